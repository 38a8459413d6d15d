"""Python face of the warm-prefix cache, the block hashes and the memory budget.

Names follow the reference: `BlockHash.{root,for_session,chain}`,
`BlockAwarePrefixCache.{match_prefix,insert,evict_lru_block,estimated_bytes}`
(src/serve/cache.rs:11-219) and `MemoryGuard.check_allocation`
(src/memory_guard.rs:331-370). The logic lives in libsgk.so.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _ffi
from .resident import InferError, check


def _h32(b: bytes):
    return (C.c_uint8 * 32).from_buffer_copy(b)


def _tokens(tokens) -> np.ndarray:
    return np.ascontiguousarray(tokens, dtype=np.uint64)


class BlockHash:
    @staticmethod
    def root() -> bytes:
        out = (C.c_uint8 * 32)()
        _ffi.lib().sgk_hash_root(out)
        return bytes(out)

    @staticmethod
    def for_session(session_key) -> bytes:
        out = (C.c_uint8 * 32)()
        if session_key is None:
            _ffi.lib().sgk_hash_for_session(None, 0, 0, out)
        else:
            raw = session_key.encode()
            _ffi.lib().sgk_hash_for_session(raw, len(raw), 1, out)
        return bytes(out)

    @staticmethod
    def chain(prev: bytes, tokens) -> bytes:
        t = _tokens(tokens)
        out = (C.c_uint8 * 32)()
        _ffi.lib().sgk_hash_chain(_h32(prev), t.ctypes.data, t.size, out)
        return bytes(out)


class PrefixBlockHit:
    def __init__(self, tokens, hash_, entry):
        self.tokens, self.hash, self.entry = tokens, hash_, entry


class BlockAwarePrefixCache:
    """pool=None gives the bookkeeping-only cache (no device involved)."""

    def __init__(self, block_tokens, capacity, blocks_per_session=None, pool=None, budget_bytes=0):
        self.L = _ffi.lib()
        self.pool = pool
        per = capacity if blocks_per_session is None else blocks_per_session
        h = C.c_void_p()
        check(self.L.sgk_prefix_create(pool.h if pool is not None else None, block_tokens, capacity, per,
                                       budget_bytes, C.byref(h)))
        self.h = h
        if pool is not None and pool.state is not None:
            pool.state._adopt(self)

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_prefix_destroy(self.h)
            self.h = None

    def block_tokens(self):
        return self.L.sgk_prefix_block_tokens(self.h)

    def match_prefix(self, root: bytes, tokens):
        t = _tokens(tokens)
        n_out, entry, h_out = C.c_int64(), C.c_uint64(), (C.c_uint8 * 32)()
        check(self.L.sgk_prefix_match(self.h, _h32(root), t.ctypes.data, t.size, C.byref(n_out), h_out,
                                      C.byref(entry)))
        if entry.value == 0:
            return None
        return PrefixBlockHit(n_out.value, bytes(h_out), entry.value)

    def insert(self, session: bytes, hash_: bytes, tokens: int, seq=None, linear_state=None, stream=None) -> bool:
        ins = C.c_int32()
        check(self.L.sgk_prefix_insert(self.h, _h32(session), _h32(hash_), tokens,
                                       seq.h if seq is not None else None,
                                       linear_state.h if linear_state is not None else None, stream, C.byref(ins)))
        return bool(ins.value)

    def insert_chain(self, root: bytes, tokens, seq, from_tokens=0, stream=None):
        """Remembers every full block of the prompt beyond from_tokens in one call (the loop of
        prefill_prompt_state, src/serve/state.rs:596-604). Returns (blocks inserted, last hash)."""
        t = _tokens(tokens)
        ins, h_out = C.c_int32(), (C.c_uint8 * 32)()
        check(self.L.sgk_prefix_insert_chain(self.h, _h32(root), t.ctypes.data, t.size, from_tokens,
                                             seq.h if seq is not None else None, stream, C.byref(ins), h_out))
        return ins.value, bytes(h_out)

    def pinned_bytes(self):
        """Distinct pages the cache pins x page bytes + state snapshots: what the budget bounds."""
        return self.L.sgk_prefix_pinned_bytes(self.h)

    def restore(self, hit_or_entry, seq, linear_state=None, share=False, stream=None) -> int:
        entry = hit_or_entry.entry if isinstance(hit_or_entry, PrefixBlockHit) else hit_or_entry
        copied = C.c_int64()
        check(self.L.sgk_prefix_restore(self.h, entry, seq.h, linear_state.h if linear_state is not None else None,
                                        stream, 1 if share else 0, C.byref(copied)))
        return copied.value

    def evict_lru_block(self):
        ev, b = C.c_int32(), C.c_int64()
        check(self.L.sgk_prefix_evict_lru(self.h, C.byref(ev), C.byref(b)))
        return b.value if ev.value else None

    def estimated_bytes(self):
        return self.L.sgk_prefix_bytes(self.h)

    def __len__(self):
        return self.L.sgk_prefix_len(self.h)

    def evicted_count(self):
        return self.L.sgk_prefix_evicted_count(self.h)

    def session_block_count(self, session: bytes):
        return self.L.sgk_prefix_session_count(self.h, _h32(session))

    def _dump(self, which):
        n = self.L.sgk_prefix_dump(self.h, which, 0, None, None, None)
        if n == 0:
            return []
        s, h, t = (C.c_uint8 * (32 * n))(), (C.c_uint8 * (32 * n))(), (C.c_int64 * n)()
        self.L.sgk_prefix_dump(self.h, which, n, s, h, t)
        return [(bytes(s[32 * i:32 * i + 32]), bytes(h[32 * i:32 * i + 32]), t[i]) for i in range(n)]

    def entries(self):
        """Live entries, most recent first: (session, hash, tokens)."""
        return self._dump(0)

    def evicted(self):
        """Every entry that left the cache, in eviction order."""
        return self._dump(1)


class DecoderPrefixCache:
    """The decoder-internal prefix cache (src/decoder/generation.rs:2998-3139): whole prompts, most
    recent first, capacity RETI_RUST_PREFIX_CACHE_CAP (4 by default)."""

    def __init__(self, pool=None, capacity=4):
        self.L = _ffi.lib()
        self.pool = pool
        h = C.c_void_p()
        check(self.L.sgk_dprefix_create(pool.h if pool is not None else None, capacity, C.byref(h)))
        self.h = h
        if pool is not None and pool.state is not None:
            pool.state._adopt(self)

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_dprefix_destroy(self.h)
            self.h = None

    def get(self, prompt, seq=None, linear_state=None, stream=None) -> int:
        """prefix_cache_get up to the suffix: rows of the longest cached prefix become seq's; returns
        their number (0: miss)."""
        t = _tokens(prompt)
        n = C.c_int64()
        check(self.L.sgk_dprefix_get(self.h, t.ctypes.data, t.size, seq.h if seq is not None else None,
                                     linear_state.h if linear_state is not None else None, stream, C.byref(n)))
        return n.value

    def put(self, prompt, seq=None, linear_state=None, stream=None):
        t = _tokens(prompt)
        check(self.L.sgk_dprefix_put(self.h, t.ctypes.data, t.size, seq.h if seq is not None else None,
                                     linear_state.h if linear_state is not None else None, stream))

    def __len__(self):
        return self.L.sgk_dprefix_len(self.h)

    def entries(self):
        """Token lists, most recent first."""
        out = []
        for i in range(len(self)):
            n = self.L.sgk_dprefix_entry_tokens(self.h, i, None, 0)
            buf = np.zeros(max(n, 1), np.uint64)
            self.L.sgk_dprefix_entry_tokens(self.h, i, buf.ctypes.data, n)
            out.append([int(x) for x in buf[:n]])
        return out


def longest_prefix_entry_index(entries, prompt):
    """src/decoder/generation.rs:190-204."""
    flat = _tokens([t for e in entries for t in e])
    lens = np.ascontiguousarray([len(e) for e in entries], dtype=np.uintp)
    p = _tokens(prompt)
    idx = _ffi.lib().sgk_longest_prefix_entry_index(flat.ctypes.data, lens.ctypes.data, len(entries), p.ctypes.data,
                                                    p.size)
    return None if idx < 0 else idx


class MemoryGuard:
    """MemoryGuard over device bytes; a cap of None is absent."""

    def __init__(self, static_cap=None, total_memory=None, headroom=0, device_cap=None):
        self.L = _ffi.lib()
        h = C.c_void_p()
        check(self.L.sgk_budget_create(static_cap or 0, total_memory or 0, headroom, device_cap or 0, C.byref(h)))
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_budget_destroy(self.h)
            self.h = None

    def set_usage(self, current, reserved=0):
        self.L.sgk_budget_set_usage(self.h, current, reserved)

    def limit_bytes(self):
        out = C.c_uint64()
        return out.value if self.L.sgk_budget_limit(self.h, C.byref(out)) else None

    def check_allocation(self, requested):
        """Raises InferError(kind='MemoryGuard') when projected > limit; returns (projected, available)."""
        proj, avail = C.c_uint64(), C.c_uint64()
        check(self.L.sgk_budget_check_allocation(self.h, requested, C.byref(proj), C.byref(avail)))
        return proj.value, avail.value

    def projection_over_limit(self, requested):
        proj, avail = C.c_uint64(), C.c_uint64()
        rc = self.L.sgk_budget_check_allocation(self.h, requested, C.byref(proj), C.byref(avail))
        return (proj.value, avail.value) if rc != 0 else None
