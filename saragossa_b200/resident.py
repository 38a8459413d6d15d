"""Python face of the C ABI, named after the reference's Rust surface.

`DecodeResidentState.full_attention(...)` returns a `FullAttentionState` with the
methods of the reference's `FullAttentionMetalState`
(src/decode_resident/attention.rs:446-1038): seed, append_row, truncate,
attention_decode[_windowed], encode_append_kv, encode_attention_decode_windowed,
keys()/values(). Failures raise `InferError` whose `kind` is the reference's
error variant (src/error.rs:12-75). Everything here only forwards to libsgk.so;
there is no computation in Python.
"""
from __future__ import annotations

import ctypes as C
import weakref

import numpy as np

from . import _ffi

KV_F32, KV_BF16, KV_U8G32 = 0, 1, 2
PAGE_TOKENS = 16
_KINDS = {1: "Dimension", 2: "Config", 3: "Backend", 4: "MemoryGuard", 5: "Shape", 6: "Timeout"}


class InferError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{_KINDS.get(code, code)}: {message}")
        self.code = code
        self.kind = _KINDS.get(code, str(code))


def check(rc: int) -> None:
    if rc != 0:
        raise InferError(rc, _ffi.last_error())


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


class Rope(C.Structure):
    """sgk_rope: RopeParams + rope_dims + eps + pairing style."""
    _fields_ = [("rope_dims", C.c_int32), ("frequency_dim", C.c_int32), ("theta", C.c_float),
                ("position_scale", C.c_float), ("eps", C.c_float), ("interleaved", C.c_int32)]


def encode_gated_delta_step_batch(states, layer, shape, d_q, d_k, d_v, d_g, d_beta, d_out, stream=None):
    """One gated-delta token for several sequences in one launch; inputs are [len(states)][...]."""
    arr = (C.c_void_p * len(states))(*[s.h for s in states])
    sh = LinearShape(*shape)
    check(_ffi.lib().sgk_linstate_enqueue_gated_delta_step_batch(arr, len(states), stream, layer, C.byref(sh), d_q.ptr,
                                                                 d_k.ptr, d_v.ptr, d_g.ptr, d_beta.ptr, d_out.ptr))


class AffineWeight(C.Structure):
    """sgk_affine_weight: device pointers of an affine-quantised [rows][cols] weight."""
    _fields_ = [("d_packed", C.c_void_p), ("d_scales", C.c_void_p), ("d_biases", C.c_void_p), ("bits", C.c_int32),
                ("group_size", C.c_int32)]


class TokenIO(C.Structure):
    """sgk_token_io: what the whole-token graph reads and writes around the layers."""
    _fields_ = [("d_table", C.c_void_p), ("table_dtype", C.c_int32), ("vocab", C.c_int64), ("hidden", C.c_int32),
                ("embedding_scale", C.c_float), ("recast_bf16", C.c_int32), ("d_x", C.c_void_p),
                ("d_lm_weight", C.c_void_p), ("lm_weight_dtype", C.c_int32), ("d_final", C.c_void_p),
                ("table_affine", C.c_void_p), ("lm_affine", C.c_void_p)]


class LinearShape(C.Structure):
    """sgk_linear_shape."""
    _fields_ = [("num_key_heads", C.c_int32), ("num_value_heads", C.c_int32), ("key_head_dim", C.c_int32),
                ("value_head_dim", C.c_int32)]


def make_rope(rope_dims, theta, eps=1e-6, frequency_dim=None, position_scale=1.0, interleaved=False) -> Rope:
    return Rope(rope_dims, rope_dims if frequency_dim is None else frequency_dim, theta, position_scale, eps,
                1 if interleaved else 0)


class DeviceBuffer:
    """A device allocation owned through the ABI (f32 unless stated)."""

    def __init__(self, state: "DecodeResidentState", nbytes: int):
        self.state = state
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(state.L.sgk_util_malloc(state.h, self.nbytes, C.byref(p)))
        self.ptr = p.value
        state._adopt(self)

    def upload(self, array: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(array)
        assert a.nbytes <= self.nbytes
        check(self.state.L.sgk_util_h2d(self.state.h, self.ptr, _ptr(a), a.nbytes))
        return self

    def download(self, dtype=np.float32, count=None) -> np.ndarray:
        n = self.nbytes // np.dtype(dtype).itemsize if count is None else count
        out = np.empty(n, dtype=dtype)
        check(self.state.L.sgk_util_d2h(self.state.h, _ptr(out), self.ptr, out.nbytes))
        return out

    def free(self):
        if self.ptr:
            self.state.L.sgk_util_free(self.state.h, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class _RawPtr:
    """A bare device address where the wrappers expect an object with `.ptr`."""

    def __init__(self, ptr):
        self.ptr = ptr


class Exchange:
    """One rank's end of the output exchange between GPUs that share a sequence by KV-head group
    (sgk_exchange_*): `handle` goes to the peers, `connect` takes theirs, `enqueue` is one kernel."""

    def __init__(self, state: "DecodeResidentState", rank: int, n_ranks: int):
        self.state, self.L, self.rank, self.n_ranks = state, state.L, rank, n_ranks
        h, handle = C.c_void_p(), (C.c_uint8 * 64)()
        check(self.L.sgk_exchange_create(state.h, rank, n_ranks, C.byref(h), handle))
        self.h, self.handle = h, bytes(handle)
        state._adopt(self)

    def connect(self, peer_rank: int, peer_handle: bytes):
        check(self.L.sgk_exchange_connect(self.h, peer_rank, (C.c_uint8 * 64).from_buffer_copy(peer_handle)))

    def enqueue(self, local_row_ptr: int, peer_row_ptrs, slice_offset: int, slice_floats: int, stream=None):
        """local_row_ptr: device address of this rank's row; peer_row_ptrs[p]: the same row in peer p's
        memory as mapped here (entry `rank` ignored)."""
        rows = (C.c_void_p * self.n_ranks)(*[None if p == self.rank else int(peer_row_ptrs[p])
                                              for p in range(self.n_ranks)])
        check(self.L.sgk_exchange_enqueue(self.h, stream, local_row_ptr, rows, slice_offset, slice_floats))

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_exchange_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TokenWindow:
    """The 4-deep submission window of the resident decode loop
    (src/decoder/resident/decode.rs:114-173): a device ring of token indices."""

    def __init__(self, state: "DecodeResidentState", depth: int = 4):
        self.state, self.L = state, state.L
        h = C.c_void_p()
        check(self.L.sgk_token_window_create(state.h, depth, C.byref(h)))
        self.h = h
        state._adopt(self)

    def output_slot(self):
        """Device word the next token's argmax writes; None while the window is full."""
        p = self.L.sgk_token_window_output_slot(self.h)
        return _RawPtr(p) if p else None

    def previous_slot(self):
        """Device word the last submitted token wrote; None before the first submit."""
        p = self.L.sgk_token_window_previous_slot(self.h)
        return _RawPtr(p) if p else None

    def submit(self, stream=None):
        check(self.L.sgk_token_window_submit(self.h, stream))

    def pop(self) -> int:
        tok = C.c_int32(0)
        check(self.L.sgk_token_window_pop(self.h, C.byref(tok)))
        return int(tok.value)

    def drain(self):
        check(self.L.sgk_token_window_drain(self.h))

    @property
    def inflight(self) -> int:
        return int(self.L.sgk_token_window_inflight(self.h))

    @property
    def enqueued(self) -> int:
        return int(self.L.sgk_token_window_enqueued(self.h))

    @property
    def depth(self) -> int:
        return int(self.L.sgk_token_window_depth(self.h))

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_token_window_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DecodeResidentState:
    """DecodeResidentState::new (src/decode_resident/arena.rs:247-349)."""

    def __init__(self, device: int = 0):
        self.L = _ffi.lib()
        h = C.c_void_p()
        check(self.L.sgk_state_create(device, C.byref(h)))
        self.h = h
        self.device = device
        self._children = []

    def _adopt(self, child):
        """Objects made from this state are closed with it (newest first): a handle that
        outlives its state must never reach the library."""
        self._children.append(weakref.ref(child))
        if len(self._children) > 4096:
            self._children = [r for r in self._children if r() is not None]

    def close(self):
        if getattr(self, "h", None):
            for ref in reversed(self._children):
                child = ref()
                if child is not None:
                    try:
                        (child.free if isinstance(child, DeviceBuffer) else child.close)()
                    except Exception:
                        pass
            self._children = []
            self.L.sgk_state_destroy(self.h)
            self.h = None

    @property
    def stream(self) -> int:
        return self.L.sgk_state_stream(self.h)

    def sync(self):
        check(self.L.sgk_state_sync(self.h))

    def device_status(self) -> int:
        s = C.c_int32()
        check(self.L.sgk_state_device_status(self.h, C.byref(s)))
        return s.value

    def set_concurrent_streams(self, enabled: bool):
        """Says that launches of this state may run on two streams at once (default: they do not)."""
        check(self.L.sgk_state_set_concurrent_streams(self.h, 1 if enabled else 0))

    def launches(self) -> int:
        """Kernels launched so far through this state."""
        return int(self.L.sgk_state_launches(self.h))

    def chain_begin(self, stream=None):
        """Opens a token chain on `stream`: the enqueues up to chain_end are one decode token."""
        check(self.L.sgk_state_chain_begin(self.h, stream))

    def chain_end(self):
        check(self.L.sgk_state_chain_end(self.h))

    def selftest_wait_timeout(self):
        """Runs the kernel whose wait must expire; raises InferError(kind='Timeout') when it did."""
        check(self.L.sgk_state_selftest_wait_timeout(self.h))

    def full_attention(self, capacity, q_heads, kv_heads, head_dim, dtype=KV_F32, shuffled_seed=None):
        """state.full_attention(capacity, q, kv, hd, sampled) (attention.rs:26-108)."""
        h = C.c_void_p()
        if shuffled_seed is None:
            check(self.L.sgk_kv_create(self.h, capacity, q_heads, kv_heads, head_dim, dtype, PAGE_TOKENS, C.byref(h)))
        else:
            check(self.L.sgk_kv_create_shuffled(self.h, capacity, q_heads, kv_heads, head_dim, dtype, shuffled_seed,
                                                C.byref(h)))
        return FullAttentionState(self, h, owned=True)

    def pool(self, layers, kv_heads, head_dim, dtype, num_pages, max_seqs, max_seq_tokens):
        return PagePool(self, layers, kv_heads, head_dim, dtype, num_pages, max_seqs, max_seq_tokens)

    def alloc(self, nbytes) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes)

    def upload(self, array) -> DeviceBuffer:
        a = np.ascontiguousarray(array)
        return DeviceBuffer(self, max(a.nbytes, 16)).upload(a)

    def encode_lm_head_argmax(self, d_weight, weight_dtype, vocab, hidden, d_x, d_index_out, n_rows=1,
                              index_offset=0, d_value_out=None, stream=None):
        """encode_lm_head_argmax for a dense biasless weight (src/metal_backend/lm_head.rs:288-337):
        the token index stays on the device. n_rows > 1 is the verify form (lm_head.rs:766-820)."""
        check(self.L.sgk_lm_head_enqueue_argmax(self.h, stream, d_weight.ptr, weight_dtype, vocab, hidden, d_x.ptr,
                                                n_rows, index_offset, d_index_out.ptr,
                                                d_value_out.ptr if d_value_out is not None else None))

    def upload_affine(self, packed, scales_bf16, biases_bf16, bits, group_size):
        """Uploads an affine-quantised weight (u32 codes, bf16 scale / bias bits) and returns its descriptor;
        the descriptor keeps the device buffers alive."""
        bufs = (self.upload(np.ascontiguousarray(packed, np.uint32)), self.upload(np.ascontiguousarray(scales_bf16, np.uint16)),
                self.upload(np.ascontiguousarray(biases_bf16, np.uint16)))
        w = AffineWeight(bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bits, group_size)
        w._keep = bufs
        return w

    def encode_lm_head_argmax_affine(self, weight, vocab, hidden, d_x, d_index_out, n_rows=1, index_offset=0,
                                     d_value_out=None, stream=None):
        """encode_affine_argmax_qmv_fast (src/metal_backend/lm_head.rs:934-990): argmax over an affine-quantised weight."""
        check(self.L.sgk_lm_head_enqueue_argmax_affine(self.h, stream, C.byref(weight), vocab, hidden, d_x.ptr, n_rows,
                                                       index_offset, d_index_out.ptr,
                                                       d_value_out.ptr if d_value_out is not None else None))

    def encode_embedding_from_index_affine(self, table, vocab, hidden, d_index, d_out, embedding_scale=1.0,
                                           recast_bf16=False, stream=None):
        index = d_index.ptr if hasattr(d_index, "ptr") else d_index
        check(self.L.sgk_embed_enqueue_from_index_affine(self.h, stream, C.byref(table), vocab, hidden, index,
                                                         embedding_scale, int(recast_bf16), d_out.ptr))

    def encode_embedding_from_index(self, d_table, table_dtype, vocab, hidden, d_index, d_out, embedding_scale=1.0,
                                    recast_bf16=False, stream=None):
        """encode_embedding_from_index_buffers_scaled (src/metal_backend/matmul_encode.rs:424-444): the next
        token's input row, looked up by an index on the device. d_index: a DeviceBuffer or a raw device address."""
        index = d_index.ptr if hasattr(d_index, "ptr") else d_index
        check(self.L.sgk_embed_enqueue_from_index(self.h, stream, d_table.ptr, table_dtype, vocab, hidden, index,
                                                  embedding_scale, int(recast_bf16), d_out.ptr))

    def peer_export(self, buf) -> bytes:
        """IPC handle (64 bytes) of a device allocation of this process, for the other ranks."""
        h = (C.c_uint8 * 64)()
        check(self.L.sgk_peer_export(self.h, buf.ptr, h))
        return bytes(h)

    def peer_open(self, handle: bytes) -> "_RawPtr":
        """Maps a peer's allocation; the result stands where a device buffer is expected."""
        h = (C.c_uint8 * 64).from_buffer_copy(handle)
        p = C.c_void_p()
        check(self.L.sgk_peer_open(self.h, h, C.byref(p)))
        return _RawPtr(p.value)

    def peer_close(self, mapped):
        check(self.L.sgk_peer_close(self.h, mapped.ptr))

    def exchange(self, rank, n_ranks) -> "Exchange":
        return Exchange(self, rank, n_ranks)

    def token_window(self, depth=4) -> "TokenWindow":
        return TokenWindow(self, depth)

    def argmax_linear_biasless(self, x, weight):
        """argmax_linear_biasless (src/metal_backend/lm_head.rs:150-182): host x [hidden] or [rows][hidden]
        and host weight [vocab][hidden] (float32, or uint16 holding bf16 bit patterns) -> indices."""
        x = _f32(x)
        w = np.ascontiguousarray(weight)
        if w.dtype not in (np.float32, np.uint16):
            raise InferError(2, f"argmax: weight dtype {w.dtype}, expected float32 or uint16 (bf16 bits)")
        if w.ndim != 2 or x.shape[-1] != w.shape[1]:
            raise InferError(1, f"argmax: x {x.shape} against weight {w.shape}")
        rows = 1 if x.ndim == 1 else x.shape[0]
        d_w, d_x = self.upload(w), self.upload(x)
        d_i = self.alloc(4 * max(rows, 1))
        try:
            self.encode_lm_head_argmax(d_w, KV_BF16 if w.dtype == np.uint16 else KV_F32, w.shape[0], w.shape[1], d_x,
                                       d_i, n_rows=rows)
            self.sync()
            out = d_i.download(np.int32, rows)
        finally:
            for b in (d_w, d_x, d_i):
                b.free()
        return int(out[0]) if x.ndim == 1 else out

    def fill_normal(self, buf: DeviceBuffer, n, seed, stream_id, index0=0, stream=None):
        check(self.L.sgk_util_fill_normal(self.h, stream, buf.ptr, n, seed, stream_id, index0))

    def rms_norm_rope_decode(self, x, weight, heads, head_dim, rope: Rope, position):
        """DecodeResidentState::rms_norm_rope_decode (attention.rs:386-444)."""
        x, w = _f32(x).ravel(), _f32(weight).ravel()
        out = np.empty(heads * head_dim, np.float32)
        check(self.L.sgk_rms_norm_rope_decode(self.h, _ptr(x), _ptr(w), heads, head_dim, C.byref(rope), position,
                                              _ptr(out)))
        return out

    def copy_blocks(self, dst: DeviceBuffer, src: DeviceBuffer, n_pages, page_bytes, dst_pages=None, src_pages=None,
                    stream=None):
        check(self.L.sgk_util_copy_blocks(self.h, stream, dst.ptr, src.ptr,
                                          None if dst_pages is None else dst_pages.ptr,
                                          None if src_pages is None else src_pages.ptr, n_pages, page_bytes))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PagePool:
    def __init__(self, state, layers, kv_heads, head_dim, dtype, num_pages, max_seqs, max_seq_tokens):
        self.state = state
        self.L = _ffi.lib()
        h = C.c_void_p()
        check(self.L.sgk_pool_create(state.h if state is not None else None, layers, kv_heads, head_dim, dtype,
                                     PAGE_TOKENS, num_pages, max_seqs, max_seq_tokens, C.byref(h)))
        self.h = h
        self.layers, self.kv_heads, self.head_dim, self.dtype = layers, kv_heads, head_dim, dtype
        if state is not None:
            state._adopt(self)

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_pool_destroy(self.h)
            self.h = None

    num_pages = property(lambda s: s.L.sgk_pool_num_pages(s.h))
    free_pages = property(lambda s: s.L.sgk_pool_free_pages(s.h))
    page_bytes = property(lambda s: s.L.sgk_pool_page_bytes(s.h))
    used_bytes = property(lambda s: s.L.sgk_pool_used_bytes(s.h))

    def shuffle_free_list(self, seed):
        check(self.L.sgk_pool_shuffle_free_list(self.h, seed))

    def refcount(self, page):
        out = C.c_int32()
        check(self.L.sgk_pool_page_refcount(self.h, page, C.byref(out)))
        return out.value

    def set_scrub_on_free(self, enabled=True):
        check(self.L.sgk_pool_set_scrub_on_free(self.h, int(enabled)))

    def sequence(self, capacity_tokens):
        return Sequence(self, capacity_tokens)


class Sequence:
    def __init__(self, pool: PagePool, capacity_tokens):
        self.pool = pool
        self.L = pool.L
        h = C.c_void_p()
        check(self.L.sgk_seq_create(pool.h, capacity_tokens, C.byref(h)))
        self.h = h
        if pool.state is not None:
            pool.state._adopt(self)

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_seq_destroy(self.h)
            self.h = None

    def reserve(self, tokens):
        check(self.L.sgk_seq_reserve(self.h, tokens))

    def reset(self, stream=None):
        """Empties the sequence (pages back to the pool, cursors to 0) for its next use."""
        check(self.L.sgk_seq_reset(self.h, stream))

    def block_table(self):
        n = C.c_int64()
        check(self.L.sgk_seq_block_table(self.h, None, 0, C.byref(n)))
        out = np.empty(n.value, np.int32)
        check(self.L.sgk_seq_block_table(self.h, _ptr(out), n.value, C.byref(n)))
        return out

    def release_before(self, row):
        check(self.L.sgk_seq_release_before(self.h, row))

    def layer(self, layer, q_heads):
        h = C.c_void_p()
        check(self.L.sgk_seq_layer(self.h, layer, q_heads, C.byref(h)))
        return FullAttentionState(self.pool.state, h, owned=False)


class FullAttentionState:
    """FullAttentionMetalState (src/decode_resident/attention.rs:446-1038)."""

    def __init__(self, state: DecodeResidentState, handle, owned: bool):
        self.state = state
        self.L = _ffi.lib()
        self.h = handle
        self.owned = owned
        if state is not None:
            state._adopt(self)

    def close(self):
        if self.owned and getattr(self, "h", None):
            self.L.sgk_kv_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def len(self):
        return self.L.sgk_kv_len(self.h)

    def capacity(self):
        return self.L.sgk_kv_capacity(self.h)

    def kv_dim(self):
        return self.L.sgk_kv_kv_dim(self.h)

    def q_heads(self):
        return self.L.sgk_kv_q_heads(self.h)

    def kv_heads(self):
        return self.L.sgk_kv_kv_heads(self.h)

    def head_dim(self):
        return self.L.sgk_kv_head_dim(self.h)

    def dtype(self):
        return self.L.sgk_kv_dtype(self.h)

    def byte_len(self):
        return self.L.sgk_kv_byte_len(self.h)

    def truncate(self, n):
        check(self.L.sgk_kv_truncate(self.h, n))

    def seed(self, keys_rows, values_rows, n_rows):
        k, v = _f32(keys_rows).ravel(), _f32(values_rows).ravel()
        check(self.L.sgk_kv_seed_f32(self.h, _ptr(k), k.size, _ptr(v), v.size, n_rows))

    def append_row(self, key, value):
        k, v = _f32(key).ravel(), _f32(value).ravel()
        check(self.L.sgk_kv_append_row_f32(self.h, _ptr(k), k.size, _ptr(v), v.size))

    def append_batch(self, keys, values, n_rows=None):
        k, v = _f32(keys), _f32(values)
        n = k.shape[0] if n_rows is None else n_rows
        check(self.L.sgk_kv_append_rows_f32(self.h, _ptr(k), k.size, _ptr(v), v.size, n))

    def encode_append_kv(self, d_k: DeviceBuffer, d_v: DeviceBuffer, stream=None):
        check(self.L.sgk_kv_enqueue_append(self.h, stream, d_k.ptr if d_k else None, d_v.ptr if d_v else None))

    def encode_append_rows(self, d_k: DeviceBuffer, d_v: DeviceBuffer, n_rows, stream=None):
        check(self.L.sgk_kv_enqueue_append_rows(self.h, stream, d_k.ptr, d_v.ptr, n_rows))

    def encode_rope_append(self, d_k_raw, d_v, d_weight, rope: Rope, stream=None):
        check(self.L.sgk_kv_enqueue_rope_append(self.h, stream, d_k_raw.ptr, d_v.ptr, d_weight.ptr, C.byref(rope)))

    def encode_verify_rows(self, d_k, d_v, d_q, d_out, n_rows, sliding_window=0, attn_scalar=0.0, stream=None):
        """Speculative verify: n_rows x (append, attention over rows 0..len+r), in stream order."""
        check(self.L.sgk_kv_enqueue_verify_rows(self.h, stream, d_k.ptr, d_v.ptr, d_q.ptr, d_out.ptr, n_rows,
                                                sliding_window, attn_scalar))

    def encode_rope_append_rows(self, d_k_raw, d_v, n_rows, d_weight, rope: Rope, stream=None):
        """Prefill producer: n_rows raw K rows normalised, rotated and stored at rows len.. in one launch."""
        check(self.L.sgk_kv_enqueue_rope_append_rows(self.h, stream, d_k_raw.ptr, d_v.ptr, n_rows, d_weight.ptr,
                                                     C.byref(rope)))

    def attention_decode(self, q, attn_scalar=0.0):
        return self.attention_decode_windowed(q, 0, attn_scalar)

    def attention_decode_windowed(self, q, window_start, attn_scalar=0.0):
        q = _f32(q).ravel()
        out = np.empty(self.q_heads() * self.head_dim(), np.float32)
        check(self.L.sgk_kv_attention_decode(self.h, _ptr(q), q.size, window_start, attn_scalar, _ptr(out)))
        return out

    def encode_attention_decode_windowed(self, d_q, d_out, window_start=0, attn_scalar=0.0, stream=None):
        check(self.L.sgk_kv_enqueue_attention(self.h, stream, d_q.ptr if d_q else None,
                                              d_out.ptr if d_out else None, window_start, attn_scalar))

    def encode_attention_decode_noalloc(self, d_q, d_out, window_start=0, attn_scalar=0.0, stream=None):
        """Same result as encode_attention_decode_windowed, for callers that cannot allocate device
        memory: the split-K workspace is the library's static 4 MiB device array. Make the first call
        on a device before any stream capture, and do not let two such calls overlap on the GPU."""
        check(self.L.sgk_kv_enqueue_attention_noalloc(self.h, stream, d_q.ptr if d_q else None,
                                                      d_out.ptr if d_out else None, window_start, attn_scalar))

    def encode_append_attention(self, d_k, d_v, d_q, d_out, sliding_window=0, attn_scalar=0.0, stream=None):
        check(self.L.sgk_kv_enqueue_append_attention(self.h, stream, d_k.ptr, d_v.ptr, d_q.ptr, d_out.ptr,
                                                     sliding_window, attn_scalar))

    def _gather(self, row0, n):
        n = self.len() - row0 if n is None else n
        dt = {KV_F32: np.float32, KV_BF16: np.uint16}[self.dtype()]
        k = np.empty((n, self.kv_dim()), dt)
        v = np.empty((n, self.kv_dim()), dt)
        check(self.L.sgk_kv_gather_rows(self.h, row0, n, _ptr(k), _ptr(v)))
        return k, v

    def keys(self, row0=0, n=None):
        """kv.keys() read-back: rows in the storage type (bf16 as bit patterns)."""
        return self._gather(row0, n)[0]

    def values(self, row0=0, n=None):
        return self._gather(row0, n)[1]

    def gather_rows(self, row0=0, n=None):
        return self._gather(row0, n)

    def gather_rows_f32(self, row0=0, n=None):
        n = self.len() - row0 if n is None else n
        k = np.empty((n, self.kv_dim()), np.float32)
        v = np.empty((n, self.kv_dim()), np.float32)
        check(self.L.sgk_kv_gather_rows_f32(self.h, row0, n, _ptr(k), _ptr(v)))
        return k, v

    def gather_rows_u8(self, row0=0, n=None):
        n = self.len() - row0 if n is None else n
        d, g = self.kv_dim(), self.kv_dim() // 32
        out = [np.empty((n, d), np.uint8), np.empty((n, g), np.uint16), np.empty((n, g), np.uint16),
               np.empty((n, d), np.uint8), np.empty((n, g), np.uint16), np.empty((n, g), np.uint16)]
        check(self.L.sgk_kv_gather_rows_u8(self.h, row0, n, *[_ptr(a) for a in out]))
        return out

    def block_table(self):
        n = C.c_int64()
        check(self.L.sgk_kv_block_table(self.h, None, 0, C.byref(n)))
        out = np.empty(n.value, np.int32)
        check(self.L.sgk_kv_block_table(self.h, _ptr(out), n.value, C.byref(n)))
        return out

    def set_attention_kernel(self, which):
        check(self.L.sgk_kv_set_attention_kernel(self.h, which))


class Batch:
    """n sequences of one layer decoded in one launch."""

    def __init__(self, state: DecodeResidentState, kvs):
        self.state, self.L, self.kvs = state, _ffi.lib(), list(kvs)
        arr = (C.c_void_p * len(self.kvs))(*[kv.h for kv in self.kvs])
        h = C.c_void_p()
        check(self.L.sgk_batch_create(state.h, arr, len(self.kvs), C.byref(h)))
        self.h = h
        state._adopt(self)

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_batch_destroy(self.h)
            self.h = None

    def enqueue_append(self, d_k, d_v, stream=None):
        check(self.L.sgk_batch_enqueue_append(self.h, stream, d_k.ptr, d_v.ptr))

    def enqueue_attention(self, d_q, d_out, sliding_window=0, attn_scalar=0.0, stream=None):
        check(self.L.sgk_batch_enqueue_attention(self.h, stream, d_q.ptr, d_out.ptr, sliding_window, attn_scalar))

    def enqueue_step(self, d_k, d_v, d_q, d_out, sliding_window=0, attn_scalar=0.0, stream=None):
        check(self.L.sgk_batch_enqueue_step(self.h, stream, d_k.ptr, d_v.ptr, d_q.ptr, d_out.ptr, sliding_window,
                                            attn_scalar))

    def enqueue_step_exchange(self, d_k, d_v, d_q, ex, local_row_ptr, peer_row_ptrs, slice_offset, sliding_window=0,
                              attn_scalar=0.0, stream=None):
        """enqueue_step whose launch also stores its outputs into the peers' rows and exchanges flags with
        them (sgk_batch_enqueue_step_exchange)."""
        rows = (C.c_void_p * ex.n_ranks)(*[None if p == ex.rank else int(peer_row_ptrs[p]) for p in range(ex.n_ranks)])
        check(self.L.sgk_batch_enqueue_step_exchange(self.h, stream, d_k.ptr, d_v.ptr, d_q.ptr, ex.h, local_row_ptr, rows,
                                                     slice_offset, sliding_window, attn_scalar))

    def enqueue_verify_rows(self, d_k, d_v, d_q, d_out, n_rows, sliding_window=0, attn_scalar=0.0, stream=None):
        """Speculative verify of n_rows draft rows for every sequence; inputs [n_rows][n_seq][...]."""
        check(self.L.sgk_batch_enqueue_verify_rows(self.h, stream, d_k.ptr, d_v.ptr, d_q.ptr, d_out.ptr, n_rows,
                                                   sliding_window, attn_scalar))

    def set_splits(self, splits):
        check(self.L.sgk_batch_set_splits(self.h, splits))

    def last_splits(self):
        s = C.c_int32()
        check(self.L.sgk_batch_get_splits(self.h, C.byref(s)))
        return s.value

    def set_kernel(self, which):
        check(self.L.sgk_batch_set_kernel(self.h, which))

    def last_kernel(self):
        s = C.c_int32()
        check(self.L.sgk_batch_last_kernel(self.h, C.byref(s)))
        return s.value


class Step:
    """Every layer of a batch: one decode token = one stream submission."""

    def __init__(self, state: DecodeResidentState, batches):
        self.state, self.L, self.batches = state, _ffi.lib(), list(batches)
        arr = (C.c_void_p * len(self.batches))(*[b.h for b in self.batches])
        h = C.c_void_p()
        check(self.L.sgk_step_create(state.h, arr, len(self.batches), C.byref(h)))
        self.h = h
        state._adopt(self)

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_step_destroy(self.h)
            self.h = None

    @staticmethod
    def _windows(w):
        if w is None:
            return None, None
        arr = np.ascontiguousarray(w, dtype=np.int64)
        return arr, _ptr(arr)

    def enqueue(self, d_k, d_v, d_q, d_out, sliding_windows=None, attn_scalar=0.0, stream=None):
        keep, p = self._windows(sliding_windows)
        check(self.L.sgk_step_enqueue(self.h, stream, d_k.ptr, d_v.ptr, d_q.ptr, d_out.ptr, p, attn_scalar))

    def capture(self, d_k, d_v, d_q, d_out, sliding_windows=None, attn_scalar=0.0):
        keep, p = self._windows(sliding_windows)
        check(self.L.sgk_step_capture(self.h, d_k.ptr, d_v.ptr, d_q.ptr, d_out.ptr, p, attn_scalar))

    def replay(self, stream=None):
        check(self.L.sgk_step_replay(self.h, stream))

    def token_capture(self, window, d_table, table_dtype, vocab, hidden, d_x, d_lm_weight, lm_weight_dtype, d_final,
                      d_k, d_v, d_q, d_out, sliding_windows=None, attn_scalar=0.0, embedding_scale=1.0,
                      recast_bf16=False, table_affine=None, lm_affine=None):
        """The whole token as ONE graph per ring slot: embedding lookup by the previous token's index,
        every layer, greedy epilogue into the window (sgk_token_capture)."""
        keep, p = self._windows(sliding_windows)
        io = TokenIO(d_table.ptr if d_table is not None else None, table_dtype, vocab, hidden, embedding_scale,
                     1 if recast_bf16 else 0, d_x.ptr, d_lm_weight.ptr if d_lm_weight is not None else None,
                     lm_weight_dtype, d_final.ptr,
                     C.addressof(table_affine) if table_affine is not None else None,
                     C.addressof(lm_affine) if lm_affine is not None else None)
        check(self.L.sgk_token_capture(self.h, window.h, C.byref(io), d_k.ptr, d_v.ptr, d_q.ptr, d_out.ptr, p,
                                       attn_scalar))

    def token_seed(self, first_token: int, stream=None):
        check(self.L.sgk_token_seed(self.h, first_token, stream))

    def token_submit(self, stream=None):
        """One submission = one token."""
        check(self.L.sgk_token_submit(self.h, stream))

    def run_host(self, k, v, q, out, sliding_windows=None, attn_scalar=0.0):
        keep, p = self._windows(sliding_windows)
        check(self.L.sgk_step_run_host(self.h, _ptr(k), _ptr(v), _ptr(q), _ptr(out), p, attn_scalar))

    def launches(self):
        return self.L.sgk_step_launches(self.h)


class LinearAttentionState:
    """LinearAttentionMetalState of all recurrent layers (src/metal_backend/mod.rs:507-531)."""

    def __init__(self, state, layers=None, conv_len=None, ssm_len=None, ssm_bf16=False, handle=None):
        self.state, self.L = state, _ffi.lib()
        if handle is None:
            handle = C.c_void_p()
            check(self.L.sgk_linstate_create(state.h, layers, conv_len, ssm_len, int(ssm_bf16), C.byref(handle)))
        self.h = handle
        self.layers, self.conv_len, self.ssm_len, self.ssm_bf16 = layers, conv_len, ssm_len, ssm_bf16
        state._adopt(self)

    def close(self):
        if getattr(self, "h", None):
            self.L.sgk_linstate_destroy(self.h)
            self.h = None

    def estimated_bytes(self):
        return self.L.sgk_linstate_bytes(self.h)

    def write(self, layer, conv, ssm):
        c, s = _f32(conv).ravel(), _f32(ssm).ravel()
        assert c.size == self.conv_len and s.size == self.ssm_len
        check(self.L.sgk_linstate_write(self.h, layer, _ptr(c), _ptr(s)))

    def read(self, layer):
        c, s = np.empty(self.conv_len, np.float32), np.empty(self.ssm_len, np.float32)
        check(self.L.sgk_linstate_read(self.h, layer, _ptr(c), _ptr(s)))
        return c, s

    def snapshot(self, stream=None):
        h = C.c_void_p()
        check(self.L.sgk_linstate_snapshot(self.h, stream, C.byref(h)))
        return LinearAttentionState(self.state, self.layers, self.conv_len, self.ssm_len, self.ssm_bf16, handle=h)

    def restore(self, snapshot, stream=None):
        check(self.L.sgk_linstate_restore(self.h, stream, snapshot.h))

    def encode_conv_seq(self, layer, d_qkv, d_weight, conv_dim, conv_kernel_dim, n_tokens, d_out, stream=None):
        """depthwise_causal_conv over n_tokens tokens of the prompt, the window kept in registers."""
        check(self.L.sgk_linstate_enqueue_conv_seq(self.h, stream, layer, d_qkv.ptr, d_weight.ptr, conv_dim,
                                                   conv_kernel_dim, n_tokens, d_out.ptr))

    def encode_gated_delta_seq(self, layer, shape, d_q, d_k, d_v, d_g, d_beta, n_tokens, d_out, stream=None):
        """gated_delta over n_tokens tokens, the state kept in registers and written back once."""
        sh = LinearShape(*shape)
        check(self.L.sgk_linstate_enqueue_gated_delta_seq(self.h, stream, layer, C.byref(sh), d_q.ptr, d_k.ptr,
                                                          d_v.ptr, d_g.ptr, d_beta.ptr, n_tokens, d_out.ptr))

    def encode_capture(self, capture, stream=None):
        """encode_capture_linear_attn_state: copy into an existing state of the same shape (no allocation)."""
        check(self.L.sgk_linstate_enqueue_capture(self.h, stream, capture.h))

    def encode_conv_step(self, layer, d_qkv, d_weight, conv_dim, conv_kernel_dim, d_out, stream=None):
        """depthwise_causal_conv for one token (src/linear_attention.rs:802-852)."""
        check(self.L.sgk_linstate_enqueue_conv_step(self.h, stream, layer, d_qkv.ptr, d_weight.ptr, conv_dim,
                                                    conv_kernel_dim, d_out.ptr))

    def encode_decode_step(self, layer, shape, d_qkv, d_conv_weight, conv_kernel_dim, d_beta_input, d_gate_input,
                           d_a_log, d_dt_bias, d_out, stream=None):
        """conv + SiLU + unit norms + gates + gated delta of one token in one launch
        (src/linear_attention.rs:313-342); shape = (H_k, H_v, 128, 128)."""
        sh = LinearShape(*shape)
        check(self.L.sgk_linstate_enqueue_decode_step(self.h, stream, layer, C.byref(sh), d_qkv.ptr, d_conv_weight.ptr,
                                                      conv_kernel_dim, d_beta_input.ptr, d_gate_input.ptr,
                                                      d_a_log.ptr, d_dt_bias.ptr, d_out.ptr))

    def encode_gated_delta_step(self, layer, shape, d_q, d_k, d_v, d_g, d_beta, d_out, stream=None):
        """gated_delta for one token (src/linear_attention.rs:896-991); shape = (H_k, H_v, d_k, d_v)."""
        sh = LinearShape(*shape)
        check(self.L.sgk_linstate_enqueue_gated_delta_step(self.h, stream, layer, C.byref(sh), d_q.ptr, d_k.ptr,
                                                           d_v.ptr, d_g.ptr, d_beta.ptr, d_out.ptr))
