"""ctypes front end of the CPU oracle (oracle/_build/libsgo.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's cpu_baseline / reference legs, never by the product package. The
oracle is a C++ restatement of the reference's CPU path; each wrapper names the
reference function it stands for.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libsgo.so")

OK, ERR_DIMENSION, ERR_CONFIG, ERR_BACKEND, ERR_MEMORY_GUARD, ERR_SHAPE = range(6)
KV_F32, KV_BF16, KV_U8G32 = 0, 1, 2
ROPE_INTERLEAVED, ROPE_HALVES = 0, 1


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc only, a few seconds)."""
    srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith((".cpp", ".hpp"))]
    stale = (not os.path.exists(_SO)) or any(
        os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _declare(L):
    sz, f, i32, u64, vp = C.c_size_t, C.c_float, C.c_int32, C.c_uint64, C.c_void_p
    pf = C.POINTER(C.c_float)
    pu8, pu16, pu64, psz = (C.POINTER(C.c_uint8), C.POINTER(C.c_uint16), C.POINTER(C.c_uint64),
                            C.POINTER(C.c_size_t))
    sig = {
        "sgo_f32_to_bf16_bits": (C.c_uint16, [f]),
        "sgo_bf16_round_f32": (f, [f]),
        "sgo_bf16_round_array": (None, [pf, sz, pf]),
        "sgo_f32_to_bf16_array": (None, [pf, sz, pu16]),
        "sgo_cache_new": (vp, []),
        "sgo_cache_free": (None, [vp]),
        "sgo_cache_append": (i32, [vp, pf, sz, sz, pf, sz, sz, sz]),
        "sgo_cache_append_batch": (i32, [vp, pf, sz, sz, pf, sz, sz, sz]),
        "sgo_cache_len": (sz, [vp]),
        "sgo_cache_truncate": (i32, [vp, sz]),
        "sgo_cache_keys": (pf, [vp]),
        "sgo_cache_values": (pf, [vp]),
        "sgo_rkv_new": (i32, [sz, sz, sz, sz, i32, C.POINTER(vp)]),
        "sgo_rkv_free": (None, [vp]),
        "sgo_rkv_seed": (i32, [vp, pf, sz, pf, sz, sz]),
        "sgo_rkv_append_row": (i32, [vp, pf, sz, pf, sz]),
        "sgo_rkv_truncate": (i32, [vp, sz]),
        "sgo_rkv_len": (sz, [vp]),
        "sgo_rkv_keys": (pf, [vp]),
        "sgo_rkv_values": (pf, [vp]),
        "sgo_rkv_attention": (i32, [vp, pf, sz, f, C.c_int, pf]),
        "sgo_cached_attention_one": (i32, [pf, sz, pf, pf, sz, sz, sz, sz, f, i32, sz, C.c_int, pf]),
        "sgo_attention_windowed": (i32, [pf, pf, pf, sz, sz, sz, sz, sz, f, C.c_int, pf]),
        "sgo_softmax_in_place": (None, [pf, sz, f]),
        "sgo_rope_rotations": (None, [sz, sz, f, sz, f, pf, pf]),
        "sgo_rms_norm_heads": (i32, [pf, sz, sz, sz, pf, f, pf]),
        "sgo_apply_rope_heads_at": (i32, [pf, sz, sz, sz, sz, f, sz, f, sz, i32, pf]),
        "sgo_rms_norm_rope_heads_at": (i32, [pf, sz, sz, sz, sz, pf, f, f, sz, f, sz, i32, pf]),
        "sgo_quantize_row_u8": (None, [pf, sz, pu8, pu16, pu16]),
        "sgo_dequantize_row_u8": (None, [pu8, pu16, pu16, sz, pf]),
        "sgo_sha256": (None, [pu8, sz, pu8]),
        "sgo_hash_root": (None, [pu8]),
        "sgo_hash_for_session": (None, [C.c_char_p, sz, i32, pu8]),
        "sgo_hash_chain": (None, [pu8, pu64, sz, pu8]),
        "sgo_prefix_new": (vp, [sz, sz, sz]),
        "sgo_prefix_free": (None, [vp]),
        "sgo_prefix_block_tokens": (sz, [vp]),
        "sgo_prefix_match": (i32, [vp, pu8, pu64, sz, psz, pu8, pu64]),
        "sgo_prefix_insert": (sz, [vp, pu8, pu8, sz, u64, sz]),
        "sgo_prefix_evict_lru": (i32, [vp, psz]),
        "sgo_prefix_bytes": (sz, [vp]),
        "sgo_prefix_len": (sz, [vp]),
        "sgo_prefix_session_count": (sz, [vp, pu8]),
        "sgo_prefix_dump": (sz, [vp, i32, sz, pu8, pu8, psz, pu64]),
        "sgo_longest_prefix_entry_index": (C.c_long, [pu64, psz, sz, pu64, sz]),
        "sgo_guard_new": (vp, [i32, u64, i32, u64, u64, i32, u64]),
        "sgo_guard_free": (None, [vp]),
        "sgo_guard_set": (None, [vp, u64, u64]),
        "sgo_guard_limit": (i32, [vp, pu64]),
        "sgo_guard_check": (i32, [vp, u64, pu64, pu64]),
        "sgo_linear_restore_check": (i32, [sz, sz, i32, sz, sz, i32]),
        "sgo_gated_delta_step": (i32, [pf, pf, pf, pf, pf, sz, sz, sz, sz, pf, sz, pf]),
        "sgo_depthwise_conv_step": (i32, [pf, pf, sz, sz, pf, sz, pf]),
        "sgo_lm_head_argmax": (i32, [pf, sz, sz, pf, psz, pf]),
        "sgo_embed_gather": (i32, [pf, sz, sz, sz, f, i32, pf]),
        "sgo_pseudo": (f, [u64]),
        "sgo_pseudo_array": (None, [u64, sz, pf]),
        "sgo_splitmix64": (u64, [u64]),
        "sgo_normal8": (f, [u64, u64, u64]),
        "sgo_fill_normal8": (None, [pf, sz, u64, u64, u64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args


# ---- bf16 -----------------------------------------------------------------
def bf16_round(a):
    a = _f32(a)
    out = np.empty_like(a)
    lib().sgo_bf16_round_array(_fp(a), a.size, _fp(out))
    return out


def f32_to_bf16_bits(a):
    a = _f32(a)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().sgo_f32_to_bf16_array(_fp(a), a.size, out.ctypes.data_as(C.POINTER(C.c_uint16)))
    return out


# ---- caches -----------------------------------------------------------------
class LayerKvCache:
    """src/decoder/attention_cache.rs:7-100."""

    def __init__(self):
        self._h = lib().sgo_cache_new()

    def __del__(self):
        if getattr(self, "_h", None):
            lib().sgo_cache_free(self._h)
            self._h = None

    def append(self, key, value, expected_dim):
        k, v = _f32(np.atleast_2d(key)), _f32(np.atleast_2d(value))
        return lib().sgo_cache_append(self._h, _fp(k), k.shape[0], k.shape[1], _fp(v), v.shape[0],
                                      v.shape[1], expected_dim)

    def append_batch(self, key, value, expected_dim):
        k, v = _f32(np.atleast_2d(key)), _f32(np.atleast_2d(value))
        return lib().sgo_cache_append_batch(self._h, _fp(k), k.shape[0], k.shape[1], _fp(v),
                                            v.shape[0], v.shape[1], expected_dim)

    def len(self):
        return lib().sgo_cache_len(self._h)

    def truncate(self, n):
        return lib().sgo_cache_truncate(self._h, n)

    def _view(self, ptr, dim):
        n = self.len() * dim
        if n == 0:
            return np.zeros((0, dim), np.float32)
        return np.ctypeslib.as_array(ptr, shape=(n,)).reshape(-1, dim).copy()

    def keys(self, dim):
        return self._view(lib().sgo_cache_keys(self._h), dim)

    def values(self, dim):
        return self._view(lib().sgo_cache_values(self._h), dim)


class ResidentKv:
    """FullAttentionMetalState semantics, src/decode_resident/attention.rs:56-108,501-644."""

    def __init__(self, capacity, q_heads, kv_heads, head_dim, dtype=KV_F32):
        h = C.c_void_p()
        st = lib().sgo_rkv_new(capacity, q_heads, kv_heads, head_dim, dtype, C.byref(h))
        self.status = st
        self._h = h if st == OK else None
        self.q_heads, self.kv_heads, self.head_dim = q_heads, kv_heads, head_dim
        self.kv_dim = kv_heads * head_dim

    def __del__(self):
        if getattr(self, "_h", None):
            lib().sgo_rkv_free(self._h)
            self._h = None

    def seed(self, k, v, n_rows):
        k, v = _f32(k).ravel(), _f32(v).ravel()
        return lib().sgo_rkv_seed(self._h, _fp(k), k.size, _fp(v), v.size, n_rows)

    def append_row(self, k, v):
        k, v = _f32(k).ravel(), _f32(v).ravel()
        return lib().sgo_rkv_append_row(self._h, _fp(k), k.size, _fp(v), v.size)

    def truncate(self, n):
        return lib().sgo_rkv_truncate(self._h, n)

    def len(self):
        return lib().sgo_rkv_len(self._h)

    def keys(self):
        n = self.len() * self.kv_dim
        return np.ctypeslib.as_array(lib().sgo_rkv_keys(self._h), shape=(n,)).reshape(-1, self.kv_dim).copy()

    def values(self):
        n = self.len() * self.kv_dim
        return np.ctypeslib.as_array(lib().sgo_rkv_values(self._h), shape=(n,)).reshape(-1, self.kv_dim).copy()

    def attention(self, q, window_start=0, attn_scalar=None, threads=1):
        q = _f32(q).ravel()
        out = np.empty(self.q_heads * self.head_dim, np.float32)
        scalar = float(self.head_dim if attn_scalar is None else attn_scalar)
        st = lib().sgo_rkv_attention(self._h, _fp(q), window_start, scalar, threads, _fp(out))
        return st, out


def cached_attention_one(q, keys, values, q_heads, kv_heads, head_dim, attn_scalar=None,
                         sliding_window=None, threads=1):
    """src/decoder/attention_ops.rs:889-974."""
    q, keys, values = _f32(q).ravel(), _f32(keys), _f32(values)
    cache_len = keys.size // (kv_heads * head_dim) if kv_heads * head_dim else 0
    out = np.zeros(q_heads * head_dim, np.float32)
    scalar = float(head_dim if attn_scalar is None else attn_scalar)
    st = lib().sgo_cached_attention_one(
        _fp(q), q.size, _fp(keys), _fp(values), cache_len, q_heads, kv_heads, head_dim, scalar,
        0 if sliding_window is None else 1, 0 if sliding_window is None else sliding_window,
        threads, _fp(out))
    return st, out


def attention_windowed(q, keys, values, length, window_start, q_heads, kv_heads, head_dim,
                       attn_scalar=None, threads=1):
    q, keys, values = _f32(q).ravel(), _f32(keys), _f32(values)
    out = np.zeros(q_heads * head_dim, np.float32)
    scalar = float(head_dim if attn_scalar is None else attn_scalar)
    st = lib().sgo_attention_windowed(_fp(q), _fp(keys), _fp(values), length, window_start, q_heads,
                                      kv_heads, head_dim, scalar, threads, _fp(out))
    return st, out


def softmax(values, temperature=1.0):
    v = _f32(values).copy()
    lib().sgo_softmax_in_place(_fp(v), v.size, temperature)
    return v


# ---- norm / rope ---------------------------------------------------------------
def rope_rotations(position, rope_dims, theta, frequency_dim, position_scale=1.0):
    cos = np.empty(rope_dims // 2, np.float32)
    sin = np.empty(rope_dims // 2, np.float32)
    lib().sgo_rope_rotations(position, rope_dims, theta, frequency_dim, position_scale, _fp(cos), _fp(sin))
    return cos, sin


def rms_norm_heads(x, heads, head_dim, weight, eps):
    x, w = _f32(np.atleast_2d(x)), _f32(weight)
    out = np.empty_like(x)
    st = lib().sgo_rms_norm_heads(_fp(x), x.shape[0], heads, head_dim, _fp(w), eps, _fp(out))
    return st, out


def apply_rope_heads_at(x, heads, head_dim, rope_dims, theta, frequency_dim, position_scale,
                        position_offset, style):
    x = _f32(np.atleast_2d(x))
    out = np.empty_like(x)
    st = lib().sgo_apply_rope_heads_at(_fp(x), x.shape[0], heads, head_dim, rope_dims, theta,
                                       frequency_dim, position_scale, position_offset, style, _fp(out))
    return st, out


def rms_norm_rope_heads_at(x, heads, head_dim, rope_dims, weight, eps, theta, frequency_dim,
                           position_scale, position_offset, style=ROPE_HALVES):
    x, w = _f32(np.atleast_2d(x)), _f32(weight)
    out = np.empty_like(x)
    st = lib().sgo_rms_norm_rope_heads_at(_fp(x), x.shape[0], heads, head_dim, rope_dims, _fp(w), eps,
                                          theta, frequency_dim, position_scale, position_offset,
                                          style, _fp(out))
    return st, out


# ---- u8 group-32 -------------------------------------------------------------------
def quantize_row_u8(x):
    x = _f32(x).ravel()
    codes = np.empty(x.size, np.uint8)
    scale = np.empty(x.size // 32, np.uint16)
    bias = np.empty(x.size // 32, np.uint16)
    lib().sgo_quantize_row_u8(_fp(x), x.size, codes.ctypes.data_as(C.POINTER(C.c_uint8)),
                              scale.ctypes.data_as(C.POINTER(C.c_uint16)),
                              bias.ctypes.data_as(C.POINTER(C.c_uint16)))
    return codes, scale, bias


def dequantize_row_u8(codes, scale, bias):
    codes = np.ascontiguousarray(codes, np.uint8).ravel()
    scale = np.ascontiguousarray(scale, np.uint16).ravel()
    bias = np.ascontiguousarray(bias, np.uint16).ravel()
    out = np.empty(codes.size, np.float32)
    lib().sgo_dequantize_row_u8(codes.ctypes.data_as(C.POINTER(C.c_uint8)),
                                scale.ctypes.data_as(C.POINTER(C.c_uint16)),
                                bias.ctypes.data_as(C.POINTER(C.c_uint16)), codes.size, _fp(out))
    return out


# ---- hashes / prefix cache -------------------------------------------------------------
def _h32():
    return (C.c_uint8 * 32)()


def sha256(data: bytes) -> bytes:
    out = _h32()
    buf = (C.c_uint8 * max(len(data), 1)).from_buffer_copy(data or b"\0")
    lib().sgo_sha256(buf, len(data), out)
    return bytes(out)


def hash_root() -> bytes:
    out = _h32()
    lib().sgo_hash_root(out)
    return bytes(out)


def hash_for_session(key) -> bytes:
    out = _h32()
    if key is None:
        lib().sgo_hash_for_session(None, 0, 0, out)
    else:
        raw = key.encode()
        lib().sgo_hash_for_session(raw, len(raw), 1, out)
    return bytes(out)


def _tok(tokens):
    return np.ascontiguousarray(tokens, dtype=np.uint64)


def _pu64(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint64))


def _h(b: bytes):
    return (C.c_uint8 * 32).from_buffer_copy(b)


def hash_chain(prev: bytes, tokens) -> bytes:
    t = _tok(tokens)
    out = _h32()
    lib().sgo_hash_chain(_h(prev), _pu64(t), t.size, out)
    return bytes(out)


class BlockAwarePrefixCache:
    """src/serve/cache.rs:74-219. payload is an opaque snapshot id."""

    def __init__(self, block_tokens, capacity, blocks_per_session=None):
        per = capacity if blocks_per_session is None else blocks_per_session
        self._p = lib().sgo_prefix_new(block_tokens, capacity, per)

    def __del__(self):
        if getattr(self, "_p", None):
            lib().sgo_prefix_free(self._p)
            self._p = None

    def block_tokens(self):
        return lib().sgo_prefix_block_tokens(self._p)

    def match_prefix(self, root: bytes, tokens):
        t = _tok(tokens)
        n_out, h_out, p_out = C.c_size_t(), _h32(), C.c_uint64()
        hit = lib().sgo_prefix_match(self._p, _h(root), _pu64(t), t.size, C.byref(n_out), h_out,
                                     C.byref(p_out))
        if not hit:
            return None
        return {"tokens": n_out.value, "hash": bytes(h_out), "payload": p_out.value}

    def insert(self, session: bytes, hash_: bytes, tokens: int, payload: int = 0, nbytes: int = 0):
        return lib().sgo_prefix_insert(self._p, _h(session), _h(hash_), tokens, payload, nbytes)

    def evict_lru_block(self):
        b = C.c_size_t()
        return b.value if lib().sgo_prefix_evict_lru(self._p, C.byref(b)) else None

    def estimated_bytes(self):
        return lib().sgo_prefix_bytes(self._p)

    def __len__(self):
        return lib().sgo_prefix_len(self._p)

    def session_block_count(self, session: bytes):
        return lib().sgo_prefix_session_count(self._p, _h(session))

    def _dump(self, which):
        n = lib().sgo_prefix_dump(self._p, which, 0, None, None, None, None)
        if n == 0:
            return []
        s = (C.c_uint8 * (32 * n))()
        h = (C.c_uint8 * (32 * n))()
        t = (C.c_size_t * n)()
        p = (C.c_uint64 * n)()
        lib().sgo_prefix_dump(self._p, which, n, s, h, t, p)
        return [(bytes(s[32 * i:32 * i + 32]), bytes(h[32 * i:32 * i + 32]), t[i], p[i]) for i in range(n)]

    def entries(self):
        return self._dump(0)

    def evicted(self):
        return self._dump(1)


def longest_prefix_entry_index(entries, prompt):
    flat = _tok([t for e in entries for t in e]) if entries else _tok([])
    lens = np.ascontiguousarray([len(e) for e in entries], dtype=np.uintp)
    p = _tok(prompt)
    idx = lib().sgo_longest_prefix_entry_index(_pu64(flat), lens.ctypes.data_as(C.POINTER(C.c_size_t)),
                                               len(entries), _pu64(p), p.size)
    return None if idx < 0 else idx


class MemoryGuard:
    """src/memory_guard.rs:155-185,331-370."""

    def __init__(self, static_cap=None, host_memory=None, headroom=0, device_cap=None):
        self._g = lib().sgo_guard_new(static_cap is not None, static_cap or 0, host_memory is not None,
                                      host_memory or 0, headroom, device_cap is not None, device_cap or 0)

    def __del__(self):
        if getattr(self, "_g", None):
            lib().sgo_guard_free(self._g)
            self._g = None

    def set(self, current, reserved=0):
        lib().sgo_guard_set(self._g, current, reserved)

    def limit(self):
        out = C.c_uint64()
        return out.value if lib().sgo_guard_limit(self._g, C.byref(out)) else None

    def check_allocation(self, requested):
        proj, avail = C.c_uint64(), C.c_uint64()
        ok = lib().sgo_guard_check(self._g, requested, C.byref(proj), C.byref(avail))
        return bool(ok), proj.value, avail.value


def linear_restore_check(conv_a, ssm_a, bf16_a, conv_b, ssm_b, bf16_b):
    return lib().sgo_linear_restore_check(conv_a, ssm_a, int(bf16_a), conv_b, ssm_b, int(bf16_b))


def gated_delta_step(q, k, v, g, beta, num_key_heads, num_value_heads, key_head_dim, value_head_dim, ssm):
    """One token of src/linear_attention.rs:896-991; returns (status, out, new_ssm)."""
    q, k, v, g, beta = (_f32(x).ravel() for x in (q, k, v, g, beta))
    state = _f32(ssm).ravel().copy()
    out = np.empty(num_value_heads * value_head_dim, np.float32)
    st = lib().sgo_gated_delta_step(_fp(q), _fp(k), _fp(v), _fp(g), _fp(beta), num_key_heads, num_value_heads,
                                    key_head_dim, value_head_dim, _fp(state), state.size, _fp(out))
    return st, out, state


def depthwise_conv_step(qkv, weight, kernel, history):
    """One token of src/linear_attention.rs:802-852; returns (status, out, new_history)."""
    qkv, weight = _f32(qkv).ravel(), _f32(weight).ravel()
    hist = _f32(history).ravel().copy()
    out = np.empty(qkv.size, np.float32)
    st = lib().sgo_depthwise_conv_step(_fp(qkv), _fp(weight), qkv.size, kernel, _fp(hist), hist.size, _fp(out))
    return st, out, hist


def silu(x):
    """src/activation.rs:14-16: v / (1 + exp(-v)) in f32."""
    x = _f32(x)
    return (x / (np.float32(1.0) + np.exp(-x, dtype=np.float32))).astype(np.float32)


def rms_norm_heads_unit(x, heads, head_dim, eps=1.0e-6):
    """src/linear_attention.rs:1029-1050: per head x / sqrt(mean(x^2) + eps), the squares summed in
    order in f32."""
    x = _f32(x).reshape(heads, head_dim)
    out = np.empty_like(x)
    for h in range(heads):
        acc = np.float32(0.0)
        for v in x[h]:
            acc = np.float32(acc + np.float32(v * v))
        inv = np.float32(1.0) / np.sqrt(np.float32(acc / np.float32(head_dim)) + np.float32(eps), dtype=np.float32)
        out[h] = x[h] * inv
    return out.ravel()


def key_scale(head_dim, squared):
    """src/linear_attention.rs:1203-1210."""
    inv = np.float32(np.power(np.float32(head_dim), np.float32(-0.5)))
    return np.float32(inv * inv) if squared else inv


def compute_decay(gate_input, a_log, dt_bias):
    """src/linear_attention.rs:1122-1146 with softplus :1218-1224 (identity above 20)."""
    arg = (_f32(gate_input) + _f32(dt_bias)).astype(np.float32)
    with np.errstate(over="ignore"):
        soft = np.where(arg > 20.0, arg, np.log(np.float32(1.0) + np.exp(arg, dtype=np.float32), dtype=np.float32))
    return np.exp(-np.exp(_f32(a_log), dtype=np.float32) * soft.astype(np.float32), dtype=np.float32)


def sigmoid(x):
    """src/linear_attention.rs:1213-1215."""
    return (np.float32(1.0) / (np.float32(1.0) + np.exp(-_f32(x), dtype=np.float32))).astype(np.float32)


def linear_decode_step(qkv, conv_weight, kernel, history, beta_input, gate_input, a_log, dt_bias, num_key_heads,
                       num_value_heads, key_head_dim, value_head_dim, ssm):
    """One token of a recurrent layer between its projections, in the CPU order of
    src/linear_attention.rs:313-342: conv -> silu -> unit RMS norm of q and k times key_scale ->
    sigmoid / decay gates -> gated_delta. Returns (status, out, new_history, new_ssm, parts) where
    parts holds the intermediate q, k, v, beta, g."""
    st, conv, hist = depthwise_conv_step(qkv, conv_weight, kernel, history)
    if st != 0:
        return st, None, None, None, None
    act = silu(conv)
    key_dim = num_key_heads * key_head_dim
    q = rms_norm_heads_unit(act[:key_dim], num_key_heads, key_head_dim) * key_scale(key_head_dim, True)
    k = rms_norm_heads_unit(act[key_dim:2 * key_dim], num_key_heads, key_head_dim) * key_scale(key_head_dim, False)
    v = act[2 * key_dim:]
    beta = sigmoid(beta_input)
    g = compute_decay(gate_input, a_log, dt_bias)
    st, out, new_ssm = gated_delta_step(q.astype(np.float32), k.astype(np.float32), v, g, beta, num_key_heads,
                                        num_value_heads, key_head_dim, value_head_dim, ssm)
    return st, out, hist, new_ssm, {"q": q, "k": k, "v": v, "beta": beta, "g": g}


def lm_head_argmax(weight, x):
    """First maximum of W . x (src/sampling.rs:49-62); weight [vocab][hidden]; returns (status, index, value)."""
    weight, x = _f32(weight), _f32(x).ravel()
    vocab = weight.shape[0] if weight.ndim == 2 else 0
    idx, val = C.c_size_t(0), C.c_float(0.0)
    st = lib().sgo_lm_head_argmax(_fp(weight.ravel()), vocab, x.size, _fp(x), C.byref(idx), C.byref(val))
    return st, int(idx.value), float(val.value)


def embed_gather(table, token, scale=1.0, recast_bf16=False):
    """src/kernels.metal:308-325; table [vocab][dim]; returns the row, or None for a token outside the table."""
    table = _f32(table)
    out = np.zeros(table.shape[1], np.float32)
    hit = lib().sgo_embed_gather(_fp(table.ravel()), table.shape[0], table.shape[1], token, scale, int(recast_bf16),
                                 _fp(out))
    return out if hit else None


# ---- generators ----------------------------------------------------------------------
def pseudo(seed0, n=None):
    """src/decode_resident/tests.rs:544-547, vectorised over seed0..seed0+n."""
    if n is None:
        return lib().sgo_pseudo(seed0)
    out = np.empty(n, np.float32)
    lib().sgo_pseudo_array(seed0, n, _fp(out))
    return out


def fill_normal8(n, seed, stream, index0=0):
    out = np.empty(n, np.float32)
    lib().sgo_fill_normal8(_fp(out), n, seed, stream, index0)
    return out


def affine_dequantize(packed, scales_bf16, biases_bf16, bits, group_size, rows, cols):
    """AffineQuantizedTensor::dequantize (src/quantization.rs:131-179, bitpacked_value :208-228):
    code of column c sits at bit offset c * bits of its row, LSB first inside 32-bit words; value =
    code * scale + bias in f32 with the group's scale and bias (stored as bf16 here, as the Metal
    buffers of src/metal_backend/lm_head.rs:960-963 hold them). numpy restatement for 4 and 8 bits
    (both divide 32: no code straddles a word)."""
    assert bits in (4, 8) and cols % group_size == 0
    packed = np.ascontiguousarray(packed, np.uint32).reshape(rows, cols * bits // 32)
    per_word = 32 // bits
    shifts = (np.arange(per_word, dtype=np.uint32) * bits)[None, None, :]
    codes = ((packed[:, :, None] >> shifts) & np.uint32((1 << bits) - 1)).reshape(rows, cols).astype(np.float32)
    # scales and biases as bf16 bit patterns (the Metal buffers), or as f32 (the reference's CPU tensors)
    to_f32 = lambda b: (_f32(b) if np.asarray(b).dtype == np.float32
                        else (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32))
    scale = np.repeat(to_f32(scales_bf16).reshape(rows, cols // group_size), group_size, axis=1)
    bias = np.repeat(to_f32(biases_bf16).reshape(rows, cols // group_size), group_size, axis=1)
    return (codes * scale).astype(np.float32) + bias


def affine_pack(codes, bits):
    """Inverse of the unpacking above: codes [rows][cols] -> u32 words, LSB first."""
    codes = np.ascontiguousarray(codes, np.uint32)
    rows, cols = codes.shape
    per_word = 32 // bits
    c = codes.reshape(rows, cols // per_word, per_word)
    shifts = (np.arange(per_word, dtype=np.uint32) * bits)[None, None, :]
    return np.bitwise_or.reduce(c << shifts, axis=2).astype(np.uint32)


class DecoderPrefixCache:
    """The decoder-internal prefix cache, bookkeeping only (src/decoder/generation.rs:2998-3139):
    get = longest_prefix_entry_index, remove, re-insert at the front (:3003-3013); when the hit is
    shorter than the prompt the caller extends it and puts the whole prompt (:3019-3022); put =
    drop the entry with the same tokens, insert at the front, truncate to the capacity (:3118-3137)."""

    def __init__(self, capacity=4):
        self.capacity = capacity
        self.entries = []          # token lists, front = most recent

    def get(self, prompt):
        idx = longest_prefix_entry_index(self.entries, prompt)
        if idx is None:
            return 0
        entry = self.entries.pop(idx)
        self.entries.insert(0, entry)
        cached = len(entry)
        if cached < len(prompt):
            self.put(prompt)
        return cached

    def put(self, prompt):
        if self.capacity == 0:
            return
        prompt = list(prompt)
        if prompt in self.entries:
            self.entries.remove(prompt)
        self.entries.insert(0, prompt)
        del self.entries[self.capacity:]
