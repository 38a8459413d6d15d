"""The allocation-free attention entry point (sgk_kv_enqueue_attention_noalloc).

Some callers cannot call cudaMalloc: a host that has given the whole device to its own arena,
a serving loop that must not take cudaMalloc's implicit device synchronisation, or code that
runs while a stream is being captured. For them the library keeps the split-K workspace in one
static 4 MiB device array. This file checks, through the C ABI, that the entry point gives the
same answer as the regular one (which allocates its workspace) on two calls in a row, that the
array's left-over contents do not leak from one call into the next, and that shapes beyond the
stated maximum are refused. It is named so that pytest collects it last.
"""
import numpy as np
import pytest

import saragossa_b200 as sg
from oracle import sgo

pytestmark = pytest.mark.gpu


def _close(a, b):
    # the tolerance of the attention parity tests: 2e-2 relative + 1e-3 absolute
    return np.all(np.abs(a - b) <= 2e-2 * np.abs(b) + 1e-3)


@pytest.mark.parametrize("shape", [
    (32, 4, 128, sg.KV_BF16, 8200),    # tensor-core kernel, 64 splits, two merge levels
    (16, 2, 256, sg.KV_BF16, 1500),    # tensor-core kernel, head_dim 256
    (16, 2, 256, sg.KV_F32, 300),      # generic kernel
    (8, 4, 64, sg.KV_U8G32, 700),      # generic kernel, u8 pages
    (16, 2, 256, sg.KV_U8G32, 2100),   # tensor-core kernel over u8 group-32 pages
])
def test_noalloc_matches_regular_entry_point_twice(shape):
    q_heads, kv_heads, hd, dtype, n = shape
    kv_dim, q_dim = kv_heads * hd, q_heads * hd
    st = sg.DecodeResidentState(0)
    kv = st.full_attention(n + 4, q_heads, kv_heads, hd, dtype, shuffled_seed=5)
    kv.seed(sgo.fill_normal8(n * kv_dim, 30, 0), sgo.fill_normal8(n * kv_dim, 30, 1), n)
    d_out_ref, d_out = st.alloc(q_dim * 4), st.alloc(q_dim * 4)
    for call in range(2):                               # two calls in a row share the static array
        q = sgo.fill_normal8(q_dim, 31, call)
        d_q = st.upload(q)
        window_start = 0 if call == 0 else 37
        kv.encode_attention_decode_windowed(d_q, d_out_ref, window_start)       # allocates its workspace
        d_out.upload(np.full(q_dim, np.nan, np.float32))
        kv.encode_attention_decode_noalloc(d_q, d_out, window_start)           # allocates nothing
        st.sync()
        want, got = d_out_ref.download(), d_out.download()
        assert np.isfinite(got).all()
        assert _close(got, want), np.abs(got - want).max()
        assert np.abs(got - want).max() <= 1e-5          # in practice the same kernel: far inside the bound
    # a different KV state right after: left-overs of the previous calls must not matter
    other = st.full_attention(64, q_heads, kv_heads, hd, dtype)
    other.seed(sgo.fill_normal8(50 * kv_dim, 32, 0), sgo.fill_normal8(50 * kv_dim, 32, 1), 50)
    q = sgo.fill_normal8(q_dim, 33, 0)
    d_q = st.upload(q)
    other.encode_attention_decode_noalloc(d_q, d_out)
    st.sync()
    ref = sgo.ResidentKv(64, q_heads, kv_heads, hd, dtype)
    ref.seed(sgo.fill_normal8(50 * kv_dim, 32, 0), sgo.fill_normal8(50 * kv_dim, 32, 1), 50)
    _, want = ref.attention(q)
    assert _close(d_out.download(), want)
    assert st.device_status() == 0
    other.close()
    kv.close()
    st.close()


def test_noalloc_rejects_what_it_cannot_hold():
    st = sg.DecodeResidentState(0)
    big = st.full_attention(16, 128, 8, 256, sg.KV_BF16)          # q_heads * head_dim = 32768 > 16384
    big.append_row(np.zeros(8 * 256, np.float32), np.zeros(8 * 256, np.float32))
    d_q, d_out = st.alloc(128 * 256 * 4), st.alloc(128 * 256 * 4)
    with pytest.raises(sg.InferError) as e:
        big.encode_attention_decode_noalloc(d_q, d_out)
    assert e.value.kind == "Config" and "exceeds the maximum" in str(e.value)
    big.encode_attention_decode_windowed(d_q, d_out)              # the allocating entry point takes it
    st.sync()
    small = st.full_attention(16, 4, 2, 64, sg.KV_F32)
    with pytest.raises(sg.InferError) as e:
        small.encode_attention_decode_noalloc(d_q, d_out)         # same errors as the regular call
    assert e.value.kind == "Dimension"
    small.append_row(np.zeros(128, np.float32), np.zeros(128, np.float32))
    with pytest.raises(sg.InferError) as e:
        small.encode_attention_decode_noalloc(d_q, d_out, window_start=1)
    assert e.value.kind == "Dimension"
    with pytest.raises(sg.InferError) as e:
        small.encode_attention_decode_noalloc(None, d_out)
    assert e.value.kind == "Backend"
    big.close()
    small.close()
    st.close()
