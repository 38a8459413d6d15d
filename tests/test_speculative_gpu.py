"""Speculative decoding on the KV path: multi-row verify (serial append + causal attention per
row, src/decode_resident/layers.rs:1295-1433 and src/decoder/attention_ops.rs:976-1017), rollback
by truncate (src/decoder/generation.rs:1019-1022) and the per-row captures of the recurrent state
(src/metal_backend/linear_attention.rs:44-127), through the C ABI against the oracle."""
import numpy as np
import pytest

import saragossa_b200 as sg
from oracle import sgo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def state():
    st = sg.DecodeResidentState(0)
    yield st
    assert st.device_status() == 0
    st.close()


def _rows(n, dim, seed, stream):
    return sgo.fill_normal8(n * dim, seed, stream).reshape(n, dim)


@pytest.mark.parametrize("dtype", [sg.KV_F32, sg.KV_BF16, sg.KV_U8G32])
@pytest.mark.parametrize("shape", [(32, 4, 128), (16, 2, 256)])
def test_verify_rows_equal_serial_decode_and_the_oracle(state, dtype, shape):
    q_heads, kv_heads, hd = shape
    kv_dim, q_dim = kv_heads * hd, q_heads * hd
    n0, rows = 300 + 13, 5          # the draft rows cross a page boundary
    k0, v0 = _rows(n0, kv_dim, 3, 0), _rows(n0, kv_dim, 3, 1)
    kd, vd, qd = _rows(rows, kv_dim, 3, 2), _rows(rows, kv_dim, 3, 3), _rows(rows, q_dim, 3, 4)
    ref = sgo.ResidentKv(n0 + rows, q_heads, kv_heads, hd, dtype)
    ref.seed(k0, v0, n0)
    spec = state.full_attention(n0 + rows, q_heads, kv_heads, hd, dtype, shuffled_seed=4)
    solo = state.full_attention(n0 + rows, q_heads, kv_heads, hd, dtype, shuffled_seed=5)
    spec.seed(k0, v0, n0)
    solo.seed(k0, v0, n0)
    d_out = state.alloc(4 * rows * q_dim)
    spec.encode_verify_rows(state.upload(kd), state.upload(vd), state.upload(qd), d_out, rows)
    d_one = state.alloc(4 * q_dim)
    outs = []
    for r in range(rows):
        solo.encode_append_attention(state.upload(kd[r]), state.upload(vd[r]), state.upload(qd[r]), d_one)
        state.sync()
        outs.append(d_one.download(count=q_dim))
    state.sync()
    got = d_out.download(count=rows * q_dim).reshape(rows, q_dim)
    assert spec.len() == solo.len() == n0 + rows
    tol_rel, tol_abs = (1e-4, 1e-5) if dtype == sg.KV_F32 else (2e-2, 1e-3)
    for r in range(rows):
        np.testing.assert_array_equal(got[r], outs[r])            # the same launches, row by row
        ref.append_row(kd[r], vd[r])
        _, want = ref.attention(qd[r], threads=8)                 # row r sees rows 0 .. n0 + r
        assert np.all(np.abs(got[r] - want) <= tol_rel * np.abs(want) + tol_abs), (r, np.abs(got[r] - want).max())
    sk, sv = spec.gather_rows_f32()
    np.testing.assert_array_equal(sk, ref.keys())
    np.testing.assert_array_equal(sv, ref.values())
    with pytest.raises(sg.InferError) as e:                       # overflow: nothing is written
        spec.encode_verify_rows(state.upload(kd), state.upload(vd), state.upload(qd), d_out, 1)
    assert e.value.kind == "Dimension" and spec.len() == n0 + rows
    spec.close()
    solo.close()


@pytest.mark.parametrize("dtype", [sg.KV_BF16, sg.KV_U8G32])
def test_rollback_after_verify_leaves_no_trace(state, dtype):
    # accept 2 of 4 draft rows: truncate, then decode on; a sequence that never speculated gives
    # the same bits (truncate never clears memory: the stale rows are simply overwritten)
    q_heads, kv_heads, hd = 8, 2, 128
    kv_dim, q_dim = kv_heads * hd, q_heads * hd
    n0, rows, accepted, more = 70, 4, 2, 6
    k0, v0 = _rows(n0, kv_dim, 9, 0), _rows(n0, kv_dim, 9, 1)
    kd, vd, qd = _rows(rows, kv_dim, 9, 2), _rows(rows, kv_dim, 9, 3), _rows(rows, q_dim, 9, 4)
    km, vm, qm = _rows(more, kv_dim, 9, 5), _rows(more, kv_dim, 9, 6), _rows(more, q_dim, 9, 7)
    spec = state.full_attention(n0 + rows + more, q_heads, kv_heads, hd, dtype)
    plain = state.full_attention(n0 + rows + more, q_heads, kv_heads, hd, dtype)
    spec.seed(k0, v0, n0)
    plain.seed(k0, v0, n0)
    d_out = state.alloc(4 * rows * q_dim)
    spec.encode_verify_rows(state.upload(kd), state.upload(vd), state.upload(qd), d_out, rows)
    state.sync()
    spec.truncate(n0 + accepted)
    assert spec.len() == n0 + accepted
    plain.encode_verify_rows(state.upload(kd[:accepted]), state.upload(vd[:accepted]), state.upload(qd[:accepted]),
                             d_out, accepted)
    state.sync()
    a, b = state.alloc(4 * q_dim), state.alloc(4 * q_dim)
    for r in range(more):
        spec.encode_append_attention(state.upload(km[r]), state.upload(vm[r]), state.upload(qm[r]), a)
        plain.encode_append_attention(state.upload(km[r]), state.upload(vm[r]), state.upload(qm[r]), b)
        state.sync()
        np.testing.assert_array_equal(a.download(count=q_dim), b.download(count=q_dim))
    sk, sv = spec.gather_rows_f32()
    pk, pv = plain.gather_rows_f32()
    np.testing.assert_array_equal(sk, pk)
    np.testing.assert_array_equal(sv, pv)
    with pytest.raises(sg.InferError) as e:                       # the cursor may not pass the capacity
        spec.truncate(n0 + rows + more + 1)                       # (src/decode_resident/attention.rs:501-510)
    assert e.value.kind == "Dimension"
    spec.close()
    plain.close()


def test_batched_verify_is_per_sequence_identical(state):
    # three sequences of different lengths verified together: each one's rows equal its solo verify
    q_heads, kv_heads, hd, rows = 16, 4, 128, 3
    kv_dim, q_dim = kv_heads * hd, q_heads * hd
    lens = [40, 1000, 333]
    pool = state.pool(1, kv_heads, hd, sg.KV_BF16, num_pages=200, max_seqs=8, max_seq_tokens=1100)
    pool.shuffle_free_list(3)
    seqs = [pool.sequence(1100) for _ in lens]
    solos = [state.full_attention(1100, q_heads, kv_heads, hd, sg.KV_BF16) for _ in lens]
    kvs = []
    for i, n in enumerate(lens):
        k, v = _rows(n, kv_dim, 20 + i, 0), _rows(n, kv_dim, 20 + i, 1)
        kv = seqs[i].layer(0, q_heads)
        kv.seed(k, v, n)
        solos[i].seed(k, v, n)
        kvs.append(kv)
    kd = _rows(rows * len(lens), kv_dim, 30, 0).reshape(rows, len(lens), kv_dim)
    vd = _rows(rows * len(lens), kv_dim, 30, 1).reshape(rows, len(lens), kv_dim)
    qd = _rows(rows * len(lens), q_dim, 30, 2).reshape(rows, len(lens), q_dim)
    batch = sg.Batch(state, kvs)
    d_out = state.alloc(4 * rows * len(lens) * q_dim)
    batch.enqueue_verify_rows(state.upload(kd), state.upload(vd), state.upload(qd), d_out, rows)
    state.sync()
    got = d_out.download(count=rows * len(lens) * q_dim).reshape(rows, len(lens), q_dim)
    d_solo = state.alloc(4 * rows * q_dim)
    for i in range(len(lens)):
        solos[i].encode_verify_rows(state.upload(np.ascontiguousarray(kd[:, i])), state.upload(np.ascontiguousarray(vd[:, i])),
                                    state.upload(np.ascontiguousarray(qd[:, i])), d_solo, rows)
        state.sync()
        want = d_solo.download(count=rows * q_dim).reshape(rows, q_dim)
        np.testing.assert_allclose(got[:, i], want, rtol=2e-2, atol=1e-3)
        assert kvs[i].len() == lens[i] + rows
    batch.close()
    for s in solos:
        s.close()
    for s in seqs:
        s.close()
    pool.close()


def test_recurrent_state_captures_roll_back_to_the_accepted_row(state):
    # verify advances the recurrent state once per draft row and captures it after each row into
    # states made ahead (no allocation while encoding); accepting row a means restoring capture a
    shape = (2, 4, 128, 64)
    hk, hv, dk, dv = shape
    rows, accepted = 4, 1
    ssm_len = hv * dv * dk
    conv_dim, kernel = 2 * hk * dk + hv * dv, 4
    conv_len = (kernel - 1) * conv_dim
    ls = sg.LinearAttentionState(state, 2, conv_len, ssm_len)
    plain = sg.LinearAttentionState(state, 2, conv_len, ssm_len)
    for layer in range(2):
        c, s = sgo.fill_normal8(conv_len, 50, layer), sgo.fill_normal8(ssm_len, 51, layer) * np.float32(0.1)
        ls.write(layer, c, s)
        plain.write(layer, c, s)
    captures = [sg.LinearAttentionState(state, 2, conv_len, ssm_len) for _ in range(rows)]
    d_w = state.upload(sgo.fill_normal8(conv_dim * kernel, 52, 0))
    d_y, d_c = state.alloc(4 * hv * dv), state.alloc(4 * conv_dim)

    def advance(target, r):
        for layer in range(2):
            ins = [sgo.fill_normal8(n, 60 + r, 10 * layer + j) * np.float32(sc) for j, (n, sc) in enumerate(
                [(hk * dk, 1.0 / dk), (hk * dk, dk ** -0.5), (hv * dv, 1.0)])]
            g = np.full(hv, 0.95, np.float32)
            beta = np.full(hv, 0.4, np.float32)
            target.encode_conv_step(layer, state.upload(sgo.fill_normal8(conv_dim, 61 + r, layer)), d_w, conv_dim, kernel, d_c)
            target.encode_gated_delta_step(layer, shape, *[state.upload(a) for a in ins + [g, beta]], d_y)

    for r in range(rows):
        advance(ls, r)
        ls.encode_capture(captures[r])
    state.sync()
    ls.restore(captures[accepted])
    for r in range(accepted + 1):
        advance(plain, r)
    state.sync()
    for layer in range(2):
        c0, s0 = ls.read(layer)
        c1, s1 = plain.read(layer)
        np.testing.assert_array_equal(c0, c1)
        np.testing.assert_array_equal(s0, s1)
    other = sg.LinearAttentionState(state, 2, conv_len, ssm_len, ssm_bf16=True)
    with pytest.raises(sg.InferError) as e:                       # capture of another shape
        ls.encode_capture(other)
    assert e.value.kind == "Shape"
    for s in captures + [ls, plain, other]:
        s.close()
