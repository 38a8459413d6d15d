"""The oracle's one-token Gated DeltaNet and depthwise-conv steps against what the reference's
own tests assert (src/linear_attention/tests.rs): the naive recurrence written term by term,
the shapes and synthetic inputs of gated_delta_matches_naive_oracle_across_lengths_and_gqa_heads,
the zero-state closed form, and invariance under any split of the sequence."""
import numpy as np
import pytest

from oracle import sgo

# The two shapes of src/linear_attention/tests.rs:305-324: (H_k, H_v, d_k, d_v).
SHAPES = [(2, 4, 8, 6), (1, 4, 128, 128)]
CHUNK_BOUNDARY_LENGTHS = [1, 15, 16, 17, 55]  # tests.rs:142


class Lcg:
    """The tests' deterministic generator: Knuth's 64-bit LCG, top 24 bits as a fraction
    (src/linear_attention/tests.rs:83-106)."""

    def __init__(self, seed):
        self.state = seed

    def fill(self, n, lo, hi):
        out = np.empty(n, np.float32)
        lo, hi = np.float32(lo), np.float32(hi)
        for i in range(n):
            self.state = (self.state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
            unit = np.float32((self.state >> 40) & 0xFFFFFF) / np.float32(16777216.0)
            out[i] = lo + (hi - lo) * unit
        return out


def gdn_inputs(shape, seq, seed):
    """synthetic_gdn_inputs (tests.rs:119-138)."""
    hk, hv, dk, dv = shape
    rng = Lcg(seed)
    qa, ka = np.float32(dk) ** np.float32(-1.0), np.float32(dk) ** np.float32(-0.5)
    return (rng.fill(seq * hk * dk, -qa, qa).reshape(seq, -1), rng.fill(seq * hk * dk, -ka, ka).reshape(seq, -1),
            rng.fill(seq * hv * dv, -1.0, 1.0).reshape(seq, -1), rng.fill(seq * hv, 0.9, 0.999).reshape(seq, -1),
            rng.fill(seq * hv, 0.1, 0.9).reshape(seq, -1))


def naive_f64(q, k, v, g, beta, shape, state):
    """The module's equations in float64 on whole matrices: an independent formulation."""
    hk, hv, dk, dv = shape
    rep = hv // hk
    S = state.astype(np.float64).reshape(hv, dv, dk).copy()
    ys = []
    for t in range(q.shape[0]):
        y = np.empty((hv, dv))
        for h in range(hv):
            kt = k[t].reshape(hk, dk)[h // rep].astype(np.float64)
            qt = q[t].reshape(hk, dk)[h // rep].astype(np.float64)
            S[h] *= float(g[t, h])
            delta = float(beta[t, h]) * (v[t].reshape(hv, dv)[h].astype(np.float64) - S[h] @ kt)
            S[h] += np.outer(delta, kt)
            y[h] = S[h] @ qt
        ys.append(y.ravel())
    return np.array(ys), S.ravel()


def run_steps(q, k, v, g, beta, shape, state):
    hk, hv, dk, dv = shape
    ys = []
    for t in range(q.shape[0]):
        st, y, state = sgo.gated_delta_step(q[t], k[t], v[t], g[t], beta[t], hk, hv, dk, dv, state)
        assert st == sgo.OK
        ys.append(y)
    return np.array(ys), state


@pytest.mark.parametrize("ci", [0, 1])
@pytest.mark.parametrize("li", [0, 2, 3])
def test_gated_delta_matches_the_equations(ci, li):
    shape, seq = SHAPES[ci], CHUNK_BOUNDARY_LENGTHS[li]
    hk, hv, dk, dv = shape
    q, k, v, g, beta = gdn_inputs(shape, seq, 0x5EED0000 + ci * 16 + li)
    ys, state = run_steps(q, k, v, g, beta, shape, np.zeros(hv * dv * dk, np.float32))
    ref_y, ref_s = naive_f64(q, k, v, g, beta, shape, np.zeros(hv * dv * dk))
    np.testing.assert_allclose(ys, ref_y, rtol=0, atol=2e-6)
    np.testing.assert_allclose(state, ref_s, rtol=0, atol=2e-6)


def test_zero_state_closed_form_and_gqa_head_mapping():
    # from S = 0: kv = 0, delta = beta*v, S = delta k^T, y = delta (k.q); value head h reads
    # key head h // repeat (src/linear_attention.rs:940-945)
    shape = (2, 4, 8, 6)
    hk, hv, dk, dv = shape
    q, k, v, g, beta = gdn_inputs(shape, 1, 99)
    st, y, s = sgo.gated_delta_step(q[0], k[0], v[0], g[0], beta[0], hk, hv, dk, dv, np.zeros(hv * dv * dk, np.float32))
    assert st == sgo.OK
    for h in range(hv):
        kh = k[0].reshape(hk, dk)[h // 2]
        qh = q[0].reshape(hk, dk)[h // 2]
        delta = (v[0].reshape(hv, dv)[h] - np.float32(0.0)) * beta[0, h]
        np.testing.assert_array_equal(s.reshape(hv, dv, dk)[h], np.float32(0.0) + delta[:, None] * kh[None, :])
        np.testing.assert_allclose(y.reshape(hv, dv)[h], delta * np.dot(kh.astype(np.float64), qh), atol=1e-7)


def test_any_split_of_the_sequence_gives_the_same_bits():
    # gated_delta_invariant_par_decoupage_en_chunks (tests.rs:379-445): the state carries
    # everything, so stopping and resuming anywhere changes nothing
    shape = (2, 4, 8, 6)
    hk, hv, dk, dv = shape
    q, k, v, g, beta = gdn_inputs(shape, 23, 7)
    full_y, full_s = run_steps(q, k, v, g, beta, shape, np.zeros(hv * dv * dk, np.float32))
    state, ys = np.zeros(hv * dv * dk, np.float32), []
    for lo, hi in [(0, 5), (5, 6), (6, 23)]:
        y, state = run_steps(q[lo:hi], k[lo:hi], v[lo:hi], g[lo:hi], beta[lo:hi], shape, state.copy())
        ys.append(y)
    np.testing.assert_array_equal(np.concatenate(ys), full_y)
    np.testing.assert_array_equal(state, full_s)


def test_gated_delta_rejects_incompatible_heads_and_state_length():
    # linear_attention_rejects_incompatible_heads (tests.rs:184-198); ensure_ssm_cache (:994-1024)
    z = np.zeros(64, np.float32)
    st, _, _ = sgo.gated_delta_step(z[:24], z[:24], z[:12], z[:2], z[:2], 3, 2, 8, 6, np.zeros(2 * 6 * 8, np.float32))
    assert st == sgo.ERR_DIMENSION
    st, _, _ = sgo.gated_delta_step(z[:8], z[:8], z[:12], z[:2], z[:2], 1, 2, 8, 6, np.zeros(17, np.float32))
    assert st == sgo.ERR_DIMENSION


def test_conv_step_is_the_causal_convolution_of_the_whole_sequence():
    # depthwise_causal_conv (src/linear_attention.rs:802-852): output t = sum_k w[c][k] * x[t-(K-1)+k][c]
    # with zeros before the start; the history afterwards is the last K-1 inputs
    conv_dim, kernel, seq = 10, 4, 9
    x = sgo.fill_normal8(seq * conv_dim, 3, 0).reshape(seq, conv_dim)
    w = sgo.fill_normal8(conv_dim * kernel, 3, 1).reshape(conv_dim, kernel)
    hist = np.zeros((kernel - 1) * conv_dim, np.float32)
    outs = []
    for t in range(seq):
        st, o, hist = sgo.depthwise_conv_step(x[t], w, kernel, hist)
        assert st == sgo.OK
        outs.append(o)
    padded = np.concatenate([np.zeros((kernel - 1, conv_dim), np.float32), x])
    for t in range(seq):
        acc = np.zeros(conv_dim, np.float32)
        for kk in range(kernel):
            acc = acc + padded[t + kk] * w[:, kk]
        np.testing.assert_array_equal(outs[t], acc)
    np.testing.assert_array_equal(hist.reshape(kernel - 1, conv_dim), x[-(kernel - 1):])
    st, _, _ = sgo.depthwise_conv_step(x[0], w, kernel, np.zeros(5, np.float32))
    assert st == sgo.ERR_DIMENSION


def test_decode_step_helpers_known_answers():
    """silu's known values (src/activation.rs:62-69), key_scale, sigmoid, softplus's linear branch and
    a unit RMS norm worked by hand: the pieces the one-launch decode step is checked against."""
    out = sgo.silu(np.array([-1.0, 0.0, 1.0], np.float32))
    assert abs(out[0] - -0.26894143) < 1e-6 and out[1] == 0.0 and abs(out[2] - 0.7310586) < 1e-6
    assert sgo.key_scale(128, False) == np.float32(128.0) ** np.float32(-0.5)
    assert abs(float(sgo.key_scale(128, True)) - 1.0 / 128.0) < 1e-9
    assert abs(float(sgo.sigmoid(np.array([0.0], np.float32))[0]) - 0.5) < 1e-7
    # softplus(25) = 25 (linear branch), softplus(0) = ln 2; decay = exp(-exp(a_log) * softplus)
    g = sgo.compute_decay(np.array([25.0, 0.0], np.float32), np.array([0.0, 0.0], np.float32), np.array([0.0, 0.0], np.float32))
    assert abs(float(g[0]) - np.exp(-25.0)) < 1e-12 and abs(float(g[1]) - 0.5) < 1e-6
    x = np.array([3.0, 4.0, 0.0, 0.0], np.float32)          # mean square 6.25 -> rms 2.5
    n = sgo.rms_norm_heads_unit(x, 1, 4, eps=0.0)
    assert np.allclose(n, [1.2, 1.6, 0.0, 0.0], atol=1e-7)
    two = sgo.rms_norm_heads_unit(np.concatenate([x, 2 * x]), 2, 4, eps=0.0)
    assert np.allclose(two[:4], two[4:], atol=1e-7)          # a head's scale does not matter


def test_decode_step_is_the_composition_of_its_pieces():
    hk, hv, d = 2, 4, 128
    conv_dim, kernel = 2 * hk * d + hv * d, 4
    qkv = sgo.fill_normal8(conv_dim, 3, 0)
    w = sgo.fill_normal8(conv_dim * kernel, 3, 1) * np.float32(0.5)
    hist = sgo.fill_normal8((kernel - 1) * conv_dim, 3, 2)
    ssm = sgo.fill_normal8(hv * d * d, 3, 3) * np.float32(0.1)
    bi, gi = sgo.fill_normal8(hv, 3, 4), sgo.fill_normal8(hv, 3, 5)
    a_log, dt = sgo.fill_normal8(hv, 3, 6) * np.float32(0.3), sgo.fill_normal8(hv, 3, 7) * np.float32(0.3)
    st, out, new_hist, new_ssm, parts = sgo.linear_decode_step(qkv, w, kernel, hist, bi, gi, a_log, dt, hk, hv, d, d, ssm)
    assert st == 0 and np.isfinite(out).all()
    # the history slid by one token and q, k have unit RMS times their scales
    assert np.array_equal(new_hist.reshape(kernel - 1, conv_dim)[-1], qkv)
    assert np.array_equal(new_hist.reshape(kernel - 1, conv_dim)[:-1], hist.reshape(kernel - 1, conv_dim)[1:])
    q = parts["q"].reshape(hk, d)
    assert np.allclose(np.sqrt((q.astype(np.float64) ** 2).mean(axis=1)), 1.0 / 128.0, rtol=1e-4)
    k = parts["k"].reshape(hk, d)
    assert np.allclose(np.sqrt((k.astype(np.float64) ** 2).mean(axis=1)), 128.0 ** -0.5, rtol=1e-4)
    assert ((parts["g"] > 0) & (parts["g"] < 1)).all() and ((parts["beta"] > 0) & (parts["beta"] < 1)).all()
