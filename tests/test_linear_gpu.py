"""GPU parity of the one-token Gated DeltaNet and depthwise-conv steps on the linear-attention
state, through the C ABI, against the oracle. Tolerances are the reference's for its own Metal
kernels against its CPU path: 1e-5 for f32 state and output, 5e-4 / 2e-4 for output / state with a
bf16 state (or one bf16 rounding step, where the stored value is large enough for a step to exceed 2e-4) (src/metal_backend/tests/linear_attention.rs:200-201,322-330). The conv step keeps the
CPU's summation order and is bit-exact."""
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


def _inputs(shape, seed, t):
    hk, hv, dk, dv = shape
    q = sgo.fill_normal8(hk * dk, seed, 5 * t) / np.float32(dk)
    k = sgo.fill_normal8(hk * dk, seed, 5 * t + 1) / np.float32(np.sqrt(dk))
    v = sgo.fill_normal8(hv * dv, seed, 5 * t + 2)
    u = sgo.fill_normal8(2 * hv, seed, 5 * t + 3)
    g = (np.float32(0.95) + np.float32(0.01) * np.clip(u[:hv], -4, 4)).astype(np.float32)
    beta = (np.float32(0.5) + np.float32(0.1) * np.clip(u[hv:], -3.9, 3.9)).astype(np.float32)
    return q, k, v, g, beta


@pytest.mark.parametrize("shape", [(2, 4, 8, 6), (1, 4, 128, 128), (16, 32, 128, 128), (2, 6, 96, 40), (1, 2, 256, 16)])
@pytest.mark.parametrize("ssm_bf16", [False, True])
def test_gated_delta_steps_match_the_oracle(state, shape, ssm_bf16):
    hk, hv, dk, dv = shape
    layers, layer, steps = 2, 1, 6
    ssm_len = hv * dv * dk
    ls = sg.LinearAttentionState(state, layers, 0, ssm_len, ssm_bf16=ssm_bf16)
    ref = sgo.fill_normal8(ssm_len, 11, 0) * np.float32(0.1)
    if ssm_bf16:
        ref = sgo.bf16_round(ref)
    other = sgo.fill_normal8(ssm_len, 11, 1)
    if ssm_bf16:
        other = sgo.bf16_round(other)
    ls.write(layer, np.zeros(0, np.float32), ref)
    ls.write(0, np.zeros(0, np.float32), other)
    d_out = state.alloc(4 * hv * dv)
    y_tol, s_tol = (5e-4, 2e-4) if ssm_bf16 else (1e-5, 1e-5)
    for t in range(steps):
        q, k, v, g, beta = _inputs(shape, 23, t)
        bufs = [state.upload(a) for a in (q, k, v, g, beta)]
        ls.encode_gated_delta_step(layer, shape, *bufs, d_out)
        st, y_ref, ref = sgo.gated_delta_step(q, k, v, g, beta, hk, hv, dk, dv, ref)
        assert st == sgo.OK
        if ssm_bf16:
            ref = sgo.bf16_round(ref)
        state.sync()
        np.testing.assert_allclose(d_out.download(count=hv * dv), y_ref, rtol=0, atol=y_tol)
        _, got = ls.read(layer)
        if ssm_bf16:
            # stored values agree to the reference's tolerance, or sit one bf16 step apart where
            # the last bit of a sum moved the rounding (a step is 2^-8 relative at most)
            diff = np.abs(got - ref)
            bad = np.nonzero(diff > np.maximum(s_tol, np.abs(ref) * 2.0 ** -7))[0]
            assert bad.size == 0, (t, bad[:8], got[bad[:8]], ref[bad[:8]])
            assert np.mean(got != ref) < 0.02
            ref = got  # follow the device so the next step compares one update, not drift
        else:
            np.testing.assert_allclose(got, ref, rtol=0, atol=s_tol)
    _, untouched = ls.read(0)
    np.testing.assert_array_equal(untouched, other)
    ls.close()


def test_gated_delta_rejects_what_the_reference_rejects(state):
    ls = sg.LinearAttentionState(state, 1, 0, 4 * 6 * 8)
    z = state.alloc(4096)
    with pytest.raises(sg.InferError) as e:  # value heads not a multiple of key heads
        ls.encode_gated_delta_step(0, (3, 4, 8, 6), z, z, z, z, z, z)
    assert e.value.kind == "Dimension"
    with pytest.raises(sg.InferError) as e:  # state length does not match the shape
        ls.encode_gated_delta_step(0, (2, 4, 8, 7), z, z, z, z, z, z)
    assert e.value.kind == "Dimension"
    with pytest.raises(sg.InferError) as e:
        ls.encode_gated_delta_step(1, (2, 4, 8, 6), z, z, z, z, z, z)
    assert e.value.kind == "Dimension"
    with pytest.raises(sg.InferError) as e:
        ls.encode_conv_step(0, z, z, 16, 4, z)  # no conv history of that size
    assert e.value.kind == "Dimension"
    ls.close()


@pytest.mark.parametrize("conv_dim,kernel", [(10, 4), (8192, 4), (777, 2), (64, 1)])
def test_conv_steps_are_bit_exact_and_slide_the_history(state, conv_dim, kernel):
    layers, layer, steps = 2, 0, 7
    conv_len = (kernel - 1) * conv_dim
    ls = sg.LinearAttentionState(state, layers, conv_len, 8)
    hist = sgo.fill_normal8(conv_len, 5, 0)
    ls.write(layer, hist, np.zeros(8, np.float32))
    w = sgo.fill_normal8(conv_dim * kernel, 5, 1)
    d_w, d_out = state.upload(w), state.alloc(4 * conv_dim)
    for t in range(steps):
        x = sgo.fill_normal8(conv_dim, 6, t)
        ls.encode_conv_step(layer, state.upload(x), d_w, conv_dim, kernel, d_out)
        st, o_ref, hist = sgo.depthwise_conv_step(x, w, kernel, hist)
        assert st == sgo.OK
        state.sync()
        np.testing.assert_array_equal(d_out.download(count=conv_dim), o_ref)
        got, _ = ls.read(layer)
        np.testing.assert_array_equal(got, hist)
    ls.close()


def test_recurrent_state_survives_a_prefix_snapshot_between_steps(state):
    # the warm-prefix flow on a hybrid model: advance, snapshot, advance, restore, advance again:
    # the replay from the snapshot reproduces the first continuation bit for bit
    shape = (2, 4, 128, 64)
    hk, hv, dk, dv = shape
    conv_dim, kernel = 2 * hk * dk + hv * dv, 4
    ls = sg.LinearAttentionState(state, 1, (kernel - 1) * conv_dim, hv * dv * dk)
    d_out, d_cout = state.alloc(4 * hv * dv), state.alloc(4 * conv_dim)
    d_w = state.upload(sgo.fill_normal8(conv_dim * kernel, 9, 9))

    def advance(t):
        q, k, v, g, beta = _inputs(shape, 31, t)
        ls.encode_conv_step(0, state.upload(sgo.fill_normal8(conv_dim, 32, t)), d_w, conv_dim, kernel, d_cout)
        ls.encode_gated_delta_step(0, shape, *[state.upload(a) for a in (q, k, v, g, beta)], d_out)
        state.sync()
        return d_out.download(count=hv * dv), d_cout.download(count=conv_dim)

    for t in range(3):
        advance(t)
    snap = ls.snapshot()
    first = [advance(t) for t in range(3, 6)]
    end_conv, end_ssm = ls.read(0)
    ls.restore(snap)
    again = [advance(t) for t in range(3, 6)]
    for (y0, c0), (y1, c1) in zip(first, again):
        np.testing.assert_array_equal(y0, y1)
        np.testing.assert_array_equal(c0, c1)
    conv2, ssm2 = ls.read(0)
    np.testing.assert_array_equal(conv2, end_conv)
    np.testing.assert_array_equal(ssm2, end_ssm)
    snap.close()
    ls.close()


@pytest.mark.parametrize("ssm_bf16", [False, True])
def test_batched_gated_delta_equals_one_launch_per_sequence(state, ssm_bf16):
    # the batch launch (four rows per warp at this size) and the single-sequence launch (one row
    # per warp) do the same arithmetic per row: identical bits per sequence
    shape, n = (16, 32, 128, 128), 5
    hk, hv, dk, dv = shape
    ssm_len = hv * dv * dk
    solo = [sg.LinearAttentionState(state, 1, 0, ssm_len, ssm_bf16=ssm_bf16) for _ in range(n)]
    both = [sg.LinearAttentionState(state, 1, 0, ssm_len, ssm_bf16=ssm_bf16) for _ in range(n)]
    inits = []
    for i in range(n):
        init = sgo.fill_normal8(ssm_len, 40, i) * np.float32(0.1)
        inits.append(sgo.bf16_round(init) if ssm_bf16 else init)
        solo[i].write(0, np.zeros(0, np.float32), init)
        both[i].write(0, np.zeros(0, np.float32), init)
    ins = [_inputs(shape, 41 + i, 0) for i in range(n)]
    stacked = [state.upload(np.stack([ins[i][j] for i in range(n)])) for j in range(5)]
    d_out = state.alloc(4 * n * hv * dv)
    sg.encode_gated_delta_step_batch(both, 0, shape, *stacked, d_out)
    state.sync()
    y_batch = d_out.download(count=n * hv * dv).reshape(n, -1)
    d_one = state.alloc(4 * hv * dv)
    for i in range(n):
        solo[i].encode_gated_delta_step(0, shape, *[state.upload(a) for a in ins[i]], d_one)
        state.sync()
        np.testing.assert_array_equal(y_batch[i], d_one.download(count=hv * dv))
        np.testing.assert_array_equal(both[i].read(0)[1], solo[i].read(0)[1])
        st, y_ref, _ = sgo.gated_delta_step(*ins[i], hk, hv, dk, dv, inits[i])
        assert st == sgo.OK
        np.testing.assert_allclose(y_batch[i], y_ref, rtol=0, atol=5e-4 if ssm_bf16 else 1e-5)
    with pytest.raises(sg.InferError) as e:
        sg.encode_gated_delta_step_batch(both * 13, 0, shape, *stacked, d_out)  # 65 states
    assert e.value.kind == "Config"
    for s in solo + both:
        s.close()


@pytest.mark.parametrize("shape", [(2, 4, 8, 6), (1, 4, 128, 128), (2, 6, 96, 40)])
@pytest.mark.parametrize("ssm_bf16", [False, True])
def test_gated_delta_sequence_equals_the_step_loop(state, shape, ssm_bf16):
    # linear_attn_gated_delta_seq_dk128_matches_step_loop (src/metal_backend/tests/linear_attention.rs:206-403):
    # the prompt form keeps the state in registers over the tokens. f32 state: the same arithmetic
    # as the step form, identical bits; bf16 state: rounded once at the end instead of per token,
    # inside the reference's 5e-4 / 2e-4. Both against the oracle's token loop.
    hk, hv, dk, dv = shape
    tokens = 17
    ssm_len = hv * dv * dk
    init = sgo.fill_normal8(ssm_len, 70, 0) * np.float32(0.1)
    if ssm_bf16:
        init = sgo.bf16_round(init)
    seq_state = sg.LinearAttentionState(state, 1, 0, ssm_len, ssm_bf16=ssm_bf16)
    loop_state = sg.LinearAttentionState(state, 1, 0, ssm_len, ssm_bf16=ssm_bf16)
    seq_state.write(0, np.zeros(0, np.float32), init)
    loop_state.write(0, np.zeros(0, np.float32), init)
    ins = [_inputs(shape, 71, t) for t in range(tokens)]
    stacked = [state.upload(np.stack([ins[t][j] for t in range(tokens)])) for j in range(5)]
    d_seq = state.alloc(4 * tokens * hv * dv)
    seq_state.encode_gated_delta_seq(0, shape, *stacked, tokens, d_seq)
    d_one = state.alloc(4 * hv * dv)
    ref, ys_loop, ys_ref = init.copy(), [], []
    for t in range(tokens):
        loop_state.encode_gated_delta_step(0, shape, *[state.upload(a) for a in ins[t]], d_one)
        state.sync()
        ys_loop.append(d_one.download(count=hv * dv))
        st, y, ref = sgo.gated_delta_step(*ins[t], hk, hv, dk, dv, ref)      # f32 over the whole sequence
        assert st == sgo.OK
        ys_ref.append(y)
    state.sync()
    ys_seq = d_seq.download(count=tokens * hv * dv).reshape(tokens, -1)
    _, s_seq = seq_state.read(0)
    _, s_loop = loop_state.read(0)
    if not ssm_bf16:
        np.testing.assert_array_equal(ys_seq, np.array(ys_loop))
        np.testing.assert_array_equal(s_seq, s_loop)
        np.testing.assert_allclose(ys_seq, np.array(ys_ref), rtol=0, atol=1e-5)
        np.testing.assert_allclose(s_seq, ref, rtol=0, atol=1e-5)
    else:
        np.testing.assert_allclose(ys_seq, np.array(ys_ref), rtol=0, atol=5e-4)
        assert np.all(np.abs(s_seq - sgo.bf16_round(ref)) <= np.maximum(2e-4, np.abs(ref) * 2.0 ** -7))
        np.testing.assert_allclose(ys_seq, np.array(ys_loop), rtol=0, atol=5e-3)   # per-token rounding drifts
    seq_state.close()
    loop_state.close()


@pytest.mark.parametrize("conv_dim,kernel", [(8192, 4), (100, 2), (33, 7)])
def test_conv_sequence_equals_the_step_loop_bit_for_bit(state, conv_dim, kernel):
    tokens = 21
    conv_len = (kernel - 1) * conv_dim
    a = sg.LinearAttentionState(state, 1, conv_len, 8)
    b = sg.LinearAttentionState(state, 1, conv_len, 8)
    hist = sgo.fill_normal8(conv_len, 80, 0)
    a.write(0, hist, np.zeros(8, np.float32))
    b.write(0, hist, np.zeros(8, np.float32))
    w = sgo.fill_normal8(conv_dim * kernel, 80, 1)
    x = sgo.fill_normal8(tokens * conv_dim, 80, 2).reshape(tokens, conv_dim)
    d_w = state.upload(w)
    d_all, d_one = state.alloc(4 * tokens * conv_dim), state.alloc(4 * conv_dim)
    a.encode_conv_seq(0, state.upload(x), d_w, conv_dim, kernel, tokens, d_all)
    state.sync()
    got = d_all.download(count=tokens * conv_dim).reshape(tokens, conv_dim)
    ref_hist = hist
    for t in range(tokens):
        b.encode_conv_step(0, state.upload(x[t]), d_w, conv_dim, kernel, d_one)
        st, o_ref, ref_hist = sgo.depthwise_conv_step(x[t], w, kernel, ref_hist)
        assert st == sgo.OK
        state.sync()
        np.testing.assert_array_equal(got[t], d_one.download(count=conv_dim))
        np.testing.assert_array_equal(got[t], o_ref)
    np.testing.assert_array_equal(a.read(0)[0], b.read(0)[0])
    np.testing.assert_array_equal(a.read(0)[0], ref_hist)
    with pytest.raises(sg.InferError) as e:
        a.encode_conv_seq(0, d_all, d_w, conv_dim, 17, 1, d_one)
    assert e.value.kind in ("Config", "Dimension")
    a.close()
    b.close()


@pytest.mark.parametrize("graph", [False, True])
def test_token_chain_of_recurrent_layers_equals_plain_enqueues(state, graph):
    """Inside a token chain the conv and gated-delta launches of consecutive layers overlap their
    neighbours (each reads its own layer's state before it waits for the launch before it, its
    inputs after). Outputs, recurrent states and conv histories must be what the same enqueues
    give outside a chain, bit for bit, in stream mode and captured into a CUDA graph."""
    import torch
    shape = (2, 4, 128, 64)
    hk, hv, dk, dv = shape
    layers, kernel, tokens = 3, 4, 3
    conv_dim = 2 * hk * dk + hv * dv
    ssm_len = hv * dv * dk
    w = [sgo.fill_normal8(conv_dim * kernel, 41, layer) * np.float32(0.5) for layer in range(layers)]
    results = []
    for chained in (False, True):
        ls = sg.LinearAttentionState(state, layers, (kernel - 1) * conv_dim, ssm_len)
        for layer in range(layers):
            ls.write(layer, sgo.fill_normal8((kernel - 1) * conv_dim, 42, layer),
                     sgo.fill_normal8(ssm_len, 43, layer) * np.float32(0.1))
        d_w = [state.upload(x) for x in w]
        d_x, d_in = state.alloc(4 * conv_dim * layers), [state.alloc(4 * n * layers) for n in (hk * dk, hk * dk, hv * dv, hv, hv)]
        d_c, d_y = state.alloc(4 * conv_dim * layers), state.alloc(4 * hv * dv * layers)
        stream = torch.cuda.Stream()

        def token():
            if chained:
                state.chain_begin(stream.cuda_stream)
            for layer in range(layers):
                ls.encode_conv_step(layer, _Off(d_x, 4 * conv_dim * layer), d_w[layer], conv_dim, kernel,
                                    _Off(d_c, 4 * conv_dim * layer), stream=stream.cuda_stream)
                ls.encode_gated_delta_step(layer, shape, *[_Off(b, 4 * n * layer) for b, n in zip(d_in, (hk * dk, hk * dk, hv * dv, hv, hv))],
                                           _Off(d_y, 4 * hv * dv * layer), stream=stream.cuda_stream)
            if chained:
                state.chain_end()

        g = None
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                token()
            # the capture ran nothing: the states are still the written ones
        got = []
        for t in range(tokens):
            d_x.upload(sgo.fill_normal8(conv_dim * layers, 44, t))
            for i, (b, n) in enumerate(zip(d_in, (hk * dk, hk * dk, hv * dv, hv, hv))):
                vals = sgo.fill_normal8(n * layers, 45, 5 * t + i)
                if i >= 3:
                    vals = (np.float32(0.9) + np.float32(0.01) * np.clip(vals, -4, 4)).astype(np.float32)
                elif i < 2:
                    vals = vals / np.float32(dk if i == 0 else np.sqrt(dk))
                b.upload(vals)
            state.sync()
            if g is not None:
                with torch.cuda.stream(stream):
                    g.replay()
            else:
                token()
            stream.synchronize()
            got.append((d_c.download(count=conv_dim * layers).copy(), d_y.download(count=hv * dv * layers).copy()))
        states = [ls.read(layer) for layer in range(layers)]
        results.append((got, states))
        ls.close()
    plain, chain = results
    for (c0, y0), (c1, y1) in zip(plain[0], chain[0]):
        assert np.array_equal(c0, c1) and np.array_equal(y0, y1)
    for (h0, s0), (h1, s1) in zip(plain[1], chain[1]):
        assert np.array_equal(h0, h1) and np.array_equal(s0, s1)


class _Off:
    """A device buffer seen from a byte offset."""

    def __init__(self, buf, offset):
        self.ptr = buf.ptr + offset


@pytest.mark.parametrize("shape,kernel", [((2, 4, 128, 128), 4), ((16, 32, 128, 128), 4), ((1, 2, 128, 128), 2),
                                          ((2, 2, 128, 128), 7)])
@pytest.mark.parametrize("ssm_bf16", [False, True])
def test_one_launch_decode_step_matches_the_cpu_order(state, shape, kernel, ssm_bf16):
    """conv + SiLU + unit RMS norm + gates + gated delta of a token in ONE launch against the
    composition of the oracle's pieces (src/linear_attention.rs:313-342), over several tokens so
    that the history (shifted by whichever block of a key head arrives last) and the state carry
    over: the history is bit-exact, output and state are inside the reference's bounds for its own
    fused dispatches (1e-5 with an f32 state; 5e-4 / one bf16 step with a bf16 state)."""
    hk, hv, dk, dv = shape
    conv_dim, ssm_len = 2 * hk * dk + hv * dv, hv * dv * dk
    w = sgo.fill_normal8(conv_dim * kernel, 61, 0) * np.float32(0.5)
    a_log = sgo.fill_normal8(hv, 61, 1) * np.float32(0.3)
    dt_bias = sgo.fill_normal8(hv, 61, 2) * np.float32(0.3)
    hist = sgo.fill_normal8((kernel - 1) * conv_dim, 61, 3)
    ssm = sgo.fill_normal8(ssm_len, 61, 4) * np.float32(0.1)
    ls = sg.LinearAttentionState(state, 2, (kernel - 1) * conv_dim, ssm_len, ssm_bf16=ssm_bf16)
    ls.write(1, hist, ssm)
    if ssm_bf16:
        ssm = sgo.bf16_round(ssm)
    d_w, d_al, d_dt = state.upload(w), state.upload(a_log), state.upload(dt_bias)
    d_out = state.alloc(4 * hv * dv)
    for t in range(4):
        qkv = sgo.fill_normal8(conv_dim, 62, 3 * t)
        bi = sgo.fill_normal8(hv, 62, 3 * t + 1)
        gi = sgo.fill_normal8(hv, 62, 3 * t + 2) + (np.float32(24.0) if t == 2 else np.float32(0.0))   # softplus's linear branch
        st, want, hist, new_ssm, _ = sgo.linear_decode_step(qkv, w, kernel, hist, bi, gi, a_log, dt_bias, hk, hv, dk, dv, ssm)
        assert st == 0
        ls.encode_decode_step(1, shape, state.upload(qkv), d_w, kernel, state.upload(bi), state.upload(gi), d_al, d_dt, d_out)
        state.sync()
        got = d_out.download(count=hv * dv)
        got_hist, got_ssm = ls.read(1)
        assert np.array_equal(got_hist, hist)
        if ssm_bf16:
            assert np.all(np.abs(got - want) <= 5e-4)
            step = np.maximum(2e-4, np.abs(new_ssm) * np.float32(2.0 ** -7))
            assert np.all(np.abs(got_ssm - new_ssm) <= step)
            ssm = got_ssm          # the stored state is what the next token starts from
        else:
            assert np.all(np.abs(got - want) <= 1e-5)
            assert np.all(np.abs(got_ssm - new_ssm) <= 1e-5)
            ssm = new_ssm
    # layer 0 was never touched
    h0, s0 = ls.read(0)
    assert not h0.any() and not s0.any()
    with pytest.raises(sg.InferError) as e:
        ls.encode_decode_step(1, (hk, hv, 64, 128), state.upload(qkv), d_w, kernel, state.upload(bi), state.upload(gi), d_al, d_dt, d_out)
    assert e.value.kind == "Config"
    ls.close()


@pytest.mark.parametrize("graph", [False, True])
def test_token_chain_of_one_launch_decode_steps_equals_plain_enqueues(state, graph):
    """The one-launch decode steps of consecutive layers as a token chain: each launch reads its own
    layer's state rows, taps and conv history before it waits for the launch before it. Outputs,
    states and histories (shifted by whichever block arrives last) equal the plain enqueues bit for
    bit over several tokens, in stream mode and as a CUDA graph."""
    import torch
    shape = (2, 4, 128, 128)
    hk, hv, dk, dv = shape
    layers, kernel, tokens = 4, 4, 3
    conv_dim, ssm_len = 2 * hk * dk + hv * dv, hv * dv * dk
    w = [sgo.fill_normal8(conv_dim * kernel, 51, layer) * np.float32(0.5) for layer in range(layers)]
    results = []
    for chained in (False, True):
        ls = sg.LinearAttentionState(state, layers, (kernel - 1) * conv_dim, ssm_len)
        for layer in range(layers):
            ls.write(layer, sgo.fill_normal8((kernel - 1) * conv_dim, 52, layer),
                     sgo.fill_normal8(ssm_len, 53, layer) * np.float32(0.1))
        d_w = [state.upload(x) for x in w]
        d_x = state.alloc(4 * conv_dim * layers)
        d_gates = [state.alloc(4 * hv * layers) for _ in range(4)]      # beta_input, gate_input, a_log, dt_bias
        d_y = state.alloc(4 * hv * dv * layers)
        stream = torch.cuda.Stream()

        def token():
            if chained:
                state.chain_begin(stream.cuda_stream)
            for layer in range(layers):
                ls.encode_decode_step(layer, shape, _Off(d_x, 4 * conv_dim * layer), d_w[layer], kernel,
                                      *[_Off(b, 4 * hv * layer) for b in d_gates], _Off(d_y, 4 * hv * dv * layer),
                                      stream=stream.cuda_stream)
            if chained:
                state.chain_end()

        g = None
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                token()
        got = []
        for t in range(tokens):
            d_x.upload(sgo.fill_normal8(conv_dim * layers, 54, t))
            for i, b in enumerate(d_gates):
                b.upload(sgo.fill_normal8(hv * layers, 55, 4 * t + i) * np.float32(0.5))
            state.sync()
            if g is not None:
                with torch.cuda.stream(stream):
                    g.replay()
            else:
                token()
            stream.synchronize()
            got.append(d_y.download(count=hv * dv * layers).copy())
        results.append((got, [ls.read(layer) for layer in range(layers)]))
        ls.close()
    plain, chain = results
    for y0, y1 in zip(plain[0], chain[0]):
        assert np.isfinite(y0).all() and np.array_equal(y0, y1)
    for (h0, s0), (h1, s1) in zip(plain[1], chain[1]):
        assert np.array_equal(h0, h1) and np.array_equal(s0, s1)
