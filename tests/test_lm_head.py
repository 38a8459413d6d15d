"""Greedy epilogue (W . x then the first maximum): the CPU restatement against hand-worked cases
and the reference's tie rule (src/sampling.rs:49-62), and the CUDA kernel against it through
the C ABI."""
import numpy as np
import pytest

from oracle import sgo


@pytest.fixture(scope="module")
def gpu_state():
    import saragossa_b200 as sg
    st = sg.DecodeResidentState(0)
    yield st
    assert st.device_status() == 0
    st.close()


def _bf16_bits(a):
    bits = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def _widen(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def test_oracle_first_maximum_and_hand_case():
    w = np.array([[1, 0], [0, 2], [3, 0], [0, 2]], np.float32)
    st, idx, val = sgo.lm_head_argmax(w, [1.0, 1.0])
    assert (st, idx, val) == (0, 2, 3.0)
    # a tie keeps the first index (src/sampling.rs:57: only a strictly greater value replaces the best)
    st, idx, val = sgo.lm_head_argmax(w, [0.0, 1.0])
    assert (st, idx, val) == (0, 1, 2.0)
    # all-negative logits: the first row still counts
    st, idx, val = sgo.lm_head_argmax(-w, [1.0, 1.0])
    assert (st, idx, val) == (0, 0, -1.0)


def test_oracle_empty_vocab_is_an_error():
    st, _, _ = sgo.lm_head_argmax(np.zeros((0, 8), np.float32), np.zeros(8, np.float32))
    assert st != 0


def test_oracle_matches_numpy_argmax():
    rng = np.random.default_rng(5)
    w = rng.standard_normal((300, 64)).astype(np.float32)
    x = rng.standard_normal(64).astype(np.float32)
    st, idx, val = sgo.lm_head_argmax(w, x)
    logits = w.astype(np.float64) @ x.astype(np.float64)
    assert st == 0 and idx == int(np.argmax(logits))
    assert abs(val - logits[idx]) <= 1e-4 * max(1.0, abs(logits[idx]))


def _separated_case(rng, vocab, hidden, rows, winners, bf16):
    """Random weights with one planted row per activation row whose logit clears the rest by a margin
    far above any f32 summation-order difference."""
    w = (rng.standard_normal((vocab, hidden)) * 0.05).astype(np.float32)
    x = rng.standard_normal((rows, hidden)).astype(np.float32)
    for r, win in enumerate(winners):
        w[win] = x[r] / np.linalg.norm(x[r]) * 2.0
    if bf16:
        bits = _bf16_bits(w)
        return bits, _widen(bits), x
    return w, w, x


@pytest.mark.gpu
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("vocab,hidden", [(1, 8), (7, 64), (1000, 256), (4097, 2048), (151936, 1024)])
def test_kernel_matches_oracle(gpu_state, bf16, vocab, hidden):
    rng = np.random.default_rng(vocab * 7 + hidden)
    win = int(rng.integers(0, vocab))
    wdev, wref, x = _separated_case(rng, vocab, hidden, 1, [win], bf16)
    st, want, want_val = sgo.lm_head_argmax(wref, x[0])
    assert st == 0 and want == win
    got = gpu_state.argmax_linear_biasless(x[0], wdev)
    assert got == want


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [2, 3, 4, 5, 8])
def test_kernel_verify_rows_share_one_pass(gpu_state, rows):
    rng = np.random.default_rng(rows)
    vocab, hidden = 5000, 512
    winners = [int(v) for v in rng.integers(0, vocab, rows)]
    wdev, wref, x = _separated_case(rng, vocab, hidden, rows, winners, True)
    got = gpu_state.argmax_linear_biasless(x, wdev)
    for r in range(rows):
        st, want, _ = sgo.lm_head_argmax(wref, x[r])
        assert st == 0 and int(got[r]) == want == winners[r]


@pytest.mark.gpu
@pytest.mark.parametrize("hidden", [8, 24, 40, 136, 1000])
def test_kernel_bf16_ragged_hidden(gpu_state, hidden):
    """hidden that is not a multiple of the 32-wide chunk or of the 128-wide unrolled step."""
    rng = np.random.default_rng(hidden)
    vocab = 333
    winners = [int(v) for v in rng.integers(0, vocab, 3)]
    wdev, wref, x = _separated_case(rng, vocab, hidden, 3, winners, True)
    got = gpu_state.argmax_linear_biasless(x, wdev)
    assert [int(v) for v in got] == winners


@pytest.mark.gpu
def test_kernel_bf16_logit_is_close_and_independent_of_the_other_rows(gpu_state):
    import saragossa_b200 as sg
    rng = np.random.default_rng(9)
    vocab, hidden, rows = 3000, 2560, 8
    w = (rng.standard_normal((vocab, hidden)) * 0.02).astype(np.float32)
    bits = _bf16_bits(w)
    x = rng.standard_normal((rows, hidden)).astype(np.float32)
    d_w, d_x = gpu_state.upload(bits), gpu_state.upload(x)
    d_i, d_v = gpu_state.alloc(32), gpu_state.alloc(32)
    gpu_state.encode_lm_head_argmax(d_w, sg.KV_BF16, vocab, hidden, d_x, d_i, n_rows=rows, d_value_out=d_v)
    gpu_state.sync()
    idx8, val8 = d_i.download(np.int32, rows), d_v.download(np.float32, rows)
    logits = _widen(bits).astype(np.float64) @ x.astype(np.float64).T  # [vocab][rows]
    for r in range(rows):
        # random logits have no planted margin: accept the index if its exact logit is within the error bound of the best
        assert logits[idx8[r], r] >= logits[:, r].max() - 2e-4
        assert abs(val8[r] - logits[idx8[r], r]) <= 2e-4   # |logit| ~ 1; hi+lo activation, f32 accumulation
        d_x1 = gpu_state.upload(x[r])
        gpu_state.encode_lm_head_argmax(d_w, sg.KV_BF16, vocab, hidden, d_x1, d_i, n_rows=1, d_value_out=d_v)
        gpu_state.sync()
        assert int(d_i.download(np.int32, 1)[0]) == int(idx8[r])
        assert d_v.download(np.float32, 1)[0].tobytes() == val8[r].tobytes()   # bit for bit


@pytest.mark.gpu
def test_kernel_tie_goes_to_the_lowest_index_and_value_is_returned(gpu_state):
    import saragossa_b200 as sg
    vocab, hidden = 20000, 64
    w = np.zeros((vocab, hidden), np.float32)
    x = np.zeros(hidden, np.float32)
    x[3] = 1.0
    for row in (19999, 4321, 777, 12000):  # exactly equal logits, far apart in the grid
        w[row, 3] = 1.5
    w[5, 3] = -4.0
    st, want, want_val = sgo.lm_head_argmax(w, x)
    assert (st, want, want_val) == (0, 777, 1.5)
    d_w, d_x = gpu_state.upload(w), gpu_state.upload(x)
    d_i, d_v = gpu_state.alloc(16), gpu_state.alloc(16)
    for _ in range(3):  # the workspace is clean again after every launch
        gpu_state.encode_lm_head_argmax(d_w, sg.KV_F32, vocab, hidden, d_x, d_i, index_offset=100, d_value_out=d_v)
        gpu_state.sync()
        assert int(d_i.download(np.int32, 1)[0]) == 777 + 100
        assert float(d_v.download(np.float32, 1)[0]) == 1.5
    # all logits negative: ordering of negative floats
    w2 = -np.abs(np.random.default_rng(1).standard_normal((300, hidden)).astype(np.float32)) - 0.1
    st, want, want_val = sgo.lm_head_argmax(w2, x)
    d_w2 = gpu_state.upload(w2)
    gpu_state.encode_lm_head_argmax(d_w2, sg.KV_F32, 300, hidden, d_x, d_i, d_value_out=d_v)
    gpu_state.sync()
    assert int(d_i.download(np.int32, 1)[0]) == want
    assert float(d_v.download(np.float32, 1)[0]) == want_val


@pytest.mark.gpu
def test_kernel_rejects_bad_shapes(gpu_state):
    import saragossa_b200 as sg
    d = gpu_state.alloc(1024)
    for kw in (dict(vocab=0, hidden=8), dict(vocab=4, hidden=12), dict(vocab=4, hidden=8, n_rows=9),
               dict(vocab=4, hidden=8, n_rows=0), dict(vocab=4, hidden=16384, n_rows=4), dict(vocab=4, hidden=16384, n_rows=4, dtype=1)):
        with pytest.raises(sg.InferError):
            gpu_state.encode_lm_head_argmax(d, kw.get("dtype", sg.KV_F32), kw["vocab"], kw["hidden"], d, d,
                                            n_rows=kw.get("n_rows", 1))
    with pytest.raises(sg.InferError):
        gpu_state.encode_lm_head_argmax(d, sg.KV_U8G32, 4, 8, d, d)
