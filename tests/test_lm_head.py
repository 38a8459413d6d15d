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
def test_kernel_bf16_large_vocabulary_whole_rounds_and_left_over_tiles(gpu_state):
    """A vocabulary of two whole rounds of tiles per warp plus left-over tiles and a ragged last
    tile, at a hidden size where eight activation rows get half the blocks of one row (one block
    per SM instead of two): planted maxima in the whole rounds, among the left-over tiles and in
    the last tile are found, and a row's logit has the same bits alone and among eight rows."""
    import torch
    import saragossa_b200 as sg
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    widest = sms * 2 * 8
    vocab, hidden, rows = 16 * (2 * widest + 37) + 3, 4096, 8
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    w = (torch.randn(vocab, hidden, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    x = torch.randn(rows, hidden, device=dev, generator=gen)
    planted = [vocab - 1, 16 * 2 * widest + 5, 7, 16 * widest + 3, vocab - 30, 12345, 16 * 2 * widest - 1, 16 * (2 * widest + 36)]
    for r, row in enumerate(planted):
        x[r] += w[row].float() * 40.0
    logits = x.double() @ w.double().T                                  # [rows][vocab]
    want = torch.argmax(logits, dim=1).cpu().numpy()
    assert list(want) == planted

    class P:
        def __init__(self, t):
            self.ptr = t.data_ptr()

    idx, val = torch.zeros(8, dtype=torch.int32, device=dev), torch.zeros(8, dtype=torch.float32, device=dev)
    got = {}
    for n in (1, 8):
        gpu_state.encode_lm_head_argmax(P(w), sg.KV_BF16, vocab, hidden, P(x), P(idx), n_rows=n, d_value_out=P(val))
        gpu_state.sync()
        torch.cuda.synchronize()
        i, v = idx.cpu().numpy()[:n], val.cpu().numpy()[:n]
        for r in range(n):
            assert int(i[r]) == planted[r]
            exact = float(logits[r, planted[r]].item())
            assert abs(float(v[r]) - exact) <= 2e-4 * max(1.0, abs(exact))
        got[n] = v.copy()
    assert got[1][0].tobytes() == got[8][0].tobytes()


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


# ---- token feed: embedding lookup by a device index, and the submission window -------------------
def test_oracle_embed_gather_known_answers():
    # embedding_gather_from_index_applies_gemma_scale (src/metal_backend/tests/buffers_core.rs:64-89)
    table = np.array([[1.0, -2.0, 3.0, -4.0], [0.5, 1.5, -2.5, 4.5]], np.float32)
    assert sgo.embed_gather(table, 1, 3.0).tolist() == [1.5, 4.5, -7.5, 13.5]
    # embedding_gather_recast_is_opt_in_and_bf16_exact (:91-133)
    row = np.array([[1.001, -2.003, 3.007, -4.015]], np.float32)
    assert sgo.embed_gather(row, 0).tobytes() == row[0].tobytes()
    assert sgo.embed_gather(row, 0, 1.0, True).tobytes() == _widen(_bf16_bits(row[0])).tobytes()
    assert sgo.embed_gather(row, 1) is None   # outside the table: nothing written


@pytest.mark.gpu
def test_embedding_from_device_index_matches_oracle(gpu_state):
    import saragossa_b200 as sg
    table = np.array([[1.0, -2.0, 3.0, -4.0], [0.5, 1.5, -2.5, 4.5]], np.float32)
    d_t, d_i, d_o = gpu_state.upload(table), gpu_state.upload(np.array([1], np.int32)), gpu_state.alloc(16)
    gpu_state.encode_embedding_from_index(d_t, sg.KV_F32, 2, 4, d_i, d_o, embedding_scale=3.0)
    gpu_state.sync()
    assert d_o.download(np.float32, 4).tolist() == [1.5, 4.5, -7.5, 13.5]
    row = np.array([[1.001, -2.003, 3.007, -4.015]], np.float32)
    d_r, d_z = gpu_state.upload(row), gpu_state.upload(np.array([0], np.int32))
    for recast in (False, True):
        gpu_state.encode_embedding_from_index(d_r, sg.KV_F32, 1, 4, d_z, d_o, recast_bf16=recast)
        gpu_state.sync()
        assert d_o.download(np.float32, 4).tobytes() == sgo.embed_gather(row, 0, 1.0, recast).tobytes()
    # an index outside the table writes nothing (and does not fault)
    before = d_o.download(np.float32, 4).copy()
    for bad in (1, -1, 2**31 - 1):
        d_b = gpu_state.upload(np.array([bad], np.int32))
        gpu_state.encode_embedding_from_index(d_r, sg.KV_F32, 1, 4, d_b, d_o)
        gpu_state.sync()
        assert d_o.download(np.float32, 4).tobytes() == before.tobytes()
    # bf16 table, larger row
    rng = np.random.default_rng(3)
    big = rng.standard_normal((50, 1000)).astype(np.float32)
    bits = _bf16_bits(big)
    d_bt, d_bo = gpu_state.upload(bits), gpu_state.alloc(4000)
    d_bi = gpu_state.upload(np.array([37], np.int32))
    gpu_state.encode_embedding_from_index(d_bt, sg.KV_BF16, 50, 1000, d_bi, d_bo, embedding_scale=0.25)
    gpu_state.sync()
    assert d_bo.download(np.float32, 1000).tobytes() == sgo.embed_gather(_widen(bits), 37, 0.25).tobytes()


def _toy_model(seed, vocab=600, hidden=64):
    """A closed token loop: next = argmax(W . (E[token] * scale)). W's rows are planted so that the chain
    is a fixed permutation with wide margins."""
    rng = np.random.default_rng(seed)
    emb = rng.standard_normal((vocab, hidden)).astype(np.float32)
    perm = rng.permutation(vocab)
    w = (rng.standard_normal((vocab, hidden)) * 0.02).astype(np.float32)
    for tok in range(vocab):
        w[perm[tok]] += emb[tok] / np.linalg.norm(emb[tok]) * 3.0
    return emb, w, perm


def _oracle_chain(emb, w, first, n, scale):
    out, tok = [], first
    for _ in range(n):
        st, tok, _ = sgo.lm_head_argmax(w, sgo.embed_gather(emb, tok, scale))
        assert st == 0
        out.append(tok)
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("depth", [1, 4])
def test_token_window_keeps_the_token_on_the_device(gpu_state, depth):
    """The decode loop of src/decoder/resident/decode.rs:114-173 on a toy model: up to `depth` tokens are
    enqueued before the oldest is read back; token n+1 reads token n's index from the device ring."""
    import saragossa_b200 as sg
    emb, w, perm = _toy_model(21)
    vocab, hidden = emb.shape
    first, n, scale = 5, 23, 1.5
    want = _oracle_chain(emb, w, first, n, scale)
    assert len(set(want)) > 10   # the chain really moves
    d_e, d_w = gpu_state.upload(emb), gpu_state.upload(w)
    d_x = gpu_state.alloc(4 * hidden)
    d_first = gpu_state.upload(np.array([first], np.int32))
    win = gpu_state.token_window(depth)
    assert win.depth == depth and win.previous_slot() is None
    got, enq = [], 0
    while len(got) < n:
        while enq < n and win.inflight < depth:
            src = win.previous_slot() or d_first
            gpu_state.encode_embedding_from_index(d_e, sg.KV_F32, vocab, hidden, src, d_x, embedding_scale=scale)
            gpu_state.encode_lm_head_argmax(d_w, sg.KV_F32, vocab, hidden, d_x, win.output_slot())
            win.submit()
            enq += 1
        got.append(win.pop())
    assert got == want
    assert win.inflight == 0 and win.enqueued == n
    with pytest.raises(sg.InferError):
        win.pop()   # nothing in flight
    win.close()


@pytest.mark.gpu
def test_token_window_full_and_stop_token_drain(gpu_state):
    import saragossa_b200 as sg
    emb, w, perm = _toy_model(22)
    vocab, hidden = emb.shape
    want = _oracle_chain(emb, w, 9, 12, 1.0)
    stop = want[5]
    d_e, d_w, d_x = gpu_state.upload(emb), gpu_state.upload(w), gpu_state.alloc(4 * hidden)
    d_first = gpu_state.upload(np.array([9], np.int32))
    win = gpu_state.token_window(4)
    got, enq, stopped = [], 0, False
    while not stopped:
        while enq < 12 and win.inflight < win.depth:
            src = win.previous_slot() or d_first
            gpu_state.encode_embedding_from_index(d_e, sg.KV_F32, vocab, hidden, src, d_x)
            gpu_state.encode_lm_head_argmax(d_w, sg.KV_F32, vocab, hidden, d_x, win.output_slot())
            win.submit()
            enq += 1
        assert win.inflight == 4 and win.output_slot() is None   # full: no slot to write
        with pytest.raises(sg.InferError) as err:
            win.submit()
        assert err.value.kind == "Dimension"
        tok = win.pop()
        if tok == stop:
            stopped = True
        else:
            got.append(tok)
    assert got == want[:5]
    assert win.inflight == 3   # tokens enqueued past the stop token are still running
    win.drain()
    assert win.inflight == 0
    assert gpu_state.device_status() == 0
    win.close()


@pytest.mark.gpu
@pytest.mark.parametrize("depth", [1, 4])
def test_whole_token_is_one_graph_submission(gpu_state, depth):
    """sgk_token_capture: embedding lookup by the previous token's index, every layer's fused
    append + attention and the greedy epilogue into the window's ring are ONE graph per ring slot,
    and a token is ONE submission (src/decoder/resident/decode.rs:183-458, one command buffer per
    token). The token chain must be the oracle's, the layers must have appended a row per token,
    and their outputs must be what the same step gives outside the graph."""
    import saragossa_b200 as sg
    emb, w, perm = _toy_model(23)
    vocab, hidden = emb.shape
    first, n, scale = 7, 19, 1.25
    want = _oracle_chain(emb, w, first, n, scale)
    q_heads, kv_heads, hd, layers, n0 = 4, 2, 128, 3, 70
    kv_dim, q_dim = kv_heads * hd, q_heads * hd
    outs = []
    for mode in ("graph", "plain"):
        pool = gpu_state.pool(layers, kv_heads, hd, sg.KV_BF16, num_pages=16, max_seqs=1, max_seq_tokens=160)
        seq = pool.sequence(n0 + n + 8)
        kvs = [seq.layer(layer, q_heads) for layer in range(layers)]
        for layer, kv in enumerate(kvs):
            kv.seed(sgo.fill_normal8(n0 * kv_dim, 51, 2 * layer).reshape(n0, kv_dim),
                    sgo.fill_normal8(n0 * kv_dim, 51, 2 * layer + 1).reshape(n0, kv_dim), n0)
        batches = [sg.Batch(gpu_state, [kv]) for kv in kvs]
        step = sg.Step(gpu_state, batches)
        d_k = gpu_state.upload(sgo.fill_normal8(layers * kv_dim, 52, 0))
        d_v = gpu_state.upload(sgo.fill_normal8(layers * kv_dim, 52, 1))
        d_q = gpu_state.upload(sgo.fill_normal8(layers * q_dim, 52, 2))
        d_out = gpu_state.alloc(4 * layers * q_dim)
        if mode == "graph":
            d_e, d_w, d_x = gpu_state.upload(emb), gpu_state.upload(w), gpu_state.alloc(4 * hidden)
            win = gpu_state.token_window(depth)
            launches0 = step.launches()
            step.token_capture(win, d_e, sg.KV_F32, vocab, hidden, d_x, d_w, sg.KV_F32, d_x, d_k, d_v, d_q, d_out,
                               embedding_scale=scale)
            assert all(kv.len() == n0 for kv in kvs)          # a capture runs nothing
            step.token_seed(first)
            got, enq = [], 0
            while len(got) < n:
                while enq < n and win.inflight < depth:
                    step.token_submit()
                    enq += 1
                if enq < n:
                    with pytest.raises(sg.InferError):
                        step.token_submit()                    # the window is full
                got.append(win.pop())
            assert got == want
            assert step.launches() - launches0 == n * (layers + 2)   # embed + layers + epilogue per token
            win.close()
        else:
            for _ in range(n):
                step.enqueue(d_k, d_v, d_q, d_out)
        gpu_state.sync()
        assert all(kv.len() == n0 + n for kv in kvs)
        outs.append((d_out.download().copy(), [kv.gather_rows_f32(n0 - 1, n + 1) for kv in kvs]))
        step.close()
        for b in batches:
            b.close()
        seq.close()
        pool.close()
    assert np.array_equal(outs[0][0], outs[1][0])
    for a, b in zip(outs[0][1], outs[1][1]):
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    assert gpu_state.device_status() == 0


def _affine_weight(vocab, hidden, bits, group, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 1 << bits, size=(vocab, hidden), dtype=np.uint32)
    groups = hidden // group
    scales = _bf16_bits((rng.uniform(0.5, 1.5, size=(vocab, groups)) * (0.02 / (1 << bits))).astype(np.float32))
    biases = _bf16_bits((rng.normal(0, 0.01, size=(vocab, groups))).astype(np.float32))
    return sgo.affine_pack(codes, bits), scales, biases


def test_oracle_affine_dequantize_known_answers():
    """The unpacking order of src/quantization.rs:208-228 (LSB first) and value = code * scale + bias."""
    packed = np.array([[0x76543210, 0xFEDCBA98]], np.uint32)                   # 16 four-bit codes 0..15
    one, two = _bf16_bits(np.array([1.0], np.float32)), _bf16_bits(np.array([2.0], np.float32))
    w = sgo.affine_dequantize(packed, np.repeat(two, 1), np.repeat(one, 1), 4, 16, 1, 16)
    assert np.array_equal(w[0], 2.0 * np.arange(16, dtype=np.float32) + 1.0)
    packed8 = np.array([[0x04030201, 0xFF070605]], np.uint32)
    w8 = sgo.affine_dequantize(packed8, np.repeat(one, 1), np.repeat(two, 1), 8, 8, 1, 8)
    assert np.array_equal(w8[0], np.array([1, 2, 3, 4, 5, 6, 7, 255], np.float32) + 2.0)
    codes = np.arange(64, dtype=np.uint32).reshape(2, 32) % 16
    assert np.array_equal(sgo.affine_dequantize(sgo.affine_pack(codes, 4), np.repeat(one, 2), np.repeat(_bf16_bits(np.zeros(1, np.float32)), 2),
                                                4, 32, 2, 32), codes.astype(np.float32))


def test_oracle_affine_dequantize_replays_the_reference_known_answers():
    """The reference's own dequantisation cases (src/quantization.rs:386-418): an 8-bit weight of two
    rows in groups of 2 with scale 1/255, and a 4-bit row in groups of 4 with scales (1/15, 2) and
    biases (0, -1); words packed LSB first (pack_lanes, :538-543); tolerance 1e-6 (:560-565)."""
    pack = lambda values, bits: np.uint32(sum(int(v) << (i * bits) for i, v in enumerate(values)))
    packed = np.array([[pack([255, 0, 0, 0], 8)], [pack([0, 255, 0, 0], 8)]], np.uint32)
    scales = np.full((2, 2), 1.0 / 255.0, np.float32)
    dense = sgo.affine_dequantize(packed, scales, np.zeros((2, 2), np.float32), 8, 2, 2, 4)
    assert np.all(np.abs(dense.ravel() - np.array([1, 0, 0, 0, 0, 1, 0, 0], np.float32)) <= 1e-6)
    packed4 = np.array([[pack([15, 0, 7, 8, 1, 2, 3, 4], 4)]], np.uint32)
    dense4 = sgo.affine_dequantize(packed4, np.array([[1.0 / 15.0, 2.0]], np.float32), np.array([[0.0, -1.0]], np.float32),
                                   4, 4, 1, 8)
    want = np.array([1.0, 0.0, 7.0 / 15.0, 8.0 / 15.0, 1.0, 3.0, 5.0, 7.0], np.float32)
    assert np.all(np.abs(dense4.ravel() - want) <= 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("bits,group", [(4, 64), (8, 64), (4, 128), (8, 128)])
@pytest.mark.parametrize("rows", [1, 3, 8])
def test_affine_lm_head_matches_oracle(gpu_state, bits, group, rows):
    """Greedy epilogue over an affine-quantised weight: the index is the oracle's (argmax over the
    dequantised weight, first maximum), the winning logit is within 2e-4 of the f64 value, planted
    maxima are found, and a row's answer does not depend on the rows that share the pass."""
    vocab, hidden = 5003, 1280
    packed, scales, biases = _affine_weight(vocab, hidden, bits, group, 70 + bits + group)
    w = sgo.affine_dequantize(packed, scales, biases, bits, group, vocab, hidden)
    x = sgo.fill_normal8(rows * hidden, 71, bits).reshape(rows, hidden)
    # push one vocabulary row per activation row towards the top: x gets that row's deviation from the mean row
    mean = w.mean(axis=0)
    for r in range(rows):
        x[r] += (w[(977 * (r + 1)) % vocab] - mean) * np.float32(400.0)
    d_w = gpu_state.upload_affine(packed, scales, biases, bits, group)
    d_x = gpu_state.upload(x)
    d_idx, d_val = gpu_state.alloc(4 * 8), gpu_state.alloc(4 * 8)
    gpu_state.encode_lm_head_argmax_affine(d_w, vocab, hidden, d_x, d_idx, n_rows=rows, d_value_out=d_val)
    gpu_state.sync()
    idx, val = d_idx.download(np.int32, rows), d_val.download(np.float32, rows)
    logits = w.astype(np.float64) @ x.astype(np.float64).T
    for r in range(rows):
        st, want, _ = sgo.lm_head_argmax(w, x[r])
        assert st == 0 and int(idx[r]) == want
        if group == 64:
            assert want == (977 * (r + 1)) % vocab          # the planted row wins where the groups are fine enough
        assert abs(float(val[r]) - logits[want, r]) <= 2e-4 * max(1.0, abs(logits[want, r]))
    # one row alone gives the same bits as the same row among others
    if rows > 1:
        gpu_state.encode_lm_head_argmax_affine(d_w, vocab, hidden, d_x, d_idx, n_rows=1, d_value_out=d_val)
        gpu_state.sync()
        assert d_idx.download(np.int32, 1)[0] == idx[0]


@pytest.mark.gpu
@pytest.mark.parametrize("bits,group", [(4, 64), (8, 64), (4, 128), (8, 128)])
def test_affine_lm_head_large_vocabulary_same_answer_from_every_kernel(gpu_state, bits, group):
    """A vocabulary of several whole rounds of tiles per warp plus left-over tiles and a last tile
    of fewer than 16 rows: index and logit are the oracle's, and row 0 gets the same logit bits
    alone, among three rows (hi and lo halves of the activation in one product) and among eight
    rows (a product each)."""
    import torch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    vocab, hidden = 16 * (sms * 8 * 2 + 29) + 5, 1024
    packed, scales, biases = _affine_weight(vocab, hidden, bits, group, 40 + bits + group)
    w = sgo.affine_dequantize(packed, scales, biases, bits, group, vocab, hidden)
    x = sgo.fill_normal8(8 * hidden, 72, bits).reshape(8, hidden)
    mean = w.mean(axis=0)
    planted = [vocab - 3, 16 * sms * 8 * 2 + 7, 5, 16 * sms * 8 + 1, 977, 4242, vocab - 40, 16 * sms * 8 * 2 - 1]
    for r in range(8):
        x[r] += (w[planted[r]] - mean) * np.float32(400.0)
    d_w = gpu_state.upload_affine(packed, scales, biases, bits, group)
    d_x = gpu_state.upload(x)
    d_idx, d_val = gpu_state.alloc(4 * 8), gpu_state.alloc(4 * 8)
    logits = w.astype(np.float64) @ x.astype(np.float64).T
    want = logits.argmax(axis=0)
    got = {}
    for rows in (1, 3, 8):
        gpu_state.encode_lm_head_argmax_affine(d_w, vocab, hidden, d_x, d_idx, n_rows=rows, d_value_out=d_val)
        gpu_state.sync()
        idx, val = d_idx.download(np.int32, rows), d_val.download(np.float32, rows)
        for r in range(rows):
            assert int(idx[r]) == int(want[r])
            assert abs(float(val[r]) - logits[want[r], r]) <= 2e-4 * max(1.0, abs(logits[want[r], r]))
        got[rows] = val.copy()
    assert got[1][0].tobytes() == got[3][0].tobytes() == got[8][0].tobytes()
    assert got[3][:3].tobytes() == got[8][:3].tobytes()
    assert gpu_state.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [4, 8])
def test_affine_embedding_lookup_is_the_dequantised_row(gpu_state, bits):
    vocab, hidden, group = 301, 256, 64
    packed, scales, biases = _affine_weight(vocab, hidden, bits, group, 90 + bits)
    w = sgo.affine_dequantize(packed, scales, biases, bits, group, vocab, hidden)
    d_t = gpu_state.upload_affine(packed, scales, biases, bits, group)
    d_out = gpu_state.alloc(4 * hidden)
    for token, scale in ((0, 1.0), (300, 1.5), (123, 0.25)):
        d_i = gpu_state.upload(np.array([token], np.int32))
        gpu_state.encode_embedding_from_index_affine(d_t, vocab, hidden, d_i, d_out, embedding_scale=scale)
        gpu_state.sync()
        assert np.array_equal(d_out.download(), w[token] * np.float32(scale))
    d_out.upload(np.full(hidden, 7.0, np.float32))
    d_i = gpu_state.upload(np.array([vocab], np.int32))                    # outside the table: nothing is written
    gpu_state.encode_embedding_from_index_affine(d_t, vocab, hidden, d_i, d_out)
    gpu_state.sync()
    assert np.array_equal(d_out.download(), np.full(hidden, 7.0, np.float32))
    with pytest.raises(Exception):
        bad = gpu_state.upload_affine(packed, scales, biases, 6, group)
        gpu_state.encode_embedding_from_index_affine(bad, vocab, hidden, d_i, d_out)
