"""GPU parity tests of the warm-prefix cache and the linear-attention state: snapshot,
restore (physical copy and copy-on-write sharing), eviction under a byte budget, and the
state container, all through the C ABI."""
import numpy as np
import pytest

import saragossa_b200 as sg
from oracle import sgo

pytestmark = pytest.mark.gpu

LAYERS, Q_HEADS, KV_HEADS, HD = 3, 8, 2, 128
KV_DIM = KV_HEADS * HD


@pytest.fixture(scope="module")
def state():
    st = sg.DecodeResidentState(0)
    yield st
    assert st.device_status() == 0
    st.close()


def _rows(n, seed, stream):
    return sgo.fill_normal8(n * KV_DIM, seed, stream).reshape(n, KV_DIM)


def _fill(seq, n, seed):
    kvs, data = [], []
    for layer in range(LAYERS):
        kv = seq.layer(layer, Q_HEADS)
        k, v = _rows(n, seed, 2 * layer), _rows(n, seed, 2 * layer + 1)
        kv.seed(k, v, n)
        kvs.append(kv)
        data.append((k, v))
    return kvs, data


def _chain(root, toks, block):
    hashes, prev = [], root
    for i in range(len(toks) // block):
        prev = sg.BlockHash.chain(prev, toks[i * block:(i + 1) * block])
        hashes.append(prev)
    return hashes


@pytest.mark.parametrize("dtype", [sg.KV_BF16, sg.KV_F32, sg.KV_U8G32])
def test_snapshot_restore_copy_is_bit_exact_and_never_aliased(state, dtype):
    # snapshot + copy + restore of src/decoder/generation.rs:2834-2892: the restored sequence
    # holds the same rows, in pages of its own
    n, block = 96, 32
    pool = state.pool(LAYERS, KV_HEADS, HD, dtype, num_pages=40, max_seqs=4, max_seq_tokens=256)
    pool.shuffle_free_list(2)
    cache = sg.BlockAwarePrefixCache(block, 16, pool=pool)
    src = pool.sequence(256)
    kvs, data = _fill(src, n + 5, seed=7)
    root = sg.BlockHash.for_session("sess")
    toks = list(range(100, 100 + n + 5))
    for i, h in enumerate(_chain(root, toks, block)):
        assert cache.insert(root, h, (i + 1) * block, seq=src)
    hit = cache.match_prefix(root, toks)
    assert hit.tokens == n
    dst = pool.sequence(256)
    copied = cache.restore(hit, dst)
    assert copied == (n // 16) * pool.page_bytes
    assert not set(dst.block_table()) & set(src.block_table())          # never aliased
    for layer in range(LAYERS):
        kv = dst.layer(layer, Q_HEADS)
        assert kv.len() == n
        gk, gv = kv.gather_rows_f32()
        sk, sv = kvs[layer].gather_rows_f32(0, n)
        assert np.array_equal(gk, sk) and np.array_equal(gv, sv)         # block copy: bit-exact
        ref = sgo.ResidentKv(n, Q_HEADS, KV_HEADS, HD, dtype)
        ref.seed(data[layer][0][:n], data[layer][1][:n], n)
        assert np.array_equal(gk, ref.keys())
    # the restored sequence extends on its own pages; the source is untouched
    kv0 = dst.layer(0, Q_HEADS)
    extra_k, extra_v = _rows(3, 8, 0), _rows(3, 8, 1)
    kv0.append_batch(extra_k, extra_v)
    assert kv0.len() == n + 3 and kvs[0].len() == n + 5
    sk, _ = kvs[0].gather_rows_f32(0, n + 5)
    ref = sgo.ResidentKv(n + 5, Q_HEADS, KV_HEADS, HD, dtype)
    ref.seed(data[0][0], data[0][1], n + 5)
    assert np.array_equal(sk, ref.keys())
    q = sgo.fill_normal8(Q_HEADS * HD, 9, 0)
    ref2 = sgo.ResidentKv(n + 3, Q_HEADS, KV_HEADS, HD, dtype)
    ref2.seed(np.concatenate([data[0][0][:n], extra_k]), np.concatenate([data[0][1][:n], extra_v]), n + 3)
    _, want = ref2.attention(q)
    got = kv0.attention_decode(q)
    assert np.all(np.abs(got - want) <= 2e-2 * np.abs(want) + 1e-3)
    dst.close()
    src.close()
    cache.close()
    assert pool.free_pages == 40
    pool.close()


def test_shared_restore_copies_on_write(state):
    n, block = 64, 16
    pool = state.pool(LAYERS, KV_HEADS, HD, sg.KV_BF16, num_pages=32, max_seqs=4, max_seq_tokens=128)
    cache = sg.BlockAwarePrefixCache(block, 16, pool=pool)
    src = pool.sequence(128)
    kvs, data = _fill(src, n, seed=11)
    root = sg.BlockHash.root()
    toks = list(range(n))
    for i, h in enumerate(_chain(root, toks, block)):
        cache.insert(root, h, (i + 1) * block, seq=src)
    free = pool.free_pages
    dst = pool.sequence(128)
    assert cache.restore(cache.match_prefix(root, toks), dst, share=True) == 0
    assert pool.free_pages == free and list(dst.block_table()) == list(src.block_table())
    kv = dst.layer(1, Q_HEADS)
    kv.truncate(n - 3)                       # back into a shared page, then write: copy-on-write
    new_k, new_v = _rows(1, 12, 0), _rows(1, 12, 1)
    kv.append_row(new_k[0], new_v[0])
    assert pool.free_pages == free - 1
    assert dst.block_table()[-1] != src.block_table()[-1] and list(dst.block_table()[:-1]) == list(src.block_table()[:-1])
    sk, sv = kvs[1].gather_rows_f32()
    ref = sgo.ResidentKv(n, Q_HEADS, KV_HEADS, HD, sg.KV_BF16)
    ref.seed(data[1][0], data[1][1], n)
    assert np.array_equal(sk, ref.keys()) and np.array_equal(sv, ref.values())      # the source did not change
    gk, _ = kv.gather_rows_f32()
    assert np.array_equal(gk[:n - 3], ref.keys()[:n - 3])
    assert np.array_equal(gk[n - 3], sgo.bf16_round(new_k[0]))
    other = dst.layer(2, Q_HEADS)             # another layer of the same page came along with the copy
    ok, _ = other.gather_rows_f32()
    ref2 = sgo.ResidentKv(n, Q_HEADS, KV_HEADS, HD, sg.KV_BF16)
    ref2.seed(data[2][0], data[2][1], n)
    assert np.array_equal(ok, ref2.keys())
    dst.close()
    src.close()
    cache.close()
    assert pool.free_pages == 32
    pool.close()


def test_budget_eviction_order_and_scrub(state):
    """LRU eviction under a byte budget follows the reference's order (root-most block of a
    touched chain first, src/serve/cache.rs:131-148,196-198); freed pages are scrubbed."""
    block = 16
    pool = state.pool(LAYERS, KV_HEADS, HD, sg.KV_BF16, num_pages=48, max_seqs=6, max_seq_tokens=128)
    pool.set_scrub_on_free(True)
    budget = 7 * pool.page_bytes
    cache = sg.BlockAwarePrefixCache(block, 64, pool=pool, budget_bytes=budget)
    ref = sgo.BlockAwarePrefixCache(block, 64)
    seqs = {}
    for name in ("a", "b", "c"):
        seq = pool.sequence(128)
        _fill(seq, 64, seed=ord(name))
        seqs[name] = seq
    pins = {}
    for name in ("a", "b", "a", "c"):
        root = sg.BlockHash.for_session(name)
        toks = [ord(name) * 100 + i for i in range(64)]
        hit = cache.match_prefix(root, toks)
        want = ref.match_prefix(root, toks)
        assert (hit is None) == (want is None) and (hit is None or hit.tokens == want["tokens"])
        for i, h in enumerate(_chain(root, toks, block)):
            pages = list(seqs[name].block_table()[:i + 1])
            skip = False
            while True:   # the budget loop runs before the insert, an older duplicate still cached
                live = set(p for e in ref.entries() for p in pins[e[1]])
                if (len(live | set(pages))) * pool.page_bytes <= budget:
                    break
                if ref.evict_lru_block() is None:
                    skip = True
                    break
            pins[h] = pages
            assert cache.insert(root, h, (i + 1) * block, seq=seqs[name]) == (not skip)
            if not skip:
                ref.insert(root, h, (i + 1) * block)
            assert [e[1] for e in cache.entries()] == [e[1] for e in ref.entries()]
    assert cache.evicted() == [(s, h, t) for s, h, t, _ in ref.evicted()] and len(cache.evicted()) >= 4
    # drop the live sequences: pages only the evicted entries held are free now and were zeroed
    tables = {name: list(seq.block_table()) for name, seq in seqs.items()}
    for seq in seqs.values():
        seq.close()
    held = set(p for e in cache.entries() for p in pins[e[1]])
    assert pool.num_pages - pool.free_pages == len(held)
    fresh = pool.sequence(128)
    fresh.reserve(64)
    kv = fresh.layer(0, Q_HEADS)
    kv.truncate(64)
    gk, gv = kv.gather_rows_f32()
    assert not gk.any() and not gv.any()          # recycled pages carry no stale K/V
    fresh.close()
    cache.close()
    assert pool.free_pages == 48
    pool.close()


def test_linear_state_snapshot_restore_roundtrip(state):
    # linear_attn_state_snapshot_restore_roundtrip, src/metal_backend/tests/linear_attention.rs:11-47
    h_v, d_v, d_k, conv_k, conv_dim = 4, 8, 8, 4, 64
    conv_len, ssm_len = (conv_k - 1) * conv_dim, h_v * d_v * d_k
    conv_seed = (1.0 + np.arange(conv_len)).astype(np.float32)
    ssm_seed = (1000.0 + np.arange(ssm_len)).astype(np.float32)
    ls = sg.LinearAttentionState(state, 1, conv_len, ssm_len)
    assert ls.estimated_bytes() == (conv_len + ssm_len) * 4
    ls.write(0, conv_seed, ssm_seed)
    snap = ls.snapshot()
    state.sync()
    ls.write(0, np.zeros(conv_len), np.zeros(ssm_len))             # corrupt in place
    assert ls.read(0)[0][1] == 0.0
    ls.restore(snap)
    conv, ssm = ls.read(0)
    assert np.array_equal(conv, conv_seed) and np.array_equal(ssm, ssm_seed)      # bit for bit
    bad = sg.LinearAttentionState(state, 1, conv_len, ssm_len, ssm_bf16=True)
    with pytest.raises(sg.InferError) as e:
        ls.restore(bad)
    assert e.value.kind == "Shape"
    for x in (ls, snap, bad):
        x.close()


def test_linear_state_config3_shape_and_prefix_entry(state):
    """30 recurrent layers of 32 x 128 x 128 f32 (config 3) ride along with a prefix entry."""
    layers, ssm_len, conv_len = 30, 32 * 128 * 128, 3 * 1024
    ls = sg.LinearAttentionState(state, layers, conv_len, ssm_len)
    want = []
    for layer in range(layers):
        c = sgo.fill_normal8(conv_len, 20, 2 * layer)
        s = sgo.fill_normal8(ssm_len, 20, 2 * layer + 1)
        ls.write(layer, c, s)
        want.append((c, s))
    pool = state.pool(LAYERS, KV_HEADS, HD, sg.KV_BF16, num_pages=16, max_seqs=2, max_seq_tokens=64)
    cache = sg.BlockAwarePrefixCache(16, 8, pool=pool)
    seq = pool.sequence(64)
    _fill(seq, 32, seed=3)
    root = sg.BlockHash.root()
    toks = list(range(32))
    for i, h in enumerate(_chain(root, toks, 16)):
        cache.insert(root, h, 16 * (i + 1), seq=seq, linear_state=ls)
    assert cache.estimated_bytes() == 2 * (pool.page_bytes + ls.estimated_bytes())
    for layer in range(layers):                                     # the live state moves on
        ls.write(layer, np.zeros(conv_len), np.ones(ssm_len))
    dst = pool.sequence(64)
    copied = cache.restore(cache.match_prefix(root, toks), dst, linear_state=ls)
    assert copied >= 2 * pool.page_bytes + ls.estimated_bytes()
    for layer in (0, 13, 29):
        c, s = ls.read(layer)
        assert np.array_equal(c, want[layer][0]) and np.array_equal(s, want[layer][1])
    bf = sg.LinearAttentionState(state, 2, 0, 256, ssm_bf16=True)
    vals = sgo.fill_normal8(256, 21, 0)
    bf.write(1, np.zeros(0), vals)
    assert np.array_equal(bf.read(1)[1], sgo.bf16_round(vals)) and bf.estimated_bytes() == 2 * 256 * 2
    for x in (dst, seq):
        x.close()
    cache.close()
    pool.close()
    ls.close()
    bf.close()


def test_decoder_prefix_cache_restores_rows_and_never_aliases_them(state):
    """prefix_cache_get / _put (src/decoder/generation.rs:2998-3139) over pages: a hit gives the new
    sequence exactly the cached rows; its appends (the suffix of the prompt) copy the shared last
    page first, so the entry and the sequence that made it keep their rows bit for bit."""
    layers, q_heads, kv_heads, hd = 2, 4, 2, 64
    kv_dim = kv_heads * hd
    pool = state.pool(layers, kv_heads, hd, sg.KV_BF16, num_pages=32, max_seqs=4, max_seq_tokens=128)
    cache = sg.DecoderPrefixCache(pool, capacity=2)
    prompt = list(range(35))                      # 2 full pages + 3 rows of a third

    def rows(layer, which, p0, p1):
        return sgo.fill_normal8((p1 - p0) * kv_dim, 61, 2 * layer + which, p0 * kv_dim).reshape(p1 - p0, kv_dim)

    a = pool.sequence(128)
    kva = [a.layer(layer, q_heads) for layer in range(layers)]
    for layer, kv in enumerate(kva):
        kv.append_batch(rows(layer, 0, 0, 35), rows(layer, 1, 0, 35))
    cache.put(prompt, a)
    b = pool.sequence(128)
    longer = prompt + [100, 101, 102, 103, 104]
    assert cache.get(longer, b) == 35
    kvb = [b.layer(layer, q_heads) for layer in range(layers)]
    for layer, kv in enumerate(kvb):
        assert kv.len() == 35
        gk, gv = kv.gather_rows_f32()
        assert np.array_equal(gk, sgo.bf16_round(rows(layer, 0, 0, 35))) and np.array_equal(gv, sgo.bf16_round(rows(layer, 1, 0, 35)))
        kv.append_batch(rows(layer, 0, 35, 40), rows(layer, 1, 35, 40))       # the suffix: copies the shared page first
    cache.put(longer, b)
    for layer, kv in enumerate(kva):                                           # the first sequence goes on too
        kv.append_batch(rows(layer, 0, 50, 53), rows(layer, 1, 50, 53))
    assert list(a.block_table())[:2] == list(b.block_table())[:2]               # full pages stay shared
    assert a.block_table()[2] != b.block_table()[2]                             # the written one does not
    c = pool.sequence(128)
    assert cache.get(prompt, c) == 35                                           # the shorter entry is intact
    for layer in range(layers):
        gk, gv = c.layer(layer, q_heads).gather_rows_f32()
        assert np.array_equal(gk, sgo.bf16_round(rows(layer, 0, 0, 35))) and np.array_equal(gv, sgo.bf16_round(rows(layer, 1, 0, 35)))
        gk, gv = kvb[layer].gather_rows_f32()
        assert np.array_equal(gk, sgo.bf16_round(rows(layer, 0, 0, 40)))
        gk, gv = kva[layer].gather_rows_f32()
        assert np.array_equal(gk[35:], sgo.bf16_round(rows(layer, 0, 50, 53)))
    d = pool.sequence(128)
    assert cache.get(longer + [9], d) == 40 and cache.entries()[0] == longer
    assert cache.get([77, 1], d) == 0 and d.layer(0, q_heads).len() == 40       # a miss leaves the sequence alone
    for s_ in (a, b, c, d):
        s_.close()
    cache.close()
    assert pool.free_pages == 32
    pool.close()


def _busy(stream, torch):
    """Keeps `stream` busy for tens of milliseconds, so that what is enqueued behind it has not run
    when the host goes on."""
    with torch.cuda.stream(stream):
        x = torch.ones((4096, 4096), device="cuda", dtype=torch.float32)
        for _ in range(60):
            x = (x @ x) * 1e-4
    return x


def test_destroy_and_restore_wait_for_the_caller_stream_used_last(state):
    """An attention launch sits behind a long computation on a caller's stream. The sequence it
    reads is then (a) destroyed, with its pages handed to another sequence that overwrites them
    through the state's own stream, and (b) in a second round, overwritten by a prefix restore on
    the state's own stream. Both calls order themselves after the caller stream used last, so the
    waiting launch still sees the rows it was enqueued for."""
    import torch
    n, block = 64, 32
    pool = state.pool(1, KV_HEADS, HD, sg.KV_BF16, num_pages=8, max_seqs=4, max_seq_tokens=64)
    q = sgo.fill_normal8(Q_HEADS * HD, 31, 0)
    d_q, d_out = state.upload(q), state.alloc(4 * Q_HEADS * HD)
    side = torch.cuda.Stream()

    def reference(k, v):
        ref = sgo.ResidentKv(n, Q_HEADS, KV_HEADS, HD, sg.KV_BF16)
        ref.seed(k, v, n)
        return ref.attention(q)[1]

    # (a) destroy
    a = pool.sequence(64)
    kv = a.layer(0, Q_HEADS)
    ka, va = _rows(n, 32, 0), _rows(n, 32, 1)
    kv.seed(ka, va, n)
    keep = _busy(side, torch)
    kv.encode_attention_decode_windowed(d_q, d_out, stream=side.cuda_stream)
    a.close()                                     # must wait for the side stream
    b = pool.sequence(64)
    b2 = pool.sequence(64)                        # the pool has 8 pages: a's four are among these eight
    for s_, seed in ((b, 33), (b2, 34)):
        s_.layer(0, Q_HEADS).seed(_rows(n, seed, 0), _rows(n, seed, 1), n)
    side.synchronize()
    got = d_out.download(count=Q_HEADS * HD)
    want = reference(ka, va)
    assert np.all(np.abs(got - want) <= 2e-2 * np.abs(want) + 1e-3)
    b2.close()

    # (b) restore on the state's own stream while a launch on the side stream still has to read the sequence
    cache = sg.BlockAwarePrefixCache(block, 16, pool=pool)
    root = sg.BlockHash.for_session("s")
    toks = list(range(n))
    for i, h in enumerate(_chain(root, toks, block)):
        assert cache.insert(root, h, (i + 1) * block, seq=b)
    c = pool.sequence(64)
    kc, vc = _rows(n, 35, 0), _rows(n, 35, 1)
    kvc = c.layer(0, Q_HEADS)
    kvc.seed(kc, vc, n)
    keep2 = _busy(side, torch)
    kvc.encode_attention_decode_windowed(d_q, d_out, stream=side.cuda_stream)
    hit = cache.match_prefix(root, toks)
    assert hit.tokens == n
    cache.restore(hit, c)                         # own stream: ordered after the side stream
    side.synchronize()
    state.sync()
    got = d_out.download(count=Q_HEADS * HD)
    want = reference(kc, vc)
    assert np.all(np.abs(got - want) <= 2e-2 * np.abs(want) + 1e-3)
    # and the sequence now holds the restored rows
    gk, _ = kvc.gather_rows_f32()
    bk, _ = b.layer(0, Q_HEADS).gather_rows_f32()
    assert np.array_equal(gk, bk)
    del keep, keep2
    c.close()
    b.close()
    cache.close()
    pool.close()
