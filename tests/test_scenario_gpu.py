"""Scenario-level parity on the GPU, at sizes the oracle finishes in seconds:
* the multi-turn warm-prefix workload (config 4 shape family): sessions picked by a Zipf
  draw, restore of the matched blocks, append of new tokens, decode, re-insert, LRU eviction
  under a byte budget; every restored cache must hold exactly the rows the oracle holds and
  the evicted keys must come out in the reference's order;
* box-style serving with sliding-window and global layers (config 5 shape family): pages
  wholly before the window are released while decoding, outputs stay equal to the oracle."""
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


def _row(session, layer, which, pos, kv_dim):
    # content of row `pos` of a session: a function of (session, layer, K|V, position) only
    return sgo.fill_normal8(kv_dim, 100 + session, 2 * layer + which, pos * kv_dim)


def _rows(session, layer, which, p0, p1, kv_dim):
    return sgo.fill_normal8((p1 - p0) * kv_dim, 100 + session, 2 * layer + which, p0 * kv_dim).reshape(p1 - p0, kv_dim)


def test_multi_turn_prefix_cache_under_budget(state):
    layers, q_heads, kv_heads, hd, block = 3, 8, 2, 128, 16
    kv_dim = kv_heads * hd
    n_sessions, turns = 6, 40
    pool = state.pool(layers, kv_heads, hd, sg.KV_BF16, num_pages=160, max_seqs=4, max_seq_tokens=1024)
    pool.shuffle_free_list(4)
    budget = 40 * pool.page_bytes
    cache = sg.BlockAwarePrefixCache(block, 10_000, pool=pool, budget_bytes=budget)
    ref = sgo.BlockAwarePrefixCache(block, 10_000)
    pins = {}
    rng = np.random.default_rng(1)
    lengths = {s: int(rng.integers(40, 160)) for s in range(n_sessions)}          # history so far
    weights = 1.0 / np.arange(1, n_sessions + 1) ** 1.1                            # Zipf s = 1.1
    weights /= weights.sum()
    reused_total = 0
    for turn in range(turns):
        s = int(rng.choice(n_sessions, p=weights))
        root = sg.BlockHash.for_session(f"session-{s}")
        new_len = lengths[s] + int(rng.integers(8, 48))
        toks = [s * 100_000 + i for i in range(new_len)]
        hit = cache.match_prefix(root, toks)
        want = ref.match_prefix(root, toks)
        assert (hit is None) == (want is None)
        seq = pool.sequence(1024)
        reused = 0
        if hit is not None:
            assert hit.tokens == want["tokens"] and hit.hash == want["hash"]
            copied = cache.restore(hit, seq)                       # physical copy: never aliased
            assert copied == hit.tokens // 16 * pool.page_bytes
            reused = hit.tokens
        reused_total += reused
        kvs = [seq.layer(layer, q_heads) for layer in range(layers)]
        for layer, kv in enumerate(kvs):                             # the rest of the prompt is "prefilled"
            assert kv.len() == reused
            kv.append_batch(_rows(s, layer, 0, reused, new_len, kv_dim), _rows(s, layer, 1, reused, new_len, kv_dim))
        # the cache must now hold exactly the session's rows, restored part included
        layer = turn % layers
        gk, gv = kvs[layer].gather_rows_f32()
        assert np.array_equal(gk, sgo.bf16_round(_rows(s, layer, 0, 0, new_len, kv_dim)))
        assert np.array_equal(gv, sgo.bf16_round(_rows(s, layer, 1, 0, new_len, kv_dim)))
        # a few decode steps, checked against the oracle on one layer
        oracle_kv = sgo.ResidentKv(new_len + 4, q_heads, kv_heads, hd, sg.KV_BF16)
        oracle_kv.seed(_rows(s, layer, 0, 0, new_len, kv_dim), _rows(s, layer, 1, 0, new_len, kv_dim), new_len)
        for step in range(2):
            pos = new_len + step
            for l2, kv in enumerate(kvs):
                kv.append_row(_row(s, l2, 0, pos, kv_dim), _row(s, l2, 1, pos, kv_dim))
            oracle_kv.append_row(_row(s, layer, 0, pos, kv_dim), _row(s, layer, 1, pos, kv_dim))
            q = sgo.fill_normal8(q_heads * hd, 7, turn, step)
            _, want_out = oracle_kv.attention(q, threads=4)
            got = kvs[layer].attention_decode(q)
            assert np.all(np.abs(got - want_out) <= 2e-2 * np.abs(want_out) + 1e-3)
        new_len += 2
        toks = [s * 100_000 + i for i in range(new_len)]
        # remember every full block that is new (the serve loop, src/serve/state.rs:596-603)
        prev = root
        for i in range(new_len // block):
            prev = sg.BlockHash.chain(prev, toks[i * block:(i + 1) * block])
            if (i + 1) * block <= reused:
                continue
            pages = list(seq.block_table()[:i + 1])
            skip = False
            while True:                                               # oracle side of the budget loop, which
                # runs before the insert: an older duplicate of the block is still cached then
                live = set(p for e in ref.entries() for p in pins[e[1]])
                if len(live | set(pages)) * pool.page_bytes <= budget:
                    break
                if ref.evict_lru_block() is None:
                    skip = True
                    break
            pins[prev] = pages
            assert cache.insert(root, prev, (i + 1) * block, seq=seq) == (not skip)
            if not skip:
                ref.insert(root, prev, (i + 1) * block)
        assert [e[1] for e in cache.entries()] == [e[1] for e in ref.entries()]
        lengths[s] = new_len
        seq.close()
    assert cache.evicted() == [(a, b, c) for a, b, c, _ in ref.evicted()]
    assert len(cache.evicted()) > 10 and reused_total > 500          # eviction and reuse both happened
    cache.close()
    assert pool.free_pages == 160
    pool.close()


def test_sliding_and_global_layers_with_page_release(state):
    """Layers alternate 5 sliding : 1 global (global iff (i+1) % 6 == 0, src/decoder.rs:890-898);
    sliding layers live in their own pool and give back pages that fell out of the window."""
    q_heads, kv_heads, hd, window = 8, 4, 256, 64
    kv_dim, q_dim = kv_heads * hd, q_heads * hd
    n_layers = 6
    sliding_layers = [i for i in range(n_layers) if (i + 1) % 6 != 0]
    global_layers = [i for i in range(n_layers) if (i + 1) % 6 == 0]
    lens = [200, 70, 333]
    steps = 40
    pool_s = state.pool(len(sliding_layers), kv_heads, hd, sg.KV_BF16, 3 * 24 + 8, 4, 512)
    pool_g = state.pool(len(global_layers), kv_heads, hd, sg.KV_BF16, 3 * 26 + 8, 4, 512)
    seqs_s = [pool_s.sequence(512) for _ in lens]
    seqs_g = [pool_g.sequence(512) for _ in lens]
    refs = {}
    kv_of = {}
    for b, n in enumerate(lens):
        for layer in range(n_layers):
            if layer in sliding_layers:
                kv = seqs_s[b].layer(sliding_layers.index(layer), q_heads)
            else:
                kv = seqs_g[b].layer(global_layers.index(layer), q_heads)
            k, v = _rows(b, layer, 0, 0, n, kv_dim), _rows(b, layer, 1, 0, n, kv_dim)
            kv.seed(k, v, n)
            r = sgo.ResidentKv(n + steps, q_heads, kv_heads, hd, sg.KV_BF16)
            r.seed(k, v, n)
            refs[b, layer], kv_of[b, layer] = r, kv
    batches = {layer: sg.Batch(state, [kv_of[b, layer] for b in range(len(lens))]) for layer in range(n_layers)}
    B = len(lens)
    d_k, d_v, d_q, d_out = (state.alloc(B * kv_dim * 4), state.alloc(B * kv_dim * 4), state.alloc(B * q_dim * 4),
                            state.alloc(B * q_dim * 4))
    used_before = pool_s.num_pages - pool_s.free_pages
    for t in range(steps):
        for layer in range(n_layers):
            k_new = np.stack([_row(b, layer, 0, lens[b] + t, kv_dim) for b in range(B)])
            v_new = np.stack([_row(b, layer, 1, lens[b] + t, kv_dim) for b in range(B)])
            q = sgo.fill_normal8(B * q_dim, 9, layer, t * B * q_dim).reshape(B, q_dim)
            d_k.upload(k_new), d_v.upload(v_new), d_q.upload(q)
            sw = window if layer in sliding_layers else 0
            batches[layer].enqueue_step(d_k, d_v, d_q, d_out, sliding_window=sw)
            state.sync()
            out = d_out.download().reshape(B, q_dim)
            for b in range(B):
                r = refs[b, layer]
                r.append_row(k_new[b], v_new[b])
                ws = max(r.len() - window, 0) if sw else 0          # len.saturating_sub(window)
                _, want = r.attention(q[b], window_start=ws, threads=4)
                assert np.all(np.abs(out[b] - want) <= 2e-2 * np.abs(want) + 1e-3), (t, layer, b)
        for b in range(B):                                           # rows before the window are never read again
            seqs_s[b].release_before(max(lens[b] + t + 1 - window, 0))
    held = pool_s.num_pages - pool_s.free_pages
    assert held <= B * (window // 16 + 2) < used_before              # only the windows stay resident
    assert pool_g.num_pages - pool_g.free_pages == sum((n + steps + 15) // 16 for n in lens)
    for b in batches.values():
        b.close()
    for s in seqs_s + seqs_g:
        s.close()
    pool_s.close()
    pool_g.close()
