"""CPU-side checks of libsgk.so: every symbol sgk.h declares is exported, the
host-only logic (hashes, prefix-cache bookkeeping, budget, page accounting)
agrees with the oracle, and nothing computes without a GPU."""
import ctypes as C
import random
import re

import numpy as np
import pytest

import saragossa_b200 as sg
from oracle import sgo
from saragossa_b200 import _ffi


def test_library_exports_every_declared_symbol():
    protos = _ffi.parse_header()
    text = open(_ffi.HEADER).read()
    declared = set(re.findall(r"\b(sgk_[a-z0-9_]+)\s*\(", text))
    assert declared == set(protos), declared ^ set(protos)
    handle = C.CDLL(_ffi.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), name
    assert len(declared) >= 90


def test_no_cpu_fallback_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(sg.InferError) as err:
        sg.DecodeResidentState(0)
    assert err.value.kind == "Backend" and "no CPU path" in str(err.value)


def test_block_hashes_match_oracle():
    assert sg.BlockHash.root() == sgo.hash_root() == bytes(32)
    for key in (None, "", "alpha", "agent-b", "é" * 40):
        assert sg.BlockHash.for_session(key) == sgo.hash_for_session(key)
    rng = random.Random(3)
    prev = sg.BlockHash.for_session("s")
    for n in (0, 1, 2, 3, 7, 16, 256):
        toks = [rng.randrange(0, 2 ** 63) for _ in range(n)]
        got = sg.BlockHash.chain(prev, toks)
        assert got == sgo.hash_chain(prev, toks)
        prev = got


def _trace(seed, n_ops, block_tokens, capacity, per_session):
    """Random serve-like trace replayed on the oracle and on libsgk."""
    rng = random.Random(seed)
    ours = sg.BlockAwarePrefixCache(block_tokens, capacity, per_session)
    ref = sgo.BlockAwarePrefixCache(block_tokens, capacity, per_session)
    sessions = [None, "a", "b", "c"]
    prompts = [[rng.randrange(0, 5) for _ in range(rng.randrange(1, 7) * block_tokens + rng.randrange(0, block_tokens))]
               for _ in range(6)]
    for _ in range(n_ops):
        op = rng.random()
        root = sg.BlockHash.for_session(rng.choice(sessions))
        toks = rng.choice(prompts)
        if op < 0.45:
            hit, want = ours.match_prefix(root, toks), ref.match_prefix(root, toks)
            assert (hit is None) == (want is None)
            if hit is not None:
                assert (hit.tokens, hit.hash) == (want["tokens"], want["hash"])
        elif op < 0.9:
            # what prefill_prompt_state does: remember every full block of the prompt
            prev = root
            for i in range(len(toks) // block_tokens):
                prev = sg.BlockHash.chain(prev, toks[i * block_tokens:(i + 1) * block_tokens])
                if rng.random() < 0.7:
                    ours.insert(root, prev, (i + 1) * block_tokens)
                    ref.insert(root, prev, (i + 1) * block_tokens)
        else:
            got, want = ours.evict_lru_block(), ref.evict_lru_block()
            assert (got is None) == (want is None)
        assert [(s, h, t) for s, h, t in ours.entries()] == [(s, h, t) for s, h, t, _ in ref.entries()]
    assert ours.evicted() == [(s, h, t) for s, h, t, _ in ref.evicted()]
    assert len(ours) == len(ref)
    return len(ours.evicted())


@pytest.mark.parametrize("cfg", [(1, 2, 2), (2, 8, 8), (2, 5, 2), (3, 4, 1), (16, 12, 6)])
def test_prefix_cache_trace_matches_oracle(cfg):
    evicted = sum(_trace(seed, 300, *cfg) for seed in range(4))
    assert evicted > 0


def test_reference_prefix_cases_through_the_abi():
    # the ordering assertions of src/serve/cache.rs:341-466, through libsgk
    cache = sg.BlockAwarePrefixCache(1, 2, 1)
    alpha, beta = sg.BlockHash.for_session("agent-a"), sg.BlockHash.for_session("agent-b")
    beta_first = sg.BlockHash.chain(beta, [9])
    alpha_first = sg.BlockHash.chain(alpha, [1])
    alpha_second = sg.BlockHash.chain(alpha_first, [2])
    cache.insert(beta, beta_first, 1)
    cache.insert(alpha, alpha_first, 1)
    cache.insert(alpha, alpha_second, 2)
    assert [e[1] for e in cache.entries()] == [alpha_second, beta_first]
    assert cache.match_prefix(beta, [9]).hash == beta_first
    assert cache.session_block_count(alpha) == 1
    zero = sg.BlockAwarePrefixCache(1, 0)
    assert zero.insert(alpha, alpha_first, 1) is False and zero.match_prefix(alpha, [1]) is None
    assert sg.BlockAwarePrefixCache(0, 4).block_tokens() == 1     # block_tokens.max(1), cache.rs:111


def test_longest_prefix_entry_index_matches_oracle():
    entries = [[1, 2], [1, 2, 3], [1]]
    for prompt in ([1, 2, 3, 4], [1, 9], [9], [1, 2], []):
        assert sg.longest_prefix_entry_index(entries, prompt) == sgo.longest_prefix_entry_index(entries, prompt)


def test_budget_matches_oracle_guard():
    # src/memory_guard.rs:734-788
    g = sg.MemoryGuard(static_cap=900, total_memory=1200, headroom=200, device_cap=700)
    assert g.limit_bytes() == 700
    g = sg.MemoryGuard(static_cap=150)
    g.set_usage(100)
    assert g.check_allocation(50) == (150, 50)
    with pytest.raises(sg.InferError) as err:
        g.check_allocation(51)
    assert err.value.kind == "MemoryGuard"
    assert g.projection_over_limit(51) == (151, 50)
    rng = random.Random(0)
    for _ in range(200):
        caps = [rng.choice([None, rng.randrange(1, 1000)]) for _ in range(3)]
        head = rng.randrange(0, 300)
        ours = sg.MemoryGuard(static_cap=caps[0], total_memory=caps[1], headroom=head, device_cap=caps[2])
        ref = sgo.MemoryGuard(static_cap=caps[0], host_memory=caps[1], headroom=head, device_cap=caps[2])
        assert ours.limit_bytes() == ref.limit()
        cur, res, req = rng.randrange(0, 600), rng.randrange(0, 200), rng.randrange(0, 400)
        ours.set_usage(cur, res)
        ref.set(cur, res)
        assert (ours.projection_over_limit(req) is None) == ref.check_allocation(req)[0]


def test_host_only_pool_accounting_and_budget_eviction():
    """Page sharing, copy-free restore and the budget loop on a bookkeeping-only pool."""
    pool = sg.PagePool(None, layers=2, kv_heads=2, head_dim=64, dtype=sg.KV_BF16, num_pages=64, max_seqs=8,
                       max_seq_tokens=512)
    page_bytes = pool.page_bytes
    assert page_bytes == 2 * 2 * 2 * 16 * 64 * 2
    budget = 8 * page_bytes
    cache = sg.BlockAwarePrefixCache(16, 100, pool=pool, budget_bytes=budget)
    ref = sgo.BlockAwarePrefixCache(16, 100)
    pins, seqs = {}, {}
    for name in ("a", "b", "c", "b", "a", "c", "c", "a"):
        root = sg.BlockHash.for_session(name)
        if name not in seqs:
            seq = pool.sequence(512)
            seq.reserve(5 * 16)
            for layer in range(2):
                seq.layer(layer, 4).truncate(80)     # the cursors, moved the host-only way
            seqs[name] = seq
        seq = seqs[name]
        toks = [ord(name) * 1000 + i for i in range(80)]
        prev = root
        for i in range(5):
            prev = sg.BlockHash.chain(prev, toks[16 * i:16 * i + 16])
            # oracle side: the reference's loop with this build's accounting (unique pinned pages)
            pages = list(seq.block_table()[:i + 1])
            skip = False
            while True:
                # the budget loop runs before the insert, with an older duplicate of the block still
                # cached (src/serve/state.rs:627-635 before cache.rs:165-169)
                live = set(p for e in ref.entries() for p in pins[e[1]])
                fresh = len(set(pages) - live)
                if (len(live) + fresh) * page_bytes <= budget:
                    break
                if ref.evict_lru_block() is None:
                    skip = True      # cache ran empty and the block still does not fit: not remembered
                    break
            pins[prev] = pages
            inserted = cache.insert(root, prev, 16 * (i + 1), seq=seq)
            assert inserted == (not skip)
            if not skip:
                ref.insert(root, prev, 16 * (i + 1))
            assert [e[1] for e in cache.entries()] == [e[1] for e in ref.entries()]
    assert cache.evicted() == [(s, h, t) for s, h, t, _ in ref.evicted()]
    assert len(cache.evicted()) > 0 and len(cache) > 0
    # an entry pins its whole prefix, and the cache holds every page of a chain once however many
    # entries lie on it: the first page is held by the sequence and by ONE run of the cache
    root = sg.BlockHash.for_session("a")
    toks = [ord("a") * 1000 + i for i in range(80)]
    hit = cache.match_prefix(root, toks)
    assert hit is not None and hit.tokens == 80
    first = int(seqs["a"].block_table()[0])
    assert sum(1 for e in cache.entries() if e[0] == root) > 1
    holders = 1
    assert pool.refcount(first) == 1 + holders
    free_before = pool.free_pages
    other = pool.sequence(512)
    cache.restore(hit, other, share=True)
    assert pool.free_pages == free_before            # sharing takes no page
    assert list(other.block_table()) == list(seqs["a"].block_table()[:5])
    assert pool.refcount(first) == 2 + holders
    other.close()
    for seq in seqs.values():
        seq.close()
    cache.close()
    assert pool.free_pages == 64
    pool.close()


def test_large_prefix_cache_trace_matches_oracle():
    """Thousands of 16-token blocks: the hash index and the relinked list give the same hits, the
    same entry order and the same evicted keys as the reference's Vec scans, op by op."""
    rng = random.Random(11)
    block, capacity, per_session = 16, 3000, 1200
    ours = sg.BlockAwarePrefixCache(block, capacity, per_session)
    ref = sgo.BlockAwarePrefixCache(block, capacity, per_session)
    sessions = [None] + [f"s{i}" for i in range(5)]
    system = [rng.randrange(0, 50000) for _ in range(40 * block)]
    prompts = [system[:rng.randrange(8, 41) * block] + [rng.randrange(0, 50000) for _ in range(rng.randrange(1, 60) * block)]
               for _ in range(24)]
    ops = 0
    for step in range(3000):
        root = sg.BlockHash.for_session(rng.choice(sessions))
        toks = rng.choice(prompts)
        op = rng.random()
        if op < 0.5:
            hit, want = ours.match_prefix(root, toks), ref.match_prefix(root, toks)
            assert (hit is None) == (want is None)
            if hit is not None:
                assert (hit.tokens, hit.hash) == (want["tokens"], want["hash"])
                ops += hit.tokens // block        # blocks looked up and moved to the front
            ops += 1
        elif op < 0.97:
            hit = ref.match_prefix(root, toks)
            ours.match_prefix(root, toks)
            start = hit["tokens"] if hit is not None else 0
            inserted, last = ours.insert_chain(root, toks, None, from_tokens=start)
            prev = root
            for i in range(len(toks) // block):
                prev = sg.BlockHash.chain(prev, toks[i * block:(i + 1) * block])
                if (i + 1) * block > start:
                    ref.insert(root, prev, (i + 1) * block)
                    ops += 1
            assert last == prev and inserted == len(toks) // block - start // block
        else:
            for _ in range(rng.randrange(1, 40)):
                got, want = ours.evict_lru_block(), ref.evict_lru_block()
                assert (got is None) == (want is None)
                ops += 1
        if step % 50 == 0:
            assert [(s, h, t) for s, h, t in ours.entries()] == [(s, h, t) for s, h, t, _ in ref.entries()]
    assert [(s, h, t) for s, h, t in ours.entries()] == [(s, h, t) for s, h, t, _ in ref.entries()]
    assert ours.evicted() == [(s, h, t) for s, h, t, _ in ref.evicted()]
    assert ops > 50_000 and len(ours) > 2000 and len(ours.evicted()) > 1000, (ops, len(ours), len(ours.evicted()))


def test_failed_restore_leaves_the_sequence_as_it_was():
    """A physical restore that the pool cannot hold fails with MemoryGuard before anything is
    touched: the sequence keeps its pages, its block table and its cursors."""
    pool = sg.PagePool(None, layers=1, kv_heads=1, head_dim=64, dtype=sg.KV_BF16, num_pages=12, max_seqs=4,
                       max_seq_tokens=256)
    cache = sg.BlockAwarePrefixCache(16, 100, pool=pool)
    a = pool.sequence(128)
    a.reserve(6 * 16)
    a.layer(0, 1).truncate(96)
    root = sg.BlockHash.for_session("a")
    toks = list(range(96))
    assert cache.insert_chain(root, toks, a)[0] == 6
    hit = cache.match_prefix(root, toks)
    assert hit.tokens == 96
    b = pool.sequence(128)
    b.reserve(2 * 16)
    b.layer(0, 1).truncate(20)
    table_before, free_before = list(b.block_table()), pool.free_pages
    assert free_before == 4                      # 6 + 2 of 12 in use: 6 needed, 4 free + 2 of its own
    c = pool.sequence(128)
    c.reserve(16)                                # now 3 free + 2 own = 5 < 6
    with pytest.raises(sg.InferError) as e:
        cache.restore(hit, b)
    assert e.value.kind == "MemoryGuard"
    assert list(b.block_table()) == table_before and b.layer(0, 1).len() == 20
    assert pool.free_pages == 3
    c.close()
    assert cache.restore(hit, b) == 6 * pool.page_bytes    # 4 free + 2 own: fits, by giving its own pages back first
    assert b.layer(0, 1).len() == 96 and pool.free_pages == 0
    for s in (a, b):
        s.close()
    cache.close()
    assert pool.free_pages == 12
    pool.close()


def test_decoder_prefix_cache_matches_the_oracle_and_shares_pages():
    """The decoder-internal prefix cache (src/decoder/generation.rs:2998-3139) on a bookkeeping pool:
    hits, order and capacity follow the restated reference logic on a random trace; an entry holds its
    prompt's pages by reference and a restored sequence shares them."""
    rng = random.Random(5)
    ours = sg.DecoderPrefixCache(None, capacity=4)
    ref = sgo.DecoderPrefixCache(4)
    base = [[rng.randrange(0, 4) for _ in range(rng.randrange(1, 9))] for _ in range(6)]
    for _ in range(400):
        prompt = list(rng.choice(base)) + [rng.randrange(0, 4) for _ in range(rng.randrange(0, 4))]
        got = ours.get(prompt)
        if 0 < got < len(prompt):
            ours.put(prompt)                     # the caller's half of prefix_cache_get (:3019-3022)
        if got == 0 and rng.random() < 0.7:
            ours.put(prompt)                     # a cold prefill ends with a put
            want = ref.get(prompt)
            ref.put(prompt)
        else:
            want = ref.get(prompt)
        assert got == want
        assert ours.entries() == ref.entries
    assert len(ours) == 4
    zero = sg.DecoderPrefixCache(None, capacity=0)
    zero.put([1, 2, 3])
    assert len(zero) == 0 and zero.get([1, 2, 3]) == 0
    ours.close()
    zero.close()
    # pages: an entry pins ceil(n / 16) pages of its sequence; a hit shares them with the new sequence
    pool = sg.PagePool(None, layers=1, kv_heads=1, head_dim=64, dtype=sg.KV_BF16, num_pages=16, max_seqs=4,
                       max_seq_tokens=128)
    cache = sg.DecoderPrefixCache(pool, capacity=2)
    a = pool.sequence(128)
    a.reserve(40)
    a.layer(0, 1).truncate(40)
    prompt = list(range(40))
    cache.put(prompt, a)
    table = list(a.block_table())
    assert [pool.refcount(p) for p in table[:3]] == [2, 2, 2]
    b = pool.sequence(128)
    assert cache.get(prompt + [7, 8], b) == 40
    assert list(b.block_table()) == table[:3] and b.layer(0, 1).len() == 40
    assert [pool.refcount(p) for p in table[:3]] == [3, 3, 3]
    with pytest.raises(sg.InferError):
        cache.put(list(range(50)), a)            # the sequence holds 40 rows only
    a.close()
    b.close()
    assert pool.free_pages == 13                  # the entry alone still pins its three pages
    cache.close()
    assert pool.free_pages == 16
    pool.close()
