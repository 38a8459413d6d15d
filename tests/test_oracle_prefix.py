"""Pins the oracle's bookkeeping half (hash chain, LRU prefix cache, budget,
linear-state container) against the reference's own unit tests."""
import hashlib
import struct

import numpy as np

from oracle import sgo


def test_sha256_fips_vectors_and_hashlib():
    # FIPS 180-4 examples (the reference tests never check a digest value: parity unpinned there)
    assert sgo.sha256(b"abc").hex() == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    assert sgo.sha256(b"").hex() == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    m = b"abcdbcdecdefdefgefghfghighijhijkijkljklmklmnlmnomnopnopq"
    assert sgo.sha256(m).hex() == "248d6a61d20638b8e5c026930c3e6039a33ce45964ff2167f6ecedd419db06c1"
    rng = np.random.default_rng(1)
    for n in (1, 55, 56, 63, 64, 65, 119, 120, 1000):
        data = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        assert sgo.sha256(data) == hashlib.sha256(data).digest()


def test_chain_is_sha256_of_prev_and_le_u64_tokens():
    # src/serve/cache.rs:37-46
    root = sgo.hash_root()
    assert root == bytes(32)
    toks = [1, 2, 70000, 2 ** 40 + 5]
    want = hashlib.sha256(root + b"".join(struct.pack("<Q", t) for t in toks)).digest()
    assert sgo.hash_chain(root, toks) == want
    assert sgo.hash_for_session("alpha") == hashlib.sha256(b"alpha").digest()
    assert sgo.hash_for_session("") == root and sgo.hash_for_session(None) == root


def test_chained_hash_depends_on_previous_block():
    # src/serve/cache.rs:281-288
    first = sgo.hash_chain(sgo.hash_root(), [1, 2])
    assert sgo.hash_chain(first, [3, 4]) != sgo.hash_chain(sgo.hash_root(), [3, 4])


def test_session_roots_are_deterministic_and_disjoint():
    # src/serve/cache.rs:290-298, 300-309
    assert sgo.hash_for_session("alpha") == sgo.hash_for_session("alpha")
    assert sgo.hash_for_session("alpha") != sgo.hash_for_session("beta")
    assert sgo.hash_chain(sgo.hash_for_session(None), [1, 2, 3]) == sgo.hash_chain(sgo.hash_root(), [1, 2, 3])


def test_prefix_cache_matches_longest_chain():
    # src/serve/cache.rs:311-339
    cache = sgo.BlockAwarePrefixCache(2, 8)
    root = sgo.hash_root()
    first = sgo.hash_chain(root, [1, 2])
    second = sgo.hash_chain(first, [3, 4])
    cache.insert(root, first, 2, payload=2)
    cache.insert(root, second, 4, payload=4)
    hit = cache.match_prefix(root, [1, 2, 3, 4, 5])
    assert hit["tokens"] == 4 and hit["hash"] == second and hit["payload"] == 4


def test_prefix_cache_evicts_lru_block():
    # src/serve/cache.rs:341-375
    cache = sgo.BlockAwarePrefixCache(1, 2)
    root = sgo.hash_root()
    first = sgo.hash_chain(root, [1])
    second = sgo.hash_chain(first, [2])
    third = sgo.hash_chain(second, [3])
    for h, n in ((first, 1), (second, 2), (third, 3)):
        cache.insert(root, h, n, payload=n)
    assert cache.match_prefix(root, [1]) is None
    assert cache.match_prefix(root, [1, 2, 3]) is None     # orphaned descendants cannot be reached
    assert [e[2] for e in cache.evicted()] == [1]


def test_default_session_cap_keeps_global_lru_order():
    # src/serve/cache.rs:377-419
    cache = sgo.BlockAwarePrefixCache(1, 2)
    alpha, beta = sgo.hash_for_session("agent-a"), sgo.hash_for_session("agent-b")
    beta_first = sgo.hash_chain(beta, [9])
    alpha_first = sgo.hash_chain(alpha, [1])
    alpha_second = sgo.hash_chain(alpha_first, [2])
    cache.insert(beta, beta_first, 1)
    cache.insert(alpha, alpha_first, 1)
    cache.insert(alpha, alpha_second, 2)
    assert [e[1] for e in cache.entries()] == [alpha_second, alpha_first]
    assert cache.match_prefix(beta, [9]) is None


def test_reduced_session_cap_evicts_only_that_session_first():
    # src/serve/cache.rs:421-466
    cache = sgo.BlockAwarePrefixCache(1, 2, 1)
    alpha, beta = sgo.hash_for_session("agent-a"), sgo.hash_for_session("agent-b")
    beta_first = sgo.hash_chain(beta, [9])
    alpha_first = sgo.hash_chain(alpha, [1])
    alpha_second = sgo.hash_chain(alpha_first, [2])
    cache.insert(beta, beta_first, 1)
    cache.insert(alpha, alpha_first, 1)
    cache.insert(alpha, alpha_second, 2)
    assert [e[1] for e in cache.entries()] == [alpha_second, beta_first]
    assert cache.match_prefix(beta, [9])["hash"] == beta_first
    assert cache.session_block_count(alpha) == 1


def test_prefix_cache_does_not_match_across_sessions():
    # src/serve/cache.rs:468-493
    cache = sgo.BlockAwarePrefixCache(2, 8)
    alpha, beta = sgo.hash_for_session("agent-a"), sgo.hash_for_session("agent-b")
    first = sgo.hash_chain(alpha, [1, 2])
    second = sgo.hash_chain(first, [3, 4])
    cache.insert(alpha, first, 2)
    cache.insert(alpha, second, 4)
    assert first != sgo.hash_chain(beta, [1, 2])
    assert cache.match_prefix(beta, [1, 2, 3, 4]) is None
    assert cache.match_prefix(alpha, [1, 2, 3, 4])["tokens"] == 4


def test_match_touch_order_makes_the_root_block_least_recent():
    # src/serve/cache.rs:131-148: blocks are touched root -> leaf, each moved to the front
    cache = sgo.BlockAwarePrefixCache(1, 8)
    root = sgo.hash_root()
    hs, prev = [], root
    for i, t in enumerate([5, 6, 7]):
        prev = sgo.hash_chain(prev, [t])
        hs.append(prev)
        cache.insert(root, prev, i + 1, payload=i + 1)
    other = sgo.hash_chain(root, [99])
    cache.insert(root, other, 1, payload=99)
    assert cache.match_prefix(root, [5, 6, 7, 8])["tokens"] == 3
    assert [e[3] for e in cache.entries()] == [3, 2, 1, 99]
    assert cache.evict_lru_block() is not None and [e[3] for e in cache.entries()] == [3, 2, 1]
    cache.evict_lru_block()
    assert [e[3] for e in cache.entries()] == [3, 2]       # root-most block left first
    assert cache.estimated_bytes() == 0
    zero = sgo.BlockAwarePrefixCache(1, 0)
    assert zero.insert(root, hs[0], 1) == 0 and zero.match_prefix(root, [5]) is None


def test_longest_prefix_entry_index():
    # prefix_cache_selects_longest_append_prefix, src/decoder/tests.rs:428-466
    entries = [[1, 2], [1, 2, 3], [1]]
    assert sgo.longest_prefix_entry_index(entries, [1, 2, 3, 4]) == 1
    assert sgo.longest_prefix_entry_index(entries, [1, 9]) == 2
    assert sgo.longest_prefix_entry_index(entries, [9]) is None


def test_memory_guard_limits_and_boundaries():
    # src/memory_guard.rs:734-788
    g = sgo.MemoryGuard(static_cap=900, host_memory=1200, headroom=200, device_cap=700)
    assert g.limit() == 700
    g = sgo.MemoryGuard(static_cap=150)
    g.set(100)
    assert g.check_allocation(50)[0]
    ok, projected, available = g.check_allocation(51)
    assert not ok and projected == 151 and available == 50
    g = sgo.MemoryGuard(static_cap=180)
    g.set(100, reserved=60)
    assert g.check_allocation(20)[0] and not g.check_allocation(21)[0]
    g.set(100, reserved=0)
    assert g.check_allocation(80)[0]
    assert sgo.MemoryGuard().limit() is None and sgo.MemoryGuard().check_allocation(1 << 60)[0]


def test_linear_state_restore_validates_shape():
    # src/metal_backend/linear_attention.rs:3133-3149
    assert sgo.linear_restore_check(192, 256, False, 192, 256, False) == sgo.OK
    assert sgo.linear_restore_check(192, 256, False, 191, 256, False) == sgo.ERR_SHAPE
    assert sgo.linear_restore_check(192, 256, False, 192, 256, True) == sgo.ERR_SHAPE
