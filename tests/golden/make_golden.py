"""Writes the golden fixtures of this folder from the CPU oracle (oracle/), which is itself
pinned to the reference's own known answers by tests/test_oracle_*.py. Inputs come from the
integer-exact generator (seed, stream, index), so a fixture stores only the seeds and the
expected outputs. Run from the repository root:  python tests/golden/make_golden.py

The reference is a Rust crate and cannot be run where these are made; the fixtures freeze what
the pinned restatement computes, so that the CUDA path is also checked against files that do
not move when the oracle is edited (tests/test_golden.py)."""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import sgo  # noqa: E402

ATTENTION_CASES = [  # name, q_heads, kv_heads, head_dim, dtype, rows, window_start
    ("attn_f32_c1shape", 32, 8, 128, sgo.KV_F32, 200, 0),
    ("attn_bf16_c2shape", 32, 4, 128, sgo.KV_BF16, 531, 0),
    ("attn_bf16_c5shape_window", 8, 4, 256, sgo.KV_BF16, 300, 77),
    ("attn_u8_c3shape", 16, 2, 256, sgo.KV_U8G32, 259, 0),
]


def attention_case(name, q_heads, kv_heads, hd, dtype, rows, ws, seed):
    kv_dim = kv_heads * hd
    k = sgo.fill_normal8(rows * kv_dim, seed, 0).reshape(rows, kv_dim)
    v = sgo.fill_normal8(rows * kv_dim, seed, 1).reshape(rows, kv_dim)
    q = sgo.fill_normal8(q_heads * hd, seed, 2)
    ref = sgo.ResidentKv(rows, q_heads, kv_heads, hd, dtype)
    assert ref.seed(k, v, rows) == sgo.OK
    st, out = ref.attention(q, window_start=ws, threads=4)
    assert st == sgo.OK
    return {"out": out, "stored_k_row0": ref.keys()[0], "stored_v_last": ref.values()[-1]}


def main():
    meta = {"generator": "oracle.sgo.fill_normal8(n, seed, stream)", "cases": {}}
    arrays = {}
    for i, (name, qh, kvh, hd, dtype, rows, ws) in enumerate(ATTENTION_CASES):
        seed = 100 + i
        res = attention_case(name, qh, kvh, hd, dtype, rows, ws, seed)
        meta["cases"][name] = {"q_heads": qh, "kv_heads": kvh, "head_dim": hd, "dtype": int(dtype), "rows": rows,
                               "window_start": ws, "seed": seed}
        for key, val in res.items():
            arrays[f"{name}.{key}"] = val

    # u8 group-32 quantiser: codes and bf16 scale/bias bits of one seeded row, ranges from tiny to large
    x = sgo.fill_normal8(512, 200, 0)
    x[:32] *= np.float32(1e-3)
    x[32:64] *= np.float32(300.0)
    x[64:96] = np.float32(1.25)            # a constant group: the scale floor
    codes, scale, bias = sgo.quantize_row_u8(x)
    meta["cases"]["quantise_u8"] = {"seed": 200, "n": 512, "edits": "x[:32]*=1e-3; x[32:64]*=300; x[64:96]=1.25"}
    arrays["quantise_u8.codes"], arrays["quantise_u8.scale_bits"], arrays["quantise_u8.bias_bits"] = codes, scale, bias

    # RMSNorm + RoPE at a position, both pairing styles
    heads, hd, rope_dims, theta, pos = 4, 128, 64, 1_000_000.0, 4097
    xr = sgo.fill_normal8(heads * hd, 201, 0)
    w = np.float32(0.75) + np.abs(sgo.fill_normal8(hd, 201, 1)) * np.float32(0.1)
    for style, label in ((sgo.ROPE_HALVES, "halves"), (sgo.ROPE_INTERLEAVED, "interleaved")):
        st, out = sgo.rms_norm_rope_heads_at(xr[None], heads, hd, rope_dims, w, 1e-6, theta, rope_dims, 1.0, pos, style)
        assert st == sgo.OK
        arrays[f"rope_{label}.out"] = out.ravel()
    meta["cases"]["rope"] = {"heads": heads, "head_dim": hd, "rope_dims": rope_dims, "theta": theta, "position": pos,
                             "eps": 1e-6, "seed": 201}

    # one Gated DeltaNet token and one conv token on seeded state
    hk, hv, dk, dv = 2, 4, 128, 32
    ssm = sgo.fill_normal8(hv * dv * dk, 202, 0) * np.float32(0.1)
    qg = sgo.fill_normal8(hk * dk, 202, 1) / np.float32(dk)
    kg = sgo.fill_normal8(hk * dk, 202, 2) / np.float32(np.sqrt(dk))
    vg = sgo.fill_normal8(hv * dv, 202, 3)
    g = np.linspace(0.9, 0.99, hv).astype(np.float32)
    beta = np.linspace(0.2, 0.8, hv).astype(np.float32)
    st, y, new_ssm = sgo.gated_delta_step(qg, kg, vg, g, beta, hk, hv, dk, dv, ssm)
    assert st == sgo.OK
    arrays["gated_delta.y"], arrays["gated_delta.ssm_checksum"] = y, np.array([new_ssm.astype(np.float64).sum()])
    arrays["gated_delta.ssm_head"] = new_ssm[:256]
    meta["cases"]["gated_delta"] = {"shape": [hk, hv, dk, dv], "seed": 202}

    # hash chain and the eviction order of a fixed operation trace (src/serve/cache.rs)
    root = sgo.hash_for_session("golden-session")
    chain, prev = [], root
    for b in range(6):
        prev = sgo.hash_chain(prev, list(range(16 * b, 16 * b + 16)))
        chain.append(prev.hex())
    cache = sgo.BlockAwarePrefixCache(16, 4, 3)
    toks = list(range(96))
    prev, hashes = root, []
    for b in range(6):
        prev = sgo.hash_chain(prev, toks[16 * b:16 * b + 16])
        hashes.append(prev)
        cache.insert(root, prev, 16 * (b + 1), payload=b, nbytes=1000 + b)
        if b == 3:
            cache.match_prefix(root, toks[:64])
    order = [(h.hex()[:16], t, p) for (_, h, t, p) in cache.evicted()]
    left = [(h.hex()[:16], t, p) for (_, h, t, p) in cache.entries()]
    meta["cases"]["prefix"] = {"session_root": root.hex(), "chain": chain, "evicted_in_order": order, "entries_front_to_back": left,
                               "sha256_abc": hashlib.sha256(b"abc").hexdigest()}

    np.savez_compressed(os.path.join(HERE, "kv_path_golden.npz"), **arrays)
    with open(os.path.join(HERE, "kv_path_golden.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print("wrote", len(arrays), "arrays;", os.path.getsize(os.path.join(HERE, "kv_path_golden.npz")), "bytes")


if __name__ == "__main__":
    main()
