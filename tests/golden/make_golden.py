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


def decode_step_inputs(seed):
    hk, hv, d, kernel = 2, 4, 128, 4
    conv_dim = 2 * hk * d + hv * d
    f = lambda n, stream, scale=1.0: sgo.fill_normal8(n, seed, stream) * np.float32(scale)
    return {"qkv": f(conv_dim, 0), "w": f(conv_dim * kernel, 1, 0.5), "hist": f((kernel - 1) * conv_dim, 2),
            "ssm": f(hv * d * d, 3, 0.1), "beta_in": f(hv, 4), "gate_in": f(hv, 5), "a_log": f(hv, 6, 0.3),
            "dt_bias": f(hv, 7, 0.3), "shape": (hk, hv, d, d), "kernel": kernel, "conv_dim": conv_dim}


def decode_step_case(seed):
    i = decode_step_inputs(seed)
    hk, hv, dk, dv = i["shape"]
    st, out, hist, ssm, parts = sgo.linear_decode_step(i["qkv"], i["w"], i["kernel"], i["hist"], i["beta_in"], i["gate_in"],
                                                       i["a_log"], i["dt_bias"], hk, hv, dk, dv, i["ssm"])
    assert st == sgo.OK
    return {"y": out, "hist_last": hist[-i["conv_dim"]:], "ssm_head": ssm[:256],
            "ssm_checksum": np.array([ssm.astype(np.float64).sum()]), "q": parts["q"].astype(np.float32),
            "g": parts["g"], "beta": parts["beta"]}


AFFINE_VOCAB, AFFINE_HIDDEN = 2051, 512


def affine_case(seed, bits):
    """Codes, bf16 scales and biases of a [2051][512] weight in groups of 64 and one activation row, all from
    the integer-exact generator."""
    n, groups = AFFINE_VOCAB * AFFINE_HIDDEN, AFFINE_VOCAB * (AFFINE_HIDDEN // 64)
    top = (1 << bits) - 1
    raw = sgo.fill_normal8(n, seed + bits, 0)
    codes = np.clip(np.floor(raw * np.float32(top / 6.0) + np.float32(top / 2.0)), 0, top).astype(np.uint32)
    scales = sgo.f32_to_bf16_bits((np.float32(1.0) + np.abs(sgo.fill_normal8(groups, seed + bits, 1))) * np.float32(0.02 / (top + 1)))
    biases = sgo.f32_to_bf16_bits(sgo.fill_normal8(groups, seed + bits, 2) * np.float32(0.01))
    x = sgo.fill_normal8(AFFINE_HIDDEN, seed, 9)
    return sgo.affine_pack(codes.reshape(AFFINE_VOCAB, AFFINE_HIDDEN), bits), scales, biases, x


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

    # the whole decode step of a recurrent layer (conv, SiLU, unit norms, gates, gated delta)
    res = decode_step_case(203)
    for key, val in res.items():
        arrays[f"decode_step.{key}"] = val
    meta["cases"]["decode_step"] = {"shape": [2, 4, 128, 128], "kernel": 4, "seed": 203}

    # greedy epilogue over an affine-quantised weight: the winning row and its logit
    for bits in (8, 4):
        packed, scales, biases, x = affine_case(204, bits)
        w = sgo.affine_dequantize(packed, scales, biases, bits, 64, AFFINE_VOCAB, AFFINE_HIDDEN)
        logits = w.astype(np.float64) @ x.astype(np.float64)
        st, idx, _ = sgo.lm_head_argmax(w, x)
        assert st == sgo.OK and idx == int(np.argmax(logits))
        arrays[f"affine_u{bits}.index"] = np.array([idx], np.int64)
        arrays[f"affine_u{bits}.logit"] = np.array([logits[idx]], np.float64)
        arrays[f"affine_u{bits}.row_head"] = w[idx, :64]
    meta["cases"]["affine_lm_head"] = {"vocab": AFFINE_VOCAB, "hidden": AFFINE_HIDDEN, "group": 64, "seed": 204}

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
