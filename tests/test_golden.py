"""The committed fixtures of tests/golden/ (made by tests/golden/make_golden.py from the pinned
oracle): on CPU the oracle must still reproduce them bit for bit and the product's host-side
hashing / eviction bookkeeping must give the same digests and the same order; on the GPU the CUDA
path is compared with the files themselves, without running the oracle."""
import json
import os
import sys

import numpy as np
import pytest

import saragossa_b200 as sg
from oracle import sgo

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, HERE)
import make_golden  # noqa: E402  (the generator of the fixtures: its input builders are reused here)
META = json.load(open(os.path.join(HERE, "kv_path_golden.json")))["cases"]
GOLD = np.load(os.path.join(HERE, "kv_path_golden.npz"))
ATTN = [n for n in META if n.startswith("attn_")]


def _attn_inputs(c):
    kv_dim = c["kv_heads"] * c["head_dim"]
    k = sgo.fill_normal8(c["rows"] * kv_dim, c["seed"], 0).reshape(c["rows"], kv_dim)
    v = sgo.fill_normal8(c["rows"] * kv_dim, c["seed"], 1).reshape(c["rows"], kv_dim)
    q = sgo.fill_normal8(c["q_heads"] * c["head_dim"], c["seed"], 2)
    return k, v, q


def _quant_input():
    x = sgo.fill_normal8(512, 200, 0)
    x[:32] *= np.float32(1e-3)
    x[32:64] *= np.float32(300.0)
    x[64:96] = np.float32(1.25)
    return x


# ---- CPU: the oracle has not drifted from the files ------------------------------------
@pytest.mark.parametrize("name", ATTN)
def test_oracle_reproduces_attention_fixture(name):
    c = META[name]
    k, v, q = _attn_inputs(c)
    ref = sgo.ResidentKv(c["rows"], c["q_heads"], c["kv_heads"], c["head_dim"], c["dtype"])
    assert ref.seed(k, v, c["rows"]) == sgo.OK
    st, out = ref.attention(q, window_start=c["window_start"], threads=2)
    assert st == sgo.OK
    np.testing.assert_array_equal(out, GOLD[f"{name}.out"])
    np.testing.assert_array_equal(ref.keys()[0], GOLD[f"{name}.stored_k_row0"])
    np.testing.assert_array_equal(ref.values()[-1], GOLD[f"{name}.stored_v_last"])


def test_oracle_reproduces_quantiser_rope_and_recurrence_fixtures():
    codes, scale, bias = sgo.quantize_row_u8(_quant_input())
    np.testing.assert_array_equal(codes, GOLD["quantise_u8.codes"])
    np.testing.assert_array_equal(scale, GOLD["quantise_u8.scale_bits"])
    np.testing.assert_array_equal(bias, GOLD["quantise_u8.bias_bits"])
    r = META["rope"]
    x = sgo.fill_normal8(r["heads"] * r["head_dim"], r["seed"], 0)
    w = np.float32(0.75) + np.abs(sgo.fill_normal8(r["head_dim"], r["seed"], 1)) * np.float32(0.1)
    for style, label in ((sgo.ROPE_HALVES, "halves"), (sgo.ROPE_INTERLEAVED, "interleaved")):
        st, out = sgo.rms_norm_rope_heads_at(x[None], r["heads"], r["head_dim"], r["rope_dims"], w, r["eps"], r["theta"],
                                             r["rope_dims"], 1.0, r["position"], style)
        assert st == sgo.OK
        np.testing.assert_array_equal(out.ravel(), GOLD[f"rope_{label}.out"])


def test_host_hashing_and_eviction_order_match_the_fixture():
    # the product's own SHA-256 / chain / LRU bookkeeping (no device involved)
    p = META["prefix"]
    root = sg.BlockHash.for_session("golden-session")
    assert root.hex() == p["session_root"]
    cache = sg.BlockAwarePrefixCache(16, 4, 3)
    toks = list(range(96))
    prev = root
    for b in range(6):
        prev = sg.BlockHash.chain(prev, toks[16 * b:16 * b + 16])
        assert prev.hex() == p["chain"][b]
        cache.insert(root, prev, 16 * (b + 1))
        if b == 3:
            cache.match_prefix(root, toks[:64])
    assert [(h.hex()[:16], t) for (_, h, t) in cache.evicted()] == [(h, t) for (h, t, _) in p["evicted_in_order"]]
    assert [(h.hex()[:16], t) for (_, h, t) in cache.entries()] == [(h, t) for (h, t, _) in p["entries_front_to_back"]]
    cache.close()


# ---- GPU: the CUDA path against the files ------------------------------------------------------
@pytest.fixture(scope="module")
def state():
    st = sg.DecodeResidentState(0)
    yield st
    assert st.device_status() == 0
    st.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ATTN)
def test_cuda_attention_matches_fixture(state, name):
    c = META[name]
    k, v, q = _attn_inputs(c)
    kv = state.full_attention(c["rows"], c["q_heads"], c["kv_heads"], c["head_dim"], c["dtype"], shuffled_seed=1)
    kv.seed(k, v, c["rows"])
    got = kv.attention_decode_windowed(q, c["window_start"])
    want = GOLD[f"{name}.out"]
    if c["dtype"] == sg.KV_F32:
        assert np.abs(got - want).max() <= 1e-4          # the reference's f32 bound
    else:
        assert np.all(np.abs(got - want) <= 2e-2 * np.abs(want) + 1e-3)
    gk, gv = kv.gather_rows_f32()
    np.testing.assert_array_equal(gk[0], GOLD[f"{name}.stored_k_row0"])     # storage rounding: bit-exact
    np.testing.assert_array_equal(gv[-1], GOLD[f"{name}.stored_v_last"])
    kv.close()


@pytest.mark.gpu
def test_cuda_quantiser_rope_and_recurrence_match_fixtures(state):
    x = _quant_input()
    kv = state.full_attention(16, 2, 2, 256, sg.KV_U8G32)
    kv.append_row(x, x[::-1].copy())
    kc, ks, kb, _, _, _ = kv.gather_rows_u8()
    np.testing.assert_array_equal(kc[0], GOLD["quantise_u8.codes"])
    np.testing.assert_array_equal(ks[0], GOLD["quantise_u8.scale_bits"])
    np.testing.assert_array_equal(kb[0], GOLD["quantise_u8.bias_bits"])
    kv.close()
    r = META["rope"]
    xr = sgo.fill_normal8(r["heads"] * r["head_dim"], r["seed"], 0)
    w = np.float32(0.75) + np.abs(sgo.fill_normal8(r["head_dim"], r["seed"], 1)) * np.float32(0.1)
    for inter, label in ((False, "halves"), (True, "interleaved")):
        rope = sg.make_rope(r["rope_dims"], r["theta"], eps=r["eps"], interleaved=inter)
        out = state.rms_norm_rope_decode(xr, w, r["heads"], r["head_dim"], rope, r["position"])
        assert np.abs(out - GOLD[f"rope_{label}.out"]).max() <= 1e-5
    hk, hv, dk, dv = META["gated_delta"]["shape"]
    seed = META["gated_delta"]["seed"]
    ssm = sgo.fill_normal8(hv * dv * dk, seed, 0) * np.float32(0.1)
    ins = [sgo.fill_normal8(hk * dk, seed, 1) / np.float32(dk), sgo.fill_normal8(hk * dk, seed, 2) / np.float32(np.sqrt(dk)),
           sgo.fill_normal8(hv * dv, seed, 3), np.linspace(0.9, 0.99, hv).astype(np.float32),
           np.linspace(0.2, 0.8, hv).astype(np.float32)]
    ls = sg.LinearAttentionState(state, 1, 0, hv * dv * dk)
    ls.write(0, np.zeros(0, np.float32), ssm)
    d_y = state.alloc(4 * hv * dv)
    ls.encode_gated_delta_step(0, (hk, hv, dk, dv), *[state.upload(a) for a in ins], d_y)
    state.sync()
    assert np.abs(d_y.download(count=hv * dv) - GOLD["gated_delta.y"]).max() <= 1e-5
    _, new_ssm = ls.read(0)
    assert np.abs(new_ssm[:256] - GOLD["gated_delta.ssm_head"]).max() <= 1e-5
    assert abs(float(new_ssm.astype(np.float64).sum()) - float(GOLD["gated_delta.ssm_checksum"][0])) <= 1e-2
    ls.close()


# ---- the decode step of a recurrent layer and the affine-quantised greedy epilogue ------------
def test_oracle_reproduces_decode_step_and_affine_fixtures():
    res = make_golden.decode_step_case(META["decode_step"]["seed"])
    for key, val in res.items():
        np.testing.assert_array_equal(val, GOLD[f"decode_step.{key}"])
    c = META["affine_lm_head"]
    for bits in (8, 4):
        packed, scales, biases, x = make_golden.affine_case(c["seed"], bits)
        w = sgo.affine_dequantize(packed, scales, biases, bits, c["group"], c["vocab"], c["hidden"])
        st, idx, _ = sgo.lm_head_argmax(w, x)
        assert st == sgo.OK and idx == int(GOLD[f"affine_u{bits}.index"][0])
        np.testing.assert_array_equal(w[idx, :64], GOLD[f"affine_u{bits}.row_head"])


@pytest.mark.gpu
def test_cuda_decode_step_and_affine_epilogue_match_fixtures(state):
    i = make_golden.decode_step_inputs(META["decode_step"]["seed"])
    hk, hv, dk, dv = i["shape"]
    ls = sg.LinearAttentionState(state, 1, (i["kernel"] - 1) * i["conv_dim"], hv * dv * dk)
    ls.write(0, i["hist"], i["ssm"])
    d_y = state.alloc(4 * hv * dv)
    ls.encode_decode_step(0, i["shape"], state.upload(i["qkv"]), state.upload(i["w"]), i["kernel"], state.upload(i["beta_in"]),
                          state.upload(i["gate_in"]), state.upload(i["a_log"]), state.upload(i["dt_bias"]), d_y)
    state.sync()
    assert np.abs(d_y.download(count=hv * dv) - GOLD["decode_step.y"]).max() <= 1e-5
    hist, ssm = ls.read(0)
    np.testing.assert_array_equal(hist[-i["conv_dim"]:], GOLD["decode_step.hist_last"])
    assert np.abs(ssm[:256] - GOLD["decode_step.ssm_head"]).max() <= 1e-5
    assert abs(float(ssm.astype(np.float64).sum()) - float(GOLD["decode_step.ssm_checksum"][0])) <= 1e-2
    ls.close()
    c = META["affine_lm_head"]
    d_idx, d_val = state.alloc(4 * 8), state.alloc(4 * 8)
    for bits in (8, 4):
        packed, scales, biases, x = make_golden.affine_case(c["seed"], bits)
        d_w = state.upload_affine(packed, scales, biases, bits, c["group"])
        state.encode_lm_head_argmax_affine(d_w, c["vocab"], c["hidden"], state.upload(x), d_idx, n_rows=1, d_value_out=d_val)
        state.sync()
        assert int(d_idx.download(np.int32, 1)[0]) == int(GOLD[f"affine_u{bits}.index"][0])
        want = float(GOLD[f"affine_u{bits}.logit"][0])
        assert abs(float(d_val.download(np.float32, 1)[0]) - want) <= 2e-4 * max(1.0, abs(want))
