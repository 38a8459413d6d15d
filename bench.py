#!/usr/bin/env python
"""Benchmark of the KV-cache hot path (append + paged GQA decode attention) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config 2 of BASELINE.json): 48 layers, 32 Q / 4 KV heads, head_dim 128,
bf16 KV in 16-token pages behind a shuffled block table, context 32768, batch 8
independent sequences per GPU; one "step" appends one token's K/V per layer and
runs paged decode attention over the whole cache, for every layer, as ONE CUDA
graph submission. K/V and q are seeded synthetic values (integer-exact
approximately-normal generator, seed 0), generated on the device.

Prints one JSON line. `value` is the whole-job algorithmic HBM GB/s (K and V rows
read once + the appended row, summed over all GPUs, divided by the max-over-ranks
device time). `e2e` is the same metric through the host-buffer C-ABI call
(inputs copied in and outputs copied out inside the timed region).

`--impl reference` times the CPU restatement of the reference's own path
(oracle/, all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, Q_HEADS, KV_HEADS, HEAD_DIM = 48, 32, 4, 128
CTX, BATCH = 32768, 8
KV_DIM, Q_DIM = KV_HEADS * HEAD_DIM, Q_HEADS * HEAD_DIM
WORKLOAD = ("C2: Qwen3-30B-A3B-shaped KV path, 48 layers, 32Q/4KV heads, head_dim 128, bf16 KV, "
            "16-token pages, shuffled block table, ctx 32768, batch 8 per GPU")


def workload_config():
    """The `config` both arms print (the reference arm times a bounded sample of the same workload)."""
    return {"workload": WORKLOAD, "sharding": "by sequence, no collective",
            "l2": "inputs larger than L2 (24.6 GB of KV per GPU streamed per step)",
            "timing": "ours: CUDA events around K graph replays, max over ranks; reference arm: host clock around "
                      "each bounded sample (one layer of one sequence per step)"}


def ncu_traffic_ratio():
    """DRAM read+write bytes per launch of the headline kernel divided by the launch's algorithmic
    bytes, from the ncu capture whose summary sits beside this file's numbers."""
    try:
        with open(os.path.join(ROOT, "profiles", "attention_mma_hd128_c2.json")) as f:
            return float(json.load(f)["dram_bytes_over_algorithmic_bytes"])
    except Exception:
        return None


KV_DTYPE = "bf16"           # or "u8": 32 codes + bf16 scale + bf16 bias per group = 1.125 B per element


def algorithmic_bytes(rows_after_append: int) -> int:
    """K and V rows of one sequence and layer read once, plus the appended row, in storage bytes."""
    elem = 2.0 if KV_DTYPE == "bf16" else 1.125
    return int((rows_after_append * KV_DIM * 2 + KV_DIM * 2) * elem)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ts, line in self.lines:
            if t0 is not None and not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples in the timed region"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------- reference arm
def cpu_sample(threads: int, iters: int):
    """One layer of one sequence at the full context through the CPU restatement of the
    reference path (append + cached_attention_one), f32 storage of bf16-rounded values."""
    from oracle import sgo
    rows = CTX
    k = sgo.bf16_round(sgo.fill_normal8(rows * KV_DIM, 0, 0))
    v = sgo.bf16_round(sgo.fill_normal8(rows * KV_DIM, 0, 1))
    cache = sgo.LayerKvCache()
    assert cache.append_batch(k.reshape(rows, KV_DIM), v.reshape(rows, KV_DIM), KV_DIM) == sgo.OK
    times = []
    for it in range(iters):
        k_new = sgo.bf16_round(sgo.fill_normal8(KV_DIM, 1, 3 * it))
        v_new = sgo.bf16_round(sgo.fill_normal8(KV_DIM, 1, 3 * it + 1))
        q = sgo.fill_normal8(Q_DIM, 1, 3 * it + 2)
        t0 = time.perf_counter()
        assert cache.append(k_new[None], v_new[None], KV_DIM) == sgo.OK
        n = cache.len()
        out = np.zeros(Q_DIM, np.float32)
        rc = sgo.lib().sgo_cached_attention_one(
            q.ctypes.data_as(sgo.C.POINTER(sgo.C.c_float)), Q_DIM, sgo.lib().sgo_cache_keys(cache._h),
            sgo.lib().sgo_cache_values(cache._h), n, Q_HEADS, KV_HEADS, HEAD_DIM, float(HEAD_DIM), 0, 0, threads,
            out.ctypes.data_as(sgo.C.POINTER(sgo.C.c_float)))
        assert rc == sgo.OK
        times.append((time.perf_counter() - t0, algorithmic_bytes(n)))
    return times


def parity_spot(threads, rows, gpu_out, k_new, v_new, q):
    """Full-size parity point: (layer 0, sequence 0) of the last timed step against the CPU
    restatement of the reference path on the same bytes. The cache holds the 32768 seeded rows
    (generator streams 0 and 1 of seed 0) and, behind them, the row every step appended (the
    step's k / v inputs do not change between replays). Tolerance of the task for bf16 pages:
    |err| <= 2e-2 * |want| + 1e-3."""
    from oracle import sgo
    k = np.empty((rows, KV_DIM), np.float32)
    v = np.empty((rows, KV_DIM), np.float32)
    k[:CTX] = sgo.bf16_round(sgo.fill_normal8(CTX * KV_DIM, 0, 0)).reshape(CTX, KV_DIM)
    v[:CTX] = sgo.bf16_round(sgo.fill_normal8(CTX * KV_DIM, 0, 1)).reshape(CTX, KV_DIM)
    k[CTX:] = sgo.bf16_round(np.ascontiguousarray(k_new, np.float32))
    v[CTX:] = sgo.bf16_round(np.ascontiguousarray(v_new, np.float32))
    cache = sgo.LayerKvCache()
    assert cache.append_batch(k, v, KV_DIM) == sgo.OK
    want = np.zeros(Q_DIM, np.float32)
    qq = np.ascontiguousarray(q, np.float32)
    rc = sgo.lib().sgo_cached_attention_one(
        qq.ctypes.data_as(sgo.C.POINTER(sgo.C.c_float)), Q_DIM, sgo.lib().sgo_cache_keys(cache._h),
        sgo.lib().sgo_cache_values(cache._h), rows, Q_HEADS, KV_HEADS, HEAD_DIM, float(HEAD_DIM), 0, 0, threads,
        want.ctypes.data_as(sgo.C.POINTER(sgo.C.c_float)))
    assert rc == sgo.OK
    err = np.abs(gpu_out.astype(np.float64) - want.astype(np.float64))
    big = np.abs(want) >= 1e-3
    return {"rows": int(rows), "max_abs": float(err.max()),
            "max_rel": float((err[big] / np.abs(want[big])).max()) if big.any() else 0.0,
            "within_2e-2_rel_plus_1e-3_abs": bool(np.all(err <= 2e-2 * np.abs(want) + 1e-3)),
            "what": "layer 0, sequence 0 of the last timed step vs the CPU path on the same bytes"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = min(Q_HEADS, os.cpu_count() or 1)
    # each step = one (layer, sequence) unit of the workload
    cpu_sample(threads, max(1, args.warmup))
    times = cpu_sample(threads, args.steps)
    total_t = sum(t for t, _ in times)
    total_b = sum(b for _, b in times)
    gbs = total_b / total_t / 1e9
    sample = (f"{args.steps} steps, each ONE layer of ONE sequence at ctx {CTX} (of the {LAYERS} layers x "
              f"{BATCH} sequences of a full step); f32 storage of bf16-rounded K/V like the reference's bf16 oracle")
    line = {
        "impl": "reference", "metric": "decode_attn_append_hbm_gbs_32k", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_t / len(times) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(),
        "us_per_layer_per_seq": total_t / len(times) * 1e6,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm
def build_sequences(sg, st, pool, batch, ctx, capacity):
    seqs = [pool.sequence(capacity) for _ in range(batch)]
    kvs = [[seq.layer(layer, Q_HEADS) for seq in seqs] for layer in range(LAYERS)]
    chunk = 8192
    dk, dv = st.alloc(chunk * KV_DIM * 4), st.alloc(chunk * KV_DIM * 4)
    for layer in range(LAYERS):
        for s in range(batch):
            stream_id = (layer * batch + s) * 2
            for c in range(0, ctx, chunk):
                n = min(chunk, ctx - c)
                st.fill_normal(dk, n * KV_DIM, 0, stream_id, c * KV_DIM)
                st.fill_normal(dv, n * KV_DIM, 0, stream_id + 1, c * KV_DIM)
                kvs[layer][s].encode_append_rows(dk, dv, n)
    st.sync()
    dk.free()
    dv.free()
    return seqs, kvs


def timed_replays(torch, step, stream, steps, dist, world):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record(stream)
    for _ in range(steps):
        step.replay(stream.cuda_stream)
    e1.record(stream)
    stream.synchronize()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms, t0, t1


def run_ours(args):
    import torch
    import saragossa_b200 as sg

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    st = sg.DecodeResidentState(local_rank)
    K, W = args.steps, max(args.warmup, 3)
    e2e_steps = max(2, min(8, K))
    b1_steps = max(4, min(32, K))
    extra = W + K + 2 * e2e_steps + 2 + 2 * (3 + b1_steps) + 16
    capacity = ((CTX + extra + 15) // 16) * 16
    pages_per_seq = capacity // 16
    dtype = sg.KV_BF16 if KV_DTYPE == "bf16" else sg.KV_U8G32
    pool = st.pool(LAYERS, KV_HEADS, HEAD_DIM, dtype, pages_per_seq * BATCH, BATCH, capacity)
    pool.shuffle_free_list(0)
    t_seed = time.perf_counter()
    seqs, kvs = build_sequences(sg, st, pool, BATCH, CTX, capacity)
    t_seed = time.perf_counter() - t_seed
    batches = [sg.Batch(st, kvs[layer]) for layer in range(LAYERS)]
    step = sg.Step(st, batches)
    d_k, d_v = st.alloc(LAYERS * BATCH * KV_DIM * 4), st.alloc(LAYERS * BATCH * KV_DIM * 4)
    d_q, d_out = st.alloc(LAYERS * BATCH * Q_DIM * 4), st.alloc(LAYERS * BATCH * Q_DIM * 4)
    st.fill_normal(d_k, LAYERS * BATCH * KV_DIM, 0, 10_000)
    st.fill_normal(d_v, LAYERS * BATCH * KV_DIM, 0, 10_001)
    st.fill_normal(d_q, LAYERS * BATCH * Q_DIM, 0, 10_002)
    st.sync()
    step.capture(d_k, d_v, d_q, d_out)
    stream = torch.cuda.Stream()

    # ---- device-resident timing: K graph replays ----
    for _ in range(W):
        step.replay(stream.cuda_stream)
    stream.synchronize()
    rows_before = kvs[0][0].len()
    launches_before = step.launches()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    ms, t0, t1 = timed_replays(torch, step, stream, K, dist, world)
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    launches = step.launches() - launches_before
    bytes_per_gpu = sum(algorithmic_bytes(rows_before + i + 1) for i in range(K)) * LAYERS * BATCH
    value = bytes_per_gpu * world / (ms * 1e-3) / 1e9
    us_per_layer = ms * 1e3 / (K * LAYERS)
    status = st.device_status()
    # (layer 0, sequence 0) of the last timed step, for the full-context check against the CPU path
    spot_rows = kvs[0][0].len()
    spot_out = d_out.download(count=Q_DIM).copy()
    if args.skip_extras:
        if rank == 0:
            print(json.dumps({"metric": "decode_attn_append_hbm_gbs_32k", "value": value, "unit": "GB/s",
                              "n_gpus": world, "steps": K, "warmup": W, "us_per_layer": us_per_layer,
                              "gpu_launches": int(launches), "device_status": status,
                              "config": {"workload": f"other shape / subset: layers={LAYERS} batch={BATCH} ctx={CTX} "
                                                      f"q{Q_HEADS}/kv{KV_HEADS}/hd{HEAD_DIM} {KV_DTYPE}"},
                              "us_per_layer_per_seq": us_per_layer / BATCH}),
                  flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- end to end: host buffers in, host buffers out, every step ----
    pin = lambda n: torch.empty(n, dtype=torch.float32).pin_memory().numpy()
    h_k, h_v, h_q = pin(LAYERS * BATCH * KV_DIM), pin(LAYERS * BATCH * KV_DIM), pin(LAYERS * BATCH * Q_DIM)
    h_out = pin(LAYERS * BATCH * Q_DIM)
    h_k[:] = d_k.download()
    h_v[:] = d_v.download()
    h_q[:] = d_q.download()
    step.run_host(h_k, h_v, h_q, h_out)
    rows_e2e = kvs[0][0].len()
    if world > 1:
        dist.barrier()
    te = time.perf_counter()
    for _ in range(e2e_steps):
        step.run_host(h_k, h_v, h_q, h_out)
    te = time.perf_counter() - te
    if world > 1:
        t = torch.tensor([te], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        te = float(t.item())
    e2e_bytes = sum(algorithmic_bytes(rows_e2e + i + 1) for i in range(e2e_steps)) * LAYERS * BATCH
    e2e_value = e2e_bytes * world / te / 1e9
    # The same without any overlap, for a caller whose layer l+1 inputs exist only after layer l:
    # all inputs copied in, the token's graph, all outputs copied out, one after the other.
    rows_serial = kvs[0][0].len()
    ts = time.perf_counter()
    for _ in range(e2e_steps):
        d_k.upload(h_k)
        d_v.upload(h_v)
        d_q.upload(h_q)
        step.replay(stream.cuda_stream)
        stream.synchronize()
        check_out = st.L.sgk_util_d2h(st.h, h_out.ctypes.data, d_out.ptr, h_out.nbytes)
        if check_out != 0:
            raise RuntimeError("device to host copy failed")
    ts = time.perf_counter() - ts
    if world > 1:
        t = torch.tensor([ts], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts = float(t.item())
    serial_bytes = sum(algorithmic_bytes(rows_serial + i + 1) for i in range(e2e_steps)) * LAYERS * BATCH
    e2e_serial_value = serial_bytes * world / ts / 1e9
    h2d = (2 * LAYERS * BATCH * KV_DIM + LAYERS * BATCH * Q_DIM) * 4
    d2h = LAYERS * BATCH * Q_DIM * 4
    finite = bool(np.isfinite(h_out).all())

    # ---- batch 1 (single long sequence) on this GPU, same pool ----
    b1_batches = [sg.Batch(st, [kvs[layer][0]]) for layer in range(LAYERS)]
    b1_step = sg.Step(st, b1_batches)
    b1_step.capture(d_k, d_v, d_q, d_out)
    for _ in range(3):
        b1_step.replay(stream.cuda_stream)
    stream.synchronize()
    rows_b1 = kvs[0][0].len()
    ms_b1, _, _ = timed_replays(torch, b1_step, stream, b1_steps, None, 1)
    b1_bytes = sum(algorithmic_bytes(rows_b1 + i + 1) for i in range(b1_steps)) * LAYERS
    b1_us_layer = ms_b1 * 1e3 / (b1_steps * LAYERS)
    b1_gbs = b1_bytes / (ms_b1 * 1e-3) / 1e9

    # ---- one long sequence sharded by KV-head group (only where kv heads divide over the ranks) ----
    # The legs below are reported beside the headline; none of them may cost the line itself.
    head_sharded = None
    if world > 1 and KV_HEADS % world == 0:
        head_sharded = head_sharded_leg(sg, st, torch, dist, world, rank, stream)

    # The headline's pages (24.6 GB) go back before the other configurations take theirs.
    for obj in [b1_step, step] + b1_batches + batches + seqs + [pool]:
        obj.close()

    # ---- prefix restore: block copy of a 4096-token prefix on the 4B shape (config 4) ----
    restore = guarded(prefix_restore_gbs, sg, st, torch, stream)
    recurrent = guarded(gated_delta_leg, sg, st, torch, stream)
    producer = guarded(bulk_append_leg, sg, st, torch, stream)
    c3 = guarded(c3_token_leg, sg, st, torch, stream)
    c5 = guarded(c5_serving_leg, sg, st, torch, stream, dist, rank, world)
    c4 = guarded(c4_prefix_leg, sg, st, torch, stream, args.c4_turns, 128, rank, world)
    if world > 1:
        # whole job: all turns over the slowest rank's wall time (a rank that failed contributes zero turns)
        ok = isinstance(c4, dict) and "error" not in c4
        mine = [float(c4["turns_on_this_gpu"]), c4["turns_on_this_gpu"] / max(c4["turns_per_s"], 1e-9)] if ok else [0.0, 0.0]
        t_sum = torch.tensor(mine, device="cuda", dtype=torch.float64)
        t_max = t_sum.clone()
        dist.all_reduce(t_sum, op=dist.ReduceOp.SUM)
        dist.all_reduce(t_max, op=dist.ReduceOp.MAX)
        if ok:
            wall = max(float(t_max[1].item()), 1e-9)
            c4["turns_done_all_gpus"] = int(t_sum[0].item())
            c4["turns_per_s_all_gpus"] = float(t_sum[0].item()) / wall
            c4["decode_tokens_per_s_all_gpus"] = float(t_sum[0].item()) * 128 / wall
    c1 = guarded(c1_decode_leg, sg, st, torch, stream) if rank == 0 else None
    lm_head = guarded(lm_head_leg, sg, st, torch, stream)

    if rank == 0:
        peak, peak_kind = measured_peak()
        launch_us = ms * 1e3 / max(launches, 1)
        alg_per_launch = bytes_per_gpu / max(launches, 1)
        achieved = alg_per_launch / (launch_us * 1e-6) / 1e9
        threads = min(Q_HEADS, os.cpu_count() or 1)
        cpu_times = cpu_sample(threads, 25)[1:]
        cpu_gbs = sum(b for _, b in cpu_times) / sum(t for t, _ in cpu_times) / 1e9
        spot = guarded(parity_spot, threads, spot_rows, spot_out, h_k[:KV_DIM], h_v[:KV_DIM], h_q[:Q_DIM])
        ratio = ncu_traffic_ratio()
        config = workload_config() if not args.reduced else {
            "workload": f"OTHER layers={LAYERS} batch={BATCH} ctx={CTX} q{Q_HEADS}/kv{KV_HEADS}/hd{HEAD_DIM} {KV_DTYPE}"}
        line = {
            "metric": "decode_attn_append_hbm_gbs_32k", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
            "us_per_layer": us_per_layer, "us_per_layer_per_seq": us_per_layer / BATCH,
            "decode_steps_per_s": BATCH * world * K / (ms * 1e-3),
            # the other configurations and kernels, longest first; the short ones the scaling run is
            # read for come last
            "c4_prefix_turns": c4, "c1_decode": c1, "c3_hybrid_token": c3, "lm_head_argmax": lm_head,
            "bulk_append": producer, "gated_delta_step": recurrent, "prefix_restore": restore,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": alg_per_launch * ratio if ratio else None,
                         "kernel": "attention_mma_kernel<128> (fused append + paged decode attention)",
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8tbs": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": alg_per_launch, "launch_us": launch_us},
            "cpu_baseline": {"value": cpu_gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                             "sample": f"24 steps of ONE layer of ONE sequence at ctx {CTX} (about 20 s of core time) through the CPU "
                                       "restatement of the reference path (oracle/), f32 storage of bf16-rounded K/V"},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": te / e2e_steps * 1e3,
                    "no_overlap_value": e2e_serial_value, "no_overlap_ms_per_step": ts / e2e_steps * 1e3,
                    "call": "sgk_step_run_host (pinned host k,v,q in; out back; synchronous)"},
            "gpu_launches": int(launches), "clocks": clocks, "device_status": status, "outputs_finite": finite,
            "seed_seconds": t_seed,
            "c5_serving": c5,
            "batch1": {"us_per_layer": b1_us_layer, "hbm_gbs": b1_gbs, "steps": b1_steps,
                       "frac_of_peak": b1_gbs / peak, "frac_of_nominal_8tbs": b1_gbs / 8000.0},
            "head_sharded_batch1": head_sharded,
            "parity_spot": spot,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


class _Ptr:
    """Lets a torch tensor stand where the ABI face expects a device buffer."""

    def __init__(self, tensor):
        self.tensor = tensor
        self.ptr = tensor.data_ptr()


def guarded(leg, *args):
    """Runs a side measurement; a failure becomes {"error": ...} in the JSON line."""
    try:
        return leg(*args)
    except Exception as exc:  # noqa: BLE001 - whatever it was, the headline still gets printed
        return {"error": f"{type(exc).__name__}: {exc}"[:300]}


def head_sharded_leg(sg, st, torch, dist, world, rank, stream):
    """Set-up is local and may fail on one rank only, so the ranks agree on it (one all-reduce of a
    flag) before any of them enters the collective part."""
    setup, err = None, None
    try:
        setup = head_sharded_setup(sg, st, torch, world, rank)
    except Exception as exc:  # noqa: BLE001
        err = f"{type(exc).__name__}: {exc}"[:300]
    dev = torch.device("cuda", torch.cuda.current_device())
    flag = torch.tensor([0 if err else 1], device=dev, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 0:
        return {"error": err or "set-up failed on another rank"}
    return head_sharded_run(sg, st, torch, dist, world, rank, stream, *setup)


def head_sharded_setup(sg, st, torch, world, rank):
    """One long sequence (batch 1) split by KV-head group over the ranks: every rank appends and
    attends over its heads' pages, then ONE all-gather of attention outputs per layer (NCCL)."""
    from saragossa_b200 import sharding
    sh = sharding.head_shard(Q_HEADS, KV_HEADS, world, rank)
    steps = 8
    kv_loc, q_loc = sh.kv_heads * HEAD_DIM, sh.q_heads * HEAD_DIM
    capacity = ((CTX + 3 * steps + 24 + 15) // 16) * 16
    pool = st.pool(LAYERS, sh.kv_heads, HEAD_DIM, sg.KV_BF16, capacity // 16, 1, capacity)
    pool.shuffle_free_list(3)
    seq = pool.sequence(capacity)
    kvs = [seq.layer(layer, sh.q_heads) for layer in range(LAYERS)]
    chunk = 8192
    dk, dv = st.alloc(chunk * kv_loc * 4), st.alloc(chunk * kv_loc * 4)
    for layer in range(LAYERS):
        for c in range(0, CTX, chunk):
            n = min(chunk, CTX - c)
            st.fill_normal(dk, n * kv_loc, 7, (layer * world + rank) * 2, c * kv_loc)
            st.fill_normal(dv, n * kv_loc, 7, (layer * world + rank) * 2 + 1, c * kv_loc)
            kvs[layer].encode_append_rows(dk, dv, n)
    st.sync()
    dk.free()
    dv.free()
    batches = [sg.Batch(st, [kv]) for kv in kvs]
    return sh, pool, seq, batches, kv_loc, q_loc, steps, kvs


def head_sharded_run(sg, st, torch, dist, world, rank, stream, sh, pool, seq, batches, kv_loc, q_loc, steps, kvs):
    dev = torch.device("cuda", torch.cuda.current_device())
    k = torch.randn(LAYERS, kv_loc, device=dev)
    v = torch.randn(LAYERS, kv_loc, device=dev)
    q = torch.randn(LAYERS, q_loc, device=dev)
    out_loc = torch.zeros(LAYERS, q_loc, device=dev)
    out_full = torch.zeros(LAYERS, world * q_loc, device=dev)
    torch.cuda.synchronize()

    # the rows of the direct exchange: [layer][world * q_loc] in memory the peers map. Mapping may fail
    # on one rank only (no IPC between these processes): the ranks agree after every local stage.
    row = world * q_loc

    def agreed(ok):
        flag = torch.tensor([1 if ok else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return int(flag.item()) == 1

    rows = ex = None
    peer_rows, peer_error, mine = {}, None, None
    try:
        rows = st.alloc(4 * LAYERS * row)
        rows.upload(np.zeros(LAYERS * row, np.float32))
        ex = st.exchange(rank, world)
        mine = (st.peer_export(rows), ex.handle)
    except Exception as exc:  # noqa: BLE001
        peer_error = f"{type(exc).__name__}: {exc}"[:200]
    peers_ok = agreed(peer_error is None)
    if peers_ok:
        handles = [None] * world
        dist.all_gather_object(handles, mine)
        try:
            for p in range(world):
                if p != rank:
                    peer_rows[p] = st.peer_open(handles[p][0])
                    ex.connect(p, handles[p][1])
        except Exception as exc:  # noqa: BLE001
            peer_error = f"{type(exc).__name__}: {exc}"[:200]
        peers_ok = agreed(peer_error is None)

    class _At:
        def __init__(self, ptr):
            self.ptr = ptr

    def step_nccl():
        st.chain_begin(stream.cuda_stream)       # one decode token: every launch lets the next one start early
        for layer in range(LAYERS):
            batches[layer].enqueue_step(_Ptr(k[layer]), _Ptr(v[layer]), _Ptr(q[layer]), _Ptr(out_loc[layer]),
                                        stream=stream.cuda_stream)
            dist.all_gather_into_tensor(out_full[layer], out_loc[layer])
        st.chain_end()

    def step_direct():
        st.chain_begin(stream.cuda_stream)
        for layer in range(LAYERS):
            base = rows.ptr + 4 * layer * row
            batches[layer].enqueue_step(_Ptr(k[layer]), _Ptr(v[layer]), _Ptr(q[layer]), _At(base + 4 * rank * q_loc),
                                        stream=stream.cuda_stream)
            ex.enqueue(base, [0 if p == rank else peer_rows[p].ptr + 4 * layer * row for p in range(world)],
                       rank * q_loc, q_loc, stream=stream.cuda_stream)
        st.chain_end()

    def step_fused():
        st.chain_begin(stream.cuda_stream)
        for layer in range(LAYERS):
            base = rows.ptr + 4 * layer * row
            batches[layer].enqueue_step_exchange(
                _Ptr(k[layer]), _Ptr(v[layer]), _Ptr(q[layer]), ex, base,
                [0 if p == rank else peer_rows[p].ptr + 4 * layer * row for p in range(world)], rank * q_loc,
                stream=stream.cuda_stream)
        st.chain_end()

    # One decode token = 48 x (fused kernel, exchange) as ONE CUDA graph; the pages the replays
    # will append into are reserved before the capture (a replay moves only the device cursor).
    seq.reserve(((CTX + 3 * steps + 24 + 15) // 16) * 16)
    result = {}
    modes = [("nccl", step_nccl)] + ([("direct", step_direct), ("fused", step_fused)] if peers_ok else [])
    # Parity of the exchanges: the SAME decode step (same rows in the cache, same q / k / v) through
    # the NCCL all-gather and through each peer-memory form; every rank compares its whole rows, bit
    # for bit. The cursors go back between the runs (truncate never clears, the appended row is
    # simply written again).
    parity = {}
    if peers_ok:
        base_len = kvs[0].len()
        with torch.cuda.stream(stream):
            step_nccl()
            stream.synchronize()
        want = out_full.detach().cpu().numpy().copy()
        for name, one_step in modes[1:]:
            for kv in kvs:
                kv.truncate(base_len)
            st.sync()
            with torch.cuda.stream(stream):
                one_step()
                stream.synchronize()
            got = rows.download(np.float32, LAYERS * row).reshape(LAYERS, row)
            parity[name] = bool(np.array_equal(got, want))
        for kv in kvs:
            kv.truncate(base_len)
        st.sync()
        flag = torch.tensor([1 if all(parity.values()) else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity["all_ranks"] = int(flag.item()) == 1
    for name, one_step in modes:
        mode = "graph"
        with torch.cuda.stream(stream):
            one_step()
            stream.synchronize()
            dist.barrier()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    one_step()
                run = graph.replay
            except Exception:  # noqa: BLE001 - same code on every rank: they all fall back together
                mode, run = "stream", one_step
            run()
            stream.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                run()
            e1.record(stream)
            stream.synchronize()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        result[name] = (float(t.item()), mode)
    finite = bool(torch.isfinite(out_full).all().item())
    direct_complete = None
    if peers_ok:
        direct_rows = rows.download(np.float32, LAYERS * row).reshape(LAYERS, world, q_loc)
        # every slice of the last token arrived: no slice of any layer is still the initial zero row
        direct_complete = bool(np.isfinite(direct_rows).all() and (np.abs(direct_rows).max(axis=2) > 0).all())
    status = st.device_status()
    dist.barrier()
    for p in peer_rows.values():
        st.peer_close(p)
    if ex is not None:
        ex.close()
    for b in batches:
        b.close()
    seq.close()
    pool.close()
    total_bytes = sum(algorithmic_bytes(CTX + 2 + i + 1) for i in range(steps)) * LAYERS
    ms, mode = result["nccl"]
    nccl = {"us_per_layer": ms * 1e3 / (steps * LAYERS), "submission": mode, "exchange": "NCCL all-gather per layer"}
    if not peers_ok:
        return {"us_per_layer": nccl["us_per_layer"], "hbm_gbs_aggregate": total_bytes / (ms * 1e-3) / 1e9, "ranks": world,
                "kv_heads_per_rank": sh.kv_heads, "steps": steps, "outputs_finite": finite, "device_status": status,
                "submission": mode, "exchange": nccl["exchange"],
                "peer_memory_unavailable": peer_error or "on another rank"}
    ms_d, mode_d = result["direct"]
    ms_f, mode_f = result["fused"]
    return {"us_per_layer": ms_f * 1e3 / (steps * LAYERS), "hbm_gbs_aggregate": total_bytes / (ms_f * 1e-3) / 1e9,
            "ranks": world, "kv_heads_per_rank": sh.kv_heads, "steps": steps, "outputs_finite": finite,
            "all_slices_arrived": direct_complete, "device_status": status, "submission": mode_f,
            "parity_vs_nccl": parity.get("all_ranks"), "parity_fused": parity.get("fused"), "parity_direct": parity.get("direct"),
            "exchange": "fused into the attention launch (peer stores + flags)",
            "exchange_kernel_us_per_layer": ms_d * 1e3 / (steps * LAYERS),
            "nccl_all_gather_us_per_layer": nccl["us_per_layer"]}


def gated_delta_leg(sg, st, torch, stream):
    """One gated-delta token on the recurrent state of config 3's linear layers: 30 layers,
    32 value heads x 128 x 128 f32 (2 MiB per layer per sequence), 8 sequences per launch,
    so each step reads and writes 480 MiB of state once (larger than L2)."""
    layers, n, shape = 30, 8, (16, 32, 128, 128)
    hk, hv, dk, dv = shape
    ssm_len = hv * dv * dk
    states = [sg.LinearAttentionState(st, layers, 0, ssm_len) for _ in range(n)]
    bufs = []
    for j, (count, scale) in enumerate([(hk * dk, 1.0 / dk), (hk * dk, dk ** -0.5), (hv * dv, 1.0)]):
        b = st.alloc(4 * n * count)
        st.fill_normal(b, n * count, 77, j, stream=stream.cuda_stream)
        stream.synchronize()
        bufs.append(st.upload(b.download(count=n * count) * np.float32(scale)))
    bufs.append(st.upload(np.full(n * hv, 0.97, np.float32)))
    bufs.append(st.upload(np.full(n * hv, 0.5, np.float32)))
    d_out = st.alloc(4 * n * hv * dv)

    def step():
        for layer in range(layers):
            sg.encode_gated_delta_step_batch(states, layer, shape, *bufs, d_out, stream=stream.cuda_stream)

    step()
    stream.synchronize()
    # the 30 launches of a step replay as one CUDA graph, as the decode loop would issue them
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step()
    with torch.cuda.stream(stream):
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        stream.synchronize()
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    t = e0.elapsed_time(e1) * 1e-3 / (reps * layers)
    finite = bool(np.isfinite(d_out.download(count=n * hv * dv)).all())
    for s in states:
        s.close()
    nbytes = 2 * 4 * n * ssm_len
    return {"us_per_layer": t * 1e6, "hbm_gbs": nbytes / t / 1e9, "sequences": n, "state_bytes_per_layer": nbytes // 2,
            "outputs_finite": finite, "launches": (2 + 3 + reps) * layers}


def lm_head_leg(sg, st, torch, stream):
    """Greedy epilogue of a token: argmax of W . x over a dense bf16 [151936][2560] weight
    (778 MB, larger than L2, read once per launch), for one row and for the 4 rows of a
    speculative verify that share the pass."""
    vocab, hidden = 151936, 2560
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    w = (torch.randn(vocab, hidden, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    x = torch.randn(4, hidden, device=dev, generator=gen)
    idx = torch.zeros(8, dtype=torch.int32, device=dev)
    out = {"vocab": vocab, "hidden": hidden, "weight_bytes": vocab * hidden * 2}
    launches = 0
    for rows in (1, 4):
        def step():
            st.encode_lm_head_argmax(_Ptr(w), sg.KV_BF16, vocab, hidden, _Ptr(x), _Ptr(idx), n_rows=rows,
                                     stream=stream.cuda_stream)
        with torch.cuda.stream(stream):
            for _ in range(3):
                step()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            stream.synchronize()
            e0.record(stream)
            for _ in range(reps):
                step()
            e1.record(stream)
            stream.synchronize()
        launches += 3 + reps
        t = e0.elapsed_time(e1) * 1e-3 / reps
        with torch.cuda.stream(stream):      # the same launches as members of a token chain (see below)
            st.chain_begin(stream.cuda_stream)
            for _ in range(3):
                step()
            stream.synchronize()
            e0.record(stream)
            for _ in range(reps):
                step()
            e1.record(stream)
            st.chain_end()
            stream.synchronize()
        launches += 3 + reps
        t_chain = e0.elapsed_time(e1) * 1e-3 / reps
        want = torch.argmax(x[:rows] @ w.float().T, dim=1).to(torch.int32)
        out[f"rows{rows}"] = {"us": t * 1e6, "hbm_gbs": vocab * hidden * 2 / t / 1e9,
                              "in_token_chain_us": t_chain * 1e6,
                              "in_token_chain_hbm_gbs": vocab * hidden * 2 / t_chain / 1e9,
                              "matches_torch_argmax": bool((idx[:rows] == want).all().item())}
    del w
    # the same over affine-quantised weights (the format the reference's models ship in): u8 and u4
    # codes, group 64, bf16 scale and bias; bytes = codes + 4 bytes of metadata per group
    from saragossa_b200.resident import AffineWeight
    peak, _ = measured_peak()
    for bits in (8, 4):
        per_word = 32 // bits
        packed = torch.randint(0, 2 ** 31 - 1, (vocab, hidden // per_word), device=dev, generator=gen, dtype=torch.int32)
        scales = (torch.rand(vocab, hidden // 64, device=dev, generator=gen) * (0.02 / (1 << bits)) + 1e-4).to(torch.bfloat16)
        biases = (torch.randn(vocab, hidden // 64, device=dev, generator=gen) * 0.01).to(torch.bfloat16)
        wq = AffineWeight(packed.data_ptr(), scales.data_ptr(), biases.data_ptr(), bits, 64)

        def qstep():
            st.encode_lm_head_argmax_affine(wq, vocab, hidden, _Ptr(x), _Ptr(idx), n_rows=1, stream=stream.cuda_stream)
        with torch.cuda.stream(stream):
            for _ in range(3):
                qstep()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            stream.synchronize()
            e0.record(stream)
            for _ in range(reps):
                qstep()
            e1.record(stream)
            stream.synchronize()
        launches += 3 + reps
        t = e0.elapsed_time(e1) * 1e-3 / reps
        # the same launches as members of a token chain, the way the epilogue runs inside a token's
        # graph: a launch asks for its first weight tiles before it waits for the launch before it
        with torch.cuda.stream(stream):
            st.chain_begin(stream.cuda_stream)
            for _ in range(3):
                qstep()
            stream.synchronize()
            e0.record(stream)
            for _ in range(reps):
                qstep()
            e1.record(stream)
            st.chain_end()
            stream.synchronize()
        launches += 3 + reps
        t_chain = e0.elapsed_time(e1) * 1e-3 / reps
        nbytes = vocab * hidden * bits // 8 + vocab * (hidden // 64) * 4
        # reference value: dequantise on the device with torch and take the argmax
        shifts = torch.arange(per_word, device=dev, dtype=torch.int32) * bits
        codes = ((packed.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)).reshape(vocab, hidden).float()
        deq = codes * scales.float().repeat_interleave(64, dim=1) + biases.float().repeat_interleave(64, dim=1)
        want = torch.argmax(x[:1] @ deq.T, dim=1).to(torch.int32)
        out[f"affine_u{bits}_g64_rows1"] = {"us": t * 1e6, "weight_bytes": nbytes, "hbm_gbs": nbytes / t / 1e9,
                                            "frac_of_peak": nbytes / t / 1e9 / peak,
                                            "in_token_chain_us": t_chain * 1e6,
                                            "in_token_chain_frac_of_peak": nbytes / t_chain / 1e9 / peak,
                                            "matches_torch_argmax": bool((idx[:1] == want).all().item())}
        del packed, scales, biases, codes, deq
    out["launches"] = launches
    return out


def c1_decode_leg(sg, st, torch, stream):
    """Config 1 as stated (the reference's own CPU-runnable case): one sequence, 36 layers,
    32 Q / 8 KV heads, hd128, bf16 pages, context prefilled to 1024 rows, 64 decode steps of
    append + attention; the device runs each token as one CUDA graph of 36 fused launches. The
    CPU restatement of the reference path runs the same token (36 layers) a few times beside it."""
    from oracle import sgo
    layers, qh, kvh, hd, ctx, steps = 36, 32, 8, 128, 1024, 64
    kv_dim, q_dim = kvh * hd, qh * hd
    loop_tokens = 32
    cap = ctx + steps + 2 * loop_tokens + 24
    pool = st.pool(layers, kvh, hd, sg.KV_BF16, cap // 16 + 2, 1, cap)
    pool.shuffle_free_list(1)
    seq = pool.sequence(cap)
    kvs = [seq.layer(layer, qh) for layer in range(layers)]
    dk_, dv_ = st.alloc(ctx * kv_dim * 4), st.alloc(ctx * kv_dim * 4)
    for layer, kv in enumerate(kvs):
        st.fill_normal(dk_, ctx * kv_dim, 0, 2 * layer)
        st.fill_normal(dv_, ctx * kv_dim, 0, 2 * layer + 1)
        kv.encode_append_rows(dk_, dv_, ctx)
    st.sync()
    batches = [sg.Batch(st, [kv]) for kv in kvs]
    step = sg.Step(st, batches)
    d_k, d_v = st.alloc(4 * layers * kv_dim), st.alloc(4 * layers * kv_dim)
    d_q, d_out = st.alloc(4 * layers * q_dim), st.alloc(4 * layers * q_dim)
    st.fill_normal(d_k, layers * kv_dim, 1, 0)
    st.fill_normal(d_v, layers * kv_dim, 1, 1)
    st.fill_normal(d_q, layers * q_dim, 1, 2)
    st.sync()
    step.capture(d_k, d_v, d_q, d_out)
    for _ in range(3):
        step.replay(stream.cuda_stream)
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps - 3):
        step.replay(stream.cuda_stream)
    e1.record(stream)
    stream.synchronize()
    us_token = e0.elapsed_time(e1) * 1e3 / (steps - 3)
    finite = bool(np.isfinite(d_out.download(count=layers * q_dim)).all())
    token_loop = guarded(_c1_token_loop, sg, st, torch, stream, step, (d_k, d_v, d_q, d_out), q_dim, loop_tokens)
    step.close()
    for b in batches:
        b.close()
    seq.close()
    pool.close()
    # the CPU path on the same token: one layer's cache, walked 36 times per token
    threads = min(qh, os.cpu_count() or 1)
    k = sgo.bf16_round(sgo.fill_normal8(ctx * kv_dim, 0, 0)).reshape(ctx, kv_dim)
    v = sgo.bf16_round(sgo.fill_normal8(ctx * kv_dim, 0, 1)).reshape(ctx, kv_dim)
    cache = sgo.LayerKvCache()
    assert cache.append_batch(k, v, kv_dim) == sgo.OK
    q = sgo.fill_normal8(q_dim, 1, 2)
    row = sgo.bf16_round(sgo.fill_normal8(kv_dim, 1, 0))
    t_cpu = []
    for it in range(3):
        t0 = time.perf_counter()
        for _ in range(layers):
            assert cache.append(row[None], row[None], kv_dim) == sgo.OK
            rc, _ = sgo.cached_attention_one(q, np.ctypeslib.as_array(sgo.lib().sgo_cache_keys(cache._h), shape=(cache.len() * kv_dim,)),
                                             np.ctypeslib.as_array(sgo.lib().sgo_cache_values(cache._h), shape=(cache.len() * kv_dim,)),
                                             qh, kvh, hd, threads=threads)
            assert rc == sgo.OK
        t_cpu.append(time.perf_counter() - t0)
    return {"us_per_token": us_token, "us_per_layer": us_token / layers, "launches_per_token": layers,
            "cpu_port_us_per_token": min(t_cpu[1:]) * 1e6, "cpu_threads": threads, "outputs_finite": finite,
            "token_loop": token_loop,
            "shape": "batch 1, 36 layers, 32Q/8KV hd128 bf16, ctx 1024 -> 1088"}


def _c1_token_loop(sg, st, torch, stream, step, bufs, hidden, tokens):
    """The whole token as ONE submission with the index resident on the device: embedding lookup
    by the previous token's index, the 36 layers and the lm_head argmax into the window's ring are
    one CUDA graph per ring slot (sgk_token_capture; tied bf16 151 936 x 4 096 table, 1.24 GB); the
    host reads tokens back 4 behind (depth 4) or after every token (depth 1). Wall clock per token,
    host included. The activations between the pieces are not a model's (no projections or MLP
    here): shapes and dependencies are."""
    d_k, d_v, d_q, d_out = bufs
    vocab = 151936
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    table = (torch.randn(vocab, hidden, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    x = torch.zeros(hidden, device=dev)
    out = {"vocab": vocab, "hidden": hidden, "tokens": tokens, "submissions_per_token": 1,
           "launches_per_token": len(step.batches) + 2}
    for depth in (4, 1):
        win = st.token_window(depth)
        step.token_capture(win, _Ptr(table), sg.KV_BF16, vocab, hidden, _Ptr(x), _Ptr(table), sg.KV_BF16, d_out,
                           d_k, d_v, d_q, d_out)
        step.token_seed(11, stream=stream.cuda_stream)
        for _ in range(min(depth, 2)):                       # warm-up
            step.token_submit(stream.cuda_stream)
        win.drain()
        got, enq = [], 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while len(got) < tokens:
            while enq < tokens and win.inflight < depth:
                step.token_submit(stream.cuda_stream)
                enq += 1
            got.append(win.pop())
        dt = time.perf_counter() - t0
        win.close()
        out[f"depth{depth}_us_per_token"] = dt / tokens * 1e6
        out[f"depth{depth}_tokens_in_range"] = bool(all(0 <= t < vocab for t in got))
    return out


def c3_token_leg(sg, st, torch, stream):
    """Config 3 as it is stated: one sequence, 40 layers, every 4th a full-attention layer
    (16 Q / 2 KV heads, hd256, u8 group-32 pages, context 32768), the other 30 recurrent
    (32 heads x 128 x 128 f32 state + conv history of 8192 channels, kernel 4). One token of the
    whole KV path as ONE CUDA graph: fused append+attention on the attention layers, conv step and
    gated-delta step on the recurrent ones (activation, norms and gates are the caller's there);
    the same token with each recurrent layer as the one-launch decode step (conv + SiLU + norms +
    gates + gated delta) is timed beside it."""
    layers, qh, kvh, hd, ctx = 40, 16, 2, 256, CTX
    attn_layers = [i for i in range(layers) if (i + 1) % 4 == 0]
    rec_layers = [i for i in range(layers) if (i + 1) % 4 != 0]
    kv_dim, q_dim = kvh * hd, qh * hd
    shape = (16, 32, 128, 128)
    hk, hv, dk, dv = shape
    conv_dim, kernel = 2 * hk * dk + hv * dv, 4
    cap = ((ctx + 64 + 15) // 16) * 16
    pool = st.pool(len(attn_layers), kvh, hd, sg.KV_U8G32, cap // 16 + 2, 1, cap)
    pool.shuffle_free_list(5)
    seq = pool.sequence(cap)
    kvs = [seq.layer(i, qh) for i in range(len(attn_layers))]
    chunk = 8192
    dk_, dv_ = st.alloc(chunk * kv_dim * 4), st.alloc(chunk * kv_dim * 4)
    for i, kv in enumerate(kvs):
        for c in range(0, ctx, chunk):
            n = min(chunk, ctx - c)
            st.fill_normal(dk_, n * kv_dim, 3, 2 * i, c * kv_dim)
            st.fill_normal(dv_, n * kv_dim, 3, 2 * i + 1, c * kv_dim)
            kv.encode_append_rows(dk_, dv_, n)
    st.sync()
    seq.reserve(cap)
    batches = [sg.Batch(st, [kv]) for kv in kvs]
    ls = sg.LinearAttentionState(st, len(rec_layers), (kernel - 1) * conv_dim, hv * dv * dk)
    bufs = {}
    for name, n, scale in (("k", kv_dim, 1.0), ("v", kv_dim, 1.0), ("q", q_dim, 1.0), ("gq", hk * dk, 1.0 / dk),
                           ("gk", hk * dk, dk ** -0.5), ("gv", hv * dv, 1.0), ("x", conv_dim, 1.0),
                           ("w", conv_dim * kernel, 0.5)):
        b = st.alloc(4 * n)
        st.fill_normal(b, n, 4, len(bufs))
        st.sync()
        bufs[name] = st.upload(b.download(count=n) * np.float32(scale))
    bufs["g"] = st.upload(np.full(hv, 0.97, np.float32))
    bufs["beta"] = st.upload(np.full(hv, 0.5, np.float32))
    # gates of the one-launch step: sigmoid(0) = 0.5 and exp(-softplus(-3.49)) = 0.97
    bufs["beta_in"] = st.upload(np.zeros(hv, np.float32))
    bufs["gate_in"] = st.upload(np.full(hv, -3.49, np.float32))
    bufs["a_log"] = st.upload(np.zeros(hv, np.float32))
    bufs["dt_bias"] = st.upload(np.zeros(hv, np.float32))
    d_out, d_y, d_c = st.alloc(4 * q_dim), st.alloc(4 * hv * dv), st.alloc(4 * conv_dim)

    def token(one_launch):
        a = r = 0
        st.chain_begin(stream.cuda_stream)   # one decode token: every launch lets the next one start early
        for layer in range(layers):
            if layer in attn_layers:
                batches[a].enqueue_step(bufs["k"], bufs["v"], bufs["q"], d_out, stream=stream.cuda_stream)
                a += 1
            elif one_launch:
                # conv + SiLU + unit norms + gates + gated delta of the layer in one launch
                ls.encode_decode_step(r, shape, bufs["x"], bufs["w"], kernel, bufs["beta_in"], bufs["gate_in"],
                                      bufs["a_log"], bufs["dt_bias"], d_y, stream=stream.cuda_stream)
                r += 1
            else:
                ls.encode_conv_step(r, bufs["x"], bufs["w"], conv_dim, kernel, d_c, stream=stream.cuda_stream)
                ls.encode_gated_delta_step(r, shape, bufs["gq"], bufs["gk"], bufs["gv"], bufs["g"], bufs["beta"], d_y,
                                           stream=stream.cuda_stream)
                r += 1
        st.chain_end()

    def timed(one_launch):
        token(one_launch)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            token(one_launch)
        reps = 20
        with torch.cuda.stream(stream):
            for _ in range(3):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream.synchronize()
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    us = timed(False)
    us_one = timed(True)
    kv_bytes = len(attn_layers) * ctx * kv_dim * 2 * 1.125
    state_bytes = len(rec_layers) * 2 * 4 * hv * dv * dk
    finite = bool(np.isfinite(d_out.download(count=q_dim)).all() and np.isfinite(d_y.download(count=hv * dv)).all())
    for b in batches:
        b.close()
    ls.close()
    seq.close()
    pool.close()
    return {"us_per_token": us, "launches_per_token": len(attn_layers) + 2 * len(rec_layers),
            # the recurrent layers as ONE launch each, SiLU, unit norms and gates included (40 launches)
            "recurrent_layers_as_one_launch_us_per_token": us_one,
            "hbm_gbs": (kv_bytes + state_bytes) / (us * 1e-6) / 1e9, "kv_bytes": kv_bytes, "state_bytes": state_bytes,
            "outputs_finite": finite, "device_status": st.device_status(),
            "shape": "batch 1, ctx 32768: 10 x (16Q/2KV hd256 u8-g32) + 30 x (32 x 128 x 128 f32 state)"}


def c4_prefix_leg(sg, st, torch, stream, turns=2000, decode_steps=128, rank=0, world=1):
    """Config 4 as it is stated: 64 sessions on the 4B shape (36 layers, 8 KV heads, hd128, bf16,
    16-token blocks of 2.25 MiB), every prompt = a 4096-token system prefix + the session's own
    history (512..8192 tokens, seed 1) + 64..512 new tokens; 2000 turns, sessions drawn Zipf
    s=1.1; per turn: match -> restore the matched blocks (physical copy, enqueue-only) -> append
    the unmatched rows -> 128 decode tokens (every token ONE graph replay of the 36 fused
    append+attention launches) -> remember every new full block (one call); LRU eviction under an
    8 GiB budget. With several GPUs a session lives on the GPU its root hash names
    (sharding.rank_of_session) and a rank runs only its sessions' turns. A session's context stops
    growing at 32k tokens (the window of the other configs)."""
    from saragossa_b200 import sharding
    layers, qh, kvh, hd, block = 36, 32, 8, 128, 16
    kv_dim, q_dim = kvh * hd, qh * hd
    budget = 8 << 30
    max_tokens = 32768
    cap = ((max_tokens + decode_steps + 15) // 16) * 16
    page_b = layers * kvh * 2 * 16 * hd * 2
    pool = st.pool(layers, kvh, hd, sg.KV_BF16, budget // page_b + 2 * (cap // 16) + 64, 4, cap)
    pool.shuffle_free_list(8)
    cache = sg.BlockAwarePrefixCache(block, 1 << 20, pool=pool, budget_bytes=budget)
    rng = np.random.default_rng(1)
    n_sessions = 64
    lengths = [4096 + int(x) for x in rng.integers(512, 8193, size=n_sessions)]
    weights = 1.0 / np.arange(1, n_sessions + 1) ** 1.1
    weights /= weights.sum()
    roots = [sg.BlockHash.for_session(f"session-{i}") for i in range(n_sessions)]
    mine = [sharding.rank_of_session(roots[i], world) == rank for i in range(n_sessions)]
    history = [[1_000_000 * (i + 1) + j for j in range(lengths[i] - 4096)] for i in range(n_sessions)]
    chunk = 8192
    d_rows_k, d_rows_v = st.alloc(4 * chunk * kv_dim), st.alloc(4 * chunk * kv_dim)
    st.fill_normal(d_rows_k, chunk * kv_dim, 12, 0)
    st.fill_normal(d_rows_v, chunk * kv_dim, 12, 1)
    d_k, d_v = st.alloc(4 * layers * kv_dim), st.alloc(4 * layers * kv_dim)
    d_q, d_out = st.alloc(4 * layers * q_dim), st.alloc(4 * layers * q_dim)
    st.fill_normal(d_k, layers * kv_dim, 13, 0)
    st.fill_normal(d_v, layers * kv_dim, 13, 1)
    st.fill_normal(d_q, layers * q_dim, 13, 2)
    st.sync()
    sys_prefix = list(range(1, 4097))
    reused_tokens = prompt_tokens = copied_bytes = my_turns = decode_rows = 0
    phase = {"match": 0.0, "restore_enqueue": 0.0, "append_enqueue": 0.0, "capture": 0.0, "decode_enqueue": 0.0,
             "remember": 0.0, "wait": 0.0}
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(2)]
    restore_ms = decode_ms = 0.0
    # The decode lane: ONE sequence with its KV views, batches and step serves turn after turn (a
    # restore or a reset gives it the turn's prefix), so a turn allocates nothing on the device.
    lane = pool.sequence(cap)
    kvs = [lane.layer(layer, qh) for layer in range(layers)]
    batches = [sg.Batch(st, [kv]) for kv in kvs]
    step = sg.Step(st, batches)
    t0 = time.perf_counter()
    for turn in range(turns):
        s_ = int(rng.choice(n_sessions, p=weights))
        n_new = int(rng.integers(64, 513))
        if not mine[s_]:
            continue
        my_turns += 1
        root = roots[s_]
        fresh = [3_000_000_000 + turn * 1000 + i for i in range(n_new)]
        toks = sys_prefix + history[s_] + fresh
        if len(toks) > max_tokens:                   # the context window: the oldest history falls out
            toks = sys_prefix + toks[len(toks) - (max_tokens - 4096):]
        new_len = len(toks)
        t = time.perf_counter()
        hit = cache.match_prefix(root, toks)
        phase["match"] += time.perf_counter() - t
        reused = 0
        t = time.perf_counter()
        if hit is not None:
            ev[0][0].record(stream)
            copied_bytes += cache.restore(hit, lane, stream=stream.cuda_stream)
            ev[0][1].record(stream)
            reused = hit.tokens
        else:
            lane.reset(stream=stream.cuda_stream)
        phase["restore_enqueue"] += time.perf_counter() - t
        reused_tokens += reused
        prompt_tokens += new_len
        t = time.perf_counter()
        for kv in kvs:                                            # the unmatched rows are "prefilled"
            for c in range(reused, new_len, chunk):
                kv.encode_append_rows(d_rows_k, d_rows_v, min(chunk, new_len - c), stream=stream.cuda_stream)
        phase["append_enqueue"] += time.perf_counter() - t
        t = time.perf_counter()
        stream.synchronize()                                      # the capture wants the appends done
        step.capture(d_k, d_v, d_q, d_out)                        # split counts follow this turn's context
        phase["capture"] += time.perf_counter() - t
        t = time.perf_counter()
        ev[1][0].record(stream)
        for _ in range(decode_steps):
            step.replay(stream.cuda_stream)
        ev[1][1].record(stream)
        phase["decode_enqueue"] += time.perf_counter() - t
        t = time.perf_counter()
        stream.synchronize()
        phase["wait"] += time.perf_counter() - t
        if hit is not None:
            restore_ms += ev[0][0].elapsed_time(ev[0][1])
        decode_ms += ev[1][0].elapsed_time(ev[1][1])
        decode_rows += decode_steps * layers * (2 * new_len + decode_steps)
        decoded = [2_000_000_000 + turn * 1000 + i for i in range(decode_steps)]
        toks = toks + decoded
        t = time.perf_counter()
        cache.insert_chain(root, toks, lane, from_tokens=reused, stream=stream.cuda_stream)   # every new full block
        phase["remember"] += time.perf_counter() - t
        history[s_] = toks[4096:]
    step.close()
    for b in batches:
        b.close()
    lane.close()
    stream.synchronize()
    wall = time.perf_counter() - t0
    out = {"turns": turns, "turns_on_this_gpu": my_turns, "decode_steps_per_turn": decode_steps,
           "turns_per_s": my_turns / wall, "ms_per_turn": wall / max(my_turns, 1) * 1e3,
           "decode_tokens_per_s": my_turns * decode_steps / wall,
           "decode_us_per_layer": decode_ms * 1e3 / max(my_turns * decode_steps * layers, 1),
           "decode_hbm_gbs": decode_rows / 2 * kv_dim * 2 * 2 / max(decode_ms * 1e-3, 1e-9) / 1e9,
           "host_ms_per_turn": {k: v / max(my_turns, 1) * 1e3 for k, v in phase.items()},
           "prompt_tokens": prompt_tokens, "reused_tokens": reused_tokens, "hit_rate": reused_tokens / max(prompt_tokens, 1),
           "restore_bytes_read_plus_written": 2 * copied_bytes,
           "restore_gbs": 2 * copied_bytes / max(restore_ms * 1e-3, 1e-9) / 1e9,
           "evicted_blocks": cache.evicted_count(), "cache_entries": len(cache), "cache_bytes": cache.estimated_bytes(),
           "pinned_bytes": cache.pinned_bytes(), "budget_bytes": budget,
           "device_status": st.device_status(),
           "shape": "64 sessions, 36 layers x 8 KV heads x hd128 bf16, 16-token blocks (2.25 MiB), 8 GiB budget, context capped at 32k"}
    cache.close()
    pool.close()
    return out


class _Off:
    """A device pointer at a byte offset inside a DeviceBuffer (what the ctypes face reads is .ptr)."""

    def __init__(self, buf, offset):
        self.ptr = buf.ptr + offset


def c5_serving_leg(sg, st, torch, stream, dist=None, rank=0, world=1, steps=256):
    """Config 5 on every rank; a rank that fails says so in the reduction instead of leaving the
    others waiting in it."""
    try:
        out = _c5_local(sg, st, torch, stream, dist, rank, world, steps)
    except Exception as exc:  # noqa: BLE001
        out = {"error": f"{type(exc).__name__}: {exc}"[:300], "ms_total": 0.0, "alg": 0.0}
    if world > 1:
        ok = 0.0 if "error" in out else 1.0
        t = torch.tensor([out["ms_total"], out["alg"], ok], device="cuda", dtype=torch.float64)
        tmax, tmin = t.clone(), t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        if float(tmin[2].item()) < 1.0:
            return {"error": out.get("error", "another rank failed")}
        out["ms_total"], out["alg"] = float(tmax[0].item()), float(t[1].item())
    if "error" in out:
        return {"error": out["error"]}
    ms_total, alg = out.pop("ms_total"), out.pop("alg")
    ms = ms_total / steps
    out.update({"ms_per_token_step": ms, "us_per_layer": ms * 1e3 / 34,
                "decode_steps_per_s": 256 / (ms * 1e-3), "hbm_gbs": alg / (ms_total * 1e-3) / 1e9,
                "hbm_gbs_per_gpu": alg / world / (ms_total * 1e-3) / 1e9})
    return out


def _c5_local(sg, st, torch, stream, dist, rank, world, steps):
    """Config 5 as it is stated: 256 concurrent sequences, 34 layers (global iff (i + 1) % 6 == 0,
    the others sliding over 1024 rows), 8 Q / 4 KV heads, hd256, bf16 pages, context lengths
    uniform in [1024, 32768] (seed 2), sharded by sequence over the GPUs of the run
    (sharding.sequences_of_rank: 256 / N per GPU, no collective on the data path), 256 decode
    steps. Sliding layers live in their own pool and hold only the pages of the window (older
    pages are released), which is what lets one GPU hold all 256 sequences (about 118 GB instead
    of 600). One decode token for all of a GPU's sequences = 34 launches in one CUDA graph; the
    time is the max over the ranks, the rate the whole job's."""
    from saragossa_b200 import sharding
    total_seq, layers, qh, kvh, hd, window = 256, 34, 8, 4, 256, 1024
    kv_dim, q_dim = kvh * hd, qh * hd
    g_layers = [i for i in range(layers) if (i + 1) % 6 == 0]
    s_layers = [i for i in range(layers) if (i + 1) % 6 != 0]
    rng = np.random.default_rng(2)
    all_lens = [int(x) for x in rng.integers(1024, 32769, size=total_seq)]
    lens = [all_lens[i] for i in sharding.sequences_of_rank(total_seq, world, rank)]
    n_seq = len(lens)
    grow = steps + 8                       # rows appended by the warm-up and the timed steps
    cap = ((32768 + grow + 32 + 15) // 16) * 16
    own = [((n + grow + 32 + 15) // 16) * 16 for n in lens]
    pages_g = sum(c // 16 for c in own) + 8
    pages_s = n_seq * ((window + grow) // 16 + 12) + cap // 16 + 8
    pool_g = st.pool(len(g_layers), kvh, hd, sg.KV_BF16, pages_g, n_seq, cap)
    pool_s = st.pool(len(s_layers), kvh, hd, sg.KV_BF16, pages_s, n_seq, cap)
    pool_g.shuffle_free_list(6)
    pool_s.shuffle_free_list(7)
    # a capture reserves every page up to a sequence's capacity: the capacity is its own length
    # plus the rows this leg appends, not the longest context of the config
    seqs_g = [pool_g.sequence(c) for c in own]
    seqs_s = [pool_s.sequence(c) for c in own]
    chunk = 8192
    dk_, dv_ = st.alloc(chunk * kv_dim * 4), st.alloc(chunk * kv_dim * 4)
    st.fill_normal(dk_, chunk * kv_dim, 8, 0)
    st.fill_normal(dv_, chunk * kv_dim, 8, 1)
    kv_of = {}
    t_seed = time.perf_counter()
    for b, n in enumerate(lens):
        for li, layer in enumerate(g_layers):
            kv = seqs_g[b].layer(li, qh)
            for c in range(0, n, chunk):
                kv.encode_append_rows(dk_, dv_, min(chunk, n - c))
            kv_of[b, layer] = kv
        # A sliding layer is filled window by window and gives the pages behind its window back as
        # it goes, as a server does while the sequence grows: its pool never holds the whole context.
        first = True
        for c in range(0, n, window):
            for li, layer in enumerate(s_layers):
                kv = seqs_s[b].layer(li, qh) if first else kv_of[b, layer]
                kv.encode_append_rows(dk_, dv_, min(window, n - c))
                kv_of[b, layer] = kv
            first = False
            st.sync()
            seqs_s[b].release_before(max(min(c + window, n) - window, 0))
    st.sync()
    t_seed = time.perf_counter() - t_seed
    batches = [sg.Batch(st, [kv_of[b, layer] for b in range(n_seq)]) for layer in range(layers)]
    step = sg.Step(st, batches)
    d_k, d_v = st.alloc(4 * layers * n_seq * kv_dim), st.alloc(4 * layers * n_seq * kv_dim)
    d_q, d_out = st.alloc(4 * layers * n_seq * q_dim), st.alloc(4 * layers * n_seq * q_dim)
    st.fill_normal(d_k, layers * n_seq * kv_dim, 9, 0)
    st.fill_normal(d_v, layers * n_seq * kv_dim, 9, 1)
    st.fill_normal(d_q, layers * n_seq * q_dim, 9, 2)
    st.sync()
    windows = [0 if layer in g_layers else window for layer in range(layers)]
    step.capture(d_k, d_v, d_q, d_out, sliding_windows=windows)
    for _ in range(3):
        step.replay(stream.cuda_stream)
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step.replay(stream.cuda_stream)
    e1.record(stream)
    stream.synchronize()
    ms_total = e0.elapsed_time(e1)
    row_bytes = kv_dim * 2 * 2
    alg = sum(len(g_layers) * (n + 3 + i + 1) * row_bytes + len(s_layers) * min(n + 3 + i + 1, window) * row_bytes
              for n in lens for i in range(steps))
    held_s = pool_s.num_pages - pool_s.free_pages
    held_g = pool_g.num_pages - pool_g.free_pages
    finite = bool(np.isfinite(d_out.download(count=n_seq * q_dim)).all())
    status = st.device_status()
    resident_gb = (held_s * pool_s.page_bytes + held_g * pool_g.page_bytes) / 1e9
    step.close()
    for b in batches:
        b.close()
    for s_ in seqs_g + seqs_s:
        s_.close()
    pool_g.close()
    pool_s.close()
    return {"n_gpus": world, "sequences": total_seq, "sequences_per_gpu": n_seq, "decode_steps": steps,
            "ms_total": ms_total, "alg": float(alg),
            "mean_context": float(np.mean(all_lens)), "kv_resident_gb_this_gpu": resident_gb,
            "sliding_pool_pages_held": int(held_s), "sliding_pool_pages_if_kept": int(sum((n + 15) // 16 for n in lens)),
            "seed_seconds": t_seed, "outputs_finite": finite, "device_status": status,
            "shape": "5 global + 29 sliding-1024 layers, 8Q/4KV hd256 bf16, contexts U(1k,32k) seed 2, by sequence"}


def bulk_append_leg(sg, st, torch, stream):
    """The prefill-side producer on the shape of config 4 (8 KV heads x hd128): 4096 prompt rows
    of one layer per launch, f32 in (K and V), pages out; plain bf16, with RMSNorm+RoPE on K, and
    u8 group-32. Bytes = what is read plus what is written."""
    kvh, hd, rows, reps = 8, 128, 4096, 8
    kv_dim = kvh * hd
    d_k, d_v = st.alloc(4 * rows * kv_dim), st.alloc(4 * rows * kv_dim)
    st.fill_normal(d_k, rows * kv_dim, 91, 0, stream=stream.cuda_stream)
    st.fill_normal(d_v, rows * kv_dim, 91, 1, stream=stream.cuda_stream)
    d_w = st.upload(np.ones(hd, np.float32))
    rope = sg.make_rope(hd, 1_000_000.0, eps=1e-6)
    out = {}
    for name, dtype, roped, store in (("bf16", sg.KV_BF16, False, 2.0), ("bf16_rope", sg.KV_BF16, True, 2.0),
                                      ("u8", sg.KV_U8G32, False, 1.125)):
        # the layers of one prompt chunk: every layer appends the same positions (with rope, the
        # cos/sin table made for the first layer's launch serves the others)
        kvs = [st.full_attention(rows * 3, 32, kvh, hd, dtype) for _ in range(reps)]

        def one(kv):
            if roped:
                kv.encode_rope_append_rows(d_k, d_v, rows, d_w, rope, stream=stream.cuda_stream)
            else:
                kv.encode_append_rows(d_k, d_v, rows, stream=stream.cuda_stream)

        for kv in kvs:
            one(kv)
        for kv in kvs:
            one(kv)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        st.sync()
        e0.record(stream)
        for kv in kvs:
            one(kv)
        e1.record(stream)
        stream.synchronize()
        t = e0.elapsed_time(e1) * 1e-3 / reps
        nbytes = rows * kv_dim * (4 * 2 + store * 2)
        out[name] = {"us_per_launch": t * 1e6, "hbm_gbs": nbytes / t / 1e9}
        for kv in kvs:
            kv.close()
    out["shape"] = f"{rows} rows x {kvh} KV heads x hd{hd} per launch, {reps} layers of one prompt chunk"
    return out


def prefix_restore_gbs(sg, st, torch, stream):
    """Restore (physical copy) of a cached 4096-token prefix on the shape of config 4:
    36 layers x 8 KV heads x hd128 bf16, 16-token blocks of 2.25 MiB."""
    layers, kvh, hd, tokens = 36, 8, 128, 4096
    pages = tokens // 16
    pool = st.pool(layers, kvh, hd, sg.KV_BF16, 3 * pages + 8, 4, tokens + 64)
    pool.shuffle_free_list(1)
    page_bytes = pool.page_bytes
    src = pool.sequence(tokens + 64)
    src.reserve(tokens)
    for layer in range(layers):
        src.layer(layer, 32).truncate(tokens)      # the rows hold the pool's zero fill: a copy does not care
    cache = sg.BlockAwarePrefixCache(16, 100000, pool=pool)
    root = sg.BlockHash.for_session("bench")
    toks = list(range(tokens))
    prev = root
    for i in range(pages):        # every block boundary is remembered, as the serve loop does
        prev = sg.BlockHash.chain(prev, toks[16 * i:16 * i + 16])
        cache.insert(root, prev, 16 * (i + 1), seq=src)
    hit = cache.match_prefix(root, toks)
    assert hit is not None and hit.tokens == tokens
    dst = pool.sequence(tokens + 64)
    call = []
    for it in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        st.sync()
        e0.record(stream)
        copied = cache.restore(hit, dst, stream=stream.cuda_stream)
        e1.record(stream)
        stream.synchronize()
        if it >= 2:
            call.append((e0.elapsed_time(e1) * 1e-3, copied))
    t_call, copied = min(call)
    # the call only enqueues: restores issued back to back keep the device busy while the host
    # prepares the next one (a server restoring several lanes); two lanes take turns
    dst2 = pool.sequence(tokens + 64)
    burst = 8
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream.synchronize()
    e0.record(stream)
    for it in range(burst):
        cache.restore(hit, dst if it % 2 == 0 else dst2, stream=stream.cuda_stream)
    e1.record(stream)
    stream.synchronize()
    t_burst = e0.elapsed_time(e1) * 1e-3 / burst
    dst2.close()
    dst.close()
    src.close()
    cache.close()
    pool.close()
    # the block-copy kernel alone, on the same page size with shuffled source and destination lists
    n = 512
    a, b = st.alloc(n * page_bytes), st.alloc(n * page_bytes)
    rng = np.random.default_rng(0)
    src_pages = st.upload(rng.permutation(n).astype(np.int32))
    dst_pages = st.upload(rng.permutation(n).astype(np.int32))
    for _ in range(3):
        st.copy_blocks(b, a, n, page_bytes, dst_pages, src_pages, stream=stream.cuda_stream)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    e0.record(stream)
    for _ in range(reps):
        st.copy_blocks(b, a, n, page_bytes, dst_pages, src_pages, stream=stream.cuda_stream)
    e1.record(stream)
    stream.synchronize()
    t_kernel = e0.elapsed_time(e1) * 1e-3 / reps
    a.free()
    b.free()
    peak, kind = measured_peak()
    kernel_gbs = 2 * n * page_bytes / t_kernel / 1e9
    call_gbs = 2 * copied / t_call / 1e9
    return {"gbs": kernel_gbs, "frac_of_copy_peak": kernel_gbs / peak, "peak_kind": f"of {kind}",
            "kernel": "copy_pages_kernel, 512 blocks of 2.25 MiB, shuffled lists, read+write bytes / time",
            "restore_call_gbs": call_gbs, "restore_call_ms": t_call * 1e3, "restore_call_tokens": tokens,
            "restore_calls_back_to_back_gbs": 2 * copied / t_burst / 1e9,
            "restore_calls_back_to_back_frac_of_copy_peak": 2 * copied / t_burst / 1e9 / peak,
            "restore_call_bytes_copied": copied,
            "shape": "36 layers, 8 KV heads, hd128, bf16, 16-token blocks (2.25 MiB per block)"}


def run_leg(args):
    import torch
    import saragossa_b200 as sg
    torch.cuda.set_device(0)
    st = sg.DecodeResidentState(0)
    stream = torch.cuda.Stream()
    legs = {"prefix_restore": lambda: prefix_restore_gbs(sg, st, torch, stream),
            "gated_delta_step": lambda: gated_delta_leg(sg, st, torch, stream),
            "bulk_append": lambda: bulk_append_leg(sg, st, torch, stream),
            "c3_hybrid_token": lambda: c3_token_leg(sg, st, torch, stream),
            "c5_serving": lambda: c5_serving_leg(sg, st, torch, stream),
            "c4_prefix_turns": lambda: c4_prefix_leg(sg, st, torch, stream, args.c4_turns, 128),
            "c1_decode": lambda: c1_decode_leg(sg, st, torch, stream),
            "lm_head_argmax": lambda: lm_head_leg(sg, st, torch, stream)}
    print(json.dumps({args.leg: legs[args.leg]()}), flush=True)


def main():
    global LAYERS, BATCH, CTX, Q_HEADS, KV_HEADS, HEAD_DIM, KV_DIM, Q_DIM, KV_DTYPE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # profiling aids: a smaller copy of the same workload for ncu captures (not a bench value)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--ctx", type=int, default=CTX)
    ap.add_argument("--q-heads", type=int, default=Q_HEADS)
    ap.add_argument("--kv-heads", type=int, default=KV_HEADS)
    ap.add_argument("--head-dim", type=int, default=HEAD_DIM)
    ap.add_argument("--kv-dtype", default=KV_DTYPE, choices=["bf16", "u8"])
    ap.add_argument("--skip-extras", action="store_true",
                    help="only the device-resident timing (no e2e, batch-1, prefix-restore or CPU legs)")
    ap.add_argument("--leg", default=None,
                    choices=["prefix_restore", "gated_delta_step", "bulk_append", "c3_hybrid_token", "c5_serving",
                             "c4_prefix_turns", "c1_decode", "lm_head_argmax"],
                    help="profiling aid: run ONE of the side legs on one GPU and print its JSON (not a bench line)")
    ap.add_argument("--c4-turns", type=int, default=2000, help="turns of the config-4 leg (2000 as stated)")
    args = ap.parse_args()
    if args.leg:
        return run_leg(args)
    reduced = (args.layers, args.batch, args.ctx, args.q_heads, args.kv_heads, args.head_dim, args.kv_dtype) != (
        LAYERS, BATCH, CTX, Q_HEADS, KV_HEADS, HEAD_DIM, KV_DTYPE)
    LAYERS, BATCH, CTX = args.layers, args.batch, args.ctx
    Q_HEADS, KV_HEADS, HEAD_DIM, KV_DTYPE = args.q_heads, args.kv_heads, args.head_dim, args.kv_dtype
    KV_DIM, Q_DIM = KV_HEADS * HEAD_DIM, Q_HEADS * HEAD_DIM
    args.reduced = reduced
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
