"""Benchmark of the quantized-matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (benchmark config 4): the 224 Q4_0 projections of a 7B-shape Llama decoder, batch 1,
every weight a distinct buffer (3.64 GB per token, far larger than L2, so every step reads
HBM cold).  One step = one token = all projections in layer order, run as ONE persistent
kernel per GPU (`--mode graph`: one kernel per projection, recorded once as a CUDA graph).
With N > 1 ranks the weights are row-sharded and every rank ends with all rows of every
projection: the persistent kernel stores its rows into the other ranks' buffers over NVLink
from inside the GEMV epilogue (graph mode: a gather kernel after every projection).
Strong scaling: the same token stream on more GPUs.
The dominant kernel is the Q4_0 decode GEMV, so `roofline` is the headline "Q4_0 GEMV HBM
GB/s (% of peak)"; `gemv_sweep` adds benchmark config 2 (the [11008x4096] / [4096x11008]
sweep at batch 1, 4, 8 -- plus 16 and 32, which the same memory-bound kernel takes -- and the [32000x4096]
vocabulary projection of config 4 at batch 1), one launch per call, timed over rotating weight copies (300 MB,
larger than L2).

Inputs are seeded synthetic GGUF blocks with the configs' value distributions; there is no
dataset behind this path.  `--impl reference` times the CPU restatement of the reference's
own path (block dequant to fp32 + sequential fp32 dot, oracle/wf_oracle.c) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_s_7b_q4_0"
UNIT = "tok/s"
WORKLOAD = ("benchmark config 4: 7B-shape Llama decode, 224 Q4_0 projections (32 layers x "
            "{4x[4096x4096], 2x[11008x4096], [4096x11008]}), batch 1, bf16 activations, fp32 out")


# DRAM traffic of the decode kernel, from the ncu capture summarised in profiles/gemv1_program_q4_0_decode_7b.md
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch over two layers of this workload);
# traffic grows in proportion to the layers run and splits evenly over row shards.  To be re-captured whenever the
# kernel changes.
NCU_TRAFFIC_BYTES_PER_LAYER = (227.78e6 + 4.19e6) / 2


def tensor_peaks():
    """(burst, sustained) dense bf16 TFLOP/s."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured (MEASURED_PEAKS.json, cuBLAS bf16)"
    return 1590.0, 1400.0, "fallback (no MEASURED_PEAKS.json)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json, stream copy)"
    return 6650.0, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler:
    """nvidia-smi clock / throttle samples taken while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows, self.proc, self.device_index = [], None, device_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.device_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_layer_time(orc, spec, threads: int, repeats: int) -> float:
    """Seconds for one layer (7 projections, batch 1) on the CPU path."""
    from oracle import oracle as O
    from warpforge_b200 import quant as Q

    oq = {"Q4_0": O.Q4_0, "Q8_0": O.Q8_0, "Q4_K": O.Q4_K}[spec.qtype.name]
    mats = []
    for i, (name, rows, k) in enumerate(spec.projections):
        blocks = Q.synth_weight(spec.qtype, rows, k, Q.config_seed(spec.config, i))
        x = Q.bf16_bits_to_float(Q.synth_activation_bf16(1, k, Q.config_seed(spec.config, 100 + k)))
        mats.append((blocks, rows, k, x))
    best = float("inf")
    for _ in range(repeats):
        t = time.perf_counter()
        for blocks, rows, k, x in mats:
            orc.qlinear(oq, blocks, rows, k, x, nthreads=threads)
        best = min(best, time.perf_counter() - t)
    return best


def run_reference(args) -> None:
    """The reference's own CPU implementation of the path (restated in C), all host threads.
    Each step is a bounded sample: one of the 32 identical-shape layers; tokens/s follows by
    dividing by the layer count."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    from warpforge_b200.decode import LLAMA_7B_Q4_0 as spec

    orc = O.COracle()
    threads = orc.max_threads()
    for _ in range(max(args.warmup, 1)):
        cpu_layer_time(orc, spec, threads, 1)
    times = [cpu_layer_time(orc, spec, threads, 1) for _ in range(args.steps)]
    t_layer = float(np.mean(times))
    tok_s = 1.0 / (t_layer * spec.layers)
    sample = f"1 of {spec.layers} layers per step (7 projections, 114 MB of Q4_0 blocks), x{spec.layers} for a token"
    # ms_per_step is what a step really took (the one-layer sample), so that steps x ms_per_step is this run's wall time;
    # `value` is the token rate that follows for the 32 identical layers
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t_layer * 1e3, "ms_per_token_extrapolated": t_layer * spec.layers * 1e3,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "timed": sample},
            "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def gemv_sweep(ctx, hbm_peak: float) -> list:
    """benchmark config 2: cold-HBM Q4_0 GEMV at batch 1/4/8 (and 16/32) over 12 rotating weight copies."""
    from warpforge_b200 import _native as N, quant as Q
    from warpforge_b200.backend import QuantizedWeight

    out, lib, qt = [], ctx._lib, Q.QuantizationType.Q4_0
    iters = 120
    # the two shapes of config 2 at batch 1 / 4 / 8, and config 4's vocabulary projection (lm_head, 73.7 MB) at batch 1
    for rows, k, batches, copies in ((11008, 4096, (1, 4, 8, 16, 32), 12), (4096, 11008, (1, 4, 8, 16, 32), 12), (32000, 4096, (1,), 4)):
        blocks = Q.synth_q4_0(rows, k, Q.config_seed(2, rows))
        ws = [QuantizedWeight(ctx, qt, blocks, rows, k) for _ in range(copies)]
        for m in batches:
            x = Q.synth_activation_bf16(m, k, Q.config_seed(2, m))
            dx, dy = ctx.allocate(x.nbytes), ctx.allocate(m * rows * 4)
            ctx.copy_to_device(dx, x)
            for i in range(copies):
                ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, ws[i].handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0))
            ctx.synchronize()
            ctx.graph_begin()
            for i in range(iters):
                ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, ws[i % copies].handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0))
            g = ctx.graph_end()
            e0, e1 = ctx.create_event(), ctx.create_event()
            ctx.graph_launch(g)
            ctx.synchronize()
            best = float("inf")
            for _ in range(3):
                ctx.record_event(e0)
                ctx.graph_launch(g)
                ctx.record_event(e1)
                ctx.synchronize()
                best = min(best, ctx.elapsed_ms(e0, e1) / iters)
            alg = rows * qt.row_bytes(k) + x.nbytes + m * rows * 4
            gbs = alg / best / 1e6
            out.append({"shape": [rows, k], "batch": m, "us": round(best * 1e3, 3), "GB/s": round(gbs, 1),
                        "frac_of_measured_peak": round(gbs / hbm_peak, 4), "frac_of_8TBs": round(gbs / 8000.0, 4)})
            if rows == 32000:
                out[-1]["role"] = "lm_head of config 4 (not part of the timed step)"
            if m > 8:
                out[-1]["note"] = "beyond config 2's batches: the several-token decode kernel's range"
            ctx.graph_destroy(g)
            ctx.free(dx)
            ctx.free(dy)
        for w in ws:
            w.close()
    return out


def parity_stats(orc, want, got) -> dict:
    """The three error measures of the path: the reference's elementwise rule (count of failures), the largest
    error against the largest output, and against each output floored at 1 % of the output RMS."""
    d = np.abs(got.astype(np.float64) - want.astype(np.float64))
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    return {"elements": int(want.size),
            "rule_failures": int(orc.count_not_close(want, got, 1e-4, 1e-3)),
            "max_rel": float(np.max(d) / max(float(np.max(np.abs(want))), 1e-30)),
            "max_rel_floored": float(np.max(d / np.maximum(np.abs(want), max(0.01 * rms, 1e-30))))}


def step_parity(stack, rank: int, world: int, dist) -> dict:
    """After a step every rank holds all rows of every projection: compare the gathered outputs of a [4096]-wide and
    an [11008]-wide projection with the CPU oracle on rows sampled from EVERY rank's row range."""
    from oracle import oracle as O
    from warpforge_b200 import quant as Q

    orc = O.COracle()
    spec = stack.spec
    per_rank = max(8, 64 // world)
    out = {"checked": True, "rows_sampled_per_output": per_rank * world, "outputs": [], "max_rel": 0.0, "rule_failures": 0,
           "elements": 0}
    for name in ("wq", "wgate"):
        rows, k = next((r, kk) for n, r, kk in spec.projections if n == name)
        got = stack.read_output(name)
        rng = np.random.default_rng(1000 + rows)
        shard = rows // world
        sample = np.sort(np.concatenate([r * shard + rng.choice(shard, per_rank, replace=False) for r in range(world)]))
        want = orc.qlinear_rows(O.Q4_0, stack.blocks[name], k, Q.bf16_bits_to_float(stack.x_host[k]), sample, nthreads=orc.max_threads())
        st = parity_stats(orc, want, got[:, sample])
        out["outputs"].append(name)
        out["max_rel"] = max(out["max_rel"], st["max_rel"])
        out["rule_failures"] += st["rule_failures"]
        out["elements"] += st["elements"]
    if dist is not None:
        import torch

        t = torch.tensor([out["max_rel"], float(out["rule_failures"])], dtype=torch.float64)
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        out["max_rel"], out["rule_failures"] = float(mx[0]), int(sm[1])
        out["elements"] *= world
        out["ranks_checked"] = world
    out["ok"] = bool(out["max_rel"] <= 1e-3)
    return out


def gemm_leg(ctx) -> dict:
    """benchmark config 3: Q4_K prefill GEMM, M=512, N=14336, K=4096, bf16 activations, fp32 out.  Events around 64
    calls over 8 rotating weight copies (264 MB of tiles, twice L2); the activation pre-pass is part of every call."""
    from oracle import oracle as O
    from warpforge_b200 import _native as N, quant as Q
    from warpforge_b200.backend import QuantizedWeight

    rows, k, m, copies, calls = 14336, 4096, 512, 8, 64
    lib, qt = ctx._lib, Q.QuantizationType.Q4_K
    blocks = Q.synth_q4_k(rows, k, Q.config_seed(3))
    xb = Q.synth_activation_bf16(m, k, Q.config_seed(3))
    ws = [QuantizedWeight(ctx, qt, blocks, rows, k) for _ in range(copies)]
    dx, dy = ctx.allocate(xb.nbytes), ctx.allocate(m * rows * 4)
    ctx.copy_to_device(dx, xb)
    for i in range(copies):
        ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, ws[i].handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0))
    ctx.synchronize()
    e0, e1 = ctx.create_event(), ctx.create_event()
    best = float("inf")
    for _ in range(3):
        ctx.record_event(e0)
        for i in range(calls):
            ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, ws[i % copies].handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0))
        ctx.record_event(e1)
        ctx.synchronize()
        best = min(best, ctx.elapsed_ms(e0, e1) / calls)
    got = np.empty((m, rows), np.float32)
    ctx.copy_to_host(got, dy)
    orc = O.COracle()
    rng = np.random.default_rng(3)
    sample = np.sort(np.concatenate([b * 128 + rng.choice(128, 1) for b in range(rows // 128)]))
    want = orc.qlinear_rows(O.Q4_K, blocks, k, Q.bf16_bits_to_float(xb), sample, nthreads=orc.max_threads())
    par = parity_stats(orc, want, got[:, sample])
    burst, sustained, src = tensor_peaks()
    tf = 2.0 * m * rows * k / (best * 1e-3) / 1e12
    for w in ws:
        w.close()
    ctx.free(dx)
    ctx.free(dy)
    return {"workload": "benchmark config 3: Q4_K [14336x4096] x 512 bf16 tokens, fp32 out", "us": round(best * 1e3, 2),
            "TFLOP/s": round(tf, 1), "frac_of_measured_burst": round(tf / burst, 4), "frac_of_measured_sustained": round(tf / sustained, 4),
            "peak_burst_tflops": burst, "peak_sustained_tflops": sustained, "peak_source": src,
            "timed": f"{calls} calls over {copies} weight copies, activation pre-pass included, best of 3",
            "parity": dict(par, rows_sampled=int(sample.size), note="one weight row per 128-row block, all 512 tokens; the GEMM rounds each "
                           "dequantized weight once to fp16, so the elementwise rule is reported, not required")}


def q8_0_leg(ctx, hbm_peak: float) -> dict:
    """benchmark config 1: one Q8_0 linear [4096x4096], fp32 activations [1x4096], fp32 out."""
    from oracle import oracle as O
    from warpforge_b200 import _native as N, quant as Q
    from warpforge_b200.backend import QuantizedWeight

    rows, k, copies, iters = 4096, 4096, 12, 120
    lib, qt = ctx._lib, Q.QuantizationType.Q8_0
    blocks = Q.synth_q8_0(rows, k, Q.config_seed(1))
    x = Q.synth_activation_f32(1, k, Q.config_seed(1))
    ws = [QuantizedWeight(ctx, qt, blocks, rows, k) for _ in range(copies)]
    dx, dy = ctx.allocate(x.nbytes), ctx.allocate(rows * 4)
    ctx.copy_to_device(dx, x)
    for i in range(copies):
        ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, ws[i].handle, dx, N.WF_DTYPE_F32, 1, 1, dy, 1, 0))
    ctx.synchronize()
    ctx.graph_begin()
    for i in range(iters):
        ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, ws[i % copies].handle, dx, N.WF_DTYPE_F32, 1, 1, dy, 1, 0))
    g = ctx.graph_end()
    e0, e1 = ctx.create_event(), ctx.create_event()
    ctx.graph_launch(g)
    ctx.synchronize()
    best = float("inf")
    for _ in range(3):
        ctx.record_event(e0)
        ctx.graph_launch(g)
        ctx.record_event(e1)
        ctx.synchronize()
        best = min(best, ctx.elapsed_ms(e0, e1) / iters)
    got = np.empty((1, rows), np.float32)
    ctx.copy_to_host(got, dy)
    orc = O.COracle()
    par = parity_stats(orc, orc.qlinear(O.Q8_0, blocks, rows, k, x, nthreads=orc.max_threads()), got)
    alg = rows * qt.row_bytes(k) + x.nbytes + rows * 4
    gbs = alg / best / 1e6
    ctx.graph_destroy(g)
    for w in ws:
        w.close()
    ctx.free(dx)
    ctx.free(dy)
    return {"workload": "benchmark config 1: Q8_0 [4096x4096], fp32 activations [1x4096]", "us": round(best * 1e3, 3), "GB/s": round(gbs, 1),
            "frac_of_measured_peak": round(gbs / hbm_peak, 4), "timed": f"{iters} calls over {copies} weight copies in one CUDA graph, best of 3",
            "parity": par}


def fused_leg(ctx, hbm_peak: float) -> dict:
    """Config 4's stack with real data flow: the fp32 operations between the projections (rms_norm, silu * up,
    residual adds) fused into the one-token program, against the same flow as separate kernels in a CUDA graph.
    Attention is outside the path: Wo reads a fixed row standing in for its output."""
    from oracle import oracle as O
    from warpforge_b200 import quant as Q
    from warpforge_b200.decode import FusedDecoderStack

    st = FusedDecoderStack(ctx, Q.QuantizationType.Q4_0, 4096, 11008, 32, seed=4)
    e0, e1 = ctx.create_event(), ctx.create_event()
    for _ in range(3):
        st.run()
    ctx.synchronize()
    iters = 10
    ctx.record_event(e0)
    for _ in range(iters):
        st.run()
    ctx.record_event(e1)
    ctx.synchronize()
    ms_fused = ctx.elapsed_ms(e0, e1) / iters
    fused_out = {n: st.read(n) for n in ("q_0", "hmid_0", "h1", "h32")}
    # parity of the first layer against the CPU oracle on sampled rows (the whole chain is checked at small sizes in tests/)
    orc = O.COracle()
    rows = np.linspace(0, 4095, 64).astype(np.int64)
    x1 = orc.rms_norm(st.host["h0"].reshape(1, -1), st.host["gamma1_0"], st.eps)
    want_q = orc.qlinear_rows(O.Q4_0, st.blocks[0]["wq"], 4096, x1, rows, nthreads=orc.max_threads()).reshape(-1)
    want_o = orc.qlinear_rows(O.Q4_0, st.blocks[0]["wo"], 4096, st.host["attn_0"].reshape(1, -1), rows, nthreads=orc.max_threads()).reshape(-1)
    want_hmid = st.host["h0"][rows] + want_o
    rel_q = float(np.max(np.abs(fused_out["q_0"][rows] - want_q)) / np.max(np.abs(want_q)))
    rel_h = float(np.max(np.abs(fused_out["hmid_0"][rows] - want_hmid)) / np.max(np.abs(want_hmid)))
    # the same flow as separate kernels, recorded once
    st.issue_unfused()
    ctx.synchronize()
    ctx.graph_begin()
    st.issue_unfused()
    g = ctx.graph_end()
    for _ in range(2):
        ctx.graph_launch(g)
    ctx.synchronize()
    ctx.record_event(e0)
    for _ in range(iters):
        ctx.graph_launch(g)
    ctx.record_event(e1)
    ctx.synchronize()
    ms_graph = ctx.elapsed_ms(e0, e1) / iters
    unfused_h = st.read("h32")
    agree = float(np.max(np.abs(unfused_h - fused_out["h32"])) / max(float(np.max(np.abs(fused_out["h32"]))), 1e-30))
    ctx.graph_destroy(g)
    gbs = st.weight_bytes_per_token() / ms_fused / 1e6
    out = {"workload": "config 4's 224 projections with rms_norm, silu * up and the residual adds fused into the one-token program (fp32 activations flow from projection to projection; attention's output is a fixed row)",
           "tok/s": round(1e3 / ms_fused, 1), "ms_per_token": round(ms_fused, 4), "GB/s": round(gbs, 1), "frac_of_measured_peak": round(gbs / hbm_peak, 4),
           "same_flow_as_separate_kernels_in_a_graph": {"launches_per_token": 32 * 12, "tok/s": round(1e3 / ms_graph, 1), "ms_per_token": round(ms_graph, 4)},
           "parity": {"layer0_q_max_rel": rel_q, "layer0_hmid_max_rel": rel_h, "fused_vs_separate_h32_max_rel": agree, "rows_sampled": 64,
                      "ok": bool(rel_q <= 1e-3 and rel_h <= 1e-3 and agree <= 1e-3 and np.isfinite(fused_out["h32"]).all())}}
    st.close()
    return out


def config5_legs(ctx) -> list:
    """One rank's shard of benchmark config 5 (70B-shape, Q4_K, 8 row shards) on this GPU: batch-16 decode and
    2048-token prefill, three layers of distinct shard weights resident."""
    from warpforge_b200 import bench_config5

    return bench_config5.run(world=8, layers=3, iters=3, ctx=ctx)



def run_ours(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    dist = None
    if world > 1:
        import torch.distributed as dist  # control plane only: id exchange, barrier, max over ranks

        dist.init_process_group("gloo", rank=rank, world_size=world)

    from warpforge_b200.backend import CudaContext
    from warpforge_b200.decode import Communicator, LLAMA_7B_Q4_0, ProjectionStack

    ctx = CudaContext(local_rank)
    comm = None
    spec = LLAMA_7B_Q4_0
    mode = args.mode if args.mode != "auto" else "program"
    replicas = mode == "replicas"  # every rank decodes its own token stream on the whole model: no exchange at all
    if replicas:
        stack = ProjectionStack(ctx, spec, tokens=1, layers=args.layers or None)
        stack.build_program(None)
        stack.mode = "program"
    elif mode == "program":
        # one persistent kernel per token and rank; the row-shard gather is fused into the GEMV
        # epilogue (peer stores), so no communicator is needed
        stack = ProjectionStack(ctx, spec, tokens=1, rank=rank, world=world, layers=args.layers or None)
        handles = None
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, stack.export_buffers())
        stack.build_program(handles)
        stack.mode = "program"
    else:
        if world > 1:
            ids = [Communicator.create_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            comm = Communicator(ctx, ids[0], rank, world)
        stack = ProjectionStack(ctx, spec, tokens=1, comm=comm, layers=args.layers or None)
        if dist is not None:
            dist.barrier()  # the ranks enter their first gather together: its waits for the peers are bounded
        stack.record()

    def barrier():
        ctx.synchronize()
        if dist is not None:
            dist.barrier()

    for _ in range(max(args.warmup, 3)):
        stack.step()
    barrier()
    # every rank's gathered outputs against the CPU oracle, before anything is timed
    parity = None
    if not args.kernel_only and stack.layers == spec.layers or os.environ.get("WF_BENCH_PARITY"):
        parity = step_parity(stack, 0 if replicas else rank, 1 if replicas else world, None if replicas else dist)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "error": "parity check failed", "parity": parity}), flush=True)
            raise SystemExit(3)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = ctx.create_event(), ctx.create_event()
    launches0 = ctx.launch_count()
    barrier()
    ctx.record_event(e0)
    for _ in range(args.steps):
        stack.step()
    ctx.record_event(e1)
    ctx.synchronize()
    ms = ctx.elapsed_ms(e0, e1)
    launches = ctx.launch_count() - launches0
    barrier()

    # end to end through the public step call: pinned host activations in, last output out
    y_out = np.empty((1, spec.projections[-1][1]), np.float32)
    e2e_ms = float("nan")
    if not args.kernel_only:
        pinned_in = {k: ctx.host_alloc(v.nbytes) for k, v in stack.x_host.items()}
        pinned_out = ctx.host_alloc(y_out.nbytes)
        for _ in range(3):
            stack.step_host(stack.x_host, y_out, pinned_in, pinned_out)
        barrier()
        t = time.perf_counter()
        ctx.record_event(e0)
        for _ in range(args.steps):
            stack.step_host(stack.x_host, y_out, pinned_in, pinned_out)
        ctx.record_event(e1)
        ctx.synchronize()
        e2e_ms = max(ctx.elapsed_ms(e0, e1), (time.perf_counter() - t) * 1e3)
    clocks = sampler.stop() if rank == 0 else None

    if dist is not None:
        import torch

        tt = torch.tensor([ms, e2e_ms], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(tt[0]), float(tt[1])

    if rank == 0:
        hbm_peak, peak_src = measured_peaks()
        ms_step = ms / args.steps
        tok_s = 1e3 / ms_step * (world if replicas else 1)
        alg_bytes = stack.algorithmic_bytes_per_step()          # this rank's shard
        n_launch = 1 if mode in ("program", "replicas") else stack.layers * len(spec.projections)
        gbs = alg_bytes / (ms_step * 1e-3) / 1e9
        h2d = sum(v.nbytes for v in stack.x_host.values())
        line = {
            "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak" if replicas else "strong", "vs_baseline": None,
            "dtype": "bf16 activations x 4-bit codes, fp32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "parallelism": (f"{world} independent replicas, one token stream each" if replicas
                                       else f"row-sharded tp{world}" if world > 1 else "single GPU"),
                       "execution": ("one persistent kernel per token, gather fused into the GEMV epilogue (peer stores)"
                                     if mode == "program" else "one persistent kernel per token and replica" if replicas else "CUDA graph of one GEMV kernel per projection"
                                     + (" + its gather (one kernel of peer stores; NCCL with WF_GATHER=nccl)" if world > 1 else "")),
                       "l2": "inputs larger than L2: 3.64 GB of distinct weights per step", "bytes_per_token": spec.bytes_per_token()},
            "e2e": {"value": 1e3 / (e2e_ms / args.steps) * (world if replicas else 1), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(y_out.nbytes)},
            "gpu_launches": int(launches),
            "parity": parity,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": ("gemv1_program_kernel" if mode in ("program", "replicas") else "gemv1_kernel") + "<Q4_0> (one token)", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s",
                         "frac": gbs / hbm_peak, "frac_of_8TBs_nominal": gbs / 8000.0, "peak_source": peak_src,
                         "bytes_per_launch": alg_bytes / n_launch, "us_per_launch": ms_step * 1e3 / n_launch,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAYER * stack.layers / (1 if replicas else world) / n_launch,
                         "traffic_source": "ncu dram bytes of a 2-layer capture (profiles/gemv1_program_q4_0_decode_7b.md), scaled by layers (and 1 / ranks)"},
        }
        if stack.layers != spec.layers:
            line["partial"] = f"{stack.layers} of {spec.layers} layers: a profiling run, not a bench value"
        if args.kernel_only:
            line["e2e"] = None
        if world == 1 and not args.kernel_only:
            line["gemv_sweep"] = gemv_sweep(ctx, hbm_peak)
            lm = [e for e in line["gemv_sweep"] if "role" in e]
            if lm:  # the step with the vocabulary projection added (config 4 lists it separately)
                line["with_lm_head"] = {"value": 1e3 / (line["ms_per_step"] + lm[0]["us"] / 1e3), "unit": line["unit"]}
            from oracle import oracle as O

            orc = O.COracle()
            threads = orc.max_threads()
            t_layer = cpu_layer_time(orc, spec, threads, 2)
            line["cpu_baseline"] = {"value": 1.0 / (t_layer * spec.layers), "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"1 of {spec.layers} layers (7 projections), best of 2, x{spec.layers}"}
            # the other configurations of the path, each a leg of its own (not part of `value`)
            line["gemm"] = gemm_leg(ctx)
            line["q8_0_config1"] = q8_0_leg(ctx, hbm_peak)
            line["config5_rank_shard"] = config5_legs(ctx)
            line["decode_with_fused_glue"] = fused_leg(ctx, hbm_peak)
        print(json.dumps(line), flush=True)
    stack.close()
    if comm is not None:
        comm.close()
    ctx.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="auto", choices=["auto", "graph", "program", "replicas"],
                    help="program: one persistent kernel per token (default); graph: one kernel per projection in a CUDA graph; "
                         "replicas: N > 1 ranks each decode their own stream on the whole model (weak scaling, no exchange)")
    ap.add_argument("--layers", type=int, default=0,
                    help="profiling aid: run only this many of the 32 layers (the line is then marked partial and is not a bench value)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="profiling aid: only the device-timed steps (no end-to-end leg, no GEMV sweep, no CPU baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
