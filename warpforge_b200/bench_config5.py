"""Times one rank's shard of benchmark config 5 (70B-shape projection set, Q4_K, 8 row shards) on one GPU.

    python -m warpforge_b200.bench_config5 [--world 8] [--layers 5] [--iters 3]

Every rank of the row-sharded run does exactly this work between two gathers, so one GPU is enough to
measure it: rows / world of each of the seven projections of a layer, `--layers` distinct copies of each
(the weights of `--layers` layers, > 2 x L2, so every call reads its weights from HBM), walked in layer order.
Two legs: (i) batch-16 decode (16 bf16 tokens through `wf_qlinear`, which routes more than 8 tokens to the
tensor-core kernel) against the HBM roofline, (ii) a 2048-token prefill against the tensor roofline.
The per-layer time times 80 layers is the per-rank step time of the full configuration (stated as an
extrapolation in the output).  Events on the launching stream, three warm-up walks.  One JSON line per leg.

Under `python -m torch.distributed.run --nproc-per-node N -m warpforge_b200.bench_config5 --world N` the N ranks run
the configuration as it is specified: every projection row-sharded N ways, each followed by the gather of
`wf_qlinear_allgather` (peer stores / peer loads over NVLink on one node; NCCL with WF_GATHER=nccl in the
environment), so that every rank holds all rows; the time is the maximum over the ranks.  `--graph` records the
decode walk once and replays it as a CUDA graph.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import _native as N
from . import quant as Q
from .backend import CudaContext, QuantizedWeight
from .decode import LLAMA_70B_Q4_K

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def run(world: int = 8, layers: int = 5, iters: int = 3, ctx: CudaContext | None = None, legs=(("decode_batch16", 16), ("prefill_2048", 2048)),
        graph: bool = False) -> list:
    """Times the legs and returns one dict per leg (rank 0; the other ranks return an empty list)."""
    class A:
        pass

    a = A()
    a.world, a.layers, a.iters = world, layers, iters
    spec = LLAMA_70B_Q4_K
    rank, nranks = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    gather = nranks > 1
    dist = comm = None
    own_ctx = ctx is None
    if own_ctx:
        ctx = CudaContext(int(os.environ.get("LOCAL_RANK", "0")))
    results = []
    if gather:
        import torch.distributed as dist  # control plane only: id exchange, barrier, max over ranks

        from .decode import Communicator

        if a.world != nranks:
            raise SystemExit(f"--world {a.world} must equal the number of ranks {nranks}")
        dist.init_process_group("gloo", rank=rank, world_size=nranks)
        ids = [Communicator.create_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = Communicator(ctx, ids[0], rank, nranks)
    lib, h = ctx._lib, ctx.handle
    qt = spec.qtype
    weights, shard_bytes, shard_macs = [], 0, 0
    for layer in range(a.layers):
        row = []
        for i, (name, rows, k) in enumerate(spec.projections):
            r = rows // a.world
            blocks = Q.synth_weight(qt, r, k, Q.config_seed(5, layer * len(spec.projections) + i) + 7919 * rank)
            if gather:  # the upload reads this rank's rows out of the whole tensor: only those rows are filled in
                full = np.empty((rows, qt.row_bytes(k)), np.uint8)
                full[rank * r:(rank + 1) * r] = blocks
                w = QuantizedWeight(ctx, qt, full, rows, k, rank, nranks)
                del full
            else:
                w = QuantizedWeight(ctx, qt, blocks, r, k)
            row.append((name, r, k, w))
            if layer == 0:
                shard_bytes += r * qt.row_bytes(k)
                shard_macs += r * k
        weights.append(row)
    kmax = max(k for _, _, k in spec.projections)
    rmax = max(r // a.world for _, r, _ in spec.projections)
    hbm, tf, src = peaks()
    e0, e1 = ctx.create_event(), ctx.create_event()
    for leg, m in legs:
        x = Q.synth_activation_bf16(m, kmax, 5)
        dx = ctx.allocate(x.nbytes)
        ctx.copy_to_device(dx, x)
        dy = ctx.allocate(m * rmax * 4 * (nranks if gather else 1))

        def walk(s=0):
            for row in weights:
                for name, r, k, w in row:
                    # the activation buffer is read as [m, k] (row stride k): same bytes for every projection
                    if gather:
                        N.check(name, lib.wf_qlinear_allgather(h, comm.handle, w.handle, dx, N.WF_DTYPE_BF16, m, dy, s), h)
                    else:
                        N.check(name, lib.wf_qlinear(h, w.handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, s), h)

        if gather:
            dist.barrier()  # the ranks enter the first gather together (a peer-store gather waits a bounded time)
        recorded = 0
        if graph and m <= 32:  # the walk recorded once and replayed: the host's per-call cost leaves the timed region
            walk()
            ctx.synchronize()
            stream = ctx.create_stream()
            ctx.graph_begin(stream)
            walk(stream)
            recorded = ctx.graph_end(stream)

            def walk(s=0, _g=recorded, _s=stream):
                ctx.graph_launch(_g, _s)

        for _ in range(3):
            walk()
        ctx.synchronize()
        if gather:
            dist.barrier()
        ts = stream if recorded else 0
        if recorded:
            ctx.synchronize(ts)
        ctx.record_event(e0, ts)
        for _ in range(a.iters):
            walk()
        ctx.record_event(e1, ts)
        ctx.synchronize(ts)
        ms = ctx.elapsed_ms(e0, e1)
        if recorded:
            ctx.graph_destroy(recorded)
            ctx.destroy_stream(stream)
        if gather:
            import torch

            t = torch.tensor([ms], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        us_layer = ms * 1e3 / a.iters / a.layers
        out = {"leg": leg, "tokens": m, "world": a.world, "layers_resident": a.layers, "us_per_layer": round(us_layer, 1),
               "ms_per_step_80_layers_extrapolated": round(us_layer * spec.layers / 1e3, 2),
               "weight_bytes_per_layer_per_rank": shard_bytes}
        if m <= 16:
            gbs = shard_bytes / us_layer / 1e3
            out.update({"bound": "hbm", "achieved_gbs": round(gbs, 1), "peak_gbs": hbm, "frac": round(gbs / hbm, 3), "peak": src})
        else:
            tfs = 2.0 * m * shard_macs / us_layer / 1e6
            out.update({"bound": "tensor", "achieved_tflops": round(tfs, 1), "peak_tflops": tf, "frac": round(tfs / tf, 3), "peak": src})
        if gather:
            how = "gather by the library's own kernels over NVLink (no NCCL)" if comm.peer_stores else "NCCL all-gather + copy"
            out["execution"] = f"{nranks} ranks, {how} after every projection, max over ranks"
        if recorded:
            out["execution"] = out.get("execution", "one rank's shard") + "; the walk over the layers replayed from one CUDA graph"
        if rank == 0:
            results.append(out)
        ctx.free(dx)
        ctx.free(dy)
    for row in weights:
        for _, _, _, w in row:
            w.close()
    if comm is not None:
        comm.close()
    if own_ctx:
        ctx.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return results


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--layers", type=int, default=5, help="distinct layers resident (the step is extrapolated to 80)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--graph", action="store_true", help="record the decode walk once and replay it as a CUDA graph")
    a = ap.parse_args()
    for out in run(a.world, a.layers, a.iters, graph=a.graph):
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
