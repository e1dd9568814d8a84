"""Times the gather behind a row-sharded projection, one projection shape at a time, on N ranks of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29537 \
        -m warpforge_b200.bench_gather [--tokens 2048]

For each distinct [rows x k] of the 70B-shape Q4_K projection set (benchmark config 5) every rank holds rows / N rows
of three distinct weights (so that consecutive calls read different weights) and runs, twelve times each,
(a) `wf_qlinear` on its shard alone and (b) `wf_qlinear_allgather` (the same projection followed by the gather that
leaves all rows on every rank).  The difference is what the gather costs: launches, the exchange of flags, the bytes
crossing NVLink and the write of the token-major output.  CUDA events on the launching stream of rank 0, the ranks
aligned by a barrier before each timed run.  `WF_GATHER=nccl` in the environment times the NCCL route, `registers`
the register variant of the large gather.  One JSON line per shape (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import _native as N
from . import quant as Q
from .backend import CudaContext, QuantizedWeight
from .decode import LLAMA_70B_Q4_K, Communicator


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    a = ap.parse_args()
    import torch.distributed as dist  # control plane only

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = CudaContext(int(os.environ.get("LOCAL_RANK", "0")))
    ids = [Communicator.create_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    comm = Communicator(ctx, ids[0], rank, world)
    lib, h = ctx._lib, ctx.handle
    qt, m = LLAMA_70B_Q4_K.qtype, a.tokens
    route = "NCCL all-gather + copy" if not comm.peer_stores else "the library's own kernels over NVLink"
    if os.environ.get("WF_GATHER"):
        route += f" (WF_GATHER={os.environ['WF_GATHER']})"
    e0, e1 = ctx.create_event(), ctx.create_event()
    seen = set()
    for name, rows, k in LLAMA_70B_Q4_K.projections:
        if (rows, k) in seen or rows % world:
            continue
        seen.add((rows, k))
        r = rows // world
        weights = []
        for c in range(3):
            full = np.empty((rows, qt.row_bytes(k)), np.uint8)  # only this rank's rows are read by the upload
            full[rank * r:(rank + 1) * r] = Q.synth_weight(qt, r, k, 100 + c)
            weights.append(QuantizedWeight(ctx, qt, full, rows, k, rank, world))
            del full
        x = Q.synth_activation_bf16(m, k, 5)
        dx, dy = ctx.allocate(x.nbytes), ctx.allocate(m * rows * 4)
        ctx.copy_to_device(dx, x)
        us = {}
        for what in ("alone", "gathered"):
            def call(w):
                if what == "alone":
                    N.check(name, lib.wf_qlinear(h, w.handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0), h)
                else:
                    N.check(name, lib.wf_qlinear_allgather(h, comm.handle, w.handle, dx, N.WF_DTYPE_BF16, m, dy, 0), h)

            dist.barrier()
            for w in weights:
                call(w)
            ctx.synchronize()
            dist.barrier()
            ctx.record_event(e0)
            for _ in range(4):
                for w in weights:
                    call(w)
            ctx.record_event(e1)
            ctx.synchronize()
            us[what] = ctx.elapsed_ms(e0, e1) * 1e3 / 12
        if rank == 0:
            out_mb = m * rows * 4 / 1e6
            cost = us["gathered"] - us["alone"]
            print(json.dumps({"tokens": m, "rows": rows, "k": k, "ranks": world, "route": route, "output_mb": round(out_mb, 1),
                              "projection_us": round(us["alone"], 1), "with_gather_us": round(us["gathered"], 1),
                              "gather_us": round(cost, 1),
                              "arriving_gb_per_s": round(out_mb * (world - 1) / world / cost * 1e3, 0) if cost > 0 else None}), flush=True)
        for w in weights:
            w.close()
        ctx.free(dx)
        ctx.free(dy)
    dist.barrier()
    comm.close()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
