"""The N > 1 host logic on CPU: two gloo ranks each hold a row shard of a quantized weight
(the same byte ranges wf_weight_upload keeps), compute their shard with the CPU oracle, and
all-gather in the rank-major layout of CollectiveApi.allGather
(warpforge-io/.../collective/CollectiveApi.java:137-146).  Checks the shard arithmetic, the
gather layout for one token (the gathered buffer IS the output row) and the [world][m][rows]
-> [m][N] rearrangement used for several tokens."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from oracle import oracle as O
    from warpforge_b200 import quant as Q

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = O.COracle()
        rows, k, m = 64, 256, 3
        qt = Q.QuantizationType.Q4_0
        blocks = Q.synth_q4_0(rows, k, 11)               # every rank sees the full tensor ...
        x = Q.bf16_bits_to_float(Q.synth_activation_bf16(m, k, 11))
        shard_rows, row_bytes = rows // world, qt.row_bytes(k)
        row0 = rank * shard_rows                          # ... and keeps rows [row0, row0 + shard_rows)
        mine = blocks.reshape(-1)[row0 * row_bytes:(row0 + shard_rows) * row_bytes]
        y_shard = orc.qlinear(O.Q4_0, mine, shard_rows, k, x)          # [m, shard_rows]
        full = orc.qlinear(O.Q4_0, blocks, rows, k, x)
        # one token: rank-major gather of [shard_rows] floats is the output row itself
        parts = [torch.empty(shard_rows) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(y_shard[0].copy()))
        ok1 = np.array_equal(torch.cat(parts).numpy(), full[0])
        # several tokens: gather [m, shard_rows] blocks, then [world][m][rows] -> [m][N]
        blocks_g = [torch.empty(m, shard_rows) for _ in range(world)]
        dist.all_gather(blocks_g, torch.from_numpy(y_shard.copy()))
        stacked = torch.stack(blocks_g).numpy()                          # [world, m, shard_rows]
        ok2 = np.array_equal(stacked.transpose(1, 0, 2).reshape(m, rows), full)
        q.put((rank, bool(ok1), bool(ok2)))
    finally:
        dist.destroy_process_group()


def test_row_shards_gather_to_the_full_output():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True, True), (1, True, True)]
