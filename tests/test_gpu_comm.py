"""The all-gather behind a row-sharded qlinear, through the C ABI (wf_comm_get_unique_id -> wf_comm_init ->
wf_allgather / wf_qlinear_allgather), against the CPU oracle: the NCCL route and, between two GPUs, the library's
own gather kernels (tagged peer stores, peer loads out of staging areas), which must give the same bits.

A communicator of world size 1 runs on the single GPU of the test box: it exercises the run-time loading of
libnccl, communicator set-up, the gather call on the compute stream and the rank-major -> token-major copy.
With two GPUs visible the same checks run with two ranks as child processes (NVLS off), where rank r's rows
must land at r * chunk on both ranks: the contract of CollectiveApi.allGather
(warpforge-io/src/main/java/io/surfworks/warpforge/io/collective/CollectiveApi.java:137-146; mock at
.../collective/mock/CollectiveMock.java:130-142)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import oracle as O
from warpforge_b200 import quant as Q

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _check(got, want):
    assert got.shape == want.shape
    assert np.max(np.abs(got - want)) <= 1e-3 * np.max(np.abs(want))


def test_world_one_communicator_allgather_and_qlinear(oracle):
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext, QuantizedWeight
    from warpforge_b200.decode import Communicator

    ctx = CudaContext(0)
    lib = ctx._lib
    try:
        comm = Communicator(ctx, Communicator.create_unique_id(), 0, 1)
        # plain all-gather of bytes: one rank's chunk is the whole result
        src = np.arange(4096, dtype=np.uint8)
        d_src, d_dst = ctx.allocate(src.nbytes), ctx.allocate(src.nbytes)
        ctx.copy_to_device(d_src, src)
        ctx.copy_to_device(d_dst, np.zeros_like(src))
        comm.all_gather(d_src, d_dst, src.nbytes)
        ctx.synchronize()
        back = np.empty_like(src)
        ctx.copy_to_host(back, d_dst)
        assert np.array_equal(back, src)
        # sharded qlinear + gather: 1 token (gathered in place), 5 and 24 tokens (decode kernels, rank-major ->
        # token-major copy), 48 tokens (tensor-core GEMM)
        rows, k = 1040, 1024
        for qt, oq in ((Q.QuantizationType.Q4_0, O.Q4_0), (Q.QuantizationType.Q4_K, O.Q4_K)):
            blocks = Q.synth_weight(qt, rows, k, 41)
            w = QuantizedWeight(ctx, qt, blocks, rows, k, 0, 1)
            for m in (1, 5, 24, 48):
                xb = Q.synth_activation_bf16(m, k, 41 + m)
                dx, dy = ctx.allocate(xb.nbytes), ctx.allocate(m * rows * 4)
                ctx.copy_to_device(dx, xb)
                ctx._ck("wf_qlinear_allgather", lib.wf_qlinear_allgather(ctx.handle, comm.handle, w.handle, dx, N.WF_DTYPE_BF16, m, dy, 0))
                ctx.synchronize()
                got = np.empty((m, rows), np.float32)
                ctx.copy_to_host(got, dy)
                _check(got, oracle.qlinear(oq, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=oracle.max_threads()))
                ctx.free(dx)
                ctx.free(dy)
            w.close()
        # a weight shard that does not belong to this communicator's rank is refused before any GPU work
        w2 = QuantizedWeight(ctx, Q.QuantizationType.Q4_0, Q.synth_q4_0(64, 256, 1), 64, 256, 1, 2)
        dx, dy = ctx.allocate(512), ctx.allocate(64 * 4)
        assert lib.wf_qlinear_allgather(ctx.handle, comm.handle, w2.handle, dx, N.WF_DTYPE_BF16, 1, dy, 0) == N.WF_ERR_SHARD
        w2.close()
        comm.close()
    finally:
        ctx.close()


_TWO_RANK = r"""
import os, sys
sys.path.insert(0, %r)
import numpy as np
import torch.distributed as dist
from oracle import oracle as O
from warpforge_b200 import _native as N, quant as Q
from warpforge_b200.backend import CudaContext, QuantizedWeight
from warpforge_b200.decode import Communicator
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
ctx = CudaContext(int(os.environ["LOCAL_RANK"]))
ids = [Communicator.create_unique_id() if rank == 0 else None]
dist.broadcast_object_list(ids, src=0)
comm = Communicator(ctx, ids[0], rank, world)
lib, orc = ctx._lib, O.COracle()
# rank r's chunk at r * chunk
chunk = 1000
src = np.full(chunk, rank + 1, np.uint8)
d_src, d_dst = ctx.allocate(chunk), ctx.allocate(chunk * world)
ctx.copy_to_device(d_src, src)
comm.all_gather(d_src, d_dst, chunk)
ctx.synchronize()
back = np.empty(chunk * world, np.uint8)
ctx.copy_to_host(back, d_dst)
assert all((back[r * chunk:(r + 1) * chunk] == r + 1).all() for r in range(world))
rows, k = 2048, 1024
for qt, oq in ((Q.QuantizationType.Q4_0, O.Q4_0), (Q.QuantizationType.Q4_K, O.Q4_K)):
    blocks = Q.synth_weight(qt, rows, k, 43)
    w = QuantizedWeight(ctx, qt, blocks, rows, k, rank, world)
    for m in (1, 5, 24, 48):
        xb = Q.synth_activation_bf16(m, k, 43 + m)
        dx, dy = ctx.allocate(xb.nbytes), ctx.allocate(m * rows * 4)
        ctx.copy_to_device(dx, xb)
        ctx._ck("wf_qlinear_allgather", lib.wf_qlinear_allgather(ctx.handle, comm.handle, w.handle, dx, N.WF_DTYPE_BF16, m, dy, 0))
        ctx.synchronize()
        got = np.empty((m, rows), np.float32)
        ctx.copy_to_host(got, dy)
        want = orc.qlinear(oq, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=4)
        assert np.max(np.abs(got - want)) <= 1e-3 * np.max(np.abs(want)), (qt.name, m)
    w.close()
dist.barrier()
comm.close(); ctx.close(); dist.destroy_process_group()
os.write(1, f"RANK_OK {rank}\n".encode())
"""


def test_two_rank_allgather_lands_rank_major(tmp_path):
    from warpforge_b200.backend import CudaContext

    if CudaContext.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "two_rank_comm.py"
    script.write_text(_TWO_RANK % ROOT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29534", str(script)], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RANK_OK 0" in r.stdout and "RANK_OK 1" in r.stdout


_PEER_STORES = r"""
import os, sys
sys.path.insert(0, %r)
import numpy as np
import torch.distributed as dist
from oracle import oracle as O
from warpforge_b200 import _native as N, quant as Q
from warpforge_b200.backend import CudaContext, QuantizedWeight
from warpforge_b200.decode import Communicator
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
ctx = CudaContext(int(os.environ["LOCAL_RANK"]))
ids = [Communicator.create_unique_id() if rank == 0 else None for _ in range(3)]
dist.broadcast_object_list(ids, src=0)
peer = Communicator(ctx, ids[0], rank, world)
os.environ["WF_GATHER"] = "nccl"
nccl = Communicator(ctx, ids[1], rank, world)
os.environ["WF_GATHER"] = "registers"   # large gathers by loads into registers instead of bulk copies through shared memory
regs = Communicator(ctx, ids[2], rank, world)
del os.environ["WF_GATHER"]
assert peer.peer_stores and regs.peer_stores and not nccl.peer_stores
lib, orc = ctx._lib, O.COracle()
rows, k = 2048 + 64 * world, 1024     # 1056 or so rows per rank: a ragged last row tile
rows -= rows %% world
def gathered(comm, w, dx, dtype, m, dy):
    ctx.copy_to_device(dy, np.full((m, rows), np.nan, np.float32))
    ctx._ck("wf_qlinear_allgather", lib.wf_qlinear_allgather(ctx.handle, comm.handle, w.handle, dx, dtype, m, dy, 0))
    ctx.synchronize()
    got = np.empty((m, rows), np.float32)
    ctx.copy_to_host(got, dy)
    return got
calls = 0
for qt, oq in ((Q.QuantizationType.Q4_0, O.Q4_0), (Q.QuantizationType.Q8_0, O.Q8_0), (Q.QuantizationType.Q4_K, O.Q4_K)):
    blocks = Q.synth_weight(qt, rows, k, 47)
    w = QuantizedWeight(ctx, qt, blocks, rows, k, rank, world)
    for m, f32 in ((1, False), (1, True), (2, False), (5, True), (16, False), (32, False), (48, False), (70, True), (200, False)):
        xb = Q.synth_activation_bf16(m, k, 47 + m)
        xf = Q.bf16_bits_to_float(xb)
        src = xf.astype(np.float32) if f32 else xb
        dx, dy = ctx.allocate(src.nbytes), ctx.allocate(m * rows * 4)
        ctx.copy_to_device(dx, src)
        dtype = N.WF_DTYPE_F32 if f32 else N.WF_DTYPE_BF16
        a = gathered(peer, w, dx, dtype, m, dy)
        b = gathered(nccl, w, dx, dtype, m, dy)
        a2 = gathered(peer, w, dx, dtype, m, dy)   # an odd number of peer gathers per case: both halves of the landing buffer take every shape
        calls += 2
        assert np.array_equal(a, b) and np.array_equal(a, a2), (qt.name, m, f32)
        if m > 32:
            assert np.array_equal(gathered(regs, w, dx, dtype, m, dy), b), (qt.name, m, f32, "registers")
        want = orc.qlinear(oq, blocks, rows, k, xf, nthreads=4)
        assert np.max(np.abs(a - want)) <= 1e-3 * np.max(np.abs(want)), (qt.name, m)
        ctx.free(dx); ctx.free(dy)
    # a recorded run of gathers replays: the gather counts live on the device.  3 tokens: tagged stores into the
    # peers' landing buffers; 40 tokens: the tensor-core kernel, blocks read out of the peers' staging areas
    for m in (3, 40):
        xb = Q.synth_activation_bf16(m, k, 5)
        dx, dy, dz = ctx.allocate(xb.nbytes), ctx.allocate(m * rows * 4), ctx.allocate(m * rows * 4)
        ctx.copy_to_device(dx, xb)
        want = gathered(nccl, w, dx, N.WF_DTYPE_BF16, m, dy)
        s = ctx.create_stream()
        ctx.graph_begin(s)
        for out in (dy, dz, dy):
            ctx._ck("wf_qlinear_allgather", lib.wf_qlinear_allgather(ctx.handle, peer.handle, w.handle, dx, N.WF_DTYPE_BF16, m, out, s))
        g = ctx.graph_end(s)
        for _ in range(3):
            ctx.copy_to_device(dy, np.zeros((m, rows), np.float32))
            ctx.copy_to_device(dz, np.zeros((m, rows), np.float32))
            ctx.graph_launch(g, s)
            ctx.synchronize(s)
            for buf in (dy, dz):
                got = np.empty((m, rows), np.float32)
                ctx.copy_to_host(got, buf)
                assert np.array_equal(got, want), qt.name
        ctx.graph_destroy(g)
        ctx.destroy_stream(s)
    w.close()
# strips of 17 KB per (rank, token): the bulk copies through shared memory, two pieces per strip, the second a short one
rows, k = 4352 * world, 512
qt = Q.QuantizationType.Q4_0
blocks = Q.synth_weight(qt, rows, k, 53)
w = QuantizedWeight(ctx, qt, blocks, rows, k, rank, world)
for m in (40, 130):
    xb = Q.synth_activation_bf16(m, k, 53 + m)
    dx, dy = ctx.allocate(xb.nbytes), ctx.allocate(m * rows * 4)
    ctx.copy_to_device(dx, xb)
    a = gathered(peer, w, dx, N.WF_DTYPE_BF16, m, dy)
    assert np.array_equal(a, gathered(nccl, w, dx, N.WF_DTYPE_BF16, m, dy)), ("bulk", m)
    assert np.array_equal(a, gathered(regs, w, dx, N.WF_DTYPE_BF16, m, dy)), ("registers", m)
    assert np.array_equal(a, gathered(peer, w, dx, N.WF_DTYPE_BF16, m, dy)), ("bulk again", m)
    want = orc.qlinear(O.Q4_0, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=4)
    assert np.max(np.abs(a - want)) <= 1e-3 * np.max(np.abs(want)), m
    ctx.free(dx); ctx.free(dy)
# Failure detection without a GPU fault: rank 1 never enters these gathers.  Rank 0's waits run out (0.3 s here), its
# kernels end by themselves, the next synchronisation reports WF_ERR_DEVICE_WAIT, its own columns are right and the
# context stays usable.  Rank 1 keeps its buffers mapped until rank 0 is through.
os.environ["WF_GATHER_WAIT_MS"] = "300"
ids = [Communicator.create_unique_id() if rank == 0 else None]
dist.broadcast_object_list(ids, src=0)
short = Communicator(ctx, ids[0], rank, world)
del os.environ["WF_GATHER_WAIT_MS"]
assert short.peer_stores
r = rows // world
if rank == 0:
    import time
    for m in (3, 40):
        xb = Q.synth_activation_bf16(m, k, 59 + m)
        dx, dy = ctx.allocate(xb.nbytes), ctx.allocate(m * rows * 4)
        ctx.copy_to_device(dx, xb)
        ctx.copy_to_device(dy, np.zeros((m, rows), np.float32))
        t0 = time.time()
        ctx._ck("wf_qlinear_allgather", lib.wf_qlinear_allgather(ctx.handle, short.handle, w.handle, dx, N.WF_DTYPE_BF16, m, dy, 0))
        try:
            ctx.synchronize()
            raise SystemExit("the gather of an absent peer did not report its wait")
        except N.WfError as err:
            assert err.status == N.WF_ERR_DEVICE_WAIT, err.status
        assert time.time() - t0 < 5.0
        got = np.empty((m, rows), np.float32)
        ctx.copy_to_host(got, dy)
        want = orc.qlinear(O.Q4_0, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=4)
        if m <= 32:  # the decode kernels write this rank's columns into y themselves
            assert np.max(np.abs(got[:, :r] - want[:, :r])) <= 1e-3 * np.max(np.abs(want)), m
        ctx.synchronize()  # the status was cleared by reporting it
        ctx.free(dx); ctx.free(dy)
dist.barrier()
w.close()
short.close()
dist.barrier()
peer.close(); nccl.close(); regs.close(); ctx.close(); dist.destroy_process_group()
os.write(1, f"RANK_OK {rank}\n".encode())
"""


def test_two_rank_peer_store_gather_equals_nccl_gather(tmp_path):
    """Small gathers go by 8-byte tagged stores into the peers' landing buffers; the result must be bit-identical to
    the NCCL all-gather + copy of a second communicator that was told to stay on NCCL, eagerly and from a replayed graph."""
    from warpforge_b200.backend import CudaContext

    if CudaContext.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "peer_store_gather.py"
    script.write_text(_PEER_STORES % ROOT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29535", str(script)], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RANK_OK 0" in r.stdout and "RANK_OK 1" in r.stdout
