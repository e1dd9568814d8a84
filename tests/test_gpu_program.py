"""The decode step as one persistent kernel (wf_program_*): its outputs must agree with those of
the same projections run one kernel at a time and with the CPU oracle.  The program and the
per-projection kernels cut a row's k-range into different pieces (the program cuts projections that
share their activations as one list of row-tiles; the per-projection kernels cut K into slices): the
same exact block sums, a different order of the final fp32 additions -- equal to 1e-5 of the output
scale, and the same bits from run to run.  A two-rank variant (row-sharded, gather fused into the epilogue over peer
memory) runs when two GPUs are visible."""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import oracle as O
from warpforge_b200 import quant as Q

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _same_as_per_op(got, ref, tokens, name):
    assert np.max(np.abs(got - ref)) <= 1e-5 * np.max(np.abs(ref)), name



@pytest.mark.parametrize("tokens", [1, 3])
def test_program_equals_per_op_kernels(oracle, tokens):
    from warpforge_b200.backend import CudaContext
    from warpforge_b200.decode import LLAMA_7B_Q4_0, ProjectionStack

    ctx = CudaContext(0)
    try:
        st = ProjectionStack(ctx, LLAMA_7B_Q4_0, tokens=tokens, layers=2)
        st._issue()
        ctx.synchronize()
        ref = {n: st.read_output(n) for n, _, _ in st.spec.projections}
        for n, ptr in st.y_dev.items():
            ctx.copy_to_device(ptr, np.zeros_like(ref[n]))
        st.build_program()
        st.run_program()
        ctx.synchronize()
        first = {n: st.read_output(n) for n, _, _ in st.spec.projections}
        st.run_program()  # twice: the second run starts from the state the first one left
        ctx.synchronize()  # also reports a bounded wait that ran out
        for name, rows, k in st.spec.projections:
            got = st.read_output(name)
            assert np.array_equal(got.view(np.uint32), first[name].view(np.uint32)), name + ": not the same bits from run to run"
            _same_as_per_op(got, ref[name], tokens, name)
            want = oracle.qlinear(O.Q4_0, st.blocks[name], rows, k, Q.bf16_bits_to_float(st.x_host[k]), nthreads=oracle.max_threads())
            assert np.max(np.abs(got - want)) <= 1e-3 * np.max(np.abs(want))
        st.close()
    finally:
        ctx.close()


@pytest.mark.parametrize("qname", ["Q4_0", "Q4_1", "Q8_0", "Q4_K", "Q5_0"])
@pytest.mark.parametrize("tokens", [1, 5])
def test_program_every_quantization_type(oracle, qname, tokens):
    """A small two-layer stack per type: the program's outputs equal the per-projection kernels' (bit for bit with
    several tokens) and the oracle within the matmul tolerance (1 token: the integer one-token kernel, 5: the
    eight-column one)."""
    from warpforge_b200.backend import CudaContext
    from warpforge_b200.decode import ProjectionStack, StackSpec

    qt = Q.QuantizationType[qname]
    oq = {"Q4_0": O.Q4_0, "Q4_1": O.Q4_1, "Q8_0": O.Q8_0, "Q4_K": O.Q4_K, "Q5_0": O.Q5_0}[qname]
    spec = StackSpec("small " + qname, qt, 2, (("wq", 512, 512), ("wk", 512, 512), ("wo", 512, 512), ("wgate", 1280, 512),
                                                ("wup", 1280, 512), ("wdown", 512, 1280)), 0)
    ctx = CudaContext(0)
    try:
        st = ProjectionStack(ctx, spec, tokens=tokens)
        st._issue()
        ctx.synchronize()
        ref = {n: st.read_output(n) for n, _, _ in st.spec.projections}
        for n, ptr in st.y_dev.items():
            ctx.copy_to_device(ptr, np.zeros_like(ref[n]))
        st.build_program()
        for _ in range(2):
            st.run_program()
        ctx.synchronize()
        for name, rows, k in st.spec.projections:
            got = st.read_output(name)
            _same_as_per_op(got, ref[name], tokens, name)
            want = oracle.qlinear(oq, st.blocks[name], rows, k, Q.bf16_bits_to_float(st.x_host[k]), nthreads=oracle.max_threads())
            assert np.max(np.abs(got - want)) <= 1e-3 * np.max(np.abs(want)), name
        st.close()
    finally:
        ctx.close()


def test_program_rejects_bad_arguments():
    import ctypes

    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext

    ctx = CudaContext(0)
    try:
        prog = ctypes.c_int64()
        one = (ctypes.c_int64 * 1)(1)
        flags = (ctypes.c_int * 1)(1)
        lib = ctx._lib
        assert lib.wf_program_create(ctx.handle, 1, one, one, one, flags, 1, 1, 0, None, ctypes.byref(prog)) == N.WF_ERR_INVALID_HANDLE
        assert lib.wf_program_create(ctx.handle, 1, one, one, one, flags, 9, 1, 0, None, ctypes.byref(prog)) == N.WF_ERR_SHAPE
        assert lib.wf_program_create(ctx.handle, 1, one, one, one, flags, 1, 2, 0, None, ctypes.byref(prog)) == N.WF_ERR_INVALID_ARGUMENT
        assert lib.wf_program_run(ctx.handle, 1234, 0) == N.WF_ERR_INVALID_HANDLE
    finally:
        ctx.close()


def test_peer_wait_runs_out_and_is_reported(oracle):
    """Failure detection without a GPU fault: rank 0 of a two-rank program runs alone, so the rows
    of the absent rank never land.  The kernel's bounded waits run out, the kernel ends by itself,
    the next synchronisation reports WF_ERR_DEVICE_WAIT, and the context stays usable."""
    import ctypes

    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext, QuantizedWeight

    ctx = CudaContext(0)
    lib = ctx._lib
    try:
        rows, k, world = 256, 256, 2
        qt = Q.QuantizationType.Q4_0
        blocks = Q.synth_q4_0(rows, k, 31)
        xb = Q.synth_activation_bf16(1, k, 31)
        dx = ctx.allocate(xb.nbytes)
        ctx.copy_to_device(dx, xb)
        ws = [QuantizedWeight(ctx, qt, blocks, rows, k, 0, world) for _ in range(2)]  # rank 0's shard, twice
        ys = [ctx.allocate(rows * 4) for _ in range(2)]
        landing = []
        for _ in range(2 * world):  # [op][rank]; the "peer" buffers are local memory nobody reads
            p = ctx.allocate(rows * 8)
            ctx.copy_to_device(p, np.zeros(rows * 8, np.uint8))
            landing.append(p)
        arr = lambda v, t: (t * len(v))(*v)
        prog = ctypes.c_int64()
        N.check("create", lib.wf_program_create(
            ctx.handle, 2, arr([w.handle for w in ws], ctypes.c_int64), arr([dx, dx], ctypes.c_int64), arr(ys, ctypes.c_int64),
            arr([N.WF_OP_NEW_X, N.WF_OP_NEW_X | N.WF_OP_DEPENDS], ctypes.c_int), 1, world, 0, arr(landing, ctypes.c_int64),
            ctypes.byref(prog)), ctx.handle)
        N.check("run", lib.wf_program_run(ctx.handle, prog.value, 0), ctx.handle)
        with pytest.raises(N.WfError) as err:
            ctx.synchronize()
        assert err.value.status == N.WF_ERR_DEVICE_WAIT
        # rank 0's own rows were still computed correctly
        got = np.empty((1, rows), np.float32)
        ctx.copy_to_host(got, ys[0])
        want = oracle.qlinear(O.Q4_0, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=2)
        half = rows // world
        assert np.max(np.abs(got[:, :half] - want[:, :half])) <= 1e-3 * np.max(np.abs(want))
        N.check("destroy", lib.wf_program_destroy(ctx.handle, prog.value), ctx.handle)
        # the context is still usable: an ordinary call gives the right answer and a clean status
        w = QuantizedWeight(ctx, qt, blocks, rows, k)
        dy = ctx.allocate(rows * 4)
        N.check("qlinear", lib.wf_qlinear(ctx.handle, w.handle, dx, N.WF_DTYPE_BF16, 1, 1, dy, 1, 0), ctx.handle)
        ctx.synchronize()
        ctx.copy_to_host(got, dy)
        assert np.max(np.abs(got - want)) <= 1e-3 * np.max(np.abs(want))
    finally:
        ctx.close()


def test_absent_rank_ends_a_long_program_within_one_timeout():
    """The failure is latched: after the first wait for the absent rank's rows has run out, the remaining
    projections of the program neither poll landing buffers nor spin at grid barriers, so an 8-projection
    program ends about as fast as a 2-projection one (not one timeout per projection)."""
    import ctypes
    import time

    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext, QuantizedWeight

    ctx = CudaContext(0)
    lib = ctx._lib
    try:
        rows, k, world, n_ops = 256, 256, 2, 8
        qt = Q.QuantizationType.Q4_0
        blocks = Q.synth_q4_0(rows, k, 33)
        xb = Q.synth_activation_bf16(1, k, 33)
        dx = ctx.allocate(xb.nbytes)
        ctx.copy_to_device(dx, xb)
        ws = [QuantizedWeight(ctx, qt, blocks, rows, k, 0, world) for _ in range(n_ops)]
        ys = [ctx.allocate(rows * 4) for _ in range(n_ops)]
        landing = []
        for _ in range(n_ops * world):
            p = ctx.allocate(rows * 8)
            ctx.copy_to_device(p, np.zeros(rows * 8, np.uint8))
            landing.append(p)
        arr = lambda v, t: (t * len(v))(*v)
        flags = [N.WF_OP_NEW_X] + [N.WF_OP_NEW_X | N.WF_OP_DEPENDS] * (n_ops - 1)

        def timed(n):
            prog = ctypes.c_int64()
            N.check("create", lib.wf_program_create(
                ctx.handle, n, arr([w.handle for w in ws[:n]], ctypes.c_int64), arr([dx] * n, ctypes.c_int64),
                arr(ys[:n], ctypes.c_int64), arr(flags[:n], ctypes.c_int), 1, world, 0, arr(landing[:n * world], ctypes.c_int64),
                ctypes.byref(prog)), ctx.handle)
            t = time.perf_counter()
            N.check("run", lib.wf_program_run(ctx.handle, prog.value, 0), ctx.handle)
            with pytest.raises(N.WfError) as err:
                ctx.synchronize()
            dt = time.perf_counter() - t
            assert err.value.status == N.WF_ERR_DEVICE_WAIT
            N.check("destroy", lib.wf_program_destroy(ctx.handle, prog.value), ctx.handle)
            return dt

        t2, t8 = timed(2), timed(n_ops)
        assert t8 <= 2.0 * t2 + 0.5, f"8 projections took {t8:.2f} s, 2 took {t2:.2f} s"
        assert t8 < 20.0
    finally:
        ctx.close()


_TWO_RANK = r"""
import os, sys
sys.path.insert(0, %r)
import numpy as np
import torch.distributed as dist
from oracle import oracle as O
from warpforge_b200 import quant as Q
from warpforge_b200.backend import CudaContext
from warpforge_b200.decode import ProjectionStack, LLAMA_7B_Q4_0
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
ctx = CudaContext(int(os.environ["LOCAL_RANK"]))
st = ProjectionStack(ctx, LLAMA_7B_Q4_0, tokens=1, layers=2, rank=rank, world=world)
handles = [None] * world
dist.all_gather_object(handles, st.export_buffers())
st.build_program(handles)
dist.barrier()
for _ in range(2):
    st.run_program()
ctx.synchronize()
orc = O.COracle()
for name, rows, k in st.spec.projections:
    got = st.read_output(name)
    want = orc.qlinear(O.Q4_0, st.blocks[name], rows, k, Q.bf16_bits_to_float(st.x_host[k]), nthreads=4)
    assert np.max(np.abs(got - want)) <= 1e-3 * np.max(np.abs(want)), name
dist.barrier()
st.close(); ctx.close(); dist.destroy_process_group()
os.write(1, f"RANK_OK {rank}\n".encode())  # one write per rank: the two ranks share the pipe
"""


def test_two_rank_program_gathers_through_peer_memory(tmp_path):
    from warpforge_b200.backend import CudaContext

    if CudaContext.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "two_rank.py"
    script.write_text(_TWO_RANK % ROOT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29533", str(script)], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RANK_OK 0" in r.stdout and "RANK_OK 1" in r.stdout


def test_weight_held_by_a_program_cannot_be_freed():
    """The program's op list points into the weights' device memory: wf_weight_free refuses while the program
    lives and works once it is destroyed."""
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext
    from warpforge_b200.decode import LLAMA_7B_Q4_0, ProjectionStack

    ctx = CudaContext(0)
    try:
        st = ProjectionStack(ctx, LLAMA_7B_Q4_0, tokens=1, layers=1)
        st.build_program()
        w = st.weights[0][0]
        assert ctx._lib.wf_weight_free(ctx.handle, w.handle) == N.WF_ERR_IN_USE
        st.run_program()  # still whole
        ctx.synchronize()
        st.close()  # destroys the program first, then frees every weight
    finally:
        ctx.close()


def test_step_from_host_buffers_in_one_call(oracle):
    """wf_program_step_host: activations from pinned host memory, the program, the last output back, one call."""
    from warpforge_b200.backend import CudaContext
    from warpforge_b200.decode import LLAMA_7B_Q4_0, ProjectionStack

    ctx = CudaContext(0)
    try:
        st = ProjectionStack(ctx, LLAMA_7B_Q4_0, tokens=1, layers=1)
        st.mode = "program"
        st.build_program()
        name, rows, k = st.spec.projections[-1]
        pinned_in = {kk: ctx.host_alloc(v.nbytes) for kk, v in st.x_host.items()}
        y_out = np.zeros((1, rows), np.float32)
        pinned_out = ctx.host_alloc(y_out.nbytes)
        # other activations than the ones uploaded at construction: the call must bring them over itself
        x_new = {kk: Q.synth_activation_bf16(1, kk, 900 + kk) for kk in st.x_host}
        st.step_host(x_new, y_out, pinned_in, pinned_out)
        want = oracle.qlinear(O.Q4_0, st.blocks[name], rows, k, Q.bf16_bits_to_float(x_new[k]), nthreads=oracle.max_threads())
        assert np.max(np.abs(y_out - want)) <= 1e-3 * np.max(np.abs(want))
        st.close()
    finally:
        ctx.close()


@pytest.mark.parametrize("seed", [1, 2])
def test_random_one_token_programs(oracle, seed):
    """Seeded random op lists: 1 - 9 projections of random row counts (one row to 6000) over up to three input widths,
    some sharing the staged activations with their predecessor (cut as one list of row-tiles), some staging anew after
    a barrier; every output against the oracle, after the program has run twice."""
    import ctypes

    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext, QuantizedWeight

    types = [(Q.QuantizationType.Q4_0, O.Q4_0), (Q.QuantizationType.Q8_0, O.Q8_0), (Q.QuantizationType.Q4_K, O.Q4_K), (Q.QuantizationType.Q4_1, O.Q4_1)]
    rng = np.random.default_rng(seed)
    ctx = CudaContext(0)
    lib = ctx._lib
    try:
        for it in range(12):
            qt, oq = types[rng.integers(len(types))]
            blk = 256 if qt == Q.QuantizationType.Q4_K else 32
            widths = [blk * int(rng.integers(1, 12288 // blk + 1)) for _ in range(3)]
            ops, xs, prev_k = [], {}, None
            for _ in range(int(rng.integers(1, 10))):
                k = widths[rng.integers(3)] if (prev_k is None or rng.random() < 0.4) else prev_k
                rows = int(rng.choice([1, 16, 33, 100, 512, 1000, 2368, 4096, 6000]))
                ops.append((rows, k, 3 if (prev_k is None or k != prev_k or rng.random() < 0.4) else 0))
                prev_k = k
                if k not in xs:
                    xb = Q.synth_activation_bf16(1, k, 77 + k)
                    d = ctx.allocate(xb.nbytes)
                    ctx.copy_to_device(d, xb)
                    xs[k] = (xb, d)
            blocks = [Q.synth_weight(qt, rows, k, 500 + it * 20 + i) for i, (rows, k, _) in enumerate(ops)]
            ws = [QuantizedWeight(ctx, qt, b, rows, k) for b, (rows, k, _) in zip(blocks, ops)]
            ys = [ctx.allocate(rows * 4) for rows, _, _ in ops]
            arr = lambda v, t: (t * len(v))(*v)
            prog = ctypes.c_int64()
            ctx._ck("wf_program_create", lib.wf_program_create(
                ctx.handle, len(ops), arr([w.handle for w in ws], ctypes.c_int64), arr([xs[k][1] for _, k, _ in ops], ctypes.c_int64),
                arr(ys, ctypes.c_int64), arr([f for _, _, f in ops], ctypes.c_int), 1, 1, 0, None, ctypes.byref(prog)))
            for _ in range(2):
                ctx._ck("wf_program_run", lib.wf_program_run(ctx.handle, prog.value, 0))
            ctx.synchronize()
            for i, (rows, k, _) in enumerate(ops):
                got = np.empty((1, rows), np.float32)
                ctx.copy_to_host(got, ys[i])
                want = oracle.qlinear(oq, blocks[i], rows, k, Q.bf16_bits_to_float(xs[k][0]), nthreads=oracle.max_threads())
                rel = float(np.max(np.abs(got - want)) / max(float(np.max(np.abs(want))), 1e-30))
                assert np.isfinite(got).all() and rel <= 1e-3, f"{qt.name} program {it} op {i} of {ops}: {rel:.3e}"
            ctx._ck("wf_program_destroy", lib.wf_program_destroy(ctx.handle, prog.value))
            for w in ws:
                w.close()
            for p in ys + [d for _, d in xs.values()]:
                ctx.free(p)
    finally:
        ctx.close()
