"""wf_qlinear_noalloc -- the entry point for hosts that may not allocate device memory once
they are running (all memory already handed to their own arena, or a no-allocation rule in a
serving loop, where cudaMalloc could fail or stall the device).  Called through the C ABI on
device buffers and compared with the ordinary wf_qlinear (same bits: the same kernels with the
same work split) and with the CPU oracle, twice in a row with different shapes, because both calls share one statically sized work array that keeps the previous
call's contents.  Collected last so that a run stopping at the first failure has already
run everything else; it needs nothing from the other tests."""
import ctypes

import numpy as np
import pytest

from warpforge_b200 import quant as Q

pytestmark = pytest.mark.gpu

MAXREL = 1e-3  # same bound as tests/test_gpu_parity.py


def _oracle_result(qt, rows, k, m, seed):
    from oracle import oracle as O

    orc = O.COracle()
    oq = {"Q4_0": O.Q4_0, "Q4_K": O.Q4_K}[qt.name]
    blocks = Q.synth_weight(qt, rows, k, seed)
    xb = Q.synth_activation_bf16(m, k, seed)
    return orc.qlinear(oq, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=orc.max_threads())


def _run_both(ctx, lib, N, qt, rows, k, m, seed):
    from warpforge_b200.backend import QuantizedWeight

    blocks = Q.synth_weight(qt, rows, k, seed)
    xb = Q.synth_activation_bf16(m, k, seed)
    w = QuantizedWeight(ctx, qt, blocks, rows, k)
    dx = ctx.allocate(xb.nbytes)
    ctx.copy_to_device(dx, xb)
    dy_ref, dy_new = ctx.allocate(m * rows * 4), ctx.allocate(m * rows * 4)
    ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, w.handle, dx, N.WF_DTYPE_BF16, 1, m, dy_ref, 1, 0))
    ctx._ck("wf_qlinear_noalloc", lib.wf_qlinear_noalloc(ctx.handle, w.handle, dx, N.WF_DTYPE_BF16, m, dy_new, 0))
    ctx.synchronize()
    ref, new = np.empty((m, rows), np.float32), np.empty((m, rows), np.float32)
    ctx.copy_to_host(ref, dy_ref)
    ctx.copy_to_host(new, dy_new)
    w.close()
    for p in (dx, dy_ref, dy_new):
        ctx.free(p)
    return ref, new


def test_noalloc_matches_qlinear_twice_in_a_row():
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext

    ctx = CudaContext(0)
    lib = ctx._lib
    try:
        # first call: many CTAs exchange partial rows; second call: a different type and a
        # smaller shape, so stale slots from the first call would show up if they were not cleared
        for qt, rows, k, m, seed in ((Q.QuantizationType.Q4_0, 4096, 11008, 3, 31), (Q.QuantizationType.Q4_K, 1000, 2048, 1, 32)):
            ref, new = _run_both(ctx, lib, N, qt, rows, k, m, seed)
            assert np.isfinite(ref).all() and np.abs(ref).max() > 0
            # the same kernels with the same work split: the same bits
            assert np.array_equal(new.view(np.uint32), ref.view(np.uint32)), f"{qt.name} [{rows}x{k}] m={m}: differs from wf_qlinear"
            want = _oracle_result(qt, rows, k, m, seed)
            rel = float(np.max(np.abs(new - want)) / np.max(np.abs(want)))
            assert rel <= MAXREL, f"{qt.name} [{rows}x{k}] m={m}: max err / max|y| against the CPU = {rel:.3e}"
        # argument checks happen before any GPU work
        assert lib.wf_qlinear_noalloc(ctx.handle, 12345, 1, N.WF_DTYPE_BF16, 1, 1, 0) == N.WF_ERR_INVALID_HANDLE
    finally:
        ctx.close()
