"""GPU parity of the tensor-core prefill GEMM (more than 8 bf16 tokens), through the C ABI,
against the CPU oracle.  The GEMM rounds each dequantized weight once to fp16 (relative 2^-12)
and accumulates exact products in fp32, so the bars are: max|d| / max|y| <= 1e-3 (the stated
tolerance) and rms(d) / rms(y) <= 3e-4; the elementwise 1e-3*|y| rule cannot hold for outputs
that cancel to nearly zero with any 16-bit weight operand and is reported, not asserted."""
import numpy as np
import pytest

from oracle import oracle as O
from warpforge_b200 import quant as Q

pytestmark = pytest.mark.gpu

QT = {"q4_0": (Q.QuantizationType.Q4_0, O.Q4_0), "q8_0": (Q.QuantizationType.Q8_0, O.Q8_0),
      "q4_k": (Q.QuantizationType.Q4_K, O.Q4_K), "q4_1": (Q.QuantizationType.Q4_1, O.Q4_1),
      "q5_0": (Q.QuantizationType.Q5_0, O.Q5_0)}


@pytest.fixture(scope="module")
def backend():
    from warpforge_b200.backend import NvidiaBackend

    b = NvidiaBackend(0)
    yield b
    b.close()


def _gemm(backend, w, xb):
    from warpforge_b200.backend import DotGeneralOp, LINEAR_DIMS, Tensor

    return backend.execute(DotGeneralOp(LINEAR_DIMS, (xb.shape[0], w.rows)), [Tensor.from_bf16_bits(xb), w])[0].data


def _check(got, want):
    d = got.astype(np.float64) - want.astype(np.float64)
    rel_max = float(np.max(np.abs(d)) / np.max(np.abs(want)))
    rel_rms = float(np.sqrt(np.mean(d * d)) / np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    assert rel_max <= 1e-3 and rel_rms <= 3e-4, f"max err / max|y| = {rel_max:.3e}, rms err / rms y = {rel_rms:.3e}"


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k", "q4_1", "q5_0"])
@pytest.mark.parametrize("rows,k,m", [(128, 256, 16), (256, 1024, 64), (1000, 2048, 300), (136, 512, 9), (4096, 4096, 33),
                                      (256, 1024, 513), (384, 1280, 700), (2048, 512, 1024),
                                      # enough tiles for the token tiles of 2 x 256: a last tile with one half, rows not a multiple of 128
                                      (4800, 256, 513), (4864, 512, 700)])
def test_gemm_matches_oracle(backend, oracle, name, rows, k, m):
    qt, oq = QT[name]
    blocks = Q.synth_weight(qt, rows, k, 77 + rows + m)
    xb = Q.synth_activation_bf16(m, k, 77 + rows + m)
    w = backend.upload_weight(qt, blocks, rows, k)
    got = _gemm(backend, w, xb)
    want = oracle.qlinear(oq, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=oracle.max_threads())
    _check(got, want)
    w.close()


def test_gemm_wide_dynamic_range_rows(backend, oracle):
    """Token rows far outside fp16's range (1e-30 and 1e30) survive the fp16 operand path."""
    rows, k, m = 256, 1024, 16
    blocks = Q.synth_q4_0(rows, k, 5)
    x = Q.synth_activation_f32(m, k, 5)
    x[3] *= 1e30
    x[7] *= 1e-30
    x[9] = 0.0
    xb = Q.float_to_bf16_bits(x).reshape(m, k)
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blocks, rows, k)
    got = _gemm(backend, w, xb)
    want = oracle.qlinear(O.Q4_0, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=4)
    for r in range(m):
        if r == 9:
            assert np.all(got[r] == 0.0)
        else:
            _check(got[r:r + 1], want[r:r + 1])
    w.close()


def test_config3_q4k_prefill_sampled_rows(backend, oracle):
    """benchmark config 3 at full size (M=512, N=14336, K=4096, Q4_K).  The oracle checks three weight rows out of
    every block of 128 (the GEMM's row tile: 112 blocks, 336 rows) for all 512 tokens; linearity over the tokens is
    checked for ALL 14336 outputs against the dequantized weight in float64; two calls give the same bits."""
    rows, k, m = 14336, 4096, 512
    blocks = Q.synth_q4_k(rows, k, Q.config_seed(3))
    xb = Q.synth_activation_bf16(m, k, Q.config_seed(3))
    w = backend.upload_weight(Q.QuantizationType.Q4_K, blocks, rows, k)
    got = _gemm(backend, w, xb)
    rng = np.random.default_rng(3)
    sample = np.sort(np.concatenate([b * 128 + rng.choice(128, 3, replace=False) for b in range(rows // 128)]))
    want = oracle.qlinear_rows(O.Q4_K, blocks, k, Q.bf16_bits_to_float(xb), sample, nthreads=oracle.max_threads())
    _check(got[:, sample], want)
    # linearity over tokens: the column sum of y equals y of the summed activations, every output column
    xs = Q.bf16_bits_to_float(xb).astype(np.float64).sum(axis=0, keepdims=True)
    wf = oracle.dequant(O.Q4_K, blocks, rows * k).reshape(rows, k)
    want_sum = np.concatenate([(xs @ wf[i:i + 1024].astype(np.float64).T)[0] for i in range(0, rows, 1024)])
    col_sum = got.astype(np.float64).sum(axis=0)
    assert np.max(np.abs(col_sum - want_sum)) <= 1e-3 * np.max(np.abs(want_sum))
    again = _gemm(backend, w, xb)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
    w.close()


def test_gemm_recorded_in_a_graph_replays_with_new_activations(oracle):
    """A many-token wf_qlinear recorded once into a CUDA graph and replayed with different activations: the pieces of
    tiles shared between CTAs are matched by a generation the kernel counts itself, so a replay can never take a
    previous replay's piece for its own."""
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext, QuantizedWeight

    ctx = CudaContext(0)
    lib = ctx._lib
    try:
        rows, k, m = 1000, 2048, 64  # 8 row tiles x 16 k-steps over 148 CTAs: every tile is shared by several CTAs
        blocks = Q.synth_q4_k(rows, k, 91)
        w = QuantizedWeight(ctx, Q.QuantizationType.Q4_K, blocks, rows, k)
        xs = [Q.synth_activation_bf16(m, k, 91 + i) for i in range(4)]
        dx, dy = ctx.allocate(xs[0].nbytes), ctx.allocate(m * rows * 4)
        ctx.copy_to_device(dx, xs[0])
        ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, w.handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0))  # eager: allocates scratch
        ctx.synchronize()
        ctx.graph_begin()
        ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, w.handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0))
        g = ctx.graph_end()
        got = np.empty((m, rows), np.float32)
        for x in xs[1:]:
            ctx.copy_to_device(dx, x)
            ctx.graph_launch(g)
            ctx.synchronize()
            ctx.copy_to_host(got, dy)
            _check(got, oracle.qlinear(O.Q4_K, blocks, rows, k, Q.bf16_bits_to_float(x), nthreads=oracle.max_threads()))
        ctx.graph_destroy(g)
        w.close()
    finally:
        ctx.close()


def test_recording_refuses_to_allocate():
    """A many-token wf_qlinear recorded without having run once would have to allocate its scratch inside the
    recording: it is refused with a status of its own, the recording stays usable, and after one eager call the
    same recording works."""
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext, QuantizedWeight

    ctx = CudaContext(0)
    lib = ctx._lib
    try:
        rows, k, m = 256, 1024, 64
        w = QuantizedWeight(ctx, Q.QuantizationType.Q4_0, Q.synth_q4_0(rows, k, 17), rows, k)
        xb = Q.synth_activation_bf16(m, k, 17)
        dx, dy = ctx.allocate(xb.nbytes), ctx.allocate(m * rows * 4)
        ctx.copy_to_device(dx, xb)
        ctx.graph_begin()
        assert lib.wf_qlinear(ctx.handle, w.handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0) == N.WF_ERR_RECORDING
        ctx.graph_destroy(ctx.graph_end())  # an empty graph: nothing was recorded, nothing was broken
        ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, w.handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0))
        ctx.synchronize()
        ctx.graph_begin()
        ctx._ck("wf_qlinear", lib.wf_qlinear(ctx.handle, w.handle, dx, N.WF_DTYPE_BF16, 1, m, dy, 1, 0))
        g = ctx.graph_end()
        ctx.graph_launch(g)
        ctx.synchronize()
        ctx.graph_destroy(g)
        w.close()
    finally:
        ctx.close()
