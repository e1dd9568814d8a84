"""The several-token decode kernel (2 .. 32 activation columns per launch) against the CPU oracle, through the
operator interface and the C ABI.  The shapes are chosen so that every way the kernel cuts a weight occurs:
one k-slice or many (K larger than what shared memory holds for the tokens at hand, a last slice shorter than
the others), teams of one to sixteen warps per unit (few rows: many warps per row-tile; many rows: several
row-tiles per warp), rows that do not fill the last row-tile, one, two and four groups of eight columns, and
fp32 activations (three bf16 columns per token, combined when the slices are added).  Tolerances: the
reference's dot_general rule and 1e-3 of the output's largest magnitude, as in test_gpu_parity.py."""
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


def _linear(backend, w, x_tensor):
    from warpforge_b200.backend import DotGeneralOp, LINEAR_DIMS

    return backend.execute(DotGeneralOp(LINEAR_DIMS, (x_tensor.shape()[0], w.rows)), [x_tensor, w])[0].data


def _check(oracle, got, want, exact64=None):
    """1e-3 of the output's largest magnitude; the reference's elementwise rule on all but 0.1 % of the elements
    (it fails where the CPU's own sequential fp32 rounding is of the size of the rule); with the exact float64
    product at hand the rule is replaced by: the GPU's error against it is at most twice the CPU's."""
    d = np.abs(got.astype(np.float64) - want.astype(np.float64))
    rel_max = float(np.max(d) / np.max(np.abs(want)))
    assert rel_max <= 1e-3, f"max err / max|y| = {rel_max:.3e}"
    if exact64 is None:
        bad = oracle.count_not_close(want, got, 1e-4, 1e-3)
        assert bad <= max(1, want.size // 1000), f"rule failures {bad}/{want.size}, max err / max|y| = {rel_max:.3e}"
    else:
        e_gpu, e_cpu = float(np.max(np.abs(got - exact64))), float(np.max(np.abs(want - exact64)))
        rms = float(np.sqrt(np.mean(exact64 ** 2)))
        assert e_gpu <= 2.0 * e_cpu + 1e-6 * rms, f"gpu err {e_gpu:.3e} vs cpu err {e_cpu:.3e} against float64"


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k", "q4_1", "q5_0"])
@pytest.mark.parametrize("rows,k,m", [
    (64, 1024, 9),      # four row-tiles: sixteen warps per unit, one group of columns and a bit
    (37, 512, 16),      # rows end inside a row-tile
    (1000, 2048, 17),   # three groups' worth of columns run as four
    (6000, 512, 24),    # many row-tiles, few k-tiles: several units per team
    (256, 11008, 32),   # K over several slices, the last one shorter (Q4_K pads K to a multiple of 256)
    (4096, 4096, 12),
])
def test_bf16_tokens_match_oracle(backend, oracle, name, rows, k, m):
    from warpforge_b200.backend import Tensor

    qt, oq = QT[name]
    if name == "q4_k" and k % 256:
        k = (k // 256) * 256
    seed = 300 + rows + k + m
    blocks = Q.synth_weight(qt, rows, k, seed)
    xb = Q.synth_activation_bf16(m, k, seed)
    w = backend.upload_weight(qt, blocks, rows, k)
    got = _linear(backend, w, Tensor.from_bf16_bits(xb))
    want = oracle.qlinear(oq, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=oracle.max_threads())
    _check(oracle, got, want)
    again = _linear(backend, w, Tensor.from_bf16_bits(xb))
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32)), "not the same bits from call to call"
    w.close()


@pytest.mark.parametrize("rows,k", [(1024, 8192), (128, 8192), (3584, 8192), (1024, 28672)])
def test_config5_shard_shapes_batch16(backend, oracle, rows, k):
    """One rank's rows of benchmark config 5's projections (70B shape, eight row shards), Q4_K, sixteen tokens."""
    from warpforge_b200.backend import Tensor

    blocks = Q.synth_q4_k(rows, k, Q.config_seed(5, rows + k))
    xb = Q.synth_activation_bf16(16, k, Q.config_seed(5, 16))
    w = backend.upload_weight(Q.QuantizationType.Q4_K, blocks, rows, k)
    got = _linear(backend, w, Tensor.from_bf16_bits(xb))
    want = oracle.qlinear(O.Q4_K, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=oracle.max_threads())
    # K up to 28672: the CPU's sequential fp32 sum is itself off by more than the elementwise rule on small outputs
    wf = oracle.dequant(O.Q4_K, blocks, rows * k).reshape(rows, k).astype(np.float64)
    _check(oracle, got, want, exact64=Q.bf16_bits_to_float(xb).astype(np.float64) @ wf.T)
    w.close()


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k"])
@pytest.mark.parametrize("m", [2, 7, 10, 11])
def test_fp32_tokens_match_oracle(backend, oracle, name, m):
    """fp32 activations: ten tokens (thirty columns) fit one launch, eleven take two."""
    from warpforge_b200.backend import Tensor

    qt, oq = QT[name]
    rows, k = 520, 4096
    blocks = Q.synth_weight(qt, rows, k, 400 + m)
    x = Q.synth_activation_f32(m, k, 400 + m)
    w = backend.upload_weight(qt, blocks, rows, k)
    got = _linear(backend, w, Tensor.from_float_array(x))
    want = oracle.qlinear(oq, blocks, rows, k, x, nthreads=oracle.max_threads())
    _check(oracle, got, want)
    w.close()


def test_integer_activations_are_exact(backend):
    """Small-integer activations and unit scales: every product and every partial sum is an integer below 2^24, so
    the result must equal the integer matrix product exactly, however K was cut into slices."""
    from warpforge_b200.backend import Tensor

    rows, k, m = 300, 11008, 16
    rng = np.random.default_rng(9)
    codes = rng.integers(0, 16, (rows, k), dtype=np.int64)
    blocks = np.zeros((rows, k // 32, 18), np.uint8)
    blocks[:, :, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    c = codes.reshape(rows, k // 32, 32)
    blocks[:, :, 2:] = (c[:, :, 0::2] | (c[:, :, 1::2] << 4)).astype(np.uint8)  # the reference's interleaved order
    x = rng.integers(-8, 9, (m, k)).astype(np.float32)
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blocks.reshape(rows, -1), rows, k)
    got = _linear(backend, w, Tensor.from_bf16_bits(Q.float_to_bf16_bits(x).reshape(m, k)))
    want = (x.astype(np.int64) @ (codes - 8).T).astype(np.float32)
    assert np.array_equal(got, want)
    w.close()


def test_recorded_in_a_graph_replays_with_new_activations(oracle):
    """A sixteen-token wf_qlinear whose K is cut into slices, recorded once and replayed with different activations:
    the arrival counters are put back to zero by the warp that completes a row-tile, so every replay starts clean."""
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext, QuantizedWeight

    ctx = CudaContext(0)
    lib = ctx._lib
    try:
        rows, k, m = 1024, 8192, 16
        blocks = Q.synth_q4_k(rows, k, 93)
        w = QuantizedWeight(ctx, Q.QuantizationType.Q4_K, blocks, rows, k)
        xs = [Q.synth_activation_bf16(m, k, 93 + i) for i in range(4)]
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
            _check(oracle, got, oracle.qlinear(O.Q4_K, blocks, rows, k, Q.bf16_bits_to_float(x), nthreads=oracle.max_threads()))
        ctx.graph_destroy(g)
        w.close()
    finally:
        ctx.close()
