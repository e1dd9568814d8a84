"""GPU parity of the fp32 operations between the projections (rms_norm, layer_norm, softmax, silu,
swiglu, add, embedding) through the C ABI against the CPU oracle.

Bars.  Element operations (silu, swiglu, add, embedding) follow the CPU arithmetic operation by
operation.  With wf_set_exact_exp(1) they are bit-exact, except that the double exp of the device and
of the host libm may round a last bit differently, so silu / swiglu allow 1 ulp on at most one element
in 10^5.  In the default mode the exponential is the fp32 one (2 ulp): silu / swiglu must stay within
8 ulp of the oracle where |x| <= 20 (sigmoid not yet rounded into 0 or 1) and meet the reference's rule
for the target, |d| <= 1e-4 + 1e-3*|expected|, everywhere.  Row
reductions are summed in another order than the CPU's one-after-another fp32 sum; they must meet the
reference's own acceptance rule for these targets, |d| <= 1e-4 + 1e-3*|expected| on every element
(warpforge-core/.../testing/ToleranceConfig.java:47-51), and the tighter max|d| <= 1e-4 * max|expected|:
the oracle's one-accumulator fp32 sum over 16384 terms drops every term below half an ulp of the running sum,
which biases it by about 2e-5 relative; the device's sums do not lose them."""
import ctypes

import numpy as np
import pytest

from warpforge_b200 import _native as N

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    from warpforge_b200.backend import NvidiaBackend

    b = NvidiaBackend(0)
    yield b
    b.close()


def _call(backend, target, *arrays):
    from warpforge_b200.backend import AddOp, CustomCallOp, Tensor

    ts = [Tensor(np.ascontiguousarray(a), "i64" if a.dtype == np.int64 else "f32") for a in arrays]
    op = AddOp(arrays[0].shape) if target == "add" else CustomCallOp(target, arrays[0].shape)
    return backend.execute(op, ts)[0].data


def _ulps(a, b):
    ai, bi = a.view(np.int32).astype(np.int64), b.view(np.int32).astype(np.int64)
    ai = np.where(ai < 0, -(ai & 0x7FFFFFFF), ai)
    bi = np.where(bi < 0, -(bi & 0x7FFFFFFF), bi)
    return np.abs(ai - bi)


def _check_rows(oracle, got, want):
    assert got.shape == want.shape
    assert oracle.count_not_close(want, got, 1e-4, 1e-3) == 0
    scale = float(np.max(np.abs(want))) or 1.0
    assert float(np.max(np.abs(got.astype(np.float64) - want))) <= 1e-4 * scale


def _check_elements(got, want):
    u = _ulps(got, want)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    u = u[~nan]
    assert u.size == 0 or (u.max() <= 1 and np.count_nonzero(u) <= max(1, u.size // 100000)), f"max ulp {u.max()}, {np.count_nonzero(u)} differ"


def _check_elements_fp32_exp(oracle, got, want, x):
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    ok = ~nan & np.isfinite(want)
    assert oracle.count_not_close(want[ok], got[ok], 1e-4, 1e-3) == 0
    near = ok & (np.abs(x) <= 20)
    assert near.sum() == 0 or _ulps(got[near], want[near]).max() <= 8


SHAPES = [(1, 4096), (16, 4096), (3, 11008), (512, 4096), (5, 1000), (7, 7), (2, 8192), (2, 16384), (4, 8196), (1, 1), (33, 130)]


@pytest.mark.parametrize("rows,n", SHAPES)
def test_rms_norm(backend, oracle, rows, n):
    rng = np.random.default_rng(rows * 31 + n)
    x = (rng.standard_normal((rows, n)) * 2.5).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    _check_rows(oracle, _call(backend, "rms_norm", x, g), oracle.rms_norm(x, g))
    _check_rows(oracle, _call(backend, "rms_norm", x), oracle.rms_norm(x))


@pytest.mark.parametrize("rows,n", SHAPES)
def test_layer_norm(backend, oracle, rows, n):
    rng = np.random.default_rng(rows * 37 + n)
    x = (rng.standard_normal((rows, n)) * 2.5 + 1.5).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    b = (0.1 * rng.standard_normal(n)).astype(np.float32)
    _check_rows(oracle, _call(backend, "layer_norm", x, g, b), oracle.layer_norm(x, g, b))
    _check_rows(oracle, _call(backend, "layer_norm", x, g), oracle.layer_norm(x, g))
    _check_rows(oracle, _call(backend, "layer_norm", x), oracle.layer_norm(x))


@pytest.mark.parametrize("rows,n", SHAPES + [(32, 512)])
def test_softmax(backend, oracle, rows, n):
    rng = np.random.default_rng(rows * 41 + n)
    x = (rng.standard_normal((rows, n)) * 4).astype(np.float32)
    for exact in (False, True):
        backend.cuda_context.set_exact_exp(exact)
        try:
            got = _call(backend, "softmax", x)
        finally:
            backend.cuda_context.set_exact_exp(False)
        _check_rows(oracle, got, oracle.softmax(x))
        assert np.allclose(got.sum(axis=-1), 1.0, atol=1e-5)


def test_reference_test_cases(backend, oracle):
    """The inputs of CustomCallKernelTest.java, with its assertions, on the device."""
    y = _call(backend, "layer_norm", np.arange(1, 9, dtype=np.float32).reshape(2, 4))
    assert np.all(np.abs(y.mean(axis=1)) < 1e-5) and np.all(np.abs(y.var(axis=1) - 1) < 1e-4)
    y = _call(backend, "softmax", np.array([1000, 1001, 1002, 1003], np.float32))
    assert np.all(np.isfinite(y)) and abs(float(y.sum()) - 1) < 1e-5 and y[0] < y[1] < y[2] < y[3]
    y = _call(backend, "silu", np.array([1.0, 2.0, -1.0], np.float32))
    assert np.allclose(y, oracle.silu(np.array([1.0, 2.0, -1.0], np.float32)), atol=1e-5, rtol=0)  # the reference test's EPSILON
    y = _call(backend, "rms_norm", np.array([[3, 4]], np.float32))
    assert abs(np.sqrt(float(np.sum(y * y)) / 2) - 1) < 1e-5


@pytest.mark.parametrize("count", [1, 3, 4096, 1000003])
def test_gelu(backend, oracle, count):
    """gelu (tanh form): the float operations in the reference's order, tanh in double as the reference calls it; a
    different libm may round the last bit of tanh differently, so 1 ulp on at most one element in 10^5."""
    rng = np.random.default_rng(count)
    a = (rng.standard_normal(count) * 3).astype(np.float32)
    if count >= 16:
        a[:8] = [0.0, -0.0, np.inf, -np.inf, np.nan, 100.0, -100.0, 1e-30]
    got, want = _call(backend, "gelu", a), oracle.gelu(a)
    _check_elements(got, want)
    y = _call(backend, "gelu", np.array([0.0, 5.0, -5.0], np.float32))  # the reference test's cases
    assert abs(float(y[0])) < 1e-5 and float(y[1]) > 4.9 and abs(float(y[2])) < 0.01


@pytest.mark.parametrize("count", [1, 3, 4096, 11008, 1000003, 512 * 11008])
def test_silu_swiglu_add(backend, oracle, count):
    rng = np.random.default_rng(count)
    a = (rng.standard_normal(count) * 4).astype(np.float32)
    b = rng.standard_normal(count).astype(np.float32)
    if count >= 16:
        a[:8] = [0.0, -0.0, np.inf, -np.inf, np.nan, 100.0, -100.0, 1e-30]
    _check_elements_fp32_exp(oracle, _call(backend, "silu", a), oracle.silu(a), a)
    _check_elements_fp32_exp(oracle, _call(backend, "swiglu", a, b), oracle.swiglu(a, b), a)
    backend.cuda_context.set_exact_exp(True)
    try:
        _check_elements(_call(backend, "silu", a), oracle.silu(a))
        _check_elements(_call(backend, "swiglu", a, b), oracle.swiglu(a, b))
    finally:
        backend.cuda_context.set_exact_exp(False)
    got, want = _call(backend, "add", a, b), oracle.add(a, b)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])


def test_embedding(backend, oracle):
    rng = np.random.default_rng(2)
    for vocab, dim, shape in ((1000, 4096, (2, 5)), (50, 7, (9,)), (32000, 4096, (64,))):
        table = rng.standard_normal((vocab, dim)).astype(np.float32)
        idx = rng.integers(0, vocab, shape).astype(np.int64)
        got = _call(backend, "embedding", idx, table)
        assert got.shape == shape + (dim,) and np.array_equal(got, oracle.embedding(idx, table))


def test_embedding_index_outside_the_table(backend):
    """The CPU backend throws; the device writes a row of zeros and the next synchronisation says so."""
    ctx = backend.cuda_context
    lib = ctx._lib
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    idx = np.array([1, 4, -1, 3], np.int64)
    d_idx, d_tab, d_y = ctx.allocate(idx.nbytes), ctx.allocate(table.nbytes), ctx.allocate(4 * 3 * 4)
    ctx.copy_to_device(d_idx, idx)
    ctx.copy_to_device(d_tab, table)
    assert lib.wf_embedding(ctx.handle, d_idx, d_tab, d_y, 4, 4, 3, 0) == N.WF_OK
    assert lib.wf_stream_sync(ctx.handle, 0) == N.WF_ERR_INDEX
    y = np.empty((4, 3), np.float32)
    ctx.copy_to_host(y, d_y)
    assert np.array_equal(y[0], table[1]) and np.array_equal(y[3], table[3]) and not y[1].any() and not y[2].any()
    assert lib.wf_stream_sync(ctx.handle, 0) == N.WF_OK  # reported once
    for p in (d_idx, d_tab, d_y):
        ctx.free(p)


def test_device_tensors_in_place_and_odd_alignment(backend, oracle):
    """Device-resident inputs (no host copies in the call), y == x, and pointers that are only
    4-byte aligned (the 16-byte paths must not be taken)."""
    ctx = backend.cuda_context
    lib = ctx._lib
    rng = np.random.default_rng(9)
    rows, n = 6, 4096
    x = rng.standard_normal((rows, n)).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    buf = ctx.allocate((rows * n + n + 8) * 4)
    for off in (0, 4):  # byte offset of x inside the allocation
        d_x, d_g = buf + off, buf + off + rows * n * 4
        ctx.copy_to_device(d_x, x)
        ctx.copy_to_device(d_g, g)
        assert lib.wf_rms_norm(ctx.handle, d_x, d_g, d_x, rows, n, 1e-5, 0) == N.WF_OK
        y = np.empty_like(x)
        ctx.copy_to_host(y, d_x)
        _check_rows(oracle, y, oracle.rms_norm(x, g))
        ctx.copy_to_device(d_x, x)
        ctx.set_exact_exp(True)
        assert lib.wf_silu(ctx.handle, d_x, d_x, rows * n, 0) == N.WF_OK
        ctx.set_exact_exp(False)
        ctx.copy_to_host(y, d_x)
        _check_elements(y, oracle.silu(x))
    ctx.free(buf)


def test_error_paths(backend):
    from warpforge_b200.backend import CustomCallOp, Tensor, UnsupportedOperationError

    ctx = backend.cuda_context
    lib = ctx._lib
    with pytest.raises(UnsupportedOperationError, match="Unknown custom_call target for CUDA: gelu_new"):
        backend.execute(CustomCallOp("gelu_new", (4,)), [Tensor(np.zeros(4, np.float32))])
    d = ctx.allocate(64)
    assert lib.wf_rms_norm(ctx.handle, 0, 0, d, 1, 4, 1e-5, 0) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_rms_norm(ctx.handle, d + 2, 0, d, 1, 4, 1e-5, 0) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_softmax(ctx.handle, d, d, 1, 0, 0) == N.WF_ERR_SHAPE
    assert lib.wf_softmax(ctx.handle, d, d, 0, 4, 0) == N.WF_OK  # no rows: nothing to do
    assert lib.wf_swiglu(ctx.handle, d, 0, d, 4, 0) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_add(ctx.handle, d, d, d, -1, 0) == N.WF_ERR_SHAPE
    assert lib.wf_embedding(ctx.handle, d, d, d, 1, 0, 4, 0) == N.WF_ERR_SHAPE
    assert lib.wf_silu(12345, d, d, 4, 0) == N.WF_ERR_INVALID_HANDLE
    ctx.free(d)
