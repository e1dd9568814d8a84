"""The oracle's fp32 glue operations against the cases of the reference's own test
(warpforge-backend-cpu/src/test/java/io/surfworks/warpforge/backend/cpu/ops/scalar/CustomCallKernelTest.java:
same inputs, same assertions, EPSILON 1e-5 there) and against an independent numpy restatement."""
import math

import numpy as np
import pytest

EPS = 1e-5


def test_layer_norm_zero_mean_unit_variance(oracle):
    y = oracle.layer_norm(np.arange(1, 9, dtype=np.float32).reshape(2, 4))
    assert y.shape == (2, 4)
    for row in y:
        assert abs(float(np.mean(row))) < EPS
        assert abs(float(np.mean((row - np.mean(row)) ** 2)) - 1.0) < 1e-4  # the reference allows 1e-4 here (eps in the denominator)


def test_layer_norm_weight_and_bias(oracle):
    y = oracle.layer_norm(np.array([[0, 1, 2, 3]], np.float32), np.full(4, 2, np.float32), np.ones(4, np.float32))
    assert abs(float(np.mean(y)) - 1.0) < EPS


def test_softmax_cases(oracle):
    y = oracle.softmax(np.array([[1, 2, 3, 4]], np.float32))
    assert abs(float(y.sum()) - 1.0) < EPS
    y = oracle.softmax(np.array([1, 2, 3, 4], np.float32))
    assert y[0] < y[1] < y[2] < y[3]
    y = oracle.softmax(np.array([1000, 1001, 1002, 1003], np.float32))
    assert np.all(np.isfinite(y)) and np.all((y >= 0) & (y <= 1)) and abs(float(y.sum()) - 1.0) < EPS


def test_silu_is_x_times_sigmoid(oracle):
    data = np.array([1.0, 2.0, -1.0, 0.0], np.float32)
    y = oracle.silu(data)
    for x, got in zip(data, y):
        assert abs(float(x) / (1 + np.float32(math.exp(-float(x)))) - got) < EPS
    assert y[3] == 0.0


def test_gelu_reference_cases(oracle):
    """CustomCallKernelTest.GeluTests: 0 at 0, close to x at 5, close to 0 at -5; and the tanh formula itself."""
    y = oracle.gelu(np.array([0.0, 5.0, -5.0, 1.0, -0.5], np.float32))
    assert abs(float(y[0])) < EPS and float(y[1]) > 4.9 and abs(float(y[2])) < 0.01
    for x, got in zip((1.0, -0.5), y[3:]):
        inner = np.float32(0.7978845608) * (np.float32(x) + np.float32(0.044715) * np.float32(x) * np.float32(x) * np.float32(x))
        assert abs(0.5 * x * (1.0 + math.tanh(float(inner))) - float(got)) < 1e-6


def test_rms_norm_normalizes_by_rms(oracle):
    y = oracle.rms_norm(np.array([[3, 4]], np.float32))
    assert abs(math.sqrt(float(np.sum(y * y)) / 2) - 1.0) < EPS
    y = oracle.rms_norm(np.array([[1, 1, 1, 1]], np.float32), np.array([2, 2, 2, 2], np.float32))
    assert np.allclose(y, 2.0, atol=1e-4)


def test_embedding_lookup(oracle):
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    y = oracle.embedding(np.array([[2, 0], [3, 3]], np.int64), table)
    assert y.shape == (2, 2, 3) and np.array_equal(y[0, 0], table[2]) and np.array_equal(y[1, 1], table[3])
    with pytest.raises(IndexError):
        oracle.embedding(np.array([4], np.int64), table)


def test_against_numpy_restatement(oracle):
    """Same formulas with numpy float32 scalars, sequential sums: bit-identical on small rows."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 37)).astype(np.float32) * 3
    g = rng.standard_normal(37).astype(np.float32)
    b = rng.standard_normal(37).astype(np.float32)
    f = np.float32
    want_rms, want_ln, want_sm = np.empty_like(x), np.empty_like(x), np.empty_like(x)
    for r in range(3):
        ss = f(0)
        for v in x[r]:
            ss = f(ss + f(v * v))
        inv = f(1) / f(np.sqrt(np.float64(f(f(ss / f(37)) + f(1e-5)))))
        want_rms[r] = (x[r] * inv).astype(f) * g
        s = f(0)
        for v in x[r]:
            s = f(s + v)
        mean = f(s / f(37))
        vs = f(0)
        for v in x[r]:
            d = f(v - mean)
            vs = f(vs + f(d * d))
        istd = f(1) / f(np.sqrt(np.float64(f(f(vs / f(37)) + f(1e-5)))))
        want_ln[r] = ((x[r] - mean).astype(f) * istd).astype(f) * g + b
        mx = x[r].max()
        e = np.exp((x[r] - mx).astype(np.float64)).astype(f)
        se = f(0)
        for v in e:
            se = f(se + v)
        want_sm[r] = e / se
    assert np.array_equal(oracle.rms_norm(x, g).view(np.uint32), want_rms.view(np.uint32))
    assert np.array_equal(oracle.layer_norm(x, g, b).view(np.uint32), want_ln.view(np.uint32))
    assert np.array_equal(oracle.softmax(x).view(np.uint32), want_sm.view(np.uint32))
    sig = f(1) / (f(1) + np.exp(-x.astype(np.float64)).astype(f))
    assert np.array_equal(oracle.silu(x).view(np.uint32), (x * sig).astype(f).view(np.uint32))
    assert np.array_equal(oracle.swiglu(x, x[::-1].copy()).view(np.uint32), ((x * sig).astype(f) * x[::-1]).astype(f).view(np.uint32))
    assert np.array_equal(oracle.add(x, x[::-1].copy()), x + x[::-1])
