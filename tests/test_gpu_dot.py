"""stablehlo.dot on the GPU (dense fp32 operands): the reference's known-answer tests for `dot`, CPU and GPU
(tests/golden/reference_kats.json: ScalarKernelTest.java:594-666, MatrixReduceKernelTest.java:151-212), replayed
through the operator interface, and random shapes against the CPU oracle bit for bit -- every output is summed over
k ascending with a separate multiply and add on both sides."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

KATS = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))


@pytest.fixture(scope="module")
def backend():
    from warpforge_b200.backend import NvidiaBackend

    b = NvidiaBackend(0)
    yield b
    b.close()


def _dot(backend, a, b):
    from warpforge_b200.backend import DotOp, Tensor

    return backend.execute(DotOp(()), [Tensor(np.ascontiguousarray(a, np.float32), "f32"), Tensor(np.ascontiguousarray(b, np.float32), "f32")])[0].data


def test_reference_dot_cases(backend):
    for k in KATS["dot"]:
        a = np.array(k["a"], np.float32).reshape(k["a_shape"])
        b = np.array(k["b"], np.float32).reshape(k["b_shape"])
        assert np.allclose(_dot(backend, a, b).ravel(), k["expected"], atol=k["tol"], rtol=0), k["source"]


@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (3, 5, 7), (64, 16, 64), (65, 17, 63), (200, 333, 129), (1, 4096, 300), (512, 1000, 1)])
def test_random_shapes_equal_the_cpu_bit_for_bit(backend, oracle, m, k, n):
    rng = np.random.default_rng(m * 1000 + k + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    got, want = _dot(backend, a, b), oracle.dot(a, b)
    assert got.shape == (m, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_vector_forms_and_errors(backend, oracle):
    from warpforge_b200.backend import DotOp, Tensor, UnsupportedOperationError

    rng = np.random.default_rng(3)
    v, w = rng.standard_normal(100).astype(np.float32), rng.standard_normal(100).astype(np.float32)
    mat = rng.standard_normal((100, 40)).astype(np.float32)
    assert np.array_equal(_dot(backend, v, w), oracle.dot(v.reshape(1, -1), w.reshape(-1, 1)).reshape(1))  # [K] x [K] -> [1]
    assert np.array_equal(_dot(backend, mat.T.copy(), v), oracle.dot(mat.T.copy(), v.reshape(-1, 1)).reshape(40))  # [M,K] x [K]
    assert np.array_equal(_dot(backend, v, mat), oracle.dot(v.reshape(1, -1), mat).reshape(40))  # [K] x [K,N]
    with pytest.raises(ValueError, match="Inner dimensions must match"):
        _dot(backend, np.zeros((2, 3), np.float32), np.zeros((4, 2), np.float32))
    with pytest.raises(UnsupportedOperationError):
        backend.execute(DotOp(()), [Tensor(np.zeros((2, 2, 2), np.float32), "f32"), Tensor(np.zeros((2, 2), np.float32), "f32")])
    with pytest.raises(ValueError, match="exactly 2 inputs"):
        backend.execute(DotOp(()), [Tensor(np.zeros((2, 2), np.float32), "f32")])
