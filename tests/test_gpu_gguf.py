"""GGUF file -> device weight through wf_gguf_upload, against the CPU oracle: the uploaded shard
dequantizes bit-for-bit to what the oracle makes of the tensor's bytes in the file, and the
linear op on it meets the matmul tolerance of the other parity tests."""
import ctypes

import numpy as np
import pytest

from oracle import oracle as O
from tests import gguf_files as G
from tests.test_gpu_parity import QT, _check_matmul, _linear
from warpforge_b200 import _native as N
from warpforge_b200 import quant as Q
from warpforge_b200.gguf import GGUF

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    from warpforge_b200.backend import NvidiaBackend

    b = NvidiaBackend(0)
    yield b
    b.close()


@pytest.fixture(scope="module")
def model_file(tmp_path_factory):
    """A small model-shaped file: one linear weight per quantization type, {k, rows} in file order,
    between tensors of other types so that offsets and alignment padding matter."""
    specs = {"q4_0": (96, 512), "q8_0": (40, 256), "q4_k": (64, 1024), "q4_1": (48, 384), "q5_0": (32, 640)}
    blocks = {n: Q.synth_weight(QT[n][0], r, k, 300 + r) for n, (r, k) in specs.items()}
    tensors = [("token_embd.weight", (8, 3), 0, np.arange(24, dtype=np.float32).tobytes())]
    for n, (r, k) in specs.items():
        tensors.append((f"blk.0.{n}.weight", (k, r), QT[n][0].ggml_type, blocks[n].tobytes()))
        tensors.append((f"blk.0.{n}.norm", (5,), 0, np.ones(5, np.float32).tobytes()))
    tensors.append(("vec_q8", (64,), 8, bytes(68)))
    p = tmp_path_factory.mktemp("gguf") / "model.gguf"
    G.write_gguf(p, tensors, metadata=[("general.architecture", G.T_STR, "llama")])
    return p, specs, blocks


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k", "q4_1", "q5_0"])
def test_upload_from_file_is_bit_exact(backend, oracle, model_file, name):
    p, specs, blocks = model_file
    rows, k = specs[name]
    with GGUF.open(p) as g:
        assert np.array_equal(g.tensor(f"blk.0.{name}.weight"), blocks[name].ravel())
        w = g.upload(backend.cuda_context, f"blk.0.{name}.weight")
    # the file is closed: the weight lives on the device
    assert (w.rows, w.k, w.qtype) == (rows, k, QT[name][0])
    want = oracle.dequant(QT[name][1], blocks[name], rows * k).reshape(rows, k)
    assert np.array_equal(w.dequantize_to_array().view(np.uint32), want.view(np.uint32))
    w.close()


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k", "q4_1", "q5_0"])
def test_sharded_upload_and_linear(backend, oracle, model_file, name):
    from warpforge_b200.backend import Tensor

    p, specs, blocks = model_file
    rows, k = specs[name]
    x = Q.synth_activation_f32(2, k, 77)
    want_y = oracle.qlinear(QT[name][1], blocks[name], rows, k, x)
    want_w = oracle.dequant(QT[name][1], blocks[name], rows * k).reshape(rows, k)
    with GGUF.open(p) as g:
        for rank in range(2):
            w = g.upload(backend.cuda_context, f"blk.0.{name}.weight", rank, 2)
            lo, hi = rank * rows // 2, (rank + 1) * rows // 2
            assert (w.rows, w.row0) == (rows // 2, lo)
            assert np.array_equal(w.dequantize_to_array().view(np.uint32), want_w[lo:hi].view(np.uint32))
            _check_matmul(oracle, _linear(backend, w, Tensor.from_float_array(x)), want_y[:, lo:hi])
            w.close()


def test_q4_0_in_ggml_order(backend, oracle, model_file):
    """The same bytes read in ggml's nibble order: equal to the oracle on the re-ordered blocks,
    and, where the package is at hand, to the gguf package's own dequantization of the file."""
    p, specs, blocks = model_file
    rows, k = specs["q4_0"]
    with GGUF.open(p) as g:
        w = g.upload(backend.cuda_context, "blk.0.q4_0.weight", q4_0_order=N.WF_Q4_0_ORDER_GGML)
    got = w.dequantize_to_array()
    w.close()
    want = oracle.dequant(O.Q4_0, O.q4_0_ggml_to_reference_order(blocks["q4_0"]), rows * k).reshape(rows, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    gguf = pytest.importorskip("gguf")
    pkg = gguf.quants.dequantize(blocks["q4_0"].reshape(-1, 18), gguf.GGMLQuantizationType.Q4_0)
    assert np.array_equal(got.view(np.uint32), pkg.astype(np.float32).reshape(rows, k).view(np.uint32))


def test_file_written_by_the_gguf_package(backend, oracle, tmp_path):
    """Quantized by the gguf package, written by its writer, uploaded from the file in ggml order:
    the device holds what the package itself dequantizes."""
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(3)
    dense = (rng.standard_normal((48, 256)) * 0.05).astype(np.float32)
    p = tmp_path / "pkg.gguf"
    wr = gguf.GGUFWriter(str(p), "llama")
    q = {}
    types = (("q4", gguf.GGMLQuantizationType.Q4_0), ("q8", gguf.GGMLQuantizationType.Q8_0), ("q41", gguf.GGMLQuantizationType.Q4_1))
    for name, t in types:
        q[name] = gguf.quants.quantize(dense, t)
        wr.add_tensor(f"{name}.weight", q[name], raw_dtype=t)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    with GGUF.open(p) as g:
        for name, t in types:
            w = g.upload(backend.cuda_context, f"{name}.weight", q4_0_order=N.WF_Q4_0_ORDER_GGML)
            assert (w.rows, w.k) == (48, 256)
            want = gguf.quants.dequantize(q[name], t).astype(np.float32)
            assert np.array_equal(w.dequantize_to_array().view(np.uint32), want.view(np.uint32))
            w.close()


def test_q4_1_in_ggml_order(backend, oracle, model_file):
    p, specs, blocks = model_file
    rows, k = specs["q4_1"]
    with GGUF.open(p) as g:
        w = g.upload(backend.cuda_context, "blk.0.q4_1.weight", q4_0_order=N.WF_Q4_0_ORDER_GGML)
    got = w.dequantize_to_array()
    w.close()
    want = oracle.dequant(O.Q4_1, O.q4_0_ggml_to_reference_order(blocks["q4_1"], header=4), rows * k).reshape(rows, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_upload_errors(backend, model_file):
    p, _, _ = model_file
    lib, ctx = backend.cuda_context._lib, backend.cuda_context.handle
    h = ctypes.c_int64()
    with GGUF.open(p) as g:
        up = lambda name, rank=0, world=1, order=0: lib.wf_gguf_upload(ctx, g.handle, name, rank, world, order, ctypes.byref(h))
        assert up(b"missing") == N.WF_ERR_INVALID_ARGUMENT
        msg = ctypes.create_string_buffer(256)
        assert lib.wf_last_error(ctx, msg, len(msg)) == N.WF_OK and b"No tensor named: missing" in msg.value
        assert up(b"vec_q8") == N.WF_ERR_SHAPE                      # 1-D
        assert up(b"token_embd.weight") == N.WF_ERR_UNSUPPORTED_TYPE  # F32
        assert up(b"blk.0.q4_0.weight", 0, 1, 7) == N.WF_ERR_INVALID_ARGUMENT
        assert up(b"blk.0.q4_0.weight", 2, 2) == N.WF_ERR_SHARD
        assert up(b"blk.0.q8_0.weight", 0, 3) == N.WF_ERR_SHARD     # 40 rows over 3 ranks
        assert lib.wf_gguf_upload(ctx, 999, b"blk.0.q4_0.weight", 0, 1, 0, ctypes.byref(h)) == N.WF_ERR_INVALID_HANDLE
        assert h.value == 0


def test_tensor_larger_than_the_staging_chunks(backend, oracle, tmp_path):
    """22 MB of blocks: the upload streams them through its two 8 MB pinned chunks (three chunks,
    the last one partial); every byte must land where a single copy would put it."""
    rows, k = 4096 + 48, 5120
    blocks = Q.synth_weight(Q.QuantizationType.Q8_0, rows, k, 9)
    p = tmp_path / "big.gguf"
    G.write_gguf(p, [("pad", (3,), 0, bytes(12)), ("big.weight", (k, rows), 8, blocks.tobytes())])
    want = oracle.dequant(O.Q8_0, blocks, rows * k).reshape(rows, k)
    with GGUF.open(p) as g:
        w = backend.upload_gguf_weight(g, "big.weight")
        assert np.array_equal(w.dequantize_to_array().view(np.uint32), want.view(np.uint32))
        half = backend.upload_gguf_weight(g, "big.weight", 1, 2)
        assert np.array_equal(half.dequantize_to_array().view(np.uint32), want[rows // 2:].view(np.uint32))


def test_rows_longer_than_a_staging_chunk(backend, oracle):
    """k = 2^20: sixteen rows already exceed 8 MB, so the chunk grows to one row tile (16, 16, 8 rows)."""
    rows, k = 40, 1 << 20
    blocks = Q.synth_weight(Q.QuantizationType.Q4_0, rows, k, 13)
    w = backend.upload_weight(Q.QuantizationType.Q4_0, blocks, rows, k)
    want = oracle.dequant(O.Q4_0, blocks, rows * k).reshape(rows, k)
    assert np.array_equal(w.dequantize_to_array().view(np.uint32), want.view(np.uint32))
    w.close()
