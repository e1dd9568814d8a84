"""The native GGUF reader (wf_gguf_*) without a GPU: the cases of the reference's own reader test
(warpforge-data/src/test/java/io/surfworks/warpforge/data/format/GGUFTest.java: simple F32 tensor,
metadata, F16, several tensors, invalid magic, file too small, unknown tensor, Q4_0 size), the format
variants the reader accepts (versions 1-3, general.alignment, arrays), corrupt files, and a file
written by the third-party gguf package read back identically."""
import ctypes
import struct

import numpy as np
import pytest

from tests import gguf_files as G
from warpforge_b200 import _native as N
from warpforge_b200.gguf import GGUF, GGUFFormatError


def f32(*v):
    return np.array(v, np.float32).tobytes()


def test_simple_f32_tensor(tmp_path):
    p = tmp_path / "simple.gguf"
    data_offset, _ = G.write_gguf(p, [("test_tensor", (2, 3), 0, f32(1, 2, 3, 4, 5, 6))])
    with GGUF.open(p) as g:
        assert g.version() == 3 and g.tensor_count() == 1
        assert g.tensor_names() == ["test_tensor"] and g.has_tensor("test_tensor") and not g.has_tensor("nope")
        info = g.tensor_info("test_tensor")
        assert info.shape == (2, 3) and info.ggml_type == 0 and info.size == 24 and info.offset == 0
        assert g.data_offset == data_offset and g.alignment == 32 and data_offset % 32 == 0
        assert np.array_equal(g.tensor("test_tensor").view(np.float32), np.arange(1, 7, dtype=np.float32))


def test_metadata(tmp_path):
    p = tmp_path / "meta.gguf"
    G.write_gguf(p, [("t", (1,), 0, f32(1))], metadata=[
        ("general.architecture", G.T_STR, "llama"), ("general.name", G.T_STR, "Test Model"),
        ("llama.block_count", G.T_U32, 32), ("x.i8", G.T_I8, -5), ("x.u64", G.T_U64, 1 << 40), ("x.flag", G.T_BOOL, 1),
        ("x.f32", G.T_F32, 0.5), ("x.f64", G.T_F64, 0.25), ("x.i16", G.T_I16, -300), ("x.u16", G.T_U16, 65535),
        ("tokens", G.T_ARR, (G.T_STR, ["a", "bc", "def"])), ("ids", G.T_ARR, (G.T_I32, list(range(20))))])
    with GGUF.open(p) as g:
        m = g.metadata()
        assert m["general.architecture"] == "llama" and m["general.name"] == "Test Model"
        assert m["llama.block_count"] == "32" and m["x.i8"] == "-5" and m["x.u64"] == str(1 << 40)
        assert m["x.flag"] == "true" and float(m["x.f32"]) == 0.5 and float(m["x.f64"]) == 0.25
        assert m["x.i16"] == "-300" and m["x.u16"] == "65535"
        assert m["tokens"] == "[a, bc, def]" and m["ids"].startswith("[0, 1, 2") and m["ids"].endswith("...]")
        assert np.array_equal(g.tensor("t").view(np.float32), [1.0])


def test_f16_and_multiple_tensors(tmp_path):
    p = tmp_path / "multi.gguf"
    h = np.array([1.0, -2.0, 0.5, 4.0], np.float16).tobytes()
    _, offs = G.write_gguf(p, [("a", (4,), 1, h), ("b", (2, 2), 0, f32(1, 2, 3, 4)), ("c", (3,), 30, struct.pack("<3i", 7, 8, 9))])
    with GGUF.open(p) as g:
        assert g.tensor_names() == ["a", "b", "c"]
        assert g.tensor_info("a").size == 8 and g.tensor_info("b").size == 16 and g.tensor_info("c").size == 12
        assert [g.tensor_info(n).offset for n in "abc"] == [offs[n] for n in "abc"] == [0, 32, 64]
        assert np.array_equal(g.tensor("a").view(np.float16), np.array([1.0, -2.0, 0.5, 4.0], np.float16))
        assert np.array_equal(g.tensor("b").view(np.float32), [1, 2, 3, 4])
        assert np.array_equal(g.tensor("c").view(np.int32), [7, 8, 9])


def test_invalid_magic(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(struct.pack("<IIqq", 0x12345678, 3, 0, 0))
    with pytest.raises(GGUFFormatError, match="Invalid GGUF magic: expected 0x46554747, got 0x12345678"):
        GGUF.open(p)


def test_file_too_small(tmp_path):
    p = tmp_path / "small.gguf"
    p.write_bytes(b"\0" * 10)
    with pytest.raises(GGUFFormatError, match="File too small to be a GGUF file: 10 bytes"):
        GGUF.open(p)
    with pytest.raises(GGUFFormatError, match="cannot open"):
        GGUF.open(tmp_path / "missing.gguf")


def test_tensor_not_found(tmp_path):
    p = tmp_path / "one.gguf"
    G.write_gguf(p, [("exists", (1,), 0, f32(1))])
    with GGUF.open(p) as g:
        with pytest.raises(ValueError, match="No tensor named: nonexistent"):
            g.tensor_info("nonexistent")
        with pytest.raises(ValueError, match="No tensor named: nonexistent"):
            g.tensor("nonexistent")


@pytest.mark.parametrize("ggml_type,elements,size", [(2, 32, 18), (2, 33, 36), (3, 64, 40), (6, 32, 22), (7, 32, 24),
                                                     (8, 32, 34), (8, 4096, 4352), (14, 256, 144), (14, 257, 288),
                                                     (16, 256, 176), (9, 40, 40), (18, 5, 10), (28, 7, 7), (29, 7, 14),
                                                     (31, 2, 16), (32, 2, 16), (26, 9, 9), (27, 9, 9)])
def test_tensor_sizes(tmp_path, ggml_type, elements, size):
    """GGUF.java:294-351 (the Q4_0 case is GGUFTest's quantized-size test)."""
    p = tmp_path / "q.gguf"
    G.write_gguf(p, [("w", (elements,), ggml_type, bytes(size))])
    with GGUF.open(p) as g:
        assert g.tensor_info("w").size == size and g.tensor("w").size == size


@pytest.mark.parametrize("version", [1, 2, 3])
def test_versions_and_alignment(tmp_path, version):
    p = tmp_path / f"v{version}.gguf"
    data_offset, offs = G.write_gguf(p, [("first", (3,), 0, f32(1, 2, 3)), ("second", (2,), 0, f32(9, 8))],
                                     metadata=[("general.name", G.T_STR, "v"), ("arr", G.T_ARR, (G.T_U8, [1, 2, 3]))],
                                     version=version, alignment=64)
    with GGUF.open(p) as g:
        assert g.version() == version and g.alignment == 64 and g.data_offset == data_offset and data_offset % 64 == 0
        assert g.tensor_info("second").offset == offs["second"] == 64
        assert np.array_equal(g.tensor("second").view(np.float32), [9, 8])
        assert g.metadata()["arr"] == "[1, 2, 3]"


@pytest.mark.parametrize("blob,msg", [
    (struct.pack("<IIqq", G.MAGIC, 4, 0, 0), "Unsupported GGUF version: 4"),
    (struct.pack("<IIqq", G.MAGIC, 0, 0, 0), "Unsupported GGUF version: 0"),
    (struct.pack("<IIqq", G.MAGIC, 3, 5, 0), "truncated|corrupt"),
    (struct.pack("<IIqq", G.MAGIC, 3, 0, 1 << 60), "corrupt"),
    (struct.pack("<IIqq", G.MAGIC, 3, 0, 1) + struct.pack("<Q", 1 << 50) + b"k" * 8, "truncated"),
    (struct.pack("<IIqq", G.MAGIC, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 13) + b"\0" * 8, "Unknown GGUF value type: 13"),
    (struct.pack("<IIqq", G.MAGIC, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<IIQ", 9, 9, 1) + b"\0" * 16, "Unknown GGUF value type: 9"),
])
def test_corrupt_headers(tmp_path, blob, msg):
    p = tmp_path / "c.gguf"
    p.write_bytes(blob)
    with pytest.raises(GGUFFormatError, match=msg):
        GGUF.open(p)


def test_unknown_ggml_type(tmp_path):
    p = tmp_path / "t.gguf"
    G.write_gguf(p, [("w", (4,), 99, bytes(4))])
    with pytest.raises(GGUFFormatError, match="Unknown GGML type: 99"):
        GGUF.open(p)


def test_directory_pointing_outside_the_file(tmp_path):
    blob, _, _ = G.gguf_bytes([("w", (1024,), 0, bytes(64))])  # claims 4096 bytes, file holds 64
    p = tmp_path / "short.gguf"
    p.write_bytes(blob)
    with GGUF.open(p) as g:
        assert g.tensor_info("w").size == 4096
        with pytest.raises(GGUFFormatError):
            g.tensor("w")


def test_handles(tmp_path):
    lib = N.load()
    assert lib.wf_gguf_close(12345) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_gguf_info(0, None, None, None, None, None, None) == N.WF_ERR_INVALID_HANDLE
    p = tmp_path / "h.gguf"
    G.write_gguf(p, [("w", (32, 4), 2, bytes(72))])
    g = GGUF.open(p)
    h = g.handle
    w = ctypes.c_int64()
    # no context: the upload is refused before anything touches a device
    assert lib.wf_gguf_upload(0, h, b"w", 0, 1, 0, ctypes.byref(w)) == N.WF_ERR_INVALID_HANDLE
    g.close()
    assert lib.wf_gguf_close(h) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_gguf_tensor_info(h, b"w", None, None, None, None, None) == N.WF_ERR_INVALID_HANDLE
    assert N.error_name(N.WF_ERR_GGUF) == "WF_ERR_GGUF"


def test_file_from_the_gguf_package(tmp_path):
    """A file written by the third-party gguf package (black box) reads back the same through the
    native reader as through that package's own reader."""
    gguf = pytest.importorskip("gguf")
    p = tmp_path / "pkg.gguf"
    rng = np.random.default_rng(7)
    w32 = rng.standard_normal((6, 64)).astype(np.float32)
    q8 = gguf.quants.quantize(rng.standard_normal((8, 128)).astype(np.float32), gguf.GGMLQuantizationType.Q8_0)
    q4 = gguf.quants.quantize(rng.standard_normal((4, 64)).astype(np.float32), gguf.GGMLQuantizationType.Q4_0)
    wr = gguf.GGUFWriter(str(p), "llama")
    wr.add_name("pkg model")
    wr.add_block_count(3)
    wr.add_tensor("dense", w32)
    wr.add_tensor("blk.0.attn_q.weight", q8, raw_dtype=gguf.GGMLQuantizationType.Q8_0)
    wr.add_tensor("blk.0.ffn_up.weight", q4, raw_dtype=gguf.GGMLQuantizationType.Q4_0)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    rd = gguf.GGUFReader(str(p))
    with GGUF.open(p) as g:
        assert g.version() == 3 and g.metadata()["general.architecture"] == "llama" and g.metadata()["general.name"] == "pkg model"
        assert g.metadata()["llama.block_count"] == "3"
        assert g.tensor_names() == [t.name for t in rd.tensors]
        assert g.data_offset == rd.data_offset and g.alignment == rd.alignment
        for t in rd.tensors:
            info = g.tensor_info(t.name)
            assert info.ggml_type == int(t.tensor_type) and info.shape == tuple(int(d) for d in t.shape)
            assert g.data_offset + info.offset == t.data_offset and info.size == t.n_bytes
            assert np.array_equal(g.tensor(t.name), np.asarray(t.data).view(np.uint8).ravel())
        assert g.tensor_info("blk.0.attn_q.weight").shape == (128, 8)  # {k, rows}
