"""Pins the CPU oracle: against the reference's own known-answer tests (transcribed in
tests/golden/reference_kats.json), against its numpy twin, and -- for Q4_K, which the
reference does not implement -- against the third-party gguf package used as a black box."""
import json
import math
import os

import numpy as np
import pytest

from oracle import oracle as O
from warpforge_b200 import quant as Q

KATS = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))


def _num(v):
    return {"inf": math.inf, "nan": math.nan}.get(v, v) if isinstance(v, str) else v


def test_fp16_kat(oracle):
    k = KATS["fp16"]
    for impl in (oracle.half_to_float, O.np_half_to_float):
        got = impl(np.array(k["bits"], np.uint16))
        for g, e, tol in zip(got, map(_num, k["expected"]), k["tol"]):
            if math.isnan(e):
                assert math.isnan(g)
            elif math.isinf(e):
                assert math.isinf(g) and g > 0
            else:
                assert abs(g - e) <= tol


def test_fp16_all_patterns_match_ieee(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    got = oracle.half_to_float(bits)
    want = bits.view(np.float16).astype(np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    # every NaN payload collapses to the canonical quiet NaN (Float.NaN), Dequantizer.java:140
    assert np.all(got[~finite].view(np.uint32) == 0x7FC00000)
    assert np.array_equal(O.np_half_to_float(bits).view(np.uint32), got.view(np.uint32))


def test_bf16_kat(oracle):
    k = KATS["bf16"]
    got = oracle.bf16_to_float(np.array(k["bits"], np.uint16))
    assert np.allclose(got, k["expected"], atol=k["tol"])
    assert np.array_equal(got, O.np_bf16_to_float(np.array(k["bits"], np.uint16)))


def test_q8_0_kat(oracle):
    k = KATS["q8_0"]
    blk = np.zeros(34, np.uint8)
    blk[:2] = np.array([k["scale_bits"]], np.uint16).view(np.uint8)
    blk[2:] = np.arange(32, dtype=np.uint8)
    for got in (oracle.dequant(O.Q8_0, blk, 32), O.np_dequant_q8_0(blk, 32)):
        for i in range(32):
            assert abs(got[i] - np.float32(i) * np.float32(0.1)) <= k["tol"]
    assert O.BLOCK_ELEMS[O.Q8_0] == k["block_size"] and O.BLOCK_BYTES[O.Q8_0] == k["bytes_per_block"]
    assert Q.QuantizationType.Q8_0.block_size() == 32 and Q.QuantizationType.Q8_0.bytes_per_block() == 34


def test_q4_0_kat_interleaved_order(oracle):
    k = KATS["q4_0"]
    blk = np.full(18, k["code_byte"], np.uint8)
    blk[:2] = np.array([k["scale_bits"]], np.uint16).view(np.uint8)
    for got in (oracle.dequant(O.Q4_0, blk, 32), O.np_dequant_q4_0(blk, 32)):
        assert np.allclose(got[0::2], k["expected_even"], atol=k["tol"])
        assert np.allclose(got[1::2], k["expected_odd"], atol=k["tol"])
    assert O.BLOCK_ELEMS[O.Q4_0] == k["block_size"] and O.BLOCK_BYTES[O.Q4_0] == k["bytes_per_block"]


def test_q4_0_order_differs_from_ggml(oracle):
    """The reference pairs byte i with elements (2i, 2i+1); ggml pairs it with (i, i+16)."""
    blk = np.zeros(18, np.uint8)
    blk[:2] = np.array([0x3C00], np.uint16).view(np.uint8)
    blk[2] = 0xF0  # low nibble 0 -> -8, high nibble 15 -> 7
    blk[3:] = 0x88
    got = oracle.dequant(O.Q4_0, blk, 32)
    assert got[0] == -8.0 and got[1] == 7.0 and np.all(got[2:] == 0.0)


def test_unsupported_type_throws(oracle):
    with pytest.raises(NotImplementedError):
        oracle.dequant(12, np.zeros(210, np.uint8), 256)  # Q6_K


def test_tail_rule(oracle):
    """blocks = ceil(n/32); writes stop at n (Dequantizer.java:205,216,252,263-276)."""
    w = Q.synth_q4_0(1, 64, 7).ravel()
    full = oracle.dequant(O.Q4_0, w, 64)
    assert np.array_equal(oracle.dequant(O.Q4_0, w, 37), full[:37])
    w8 = Q.synth_q8_0(1, 64, 7).ravel()
    assert np.array_equal(oracle.dequant(O.Q8_0, w8, 33), oracle.dequant(O.Q8_0, w8, 64)[:33])


def test_gguf_sizes():
    k = KATS["gguf_sizes"]
    assert Q.QuantizationType.Q4_0.tensor_bytes(k["q4_0"]["elements"]) == k["q4_0"]["bytes"]
    assert Q.QuantizationType.Q8_0.tensor_bytes(k["q8_0"]["elements"]) == k["q8_0"]["bytes"]
    assert Q.QuantizationType.Q4_0.compression_ratio() == k["q4_0_compression_ratio"]
    assert Q.QuantizationType.Q4_K.tensor_bytes(256) == 144


@pytest.mark.parametrize("qtype,gen", [(O.Q8_0, Q.synth_q8_0), (O.Q4_0, Q.synth_q4_0), (O.Q4_K, Q.synth_q4_k)])
def test_c_oracle_matches_numpy_twin_bitwise(oracle, qtype, gen):
    w = gen(24, 1024, 1234)
    a = oracle.dequant(qtype, w, 24 * 1024)
    b = O.np_dequant(qtype, w, 24 * 1024)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_subnormal_and_edge_scales(oracle):
    blk = np.zeros((4, 18), np.uint8)
    for i, bits in enumerate([0x0001, 0x03FF, 0x8001, 0x7BFF]):  # min/max subnormal, -subnormal, max half
        blk[i, :2] = np.array([bits], np.uint16).view(np.uint8)
        blk[i, 2:] = np.arange(16, dtype=np.uint8) * 17
    a = oracle.dequant(O.Q4_0, blk, 128)
    b = O.np_dequant_q4_0(blk, 128)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert a[2] == np.float32(-7.0) * np.float32(2.0 ** -24)  # byte 0x11: code 1 -> (1 - 8) * min subnormal


def test_q4_k_against_gguf_package(oracle):
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    w = Q.synth_q4_k(16, 1024, 99)
    want = quants.dequantize(w.reshape(-1, 144), gguf.GGMLQuantizationType.Q4_K).astype(np.float32).ravel()
    got = oracle.dequant(O.Q4_K, w, 16 * 1024)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q8_0_against_gguf_package(oracle):
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    w = Q.synth_q8_0(8, 256, 5)
    want = quants.dequantize(w.reshape(-1, 34), gguf.GGMLQuantizationType.Q8_0).astype(np.float32).ravel()
    assert np.array_equal(oracle.dequant(O.Q8_0, w, 8 * 256).view(np.uint32), want.view(np.uint32))


def test_q4_0_is_a_permutation_of_ggml_order(oracle):
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    w = Q.synth_q4_0(4, 128, 5)
    ggml = quants.dequantize(w.reshape(-1, 18), gguf.GGMLQuantizationType.Q4_0).astype(np.float32).reshape(-1, 32)
    ref = oracle.dequant(O.Q4_0, w, 4 * 128).reshape(-1, 32)
    assert np.array_equal(ref[:, 0::2], ggml[:, :16]) and np.array_equal(ref[:, 1::2], ggml[:, 16:])


def test_q4k_scale_pack_roundtrip():
    rng = np.random.default_rng(3)
    sc = rng.integers(0, 64, (50, 8), dtype=np.uint8)
    m = rng.integers(0, 64, (50, 8), dtype=np.uint8)
    sc2, m2 = O.np_q4k_scales_mins(Q.pack_q4k_scales(sc, m))
    assert np.array_equal(sc, sc2) and np.array_equal(m, m2)


def test_dot_kats(oracle):
    for k in KATS["dot"]:
        a = np.array(k["a"], np.float32).reshape(k["a_shape"])
        b = np.array(k["b"], np.float32).reshape(k["b_shape"])
        assert np.allclose(oracle.dot(a, b).ravel(), k["expected"], atol=k["tol"], rtol=0)


def test_dot_general_kats(oracle):
    tol = KATS["tolerance_dot_general"]
    for k in KATS["dot_general"]:
        lhs = np.array(k["lhs"], np.float32).reshape(k["lhs_shape"])
        rhs = np.array(k["rhs"], np.float32).reshape(k["rhs_shape"])
        got = oracle.dot_general(lhs, rhs, lhs_contract=k["lhs_contract"], rhs_contract=k["rhs_contract"])
        assert O.is_close_count(k["expected"], got, tol["atol"], tol["rtol"]) == 0
        assert oracle.count_not_close(np.array(k["expected"], np.float32), got, tol["atol"], tol["rtol"]) == 0


def test_dot_general_linear_form_and_batch(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 40)).astype(np.float32)
    w = rng.standard_normal((5, 40)).astype(np.float32)
    lin = oracle.dot_general(x, w, lhs_contract=(1,), rhs_contract=(1,))  # torch linear lowering
    assert np.array_equal(lin, oracle.linear(x, w))
    assert np.array_equal(lin, O.np_linear_sequential(x, w))
    a = rng.standard_normal((2, 3, 4)).astype(np.float32)
    b = rng.standard_normal((2, 4, 5)).astype(np.float32)
    got = oracle.dot_general(a, b, lhs_batch=(0,), rhs_batch=(0,), lhs_contract=(2,), rhs_contract=(1,))
    assert got.shape == (2, 3, 5) and np.allclose(got, a @ b, atol=1e-5)


def test_sequential_accumulation_is_not_fused(oracle):
    """One case where fused multiply-add and multiply-then-add differ in the last bit."""
    x = np.array([[1.0 + 2.0 ** -12, 1.0]], np.float32)
    w = np.array([[1.0 + 2.0 ** -12, -1.0]], np.float32)
    want = np.float32(np.float32(x[0, 0] * w[0, 0]) + np.float32(x[0, 1] * w[0, 1]))
    assert oracle.linear(x, w)[0, 0] == want
    exact = float(x[0, 0]) * float(w[0, 0]) - 1.0
    assert float(want) != exact  # the unfused result dropped the 2^-24 term


@pytest.mark.parametrize("qtype,gen,k", [(O.Q8_0, Q.synth_q8_0, 256), (O.Q4_0, Q.synth_q4_0, 256),
                                          (O.Q4_K, Q.synth_q4_k, 512)])
def test_qlinear_matches_twin_and_threads(oracle, qtype, gen, k):
    n, m = 48, 3
    w = gen(n, k, 42)
    x = Q.bf16_bits_to_float(Q.synth_activation_bf16(m, k, 42))
    y1 = oracle.qlinear(qtype, w, n, k, x, nthreads=1)
    y4 = oracle.qlinear(qtype, w, n, k, x, nthreads=4)
    twin = O.np_linear_sequential(x, O.np_dequant(qtype, w, n * k).reshape(n, k))
    assert np.array_equal(y1.view(np.uint32), y4.view(np.uint32))
    assert np.array_equal(y1.view(np.uint32), twin.view(np.uint32))
    rows = np.array([0, 5, 47, 13])
    assert np.array_equal(oracle.qlinear_rows(qtype, w, k, x, rows, nthreads=2), y1[:, rows])


def test_config1_shape_runs_on_cpu(oracle):
    """benchmark config 1: single Q8_0 linear [4096 x 4096], x fp32 [1 x 4096]."""
    w = Q.synth_q8_0(4096, 4096, Q.config_seed(1))
    x = Q.synth_activation_f32(1, 4096, Q.config_seed(1))
    y = oracle.qlinear(O.Q8_0, w, 4096, 4096, x, nthreads=oracle.max_threads())
    assert y.shape == (1, 4096) and np.isfinite(y).all()
    wf = oracle.dequant(O.Q8_0, w, 4096 * 4096).reshape(4096, 4096)
    ref64 = x.astype(np.float64) @ wf.astype(np.float64).T
    assert np.max(np.abs(y - ref64)) / np.max(np.abs(ref64)) < 1e-5


def test_q4_0_ggml_order_against_gguf_package(oracle):
    """Blocks in ggml's nibble order, rewritten to the reference's order, dequantize (by the
    reference's rule) to exactly what the gguf package makes of the original blocks."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    w = Q.synth_q4_0(8, 256, 11)
    want = quants.dequantize(w.reshape(-1, 18), gguf.GGMLQuantizationType.Q4_0).astype(np.float32).ravel()
    got = oracle.dequant(O.Q4_0, O.q4_0_ggml_to_reference_order(w), 8 * 256)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(O.np_dequant_q4_0_ggml(w, 8 * 256).view(np.uint32), want.view(np.uint32))


def test_q4_1_ggml_order_against_gguf_package(oracle):
    """Q4_1 (Dequantizer.java:304-358 has no block test in the reference): ggml-ordered blocks rewritten to
    the reference's order dequantize to what the gguf package makes of them, up to the package's fused
    d * q + m (it computes in fp32 numpy: product and sum rounded separately, as the reference does)."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    w = Q.synth_q4_1(8, 256, 12)
    want = quants.dequantize(w.reshape(-1, 20), gguf.GGMLQuantizationType.Q4_1).astype(np.float32).ravel()
    got = oracle.dequant(O.Q4_1, O.q4_0_ggml_to_reference_order(w, header=4), 8 * 256)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q5_0_against_gguf_package(oracle):
    """Q5_0 is a format the reference can only size (GGUF.java:332-351): the restatement of the public block
    format (C and numpy) is checked against the independent implementation in the gguf package, bit for bit.
    Parity with the reference itself is unpinned for this type: the reference has no dequantizer for it."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    w = Q.synth_q5_0(8, 256, 13)
    want = quants.dequantize(w.reshape(-1, 22), gguf.GGMLQuantizationType.Q5_0).astype(np.float32).ravel()
    got = oracle.dequant(O.Q5_0, w, 8 * 256)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(O.np_dequant_q5_0(w, 8 * 256).view(np.uint32), want.view(np.uint32))
    assert Q.QuantizationType.Q5_0.tensor_bytes(8 * 256) == 8 * 8 * 22 and O.BLOCK_BYTES[O.Q5_0] == 22
