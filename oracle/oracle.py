"""CPU oracle for the quantized-matmul path -- TEST INFRASTRUCTURE, not product code.

Two independent restatements of the reference's CPU arithmetic:

* ``COracle`` loads ``libwforacle.so`` (built from ``wf_oracle.c`` by the Makefile beside
  it) through ctypes.  It is the checker for full-size cases and the timed CPU baseline.
* the ``np_*`` functions are a numpy twin used to cross-check the C code on small cases.

Reference files followed (paths inside the WarpForge project):
  warpforge-data/src/main/java/io/surfworks/warpforge/data/quant/Dequantizer.java:121-147 (fp16),
  :204-221 (Q8_0), :251-279 (Q4_0, interleaved nibble order), :304-358 (Q4_1);
  warpforge-backend-cpu/src/main/java/io/surfworks/warpforge/backend/cpu/ops/scalar/DotGeneralKernel.java:85-128
  (fp32 ``sum += a*b``, k ascending, one accumulator, multiply and add rounded separately).
Q4_K is not implemented by the reference (Dequantizer.java:58-71 throws); the functions
here follow the public GGUF Q4_K block format and their parity is unpinned.

Nothing under the product package imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libwforacle.so")

Q4_0, Q4_1, Q8_0, Q4_K, Q5_0 = 2, 3, 8, 14, 6  # ggml type ids, GGUF.java:297-305
BLOCK_ELEMS = {Q4_0: 32, Q4_1: 32, Q8_0: 32, Q4_K: 256, Q5_0: 32}
BLOCK_BYTES = {Q4_0: 18, Q4_1: 20, Q8_0: 34, Q4_K: 144, Q5_0: 22}


def build(force: bool = False) -> str:
    """Compile wf_oracle.c with the Makefile beside it; returns the library path."""
    src = os.path.join(HERE, "wf_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "libwforacle.so"], check=True, capture_output=True)
    return LIB_PATH


def _ptr(a: np.ndarray, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype))


class COracle:
    """ctypes face of libwforacle.so."""

    def __init__(self, path: str | None = None):
        self.lib = ctypes.CDLL(path or build())
        L = self.lib
        u8p, f32p, i64p = (ctypes.POINTER(t) for t in (ctypes.c_uint8, ctypes.c_float, ctypes.c_int64))
        u16p = ctypes.POINTER(ctypes.c_uint16)
        L.wfo_half_to_float.restype = ctypes.c_float
        L.wfo_half_to_float.argtypes = [ctypes.c_uint16]
        L.wfo_half_to_float_array.argtypes = [u16p, f32p, ctypes.c_int64]
        L.wfo_bf16_to_float_array.argtypes = [u16p, f32p, ctypes.c_int64]
        L.wfo_dequant.restype = ctypes.c_int
        L.wfo_dequant.argtypes = [ctypes.c_int, u8p, f32p, ctypes.c_int64]
        L.wfo_dot_f32.argtypes = [f32p, f32p, f32p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
        L.wfo_dot_general_f32.restype = ctypes.c_int
        L.wfo_dot_general_f32.argtypes = [f32p, i64p, ctypes.c_int, f32p, i64p, ctypes.c_int, i64p, i64p,
                                          ctypes.c_int, i64p, i64p, ctypes.c_int, f32p]
        L.wfo_linear_f32.argtypes = [f32p, f32p, f32p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                     ctypes.c_int]
        L.wfo_qlinear.restype = ctypes.c_int
        L.wfo_qlinear.argtypes = [ctypes.c_int, u8p, ctypes.c_int64, ctypes.c_int64, f32p, ctypes.c_int64,
                                  f32p, ctypes.c_int]
        L.wfo_qlinear_rows.restype = ctypes.c_int
        L.wfo_qlinear_rows.argtypes = [ctypes.c_int, u8p, ctypes.c_int64, f32p, ctypes.c_int64, i64p,
                                       ctypes.c_int64, f32p, ctypes.c_int]
        L.wfo_count_not_close.restype = ctypes.c_int64
        L.wfo_count_not_close.argtypes = [f32p, f32p, ctypes.c_int64, ctypes.c_double, ctypes.c_double]
        L.wfo_max_threads.restype = ctypes.c_int
        i64 = ctypes.c_int64
        L.wfo_rms_norm.argtypes = [f32p, f32p, f32p, i64, i64, ctypes.c_float]
        L.wfo_layer_norm.argtypes = [f32p, f32p, f32p, f32p, i64, i64, ctypes.c_float]
        L.wfo_softmax.argtypes = [f32p, f32p, i64, i64]
        L.wfo_silu.argtypes = [f32p, f32p, i64]
        L.wfo_gelu.argtypes = [f32p, f32p, i64]
        L.wfo_swiglu.argtypes = [f32p, f32p, f32p, i64]
        L.wfo_add.argtypes = [f32p, f32p, f32p, i64]
        L.wfo_embedding.restype = ctypes.c_int
        L.wfo_embedding.argtypes = [i64p, f32p, f32p, i64, i64, i64]

    def max_threads(self) -> int:
        return int(self.lib.wfo_max_threads())

    def half_to_float(self, bits) -> np.ndarray:
        a = np.ascontiguousarray(bits, dtype=np.uint16).ravel()
        out = np.empty(a.size, np.float32)
        self.lib.wfo_half_to_float_array(_ptr(a, ctypes.c_uint16), _ptr(out, ctypes.c_float), a.size)
        return out

    def bf16_to_float(self, bits) -> np.ndarray:
        a = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(a.shape, np.float32)
        self.lib.wfo_bf16_to_float_array(_ptr(a, ctypes.c_uint16), _ptr(out, ctypes.c_float), a.size)
        return out

    def dequant(self, qtype: int, blocks, n: int) -> np.ndarray:
        b = np.ascontiguousarray(blocks, dtype=np.uint8).ravel()
        out = np.empty(n, np.float32)
        rc = self.lib.wfo_dequant(qtype, _ptr(b, ctypes.c_uint8), _ptr(out, ctypes.c_float), n)
        if rc != 0:
            raise NotImplementedError(f"Dequantization not yet implemented for: {qtype}")
        return out

    def dot(self, a, b) -> np.ndarray:
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        M, K = a.shape
        K2, N = b.shape
        assert K == K2
        c = np.empty((M, N), np.float32)
        self.lib.wfo_dot_f32(_ptr(a, ctypes.c_float), _ptr(b, ctypes.c_float), _ptr(c, ctypes.c_float), M, K, N)
        return c

    def dot_general(self, lhs, rhs, lhs_batch=(), rhs_batch=(), lhs_contract=(1,), rhs_contract=(0,)):
        lhs = np.ascontiguousarray(lhs, np.float32)
        rhs = np.ascontiguousarray(rhs, np.float32)
        lfree = [d for d in range(lhs.ndim) if d not in lhs_batch and d not in lhs_contract]
        rfree = [d for d in range(rhs.ndim) if d not in rhs_batch and d not in rhs_contract]
        oshape = [lhs.shape[d] for d in lhs_batch] + [lhs.shape[d] for d in lfree] + [rhs.shape[d] for d in rfree]
        out = np.empty(oshape, np.float32)
        mk = lambda v: np.asarray(list(v) or [0], np.int64)
        ls, rs = mk(lhs.shape), mk(rhs.shape)
        lb, rb, lc, rc_ = mk(lhs_batch), mk(rhs_batch), mk(lhs_contract), mk(rhs_contract)
        i64 = ctypes.c_int64
        rc = self.lib.wfo_dot_general_f32(_ptr(lhs, ctypes.c_float), _ptr(ls, i64), lhs.ndim,
                                          _ptr(rhs, ctypes.c_float), _ptr(rs, i64), rhs.ndim,
                                          _ptr(lb, i64), _ptr(rb, i64), len(lhs_batch),
                                          _ptr(lc, i64), _ptr(rc_, i64), len(lhs_contract),
                                          _ptr(out, ctypes.c_float))
        assert rc == 0
        return out

    def linear(self, x, w, nthreads: int = 1) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        M, K = x.shape
        N = w.shape[0]
        y = np.empty((M, N), np.float32)
        self.lib.wfo_linear_f32(_ptr(x, ctypes.c_float), _ptr(w, ctypes.c_float), _ptr(y, ctypes.c_float),
                                M, N, K, nthreads)
        return y

    def qlinear(self, qtype: int, blocks, N: int, K: int, x, nthreads: int = 1) -> np.ndarray:
        """y[M,N] = x[M,K] . dequant(blocks)[N,K]^T with the reference's accumulate rule."""
        b = np.ascontiguousarray(blocks, dtype=np.uint8).ravel()
        x = np.ascontiguousarray(x, np.float32)
        M = x.shape[0]
        assert x.shape[1] == K and b.size == N * (K // BLOCK_ELEMS[qtype]) * BLOCK_BYTES[qtype]
        y = np.empty((M, N), np.float32)
        rc = self.lib.wfo_qlinear(qtype, _ptr(b, ctypes.c_uint8), N, K, _ptr(x, ctypes.c_float), M,
                                  _ptr(y, ctypes.c_float), nthreads)
        if rc != 0:
            raise ValueError(f"wfo_qlinear failed: {rc}")
        return y

    def qlinear_rows(self, qtype: int, blocks, K: int, x, rows, nthreads: int = 1) -> np.ndarray:
        """Sampled rows: returns [M, len(rows)]."""
        b = np.ascontiguousarray(blocks, dtype=np.uint8).ravel()
        x = np.ascontiguousarray(x, np.float32)
        rows = np.ascontiguousarray(rows, np.int64)
        M = x.shape[0]
        y = np.empty((rows.size, M), np.float32)
        rc = self.lib.wfo_qlinear_rows(qtype, _ptr(b, ctypes.c_uint8), K, _ptr(x, ctypes.c_float), M,
                                       _ptr(rows, ctypes.c_int64), rows.size, _ptr(y, ctypes.c_float), nthreads)
        if rc != 0:
            raise ValueError(f"wfo_qlinear_rows failed: {rc}")
        return np.ascontiguousarray(y.T)

    # ---- the fp32 operations between the projections (CustomCallKernel.java); x is [rows, n] or flat
    @staticmethod
    def _f32(a):
        return np.ascontiguousarray(a, np.float32)

    def _opt(self, a):
        return None if a is None else _ptr(self._f32(a), ctypes.c_float)

    def rms_norm(self, x, gamma=None, eps: float = 1e-5) -> np.ndarray:
        x = self._f32(x)
        y = np.empty_like(x)
        self.lib.wfo_rms_norm(_ptr(x, ctypes.c_float), self._opt(gamma), _ptr(y, ctypes.c_float), x.size // x.shape[-1], x.shape[-1], eps)
        return y

    def layer_norm(self, x, gamma=None, beta=None, eps: float = 1e-5) -> np.ndarray:
        x = self._f32(x)
        y = np.empty_like(x)
        self.lib.wfo_layer_norm(_ptr(x, ctypes.c_float), self._opt(gamma), self._opt(beta), _ptr(y, ctypes.c_float),
                                x.size // x.shape[-1], x.shape[-1], eps)
        return y

    def softmax(self, x) -> np.ndarray:
        x = self._f32(x)
        y = np.empty_like(x)
        self.lib.wfo_softmax(_ptr(x, ctypes.c_float), _ptr(y, ctypes.c_float), x.size // x.shape[-1], x.shape[-1])
        return y

    def silu(self, x) -> np.ndarray:
        x = self._f32(x)
        y = np.empty_like(x)
        self.lib.wfo_silu(_ptr(x, ctypes.c_float), _ptr(y, ctypes.c_float), x.size)
        return y

    def gelu(self, x) -> np.ndarray:
        x = self._f32(x)
        y = np.empty_like(x)
        self.lib.wfo_gelu(_ptr(x, ctypes.c_float), _ptr(y, ctypes.c_float), x.size)
        return y

    def swiglu(self, gate, up) -> np.ndarray:
        gate, up = self._f32(gate), self._f32(up)
        y = np.empty_like(gate)
        self.lib.wfo_swiglu(_ptr(gate, ctypes.c_float), _ptr(up, ctypes.c_float), _ptr(y, ctypes.c_float), gate.size)
        return y

    def add(self, a, b) -> np.ndarray:
        a, b = self._f32(a), self._f32(b)
        y = np.empty_like(a)
        self.lib.wfo_add(_ptr(a, ctypes.c_float), _ptr(b, ctypes.c_float), _ptr(y, ctypes.c_float), a.size)
        return y

    def embedding(self, indices, table) -> np.ndarray:
        idx = np.ascontiguousarray(indices, np.int64)
        table = self._f32(table)
        y = np.empty(idx.shape + (table.shape[1],), np.float32)
        rc = self.lib.wfo_embedding(_ptr(idx, ctypes.c_int64), _ptr(table, ctypes.c_float), _ptr(y, ctypes.c_float), idx.size,
                                    table.shape[0], table.shape[1])
        if rc != 0:
            raise IndexError("embedding index outside the table")
        return y

    def count_not_close(self, expected, actual, atol=1e-4, rtol=1e-3) -> int:
        e = np.ascontiguousarray(expected, np.float32).ravel()
        a = np.ascontiguousarray(actual, np.float32).ravel()
        assert e.size == a.size
        return int(self.lib.wfo_count_not_close(_ptr(e, ctypes.c_float), _ptr(a, ctypes.c_float), e.size,
                                                atol, rtol))


# ----------------------------------------------------------------------------- numpy twin


def np_half_to_float(bits) -> np.ndarray:
    """Dequantizer.java:121-147, vectorised; NaNs come out as the canonical Float.NaN."""
    b = np.asarray(bits, dtype=np.uint16).astype(np.uint32)
    sign, exp, mant = (b >> 15) & 1, (b >> 10) & 0x1F, b & 0x3FF
    normal = ((sign << 31) | ((exp + 112) << 23) | (mant << 13)).astype(np.uint32).view(np.float32)
    sub = (mant.astype(np.float32) / np.float32(1024.0)) * np.float32(2.0 ** -14)
    sub = np.where(sign == 1, -sub, sub).astype(np.float32)
    inf = np.where(sign == 1, -np.inf, np.inf).astype(np.float32)
    nan = np.full(b.shape, 0x7FC00000, np.uint32).view(np.float32)
    out = np.where(exp == 0, sub, normal)
    out = np.where((exp == 31) & (mant == 0), inf, out)
    out = np.where((exp == 31) & (mant != 0), nan, out)
    return out.astype(np.float32)


def np_bf16_to_float(bits) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def np_dequant_q8_0(blocks, n: int) -> np.ndarray:
    blk = np.asarray(blocks, np.uint8).reshape(-1, 34)
    d = np_half_to_float(blk[:, :2].copy().view(np.uint16)[:, 0])
    q = blk[:, 2:].view(np.int8).astype(np.float32)
    return (q * d[:, None]).astype(np.float32).ravel()[:n]


def np_dequant_q4_0(blocks, n: int) -> np.ndarray:
    blk = np.asarray(blocks, np.uint8).reshape(-1, 18)
    d = np_half_to_float(blk[:, :2].copy().view(np.uint16)[:, 0])
    qs = blk[:, 2:]
    vals = np.empty((blk.shape[0], 32), np.float32)
    vals[:, 0::2] = (qs & 0x0F).astype(np.int32) - 8  # byte i -> element 2i  (low nibble)
    vals[:, 1::2] = (qs >> 4).astype(np.int32) - 8  # byte i -> element 2i+1 (high nibble)
    return (vals * d[:, None]).astype(np.float32).ravel()[:n]


def q4_0_ggml_to_reference_order(blocks, header: int = 2) -> np.ndarray:
    """Q4_0 blocks (header 2: the scale) or Q4_1 blocks (header 4: scale and min) in ggml's nibble order
    (byte i = elements i and i+16) rewritten in the order the reference's Dequantizer.java:251-279 /
    :304-358 reads (byte i = elements 2i and 2i+1); the header bytes are untouched."""
    blk = np.asarray(blocks, np.uint8).reshape(-1, header + 16).copy()
    qs = blk[:, header:]
    elems = np.concatenate([qs & 0x0F, qs >> 4], axis=1)  # [nb, 32] in element order
    blk[:, header:] = elems[:, 0::2] | (elems[:, 1::2] << 4)
    return blk.ravel()


def np_dequant_q4_0_ggml(blocks, n: int) -> np.ndarray:
    return np_dequant_q4_0(q4_0_ggml_to_reference_order(blocks), n)


def np_q4k_scales_mins(s: np.ndarray):
    """s: [nb, 12] uint8 -> (sc [nb, 8], m [nb, 8]) as in wfo_q4k_scale_min."""
    s = s.astype(np.uint8)
    sc = np.empty((s.shape[0], 8), np.uint8)
    m = np.empty((s.shape[0], 8), np.uint8)
    sc[:, :4] = s[:, 0:4] & 63
    m[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 6) << 4)
    m[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, m


def np_dequant_q4_k(blocks, n: int) -> np.ndarray:
    blk = np.asarray(blocks, np.uint8).reshape(-1, 144)
    d = np_half_to_float(blk[:, 0:2].copy().view(np.uint16)[:, 0])
    dmin = np_half_to_float(blk[:, 2:4].copy().view(np.uint16)[:, 0])
    sc, m = np_q4k_scales_mins(blk[:, 4:16])
    qs = blk[:, 16:].reshape(-1, 4, 32)
    q = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)
    dl = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    ml = (dmin[:, None] * m.astype(np.float32)).astype(np.float32)
    return ((dl[:, :, None] * q).astype(np.float32) - ml[:, :, None]).astype(np.float32).ravel()[:n]


def np_dequant_q5_0(blocks, n: int) -> np.ndarray:
    """Q5_0 (public GGUF format): d fp16, 32 high bits, 16 code bytes; element i < 16 = low nibble of byte i,
    element i + 16 = high nibble of byte i; w = d * ((nibble | bit << 4) - 16)."""
    blk = np.asarray(blocks, np.uint8).reshape(-1, 22)
    d = np_half_to_float(blk[:, :2].copy().view(np.uint16)[:, 0])
    qh = blk[:, 2:6].copy().view("<u4")[:, 0]
    qs = blk[:, 6:]
    nib = np.concatenate([qs & 0x0F, qs >> 4], axis=1).astype(np.int32)
    bits = ((qh[:, None] >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.int32)
    q = (nib | (bits << 4)) - 16
    return (q.astype(np.float32) * d[:, None]).astype(np.float32).ravel()[:n]


def np_dequant(qtype: int, blocks, n: int) -> np.ndarray:
    return {Q8_0: np_dequant_q8_0, Q4_0: np_dequant_q4_0, Q4_K: np_dequant_q4_k, Q5_0: np_dequant_q5_0}[qtype](blocks, n)


def np_linear_sequential(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y[M,N] with the reference's rule: one fp32 accumulator per output, k ascending,
    product and sum rounded separately (vectorised over outputs, never over k)."""
    x = np.asarray(x, np.float32)
    w = np.asarray(w, np.float32)
    acc = np.zeros((x.shape[0], w.shape[0]), np.float32)
    for k in range(x.shape[1]):
        acc = (acc + (x[:, k, None] * w[None, :, k]).astype(np.float32)).astype(np.float32)
    return acc


def is_close_count(expected, actual, atol=1e-4, rtol=1e-3) -> int:
    """ToleranceConfig.java:164-182 in numpy; number of elements NOT close."""
    e = np.asarray(expected, np.float64).ravel()
    a = np.asarray(actual, np.float64).ravel()
    both_nan = np.isnan(e) & np.isnan(a)
    any_nan = np.isnan(e) | np.isnan(a)
    both_inf = np.isinf(e) & np.isinf(a)
    any_inf = np.isinf(e) | np.isinf(a)
    with np.errstate(invalid="ignore"):
        close = np.abs(e - a) <= atol + rtol * np.abs(e)
    ok = np.where(both_nan, True, np.where(any_nan, False, np.where(both_inf, e == a, np.where(any_inf, False, close))))
    return int((~ok).sum())
