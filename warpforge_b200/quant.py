"""Block-quantization geometry and seeded synthetic GGUF block generators (host side).

``QuantizationType`` mirrors the members of the reference enum that this path handles
(warpforge-data/src/main/java/io/surfworks/warpforge/data/quant/QuantizationType.java:9-58):
bits per weight, compression ratio, plus the block geometry the reference spreads over
``Dequantizer.blockSize()/bytesPerBlock()`` (Dequantizer.java:199-298) and the GGUF size
table (warpforge-data/src/main/java/io/surfworks/warpforge/data/format/GGUF.java:332-351).

The generators write genuine GGUF block bytes so the same buffers feed the CPU checker,
third-party GGUF tooling and the device upload.  They only produce inputs; no arithmetic
of the product path lives here.
"""
from __future__ import annotations

import enum

import numpy as np


class QuantizationType(enum.Enum):
    """(ggml type id, bits, block elements, block bytes)."""

    Q4_0 = (2, 4, 32, 18)
    Q4_1 = (3, 4, 32, 20)
    Q5_0 = (6, 5, 32, 22)
    Q8_0 = (8, 8, 32, 34)
    Q4_K = (14, 4, 256, 144)

    @property
    def ggml_type(self) -> int:
        return self.value[0]

    def bits(self) -> int:
        return self.value[1]

    def is_quantized(self) -> bool:
        return True

    def compression_ratio(self) -> float:
        return 32.0 / self.value[1]

    def block_size(self) -> int:
        return self.value[2]

    def bytes_per_block(self) -> int:
        return self.value[3]

    def row_bytes(self, k: int) -> int:
        if k % self.block_size():
            raise ValueError(f"K={k} is not a multiple of the {self.name} block size {self.block_size()}")
        return k // self.block_size() * self.bytes_per_block()

    def tensor_bytes(self, elements: int) -> int:
        """GGUF.java:332-351: ceil(elements / block) * bytes_per_block."""
        bs = self.block_size()
        return (elements + bs - 1) // bs * self.bytes_per_block()

    @classmethod
    def from_ggml(cls, ggml_type: int) -> "QuantizationType":
        for q in cls:
            if q.ggml_type == ggml_type:
                return q
        raise ValueError(f"Unknown or unsupported GGML type for quantized matmul: {ggml_type}")


BASE_SEED = 20261125


def config_seed(config: int, matrix_index: int = 0) -> int:
    return BASE_SEED + 1000 * config + matrix_index


def float_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bits, round to nearest even (inputs are finite)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_float(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def _fp16_scales(rng: np.random.Generator, shape, s: float) -> np.ndarray:
    return (np.abs(rng.standard_normal(shape)) * s).astype(np.float32).astype(np.float16)


def synth_q8_0(n_rows: int, k: int, seed: int, scale: float = 0.02) -> np.ndarray:
    """int8 codes uniform in [-127, 127], one fp16 scale |N(0,1)|*scale per block of 32."""
    rng = np.random.Generator(np.random.PCG64(seed))
    nb = n_rows * k // 32
    out = np.empty((nb, 34), np.uint8)
    out[:, :2] = _fp16_scales(rng, nb, scale).view(np.uint8).reshape(nb, 2)
    out[:, 2:] = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(n_rows, -1)


def synth_q4_0(n_rows: int, k: int, seed: int, scale: float = 0.02) -> np.ndarray:
    """4-bit codes uniform 0..15 (value = code - 8), one fp16 scale per block of 32."""
    rng = np.random.Generator(np.random.PCG64(seed))
    nb = n_rows * k // 32
    out = np.empty((nb, 18), np.uint8)
    out[:, :2] = _fp16_scales(rng, nb, scale).view(np.uint8).reshape(nb, 2)
    out[:, 2:] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    return out.reshape(n_rows, -1)


def synth_q4_1(n_rows: int, k: int, seed: int, scale: float = 0.02) -> np.ndarray:
    """4-bit codes uniform 0..15 (value = code * scale + min), fp16 scale |N(0,1)|*scale and fp16 min
    -8 * |N(0,1)|*scale per block of 32 (the asymmetric counterpart of the Q4_0 distribution)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    nb = n_rows * k // 32
    out = np.empty((nb, 20), np.uint8)
    out[:, 0:2] = _fp16_scales(rng, nb, scale).view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = (-8 * _fp16_scales(rng, nb, scale).astype(np.float32)).astype(np.float16).view(np.uint8).reshape(nb, 2)
    out[:, 4:] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    return out.reshape(n_rows, -1)


def synth_q5_0(n_rows: int, k: int, seed: int, scale: float = 0.02) -> np.ndarray:
    """5-bit codes uniform 0..31 (value = (code - 16) * scale): fp16 scale |N(0,1)|*scale, 32 high bits and
    16 nibble bytes per block of 32, in the file's own (ggml) element order."""
    rng = np.random.Generator(np.random.PCG64(seed))
    nb = n_rows * k // 32
    out = np.empty((nb, 22), np.uint8)
    out[:, 0:2] = _fp16_scales(rng, nb, scale).view(np.uint8).reshape(nb, 2)
    out[:, 2:] = rng.integers(0, 256, size=(nb, 20), dtype=np.uint8)
    return out.reshape(n_rows, -1)


def pack_q4k_scales(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """[nb, 8] 6-bit scales and mins -> the 12-byte field of a Q4_K super-block."""
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    s = np.empty((sc.shape[0], 12), np.uint8)
    s[:, 0:4] = (sc[:, :4] & 63) | ((sc[:, 4:] >> 4) << 6)
    s[:, 4:8] = (m[:, :4] & 63) | ((m[:, 4:] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:] & 0x0F) | ((m[:, 4:] & 0x0F) << 4)
    return s


def synth_q4_k(n_rows: int, k: int, seed: int, scale: float = 0.01) -> np.ndarray:
    """256-element super-blocks: fp16 d and dmin |N(0,1)|*scale, 6-bit sub-block scales and
    mins uniform 0..63, 4-bit codes uniform."""
    rng = np.random.Generator(np.random.PCG64(seed))
    nb = n_rows * k // 256
    out = np.empty((nb, 144), np.uint8)
    out[:, 0:2] = _fp16_scales(rng, nb, scale).view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = _fp16_scales(rng, nb, scale).view(np.uint8).reshape(nb, 2)
    sc = rng.integers(0, 64, size=(nb, 8), dtype=np.uint8)
    m = rng.integers(0, 64, size=(nb, 8), dtype=np.uint8)
    out[:, 4:16] = pack_q4k_scales(sc, m)
    out[:, 16:] = rng.integers(0, 256, size=(nb, 128), dtype=np.uint8)
    return out.reshape(n_rows, -1)


def synth_weight(qtype: QuantizationType, n_rows: int, k: int, seed: int) -> np.ndarray:
    """Returns uint8 [n_rows, row_bytes] of GGUF blocks (blocks run along K inside a row)."""
    qtype.row_bytes(k)
    return {QuantizationType.Q8_0: synth_q8_0, QuantizationType.Q4_0: synth_q4_0,
            QuantizationType.Q4_1: synth_q4_1, QuantizationType.Q4_K: synth_q4_k,
            QuantizationType.Q5_0: synth_q5_0}[qtype](n_rows, k, seed)


def synth_activation_f32(m: int, k: int, seed: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed ^ 0x5A5A5A))
    return rng.standard_normal((m, k)).astype(np.float32)


def synth_activation_bf16(m: int, k: int, seed: int) -> np.ndarray:
    """bf16 bit patterns (uint16) of N(0,1) rounded to nearest even."""
    return float_to_bf16_bits(synth_activation_f32(m, k, seed)).reshape(m, k)
