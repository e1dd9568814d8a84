// GGUF blocks -> tiled device layout (one-time, at upload), and the inverse check kernel
// that dequantizes rows of the tiled layout to fp32 bit-for-bit as the CPU does
// (warpforge-data/src/main/java/io/surfworks/warpforge/data/quant/Dequantizer.java:204-221
//  for Q8_0, :251-279 for Q4_0; Q4_K per the GGUF super-block format).
#include <cuda_fp16.h>

#include "wf_common.cuh"

namespace wf {

__device__ __forceinline__ uint32_t pack8(const uint32_t (&nib)[8]) {
    uint32_t w = 0;
#pragma unroll
    for (int e = 0; e < 8; e++) w |= (nib[e] & 0xFu) << (4 * nibble_pos(e));
    return (w << PLANE_ROT) | (w >> (32 - PLANE_ROT));
}

__device__ __forceinline__ uint16_t ld_u16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// One thread per (row, 32-k block, element group q).
__global__ void repack_q4_0_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ tiles, int64_t rows,
                                   int64_t nblk, int64_t kt, int ggml_order) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * nblk * 4) return;
    int q = idx & 3;
    int64_t bk = (idx >> 2) % nblk, r = (idx >> 2) / nblk;
    const uint8_t* src = raw + (r * nblk + bk) * 18;
    uint8_t* tile = tiles + ((r >> 4) * kt + (bk >> 2)) * Tile<WF_QTYPE_Q4_0>::BYTES;
    int ri = r & 15, j = bk & 3;
    uint32_t nib[8];
    if (ggml_order) {  // files written by ggml: byte i -> elements i (low), i + 16 (high)
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint8_t b = src[2 + ((8 * q + i) & 15)];
            nib[i] = q >= 2 ? (b >> 4) : (b & 0xF);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) {  // reference order: byte i -> elements 2i (low), 2i+1 (high)
            uint8_t b = src[2 + 4 * q + i];
            nib[2 * i] = b & 0xF;
            nib[2 * i + 1] = b >> 4;
        }
    }
    *reinterpret_cast<uint32_t*>(tile + plane_word_off(ri, j, q)) = pack8(nib);
    if (q == 0)
        *reinterpret_cast<uint16_t*>(tile + Tile<WF_QTYPE_Q4_0>::SCALE_OFF + (ri & 7) * 16 + (ri >> 3) * 8 + j * 2) =
            ld_u16(src);
}

// Q4_1 (Dequantizer.java:304-358): fp16 scale, fp16 min, 16 code bytes in the same two nibble orders.
__global__ void repack_q4_1_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ tiles, int64_t rows,
                                   int64_t nblk, int64_t kt, int ggml_order) {
    using T = Tile<WF_QTYPE_Q4_1>;
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * nblk * 4) return;
    int q = idx & 3;
    int64_t bk = (idx >> 2) % nblk, r = (idx >> 2) / nblk;
    const uint8_t* src = raw + (r * nblk + bk) * 20;
    uint8_t* tile = tiles + ((r >> 4) * kt + (bk >> 2)) * T::BYTES;
    int ri = r & 15, j = bk & 3;
    uint32_t nib[8];
    if (ggml_order) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint8_t b = src[4 + ((8 * q + i) & 15)];
            nib[i] = q >= 2 ? (b >> 4) : (b & 0xF);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint8_t b = src[4 + 4 * q + i];
            nib[2 * i] = b & 0xF;
            nib[2 * i + 1] = b >> 4;
        }
    }
    *reinterpret_cast<uint32_t*>(tile + plane_word_off(ri, j, q)) = pack8(nib);
    if (q == 0) {
        const int so = (ri & 7) * 16 + (ri >> 3) * 8 + j * 2;
        *reinterpret_cast<uint16_t*>(tile + T::SCALE_OFF + so) = ld_u16(src);
        *reinterpret_cast<uint16_t*>(tile + T::MIN_OFF + so) = ld_u16(src + 2);
    }
}

__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ tiles, int64_t rows,
                                   int64_t nblk, int64_t kt) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * nblk * 4) return;
    int q = idx & 3;
    int64_t bk = (idx >> 2) % nblk, r = (idx >> 2) / nblk;
    const uint8_t* src = raw + (r * nblk + bk) * 34;
    uint8_t* tile = tiles + ((r >> 4) * kt + (bk >> 2)) * Tile<WF_QTYPE_Q8_0>::BYTES;
    int ri = r & 15, j = bk & 3;
    uint32_t hi[8], lo[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {  // q = 16*(hi-8) + lo with hi/lo the nibbles of (byte ^ 0x80)
        uint8_t u = src[2 + 8 * q + i] ^ 0x80;
        hi[i] = u >> 4;
        lo[i] = u & 0xF;
    }
    int off = plane_word_off(ri, j, q);
    *reinterpret_cast<uint32_t*>(tile + off) = pack8(hi);
    *reinterpret_cast<uint32_t*>(tile + PLANE_BYTES + off) = pack8(lo);
    if (q == 0)
        *reinterpret_cast<uint16_t*>(tile + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + (ri & 7) * 16 + (ri >> 3) * 8 + j * 2) =
            ld_u16(src);
}

// Q5_0 (22 bytes: fp16 scale, 32 high bits, 16 nibble bytes; element i < 16 = low nibble of byte i, element
// i + 16 = high nibble of byte i) into Q8_0 tiles: q = (nibble | bit << 4) - 16 is stored as the 8-bit integer
// the Q8_0 kernels expect (nibbles of q ^ 0x80), with the block's own fp16 scale.
__global__ void repack_q5_0_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ tiles, int64_t rows,
                                   int64_t nblk, int64_t kt) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * nblk * 4) return;
    int q = idx & 3;
    int64_t bk = (idx >> 2) % nblk, r = (idx >> 2) / nblk;
    const uint8_t* src = raw + (r * nblk + bk) * 22;
    uint8_t* tile = tiles + ((r >> 4) * kt + (bk >> 2)) * Tile<WF_QTYPE_Q8_0>::BYTES;
    int ri = r & 15, j = bk & 3;
    const uint32_t qh = (uint32_t)src[2] | ((uint32_t)src[3] << 8) | ((uint32_t)src[4] << 16) | ((uint32_t)src[5] << 24);
    uint32_t hi[8], lo[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = 8 * q + i;
        const uint8_t byte = src[6 + (e & 15)];
        const int nib = e < 16 ? (byte & 0xF) : (byte >> 4);
        const int v = (nib | (int)(((qh >> e) & 1u) << 4)) - 16;
        const uint8_t u = (uint8_t)v ^ 0x80;
        hi[i] = u >> 4;
        lo[i] = u & 0xF;
    }
    int off = plane_word_off(ri, j, q);
    *reinterpret_cast<uint32_t*>(tile + off) = pack8(hi);
    *reinterpret_cast<uint32_t*>(tile + PLANE_BYTES + off) = pack8(lo);
    if (q == 0)
        *reinterpret_cast<uint16_t*>(tile + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + (ri & 7) * 16 + (ri >> 3) * 8 + j * 2) =
            ld_u16(src);
}

__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, int j, uint32_t& sc, uint32_t& m) {
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// One thread per (row, super-block, sub-block jj, element group q).
__global__ void repack_q4_k_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ tiles, int64_t rows,
                                   int64_t nsb) {
    using T = Tile<WF_QTYPE_Q4_K>;
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * nsb * 32) return;
    int q = idx & 3, jj = (idx >> 2) & 7;
    int64_t sb = (idx >> 5) % nsb, r = (idx >> 5) / nsb;
    const uint8_t* src = raw + (r * nsb + sb) * 144;
    uint8_t* tile = tiles + ((r >> 4) * nsb + sb) * T::BYTES;
    int ri = r & 15;
    const uint8_t* qs = src + 16 + 32 * (jj >> 1);  // 32 bytes shared by sub-blocks 2c (low) and 2c+1 (high)
    uint32_t nib[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        uint8_t b = qs[8 * q + i];
        nib[i] = (jj & 1) ? (b >> 4) : (b & 0xF);
    }
    *reinterpret_cast<uint32_t*>(tile + (jj >> 2) * PLANE_BYTES + plane_word_off(ri, jj & 3, q)) = pack8(nib);
    if (q == 0) {
        uint32_t sc, m;
        q4k_scale_min(src + 4, jj, sc, m);
        int so = (ri & 7) * 16 + (ri >> 3) * 8 + jj;
        tile[T::SC_OFF + so] = (uint8_t)sc;
        tile[T::MN_OFF + so] = (uint8_t)m;
        if (jj == 0) {
            uint16_t* dd = reinterpret_cast<uint16_t*>(tile + T::D_OFF + (ri & 7) * 8 + (ri >> 3) * 4);
            dd[0] = ld_u16(src);
            dd[1] = ld_u16(src + 2);
        }
    }
}

cudaError_t launch_repack(int qtype, const uint8_t* d_raw, uint8_t* d_tiles, int64_t rows, int64_t k,
                          int q4_0_order, cudaStream_t s) {
    const int threads = 256;
    if (qtype == WF_QTYPE_Q4_K) {
        int64_t nsb = k / 256, n = rows * nsb * 32;
        repack_q4_k_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, s>>>(d_raw, d_tiles, rows, nsb);
    } else {
        int64_t nblk = k / 32, n = rows * nblk * 4, kt = (k + 127) / 128;
        unsigned grid = (unsigned)((n + threads - 1) / threads);
        if (qtype == WF_QTYPE_Q4_0)
            repack_q4_0_kernel<<<grid, threads, 0, s>>>(d_raw, d_tiles, rows, nblk, kt, q4_0_order == WF_Q4_0_ORDER_GGML);
        else if (qtype == WF_QTYPE_Q4_1)
            repack_q4_1_kernel<<<grid, threads, 0, s>>>(d_raw, d_tiles, rows, nblk, kt, q4_0_order == WF_Q4_0_ORDER_GGML);
        else if (qtype == WF_QTYPE_Q5_0)
            repack_q5_0_kernel<<<grid, threads, 0, s>>>(d_raw, d_tiles, rows, nblk, kt);
        else
            repack_q8_0_kernel<<<grid, threads, 0, s>>>(d_raw, d_tiles, rows, nblk, kt);
    }
    return cudaGetLastError();
}

// fp16 -> fp32 with the CPU's NaN rule: every NaN becomes the canonical quiet NaN
// (Dequantizer.java:140 returns Float.NaN); all other inputs convert exactly.
__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
    float f = __half2float(__ushort_as_half(h));
    return (f != f) ? __uint_as_float(0x7FC00000u) : f;
}

__device__ __forceinline__ uint32_t tile_nibble(const uint8_t* plane, int ri, int j, int e) {
    uint32_t w = *reinterpret_cast<const uint32_t*>(plane + plane_word_off(ri, j, e >> 3));
    w = (w >> PLANE_ROT) | (w << (32 - PLANE_ROT));
    return (w >> (4 * nibble_pos(e & 7))) & 0xF;
}

// fp32 multiply / subtract with the NaN results an x86 host produces (the CPU path runs on
// SSE): a NaN operand is returned as is (first operand first), an invalid operation
// (0 * Inf, Inf - Inf) yields the negative default NaN.  All finite results are plain IEEE.
__device__ __forceinline__ float mul_host(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    float r = __fmul_rn(a, b);
    return (r != r) ? __uint_as_float(0xFFC00000u) : r;
}
__device__ __forceinline__ float sub_host(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    float r = __fsub_rn(a, b);
    return (r != r) ? __uint_as_float(0xFFC00000u) : r;
}

__device__ __forceinline__ float add_host(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    float r = __fadd_rn(a, b);
    return (r != r) ? __uint_as_float(0xFFC00000u) : r;
}

// One thread per output element; multiply and subtract rounded separately, never fused.
__global__ void dequant_rows_kernel(const uint8_t* __restrict__ tiles, int qtype, int64_t kt, int64_t k,
                                    int64_t row0, int64_t nrows, float* __restrict__ out) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nrows * k) return;
    int64_t r = row0 + idx / k, kk = idx % k;
    int ri = r & 15;
    float v;
    if (qtype == WF_QTYPE_Q4_K) {
        using T = Tile<WF_QTYPE_Q4_K>;
        const uint8_t* tile = tiles + ((r >> 4) * kt + (kk >> 8)) * T::BYTES;
        int jj = (kk >> 5) & 7, e = kk & 31;
        uint32_t qv = tile_nibble(tile + (jj >> 2) * PLANE_BYTES, ri, jj & 3, e);
        const uint16_t* dd = reinterpret_cast<const uint16_t*>(tile + T::D_OFF + (ri & 7) * 8 + (ri >> 3) * 4);
        int so = (ri & 7) * 16 + (ri >> 3) * 8 + jj;
        float d1 = mul_host(half_bits_to_float(dd[0]), (float)tile[T::SC_OFF + so]);
        float m1 = mul_host(half_bits_to_float(dd[1]), (float)tile[T::MN_OFF + so]);
        v = sub_host(mul_host(d1, (float)qv), m1);
    } else {
        int tb = tile_bytes(qtype);
        const uint8_t* tile = tiles + ((r >> 4) * kt + (kk >> 7)) * tb;
        int j = (kk >> 5) & 3, e = kk & 31;
        int so = (ri & 7) * 16 + (ri >> 3) * 8 + j * 2;
        int qv;
        float scale;
        if (qtype == WF_QTYPE_Q4_1) {  // q * scale + min, product and sum rounded separately
            using T = Tile<WF_QTYPE_Q4_1>;
            scale = half_bits_to_float(*reinterpret_cast<const uint16_t*>(tile + T::SCALE_OFF + so));
            const float mn = half_bits_to_float(*reinterpret_cast<const uint16_t*>(tile + T::MIN_OFF + so));
            out[idx] = add_host(mul_host((float)tile_nibble(tile, ri, j, e), scale), mn);
            return;
        }
        if (qtype == WF_QTYPE_Q4_0) {
            qv = (int)tile_nibble(tile, ri, j, e) - 8;
            scale = half_bits_to_float(*reinterpret_cast<const uint16_t*>(tile + Tile<WF_QTYPE_Q4_0>::SCALE_OFF + so));
        } else {
            int hi = (int)tile_nibble(tile, ri, j, e), lo = (int)tile_nibble(tile + PLANE_BYTES, ri, j, e);
            qv = 16 * (hi - 8) + lo;
            scale = half_bits_to_float(*reinterpret_cast<const uint16_t*>(tile + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + so));
        }
        v = mul_host((float)qv, scale);
    }
    out[idx] = v;
}

cudaError_t launch_dequant_rows(const Weight& w, int64_t row0, int64_t nrows, float* d_out, cudaStream_t s) {
    int64_t n = nrows * w.g.k;
    if (n == 0) return cudaSuccess;
    const int threads = 256;
    dequant_rows_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, s>>>(w.d_tiles, w.g.qtype, w.g.kt,
                                                                                    w.g.k, row0, nrows, d_out);
    return cudaGetLastError();
}

}  // namespace wf
