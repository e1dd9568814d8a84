// Decode GEMV: y[m, rows] = x[m, K] . W[rows, K]^T for m <= 8 tokens per pass, W in the tiled
// quantized layout of wf_layout.cuh.  HBM-bound: every weight byte is read exactly once.
// A producer thread streams the CTA's contiguous share of the weight into a shared-memory
// ring with bulk asynchronous copies (cp.async.bulk + mbarrier), as far ahead as the ring
// is deep -- for the decode shapes the whole share is in flight from the first cycle --
// and sixteen consumer warps pick their tile out of each ring stage with 16-byte
// shared-memory loads.  The 4-bit codes are turned into exact small integers in bf16 with
// one rotate and one logic op per pair and contracted on the tensor cores (mma.m16n8k16,
// fp32 accumulate); block scales are applied to the fp32 block sums in registers.
//
// Codes enter the MMA with a constant offset (16 + code); the offset is cancelled by
// starting each block's accumulator at beta * (sum of the block's activations), which is
// precomputed once per launch in shared memory.  No per-weight subtraction is executed.
//
// Work split ("stream-K"): the R*KT tiles of the weight form one stream in memory order.
// A persistent grid of one CTA per SM cuts the stream into equal contiguous chunks, so
// every SM reads the same number of bytes whatever the matrix shape.  Inside a CTA the
// warps take tiles round-robin, so the CTA as a whole reads memory sequentially.  A chunk
// is a sequence of segments, one per row-tile it touches; when a warp leaves a segment it
// parks its partial sums in shared memory and bumps an arrival counter, and the last warp
// to arrive adds the sixteen partials in warp order (deterministic) -- nobody waits at a
// barrier.  A row-tile cut by a chunk boundary is finished by the CTA that holds its
// beginning: the following CTAs compute their piece first and publish it to a scratch
// slot tagged valid; the owner, which reaches that row-tile last, adds the pieces in CTA
// order, clears the tags and writes y.  The owner's wait is bounded; on expiry it sets a
// status bit instead of spinning on.
//
// Replaces the fp32 batch_matmul_f32 launch of
// warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/ops/DotGeneralKernel.java:263-281
// (PTX at .../nvidia/cuda/CudaKernels.java:4423-4585) for quantized right-hand sides.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdlib.h>

#include <algorithm>

#include "wf_common.cuh"

namespace wf {

constexpr int GEMV_WARPS = 16;                       // consumer warps
constexpr int GEMV_THREADS = (GEMV_WARPS + 1) * 32;  // + one producer warp
constexpr int GEMV_MAX_STAGES = 16;
constexpr int GEMV_BAR_SPINS = 1 << 24;
constexpr int GEMV_XCOLS = 8;  // columns of one mma n-tile
constexpr int GEMV_FIXUP_SPINS = 1 << 22;
constexpr int GEMV_SLOT_SPINS = 1 << 24;
constexpr int GEMV_CTRL_BYTES = 128 + 2 * GEMV_MAX_STAGES * 8;  // arrive[], released[], abort, full[], empty[]

struct GemvParams {
    const uint8_t* tiles;
    const void* x;
    float* y;
    uint2* scratch;
    int* status;
    int64_t ldy, col0;
    int64_t ldx;  // elements between consecutive tokens of x
    int rows, k, kt, rt;
    int m;        // tokens this pass (<= 8 for bf16, <= 2 for fp32)
    int x_f32;    // 1: x is fp32 and each token is split into 3 exact bf16 columns
    int sx;       // shared-memory row stride of staged x, in bytes
    int stages;   // ring depth, each stage holds GEMV_WARPS tiles
    int chunk_q, chunk_r;  // CTA b owns tiles [b*q + min(b,r), (b+1)*q + min(b+1,r))
    unsigned long long* timing;  // optional [ctas][8] globaltimer stamps (instrumented launches only)
};

// ---------------------------------------------------------------- small device helpers
__device__ __forceinline__ uint4 ldg_stream(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint2 ldg_stream2(const void* p) { return *reinterpret_cast<const uint2*>(p); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// arrive from the lanes whose `pred` is non-zero, without a branch
__device__ __forceinline__ void mbar_arrive_if(void* bar, uint32_t pred) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %1, 0;\n\t@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" ::"r"(smem_u32(bar)),
        "r"(pred)
        : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: false if the phase did not complete within the spin budget.
__device__ __forceinline__ bool mbar_wait(void* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .u32 n;\n\t"
        "mov.u32 n, 0;\n\t"
        "WF_WAIT_%=:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra WF_DONE_%=;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 q, n, %3;\n\t"
        "@q bra WF_WAIT_%=;\n\t"
        "WF_DONE_%=:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)GEMV_BAR_SPINS)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, void* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// A scratch slot element is {value bits, valid tag}.  It is written and read as ONE 64-bit
// access so that a reader can never see the tag of one write with the value of another.
__device__ __forceinline__ void st_slot(uint2* p, uint2 v) {
    const unsigned long long w = ((unsigned long long)v.y << 32) | v.x;
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_slot(const uint2* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}
// d = a * b + c, d and c separate so that c can come straight from another register set
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}
__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t h2) {
    return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

// Codes enter the MMA as bf16 `base + scale * code`: magic 0x4180 -> 16 + code,
// magic 0x4380 -> 256 + 16 * code (nibble in the top four mantissa bits).  Exact.
constexpr uint32_t MAGIC_16 = 0x41804180u;   // 16 + code
constexpr uint32_t MAGIC_256 = 0x43804380u;  // 256 + 16 * code

// d = c + sum over one 32-k block of (base + scale * code) * x, rows g / g+8 of the fragment.
// One asm block: three rotates and eight logic ops unpack the two words, two MMAs consume
// them.  The temporaries live inside the block so the register allocator is free to build
// the MMA operand tuples in place.
__device__ __forceinline__ void block_mma(float (&d)[4], uint32_t wg, uint32_t wh, const uint4& xb, uint32_t magic,
                                          float c0, float c1, float c2, float c3) {
    asm(
        "{\n\t"
        ".reg .b32 g1, g2, g3, h1, h2, h3, a0, a1, a2, a3, a4, a5, a6, a7;\n\t"
        "shf.r.wrap.b32 g1, %4, %4, 4;\n\t"
        "shf.r.wrap.b32 h1, %5, %5, 4;\n\t"
        "shf.r.wrap.b32 g2, %4, %4, 8;\n\t"
        "shf.r.wrap.b32 h2, %5, %5, 8;\n\t"
        "shf.r.wrap.b32 g3, %4, %4, 12;\n\t"
        "shf.r.wrap.b32 h3, %5, %5, 12;\n\t"
        "lop3.b32 a0, %4, %14, %15, 0xEA;\n\t"
        "lop3.b32 a1, %5, %14, %15, 0xEA;\n\t"
        "lop3.b32 a2, g1, %14, %15, 0xEA;\n\t"
        "lop3.b32 a3, h1, %14, %15, 0xEA;\n\t"
        "lop3.b32 a4, g2, %14, %15, 0xEA;\n\t"
        "lop3.b32 a5, h2, %14, %15, 0xEA;\n\t"
        "lop3.b32 a6, g3, %14, %15, 0xEA;\n\t"
        "lop3.b32 a7, h3, %14, %15, 0xEA;\n\t"
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {a0,a1,a2,a3}, {%6,%7}, {%10,%11,%12,%13};\n\t"
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {a4,a5,a6,a7}, {%8,%9}, {%0,%1,%2,%3};\n\t"
        "}\n"
        : "=&f"(d[0]), "=&f"(d[1]), "=&f"(d[2]), "=&f"(d[3])
        : "r"(wg), "r"(wh), "r"(xb.x), "r"(xb.y), "r"(xb.z), "r"(xb.w), "f"(c0), "f"(c1), "f"(c2), "f"(c3),
          "r"(0x00780078u), "r"(magic));
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}

// ---------------------------------------------------------------- per-format tile code
// BETA: factor on "sum of the block's activations" that cancels the offsets the codes carry
// into the MMA.
template <int QT> struct TileRegs;

template <> struct TileRegs<WF_QTYPE_Q4_0> {
    static constexpr float BETA = -24.f;  // (16 + code) - 24 = code - 8
    uint4 c[2], s;
    __device__ __forceinline__ void load(const uint8_t* t, int lane) {
        c[0] = ldg_stream(t + lane * 16);
        c[1] = ldg_stream(t + 512 + lane * 16);
        s = ldg_stream(t + Tile<WF_QTYPE_Q4_0>::SCALE_OFF + (lane >> 2) * 16);
    }
    template <int XC>
    __device__ __forceinline__ void compute(float (&acc)[4], const uint8_t* xrow, const float4* cinit, int kbase,
                                            int q) const {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint4 xb = *reinterpret_cast<const uint4*>(xrow + (size_t)(kbase + j * 32 + q * 8) * 2);
            const float4 ci = cinit[((kbase >> 5) + j) * 4 + q];
            float d[4];
            block_mma(d, word_of(c[0], j), word_of(c[1], j), xb, MAGIC_16, ci.x, ci.y, ci.z, ci.w);
            const float2 dg = half2_bits_to_float2(j < 2 ? s.x : s.y), dh = half2_bits_to_float2(j < 2 ? s.z : s.w);
            const float sg = (j & 1) ? dg.y : dg.x, sh = (j & 1) ? dh.y : dh.x;
            acc[0] = fmaf(sg, d[0], acc[0]);
            acc[2] = fmaf(sh, d[2], acc[2]);
            if (XC > 1) {
                acc[1] = fmaf(sg, d[1], acc[1]);
                acc[3] = fmaf(sh, d[3], acc[3]);
            }
        }
    }
};

template <> struct TileRegs<WF_QTYPE_Q8_0> {
    static constexpr float BETA = -400.f;  // (256 + 16 hi) + (16 + lo) - 400 = 16 (hi - 8) + lo
    uint4 c[4], s;                         // c[0..1] high plane rows g / g+8, c[2..3] low plane
    __device__ __forceinline__ void load(const uint8_t* t, int lane) {
#pragma unroll
        for (int i = 0; i < 4; i++) c[i] = ldg_stream(t + i * 512 + lane * 16);
        s = ldg_stream(t + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + (lane >> 2) * 16);
    }
    template <int XC>
    __device__ __forceinline__ void compute(float (&acc)[4], const uint8_t* xrow, const float4* cinit, int kbase,
                                            int q) const {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint4 xb = *reinterpret_cast<const uint4*>(xrow + (size_t)(kbase + j * 32 + q * 8) * 2);
            const float4 ci = cinit[((kbase >> 5) + j) * 4 + q];
            float d[4];
            block_mma(d, word_of(c[0], j), word_of(c[1], j), xb, MAGIC_256, ci.x, ci.y, ci.z, ci.w);
            block_mma(d, word_of(c[2], j), word_of(c[3], j), xb, MAGIC_16, d[0], d[1], d[2], d[3]);
            const float2 dg = half2_bits_to_float2(j < 2 ? s.x : s.y), dh = half2_bits_to_float2(j < 2 ? s.z : s.w);
            const float sg = (j & 1) ? dg.y : dg.x, sh = (j & 1) ? dh.y : dh.x;
            acc[0] = fmaf(sg, d[0], acc[0]);
            acc[2] = fmaf(sh, d[2], acc[2]);
            if (XC > 1) {
                acc[1] = fmaf(sg, d[1], acc[1]);
                acc[3] = fmaf(sh, d[3], acc[3]);
            }
        }
    }
};

// byte `i` of w times d, exactly: (2^23 + byte) * d - 2^23 * d
__device__ __forceinline__ float byte_times(uint32_t w, int i, float d, float neg_big_d) {
    const float f = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u + i));
    return fmaf(f, d, neg_big_d);
}

template <> struct TileRegs<WF_QTYPE_Q4_K> {
    static constexpr float BETA = -16.f;  // (16 + code) - 16 = code
    uint4 c[4], sc, mn;                   // c[0..1] sub-blocks 0..3 rows g / g+8, c[2..3] sub-blocks 4..7
    uint2 dd;                             // (d, dmin) of row g, of row g+8
    __device__ __forceinline__ void load(const uint8_t* t, int lane) {
        using T = Tile<WF_QTYPE_Q4_K>;
#pragma unroll
        for (int i = 0; i < 4; i++) c[i] = ldg_stream(t + i * 512 + lane * 16);
        dd = ldg_stream2(t + T::D_OFF + (lane >> 2) * 8);
        sc = ldg_stream(t + T::SC_OFF + (lane >> 2) * 16);
        mn = ldg_stream(t + T::MN_OFF + (lane >> 2) * 16);
    }
    template <int XC>
    __device__ __forceinline__ void compute(float (&acc)[4], const uint8_t* xrow, const float4* cinit, int kbase,
                                            int q) const {
        const float2 g = half2_bits_to_float2(dd.x), h = half2_bits_to_float2(dd.y);  // (d, dmin)
        const float BIG = 8388608.f;
        // the min term -dmin*m*X comes from cinit = -16*X as (dmin/16) * m * cinit
        const float gm = g.y * 0.0625f, hm = h.y * 0.0625f;
        const float ngd = -BIG * g.x, ngm = -BIG * gm, nhd = -BIG * h.x, nhm = -BIG * hm;
#pragma unroll
        for (int jj = 0; jj < 8; jj++) {
            const uint4 xb = *reinterpret_cast<const uint4*>(xrow + (size_t)(kbase + jj * 32 + q * 8) * 2);
            const float4 ci = cinit[((kbase >> 5) + jj) * 4 + q];
            float d[4];
            block_mma(d, word_of(c[(jj >> 2) * 2], jj & 3), word_of(c[(jj >> 2) * 2 + 1], jj & 3), xb, MAGIC_16, ci.x,
                      ci.y, ci.z, ci.w);
            const float ag = byte_times(jj < 4 ? sc.x : sc.y, jj & 3, g.x, ngd);  // d * sc, exact
            const float ah = byte_times(jj < 4 ? sc.z : sc.w, jj & 3, h.x, nhd);
            const float cg = byte_times(jj < 4 ? mn.x : mn.y, jj & 3, gm, ngm);  // dmin * m / 16, exact
            const float ch = byte_times(jj < 4 ? mn.z : mn.w, jj & 3, hm, nhm);
            acc[0] = fmaf(ag, d[0], fmaf(cg, ci.x, acc[0]));
            acc[2] = fmaf(ah, d[2], fmaf(ch, ci.z, acc[2]));
            if (XC > 1) {
                acc[1] = fmaf(ag, d[1], fmaf(cg, ci.y, acc[1]));
                acc[3] = fmaf(ah, d[3], fmaf(ch, ci.w, acc[3]));
            }
        }
    }
};

// ---------------------------------------------------------------- x staging
// Copies x into shared memory as bf16 rows of `kp` elements (zero beyond k), row stride sx
// bytes.  bf16 input: row = token.  fp32 input: token t becomes rows 3t, 3t+1, 3t+2 holding
// an exact three-way bf16 split (x = hi + mid + lo), so fp32 activations lose nothing.
// Also fills cinit[kp/32][4]: for block b and column pair q the float4
// {beta*X(b,2q), beta*X(b,2q+1), same, same}, X = fp32 sum of the block's 32 activations.
__device__ __forceinline__ uint32_t pack_bf16_trunc(float a, float b) {
    return (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xFFFF0000u);
}

__device__ void stage_x(const GemvParams& p, uint8_t* xs, float* cinit, int kp, float beta) {
    const int groups = kp >> 3;  // 8 elements per thread step
    const int total = p.m * groups;
    for (int idx = threadIdx.x; idx < ((total + 31) & ~31); idx += GEMV_THREADS) {  // warp-uniform trip count
        const bool live = idx < total;
        const int t = (live && p.m > 1) ? idx / groups : 0, c8 = live ? idx - t * groups : 0;
        const bool in_k = live && (c8 * 8 < p.k);
        float sum[3] = {0.f, 0.f, 0.f};
        if (!p.x_f32) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (in_k) v = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + (size_t)t * p.ldx + c8 * 8);
            if (live) *reinterpret_cast<uint4*>(xs + (size_t)t * p.sx + c8 * 16) = v;
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                sum[0] += __uint_as_float(w[i] << 16);
                sum[0] += __uint_as_float(w[i] & 0xFFFF0000u);
            }
        } else {
            float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (in_k) {
                const float4* src =
                    reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + (size_t)t * p.ldx + c8 * 8);
                const float4 a = src[0], b = src[1];
                f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
            }
            uint32_t hi[4], mid[4], lo[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float x0 = f[2 * i], x1 = f[2 * i + 1];
                const float h0 = __uint_as_float(__float_as_uint(x0) & 0xFFFF0000u);
                const float h1 = __uint_as_float(__float_as_uint(x1) & 0xFFFF0000u);
                const float r0 = x0 - h0, r1 = x1 - h1;
                const float m0 = __uint_as_float(__float_as_uint(r0) & 0xFFFF0000u);
                const float m1 = __uint_as_float(__float_as_uint(r1) & 0xFFFF0000u);
                const float l0 = r0 - m0, l1 = r1 - m1;  // at most 8 significant bits left: exact in bf16
                hi[i] = pack_bf16_trunc(h0, h1);
                mid[i] = pack_bf16_trunc(m0, m1);
                lo[i] = pack_bf16_trunc(l0, l1);
                sum[0] += h0 + h1;
                sum[1] += m0 + m1;
                sum[2] += l0 + l1;
            }
            if (live) {
                *reinterpret_cast<uint4*>(xs + (size_t)(3 * t) * p.sx + c8 * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(xs + (size_t)(3 * t + 1) * p.sx + c8 * 16) = make_uint4(mid[0], mid[1], mid[2], mid[3]);
                *reinterpret_cast<uint4*>(xs + (size_t)(3 * t + 2) * p.sx + c8 * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
        // 4 consecutive threads hold one 32-element block (groups is a multiple of 4)
#pragma unroll
        for (int s = 0; s < 3; s++) {
            sum[s] += __shfl_xor_sync(0xFFFFFFFFu, sum[s], 1);
            sum[s] += __shfl_xor_sync(0xFFFFFFFFu, sum[s], 2);
        }
        if (live && (threadIdx.x & 3) == 0) {
            float* blk = cinit + (size_t)(c8 >> 2) * 16;  // [q][4]
            const int parts = p.x_f32 ? 3 : 1;
            for (int s = 0; s < parts; s++) {
                const int col = p.x_f32 ? 3 * t + s : t;
                const float v = beta * sum[s];
                blk[(col >> 1) * 4 + (col & 1)] = v;
                blk[(col >> 1) * 4 + (col & 1) + 2] = v;
            }
        }
    }
}

// ---------------------------------------------------------------- the kernel
// XC = 1: exactly one live column (one bf16 token); XC = 8: up to 8 columns.
template <int XC> struct Slots { static constexpr int N = (XC == 1) ? 4 : 2, ELEMS = 16 * XC; };

// Shared-memory map (bytes): [0,32) arrive[8] | [32,64) released[8] | [64,68) abort flag |
// [128, 128+8*MAX_STAGES) full barriers | then empty barriers | partial sums | exchange row |
// cinit | staged x | ring stages (128-byte aligned).
template <int QT, int XC>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvParams p) {
    using T = Tile<QT>;
    using R = TileRegs<QT>;
    constexpr int NSLOT = Slots<XC>::N, ELEMS = Slots<XC>::ELEMS;
    constexpr uint32_t STAGE_BYTES = GEMV_WARPS * T::BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    int* arrive = reinterpret_cast<int*>(smem);                              // [NSLOT]
    volatile int* released = reinterpret_cast<volatile int*>(smem) + 8;      // [NSLOT]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem) + 16;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + 128);                // [stages]
    uint64_t* empty = full + GEMV_MAX_STAGES;                                // [stages]
    float* partial = reinterpret_cast<float*>(smem + GEMV_CTRL_BYTES);       // [NSLOT][GEMV_WARPS][ELEMS]
    float* exchange = partial + NSLOT * GEMV_WARPS * ELEMS;                  // [128]
    const int kp = p.kt * T::K;
    float4* cinit = reinterpret_cast<float4*>(exchange + 128);               // [kp/32][4]
    uint8_t* xs = reinterpret_cast<uint8_t*>(cinit + (kp >> 5) * 4);         // [xcols][sx]
    const int xcols = p.x_f32 ? 3 * p.m : p.m;
    uint8_t* ring = smem + (((size_t)(xs - smem) + (size_t)xcols * p.sx + 127) & ~(size_t)127);

    // warp-uniform values, obtained in a way the compiler can see is uniform
    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    const int bx = blockIdx.x;
    const int t0 = bx * p.chunk_q + min(bx, p.chunk_r);
    const int t1 = t0 + p.chunk_q + (bx < p.chunk_r ? 1 : 0);
    const int rounds = (t1 - t0 + GEMV_WARPS - 1) / GEMV_WARPS;
    const int stages = p.stages;

    // Optional timing stamps, the counterpart of the reference's SALT_TIMING kernels
    // (nvidia/cuda/CudaKernels.java:31-37): warp 0 lane 0 records globaltimer at fixed points.
    auto stamp = [&](int i) {
        if (p.timing != nullptr && threadIdx.x == 0) {
            unsigned long long tm;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm));
            p.timing[(size_t)blockIdx.x * 8 + i] = tm;
        }
    };
    stamp(0);
    if (threadIdx.x == 0) {
        for (int i = 0; i < 32; i++) reinterpret_cast<int*>(smem)[i] = 0;
        for (int s = 0; s < stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GEMV_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Producer: fill every stage right away; the weights do not depend on anything.
    auto issue_round = [&](int r) {
        const int s = r % stages;
        const int first = t0 + r * GEMV_WARPS;
        const uint32_t bytes = (uint32_t)min(GEMV_WARPS, t1 - first) * T::BYTES;
        mbar_expect_tx(&full[s], bytes);
        bulk_load(ring + (size_t)s * STAGE_BYTES, p.tiles + (size_t)first * T::BYTES, bytes, &full[s]);
    };
    if (warp == GEMV_WARPS && lane == 0)
        for (int r = 0; r < min(rounds, stages); r++) issue_round(r);

    // cinit entries of dead columns stay uninitialised: they only feed dead columns
    stage_x(p, xs, reinterpret_cast<float*>(cinit), kp, R::BETA);
    __syncthreads();
    stamp(1);

    if (warp == GEMV_WARPS) {  // producer warp: refill stages as the consumers release them
        if (lane == 0) {
            for (int r = stages; r < rounds; r++) {
                if (!mbar_wait(&empty[r % stages], ((r / stages) - 1) & 1) || *abort_flag) {
                    atomicOr(p.status, STATUS_GEMV_FIXUP_TIMEOUT);
                    *abort_flag = 1;
                    break;
                }
                issue_round(r);
            }
        }
        return;
    }

    // dead columns read the last live row: their results are computed and never stored
    const uint8_t* xrow = xs + (size_t)(g < xcols ? g : xcols - 1) * p.sx;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    int seg = 0, seg_begin = t0;
    int rt = (t0 < t1) ? t0 / p.kt : 0;
    int seg_end = min((rt + 1) * p.kt, t1);

    auto finish_segment = [&](int slot) {  // run by the last warp to arrive, all 32 lanes
        constexpr int PER_LANE = (ELEMS + 31) / 32;
        float v[PER_LANE];
#pragma unroll
        for (int u = 0; u < PER_LANE; u++) {
            const int i = lane + 32 * u;
            v[u] = 0.f;
            if (i < ELEMS) {
                const float* src = partial + (size_t)slot * GEMV_WARPS * ELEMS + i;
#pragma unroll
                for (int w = 0; w < GEMV_WARPS; w++) v[u] += src[w * ELEMS];
            }
        }
        const bool starts = seg_begin == rt * p.kt, ends = seg_end == (rt + 1) * p.kt;
        if (!starts) {  // a piece of a row-tile owned by an earlier CTA: publish it
#pragma unroll
            for (int u = 0; u < PER_LANE; u++) {
                const int i = lane + 32 * u;
                if (i < ELEMS)
                    st_slot(p.scratch + (size_t)blockIdx.x * 128 + i, make_uint2(__float_as_uint(v[u]), 1u));
            }
            return;
        }
        if (!ends) {  // owner of a row-tile that continues in the following CTAs
            const int te = (rt + 1) * p.kt;
            bool gave_up = false;
            for (int c = (int)blockIdx.x + 1; c < (int)gridDim.x && !gave_up; c++) {
                const int c0 = c * p.chunk_q + min(c, p.chunk_r), c1 = c0 + p.chunk_q + (c < p.chunk_r ? 1 : 0);
                if (c0 >= te) break;
                if (c0 == c1) continue;
#pragma unroll
                for (int u = 0; u < PER_LANE; u++) {
                    const int i = lane + 32 * u;
                    if (i >= ELEMS) continue;
                    uint2* slot_ptr = p.scratch + (size_t)c * 128 + i;
                    uint2 e;
                    int spins = 0;
                    do {
                        e = ld_slot(slot_ptr);
                        if (e.y != 0u) break;
                        __nanosleep(32);
                    } while (++spins < GEMV_FIXUP_SPINS);
                    if (e.y == 0u) {
                        atomicOr(p.status, STATUS_GEMV_FIXUP_TIMEOUT);
                        gave_up = true;
                    } else {
                        v[u] += __uint_as_float(e.x);
                        st_slot(slot_ptr, make_uint2(0u, 0u));
                    }
                }
                gave_up = __any_sync(0xFFFFFFFFu, gave_up);
            }
        }
        // element i = col * 16 + row
        if (!p.x_f32) {
#pragma unroll
            for (int u = 0; u < PER_LANE; u++) {
                const int i = lane + 32 * u, col = i >> 4, n = rt * 16 + (i & 15);
                if (i < ELEMS && col < p.m && n < p.rows) p.y[(int64_t)col * p.ldy + p.col0 + n] = v[u];
            }
        } else {  // columns 3t, 3t+1, 3t+2 are the hi / mid / lo parts of token t
#pragma unroll
            for (int u = 0; u < PER_LANE; u++)
                if (lane + 32 * u < ELEMS) exchange[lane + 32 * u] = v[u];
            __syncwarp();
            for (int i = lane; i < 16 * p.m; i += 32) {
                const int tok = i >> 4, r = i & 15, n = rt * 16 + r;
                if (n < p.rows)
                    p.y[(int64_t)tok * p.ldy + p.col0 + n] =
                        (exchange[(3 * tok + 2) * 16 + r] + exchange[(3 * tok + 1) * 16 + r]) + exchange[(3 * tok) * 16 + r];
            }
            __syncwarp();
        }
    };

    auto flush = [&]() {
        const int slot = seg % NSLOT, gen = seg / NSLOT;
        if (gen > 0) {  // the slot's previous use must have been reduced already
            int spins = 0;
            while (released[slot] < gen && ++spins < GEMV_SLOT_SPINS) {
            }
            if (released[slot] < gen && lane == 0) atomicOr(p.status, STATUS_GEMV_FIXUP_TIMEOUT);
        }
        float* mine = partial + ((size_t)slot * GEMV_WARPS + warp) * ELEMS;
        if (XC == 1) {
            if (q == 0) {
                mine[g] = acc[0];
                mine[g + 8] = acc[2];
            }
        } else {
            mine[(2 * q) * 16 + g] = acc[0];
            mine[(2 * q + 1) * 16 + g] = acc[1];
            mine[(2 * q) * 16 + g + 8] = acc[2];
            mine[(2 * q + 1) * 16 + g + 8] = acc[3];
        }
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        __syncwarp();
        int old = 0;
        if (lane == 0) {
            __threadfence_block();
            old = atomicAdd(&arrive[slot], 1);
        }
        old = __shfl_sync(0xFFFFFFFFu, old, 0);
        if (old == GEMV_WARPS * (gen + 1) - 1) {
            __threadfence_block();
            finish_segment(slot);
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                released[slot] = gen + 1;
            }
        }
        seg++;
        seg_begin = seg_end;
        rt++;  // segments advance one row-tile at a time
        seg_end = min((rt + 1) * p.kt, t1);
    };

    // Segment by segment: an inner loop over this warp's tiles of the segment (one tile per
    // ring round, nothing but wait / load / release / compute in it), then the flush.
    // Stage index and phase are tracked incrementally.
    const int n_my = (t0 + warp < t1) ? (t1 - t0 - warp + GEMV_WARPS - 1) / GEMV_WARPS : 0;
    int s = 0, t = t0 + warp;
    uint32_t phase = 0;
    const uint8_t* my_tile = ring + (size_t)warp * T::BYTES;
    const uint32_t lane_is_0 = lane == 0;
    bool failed = false;
    stamp(2);
    while (seg_begin < t1) {
        // my tiles with index below seg_end
        const int n_seg = (t < seg_end) ? (seg_end - t + GEMV_WARPS - 1) / GEMV_WARPS : 0;
        int kbase = (t - rt * p.kt) * T::K;
        for (int i = 0; i < n_seg && !failed; i++) {
            if (!mbar_wait(&full[s], phase)) {
                failed = true;
                break;
            }
            R regs;
            regs.load(my_tile + (size_t)s * STAGE_BYTES, lane);
            __syncwarp();
            mbar_arrive_if(&empty[s], lane_is_0);
            regs.template compute<XC>(acc, xrow, cinit, kbase, q);
            kbase += GEMV_WARPS * T::K;
            t += GEMV_WARPS;
            if (++s == stages) {
                s = 0;
                phase ^= 1u;
            }
        }
        flush();
    }
    stamp(4);
    // Only the last round can lack a tile for some warps, and its stage is never refilled, so
    // those warps owe the producer no release.
    if (failed) {
        if (lane == 0) atomicOr(p.status, STATUS_GEMV_FIXUP_TIMEOUT);
        *abort_flag = 1;
    }
    stamp(5);
}

// ---------------------------------------------------------------- host side
template <int XC>
static size_t gemv_fixed_smem(int kp, int xcols, int* sx_out) {
    const int sx = kp * 2 + 64;  // +64: consecutive rows start 16 banks apart
    if (sx_out) *sx_out = sx;
    size_t b = GEMV_CTRL_BYTES + (size_t)Slots<XC>::N * GEMV_WARPS * Slots<XC>::ELEMS * 4 + 128 * 4 + (size_t)(kp / 32) * 64 +
               (size_t)xcols * sx;
    return (b + 127) & ~(size_t)127;
}

constexpr size_t GEMV_SMEM_LIMIT = 227 * 1024;

// Ring depth that fits beside the staged activations (0 = does not fit at all).
template <int XC>
static int gemv_stages(int qt, int kp, int xcols) {
    const size_t fixed = gemv_fixed_smem<XC>(kp, xcols, nullptr), stage = (size_t)GEMV_WARPS * tile_bytes(qt);
    if (fixed + stage > GEMV_SMEM_LIMIT) return 0;
    return (int)std::min<size_t>((GEMV_SMEM_LIMIT - fixed) / stage, GEMV_MAX_STAGES);
}

// Largest number of tokens one pass can take: bounded by the 8 mma columns (3 per fp32
// token) and by the shared memory the staged activations and a 2-deep ring need.
int gemv_max_tokens_per_pass(const Weight& w, int x_dtype) {
    const int kp = (int)w.g.kt * tile_k(w.g.qtype);
    const int per_tok = x_dtype == WF_DTYPE_F32 ? 3 : 1;
    int best = 0;
    for (int m = 1; m * per_tok <= GEMV_XCOLS; m++)
        if (gemv_stages<8>(w.g.qtype, kp, m * per_tok) >= 2) best = m;
    if (best == 0 && per_tok == 1 && gemv_stages<1>(w.g.qtype, kp, 1) >= 1) best = 1;
    return best;
}

template <int QT, int XC>
static cudaError_t launch_one(const GemvParams& p, int grid, size_t smem, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e =
            cudaFuncSetAttribute(gemv_kernel<QT, XC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMV_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    gemv_kernel<QT, XC><<<grid, GEMV_THREADS, smem, s>>>(p);
    return cudaGetLastError();
}

template <int XC>
static cudaError_t launch_qt(int qt, const GemvParams& p, int grid, size_t smem, cudaStream_t s) {
    return qt == WF_QTYPE_Q4_0   ? launch_one<WF_QTYPE_Q4_0, XC>(p, grid, smem, s)
           : qt == WF_QTYPE_Q8_0 ? launch_one<WF_QTYPE_Q8_0, XC>(p, grid, smem, s)
                                 : launch_one<WF_QTYPE_Q4_K, XC>(p, grid, smem, s);
}

// Allocates (once per stream) the scratch slots the CTAs exchange partial row-tiles through.
// Streams get their own slots so GEMVs on different streams may overlap.
int gemv_prepare_stream(Context* c, cudaStream_t s) {
    GemvScratch& sc = c->gemv_scratch[s];
    if (sc.ctas >= c->sm_count) return WF_OK;
    if (sc.d_slots) cudaFree(sc.d_slots);
    sc.d_slots = nullptr;
    sc.ctas = 0;
    WF_CUDA(c, cudaMalloc(&sc.d_slots, (size_t)c->sm_count * 128 * sizeof(uint2)));
    WF_CUDA(c, cudaMemset(sc.d_slots, 0, (size_t)c->sm_count * 128 * sizeof(uint2)));
    sc.ctas = c->sm_count;
    return WF_OK;
}

int gemv_launch(Context* c, const GemvCall& call, cudaStream_t s) {
    const Weight& w = *call.w;
    const int qt = w.g.qtype;
    const int kp = (int)w.g.kt * tile_k(qt);
    const int per_pass = gemv_max_tokens_per_pass(w, call.x_dtype);
    if (per_pass < 1)
        return set_error(c, WF_ERR_TOO_LARGE, "K=%lld needs more shared memory than one SM has", (long long)w.g.k);
    const int64_t total = w.g.rt * w.g.kt;
    if (total >= (1LL << 31)) return set_error(c, WF_ERR_TOO_LARGE, "weight has too many tiles");
    int grid = c->sm_count;
    if ((int64_t)grid > total) grid = (int)total;
    if (grid < 1) return WF_OK;

    int prc = gemv_prepare_stream(c, s);
    if (prc != WF_OK) return prc;
    GemvScratch& sc = c->gemv_scratch[s];

    const size_t esz = call.x_dtype == WF_DTYPE_F32 ? 4 : 2;
    int max_rounds = (int)((total / grid + 1 + GEMV_WARPS - 1) / GEMV_WARPS);
    if (const char* cap = getenv("WF_GEMV_MAX_STAGES")) max_rounds = std::max(1, std::min(max_rounds, atoi(cap)));
    for (int64_t m0 = 0; m0 < call.m; m0 += per_pass) {
        GemvParams p{};
        p.tiles = w.d_tiles;
        p.x = static_cast<const uint8_t*>(call.d_x) + (size_t)m0 * w.g.k * esz;
        p.y = call.d_y + m0 * call.ldy;
        p.scratch = sc.d_slots;
        p.status = c->d_status;
        p.timing = c->salt >= 2 ? c->d_timing : nullptr;
        p.ldy = call.ldy;
        p.col0 = call.col0;
        p.ldx = w.g.k;
        p.rows = (int)w.g.rows;
        p.k = (int)w.g.k;
        p.kt = (int)w.g.kt;
        p.rt = (int)w.g.rt;
        p.chunk_q = (int)(total / grid);
        p.chunk_r = (int)(total % grid);
        p.m = (int)((call.m - m0) < per_pass ? (call.m - m0) : per_pass);
        p.x_f32 = call.x_dtype == WF_DTYPE_F32;
        const int xcols = p.x_f32 ? 3 * p.m : p.m;
        const size_t stage = (size_t)GEMV_WARPS * tile_bytes(qt);
        cudaError_t e;
        if (xcols == 1) {
            p.stages = std::min(gemv_stages<1>(qt, kp, xcols), std::max(max_rounds, 1));
            e = launch_qt<1>(qt, p, grid, gemv_fixed_smem<1>(kp, xcols, &p.sx) + p.stages * stage, s);
        } else {
            p.stages = std::min(gemv_stages<8>(qt, kp, xcols), std::max(max_rounds, 1));
            e = launch_qt<8>(qt, p, grid, gemv_fixed_smem<8>(kp, xcols, &p.sx) + p.stages * stage, s);
        }
        if (e != cudaSuccess) return cuda_status(c, e, "gemv launch");
        c->launches++;
    }
    return WF_OK;
}

// ---------------------------------------------------------------- allocation-free variant
// Fix-up slots for wf_qlinear_noalloc live in this statically sized device array instead of
// memory obtained from cudaMalloc.  Every GPU that loads the library carries its 256 KiB
// until the process exits.  One array per device is shared by all calls on that device.
constexpr int GEMV_NOALLOC_MAX_CTAS = 256;  // the kernel launches one CTA per SM
static __device__ __align__(256) uint2 g_noalloc_slots[GEMV_NOALLOC_MAX_CTAS * 128];

// In host code `g_noalloc_slots` is only a handle for the symbol, not an address the GPU can
// use; the device address is looked up once per device, with that device current.
static std::mutex g_noalloc_mu;
static uint2* g_noalloc_ptr[64] = {};

static int noalloc_slots_for_current_device(Context* c, uint2** out) {
    if (c->device < 0 || c->device >= 64) return set_error(c, WF_ERR_TOO_LARGE, "device index %d beyond 63", c->device);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[c->device]) {
        uint2* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_slots);
        if (e != cudaSuccess) return cuda_status(c, e, "cudaGetSymbolAddress(g_noalloc_slots)");
        g_noalloc_ptr[c->device] = ptr;
    }
    *out = g_noalloc_ptr[c->device];
    return WF_OK;
}

// Same kernels and the same work split as gemv_launch, but nothing is allocated: the slots
// come from the static array above and are cleared on the stream before every launch,
// because the array keeps whatever the previous call (possibly a failed one) left in it.
int gemv_launch_noalloc(Context* c, const GemvCall& call, cudaStream_t s) {
    const Weight& w = *call.w;
    const int qt = w.g.qtype;
    const int kp = (int)w.g.kt * tile_k(qt);
    const int per_pass = gemv_max_tokens_per_pass(w, call.x_dtype);
    if (per_pass < 1)
        return set_error(c, WF_ERR_TOO_LARGE, "K=%lld needs more shared memory than one SM has", (long long)w.g.k);
    const int64_t total = w.g.rt * w.g.kt;
    if (total >= (1LL << 31)) return set_error(c, WF_ERR_TOO_LARGE, "weight has too many tiles");
    if (c->sm_count > GEMV_NOALLOC_MAX_CTAS)
        return set_error(c, WF_ERR_TOO_LARGE, "device has %d SMs; the static fix-up array covers at most %d", c->sm_count,
                         GEMV_NOALLOC_MAX_CTAS);
    int grid = c->sm_count;
    if ((int64_t)grid > total) grid = (int)total;
    if (grid < 1) return WF_OK;
    uint2* slots = nullptr;
    int rc = noalloc_slots_for_current_device(c, &slots);
    if (rc != WF_OK) return rc;

    const size_t esz = call.x_dtype == WF_DTYPE_F32 ? 4 : 2;
    const int max_rounds = (int)((total / grid + 1 + GEMV_WARPS - 1) / GEMV_WARPS);
    for (int64_t m0 = 0; m0 < call.m; m0 += per_pass) {
        GemvParams p{};
        p.tiles = w.d_tiles;
        p.x = static_cast<const uint8_t*>(call.d_x) + (size_t)m0 * w.g.k * esz;
        p.y = call.d_y + m0 * call.ldy;
        p.scratch = slots;
        p.status = c->d_status;
        p.timing = nullptr;
        p.ldy = call.ldy;
        p.col0 = call.col0;
        p.ldx = w.g.k;
        p.rows = (int)w.g.rows;
        p.k = (int)w.g.k;
        p.kt = (int)w.g.kt;
        p.rt = (int)w.g.rt;
        p.chunk_q = (int)(total / grid);
        p.chunk_r = (int)(total % grid);
        p.m = (int)((call.m - m0) < per_pass ? (call.m - m0) : per_pass);
        p.x_f32 = call.x_dtype == WF_DTYPE_F32;
        const int xcols = p.x_f32 ? 3 * p.m : p.m;
        const size_t stage = (size_t)GEMV_WARPS * tile_bytes(qt);
        WF_CUDA(c, cudaMemsetAsync(slots, 0, (size_t)grid * 128 * sizeof(uint2), s));
        cudaError_t e;
        if (xcols == 1) {
            p.stages = std::min(gemv_stages<1>(qt, kp, xcols), std::max(max_rounds, 1));
            e = launch_qt<1>(qt, p, grid, gemv_fixed_smem<1>(kp, xcols, &p.sx) + p.stages * stage, s);
        } else {
            p.stages = std::min(gemv_stages<8>(qt, kp, xcols), std::max(max_rounds, 1));
            e = launch_qt<8>(qt, p, grid, gemv_fixed_smem<8>(kp, xcols, &p.sx) + p.stages * stage, s);
        }
        if (e != cudaSuccess) return cuda_status(c, e, "gemv launch (no-alloc)");
        c->launches++;
    }
    return WF_OK;
}

}  // namespace wf
