// Prefill GEMM: y[m, rows] = x[m, K] . W[rows, K]^T for many tokens, W in the tiled quantized
// layout of wf_layout.cuh, on the 5th-generation tensor cores.
//
//   D[128 weight rows x BM tokens] (fp32, in TMEM) += A[128 x 16] (fp16, smem) * B[16 x BM] (fp16, smem)
//
// Activations arrive as bf16; a small pre-pass rewrites each token row as fp16 times a power of two
// (exact: fp16 has more mantissa bits than bf16, and the per-row scale keeps the row inside fp16's
// exponent range); the epilogue multiplies the row back.
//
// Warp roles in one persistent CTA per SM (448 threads):
//   warp 0      TMA producer: activation tiles [BM tokens x 64 k] with 128-byte swizzle, two per stage
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma, commits to mbarriers; owns TMEM
//   warps 4-7   epilogue (TMEM lane quarter = warp % 4): tcgen05.ld the accumulator, store fp32 rows
//               to y, release the accumulator
//   warps 2,3,8-13  dequant: read the quantized tiles straight from global memory (coalesced 16-byte
//               loads, the layout is already fragment-ordered), unpack 4-bit codes, apply the block
//               scale and write fp16 rows into the swizzled A stage; one 16-row tile per warp and stage
// Stages hold BK = 128 k: A = 128 rows x 128 k fp16 (two 64-k swizzle spans, 32 KB), B = BM x 128 k fp16.
// The accumulator is double buffered in TMEM (2 x BM columns <= 512) so the epilogue of one tile
// overlaps the main loop of the next.  A dequant warp converts its registers to fp16 BEFORE it waits
// for the stage to be released, so only the shared-memory stores lie between "stage released" and
// "stage full again".
//
// Above 512 tokens a token tile is two halves of 256 tokens (TMEM columns 0 and 256, one accumulator each)
// that share every dequantized weight stage, and a stage holds 64 k (A 16 KB, B 2 x 32 KB): the weight
// loads and conversions per MMA halve.  The two halves have their own full / empty barriers, so the
// epilogue drains the first half while the MMAs of the second still run.
//
// Work split ("stream-K"): all (tile, k-block) steps form one sequence in tile order, cut into
// equal contiguous shares, one per CTA, so every SM does the same number of MMA steps whatever the
// tile count.  A tile cut by a share boundary is finished by the CTA that holds its first
// k-block: the CTAs holding the rest reach their piece first (it is the head of their share),
// write it to a scratch buffer and publish the launch number; the owner reaches the tile last --
// it is the last thing in its share, so all its warps are free by then: twelve of them (three per
// TMEM lane quarter) add the pieces in CTA order (deterministic) and write y.  Every wait is bounded;
// on expiry the CTA sets a status bit, stops issuing work and still frees its TMEM.
//
// Weights are rounded once to fp16 (relative 2^-12) after the exact fp32 dequantization; products
// and sums are fp32 in the tensor core.  Replaces the host transpose + batch_matmul_f32 of
// warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/ops/DotGeneralKernel.java:169-298.
#include <cuda.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "wf_common.cuh"

namespace wf {

constexpr int GEMM_BN = 128;        // weight rows per tile (UMMA M)
constexpr int GEMM_BK = 128;        // k per stage
// Build-time choices, measured on one B200 against each other (config: Q4_K [14336 x 4096], 512 / 2048 tokens):
// 8 dequant warps 77.9 / 254.6 us, 16 dequant warps 84.0 / 278.3 us; token tiles of 2 x 256 above 512 tokens
// 254.6 us against 263.6 us without them at 2048 tokens ([8192 x 8192]: 278.4 against 311.4 us).
#ifndef WF_GEMM_DQ_WARPS
#define WF_GEMM_DQ_WARPS 8
#endif
#ifndef WF_GEMM_WIDE_MIN
#define WF_GEMM_WIDE_MIN 512  // token counts above this use the 2 x 256 token tiles
#endif
constexpr int GEMM_DEQUANT_WARPS = WF_GEMM_DQ_WARPS;  // 8: a 16-row weight tile each; 16: one row half (8 rows) each
constexpr int GEMM_DQ_HALVES = 16 / GEMM_DEQUANT_WARPS;   // row halves a dequant warp converts per step
constexpr int GEMM_THREADS = (6 + GEMM_DEQUANT_WARPS) * 32;  // TMA, MMA, 4 epilogue, dequant warps
constexpr int GEMM_WAIT_SPINS = 1 << 26;
constexpr int GEMM_A_BYTES = GEMM_BN * GEMM_BK * 2;  // 32 KB
constexpr int GEMM_WIDE_BK = 64;                     // k per stage when a token tile is 2 x 256 tokens
constexpr int GEMM_WIDE_A_BYTES = GEMM_BN * GEMM_WIDE_BK * 2;  // 16 KB
constexpr int GEMM_WIDE_B_HALF = 256 * GEMM_WIDE_BK * 2;       // 32 KB: 256 tokens x 64 k
constexpr int GEMM_PIECE_TOKENS = 512;               // tokens a stream-K piece can hold

struct GemmParams {
    const uint8_t* tiles;
    float* y;
    const float* row_unscale;  // [m] power of two that undoes the pre-pass scaling of token row m
    int* status;
    int64_t ldy, col0;
    int rows, k, kt_w;   // kt_w: weight k-tiles per row-tile stripe (tile_k of the format)
    int m;               // tokens
    int bm;              // tokens per MMA (UMMA N: multiple of 16, <= 256)
    int halves;          // 1: token tiles of bm, 128-k stages, accumulator double buffered;
                         // 2: token tiles of 2 x 256 sharing each dequantized weight stage, 64-k stages
    int n_tiles, m_tiles, k_blocks;  // k_blocks = ceil(k / k per stage)
    int stages;
    uint32_t idesc;
    // stream-K: the (tile, k-block) units form one sequence, CTA b owns units [b*q + min(b,r), ...)
    int unit_q, unit_r;
    float* partial;        // [ctas][GEMM_PIECE_TOKENS][128] fp32: a CTA's piece of a tile that begins in an earlier CTA
    unsigned int* ready;   // [ctas][4] generation whose piece (per 32-row quarter) is complete in `partial`
    unsigned int* gen;     // [0] generations completed so far, [1] CTAs that have left the current launch: the kernel
                           // numbers its own launches, so a launch recorded in a CUDA graph is a new generation on every replay
};

// One CTA's share of the unit sequence, cut into segments: a segment is a run of k-blocks of one tile.
struct GemmSegment {
    int tile, kb0, kb1;  // k-blocks [kb0, kb1) of `tile`
};
__device__ __forceinline__ void cta_units(const GemmParams& p, int cta, int& u0, int& u1) {
    u0 = cta * p.unit_q + min(cta, p.unit_r);
    u1 = u0 + p.unit_q + (cta < p.unit_r ? 1 : 0);
}
// the segment that starts at unit u (u < u1)
__device__ __forceinline__ GemmSegment segment_at(const GemmParams& p, int u, int u1) {
    GemmSegment g;
    g.tile = u / p.k_blocks;
    g.kb0 = u - g.tile * p.k_blocks;
    g.kb1 = min(p.k_blocks, g.kb0 + (u1 - u));
    return g;
}

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t g_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void g_mbar_init(void* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(g_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void g_mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(g_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void g_mbar_expect_tx(void* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(g_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool g_mbar_wait(void* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .u32 n;\n\t"
        "mov.u32 n, 0;\n\t"
        "WFG_WAIT_%=:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra WFG_DONE_%=;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 q, n, %3;\n\t"
        "@q bra WFG_WAIT_%=;\n\t"
        "WFG_DONE_%=:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(g_smem_u32(bar)), "r"(parity), "r"((uint32_t)GEMM_WAIT_SPINS)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            g_smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(g_smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(void* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(g_smem_u32(smem_dst)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(g_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused with swizzle), 16 B
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                    // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- epilogue pieces (one lane = one weight row)
// r[j] = accumulator of (token m0 + j, weight row n).  Rows of y are ldy floats apart; a warp writes 32
// consecutive floats of one token row per store.  m0 is a multiple of 32, so the row scales load as float4.
__device__ __forceinline__ void store_chunk(float* __restrict__ y, int64_t ldy, int64_t col0, const float* __restrict__ unscale,
                                            const uint32_t (&r)[32], int m0, int m, int n, int rows) {
    if (n >= rows || m0 >= m) return;
    float* yp = y + (int64_t)m0 * ldy + col0 + n;
    if (m0 + 32 <= m) {
        float sc[32];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(unscale + m0) + i);
            sc[4 * i] = v.x, sc[4 * i + 1] = v.y, sc[4 * i + 2] = v.z, sc[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int j = 0; j < 32; j++) yp[(int64_t)j * ldy] = __uint_as_float(r[j]) * sc[j];
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++)
            if (m0 + j < m) yp[(int64_t)j * ldy] = __uint_as_float(r[j]) * __ldg(unscale + m0 + j);
    }
}
// A stream-K piece is token-major, 128 weight rows contiguous per token.
__device__ __forceinline__ void write_piece_chunk(float* __restrict__ piece, const uint32_t (&r)[32], int tok, int row) {
    float* pp = piece + (size_t)tok * GEMM_BN + row;
#pragma unroll
    for (int j = 0; j < 32; j++) pp[j * GEMM_BN] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void add_piece_chunk(const float* __restrict__ piece, uint32_t (&r)[32], int tok, int row) {
    const float* pp = piece + (size_t)tok * GEMM_BN + row;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = __ldcg(pp + j * GEMM_BN);  // 32 independent loads in flight
#pragma unroll
    for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) + v[j]);
}

// ---------------------------------------------------------------- dequantization to fp16
// A plane word holds the codes of 8 consecutive elements: rotated back by PLANE_ROT, nibble p of the
// low half is element 2p and nibble p of the high half element 2p + 1.  As fp16 bit patterns
//   (w & 0x000F000F) | 0x64006400  =  (1024 + e0, 1024 + e1)      codes in mantissa bits 3..0
//   (w & 0x00F000F0) | 0x54005400  =  (  64 + e2,   64 + e3)      codes in mantissa bits 7..4
// and the same two masks on the word rotated by a further 8 bits give elements 4..7.  Two rotates and
// four logic ops per 8 codes; everything after that runs on the half / float pipes.
struct Codes8 {
    uint32_t k[2];  // 1024 + code: elements (0,1), (4,5)
    uint32_t h[2];  // 64 + code:   elements (2,3), (6,7)
};
__device__ __forceinline__ Codes8 unpack8(uint32_t w) {
    const uint32_t a = __funnelshift_r(w, w, PLANE_ROT), b = __funnelshift_r(w, w, PLANE_ROT + 8);
    Codes8 c;
    c.k[0] = (a & 0x000F000Fu) | 0x64006400u;
    c.h[0] = (a & 0x00F000F0u) | 0x54005400u;
    c.k[1] = (b & 0x000F000Fu) | 0x64006400u;
    c.h[1] = (b & 0x00F000F0u) | 0x54005400u;
    return c;
}
__device__ __forceinline__ __half2 as_half2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Q4_0: s * (code - 8) with s an fp16 value.  code - 8 is exact in fp16 and the product is rounded
// once, exactly like the fp32 product rounded to fp16.
__device__ __forceinline__ uint4 word_to_half8_q4_0(uint32_t w, __half2 s2) {
    const Codes8 c = unpack8(w);
    const __half2 m1032 = __float2half2_rn(-1032.f), m72 = __float2half2_rn(-72.f);
    uint4 o;
    o.x = as_u32(__hmul2(__hadd2(as_half2(c.k[0]), m1032), s2));
    o.y = as_u32(__hmul2(__hadd2(as_half2(c.h[0]), m72), s2));
    o.z = as_u32(__hmul2(__hadd2(as_half2(c.k[1]), m1032), s2));
    o.w = as_u32(__hmul2(__hadd2(as_half2(c.h[1]), m72), s2));
    return o;
}
// Q8_0: s * (16 (hi - 8) + lo): the integer is exact in fp16 (|q| <= 128), one rounding in the product.
__device__ __forceinline__ uint4 words_to_half8_q8(uint32_t wh, uint32_t wl, __half2 s2) {
    const Codes8 h = unpack8(wh), l = unpack8(wl);
    const __half2 m1032 = __float2half2_rn(-1032.f), m72 = __float2half2_rn(-72.f);
    const __half2 m1024 = __float2half2_rn(-1024.f), m64 = __float2half2_rn(-64.f), sixteen = __float2half2_rn(16.f);
    uint4 o;
    o.x = as_u32(__hmul2(__hfma2(sixteen, __hadd2(as_half2(h.k[0]), m1032), __hadd2(as_half2(l.k[0]), m1024)), s2));
    o.y = as_u32(__hmul2(__hfma2(sixteen, __hadd2(as_half2(h.h[0]), m72), __hadd2(as_half2(l.h[0]), m64)), s2));
    o.z = as_u32(__hmul2(__hfma2(sixteen, __hadd2(as_half2(h.k[1]), m1032), __hadd2(as_half2(l.k[1]), m1024)), s2));
    o.w = as_u32(__hmul2(__hfma2(sixteen, __hadd2(as_half2(h.h[1]), m72), __hadd2(as_half2(l.h[1]), m64)), s2));
    return o;
}
// Q4_K: a * code + b in fp32 (a = d * sc and b = -dmin * m are exact in fp32), rounded once to fp16.
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 word_to_half8(uint32_t w, float a, float b) {
    const Codes8 c = unpack8(w);
    const float bk = fmaf(-1024.f, a, b), bh = fmaf(-64.f, a, b);  // the unpacked values carry 1024 / 64
    const float2 f0 = __half22float2(as_half2(c.k[0])), f1 = __half22float2(as_half2(c.h[0]));
    const float2 f2 = __half22float2(as_half2(c.k[1])), f3 = __half22float2(as_half2(c.h[1]));
    uint4 o;
    o.x = pack_half2(fmaf(a, f0.x, bk), fmaf(a, f0.y, bk));
    o.y = pack_half2(fmaf(a, f1.x, bh), fmaf(a, f1.y, bh));
    o.z = pack_half2(fmaf(a, f2.x, bk), fmaf(a, f2.y, bk));
    o.w = pack_half2(fmaf(a, f3.x, bh), fmaf(a, f3.y, bh));
    return o;
}

// A stage address of the 16-byte chunk (row r, chunk c of 16 along k): two swizzled 64-k spans
__device__ __forceinline__ uint32_t a_chunk_off(int r, int c) {
    return (uint32_t)((c >> 3) * (GEMM_BN * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

// One warp dequantizes one 16-row tile x 128 k of the stage: rows rt16*16 .. +15.  The work is split
// into load (global memory -> registers) and store (registers -> fp16 in the swizzled stage): the
// weights come from HBM, and the loads of the next step are issued into a second register set
// before the current step is converted, so their latency is off the stage hand-over path.
template <int QT> struct DequantRegs;

template <> struct DequantRegs<WF_QTYPE_Q4_0> {
    uint4 c[1];
    uint2 sc[1];
    __device__ __forceinline__ void load(const uint8_t* tile, int kb, int lane, int hsel) {
        (void)kb;
        const int g = lane >> 2;
        {
            const int h = hsel;
            c[0] = __ldg(reinterpret_cast<const uint4*>(tile + h * 512 + lane * 16));
            sc[0] = __ldg(reinterpret_cast<const uint2*>(tile + Tile<WF_QTYPE_Q4_0>::SCALE_OFF + g * 16 + h * 8));
        }
    }
    template <class F>
    __device__ __forceinline__ void convert(int lane, int hsel, F&& f) const {  // f(row half, 16-byte chunk, 8 fp16 values)
        (void)lane;
        {
            const int h = hsel;
            const __half2 s01 = as_half2(sc[0].x), s23 = as_half2(sc[0].y);  // block scales 0..3 of this row, fp16
            const __half2 s[4] = {__low2half2(s01), __high2half2(s01), __low2half2(s23), __high2half2(s23)};
            const uint32_t w[4] = {c[0].x, c[0].y, c[0].z, c[0].w};
#pragma unroll
            for (int j = 0; j < 4; j++)  // value = s * (code - 8)
                f(h, j, word_to_half8_q4_0(w[j], s[j]));
        }
    }
};

template <> struct DequantRegs<WF_QTYPE_Q4_1> {
    uint4 c[1];
    uint2 sc[1], mn[1];
    __device__ __forceinline__ void load(const uint8_t* tile, int kb, int lane, int hsel) {
        (void)kb;
        using T = Tile<WF_QTYPE_Q4_1>;
        const int g = lane >> 2;
        {
            const int h = hsel;
            c[0] = __ldg(reinterpret_cast<const uint4*>(tile + h * 512 + lane * 16));
            sc[0] = __ldg(reinterpret_cast<const uint2*>(tile + T::SCALE_OFF + g * 16 + h * 8));
            mn[0] = __ldg(reinterpret_cast<const uint2*>(tile + T::MIN_OFF + g * 16 + h * 8));
        }
    }
    template <class F>
    __device__ __forceinline__ void convert(int lane, int hsel, F&& f) const {  // f(row half, 16-byte chunk, 8 fp16 values)
        (void)lane;
        {
            const int h = hsel;
            const float2 s01 = __half22float2(as_half2(sc[0].x)), s23 = __half22float2(as_half2(sc[0].y));
            const float2 m01 = __half22float2(as_half2(mn[0].x)), m23 = __half22float2(as_half2(mn[0].y));
            const float a[4] = {s01.x, s01.y, s23.x, s23.y}, b[4] = {m01.x, m01.y, m23.x, m23.y};
            const uint32_t w[4] = {c[0].x, c[0].y, c[0].z, c[0].w};
#pragma unroll
            for (int j = 0; j < 4; j++)  // value = scale * code + min in fp32, rounded once to fp16
                f(h, j, word_to_half8(w[j], a[j], b[j]));
        }
    }
};

template <> struct DequantRegs<WF_QTYPE_Q8_0> {
    uint4 ch[1], cl[1];
    uint2 sc[1];
    __device__ __forceinline__ void load(const uint8_t* tile, int kb, int lane, int hsel) {
        (void)kb;
        const int g = lane >> 2;
        {
            const int h = hsel;
            ch[0] = __ldg(reinterpret_cast<const uint4*>(tile + h * 512 + lane * 16));
            cl[0] = __ldg(reinterpret_cast<const uint4*>(tile + PLANE_BYTES + h * 512 + lane * 16));
            sc[0] = __ldg(reinterpret_cast<const uint2*>(tile + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + g * 16 + h * 8));
        }
    }
    template <class F>
    __device__ __forceinline__ void convert(int lane, int hsel, F&& f) const {  // f(row half, 16-byte chunk, 8 fp16 values)
        (void)lane;
        {
            const int h = hsel;
            const __half2 s01 = as_half2(sc[0].x), s23 = as_half2(sc[0].y);
            const __half2 s[4] = {__low2half2(s01), __high2half2(s01), __low2half2(s23), __high2half2(s23)};
            const uint32_t wh[4] = {ch[0].x, ch[0].y, ch[0].z, ch[0].w}, wl[4] = {cl[0].x, cl[0].y, cl[0].z, cl[0].w};
#pragma unroll
            for (int j = 0; j < 4; j++)
                f(h, j, words_to_half8_q8(wh[j], wl[j], s[j]));
        }
    }
};

template <> struct DequantRegs<WF_QTYPE_Q4_K> {  // the stage is one half (plane kb & 1) of a 256-k tile
    uint4 c[1];
    uint32_t dd[1], scw[1], mnw[1];
    __device__ __forceinline__ void load(const uint8_t* tile, int kb, int lane, int hsel) {
        using T = Tile<WF_QTYPE_Q4_K>;
        const int g = lane >> 2, pl = kb & 1;
        {
            const int h = hsel;
            c[0] = __ldg(reinterpret_cast<const uint4*>(tile + pl * PLANE_BYTES + h * 512 + lane * 16));
            dd[0] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::D_OFF + g * 8 + h * 4));
            scw[0] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::SC_OFF + g * 16 + h * 8 + pl * 4));
            mnw[0] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::MN_OFF + g * 16 + h * 8 + pl * 4));
        }
    }
    template <class F>
    __device__ __forceinline__ void convert(int lane, int hsel, F&& f) const {  // f(row half, 16-byte chunk, 8 fp16 values)
        (void)lane;
        {
            const int h = hsel;
            const float2 d = __half22float2(as_half2(dd[0]));  // (d, dmin)
            const uint32_t w[4] = {c[0].x, c[0].y, c[0].z, c[0].w};
#pragma unroll
            for (int j = 0; j < 4; j++) {  // value = (d * sc) * code - dmin * m
                const float a = d.x * (float)((scw[0] >> (8 * j)) & 0xFF), b = -(d.y * (float)((mnw[0] >> (8 * j)) & 0xFF));
                f(h, j, word_to_half8(w[j], a, b));
            }
        }
    }
};

// 64-k stages (token tiles of 512): a warp converts 16 rows x 64 k of a weight tile per stage, i.e. the
// two words (32-k blocks) 2*sub and 2*sub + 1 of every lane's 16-byte piece.  `sub` counts 64-k pieces
// inside the weight tile: 0..1 for the 128-k formats, 0..3 for Q4_K (plane = sub / 2).
template <int QT> struct DequantHalf;

template <> struct DequantHalf<WF_QTYPE_Q4_0> {
    uint2 c[1];
    uint32_t sc[1];
    __device__ __forceinline__ void load(const uint8_t* tile, int sub, int lane, int hsel) {
        const int g = lane >> 2;
        {
            const int h = hsel;
            c[0] = __ldg(reinterpret_cast<const uint2*>(tile + h * 512 + lane * 16 + sub * 8));
            sc[0] = __ldg(reinterpret_cast<const uint32_t*>(tile + Tile<WF_QTYPE_Q4_0>::SCALE_OFF + g * 16 + h * 8 + sub * 4));
        }
    }
    template <class F>
    __device__ __forceinline__ void convert(int lane, int hsel, F&& f) const {  // f(row half, 16-byte chunk, 8 fp16 values)
        (void)lane;
        {
            const int h = hsel;
            const __half2 s01 = as_half2(sc[0]);
            f(h, 0, word_to_half8_q4_0(c[0].x, __low2half2(s01)));
            f(h, 1, word_to_half8_q4_0(c[0].y, __high2half2(s01)));
        }
    }
};

template <> struct DequantHalf<WF_QTYPE_Q4_1> {
    uint2 c[1];
    uint32_t sc[1], mn[1];
    __device__ __forceinline__ void load(const uint8_t* tile, int sub, int lane, int hsel) {
        using T = Tile<WF_QTYPE_Q4_1>;
        const int g = lane >> 2;
        {
            const int h = hsel;
            c[0] = __ldg(reinterpret_cast<const uint2*>(tile + h * 512 + lane * 16 + sub * 8));
            sc[0] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::SCALE_OFF + g * 16 + h * 8 + sub * 4));
            mn[0] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::MIN_OFF + g * 16 + h * 8 + sub * 4));
        }
    }
    template <class F>
    __device__ __forceinline__ void convert(int lane, int hsel, F&& f) const {  // f(row half, 16-byte chunk, 8 fp16 values)
        (void)lane;
        {
            const int h = hsel;
            const float2 s = __half22float2(as_half2(sc[0])), m = __half22float2(as_half2(mn[0]));
            f(h, 0, word_to_half8(c[0].x, s.x, m.x));
            f(h, 1, word_to_half8(c[0].y, s.y, m.y));
        }
    }
};

template <> struct DequantHalf<WF_QTYPE_Q8_0> {
    uint2 ch[1], cl[1];
    uint32_t sc[1];
    __device__ __forceinline__ void load(const uint8_t* tile, int sub, int lane, int hsel) {
        const int g = lane >> 2;
        {
            const int h = hsel;
            ch[0] = __ldg(reinterpret_cast<const uint2*>(tile + h * 512 + lane * 16 + sub * 8));
            cl[0] = __ldg(reinterpret_cast<const uint2*>(tile + PLANE_BYTES + h * 512 + lane * 16 + sub * 8));
            sc[0] = __ldg(reinterpret_cast<const uint32_t*>(tile + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + g * 16 + h * 8 + sub * 4));
        }
    }
    template <class F>
    __device__ __forceinline__ void convert(int lane, int hsel, F&& f) const {  // f(row half, 16-byte chunk, 8 fp16 values)
        (void)lane;
        {
            const int h = hsel;
            const __half2 s01 = as_half2(sc[0]);
            f(h, 0, words_to_half8_q8(ch[0].x, cl[0].x, __low2half2(s01)));
            f(h, 1, words_to_half8_q8(ch[0].y, cl[0].y, __high2half2(s01)));
        }
    }
};

template <> struct DequantHalf<WF_QTYPE_Q4_K> {
    uint2 c[1];
    uint32_t dd[1];
    uint16_t scw[1], mnw[1];  // the two 8-bit sub-block scales / mins of this 64-k piece
    __device__ __forceinline__ void load(const uint8_t* tile, int sub, int lane, int hsel) {
        using T = Tile<WF_QTYPE_Q4_K>;
        const int g = lane >> 2;
        {
            const int h = hsel;
            c[0] = __ldg(reinterpret_cast<const uint2*>(tile + (sub >> 1) * PLANE_BYTES + h * 512 + lane * 16 + (sub & 1) * 8));
            dd[0] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::D_OFF + g * 8 + h * 4));
            scw[0] = __ldg(reinterpret_cast<const uint16_t*>(tile + T::SC_OFF + g * 16 + h * 8 + sub * 2));
            mnw[0] = __ldg(reinterpret_cast<const uint16_t*>(tile + T::MN_OFF + g * 16 + h * 8 + sub * 2));
        }
    }
    template <class F>
    __device__ __forceinline__ void convert(int lane, int hsel, F&& f) const {  // f(row half, 16-byte chunk, 8 fp16 values)
        (void)lane;
        {
            const int h = hsel;
            const float2 d = __half22float2(as_half2(dd[0]));  // (d, dmin)
            const float a0 = d.x * (float)(scw[0] & 0xFF), b0 = -(d.y * (float)(mnw[0] & 0xFF));
            const float a1 = d.x * (float)(scw[0] >> 8), b1 = -(d.y * (float)(mnw[0] >> 8));
            f(h, 0, word_to_half8(c[0].x, a0, b0));
            f(h, 1, word_to_half8(c[0].y, a1, b1));
        }
    }
};

// ---------------------------------------------------------------- activation pre-pass
// One CTA per token row: x16[row] = fp16(x[row] * 2^s) with s chosen so the largest magnitude lands in
// [2^14, 2^15); unscale[row] = 2^-s.  bf16 -> fp16 is exact whenever the scaled value is a normal fp16.
// The row is read once: every thread keeps its 16-byte pieces in registers between the exponent scan
// and the conversion (up to 4 pieces = K <= 8192 at 256 threads; longer rows re-read the rest).
constexpr int XPRE_THREADS = 256, XPRE_KEEP = 4;
__global__ void __launch_bounds__(XPRE_THREADS) x_to_f16_kernel(const uint16_t* __restrict__ x, __half* __restrict__ x16,
                                                                float* __restrict__ unscale, int k) {
    __shared__ int s_emax;
    // Launched with programmatic stream serialization itself: its CTAs may be placed while the previous kernel of the
    // stream drains, but nothing is read or written before that kernel has completed (it may have produced x, and a
    // previous GEMM may still be reading the fp16 copy this kernel rewrites).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the GEMM may set itself up while the rows are converted
    const uint4* row = reinterpret_cast<const uint4*>(x + (size_t)blockIdx.x * k);  // k is a multiple of 8
    uint4* out = reinterpret_cast<uint4*>(x16 + (size_t)blockIdx.x * k);
    const int pieces = k >> 3;
    if (threadIdx.x == 0) s_emax = 0;
    __syncthreads();
    auto emax_of = [](uint4 v) {
        int m = 0;
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e0 = (w[i] >> 7) & 0xFF, e1 = (w[i] >> 23) & 0xFF;  // bf16 biased exponents
            m = max(m, e0 == 0xFF ? 0 : e0);                              // Inf / NaN do not drive the scale
            m = max(m, e1 == 0xFF ? 0 : e1);
        }
        return m;
    };
    uint4 keep[XPRE_KEEP];
    int emax = 0;
#pragma unroll
    for (int u = 0; u < XPRE_KEEP; u++) {
        const int i = threadIdx.x + u * XPRE_THREADS;
        keep[u] = i < pieces ? __ldg(row + i) : make_uint4(0, 0, 0, 0);
        emax = max(emax, emax_of(keep[u]));
    }
    for (int i = threadIdx.x + XPRE_KEEP * XPRE_THREADS; i < pieces; i += XPRE_THREADS) emax = max(emax, emax_of(__ldg(row + i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) emax = max(emax, __shfl_xor_sync(0xFFFFFFFFu, emax, o));
    if ((threadIdx.x & 31) == 0) atomicMax(&s_emax, emax);
    __syncthreads();
    emax = s_emax;
    const int shift = emax == 0 ? 0 : (127 + 14) - emax;  // multiply by 2^shift
    const float scale = __uint_as_float((uint32_t)min(max(127 + shift, 1), 254) << 23);
    auto convert = [scale](uint4 v) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 h = __floats2half2_rn(__uint_as_float(w[i] << 16) * scale, __uint_as_float(w[i] & 0xFFFF0000u) * scale);
            o[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(o[0], o[1], o[2], o[3]);
    };
#pragma unroll
    for (int u = 0; u < XPRE_KEEP; u++) {
        const int i = threadIdx.x + u * XPRE_THREADS;
        if (i < pieces) out[i] = convert(keep[u]);
    }
    for (int i = threadIdx.x + XPRE_KEEP * XPRE_THREADS; i < pieces; i += XPRE_THREADS) out[i] = convert(__ldg(row + i));
    if (threadIdx.x == 0) unscale[blockIdx.x] = __uint_as_float((uint32_t)min(max(127 - shift, 1), 254) << 23);
}

// ---------------------------------------------------------------- the kernel
// smem: [0,1024) barriers + tmem slot | stages x (A 32 KB | B bm*256 B), 1024-byte aligned
template <int QT>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* b_full = reinterpret_cast<uint64_t*>(smem);        // [8] activations landed
    uint64_t* a_full = b_full + 8;                               // [8] weights dequantized
    uint64_t* s_empty = a_full + 8;                              // [8] stage consumed by the MMA
    uint64_t* acc_full = s_empty + 8;                            // [2]
    uint64_t* acc_empty = acc_full + 2;                          // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // this launch's generation: the previous GEMM of the stream has ended before this kernel starts (the activation
    // pre-pass between them waits for it before it lets this kernel go), so its closing store is visible
    unsigned int launch_gen = ld_acquire_u32(p.gen) + 1u;
    if (launch_gen == 0u) launch_gen = 1u;  // 0 is what untouched flags hold
    const bool wide = p.halves == 2, k64 = wide;  // 64-k stages go with the two-half token tiles (alone they measured 25 % slower)
    const uint32_t a_bytes = k64 ? GEMM_WIDE_A_BYTES : GEMM_A_BYTES;
    const uint32_t b_bytes = wide ? 2u * GEMM_WIDE_B_HALF : (uint32_t)p.bm * 256;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    uint8_t* stage0 = smem + 1024;

    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int stages = p.stages;
    int u0, u1;
    cta_units(p, blockIdx.x, u0, u1);
    constexpr int TILE_BYTES = Tile<QT>::BYTES;
    constexpr int KB_PER_WTILE = Tile<QT>::K / GEMM_BK;  // stages per weight k-tile: 1 (Q4_0, Q8_0) or 2 (Q4_K)

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            g_mbar_init(&b_full[s], 1);
            g_mbar_init(&a_full[s], GEMM_DEQUANT_WARPS);
            g_mbar_init(&s_empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            g_mbar_init(&acc_full[b], 1);
            g_mbar_init(&acc_empty[b], 4);  // four epilogue warps
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto fail = [&]() {
        atomicOr(p.status, STATUS_GEMM_PIPE_TIMEOUT);
        *abort_flag = 1;
    };

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (activations)
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // the fp16 activations are the pre-pass kernel's output
            int it = 0;
            for (int u = u0; u < u1 && !*abort_flag;) {
                const GemmSegment g = segment_at(p, u, u1);
                const int mt = g.tile % p.m_tiles;
                const int nh = (wide && p.m - mt * 512 > 256) ? 2 : 1;  // 256-token halves of this tile that hold tokens
                for (int kb = g.kb0; kb < g.kb1; kb++, it++) {
                    const int s = it % stages;
                    if (it >= stages && !g_mbar_wait(&s_empty[s], ((it / stages) - 1) & 1)) { fail(); break; }
                    uint8_t* b_stage = stage0 + (size_t)s * stage_bytes + a_bytes;
                    if (wide) {  // one 64-k span per 256-token half
                        g_mbar_expect_tx(&b_full[s], (uint32_t)nh * GEMM_WIDE_B_HALF);
                        for (int h = 0; h < nh; h++)
                            tma_load_2d(b_stage + h * GEMM_WIDE_B_HALF, &xmap, kb * GEMM_WIDE_BK, mt * 512 + h * 256, &b_full[s]);
                    } else {
                        g_mbar_expect_tx(&b_full[s], b_bytes);
                        tma_load_2d(b_stage, &xmap, kb * GEMM_BK, mt * p.bm, &b_full[s]);
                        tma_load_2d(b_stage + b_bytes / 2, &xmap, kb * GEMM_BK + 64, mt * p.bm, &b_full[s]);
                    }
                }
                u += g.kb1 - g.kb0;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0 && wide) {
            // Token tile = two halves of 256 tokens, each with its own accumulator (TMEM columns 0 and 256) and its
            // own full / empty barrier; both halves consume the same dequantized weight stage.  used[h] counts
            // the tiles that have used half h (a tile's second half is skipped when it holds no tokens).
            int it = 0, used[2] = {0, 0};
            for (int u = u0; u < u1 && !*abort_flag;) {
                const GemmSegment g = segment_at(p, u, u1);
                const int mt = g.tile % p.m_tiles;
                const int nh = (p.m - mt * 512 > 256) ? 2 : 1;
                bool ok = true;
                for (int kb = g.kb0; kb < g.kb1 && ok; kb++, it++) {
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1;
                    if (!g_mbar_wait(&b_full[s], ph) || !g_mbar_wait(&a_full[s], ph)) { fail(); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = g_smem_u32(stage0 + (size_t)s * stage_bytes);
                    const uint32_t b_addr = a_addr + GEMM_WIDE_A_BYTES;
                    for (int h = 0; h < nh; h++) {
                        if (kb == g.kb0 && used[h] >= 1) {  // the epilogue must have drained this half's previous tile
                            if (!g_mbar_wait(&acc_empty[h], (used[h] - 1) & 1)) { fail(); ok = false; break; }
                            tc_fence_after();
                        }
                        const uint32_t d_tmem = tmem_base + (uint32_t)(h * 256);
#pragma unroll
                        for (int kk = 0; kk < 4; kk++) {  // 4 x K16 per 64-k stage
                            const uint64_t ad = smem_desc_sw128(a_addr + kk * 32);
                            const uint64_t bd = smem_desc_sw128(b_addr + h * GEMM_WIDE_B_HALF + kk * 32);
                            tc_mma_f16(d_tmem, ad, bd, p.idesc, ((kb - g.kb0) | kk) != 0);
                        }
                        if (kb == g.kb1 - 1) {
                            tc_commit(&acc_full[h]);
                            used[h]++;
                        }
                    }
                    if (!ok) break;
                    tc_commit(&s_empty[s]);
                }
                if (!ok) break;
                u += g.kb1 - g.kb0;
            }
        } else if (lane == 0) {
            int it = 0, local = 0;
            for (int u = u0; u < u1 && !*abort_flag; local++) {
                const GemmSegment g = segment_at(p, u, u1);
                const int buf = local & 1;
                if (local >= 2 && !g_mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1)) { fail(); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * p.bm);
                bool ok = true;
                for (int kb = g.kb0; kb < g.kb1 && ok; kb++, it++) {
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1;
                    if (!g_mbar_wait(&b_full[s], ph) || !g_mbar_wait(&a_full[s], ph)) { fail(); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = g_smem_u32(stage0 + (size_t)s * stage_bytes);
                    const uint32_t b_addr = a_addr + a_bytes;
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) {  // 8 x K16 per stage; spans of 64 k are 16 KB (A) / bm*128 B (B) apart
                        const uint64_t ad = smem_desc_sw128(a_addr + (kk >> 2) * (GEMM_BN * 128) + (kk & 3) * 32);
                        const uint64_t bd = smem_desc_sw128(b_addr + (kk >> 2) * (b_bytes / 2) + (kk & 3) * 32);
                        tc_mma_f16(d_tmem, ad, bd, p.idesc, ((kb - g.kb0) | kk) != 0);
                    }
                    tc_commit(&s_empty[s]);  // frees the stage when these MMAs have read it
                }
                if (!ok) break;
                tc_commit(&acc_full[buf]);
                u += g.kb1 - g.kb0;
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------------------------ epilogue (TMEM lane quarter = warp % 4)
        // Handles every segment except the tile this CTA owns the beginning of and shares with the following
        // CTAs: that one is always the last segment of the share and is finished by all warps together below.
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;  // weight row inside the 128-row block
        int local = 0, used[2] = {0, 0};
        bool dead = false;
        asm volatile("griddepcontrol.wait;" ::: "memory");  // the row scales are the pre-pass kernel's output
        float* mine = p.partial + (size_t)blockIdx.x * GEMM_PIECE_TOKENS * GEMM_BN;
        for (int u = u0; u < u1 && !*abort_flag && !dead; local++) {
            const GemmSegment g = segment_at(p, u, u1);
            const int nt = g.tile / p.m_tiles, mt = g.tile % p.m_tiles;
            const int n = nt * GEMM_BN + row;
            const bool starts = g.kb0 == 0, ends = g.kb1 == p.k_blocks;
            if (starts && !ends) break;
            // The tile's accumulators: one (double buffered, `local & 1`) or one per 256-token half.
            const int parts = wide ? ((p.m - mt * 512 > 256) ? 2 : 1) : 1;
            for (int h = 0; h < parts; h++) {
                const int acc = wide ? h : (local & 1);
                const uint32_t parity = wide ? (uint32_t)(used[h] & 1) : (uint32_t)((local >> 1) & 1);
                const int col_base = wide ? h * 256 : acc * p.bm;   // TMEM column of the accumulator
                const int tok_base = wide ? mt * 512 + h * 256 : mt * p.bm;
                const int piece_base = wide ? h * 256 : 0;          // token offset inside a stream-K piece
                const int ncols = wide ? 256 : p.bm;
                if (!g_mbar_wait(&acc_full[acc], parity)) { if (lane == 0) fail(); dead = true; break; }
                tc_fence_after();
                used[h]++;
                // 32 columns at a time (also past a BM that is not a multiple of 32)
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col_base;
                auto emit = [&](const uint32_t (&r)[32], int c) {
                    if (!starts) write_piece_chunk(mine, r, piece_base + c, row);  // my piece of a tile owned by an earlier CTA
                    else store_chunk(p.y, p.ldy, p.col0, p.row_unscale, r, tok_base + c, p.m, n, p.rows);
                };
                for (int c = 0; c < ncols; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + (uint32_t)c, r);
                    emit(r, c);
                }
                tc_fence_before();  // the accumulator has been read: the MMA issuer may overwrite it
                __syncwarp();
                if (lane == 0) g_mbar_arrive(&acc_empty[acc]);
            }
            if (dead) break;
            if (!starts) {  // publish this warp's 32 rows of the piece
                __threadfence();
                __syncwarp();
                if (lane == 0) st_release_u32(p.ready + blockIdx.x * 4 + quarter, launch_gen);
            }
            u += g.kb1 - g.kb0;
        }
    } else {
        // ------------------------------------------------ dequant warps 2, 3, 8..: one 16-row tile (or half of one) each per stage
        const int dw = (warp < 4) ? warp - 2 : warp - 6;  // 0 .. GEMM_DEQUANT_WARPS - 1
        // 16-row tile inside the 128-row block, and the first row half (rows g or g + 8) this warp converts
        const int dq = GEMM_DQ_HALVES == 2 ? dw : dw >> 1, hsel0 = GEMM_DQ_HALVES == 2 ? 0 : dw & 1;
        // One step: convert the registers loaded earlier into fp16 rows (still in registers), wait for the stage,
        // store them and hand the stage over.  Converting before the wait keeps the arithmetic off the path
        // between "the MMAs have released the stage" and "the stage is full again".
        const int dg = lane >> 2, dq4 = lane & 3;
        const bool odd_row = (dg & 1) != 0;
        auto finish_step = [&](const auto& regs, int it) {  // regs[GEMM_DQ_HALVES]
            const int s = it % stages;
            uint4 out[GEMM_DQ_HALVES][4];
#pragma unroll
            for (int hh = 0; hh < GEMM_DQ_HALVES; hh++)
                regs[hh].convert(lane, hsel0 + hh, [&](int, int j, uint4 v) { out[hh][j] = v; });
            if (it >= stages && !g_mbar_wait(&s_empty[s], ((it / stages) - 1) & 1)) {
                if (lane == 0) fail();
                return false;
            }
            uint8_t* a_stage = stage0 + (size_t)s * stage_bytes;
            const int nj = k64 ? 2 : 4;  // 16-byte chunks per row half and lane: 64 k or 128 k per stage
            // A 16-byte store is served eight lanes at a time, i.e. two consecutive rows x four chunks.  Under the
            // 128-byte swizzle chunks 4j .. 4j + 3 of both rows fall into the same 64-byte half of their rows, a
            // two-way bank conflict; so the odd row of each pair stores its chunks of block j ^ 1 in that slot.
#pragma unroll
            for (int hh = 0; hh < GEMM_DQ_HALVES; hh++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (j < nj) {
                        const uint4 e = out[hh][j], o = out[hh][j ^ 1];
                        const uint4 v = odd_row ? o : e;
                        *reinterpret_cast<uint4*>(a_stage + a_chunk_off(dq * 16 + dg + 8 * (hsel0 + hh), ((j ^ (int)odd_row) * 4 + dq4))) = v;
                    }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) g_mbar_arrive(&a_full[s]);
            return true;
        };
        // DEPTH register sets in turn: the loads of steps u + 1 .. u + DEPTH - 1 are in flight while step u is
        // converted.  Two sets for the 128-k steps (four measured 9 % slower: the unrolled loop is four
        // conversions long), four for the 64-k steps, which are half as long and half as large.
        auto run = [&](auto& r, auto kbw_tag, auto depth_tag) {
            constexpr int DEPTH = decltype(depth_tag)::value, KBW = decltype(kbw_tag)::value;  // KBW: stage-sized pieces per weight k-tile
            // weight tile of unit u (tile-major, k-block minor), this warp's rows of the 128-row block, and the
            // piece of it the k-block covers
            auto load = [&](auto& regs, int u) {
                const int tile = u / p.k_blocks, kb = u - tile * p.k_blocks;
                const int64_t wrt = (int64_t)(tile / p.m_tiles) * (GEMM_BN / 16) + dq;
#pragma unroll
                for (int hh = 0; hh < GEMM_DQ_HALVES; hh++)
                    regs[hh].load(p.tiles + (wrt * p.kt_w + kb / KBW) * (int64_t)TILE_BYTES, kb % KBW, lane, hsel0 + hh);
            };
#pragma unroll
            for (int d = 0; d < DEPTH - 1; d++)
                if (u0 + d < u1) load(r[d], u0 + d);
            bool ok = true;
            for (int u = u0, it = 0; u < u1 && ok && !*abort_flag; u += DEPTH) {
#pragma unroll
                for (int d = 0; d < DEPTH; d++) {  // r[d] holds step u + d; refill the set that was converted last
                    if (u + d >= u1) break;
                    if (u + d + DEPTH - 1 < u1) load(r[(d + DEPTH - 1) % DEPTH], u + d + DEPTH - 1);
                    if (!finish_step(r[d], it++)) { ok = false; break; }
                }
            }
        };
        if (k64) {
            DequantHalf<QT> r[4][GEMM_DQ_HALVES];
            run(r, std::integral_constant<int, Tile<QT>::K / GEMM_WIDE_BK>{}, std::integral_constant<int, 4>{});
        } else {
            DequantRegs<QT> r[2][GEMM_DQ_HALVES];
            run(r, std::integral_constant<int, KB_PER_WTILE>{}, std::integral_constant<int, 2>{});
        }
    }

    // ------------------------------------------------ the tile whose beginning this CTA owns and whose rest lies in the
    // following CTAs.  It is the last segment of the share, so every role has run out of work: twelve warps
    // (three per TMEM lane quarter, each taking every third group of 32 tokens) add the followers' pieces in CTA
    // order and write y.  The pieces were computed at the head of the followers' shares, long before this tail.
    if (u0 < u1 && warp < 12) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int tile = (u1 - 1) / p.k_blocks;
        const int kb0 = max(u0, tile * p.k_blocks) - tile * p.k_blocks, kb1 = u1 - tile * p.k_blocks;
        if (kb0 == 0 && kb1 < p.k_blocks) {
            const int quarter = warp & 3, slice = warp >> 2;
            const int row = quarter * 32 + lane;
            const int nt = tile / p.m_tiles, mt = tile % p.m_tiles;
            const int n = nt * GEMM_BN + row;
            // accumulator bookkeeping of the segments before this one (what the epilogue warps counted)
            int local = 0, used[2] = {0, 0};
            for (int u = u0; u < u1;) {
                const GemmSegment g = segment_at(p, u, u1);
                if (g.tile == tile) break;
                used[0]++;
                if (wide && p.m - (g.tile % p.m_tiles) * 512 > 256) used[1]++;
                local++;
                u += g.kb1 - g.kb0;
            }
            // followers: the CTAs holding the rest of the tile; this quarter's rows of their pieces must be complete
            int last_cta = (int)blockIdx.x;
            bool ok = !*abort_flag;
            const int tile_end = (tile + 1) * p.k_blocks;
            for (int c = (int)blockIdx.x + 1; c < (int)gridDim.x && ok; c++) {
                int c0, c1;
                cta_units(p, c, c0, c1);
                if (c0 >= tile_end) break;
                if (c0 == c1) continue;
                last_cta = c;
                int spins = 0;
                while (ld_acquire_u32(p.ready + c * 4 + quarter) != launch_gen && ++spins < GEMM_WAIT_SPINS) __nanosleep(64);
                if (spins >= GEMM_WAIT_SPINS) ok = false;
            }
            if (!ok && lane == 0) fail();
            const int parts = wide ? ((p.m - mt * 512 > 256) ? 2 : 1) : 1;
            for (int h = 0; h < parts && ok; h++) {
                const int acc = wide ? h : (local & 1);
                const uint32_t parity = wide ? (uint32_t)(used[h] & 1) : (uint32_t)((local >> 1) & 1);
                const int col_base = wide ? h * 256 : acc * p.bm;
                const int tok_base = wide ? mt * 512 + h * 256 : mt * p.bm;
                const int piece_base = wide ? h * 256 : 0;
                const int ncols = wide ? 256 : p.bm;
                if (!g_mbar_wait(&acc_full[acc], parity)) { if (lane == 0) fail(); break; }
                tc_fence_after();
                for (int c = slice * 32; c < ncols; c += 96) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(col_base + c), r);
                    for (int cc = (int)blockIdx.x + 1; cc <= last_cta; cc++) {  // pieces in CTA order
                        int c0, c1;
                        cta_units(p, cc, c0, c1);
                        if (c0 == c1) continue;
                        add_piece_chunk(p.partial + (size_t)cc * GEMM_PIECE_TOKENS * GEMM_BN, r, piece_base + c, row);
                    }
                    store_chunk(p.y, p.ldy, p.col0, p.row_unscale, r, tok_base + c, p.m, n, p.rows);
                }
            }
        }
    }

    // ------------------------------------------------ teardown: TMEM is freed on every path
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0) {  // the last CTA out closes the generation
        __threadfence();
        if (atomicAdd(p.gen + 1, 1u) == gridDim.x - 1) {
            p.gen[1] = 0u;
            __threadfence();
            st_release_u32(p.gen, launch_gen);
        }
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

constexpr size_t GEMM_SMEM_LIMIT = 227 * 1024;

bool gemm_supported(const Weight& w, int x_dtype, int64_t m, const void* d_x) {
    // bf16 activations, more than the 32 tokens the memory-bound decode kernel takes in one launch; K a multiple of 8 elements and a 16-byte aligned activation
    // pointer (the pre-pass reads 16-byte pieces, the TMA row stride must be a multiple of 16 bytes).  Whole
    // 128-row blocks exist for any row count: the weight buffer is padded to 8 row-tiles with zero scales.
    return x_dtype == WF_DTYPE_BF16 && m > 32 && (w.g.k % 8) == 0 && (reinterpret_cast<uintptr_t>(d_x) & 15) == 0 &&
           encode_tiled_fn() != nullptr;
}

template <int QT>
static cudaError_t gemm_launch_one(const GemmParams& p, const CUtensorMap& map, int grid, size_t smem, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    // Programmatic stream serialization: this kernel may start while the activation pre-pass (the previous launch of
    // the stream) is still running; what reads the pre-pass's output waits with griddepcontrol.wait, the rest
    // (barrier set-up, TMEM allocation, the first weight loads and conversions) runs under it.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_kernel<QT>, p, map);
}

int gemm_launch(Context* c, const GemvCall& call, cudaStream_t s) {
    const Weight& w = *call.w;
    const int qt = w.g.qtype;
    GemmParams p{};
    p.tiles = w.d_tiles;
    p.y = call.d_y;
    p.status = c->d_status;
    p.ldy = call.ldy;
    p.col0 = call.col0;
    p.rows = (int)w.g.rows;
    p.k = (int)w.g.k;
    p.kt_w = (int)w.g.kt;
    p.m = (int)call.m;
    // More than 512 tokens: token tiles of 2 x 256 that share every dequantized weight stage (half the weight
    // loads and conversions per MMA; 4 - 10 % faster at 2048 tokens, equal at 512).  Otherwise one MMA column
    // block per tile and a double-buffered accumulator.
    // The two-half tiles make stream-K pieces of 256 KB: only when there are enough tiles that a tile is cut at most
    // about twice.
    const int64_t wide_tiles = ((w.g.rows + GEMM_BN - 1) / GEMM_BN) * ((call.m + 511) / 512);
    p.halves = (call.m > WF_GEMM_WIDE_MIN && wide_tiles >= c->sm_count / 2) ? 2 : 1;
    p.bm = call.m >= 256 ? 256 : (int)((call.m + 15) / 16 * 16);
    const int tile_tokens = p.bm * p.halves, bk = p.halves == 2 ? GEMM_WIDE_BK : GEMM_BK;
    p.n_tiles = (int)((w.g.rows + GEMM_BN - 1) / GEMM_BN);
    p.m_tiles = (int)((call.m + tile_tokens - 1) / tile_tokens);
    p.k_blocks = (int)((w.g.k + bk - 1) / bk);
    const size_t stage_bytes = p.halves == 2 ? (size_t)GEMM_WIDE_A_BYTES + 2 * GEMM_WIDE_B_HALF : GEMM_A_BYTES + (size_t)p.bm * 256;
    p.stages = (int)std::min<size_t>((GEMM_SMEM_LIMIT - 1024) / stage_bytes, 8);
    // A = fp16 weights, B = fp16 activations, D = fp32; both operands K-major
    p.idesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(p.bm >> 3) << 17) | ((uint32_t)(GEMM_BN >> 4) << 24);

    // the last 128-row block may reach past the padded row-tiles: the weight buffer must cover it
    if ((int64_t)p.n_tiles * (GEMM_BN / 16) > w.g.rt_alloc)
        return set_error(c, WF_ERR_SHAPE, "weight buffer does not cover the last 128-row block");

    // activation pre-pass into the context's fp16 scratch (grown on demand)
    const int64_t x16_bytes = ((call.m * w.g.k * 2 + 255) & ~255LL) + call.m * 4;
    if (x16_bytes > c->x16_bytes) {
        const int rc = refuse_allocation_while_recording(c, s, "the fp16 activation scratch");
        if (rc != WF_OK) return rc;
        if (c->d_x16) cudaFree(c->d_x16);
        c->d_x16 = nullptr;
        c->x16_bytes = 0;
        WF_CUDA(c, cudaMalloc(&c->d_x16, (size_t)x16_bytes));
        c->x16_bytes = x16_bytes;
    }
    __half* x16 = static_cast<__half*>(c->d_x16);
    float* unscale = reinterpret_cast<float*>(static_cast<uint8_t*>(c->d_x16) + ((call.m * w.g.k * 2 + 255) & ~255LL));
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)call.m);
        cfg.blockDim = dim3(XPRE_THREADS);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        WF_CUDA(c, cudaLaunchKernelEx(&cfg, x_to_f16_kernel, static_cast<const uint16_t*>(call.d_x), x16, unscale, (int)w.g.k));
    }
    c->launches++;
    p.row_unscale = unscale;

    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)w.g.k, (cuuint64_t)call.m};
    const cuuint64_t strides[1] = {(cuuint64_t)w.g.k * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)p.bm};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(c, WF_ERR_CUDA_BASE + 1, "cuTensorMapEncodeTiled failed (%d)", (int)r);

    // stream-K shares and the scratch the CTAs hand pieces of cut tiles through
    const int64_t units = (int64_t)p.n_tiles * p.m_tiles * p.k_blocks;
    if (units >= (1LL << 31)) return set_error(c, WF_ERR_TOO_LARGE, "GEMM has too many tile steps");
    // A tile of U k-blocks shared by S CTAs costs about U / S steps plus S - 1 pieces added by its owner, a piece of
    // 256 tokens costing about two steps (smaller ones in proportion, 0.3 at least): no share is shorter than
    // sqrt(c U) steps, which bounds S for weights with few tiles.
    const double piece_steps = std::max(0.3, 2.0 * tile_tokens / 256.0);
    int min_units = 1;
    while ((double)min_units * min_units < piece_steps * (double)p.k_blocks) min_units++;
    const int grid = (int)std::min<int64_t>(c->sm_count, std::max<int64_t>(1, units / min_units));
    p.unit_q = (int)(units / grid);
    p.unit_r = (int)(units % grid);
    if (!c->d_gemm_partial) {
        const int rc = refuse_allocation_while_recording(c, s, "the GEMM's piece buffers");
        if (rc != WF_OK) return rc;
        WF_CUDA(c, cudaMalloc(&c->d_gemm_partial, (size_t)c->sm_count * GEMM_PIECE_TOKENS * GEMM_BN * sizeof(float)));
        WF_CUDA(c, cudaMalloc(&c->d_gemm_ready, ((size_t)c->sm_count * 4 + 2) * sizeof(unsigned int)));
        WF_CUDA(c, cudaMemset(c->d_gemm_ready, 0, ((size_t)c->sm_count * 4 + 2) * sizeof(unsigned int)));
    }
    p.partial = c->d_gemm_partial;
    p.ready = c->d_gemm_ready;
    p.gen = c->d_gemm_ready + (size_t)c->sm_count * 4;
    const size_t smem = 1024 + (size_t)p.stages * stage_bytes;
    cudaError_t e = qt == WF_QTYPE_Q4_0   ? gemm_launch_one<WF_QTYPE_Q4_0>(p, map, grid, smem, s)
                    : qt == WF_QTYPE_Q4_1 ? gemm_launch_one<WF_QTYPE_Q4_1>(p, map, grid, smem, s)
                    : qt == WF_QTYPE_Q8_0 ? gemm_launch_one<WF_QTYPE_Q8_0>(p, map, grid, smem, s)
                                          : gemm_launch_one<WF_QTYPE_Q4_K>(p, map, grid, smem, s);
    if (e != cudaSuccess) return cuda_status(c, e, "gemm launch");
    c->launches++;
    return WF_OK;
}

}  // namespace wf
