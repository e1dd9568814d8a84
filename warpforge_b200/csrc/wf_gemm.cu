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
// Stages hold BK = 128 k: A = 128 rows x 128 k fp16 (two 64-k swizzle spans, 32 KB), B = BM x 128 k bf16.
// The accumulator is double buffered in TMEM (2 x BM columns <= 512) so the epilogue of one tile
// overlaps the main loop of the next.
//
// Work split ("stream-K"): all (tile, k-block) steps form one sequence in tile order, cut into
// equal contiguous shares, one per CTA, so every SM does the same number of MMA steps whatever the
// tile count.  A tile cut by a share boundary is finished by the CTA that holds its first
// k-block: the CTAs holding the rest reach their piece first (it is the head of their share),
// write it to a scratch buffer and publish the launch number; the owner reaches the tile last,
// adds the pieces in CTA order (deterministic) and writes y.  The owner's wait is bounded.  Every wait is bounded; on expiry the CTA sets a status bit,
// stops issuing work and still frees its TMEM.
//
// Weights are rounded once to fp16 (relative 2^-12) after the exact fp32 dequantization; products
// and sums are fp32 in the tensor core.  Replaces the host transpose + batch_matmul_f32 of
// warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/ops/DotGeneralKernel.java:169-298.
#include <cuda.h>
#include <cuda_fp16.h>

#include "wf_common.cuh"

namespace wf {

constexpr int GEMM_BN = 128;        // weight rows per tile (UMMA M)
constexpr int GEMM_BK = 128;        // k per stage
constexpr int GEMM_THREADS = 448;   // 14 warps: TMA, MMA, 4 epilogue, 8 dequant
constexpr int GEMM_WAIT_SPINS = 1 << 26;
constexpr int GEMM_A_BYTES = GEMM_BN * GEMM_BK * 2;  // 32 KB

struct GemmParams {
    const uint8_t* tiles;
    float* y;
    const float* row_unscale;  // [m] power of two that undoes the pre-pass scaling of token row m
    int* status;
    int64_t ldy, col0;
    int rows, k, kt_w;   // kt_w: weight k-tiles per row-tile stripe (tile_k of the format)
    int m;               // tokens
    int bm;              // tokens per tile (multiple of 16, <= 256)
    int n_tiles, m_tiles, k_blocks;  // k_blocks = ceil(k / 128)
    int stages;
    uint32_t idesc;
    // stream-K: the (tile, k-block) units form one sequence, CTA b owns units [b*q + min(b,r), ...)
    int unit_q, unit_r;
    float* partial;        // [ctas][bm][128] fp32: a CTA's piece of a tile that begins in an earlier CTA
    unsigned int* ready;   // [ctas][4] launch number whose piece (per 32-row quarter) is complete in `partial`
    unsigned int launch;   // this launch's number (never 0)
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
    uint4 c[2];
    uint2 sc[2];
    __device__ __forceinline__ void load(const uint8_t* tile, int kb, int lane) {
        (void)kb;
        const int g = lane >> 2;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            c[h] = __ldg(reinterpret_cast<const uint4*>(tile + h * 512 + lane * 16));
            sc[h] = __ldg(reinterpret_cast<const uint2*>(tile + Tile<WF_QTYPE_Q4_0>::SCALE_OFF + g * 16 + h * 8));
        }
    }
    __device__ __forceinline__ void store(uint8_t* a_stage, int rt16, int lane) const {
        const int g = lane >> 2, q = lane & 3;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const __half2 s01 = as_half2(sc[h].x), s23 = as_half2(sc[h].y);  // block scales 0..3 of this row, fp16
            const __half2 s[4] = {__low2half2(s01), __high2half2(s01), __low2half2(s23), __high2half2(s23)};
            const uint32_t w[4] = {c[h].x, c[h].y, c[h].z, c[h].w};
            const int r = rt16 * 16 + g + 8 * h;
#pragma unroll
            for (int j = 0; j < 4; j++)  // value = s * (code - 8)
                *reinterpret_cast<uint4*>(a_stage + a_chunk_off(r, j * 4 + q)) = word_to_half8_q4_0(w[j], s[j]);
        }
    }
};

template <> struct DequantRegs<WF_QTYPE_Q4_1> {
    uint4 c[2];
    uint2 sc[2], mn[2];
    __device__ __forceinline__ void load(const uint8_t* tile, int kb, int lane) {
        (void)kb;
        using T = Tile<WF_QTYPE_Q4_1>;
        const int g = lane >> 2;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            c[h] = __ldg(reinterpret_cast<const uint4*>(tile + h * 512 + lane * 16));
            sc[h] = __ldg(reinterpret_cast<const uint2*>(tile + T::SCALE_OFF + g * 16 + h * 8));
            mn[h] = __ldg(reinterpret_cast<const uint2*>(tile + T::MIN_OFF + g * 16 + h * 8));
        }
    }
    __device__ __forceinline__ void store(uint8_t* a_stage, int rt16, int lane) const {
        const int g = lane >> 2, q = lane & 3;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const float2 s01 = __half22float2(as_half2(sc[h].x)), s23 = __half22float2(as_half2(sc[h].y));
            const float2 m01 = __half22float2(as_half2(mn[h].x)), m23 = __half22float2(as_half2(mn[h].y));
            const float a[4] = {s01.x, s01.y, s23.x, s23.y}, b[4] = {m01.x, m01.y, m23.x, m23.y};
            const uint32_t w[4] = {c[h].x, c[h].y, c[h].z, c[h].w};
            const int r = rt16 * 16 + g + 8 * h;
#pragma unroll
            for (int j = 0; j < 4; j++)  // value = scale * code + min in fp32, rounded once to fp16
                *reinterpret_cast<uint4*>(a_stage + a_chunk_off(r, j * 4 + q)) = word_to_half8(w[j], a[j], b[j]);
        }
    }
};

template <> struct DequantRegs<WF_QTYPE_Q8_0> {
    uint4 ch[2], cl[2];
    uint2 sc[2];
    __device__ __forceinline__ void load(const uint8_t* tile, int kb, int lane) {
        (void)kb;
        const int g = lane >> 2;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            ch[h] = __ldg(reinterpret_cast<const uint4*>(tile + h * 512 + lane * 16));
            cl[h] = __ldg(reinterpret_cast<const uint4*>(tile + PLANE_BYTES + h * 512 + lane * 16));
            sc[h] = __ldg(reinterpret_cast<const uint2*>(tile + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + g * 16 + h * 8));
        }
    }
    __device__ __forceinline__ void store(uint8_t* a_stage, int rt16, int lane) const {
        const int g = lane >> 2, q = lane & 3;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const __half2 s01 = as_half2(sc[h].x), s23 = as_half2(sc[h].y);
            const __half2 s[4] = {__low2half2(s01), __high2half2(s01), __low2half2(s23), __high2half2(s23)};
            const uint32_t wh[4] = {ch[h].x, ch[h].y, ch[h].z, ch[h].w}, wl[4] = {cl[h].x, cl[h].y, cl[h].z, cl[h].w};
            const int r = rt16 * 16 + g + 8 * h;
#pragma unroll
            for (int j = 0; j < 4; j++)
                *reinterpret_cast<uint4*>(a_stage + a_chunk_off(r, j * 4 + q)) = words_to_half8_q8(wh[j], wl[j], s[j]);
        }
    }
};

template <> struct DequantRegs<WF_QTYPE_Q4_K> {  // the stage is one half (plane kb & 1) of a 256-k tile
    uint4 c[2];
    uint32_t dd[2], scw[2], mnw[2];
    __device__ __forceinline__ void load(const uint8_t* tile, int kb, int lane) {
        using T = Tile<WF_QTYPE_Q4_K>;
        const int g = lane >> 2, pl = kb & 1;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            c[h] = __ldg(reinterpret_cast<const uint4*>(tile + pl * PLANE_BYTES + h * 512 + lane * 16));
            dd[h] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::D_OFF + g * 8 + h * 4));
            scw[h] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::SC_OFF + g * 16 + h * 8 + pl * 4));
            mnw[h] = __ldg(reinterpret_cast<const uint32_t*>(tile + T::MN_OFF + g * 16 + h * 8 + pl * 4));
        }
    }
    __device__ __forceinline__ void store(uint8_t* a_stage, int rt16, int lane) const {
        const int g = lane >> 2, q = lane & 3;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const float2 d = __half22float2(as_half2(dd[h]));  // (d, dmin)
            const uint32_t w[4] = {c[h].x, c[h].y, c[h].z, c[h].w};
            const int r = rt16 * 16 + g + 8 * h;
#pragma unroll
            for (int j = 0; j < 4; j++) {  // value = (d * sc) * code - dmin * m
                const float a = d.x * (float)((scw[h] >> (8 * j)) & 0xFF), b = -(d.y * (float)((mnw[h] >> (8 * j)) & 0xFF));
                *reinterpret_cast<uint4*>(a_stage + a_chunk_off(r, j * 4 + q)) = word_to_half8(w[j], a, b);
            }
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
    const uint32_t b_bytes = (uint32_t)p.bm * 256;
    const uint32_t stage_bytes = GEMM_A_BYTES + b_bytes;
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
            g_mbar_init(&a_full[s], 8);   // eight dequant warps
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
            int it = 0;
            for (int u = u0; u < u1 && !*abort_flag;) {
                const GemmSegment g = segment_at(p, u, u1);
                const int mt = g.tile % p.m_tiles;
                for (int kb = g.kb0; kb < g.kb1; kb++, it++) {
                    const int s = it % stages;
                    if (it >= stages && !g_mbar_wait(&s_empty[s], ((it / stages) - 1) & 1)) { fail(); break; }
                    uint8_t* b_stage = stage0 + (size_t)s * stage_bytes + GEMM_A_BYTES;
                    g_mbar_expect_tx(&b_full[s], b_bytes);
                    tma_load_2d(b_stage, &xmap, kb * GEMM_BK, mt * p.bm, &b_full[s]);
                    tma_load_2d(b_stage + b_bytes / 2, &xmap, kb * GEMM_BK + 64, mt * p.bm, &b_full[s]);
                }
                u += g.kb1 - g.kb0;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
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
                    const uint32_t b_addr = a_addr + GEMM_A_BYTES;
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
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;  // weight row inside the 128-row block
        int local = 0;
        for (int u = u0; u < u1 && !*abort_flag; local++) {
            const GemmSegment g = segment_at(p, u, u1);
            const int buf = local & 1;
            const int nt = g.tile / p.m_tiles, mt = g.tile % p.m_tiles;
            if (!g_mbar_wait(&acc_full[buf], (local >> 1) & 1)) { if (lane == 0) fail(); break; }
            tc_fence_after();
            const int n = nt * GEMM_BN + row;
            const bool starts = g.kb0 == 0, ends = g.kb1 == p.k_blocks;
            // Owner of a tile that continues in the following CTAs: their pieces must be complete.
            // They were computed at the head of those CTAs' shares, long before this tail of mine.
            int last_cta = (int)blockIdx.x;
            if (starts && !ends) {
                const int tile_end = (g.tile + 1) * p.k_blocks;
                bool gave_up = false;
                for (int c = (int)blockIdx.x + 1; c < (int)gridDim.x; c++) {
                    int c0, c1;
                    cta_units(p, c, c0, c1);
                    if (c0 >= tile_end) break;
                    if (c0 == c1) continue;
                    last_cta = c;
                    int spins = 0;  // the same quarter of the other CTA wrote the rows this warp is going to add
                    while (ld_acquire_u32(p.ready + c * 4 + quarter) != p.launch && ++spins < GEMM_WAIT_SPINS) __nanosleep(64);
                    if (spins >= GEMM_WAIT_SPINS) gave_up = true;
                }
                if (gave_up) { if (lane == 0) fail(); break; }
            }
            // room for 256 tokens per CTA: columns are moved 32 at a time, also past a BM that is not a multiple of 32
            float* mine = p.partial + (size_t)blockIdx.x * 256 * GEMM_BN;
            for (int c = 0; c < p.bm; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * p.bm + c), r);
                const int m0 = mt * p.bm + c;
                if (!starts) {  // my piece of a tile owned by an earlier CTA: token-major, 128 rows contiguous
#pragma unroll
                    for (int j = 0; j < 32; j++) mine[(size_t)(c + j) * GEMM_BN + row] = __uint_as_float(r[j]);
                    continue;
                }
                for (int cc = (int)blockIdx.x + 1; cc <= last_cta; cc++) {  // pieces in CTA order
                    int c0, c1;
                    cta_units(p, cc, c0, c1);
                    if (c0 == c1) continue;
                    const float* piece = p.partial + (size_t)cc * 256 * GEMM_BN;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldcg(piece + (size_t)(c + j) * GEMM_BN + row));
                }
                if (n < p.rows) {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (m0 + j < p.m)
                            p.y[(int64_t)(m0 + j) * p.ldy + p.col0 + n] = __uint_as_float(r[j]) * __ldg(p.row_unscale + m0 + j);
                }
            }
            tc_fence_before();
            if (!starts) {  // publish this warp's 32 rows of the piece
                __threadfence();
                __syncwarp();
                if (lane == 0) st_release_u32(p.ready + blockIdx.x * 4 + quarter, p.launch);
            }
            __syncwarp();
            if (lane == 0) g_mbar_arrive(&acc_empty[buf]);
            u += g.kb1 - g.kb0;
        }
    } else {
        // ------------------------------------------------ dequant warps 2, 3, 8..13: one 16-row tile each per stage
        const int dq = (warp < 4) ? warp - 2 : warp - 6;  // 0..7 = 16-row tile inside the 128-row block
        // weight tile of unit u (tile-major, k-block minor), this warp's 16-row tile of the 128-row block
        auto weight_tile = [&](int u) {
            const int tile = u / p.k_blocks, kb = u - tile * p.k_blocks;
            const int64_t wrt = (int64_t)(tile / p.m_tiles) * (GEMM_BN / 16) + dq;
            return p.tiles + (wrt * p.kt_w + kb / KB_PER_WTILE) * (int64_t)TILE_BYTES;
        };
        // one step: wait for the stage, convert the registers loaded one step ago, hand the stage over
        auto finish_step = [&](const DequantRegs<QT>& regs, int it) {
            const int s = it % stages;
            if (it >= stages && !g_mbar_wait(&s_empty[s], ((it / stages) - 1) & 1)) {
                if (lane == 0) fail();
                return false;
            }
            regs.store(stage0 + (size_t)s * stage_bytes, dq, lane);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) g_mbar_arrive(&a_full[s]);
            return true;
        };
        // two register sets in turn: the loads of step u + 1 are in flight while step u is converted
        DequantRegs<QT> ra, rb;
        int it = 0;
        if (u0 < u1) ra.load(weight_tile(u0), u0 % p.k_blocks, lane);
        for (int u = u0; u < u1 && !*abort_flag; u += 2, it += 2) {
            if (u + 1 < u1) rb.load(weight_tile(u + 1), (u + 1) % p.k_blocks, lane);
            if (!finish_step(ra, it)) break;
            if (u + 1 >= u1) break;
            if (u + 2 < u1) ra.load(weight_tile(u + 2), (u + 2) % p.k_blocks, lane);
            if (!finish_step(rb, it + 1)) break;
        }
    }

    // ------------------------------------------------ teardown: TMEM is freed on every path
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
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
    // bf16 activations, more than the GEMV's 8 tokens; K a multiple of 8 elements and a 16-byte aligned activation
    // pointer (the pre-pass reads 16-byte pieces, the TMA row stride must be a multiple of 16 bytes).  Whole
    // 128-row blocks exist for any row count: the weight buffer is padded to 8 row-tiles with zero scales.
    return x_dtype == WF_DTYPE_BF16 && m > 8 && (w.g.k % 8) == 0 && (reinterpret_cast<uintptr_t>(d_x) & 15) == 0 &&
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
    gemm_kernel<QT><<<grid, GEMM_THREADS, smem, s>>>(p, map);
    return cudaGetLastError();
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
    p.bm = call.m >= 256 ? 256 : (int)((call.m + 15) / 16 * 16);
    p.n_tiles = (int)((w.g.rows + GEMM_BN - 1) / GEMM_BN);
    p.m_tiles = (int)((call.m + p.bm - 1) / p.bm);
    p.k_blocks = (int)((w.g.k + GEMM_BK - 1) / GEMM_BK);
    const size_t stage_bytes = GEMM_A_BYTES + (size_t)p.bm * 256;
    p.stages = (int)std::min<size_t>((GEMM_SMEM_LIMIT - 1024) / stage_bytes, 8);
    // A = fp16 weights, B = fp16 activations, D = fp32; both operands K-major
    p.idesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(p.bm >> 3) << 17) | ((uint32_t)(GEMM_BN >> 4) << 24);

    // the last 128-row block may reach past the padded row-tiles: the weight buffer must cover it
    if ((int64_t)p.n_tiles * (GEMM_BN / 16) > w.g.rt_alloc)
        return set_error(c, WF_ERR_SHAPE, "weight buffer does not cover the last 128-row block");

    // activation pre-pass into the context's fp16 scratch (grown on demand)
    const int64_t x16_bytes = ((call.m * w.g.k * 2 + 255) & ~255LL) + call.m * 4;
    if (x16_bytes > c->x16_bytes) {
        if (c->d_x16) cudaFree(c->d_x16);
        c->d_x16 = nullptr;
        c->x16_bytes = 0;
        WF_CUDA(c, cudaMalloc(&c->d_x16, (size_t)x16_bytes));
        c->x16_bytes = x16_bytes;
    }
    __half* x16 = static_cast<__half*>(c->d_x16);
    float* unscale = reinterpret_cast<float*>(static_cast<uint8_t*>(c->d_x16) + ((call.m * w.g.k * 2 + 255) & ~255LL));
    x_to_f16_kernel<<<(unsigned)call.m, XPRE_THREADS, 0, s>>>(static_cast<const uint16_t*>(call.d_x), x16, unscale, (int)w.g.k);
    WF_CUDA(c, cudaGetLastError());
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
    const int grid = (int)std::min<int64_t>(c->sm_count, units);
    p.unit_q = (int)(units / grid);
    p.unit_r = (int)(units % grid);
    if (!c->d_gemm_partial) {
        WF_CUDA(c, cudaMalloc(&c->d_gemm_partial, (size_t)c->sm_count * 256 * GEMM_BN * sizeof(float)));
        WF_CUDA(c, cudaMalloc(&c->d_gemm_ready, (size_t)c->sm_count * 4 * sizeof(unsigned int)));
        WF_CUDA(c, cudaMemset(c->d_gemm_ready, 0, (size_t)c->sm_count * 4 * sizeof(unsigned int)));
    }
    p.partial = c->d_gemm_partial;
    p.ready = c->d_gemm_ready;
    if (++c->gemm_launches == 0) c->gemm_launches = 1;  // 0 means "nothing published"
    p.launch = c->gemm_launches;
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
