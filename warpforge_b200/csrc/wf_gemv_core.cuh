// Device-side building blocks of the decode kernels (wf_gemv.cu, wf_gemv_stream.cuh, wf_gemv_multi.cuh, wf_decode.cu):
// the per-format tile code (loads into registers, the one-token integer arithmetic on activation digits, the
// several-token bf16 arithmetic), the activation staging, the exchange of cut row-tiles between CTAs, and -- for
// the several-token program kernel only -- the shared-memory ring primitives and the walk over a CTA's share of a
// weight (producer and consumer side, segment reduction).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#include <algorithm>

#include "wf_common.cuh"

namespace wf {

constexpr int GEMV_WARPS = 16;                       // consumer warps
constexpr int GEMV_CONSUMERS = GEMV_WARPS * 32;
constexpr int GEMV_THREADS = (GEMV_WARPS + 1) * 32;  // + one producer warp
constexpr int GEMV_MAX_STAGES = 16;
// Ring depth actually used: measured on the decode shapes, 3-4 stages of 18 KB in flight per SM beat
// deeper rings by 7 % (more copies in flight only queue up in the memory system).
constexpr int GEMV_USE_STAGES = 4;
constexpr int GEMV_BAR_SPINS = 1 << 24;
constexpr int GEMV_XCOLS = 8;  // columns of one mma n-tile
constexpr int GEMV_FIXUP_SPINS = 1 << 22;
constexpr int GEMV_SLOT_SPINS = 1 << 24;
constexpr int GEMV_MAX_SLOTS = 8;  // partial-sum slots a CTA rotates through
// CTAs that share a weight of `tiles` tiles: one per SM, but never fewer than two ring rounds of tiles per CTA -- a
// small weight cut into 148 shares would spend its time in the fix-up between the CTAs that share a row-tile,
// not in reading its bytes.
inline int gemv_ctas(int sm_count, int64_t tiles) {
    const int64_t by_work = tiles / (2 * GEMV_WARPS);
    return (int)std::min<int64_t>(sm_count, std::max<int64_t>(1, by_work));
}
// control block: abort flag | full[MAX_STAGES] | empty[MAX_STAGES] | done[MAX_SLOTS] | vacant[MAX_SLOTS]
constexpr int GEMV_CTRL_BYTES = 128 + (2 * GEMV_MAX_STAGES + 2 * GEMV_MAX_SLOTS) * 8;
// XC = 1: one live column; XC = 8: up to 8.  N partial-sum slots of [GEMV_WARPS][ELEMS] floats.
template <int XC> struct Slots { static constexpr int N = (XC == 1) ? 8 : 4, ELEMS = 16 * XC; };

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
    int aligned;           // one-token kernel: 1 = chunk_q / chunk_r count whole row-tiles (no row-tile is cut between CTAs)
    unsigned long long* timing;  // optional [ctas][8] globaltimer stamps (instrumented launches only)
};

// ---------------------------------------------------------------- small device helpers
// shared-memory loads by 32-bit shared address (no generic-pointer arithmetic in the hot loop)
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint32_t v;
    asm volatile("{\n\t.reg .b16 h;\n\tld.shared.u16 h, [%1];\n\tcvt.u32.u16 %0, h;\n\t}" : "=r"(v) : "r"(a));
    return v;
}
// Streaming loads of weight tiles straight from global memory (read-only for the kernel's lifetime, no reuse:
// not kept in L1).  A warp's 16-byte loads of a plane half cover 512 contiguous bytes.
// The byte offset OFF is an immediate of the load: several loads off one lane pointer cost no address arithmetic.
template <int OFF> __device__ __forceinline__ uint4 ldg128_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ uint2 ldg64_stream(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "l"(p), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ uint32_t ldg32_stream(const uint8_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1+%2];" : "=r"(v) : "l"(p), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ uint32_t ldg16_stream(const uint8_t* p) {
    uint32_t v;
    asm volatile("{\n\t.reg .b16 h;\n\tld.global.nc.L1::no_allocate.u16 h, [%1+%2];\n\tcvt.u32.u16 %0, h;\n\t}" : "=r"(v) : "l"(p), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ uint4 lds128_at(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF));
    return v;
}
// 16-byte load by the lanes whose `pred` is non-zero; the other lanes keep what `v` held.
__device__ __forceinline__ void lds128_if(uint4& v, uint32_t a, uint32_t pred) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "r"(a), "r"(pred));
}
// Several tokens (XC = 8): per 32-k block the B fragment (8 activations of this lane's column, 16 bytes)
// and the lane's float4 of accumulator start values.
template <int XC>
__device__ __forceinline__ void fetch_block(uint32_t xaddr, uint32_t caddr, uint32_t live, uint4& xb, float4& ci) {
    (void)live;
    xb = lds128(xaddr);
    const uint4 t = lds128(caddr);
    ci = make_float4(__uint_as_float(t.x), __uint_as_float(t.y), __uint_as_float(t.z), __uint_as_float(t.w));
}
// Bytes per block in the start-value table of the several-token path: [4] float4.
template <int XC> __device__ __forceinline__ constexpr int cinit_block_bytes() { return 64; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// Barriers are addressed by their 32-bit shared-memory address throughout: no generic-pointer
// arithmetic or address-space conversion in the hot loops.
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive from the lanes whose `pred` is non-zero, without a branch
__device__ __forceinline__ void mbar_arrive_if(uint32_t bar, uint32_t pred) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %1, 0;\n\t@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" ::"r"(bar),
        "r"(pred)
        : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// The hot-loop form: one try_wait and a branch when the phase is already complete.  Otherwise spin,
// bounded, and leave early once any thread of the CTA has raised the abort word (shared address
// `abort32`); a wait that runs out raises it.  After an abort the data the caller goes on to use is
// garbage -- the kernel reports the failure through its status word and the host discards y.
__device__ __forceinline__ void mbar_wait_or_abort(uint32_t bar, uint32_t parity, uint32_t abort32) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .u32 n, a;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n\t"
        "@p bra WF_OK_%=;\n\t"
        "mov.u32 n, 0;\n\t"
        "WF_SPIN_%=:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n\t"
        "@p bra WF_OK_%=;\n\t"
        "ld.volatile.shared.u32 a, [%2];\n\t"
        "setp.ne.u32 q, a, 0;\n\t"
        "@q bra WF_OK_%=;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 q, n, %3;\n\t"
        "@q bra WF_SPIN_%=;\n\t"
        "st.volatile.shared.u32 [%2], 1;\n\t"
        "WF_OK_%=:\n\t"
        "}\n" ::"r"(bar),
        "r"(parity), "r"(abort32), "r"((uint32_t)GEMV_BAR_SPINS)
        : "memory");
}
// After an abort: give this CTA's bulk copies still in flight time to land before its shared memory
// is handed to another CTA (about a millisecond, bounded).
__device__ __forceinline__ void drain_after_abort() {
    for (int i = 0; i < 1000; i++) __nanosleep(1000);
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
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

// The A fragments of one 32-k block alone (what block_mma builds before its two MMAs): a[0..3] feed the MMA over
// elements 0..15 of the block, a[4..7] the one over elements 16..31.  For kernels that multiply one block of
// weights with several groups of eight columns.
__device__ __forceinline__ void unpack8(uint32_t (&a)[8], uint32_t wg, uint32_t wh, uint32_t magic) {
    asm("{\n\t"
        ".reg .b32 g1, g2, g3, h1, h2, h3;\n\t"
        "shf.r.wrap.b32 g1, %8, %8, 4;\n\t"
        "shf.r.wrap.b32 h1, %9, %9, 4;\n\t"
        "shf.r.wrap.b32 g2, %8, %8, 8;\n\t"
        "shf.r.wrap.b32 h2, %9, %9, 8;\n\t"
        "shf.r.wrap.b32 g3, %8, %8, 12;\n\t"
        "shf.r.wrap.b32 h3, %9, %9, 12;\n\t"
        "lop3.b32 %0, %8, %10, %11, 0xEA;\n\t"
        "lop3.b32 %1, %9, %10, %11, 0xEA;\n\t"
        "lop3.b32 %2, g1, %10, %11, 0xEA;\n\t"
        "lop3.b32 %3, h1, %10, %11, 0xEA;\n\t"
        "lop3.b32 %4, g2, %10, %11, 0xEA;\n\t"
        "lop3.b32 %5, h2, %10, %11, 0xEA;\n\t"
        "lop3.b32 %6, g3, %10, %11, 0xEA;\n\t"
        "lop3.b32 %7, h3, %10, %11, 0xEA;\n\t"
        "}\n"
        : "=&r"(a[0]), "=&r"(a[1]), "=&r"(a[2]), "=&r"(a[3]), "=&r"(a[4]), "=&r"(a[5]), "=&r"(a[6]), "=&r"(a[7])
        : "r"(wg), "r"(wh), "r"(0x00780078u), "r"(magic));
}
// One block against one group of eight columns: d = c + A . B over the 32 k of the block.
__device__ __forceinline__ void block_mma_pre(float (&d)[4], const uint32_t (&a)[8], const uint4& xb, float c0, float c1, float c2, float c3) {
    mma_bf16(d, a[0], a[1], a[2], a[3], xb.x, xb.y, c0, c1, c2, c3);
    mma_bf16(d, a[4], a[5], a[6], a[7], xb.z, xb.w, d[0], d[1], d[2], d[3]);
}
__device__ __forceinline__ float2 lds64f(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}

// ---- one token: integer MMAs, the eight accumulator columns = two blocks x four activation digits
// With a single bf16 token seven of the eight columns of the B operand would be idle, and turning 4-bit
// codes into bf16 operands costs seven half-rate integer instructions per word of eight codes.  The
// one-token path therefore runs on mma.m16n8k32.s32.u8.s8:
//   * A operand: a plane word AND 0x78787878 is four bytes 8 * code (nibble positions 0, 2, 4, 6 of the
//     rotated word sit in bits 3..6 of the four bytes); a rotation by 4 bits gives the other four codes.
//     Three integer instructions per word, no layout change.
//   * B operand: the activations of a 32-k block are written as x = X * 2^e with one exponent per block
//     and X an integer below 2^30, and X as four signed base-256 digits (exact for every element within
//     2^-22 of the block's largest; smaller ones are cut at 2^-30 of it).  The 32 k-slots of an MMA belong to
//     two different blocks (slots 0..15 / 16..31) and column n = 4 * h + digit holds digit `digit` of
//     block h in that block's slots and zeros elsewhere, so column n of the int32 accumulator is the
//     exact sum over one block and one digit.
//   * After the two MMAs of a block pair lane (g, q) holds, for rows g and g+8, digits 2(q&1), 2(q&1)+1
//     of block (q >> 1) of the pair: D = 256 * D_even + D_odd in integers, one conversion to float, one
//     product with weight scale x block exponent, one FMA into the row's accumulator.
// The constant offset of the codes (8 * (code - 8) wanted, 8 * code multiplied) enters as the int32
// start value -64 * (sum of the block's digits), prepared with the digits.
//
// Staged form of one token, per 128 k (a "unit" = four blocks j = 0..3, block pairs A = (0, 2) and
// B = (1, 3)): 1024 bytes of digits, lane L = 4 g + q reads 32 bytes at L * 32: for pair A and then for pair B
// the words {lo, hi} of the first MMA (elements 0, 4, 1, 5 of the lane's block) and {lo, hi} of the second
// (elements 2, 6, 3, 7), holding digit (g & 3) of elements 8q..8q+7 of block 2 (g >> 2) [pair A] / 2 (g >> 2) + 1
// [pair B].  A lane is a live source for the low k-slots (its block is the pair's first) when g < 4 and for
// the high k-slots otherwise; the word of the other half is zero in shared memory (cleared once per kernel and
// never written), so two plain 16-byte loads deliver the MMA operand pairs in consecutive registers.
// Per unit and lane quad position q = 2 h + p a 16-byte record {W, f, W', f'} for blocks 2h and 2h+1 and
// digit pair p: W = int32 correction beta * (256 * sum of digit 2p + sum of digit 2p+1) that cancels the
// codes' offset, f = 2^e * 256^(2 - 2p) / 8 the factor that turns the integer block sum into the block's
// value; and 8 bytes {sum of x, sum of x'} for p = 0, zeros for p = 1 (formats with a per-block minimum).

constexpr uint32_t CODE8_MASK = 0x78787878u;

// d += (8 * codes) x digits over one block pair: w00 / w10 = rows g / g+8 of the pair's first block,
// w01 / w11 = of its second block; bl = digit bytes for the low k-slots (first MMA, second MMA),
// bh = for the high k-slots.
__device__ __forceinline__ void pair_imma(int (&d)[4], uint32_t w00, uint32_t w10, uint32_t w01, uint32_t w11,
                                          uint32_t bl1, uint32_t bh1, uint32_t bl2, uint32_t bh2, uint32_t mul28) {
    // d = (not +=): the first MMA starts from zero.  bl / bh: digit bytes for the low / high k-slots, first and second MMA.
    // The rotation by four bits for the second MMA goes through the multiplier (w * 2^28 as a 64-bit product:
    // low word w << 28, high word w >> 4) and one three-input logic op ((lo | hi) & mask), which leaves two
    // instead of three instructions per word on the half-rate integer pipe.  mul28 = 2^28, kept in a register the
    // compiler cannot see through (a constant factor would be turned back into shifts).
    asm(
        "{\n\t"
        ".reg .b32 a0, a1, a2, a3, l0, l1, l2, l3, h0, h1, h2, h3;\n\t"
        ".reg .b64 p0, p1, p2, p3;\n\t"
        "and.b32 a0, %4, %12;\n\t"
        "and.b32 a1, %5, %12;\n\t"
        "and.b32 a2, %6, %12;\n\t"
        "and.b32 a3, %7, %12;\n\t"
        "mul.wide.u32 p0, %4, %13;\n\t"
        "mul.wide.u32 p1, %5, %13;\n\t"
        "mul.wide.u32 p2, %6, %13;\n\t"
        "mul.wide.u32 p3, %7, %13;\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {a0,a1,a2,a3}, {%8,%9}, {%14,%14,%14,%14};\n\t"
        "mov.b64 {l0, h0}, p0;\n\t"
        "mov.b64 {l1, h1}, p1;\n\t"
        "mov.b64 {l2, h2}, p2;\n\t"
        "mov.b64 {l3, h3}, p3;\n\t"
        "lop3.b32 a0, l0, h0, %12, 0xA8;\n\t"
        "lop3.b32 a1, l1, h1, %12, 0xA8;\n\t"
        "lop3.b32 a2, l2, h2, %12, 0xA8;\n\t"
        "lop3.b32 a3, l3, h3, %12, 0xA8;\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {a0,a1,a2,a3}, {%10,%11}, {%0,%1,%2,%3};\n\t"
        "}\n"
        : "=&r"(d[0]), "=&r"(d[1]), "=&r"(d[2]), "=&r"(d[3])
        : "r"(w00), "r"(w10), "r"(w01), "r"(w11), "r"(bl1), "r"(bh1), "r"(bl2), "r"(bh2), "r"(CODE8_MASK), "r"(mul28), "r"(0));
}

// Lane-specific shared addresses of the staged token for the tile at hand.
struct Q8Addr {
    uint32_t x;    // this lane's 32 digit bytes of the tile's first unit
    uint32_t rec;  // this lane's record of the tile's first unit
    uint32_t sx;   // this lane's pair of activation sums
};
// The B registers of a warp for one unit: {lo, hi} byte quadruples of the first and second MMA of block pair A (a)
// and of pair B (b).  For a lane that feeds the low k-slots the hi words are zero in shared memory, and vice versa.
struct Q8Digits {
    uint4 a, b;
    uint32_t mul28 = 0x10000000u | (gridDim.y >> 16);  // 2^28 (a grid has fewer than 2^16 CTAs in y), opaque to the compiler
    template <int OFF> __device__ __forceinline__ void load(uint32_t addr) {
        a = lds128_at<OFF>(addr);
        b = lds128_at<OFF + 16>(addr);
    }
};
constexpr int Q8_UNIT_BYTES = 1024;  // staged digits per 128 k: 32 lanes x 32 bytes

// 256 D_even + D_odd as a float (|D| < 2^20 for the 4-bit formats, so the integer is exact and the conversion rounds once)
__device__ __forceinline__ float digits_to_float(int de, int dodd) { return (float)(de * 256 + dodd); }
// the same for sums up to 2^24 (Q8_0: two planes combined), where 256 D would leave 32 bits; w = the offset correction,
// split so that both summands stay below 2^24 and convert exactly (one rounding in the FMA)
__device__ __forceinline__ float wide_digits_to_float(int de, int dodd, int w) {
    return fmaf((float)(de + (w >> 8)), 256.f, (float)(dodd + (w & 255)));
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
    static constexpr int BETA_INT = -64;   // one token: 8 * code - 64 = 8 * (code - 8)
    uint4 c[2], s;
    uint32_t sg2, sh2;  // one token: fp16 scales of blocks 2h, 2h+1 (h = q >> 1) for row g / row g+8
    // t = shared address of the tile + lane * 16
    template <int XC>
    __device__ __forceinline__ void load(uint32_t t, int lane) {
        c[0] = lds128(t);
        c[1] = lds128(t + 512);
        const uint32_t sb = t - lane * 16 + Tile<WF_QTYPE_Q4_0>::SCALE_OFF + (lane >> 2) * 16;
        if (XC == 1) {
            sg2 = lds32(sb + (lane & 2) * 2);
            sh2 = lds32(sb + 8 + (lane & 2) * 2);
        } else {
            s = lds128(sb);
        }
    }
    // one token: the tile straight from global memory into registers.  pc = tile + lane * 16, ps = tile + the lane's
    // scale offset (see lane_scale_offset); OFF = byte offset of the tile from those pointers, an immediate.
    static __device__ __forceinline__ int lane_scale_offset(int lane) { return (lane >> 2) * 16 + (lane & 2) * 2; }
    template <int OFF> __device__ __forceinline__ void load_global(const uint8_t* pc, const uint8_t* ps) {
        c[0] = ldg128_stream<OFF>(pc);
        c[1] = ldg128_stream<OFF + 512>(pc);
        sg2 = ldg32_stream<OFF + Tile<WF_QTYPE_Q4_0>::SCALE_OFF>(ps);
        sh2 = ldg32_stream<OFF + Tile<WF_QTYPE_Q4_0>::SCALE_OFF + 8>(ps);
    }
    // One token: lane (g, q) adds its share of rows g (acc[0]) and g+8 (acc[2]); the four lanes of a quad
    // hold different digit pairs / blocks of the same rows and are summed when the row-tile is flushed.
    // J: the tile's position after the one the addresses point at (immediate offsets).
    template <int J> __device__ __forceinline__ void compute_q8(float (&acc)[4], const Q8Addr& a, Q8Digits& dg) const {
        constexpr int TK = Tile<WF_QTYPE_Q4_0>::K;
        dg.template load<J * (TK / 128) * Q8_UNIT_BYTES>(a.x);
        const uint4 r = lds128_at<J * (TK >> 5) * 16>(a.rec);  // {W, f, W', f'}
        int da[4], db[4];
        pair_imma(da, c[0].x, c[1].x, c[0].z, c[1].z, dg.a.x, dg.a.y, dg.a.z, dg.a.w, dg.mul28);
        pair_imma(db, c[0].y, c[1].y, c[0].w, c[1].w, dg.b.x, dg.b.y, dg.b.z, dg.b.w, dg.mul28);
        const float2 sg = half2_bits_to_float2(sg2), sh = half2_bits_to_float2(sh2);
        const float ea = __uint_as_float(r.y), eb = __uint_as_float(r.w);
        const int wa = (int)r.x, wb = (int)r.z;
        acc[0] = fmaf(sg.x * ea, digits_to_float(da[0], da[1] + wa), acc[0]);
        acc[2] = fmaf(sh.x * ea, digits_to_float(da[2], da[3] + wa), acc[2]);
        acc[0] = fmaf(sg.y * eb, digits_to_float(db[0], db[1] + wb), acc[0]);
        acc[2] = fmaf(sh.y * eb, digits_to_float(db[2], db[3] + wb), acc[2]);
    }
    // Several tokens, register streaming: the tile from global memory (tile = its first byte); NG groups of eight
    // columns; xg[i] = shared address of this lane's column of group i (row + q * 16 bytes) at the slice's first k,
    // xoff = byte offset of the tile's first k in a staged row, caddr = the lane's start values of the tile's first
    // block, group 0 ([block][group][q] float4).
    __device__ __forceinline__ void load_global_n(const uint8_t* tile, int lane) {
        c[0] = ldg128_stream<0>(tile + lane * 16);
        c[1] = ldg128_stream<512>(tile + lane * 16);
        s = ldg128_stream<Tile<WF_QTYPE_Q4_0>::SCALE_OFF>(tile + (lane >> 2) * 16);
    }
    template <int NG>
    __device__ __forceinline__ void compute_n(float (&acc)[NG][4], const uint32_t (&xg)[NG], uint32_t xoff, uint32_t caddr) const {
        const float2 s0 = half2_bits_to_float2(s.x), s1 = half2_bits_to_float2(s.y);
        const float2 s2 = half2_bits_to_float2(s.z), s3 = half2_bits_to_float2(s.w);
        const float sg[4] = {s0.x, s0.y, s1.x, s1.y}, sh[4] = {s2.x, s2.y, s3.x, s3.y};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t a[8];
            unpack8(a, word_of(c[0], j), word_of(c[1], j), MAGIC_16);
#pragma unroll
            for (int gi = 0; gi < NG; gi++) {
                const uint4 xb = lds128(xg[gi] + xoff + j * 64);
                const float2 ci = lds64f(caddr + (j * NG + gi) * 32);
                float d[4];
                block_mma_pre(d, a, xb, ci.x, ci.y, ci.x, ci.y);
                acc[gi][0] = fmaf(sg[j], d[0], acc[gi][0]);
                acc[gi][2] = fmaf(sh[j], d[2], acc[gi][2]);
                acc[gi][1] = fmaf(sg[j], d[1], acc[gi][1]);
                acc[gi][3] = fmaf(sh[j], d[3], acc[gi][3]);
            }
        }
    }
    template <int XC>
    // xaddr: shared address of this lane's activations for k = kbase (row + q * 16 bytes);
    // caddr: shared address of the start value(s) of block kbase / 32; live: lane owns a live column
    __device__ __forceinline__ void compute(float (&acc)[4], uint32_t xaddr, uint32_t caddr, uint32_t live) const {
        const float2 s0 = half2_bits_to_float2(s.x), s1 = half2_bits_to_float2(s.y);  // row g, blocks 0..3
        const float2 s2 = half2_bits_to_float2(s.z), s3 = half2_bits_to_float2(s.w);  // row g + 8
        const float sg[4] = {s0.x, s0.y, s1.x, s1.y}, sh[4] = {s2.x, s2.y, s3.x, s3.y};
        uint4 xb;
        float4 ci;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            fetch_block<XC>(xaddr + j * 64, caddr + j * cinit_block_bytes<XC>(), live, xb, ci);
            float d[4];
            block_mma(d, word_of(c[0], j), word_of(c[1], j), xb, MAGIC_16, ci.x, ci.y, ci.z, ci.w);
            acc[0] = fmaf(sg[j], d[0], acc[0]);
            acc[2] = fmaf(sh[j], d[2], acc[2]);
            acc[1] = fmaf(sg[j], d[1], acc[1]);
            acc[3] = fmaf(sh[j], d[3], acc[3]);
        }
    }
};

template <> struct TileRegs<WF_QTYPE_Q4_1> {
    static constexpr float BETA = -16.f;  // (16 + code) - 16 = code; the min term is (-min / 16) * (start value)
    static constexpr int BETA_INT = 0;    // one token: codes are unsigned, nothing to cancel
    uint4 c[2], s, mn;
    uint32_t sg2, sh2, mg2, mh2;  // one token: fp16 scales and mins of blocks 2h, 2h+1 (h = q >> 1) for row g / row g+8
    template <int XC>
    __device__ __forceinline__ void load(uint32_t t, int lane) {
        using T = Tile<WF_QTYPE_Q4_1>;
        c[0] = lds128(t);
        c[1] = lds128(t + 512);
        const uint32_t sb = t - lane * 16 + T::SCALE_OFF + (lane >> 2) * 16;
        const uint32_t mb = t - lane * 16 + T::MIN_OFF + (lane >> 2) * 16;
        if (XC == 1) {
            sg2 = lds32(sb + (lane & 2) * 2);
            sh2 = lds32(sb + 8 + (lane & 2) * 2);
            mg2 = lds32(mb + (lane & 2) * 2);
            mh2 = lds32(mb + 8 + (lane & 2) * 2);
        } else {
            s = lds128(sb);
            mn = lds128(mb);
        }
    }
    // one token: the tile straight from global memory into registers (pointers and OFF as for Q4_0)
    static __device__ __forceinline__ int lane_scale_offset(int lane) { return (lane >> 2) * 16 + (lane & 2) * 2; }
    template <int OFF> __device__ __forceinline__ void load_global(const uint8_t* pc, const uint8_t* ps) {
        using T = Tile<WF_QTYPE_Q4_1>;
        c[0] = ldg128_stream<OFF>(pc);
        c[1] = ldg128_stream<OFF + 512>(pc);
        sg2 = ldg32_stream<OFF + T::SCALE_OFF>(ps);
        sh2 = ldg32_stream<OFF + T::SCALE_OFF + 8>(ps);
        mg2 = ldg32_stream<OFF + T::MIN_OFF>(ps);
        mh2 = ldg32_stream<OFF + T::MIN_OFF + 8>(ps);
    }
    // One token: 8 * code enters the MMA as is (no offset); the min term is min * (sum of the block's
    // activations), which only the lanes of the first digit pair carry (the others read zeros).
    template <int J> __device__ __forceinline__ void compute_q8(float (&acc)[4], const Q8Addr& a, Q8Digits& dg) const {
        constexpr int TK = Tile<WF_QTYPE_Q4_1>::K;
        dg.template load<J * (TK / 128) * Q8_UNIT_BYTES>(a.x);
        const uint4 r = lds128_at<J * (TK >> 5) * 16>(a.rec);
        const uint2 sx = lds64(a.sx + J * (TK >> 5) * 8);
        int da[4], db[4];
        pair_imma(da, c[0].x, c[1].x, c[0].z, c[1].z, dg.a.x, dg.a.y, dg.a.z, dg.a.w, dg.mul28);
        pair_imma(db, c[0].y, c[1].y, c[0].w, c[1].w, dg.b.x, dg.b.y, dg.b.z, dg.b.w, dg.mul28);
        const float2 sg = half2_bits_to_float2(sg2), sh = half2_bits_to_float2(sh2);
        const float2 mg = half2_bits_to_float2(mg2), mh = half2_bits_to_float2(mh2);
        const float ea = __uint_as_float(r.y), eb = __uint_as_float(r.w);
        const float xa = __uint_as_float(sx.x), xb = __uint_as_float(sx.y);
        acc[0] = fmaf(sg.x * ea, digits_to_float(da[0], da[1]), fmaf(mg.x, xa, acc[0]));
        acc[2] = fmaf(sh.x * ea, digits_to_float(da[2], da[3]), fmaf(mh.x, xa, acc[2]));
        acc[0] = fmaf(sg.y * eb, digits_to_float(db[0], db[1]), fmaf(mg.y, xb, acc[0]));
        acc[2] = fmaf(sh.y * eb, digits_to_float(db[2], db[3]), fmaf(mh.y, xb, acc[2]));
    }
    __device__ __forceinline__ void load_global_n(const uint8_t* tile, int lane) {
        using T = Tile<WF_QTYPE_Q4_1>;
        c[0] = ldg128_stream<0>(tile + lane * 16);
        c[1] = ldg128_stream<512>(tile + lane * 16);
        s = ldg128_stream<T::SCALE_OFF>(tile + (lane >> 2) * 16);
        mn = ldg128_stream<T::MIN_OFF>(tile + (lane >> 2) * 16);
    }
    template <int NG>
    __device__ __forceinline__ void compute_n(float (&acc)[NG][4], const uint32_t (&xg)[NG], uint32_t xoff, uint32_t caddr) const {
        const float2 s0 = half2_bits_to_float2(s.x), s1 = half2_bits_to_float2(s.y);
        const float2 s2 = half2_bits_to_float2(s.z), s3 = half2_bits_to_float2(s.w);
        const float2 m0 = half2_bits_to_float2(mn.x), m1 = half2_bits_to_float2(mn.y);
        const float2 m2 = half2_bits_to_float2(mn.z), m3 = half2_bits_to_float2(mn.w);
        const float sg[4] = {s0.x, s0.y, s1.x, s1.y}, sh[4] = {s2.x, s2.y, s3.x, s3.y};
        const float mg[4] = {m0.x * -0.0625f, m0.y * -0.0625f, m1.x * -0.0625f, m1.y * -0.0625f};
        const float mh[4] = {m2.x * -0.0625f, m2.y * -0.0625f, m3.x * -0.0625f, m3.y * -0.0625f};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t a[8];
            unpack8(a, word_of(c[0], j), word_of(c[1], j), MAGIC_16);
#pragma unroll
            for (int gi = 0; gi < NG; gi++) {
                const uint4 xb = lds128(xg[gi] + xoff + j * 64);
                const float2 ci = lds64f(caddr + (j * NG + gi) * 32);
                float d[4];
                block_mma_pre(d, a, xb, ci.x, ci.y, ci.x, ci.y);
                acc[gi][0] = fmaf(sg[j], d[0], fmaf(mg[j], ci.x, acc[gi][0]));
                acc[gi][2] = fmaf(sh[j], d[2], fmaf(mh[j], ci.x, acc[gi][2]));
                acc[gi][1] = fmaf(sg[j], d[1], fmaf(mg[j], ci.y, acc[gi][1]));
                acc[gi][3] = fmaf(sh[j], d[3], fmaf(mh[j], ci.y, acc[gi][3]));
            }
        }
    }
    template <int XC>
    __device__ __forceinline__ void compute(float (&acc)[4], uint32_t xaddr, uint32_t caddr, uint32_t live) const {
        const float2 s0 = half2_bits_to_float2(s.x), s1 = half2_bits_to_float2(s.y);  // row g, blocks 0..3
        const float2 s2 = half2_bits_to_float2(s.z), s3 = half2_bits_to_float2(s.w);  // row g + 8
        const float2 m0 = half2_bits_to_float2(mn.x), m1 = half2_bits_to_float2(mn.y);
        const float2 m2 = half2_bits_to_float2(mn.z), m3 = half2_bits_to_float2(mn.w);
        const float sg[4] = {s0.x, s0.y, s1.x, s1.y}, sh[4] = {s2.x, s2.y, s3.x, s3.y};
        const float mg[4] = {m0.x * -0.0625f, m0.y * -0.0625f, m1.x * -0.0625f, m1.y * -0.0625f};
        const float mh[4] = {m2.x * -0.0625f, m2.y * -0.0625f, m3.x * -0.0625f, m3.y * -0.0625f};
        uint4 xb;
        float4 ci;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            fetch_block<XC>(xaddr + j * 64, caddr + j * cinit_block_bytes<XC>(), live, xb, ci);
            float d[4];
            block_mma(d, word_of(c[0], j), word_of(c[1], j), xb, MAGIC_16, ci.x, ci.y, ci.z, ci.w);
            acc[0] = fmaf(sg[j], d[0], fmaf(mg[j], ci.x, acc[0]));
            acc[2] = fmaf(sh[j], d[2], fmaf(mh[j], ci.z, acc[2]));
            acc[1] = fmaf(sg[j], d[1], fmaf(mg[j], ci.y, acc[1]));
            acc[3] = fmaf(sh[j], d[3], fmaf(mh[j], ci.w, acc[3]));
        }
    }
};

template <> struct TileRegs<WF_QTYPE_Q8_0> {
    static constexpr float BETA = -400.f;  // (256 + 16 hi) + (16 + lo) - 400 = 16 (hi - 8) + lo
    static constexpr int BETA_INT = -1024;  // one token: 16 * (8 hi) + (8 lo) - 1024 = 8 * (16 (hi - 8) + lo)
    uint4 c[4], s;                         // c[0..1] high plane rows g / g+8, c[2..3] low plane
    uint32_t sg2, sh2;
    template <int XC>
    __device__ __forceinline__ void load(uint32_t t, int lane) {
#pragma unroll
        for (int i = 0; i < 4; i++) c[i] = lds128(t + i * 512);
        const uint32_t sb = t - lane * 16 + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + (lane >> 2) * 16;
        if (XC == 1) {
            sg2 = lds32(sb + (lane & 2) * 2);
            sh2 = lds32(sb + 8 + (lane & 2) * 2);
        } else {
            s = lds128(sb);
        }
    }
    // one token: the tile straight from global memory into registers (pointers and OFF as for Q4_0)
    static __device__ __forceinline__ int lane_scale_offset(int lane) { return (lane >> 2) * 16 + (lane & 2) * 2; }
    template <int OFF> __device__ __forceinline__ void load_global(const uint8_t* pc, const uint8_t* ps) {
        c[0] = ldg128_stream<OFF>(pc);
        c[1] = ldg128_stream<OFF + 512>(pc);
        c[2] = ldg128_stream<OFF + 1024>(pc);
        c[3] = ldg128_stream<OFF + 1536>(pc);
        sg2 = ldg32_stream<OFF + Tile<WF_QTYPE_Q8_0>::SCALE_OFF>(ps);
        sh2 = ldg32_stream<OFF + Tile<WF_QTYPE_Q8_0>::SCALE_OFF + 8>(ps);
    }
    // One token: value = 16 (hi - 8) + lo; the two planes accumulate separately and combine as integers.
    template <int J> __device__ __forceinline__ void compute_q8(float (&acc)[4], const Q8Addr& a, Q8Digits& dg) const {
        constexpr int TK = Tile<WF_QTYPE_Q8_0>::K;
        dg.template load<J * (TK / 128) * Q8_UNIT_BYTES>(a.x);
        const uint4 r = lds128_at<J * (TK >> 5) * 16>(a.rec);
        int la[4], lb[4], ha[4], hb[4];
        pair_imma(ha, c[0].x, c[1].x, c[0].z, c[1].z, dg.a.x, dg.a.y, dg.a.z, dg.a.w, dg.mul28);
        pair_imma(la, c[2].x, c[3].x, c[2].z, c[3].z, dg.a.x, dg.a.y, dg.a.z, dg.a.w, dg.mul28);
        pair_imma(hb, c[0].y, c[1].y, c[0].w, c[1].w, dg.b.x, dg.b.y, dg.b.z, dg.b.w, dg.mul28);
        pair_imma(lb, c[2].y, c[3].y, c[2].w, c[3].w, dg.b.x, dg.b.y, dg.b.z, dg.b.w, dg.mul28);
        const float2 sg = half2_bits_to_float2(sg2), sh = half2_bits_to_float2(sh2);
        const float ea = __uint_as_float(r.y), eb = __uint_as_float(r.w);
        const int wa = (int)r.x, wb = (int)r.z;
        acc[0] = fmaf(sg.x * ea, wide_digits_to_float(16 * ha[0] + la[0], 16 * ha[1] + la[1], wa), acc[0]);
        acc[2] = fmaf(sh.x * ea, wide_digits_to_float(16 * ha[2] + la[2], 16 * ha[3] + la[3], wa), acc[2]);
        acc[0] = fmaf(sg.y * eb, wide_digits_to_float(16 * hb[0] + lb[0], 16 * hb[1] + lb[1], wb), acc[0]);
        acc[2] = fmaf(sh.y * eb, wide_digits_to_float(16 * hb[2] + lb[2], 16 * hb[3] + lb[3], wb), acc[2]);
    }
    __device__ __forceinline__ void load_global_n(const uint8_t* tile, int lane) {
        c[0] = ldg128_stream<0>(tile + lane * 16);
        c[1] = ldg128_stream<512>(tile + lane * 16);
        c[2] = ldg128_stream<1024>(tile + lane * 16);
        c[3] = ldg128_stream<1536>(tile + lane * 16);
        s = ldg128_stream<Tile<WF_QTYPE_Q8_0>::SCALE_OFF>(tile + (lane >> 2) * 16);
    }
    template <int NG>
    __device__ __forceinline__ void compute_n(float (&acc)[NG][4], const uint32_t (&xg)[NG], uint32_t xoff, uint32_t caddr) const {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t ah[8], al[8];
            unpack8(ah, word_of(c[0], j), word_of(c[1], j), MAGIC_256);
            unpack8(al, word_of(c[2], j), word_of(c[3], j), MAGIC_16);
            const float2 dg = half2_bits_to_float2(j < 2 ? s.x : s.y), dh = half2_bits_to_float2(j < 2 ? s.z : s.w);
            const float sg = (j & 1) ? dg.y : dg.x, sh = (j & 1) ? dh.y : dh.x;
#pragma unroll
            for (int gi = 0; gi < NG; gi++) {
                const uint4 xb = lds128(xg[gi] + xoff + j * 64);
                const float2 ci = lds64f(caddr + (j * NG + gi) * 32);
                float d[4];
                block_mma_pre(d, ah, xb, ci.x, ci.y, ci.x, ci.y);
                block_mma_pre(d, al, xb, d[0], d[1], d[2], d[3]);
                acc[gi][0] = fmaf(sg, d[0], acc[gi][0]);
                acc[gi][2] = fmaf(sh, d[2], acc[gi][2]);
                acc[gi][1] = fmaf(sg, d[1], acc[gi][1]);
                acc[gi][3] = fmaf(sh, d[3], acc[gi][3]);
            }
        }
    }
    template <int XC>
    // xaddr: shared address of this lane's activations for k = kbase (row + q * 16 bytes);
    // caddr: shared address of the start value(s) of block kbase / 32; live: lane owns a live column
    __device__ __forceinline__ void compute(float (&acc)[4], uint32_t xaddr, uint32_t caddr, uint32_t live) const {
        uint4 xb;
        float4 ci;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            fetch_block<XC>(xaddr + j * 64, caddr + j * cinit_block_bytes<XC>(), live, xb, ci);
            float d[4];
            block_mma(d, word_of(c[0], j), word_of(c[1], j), xb, MAGIC_256, ci.x, ci.y, ci.z, ci.w);
            block_mma(d, word_of(c[2], j), word_of(c[3], j), xb, MAGIC_16, d[0], d[1], d[2], d[3]);
            const float2 dg = half2_bits_to_float2(j < 2 ? s.x : s.y), dh = half2_bits_to_float2(j < 2 ? s.z : s.w);
            const float sg = (j & 1) ? dg.y : dg.x, sh = (j & 1) ? dh.y : dh.x;
            acc[0] = fmaf(sg, d[0], acc[0]);
            acc[2] = fmaf(sh, d[2], acc[2]);
            acc[1] = fmaf(sg, d[1], acc[1]);
            acc[3] = fmaf(sh, d[3], acc[3]);
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
    static constexpr int BETA_INT = 0;    // one token: codes are unsigned, nothing to cancel
    uint4 c[4], sc, mn;                   // c[0..1] sub-blocks 0..3 rows g / g+8, c[2..3] sub-blocks 4..7
    uint2 dd;                             // (d, dmin) of row g, of row g+8
    uint32_t scg[2], sch[2], mng[2], mnh[2];  // one token, per unit u: scale / min bytes of sub-blocks 4u+2h, 4u+2h+1 (h = q >> 1), rows g / g+8
    template <int XC>
    __device__ __forceinline__ void load(uint32_t t, int lane) {
        using T = Tile<WF_QTYPE_Q4_K>;
#pragma unroll
        for (int i = 0; i < 4; i++) c[i] = lds128(t + i * 512);
        const uint32_t base = t - lane * 16;
        dd = lds64(base + T::D_OFF + (lane >> 2) * 8);
        if (XC == 1) {
            const uint32_t so = (lane >> 2) * 16 + (lane & 2);  // row g: bytes 2h, 2h+1; +4: sub-blocks 4+2h, 5+2h; +8: row g+8
#pragma unroll
            for (int u = 0; u < 2; u++) {
                scg[u] = lds16(base + T::SC_OFF + so + 4 * u);
                sch[u] = lds16(base + T::SC_OFF + so + 8 + 4 * u);
                mng[u] = lds16(base + T::MN_OFF + so + 4 * u);
                mnh[u] = lds16(base + T::MN_OFF + so + 8 + 4 * u);
            }
        } else {
            sc = lds128(base + T::SC_OFF + (lane >> 2) * 16);
            mn = lds128(base + T::MN_OFF + (lane >> 2) * 16);
        }
    }
    // one token: the tile straight from global memory into registers.  pc = tile + lane * 16, ps = tile + the lane's
    // scale offset; the (d, dmin) pairs sit at g * 8, which is half of the scale offset's g * 16: a third pointer
    // is rebuilt from ps (the lane's bit (lane & 2) is removed first).
    static __device__ __forceinline__ int lane_scale_offset(int lane) { return (lane >> 2) * 16 + (lane & 2); }
    template <int OFF> __device__ __forceinline__ void load_global(const uint8_t* pc, const uint8_t* ps) {
        using T = Tile<WF_QTYPE_Q4_K>;
        c[0] = ldg128_stream<OFF>(pc);
        c[1] = ldg128_stream<OFF + 512>(pc);
        c[2] = ldg128_stream<OFF + 1024>(pc);
        c[3] = ldg128_stream<OFF + 1536>(pc);
        const int lane = threadIdx.x & 31;
        dd = ldg64_stream<OFF + T::D_OFF>(ps - lane_scale_offset(lane) + (lane >> 2) * 8);
        // row g: bytes 2h, 2h+1; +4: sub-blocks 4+2h, 5+2h; +8: row g+8
        scg[0] = ldg16_stream<OFF + T::SC_OFF>(ps);
        scg[1] = ldg16_stream<OFF + T::SC_OFF + 4>(ps);
        sch[0] = ldg16_stream<OFF + T::SC_OFF + 8>(ps);
        sch[1] = ldg16_stream<OFF + T::SC_OFF + 12>(ps);
        mng[0] = ldg16_stream<OFF + T::MN_OFF>(ps);
        mng[1] = ldg16_stream<OFF + T::MN_OFF + 4>(ps);
        mnh[0] = ldg16_stream<OFF + T::MN_OFF + 8>(ps);
        mnh[1] = ldg16_stream<OFF + T::MN_OFF + 12>(ps);
    }
    // One token: the tile is two units of 128 k (sub-blocks 0..3 and 4..7).  8 * code enters the MMA as is;
    // the min term is (dmin * m) * (sum of the sub-block's activations), carried by the lanes of the first digit pair.
    template <int J> __device__ __forceinline__ void compute_q8(float (&acc)[4], const Q8Addr& a, Q8Digits& dg) const {
        const float2 g = half2_bits_to_float2(dd.x), h = half2_bits_to_float2(dd.y);  // (d, dmin) of rows g / g+8
        const float BIG = 8388608.f;
        const float ngd = -BIG * g.x, ngm = BIG * g.y, nhd = -BIG * h.x, nhm = BIG * h.y;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            if (u == 0) dg.template load<(2 * J) * Q8_UNIT_BYTES>(a.x);
            else dg.template load<(2 * J + 1) * Q8_UNIT_BYTES>(a.x);
            const uint4 r = u == 0 ? lds128_at<(2 * J) * 64>(a.rec) : lds128_at<(2 * J + 1) * 64>(a.rec);
            const uint2 sx = lds64(a.sx + (2 * J + u) * 32);
            int da[4], db[4];
            pair_imma(da, c[2 * u].x, c[2 * u + 1].x, c[2 * u].z, c[2 * u + 1].z, dg.a.x, dg.a.y, dg.a.z, dg.a.w, dg.mul28);
            pair_imma(db, c[2 * u].y, c[2 * u + 1].y, c[2 * u].w, c[2 * u + 1].w, dg.b.x, dg.b.y, dg.b.z, dg.b.w, dg.mul28);
            const uint32_t wsg = scg[u], wsh = sch[u], wmg = mng[u], wmh = mnh[u];
            const float ea = __uint_as_float(r.y), eb = __uint_as_float(r.w);
            const float xa = __uint_as_float(sx.x), xb = __uint_as_float(sx.y);
            // d * sc and -(dmin * m), exact
            acc[0] = fmaf(byte_times(wsg, 0, g.x, ngd) * ea, digits_to_float(da[0], da[1]),
                          fmaf(byte_times(wmg, 0, -g.y, ngm), xa, acc[0]));
            acc[2] = fmaf(byte_times(wsh, 0, h.x, nhd) * ea, digits_to_float(da[2], da[3]),
                          fmaf(byte_times(wmh, 0, -h.y, nhm), xa, acc[2]));
            acc[0] = fmaf(byte_times(wsg, 1, g.x, ngd) * eb, digits_to_float(db[0], db[1]),
                          fmaf(byte_times(wmg, 1, -g.y, ngm), xb, acc[0]));
            acc[2] = fmaf(byte_times(wsh, 1, h.x, nhd) * eb, digits_to_float(db[2], db[3]),
                          fmaf(byte_times(wmh, 1, -h.y, nhm), xb, acc[2]));
        }
    }
    __device__ __forceinline__ void load_global_n(const uint8_t* tile, int lane) {
        using T = Tile<WF_QTYPE_Q4_K>;
        c[0] = ldg128_stream<0>(tile + lane * 16);
        c[1] = ldg128_stream<512>(tile + lane * 16);
        c[2] = ldg128_stream<1024>(tile + lane * 16);
        c[3] = ldg128_stream<1536>(tile + lane * 16);
        dd = ldg64_stream<T::D_OFF>(tile + (lane >> 2) * 8);
        sc = ldg128_stream<T::SC_OFF>(tile + (lane >> 2) * 16);
        mn = ldg128_stream<T::MN_OFF>(tile + (lane >> 2) * 16);
    }
    template <int NG>
    __device__ __forceinline__ void compute_n(float (&acc)[NG][4], const uint32_t (&xg)[NG], uint32_t xoff, uint32_t caddr) const {
        const float2 g = half2_bits_to_float2(dd.x), h = half2_bits_to_float2(dd.y);  // (d, dmin)
        const float BIG = 8388608.f;
        const float gm = g.y * 0.0625f, hm = h.y * 0.0625f;
        const float ngd = -BIG * g.x, ngm = -BIG * gm, nhd = -BIG * h.x, nhm = -BIG * hm;
#pragma unroll
        for (int jj = 0; jj < 8; jj++) {
            uint32_t a[8];
            unpack8(a, word_of(c[(jj >> 2) * 2], jj & 3), word_of(c[(jj >> 2) * 2 + 1], jj & 3), MAGIC_16);
            const float ag = byte_times(jj < 4 ? sc.x : sc.y, jj & 3, g.x, ngd);
            const float ah = byte_times(jj < 4 ? sc.z : sc.w, jj & 3, h.x, nhd);
            const float cg = byte_times(jj < 4 ? mn.x : mn.y, jj & 3, gm, ngm);
            const float ch = byte_times(jj < 4 ? mn.z : mn.w, jj & 3, hm, nhm);
#pragma unroll
            for (int gi = 0; gi < NG; gi++) {
                const uint4 xb = lds128(xg[gi] + xoff + jj * 64);
                const float2 ci = lds64f(caddr + (jj * NG + gi) * 32);
                float d[4];
                block_mma_pre(d, a, xb, ci.x, ci.y, ci.x, ci.y);
                acc[gi][0] = fmaf(ag, d[0], fmaf(cg, ci.x, acc[gi][0]));
                acc[gi][2] = fmaf(ah, d[2], fmaf(ch, ci.x, acc[gi][2]));
                acc[gi][1] = fmaf(ag, d[1], fmaf(cg, ci.y, acc[gi][1]));
                acc[gi][3] = fmaf(ah, d[3], fmaf(ch, ci.y, acc[gi][3]));
            }
        }
    }
    template <int XC>
    // xaddr: shared address of this lane's activations for k = kbase (row + q * 16 bytes);
    // caddr: shared address of the start value(s) of block kbase / 32; live: lane owns a live column
    __device__ __forceinline__ void compute(float (&acc)[4], uint32_t xaddr, uint32_t caddr, uint32_t live) const {
        uint4 xb;
        float4 ci;
        const float2 g = half2_bits_to_float2(dd.x), h = half2_bits_to_float2(dd.y);  // (d, dmin)
        const float BIG = 8388608.f;
        // the min term -dmin*m*X comes from cinit = -16*X as (dmin/16) * m * cinit
        const float gm = g.y * 0.0625f, hm = h.y * 0.0625f;
        const float ngd = -BIG * g.x, ngm = -BIG * gm, nhd = -BIG * h.x, nhm = -BIG * hm;
#pragma unroll
        for (int jj = 0; jj < 8; jj++) {
            fetch_block<XC>(xaddr + jj * 64, caddr + jj * cinit_block_bytes<XC>(), live, xb, ci);
            float d[4];
            block_mma(d, word_of(c[(jj >> 2) * 2], jj & 3), word_of(c[(jj >> 2) * 2 + 1], jj & 3), xb, MAGIC_16, ci.x,
                      ci.y, ci.z, ci.w);
            const float ag = byte_times(jj < 4 ? sc.x : sc.y, jj & 3, g.x, ngd);  // d * sc, exact
            const float ah = byte_times(jj < 4 ? sc.z : sc.w, jj & 3, h.x, nhd);
            const float cg = byte_times(jj < 4 ? mn.x : mn.y, jj & 3, gm, ngm);  // dmin * m / 16, exact
            const float ch = byte_times(jj < 4 ? mn.z : mn.w, jj & 3, hm, nhm);
            acc[0] = fmaf(ag, d[0], fmaf(cg, ci.x, acc[0]));
            acc[2] = fmaf(ah, d[2], fmaf(ch, ci.z, acc[2]));
            acc[1] = fmaf(ag, d[1], fmaf(cg, ci.y, acc[1]));
            acc[3] = fmaf(ah, d[3], fmaf(ch, ci.w, acc[3]));
        }
    }
};

// ---------------------------------------------------------------- walking a CTA's share of a weight
// A CTA owns tiles [t0, t1) of the weight (row-tile major, k-tile minor), delivered through the
// ring in rounds of GEMV_WARPS consecutive tiles; consumer warp w takes tile w of every round.
// The share is a sequence of segments, one per row-tile it touches.  When a warp leaves a
// segment it parks its partial sums in slot (segment mod N) and arrives on the slot's `done`
// barrier -- nothing more, it does not wait for anybody.  One warp per segment, taken in turn,
// is the segment's reducer: one segment later, when the other warps have normally long
// arrived, it waits on `done`, adds the sixteen partials in warp order, finishes the row-tile
// (fix-up between CTAs, y) and marks the slot vacant.
struct BarrierSet {            // 32-bit shared addresses of the barrier arrays (8 bytes per barrier)
    uint32_t full, empty;      // [stages]: data of a round has landed / all warps have taken their tile
    uint32_t done, vacant;     // [Slots::N]: all warps have parked their partials / the reducer has read them
};
__device__ __forceinline__ BarrierSet barrier_set(uint8_t* smem) {
    BarrierSet b;
    b.full = smem_u32(smem + 128);
    b.empty = b.full + GEMV_MAX_STAGES * 8;
    b.done = b.empty + GEMV_MAX_STAGES * 8;
    b.vacant = b.done + GEMV_MAX_SLOTS * 8;
    return b;
}
template <int XC>
__device__ __forceinline__ void barrier_set_init(const BarrierSet& b, int stages) {
    for (int s = 0; s < stages; s++) {
        mbar_init(b.full + s * 8, 1);
        mbar_init(b.empty + s * 8, GEMV_WARPS);
    }
    for (int s = 0; s < Slots<XC>::N; s++) {
        mbar_init(b.done + s * 8, GEMV_WARPS);
        mbar_init(b.vacant + s * 8, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Position in the ring (stage, laps walked) and the number of segments flushed so far; both
// carry over from one weight to the next in the multi-op kernel.
struct WalkState {
    int s = 0;
    uint32_t lap = 0;
    int seg = 0;
    __device__ __forceinline__ void advance(int stages) {
        if (++s == stages) {
            s = 0;
            lap++;
        }
    }
};

// Producer (one thread): issue every round of the share, waiting for a stage to be released once
// the ring has been filled.  Stops early when the CTA has aborted.
template <int QT>
__device__ __forceinline__ void produce_share(const uint8_t* tiles, int t0, int t1, uint32_t ring32, const BarrierSet& bar,
                                              int stages, WalkState& pos, volatile int* abort_flag) {
    using T = Tile<QT>;
    constexpr uint32_t STAGE_BYTES = GEMV_WARPS * T::BYTES;
    const uint32_t abort32 = smem_u32(const_cast<int*>(abort_flag));
    for (int first = t0; first < t1; first += GEMV_WARPS) {
        if (pos.lap > 0) mbar_wait_or_abort(bar.empty + pos.s * 8, (pos.lap - 1) & 1, abort32);
        if (*abort_flag) return;
        const uint32_t bytes = (uint32_t)min(GEMV_WARPS, t1 - first) * T::BYTES;
        mbar_expect_tx(bar.full + pos.s * 8, bytes);
        bulk_load(ring32 + pos.s * STAGE_BYTES, tiles + (size_t)first * T::BYTES, bytes, bar.full + pos.s * 8);
        pos.advance(stages);
    }
}

// Accumulator fragment -> a partial-sum buffer, element i = column * 16 + row; clears the fragment.
template <int XC>
__device__ __forceinline__ void store_fragment(float* buf, float (&acc)[4], int g, int q) {
    if (XC == 1) {
        if (q == 0) {
            buf[g] = acc[0];
            buf[g + 8] = acc[2];
        }
    } else {
        buf[(2 * q) * 16 + g] = acc[0];
        buf[(2 * q + 1) * 16 + g] = acc[1];
        buf[(2 * q) * 16 + g + 8] = acc[2];
        buf[(2 * q + 1) * 16 + g + 8] = acc[3];
    }
    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
}

// Fix-up between CTAs.  A row-tile cut by a share boundary is finished by the CTA that holds its
// first k-tile (the owner).  The following CTAs publish their piece to their scratch slot as
// {value, 1} words; the owner adds the pieces in CTA order, clears the tags and emits the
// row-tile.  All waits are bounded; on expiry a status bit is set.
template <int ELEMS>
__device__ __forceinline__ void publish_piece(uint2* slot, const float (&v)[(ELEMS + 31) / 32], int lane, int* status) {
#pragma unroll
    for (int u = 0; u < (ELEMS + 31) / 32; u++) {
        const int i = lane + 32 * u;
        if (i >= ELEMS) continue;
        int spins = 0;  // the slot's previous content must have been taken before it is overwritten
        while (ld_slot(slot + i).y != 0u && ++spins < GEMV_FIXUP_SPINS) __nanosleep(32);
        if (spins >= GEMV_FIXUP_SPINS) atomicOr(status, STATUS_GEMV_FIXUP_TIMEOUT);
        st_slot(slot + i, make_uint2(__float_as_uint(v[u]), 1u));
    }
}
template <int ELEMS>
__device__ __forceinline__ void collect_pieces(uint2* slots, float (&v)[(ELEMS + 31) / 32], int lane, int row_end,
                                               int chunk_q, int chunk_r, int* status) {
    bool gave_up = false;
    for (int c = (int)blockIdx.x + 1; c < (int)gridDim.x && !gave_up; c++) {
        const int c0 = c * chunk_q + min(c, chunk_r), c1 = c0 + chunk_q + (c < chunk_r ? 1 : 0);
        if (c0 >= row_end) break;
        if (c0 == c1) continue;
        // all of this lane's elements of the piece are requested at once; those not yet published are polled
        constexpr int PER_LANE = (ELEMS + 31) / 32;
        uint2 e[PER_LANE];
#pragma unroll
        for (int u = 0; u < PER_LANE; u++) {
            const int i = lane + 32 * u;
            e[u] = i < ELEMS ? ld_slot(slots + (size_t)c * 128 + i) : make_uint2(0u, 1u);
        }
#pragma unroll
        for (int u = 0; u < PER_LANE; u++) {
            const int i = lane + 32 * u;
            if (i >= ELEMS) continue;
            uint2* sp = slots + (size_t)c * 128 + i;
            int spins = 0;
            while (e[u].y == 0u && ++spins < GEMV_FIXUP_SPINS) {
                __nanosleep(32);
                e[u] = ld_slot(sp);
            }
            if (e[u].y == 0u) {
                atomicOr(status, STATUS_GEMV_FIXUP_TIMEOUT);
                gave_up = true;
            } else {
                v[u] += __uint_as_float(e[u].x);
                st_slot(sp, make_uint2(0u, 0u));
            }
        }
        gave_up = __any_sync(0xFFFFFFFFu, gave_up);
    }
}

// Consumer warp: this warp's tiles of the share, segment by segment.  emit(row_tile, buf) writes
// one finished row-tile from a shared-memory buffer (element i = column * 16 + row) and is run
// by all 32 lanes of the segment's reducer.  Waits that run out raise the CTA's abort word.
template <int QT, int XC, class Emit>
__device__ __forceinline__ void consume_share(int t0, int t1, int kt, int chunk_q, int chunk_r, int warp, int lane,
                                              uint32_t ring32, const BarrierSet& bar, float* partial, int stages,
                                              WalkState& st, uint32_t x32, uint32_t c32, uint2* slots,
                                              int* status, uint32_t abort32, float (&acc)[4], Emit&& emit) {
    using T = Tile<QT>;
    using R = TileRegs<QT>;
    constexpr int NSLOT = Slots<XC>::N, ELEMS = Slots<XC>::ELEMS, PER_LANE = (ELEMS + 31) / 32;
    constexpr uint32_t STAGE_BYTES = GEMV_WARPS * T::BYTES;
    const int g = lane >> 2, q = lane & 3;
    const uint32_t my_tile = ring32 + warp * T::BYTES + lane * 16;
    const uint32_t lane_is_0 = lane == 0;

    // finish segment number sg (row-tile rt, tiles [sb, se) of it in this share)
    auto reduce = [&](int sg, int rt, int sb, int se) {
        const int slot = sg % NSLOT, gen = sg / NSLOT;
        mbar_wait_or_abort(bar.done + slot * 8, gen & 1, abort32);
        float* buf = partial + (size_t)slot * GEMV_WARPS * ELEMS;
        float v[PER_LANE];
#pragma unroll
        for (int u = 0; u < PER_LANE; u++) {
            const int i = lane + 32 * u;
            v[u] = 0.f;
            if (i < ELEMS) {
#pragma unroll
                for (int w = 0; w < GEMV_WARPS; w++) v[u] += buf[w * ELEMS + i];
            }
        }
        const bool starts = sb == rt * kt, ends = se == (rt + 1) * kt;
        if (!starts) {
            publish_piece<ELEMS>(slots + (size_t)blockIdx.x * 128, v, lane, status);
        } else {
            if (!ends) collect_pieces<ELEMS>(slots, v, lane, (rt + 1) * kt, chunk_q, chunk_r, status);
            __syncwarp();  // every lane has read what it needs of the slot: reuse its first row as emit's buffer
#pragma unroll
            for (int u = 0; u < PER_LANE; u++)
                if (lane + 32 * u < ELEMS) buf[lane + 32 * u] = v[u];
            __syncwarp();
            emit(rt, buf);
        }
        __syncwarp();
        mbar_arrive_if(bar.vacant + slot * 8, lane_is_0);
    };

    int seg_begin = t0, rt = (t0 < t1) ? t0 / kt : 0;
    int seg_end = min((rt + 1) * kt, t1);
    int t = t0 + warp;
    int prev_rt = 0, prev_begin = 0, prev_end = 0;
    bool have_prev = false;
    while (seg_begin < t1) {
        uint32_t xa = x32 + (t - rt * kt) * (T::K * 2), ca = c32 + (t - rt * kt) * ((T::K >> 5) * cinit_block_bytes<XC>());
        for (; t < seg_end; t += GEMV_WARPS) {  // my tiles below seg_end
            mbar_wait_or_abort(bar.full + st.s * 8, st.lap & 1, abort32);
            R regs;
            regs.template load<XC>(my_tile + st.s * STAGE_BYTES, lane);
            __syncwarp();
            mbar_arrive_if(bar.empty + st.s * 8, lane_is_0);
            regs.template compute<XC>(acc, xa, ca, 1u);
            xa += GEMV_WARPS * T::K * 2;
            ca += GEMV_WARPS * (T::K >> 5) * cinit_block_bytes<XC>();
            st.advance(stages);
        }
        // park my partial sums of this segment
        const int slot = st.seg % NSLOT, gen = st.seg / NSLOT;
        if (gen > 0) mbar_wait_or_abort(bar.vacant + slot * 8, (gen - 1) & 1, abort32);
        store_fragment<XC>(partial + ((size_t)slot * GEMV_WARPS + warp) * ELEMS, acc, g, q);
        __syncwarp();
        mbar_arrive_if(bar.done + slot * 8, lane_is_0);
        // the previous segment's reducer does its duty now
        if (have_prev && warp == (st.seg - 1) % GEMV_WARPS) reduce(st.seg - 1, prev_rt, prev_begin, prev_end);
        prev_rt = rt;
        prev_begin = seg_begin;
        prev_end = seg_end;
        have_prev = true;
        st.seg++;
        seg_begin = seg_end;
        rt++;
        seg_end = min((rt + 1) * kt, t1);
    }
    if (have_prev && warp == (st.seg - 1) % GEMV_WARPS) reduce(st.seg - 1, prev_rt, prev_begin, prev_end);
    // A warp without a tile in the share's last round still waits for that round and releases it,
    // so that every stage collects its GEMV_WARPS releases.  (t ran past t1 by less than a round;
    // the warp missed the last round iff the share's last round does not reach its position.)
    const int n = t1 - t0;
    if (n > 0 && (n % GEMV_WARPS) != 0 && warp >= (n % GEMV_WARPS)) {
        mbar_wait_or_abort(bar.full + st.s * 8, st.lap & 1, abort32);
        mbar_arrive_if(bar.empty + st.s * 8, lane_is_0);
        st.advance(stages);
    }
}

// ---------------------------------------------------------------- x staging
// Copies x into shared memory as bf16 rows of `kp` elements (zero beyond k), row stride sx
// bytes.  bf16 input: row = token.  fp32 input: token t becomes rows 3t, 3t+1, 3t+2 holding
// an exact three-way bf16 split (x = hi + mid + lo), so fp32 activations lose nothing.
// Also fills cinit[kp/32][4]: for block b and column pair q the float4
// {beta*X(b,2q), beta*X(b,2q+1), same, same}, X = fp32 sum of the block's 32 activations.
__device__ __forceinline__ uint32_t pack_bf16_trunc(float a, float b) {
    return (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xFFFF0000u);
}

// bf16 activations: the copy is verbatim.  Token by token (no index division), four 16-byte loads in
// flight per thread, one block sum per four consecutive lanes.
static __device__ void stage_x_bf16(const GemvParams& p, uint8_t* xs, float* cinit, int kp, float beta, int nthreads) {
    const int groups = kp >> 3, padded = (groups + 31) & ~31, kgroups = p.k >> 3;
    constexpr int U = 4;
    for (int t = 0; t < p.m; t++) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + (size_t)t * p.ldx);
        uint8_t* dst = xs + (size_t)t * p.sx;
        float* col = cinit + (t >> 1) * 4 + (t & 1);  // [block][q][4]: entries (t&1) and (t&1)+2 of quad t>>1
        for (int c0 = threadIdx.x; c0 < padded; c0 += nthreads * U) {   // warp-uniform trip counts
            uint4 pre[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int c8 = c0 + u * nthreads;
                pre[u] = make_uint4(0, 0, 0, 0);
                if (c8 < kgroups) pre[u] = __ldcg(src + c8);
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int c8 = c0 + u * nthreads;
                if ((c8 & ~31) >= padded) break;  // warp-uniform
                const uint4 v = pre[u];
                if (c8 < groups) *reinterpret_cast<uint4*>(dst + c8 * 16) = v;
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    sum += __uint_as_float(w[i] << 16);
                    sum += __uint_as_float(w[i] & 0xFFFF0000u);
                }
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                if (c8 < groups && (threadIdx.x & 3) == 0) {
                    const float v0 = beta * sum;
                    col[(c8 >> 2) * 16] = v0;
                    col[(c8 >> 2) * 16 + 2] = v0;
                }
            }
        }
    }
}

// One token for the integer path (layout and arithmetic: see pair_imma).  Per 32-k block the four
// threads that hold it find the largest magnitude, whose exponent field e (at least 40, so that every factor
// below is a normal float) fixes the block's scale: X = trunc(x * 2^(156 - e)) is an integer below 2^30,
// exact for every element within 2^-22 of the block's largest.  (X + 0x808080) XOR 0x808080 holds, byte by
// byte, the four signed base-256 digits of X.  A block holding Inf (and no NaN) is staged as signs only with
// an infinite factor, one holding a NaN with a NaN factor.  recs: 16 bytes per block of records followed by 8
// bytes per block of activation sums.
// KIND: where the token comes from.
//   XK_BF16          a bf16 row;
//   XK_F32           an fp32 row -- the same staging (an fp32 element has 24 significant bits, X keeps 30 below the
//                    block's largest magnitude, so elements within 2^-6 of it are exact and the others are cut at 2^-30 of it);
//   XK_RMSNORM_F32   (x[i] * inv) * gamma[i] of an fp32 row, inv = 1 / rms(x) worked out by the caller (cta_rms_inv),
//                    gamma = aux (may be null): rms_norm fused into the staging
//                    (warpforge-backend-cpu/src/main/java/io/surfworks/warpforge/backend/cpu/ops/scalar/CustomCallKernel.java:173-224);
//   XK_SWIGLU_F32    (x[i] * sigmoid(x[i])) * aux[i], x = the gate projection's output, aux = the up projection's:
//                    silu (CustomCallKernel.java:262-280) and the multiply fused into the staging of Wdown.
constexpr int XK_BF16 = 0, XK_F32 = 1, XK_RMSNORM_F32 = 2, XK_SWIGLU_F32 = 3;

// 1 / rms of an fp32 row for the whole CTA: rms = sqrt(sum x^2 / k + eps), the sum taken per thread, per warp, then
// over the warps in warp order (every thread of every CTA gets the same bits).  scratch: 16 floats of shared
// memory; all `nthreads` threads call it (one named barrier).
static __device__ __noinline__ float cta_rms_inv(const float* x, int k, float eps, float* scratch, int nthreads) {
    float ss = 0.f;
    const float4* src = reinterpret_cast<const float4*>(x);
    for (int i = threadIdx.x; i < (k >> 2); i += nthreads) {
        const float4 v = __ldcg(src + i);
        ss += v.x * v.x;
        ss += v.y * v.y;
        ss += v.z * v.z;
        ss += v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = ss;
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    float total = 0.f;
    for (int w = 0; w < (nthreads >> 5); w++) total += scratch[w];
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");  // scratch may be reused
    const float rms = (float)sqrt((double)(total / (float)k + eps));
    return 1.0f / rms;
}

template <int BETA_INT, int KIND>
static __device__ __noinline__ void stage_x_q8(const void* x, int k, uint8_t* xd, uint8_t* recs, int kp, int nthreads,
                                               const float* aux = nullptr, float inv = 1.f) {
    constexpr bool F32 = KIND != XK_BF16, AUX = KIND == XK_RMSNORM_F32 || KIND == XK_SWIGLU_F32;
    const int groups = kp >> 3, padded = (groups + 31) & ~31, kgroups = k >> 3;
    const uint4* src = static_cast<const uint4*>(x);
    const uint4* asrc = reinterpret_cast<const uint4*>(aux);
    const bool has_aux = AUX && aux != nullptr;
    uint8_t* sums = recs + (size_t)(kp >> 5) * 16;  // the activation sums follow the records
    constexpr int U = F32 ? 2 : 3;  // element groups in flight per thread
    for (int c0 = threadIdx.x; c0 < padded; c0 += nthreads * U) {  // warp-uniform trip counts
        uint4 pre[U], pre2[U], ax[U], ax2[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int c8 = c0 + u * nthreads;
            pre[u] = pre2[u] = make_uint4(0u, 0u, 0u, 0u);
            ax[u] = ax2[u] = make_uint4(0x3F800000u, 0x3F800000u, 0x3F800000u, 0x3F800000u);  // 1.0f
            if (c8 < kgroups) {
                if (F32) {
                    pre[u] = __ldcg(src + 2 * c8);
                    pre2[u] = __ldcg(src + 2 * c8 + 1);
                    if (has_aux) {
                        ax[u] = __ldcg(asrc + 2 * c8);
                        ax2[u] = __ldcg(asrc + 2 * c8 + 1);
                    }
                } else {
                    pre[u] = __ldcg(src + c8);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int c8 = c0 + u * nthreads;
            if ((c8 & ~31) >= padded) break;  // warp-uniform
            const uint4 v = pre[u];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            float f[8];
            if (F32) {
                const uint4 v2 = pre2[u];
                f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
                f[4] = __uint_as_float(v2.x); f[5] = __uint_as_float(v2.y); f[6] = __uint_as_float(v2.z); f[7] = __uint_as_float(v2.w);
                if (AUX) {
                    const uint4 a1 = ax[u], a2 = ax2[u];
                    const float a[8] = {__uint_as_float(a1.x), __uint_as_float(a1.y), __uint_as_float(a1.z), __uint_as_float(a1.w),
                                        __uint_as_float(a2.x), __uint_as_float(a2.y), __uint_as_float(a2.z), __uint_as_float(a2.w)};
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        if (KIND == XK_RMSNORM_F32) {
                            f[i] = f[i] * inv;
                            if (has_aux) f[i] *= a[i];
                        } else {
                            const float sig = 1.0f / (1.0f + expf(-f[i]));
                            f[i] = (f[i] * sig) * a[i];
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    f[2 * i] = __uint_as_float(w[i] << 16);
                    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
                }
            }
            float sum = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
            float amax = fmaxf(fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3]))),
                               fmaxf(fmaxf(fabsf(f[4]), fabsf(f[5])), fmaxf(fabsf(f[6]), fabsf(f[7]))));
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            const int eeff = max((int)(__float_as_uint(amax) >> 23), 40);
            const bool special = eeff == 0xFF || sum != sum;  // an Inf or a NaN in the block (a NaN makes the sum a NaN)
            const float scale = __uint_as_float((uint32_t)(283 - eeff) << 23);  // 2^(156 - e)
            uint32_t z[8];  // per element the four signed digit bytes, least significant digit in byte 0
#pragma unroll
            for (int i = 0; i < 8; i++) {
                int X = __float2int_rz(f[i] * scale);
                if (special) X = (fabsf(f[i]) == __uint_as_float(0x7F800000u)) ? (f[i] < 0.f ? -1 : 1) : 0;
                z[i] = ((uint32_t)X + 0x00808080u) ^ 0x00808080u;
            }
            // transpose to digit-major byte quadruples in the element order of the two MMAs: (0, 4, 1, 5) and (2, 6, 3, 7)
            uint32_t t1[4], t2[4];
            {
                const uint32_t P = __byte_perm(z[0], z[4], 0x5140), Q = __byte_perm(z[0], z[4], 0x7362);
                const uint32_t R = __byte_perm(z[1], z[5], 0x5140), S = __byte_perm(z[1], z[5], 0x7362);
                t1[0] = __byte_perm(P, R, 0x5410); t1[1] = __byte_perm(P, R, 0x7632);
                t1[2] = __byte_perm(Q, S, 0x5410); t1[3] = __byte_perm(Q, S, 0x7632);
            }
            {
                const uint32_t P = __byte_perm(z[2], z[6], 0x5140), Q = __byte_perm(z[2], z[6], 0x7362);
                const uint32_t R = __byte_perm(z[3], z[7], 0x5140), S = __byte_perm(z[3], z[7], 0x7362);
                t2[0] = __byte_perm(P, R, 0x5410); t2[1] = __byte_perm(P, R, 0x7632);
                t2[2] = __byte_perm(Q, S, 0x5410); t2[3] = __byte_perm(Q, S, 0x7632);
            }
            int dsum[4];
#pragma unroll
            for (int t = 0; t < 4; t++) {
                dsum[t] = BETA_INT == 0 ? 0 : __dp4a((int)t1[t], 0x01010101, __dp4a((int)t2[t], 0x01010101, 0));
                if (BETA_INT != 0) {
                    dsum[t] += __shfl_xor_sync(0xFFFFFFFFu, dsum[t], 1);
                    dsum[t] += __shfl_xor_sync(0xFFFFFFFFu, dsum[t], 2);
                }
            }
            if (c8 < groups) {
                const int b = c8 >> 2, q = c8 & 3, unit = b >> 2, j = b & 3, pair = j & 1, hcol = j >> 1;
                // lane (g = 4 hcol + digit, q): 32 bytes {lo, hi} first MMA, {lo, hi} second MMA for pair A, then pair B;
                // this block fills the lo words when it is its pair's first block (hcol 0), the hi words otherwise
                uint8_t* base = xd + (size_t)unit * Q8_UNIT_BYTES + q * 32 + pair * 16 + hcol * 4;
#pragma unroll
                for (int t = 0; t < 4; t++) {  // digit t has weight 256^t; column digit index = 3 - t (most significant first)
                    uint32_t* w = reinterpret_cast<uint32_t*>(base + (4 * hcol + (3 - t)) * 128);
                    w[0] = t1[t];
                    w[2] = t2[t];
                }
                if (q == 0) {
                    // x = X * 2^(e - 156); the MMA multiplies 8 * code; the lanes of the first digit pair hold
                    // 256^3 D + 256^2 D' = 2^16 (256 D + D')
                    float f_hi = __uint_as_float((uint32_t)(eeff - 156 - 3 + 16 + 127) << 23);
                    float f_lo = __uint_as_float((uint32_t)(eeff - 156 - 3 + 127) << 23);
                    if (special) {
                        // a NaN sum: a NaN element, or Infs of both signs (which the CPU's sum of products turns into NaN as well)
                        const bool nan = sum != sum;
                        f_hi = nan ? __uint_as_float(0x7FC00000u) : 0.f;
                        f_lo = nan ? __uint_as_float(0x7FC00000u) : __uint_as_float(0x7F800000u);
                    }
                    // block j of the unit is block (j & 1) of lane position h = j >> 1; digit pair p: record at (2 h + p) * 16
                    uint8_t* rec = recs + (size_t)unit * 64 + (size_t)(j >> 1) * 32 + (size_t)(j & 1) * 8;
                    *reinterpret_cast<uint2*>(rec) = make_uint2((uint32_t)(BETA_INT * (256 * dsum[3] + dsum[2])), __float_as_uint(f_hi));
                    *reinterpret_cast<uint2*>(rec + 16) = make_uint2((uint32_t)(BETA_INT * (256 * dsum[1] + dsum[0])), __float_as_uint(f_lo));
                    float* sp = reinterpret_cast<float*>(sums + (size_t)unit * 32 + (size_t)(j >> 1) * 16 + (size_t)(j & 1) * 4);
                    sp[0] = sum;
                    sp[2] = 0.f;
                }
            }
        }
    }
}

static __device__ void stage_x(const GemvParams& p, uint8_t* xs, float* cinit, int kp, float beta, int nthreads) {
    if (!p.x_f32) {
        stage_x_bf16(p, xs, cinit, kp, beta, nthreads);
        return;
    }
    const int groups = kp >> 3;  // 8 elements per thread step
    const int total = p.m * groups;
    constexpr int U = 4;  // bf16 path: four independent loads in flight per thread
    for (int idx0 = threadIdx.x; idx0 < ((total + 31) & ~31); idx0 += nthreads * (p.x_f32 ? 1 : U)) {  // warp-uniform trip counts
      uint4 pre[U];
      if (!p.x_f32) {
#pragma unroll
          for (int u = 0; u < U; u++) {
              const int idx = idx0 + u * nthreads;
              const int t = (idx < total && p.m > 1) ? idx / groups : 0, c8 = idx < total ? idx - t * groups : 0;
              pre[u] = make_uint4(0, 0, 0, 0);
              if (idx < total && c8 * 8 < p.k)
                  pre[u] = __ldcg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.x) + (size_t)t * p.ldx + c8 * 8));
          }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int idx = idx0 + u * nthreads;
        if ((p.x_f32 && u > 0) || (idx & ~31) >= ((total + 31) & ~31)) break;  // warp-uniform
        const bool live = idx < total;
        const int t = (live && p.m > 1) ? idx / groups : 0, c8 = live ? idx - t * groups : 0;
        const bool in_k = live && (c8 * 8 < p.k);
        float sum[3] = {0.f, 0.f, 0.f};
        if (!p.x_f32) {
            const uint4 v = pre[u];
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
                const float4 a = __ldcg(src), b = __ldcg(src + 1);
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
}

}  // namespace wf
