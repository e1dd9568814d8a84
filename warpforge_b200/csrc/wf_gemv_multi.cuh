// Decode GEMV for several tokens (2 .. 32 activation columns): y[m, rows] = x[m, K] . W[rows, K]^T, memory-bound.
//
// Every warp loads its tiles from global memory straight into registers (the tile layout is the MMA's fragment
// order) and multiplies them on mma.m16n8k16 with exact bf16 operands and fp32 accumulation: the 4-bit codes of a
// 32-k block become A fragments once (unpack8) and meet NG = 1, 2 or 4 groups of eight activation columns, so the
// integer work per weight byte does not grow with the number of tokens.  fp32 activations enter as three exact
// bf16 columns per token (x = hi + mid + lo), as in the one-pass ring kernel this replaces.
//
// Work split.  A unit is one row-tile (16 rows) times one k-slice (kc consecutive k-tiles, contiguous in memory).
// A team of W warps of one CTA owns whole units: its members cut a unit's k-tiles among themselves, keep their
// sums in registers from their first to their last tile, and hand them to the team's first member through
// shared memory (one named barrier per unit).  The number of k-slices S and the team size W are chosen on the
// host so that (i) a slice of the activations (all columns, kc tiles of k) fits in shared memory whatever K is,
// and (ii) every warp of the grid has about the same number of tiles however few rows the weight has (a
// 1024-row shard has 64 row-tiles for 2368 warps).  The CTAs are dealt to the slices round-robin (CTA c works
// on slice c mod S); the CTAs of a slice split its row-tiles evenly, and so do the teams of a CTA.  A CTA stages
// only its own slice of x.
//
// With S > 1 (or fp32 activations, whose three columns per token are combined at the end) a unit's sums go to a
// partial-sum buffer [slice][column][row]; the warp then counts itself on the row-tile's arrival counter, and
// the warp that finds all other slices already counted adds the S partial sums in slice order and stores y
// (it also puts the counter back to zero).  The order of the additions is fixed, so the result does not depend
// on which warp comes last; nobody waits for anybody.  With S = 1 and bf16 activations y is stored directly.
//
// Replaces, for up to 32 tokens, the fp32 batch_matmul_f32 launch of
// warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/ops/DotGeneralKernel.java:263-281.
#pragma once
#include "wf_gemv_stream.cuh"

namespace wf {

// weight of a staged activation byte against a streamed weight byte in the planner's estimate (measured: 1 - 3 give
// the same cuts for up to 8 columns, 2 the best ones for 16; 6 and more cut K too finely)
constexpr int GEMVN_STAGE_COST = 2;
constexpr int GEMVN_MAX_COLS = 32;
constexpr int GEMVN_MAX_SLICES = 64;
constexpr size_t GEMVN_PART_BYTES = 8u << 20;  // partial sums a launch may use (the static array of the no-alloc entry is this large)
constexpr int GEMVN_MAX_ROW_TILES = 1 << 16;   // arrival counters

struct GemvNParams {
    const uint8_t* tiles;
    const void* x;
    float* y;
    float* part;  // [slices][cols][rt * 16], used unless slices == 1 with bf16 activations
    int* count;   // [rt] arrivals per row-tile, zero between launches
    int* status;
    int64_t ldy, col0, ldx;
    int rows, k, kt, rt;
    int m, x_f32, cols;  // cols = activation columns = m (bf16) or 3 m (fp32)
    int slices, kc;      // k-slices; k-tiles per slice (the last slice may have fewer)
    int team;            // warps that share a unit (they cut its k-tiles among themselves)
    int sx;              // bytes per staged activation row
    int piece_off;       // byte offset of the team hand-over buffers in shared memory
    unsigned long long* timing;
};

template <int QT, int NG> struct GemvNGeom {
    // tiles a warp holds in registers while it multiplies: what 128 registers per thread leave room for
    static constexpr int DEPTH = (QT == WF_QTYPE_Q4_0) ? (NG == 4 ? 3 : 4) : (QT == WF_QTYPE_Q4_1) ? 3 : 2;
};

// Shared memory: start values [kc * TK / 32][NG][4] float2 | staged x [cols][sx] | team hand-over [2][16][32] NG float4.
inline size_t gemvn_smem(int qt, int kc, int cols, int ng, int team, int* sx_out, int* piece_off_out) {
    const int kslice = kc * tile_k(qt);
    const int sx = kslice * 2 + 64;  // +64: consecutive rows start 16 banks apart
    if (sx_out) *sx_out = sx;
    size_t b = 128 + (size_t)(kslice / 32) * ng * 32 + (size_t)cols * sx;
    b = (b + 127) & ~(size_t)127;
    if (piece_off_out) *piece_off_out = (int)b;
    if (team > 1) b += (size_t)2 * GEMV_WARPS * 32 * ng * 16;
    return b;
}

struct GemvNPlan {
    int slices = 0, kc = 0, team = 1;  // slices == 0: no plan fits
    bool uses_part = false;
};
// The cheapest (S, W) by the estimate "what the busiest warp moves", in sixteenths of a tile: per slice,
// ceil(row-tiles / teams of the slice) units; per unit the member's share of the kc tiles, the hand-over inside
// the team (W > 1) and the partial sums written (cols x 64 bytes, S > 1); for the warp that completes a row-tile
// the S partial sums read back and two tiles' worth of round trips; for every warp its sixteenth of the CTA's
// activation staging (cols x kc tiles of k, bf16; all CTAs of a slice read the same lines of the L2).
inline GemvNPlan gemvn_plan(int sm_count, int qt, int64_t rt, int64_t kt, int cols, bool x_f32) {
    GemvNPlan best;
    const int ng = cols <= 8 ? 1 : cols <= 16 ? 2 : 4;
    int64_t best_cost = -1;
    int last_kc = 0;
    static const int team_sizes[] = {1, 2, 3, 4, 5, 8, 16};
    for (int s = 1; s <= GEMVN_MAX_SLICES && s <= kt && s <= sm_count; s++) {
        const int kc = (int)((kt + s - 1) / s), slices = (int)((kt + kc - 1) / kc);
        if (kc == last_kc) continue;
        last_kc = kc;
        const bool part = slices > 1 || x_f32;
        if (part && (size_t)slices * cols * rt * 16 * 4 > GEMVN_PART_BYTES) continue;
        const int64_t tb = tile_bytes(qt), part16 = part ? ((int64_t)cols * 64 * 16 + tb - 1) / tb : 0;
        for (int w : team_sizes) {
            if (gemvn_smem(qt, kc, cols, ng, w, nullptr, nullptr) > 200 * 1024) continue;
            const int teams = GEMV_WARPS / w;
            int64_t cost = 0;
            for (int sl = 0; sl < slices; sl++) {
                const int64_t ctas = (sm_count - sl + slices - 1) / slices;
                const int64_t kcs = std::min<int64_t>(kc, kt - (int64_t)sl * kc);
                const int64_t units_cta = (rt + ctas - 1) / ctas, units_team = (units_cta + teams - 1) / teams;
                cost = std::max(cost, units_team * (((kcs + w - 1) / w) * 16 + (w > 1 ? 4 + w : 0) + part16));
            }
            if (part) cost += slices * part16 + 32;
            // every CTA stages cols x kc tiles of k of the activations (from L2, by all its warps together)
            cost += ((int64_t)cols * kc * tile_k(qt) * GEMVN_STAGE_COST + tb - 1) / tb;
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                best.slices = slices;
                best.kc = kc;
                best.team = w;
                best.uses_part = part;
            }
        }
    }
    return best;
}

// Stage this CTA's k-slice [k_lo, k_lo + kslice) of every token: bf16 rows of kslice elements (zero beyond k) and,
// per 32-k block, group of eight columns and column pair q, the float2 {beta X(2q), beta X(2q+1)} with X the fp32
// sum of the block's 32 activations of that column (the start values of rows g and g+8 alike).
//
// bf16 activations: the rows are copied verbatim, one bulk asynchronous copy per token straight into shared
// memory (no registers, no per-thread load latency; `bar` is an initialised mbarrier with one arrival pending),
// and the block sums are taken from shared memory afterwards, one (column, block) per thread, in the association
// ((s0 + s1) + (s2 + s3)) of four eight-element runs.
static __device__ void stage_x_slice_bulk(const GemvNParams& p, uint8_t* xs, float* cinit, int k_lo, int kslice, int ng, float beta,
                                          int nthreads, uint32_t bar, uint32_t abort32) {
    const int valid = max(0, min(kslice, p.k - k_lo));  // elements of the slice that exist
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, (uint32_t)(p.m * valid * 2));
        for (int t = 0; t < p.m; t++)
            if (valid > 0)
                bulk_load(smem_u32(xs + (size_t)t * p.sx), static_cast<const uint16_t*>(p.x) + (size_t)t * p.ldx + k_lo, (uint32_t)valid * 2, bar);
    }
    if (valid < kslice) {  // K ends inside the slice: zeros behind it (k is a multiple of 32, so whole 16-byte pieces)
        const int pieces = (kslice - valid) >> 3;
        for (int i = threadIdx.x; i < p.m * pieces; i += nthreads) {
            const int t = i / pieces, c = i - t * pieces;
            *reinterpret_cast<uint4*>(xs + (size_t)t * p.sx + (size_t)(valid + c * 8) * 2) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncthreads();
    }
    mbar_wait_or_abort(bar, 0, abort32);
    const int nblk = kslice >> 5;
    for (int i = threadIdx.x; i < p.m * nblk; i += nthreads) {
        const int t = i / nblk, b = i - t * nblk;
        const uint4* src = reinterpret_cast<const uint4*>(xs + (size_t)t * p.sx + (size_t)b * 64);
        float part[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint4 v = src[j];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                sum += __uint_as_float(w[e] << 16);
                sum += __uint_as_float(w[e] & 0xFFFF0000u);
            }
            part[j] = sum;
        }
        const float v = beta * ((part[0] + part[1]) + (part[2] + part[3]));
        cinit[(size_t)b * ng * 8 + t] = v;  // [block][group][q] float2 = [block][column]
    }
}

// fp32 activations (three bf16 columns per token), through registers.
static __device__ void stage_x_slice(const GemvNParams& p, uint8_t* xs, float* cinit, int k_lo, int kslice, int ng, float beta,
                                     int nthreads) {
    const int groups = kslice >> 3;  // 8 elements per thread step; a multiple of 4
    const int total = p.m * groups;
    const int padded = (total + 31) & ~31;
    // Every CTA of a slice reads the same activations: each starts at another place of the list (a multiple of 32
    // items, so warps and the four threads of a block stay together), or all of them would ask the same L2 lines at
    // the same moment.
    const int rot = (int)(((int64_t)(blockIdx.x / p.slices) * 2654435761LL) % (padded >> 5)) << 5;
    auto item = [&](int raw) {
        const int i = raw + rot;
        return i >= padded ? i - padded : i;
    };
    // block sums: 4 consecutive threads hold one 32-element block (groups is a multiple of 4, so they belong to one token)
    auto block_sums = [&](float (&sum)[3], bool live, int t, int c8) {
#pragma unroll
        for (int s = 0; s < 3; s++) {
            sum[s] += __shfl_xor_sync(0xFFFFFFFFu, sum[s], 1);
            sum[s] += __shfl_xor_sync(0xFFFFFFFFu, sum[s], 2);
        }
        if (live && (threadIdx.x & 3) == 0) {
            float* blk = cinit + (size_t)(c8 >> 2) * ng * 8;  // [group][q] float2 = [column]
            const int parts = p.x_f32 ? 3 : 1;
            for (int s = 0; s < parts; s++) blk[p.x_f32 ? 3 * t + s : t] = beta * sum[s];
        }
    };
    for (int raw = threadIdx.x; raw < padded; raw += nthreads) {  // warp-uniform trip counts
        const int idx = item(raw);
        const bool live = idx < total;
        const int t = live ? idx / groups : 0, c8 = live ? idx - t * groups : 0;
        const int kk = k_lo + c8 * 8;
        const bool in_k = live && kk < p.k;
        float sum[3] = {0.f, 0.f, 0.f};
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (in_k) {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + (size_t)t * p.ldx + kk);
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
        block_sums(sum, live, t, c8);
    }
}

template <int QT, int NG>
__global__ void __launch_bounds__(GEMV_CONSUMERS, 1) gemvn_kernel(const GemvNParams p) {
    using T = Tile<QT>;
    using R = TileRegs<QT>;
    constexpr int DEPTH = GemvNGeom<QT, NG>::DEPTH;
    constexpr uint32_t XSTEP = T::K * 2, CSTEP = (T::K / 32) * NG * 32;  // staged bytes per tile
    extern __shared__ __align__(128) uint8_t smem[];

    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    const int S = p.slices, slice = (int)blockIdx.x % S, idx = (int)blockIdx.x / S;
    const int ctas = ((int)gridDim.x - slice + S - 1) / S;  // CTAs working on this slice
    const int k0t = slice * p.kc, kcs = min(p.kc, p.kt - k0t);
    // teams of W warps; a team owns whole units, its members cut a unit's k-tiles among themselves
    const int W = p.team, teams = GEMV_WARPS / W;
    const int team = warp / W, member = warp - team * W;
    const bool idle = team >= teams;
    // this CTA's row-tiles of the slice, this team's share of them
    const int u0 = (int)((int64_t)idx * p.rt / ctas), u1 = (int)((int64_t)(idx + 1) * p.rt / ctas);
    const int nu = u1 - u0, tq = nu / teams, tr = nu - tq * teams;
    const int ua = idle ? 0 : u0 + team * tq + min(team, tr), ub = idle ? 0 : ua + tq + (team < tr ? 1 : 0);
    // this member's k-tiles inside every unit
    const int ma = member * kcs / W, mb = (member + 1) * kcs / W, ml = mb - ma;
    const int nt = (ub - ua) * ml;  // tiles of this warp

    auto stamp = [&](int i) {
        if (p.timing != nullptr && threadIdx.x == 0) {
            unsigned long long tm;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm));
            p.timing[(size_t)blockIdx.x * 8 + i] = tm;
        }
    };
    // Programmatic stream serialization, as in the one-token kernel: the weights depend on nothing, so the first
    // tiles are requested before the wait for the previous grid.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    stamp(3);
    R slots[DEPTH];
    const uint8_t* lptr = p.tiles + ((size_t)ua * p.kt + k0t + ma) * T::BYTES;
    int lkk = 0, lrem = nt;
    auto load_next = [&](R& slot) {
        if (lrem > 0) {
            slot.load_global_n(lptr, lane);
            lrem--;
            lptr += T::BYTES;
            if (++lkk == ml) {  // next unit: the same k-tiles of the next row-tile
                lkk = 0;
                lptr += (size_t)(p.kt - ml) * T::BYTES;
            }
        }
    };
    static_for<DEPTH>([&](auto J) { load_next(slots[decltype(J)::value]); });
    // control words: mbarrier of the activation copies at 0, abort word at 8
    if (threadIdx.x == 0) {
        *reinterpret_cast<volatile int*>(smem + 8) = 0;
        mbar_init(smem_u32(smem), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    float* cinit = reinterpret_cast<float*>(smem + 128);  // [kslice / 32][NG][4] float2
    const int kslice = kcs * T::K;
    uint8_t* xs = reinterpret_cast<uint8_t*>(cinit + (size_t)(p.kc * T::K / 32) * NG * 8);
    // team hand-over: [2][warp][lane] NG float4, after the staged activations
    float4* pieces = reinterpret_cast<float4*>(smem + p.piece_off);

    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(0);
    if (p.x_f32) stage_x_slice(p, xs, cinit, k0t * T::K, kslice, NG, R::BETA, GEMV_CONSUMERS);
    else stage_x_slice_bulk(p, xs, cinit, k0t * T::K, kslice, NG, R::BETA, GEMV_CONSUMERS, smem_u32(smem), smem_u32(smem + 8));
    __syncthreads();
    stamp(1);
    if (*reinterpret_cast<volatile int*>(smem + 8)) {  // the copies did not land in time: y would be garbage
        if (threadIdx.x == 0) atomicOr(p.status, STATUS_GEMV_FIXUP_TIMEOUT);
        drain_after_abort();
        return;
    }
    if (idle) return;

    // dead columns read the last live row: their results are computed and never stored
    uint32_t xg[NG];
#pragma unroll
    for (int gi = 0; gi < NG; gi++) xg[gi] = smem_u32(xs) + (uint32_t)min(8 * gi + g, p.cols - 1) * p.sx + q * 16 + (uint32_t)ma * XSTEP;
    const uint32_t c32 = smem_u32(cinit) + q * 8 + (uint32_t)ma * CSTEP;
    const bool direct = S == 1 && !p.x_f32;
    const int64_t prow = (int64_t)p.rt * 16;

    float acc[NG][4];
#pragma unroll
    for (int gi = 0; gi < NG; gi++) acc[gi][0] = acc[gi][1] = acc[gi][2] = acc[gi][3] = 0.f;

    // member 0 of the team, holding the unit's complete sums: store them (or count the slice in and add the slices)
    auto store_unit = [&](int u) {
        const int r0 = u * 16 + g, r1 = r0 + 8;
        if (direct) {
#pragma unroll
            for (int gi = 0; gi < NG; gi++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int col = 8 * gi + 2 * q + e;
                    if (col < p.cols) {
                        if (r0 < p.rows) p.y[(int64_t)col * p.ldy + p.col0 + r0] = acc[gi][e];
                        if (r1 < p.rows) p.y[(int64_t)col * p.ldy + p.col0 + r1] = acc[gi][2 + e];
                    }
                }
            return;
        }
        float* mine = p.part + (int64_t)slice * p.cols * prow;
#pragma unroll
        for (int gi = 0; gi < NG; gi++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int col = 8 * gi + 2 * q + e;
                if (col < p.cols) {
                    __stcg(mine + (int64_t)col * prow + r0, acc[gi][e]);
                    __stcg(mine + (int64_t)col * prow + r1, acc[gi][2 + e]);
                }
            }
        // count this slice in; the warp that completes the row-tile adds the slices in order
        __syncwarp();
        int old = 0;
        if (lane == 0) {
            __threadfence();
            old = atomicAdd(p.count + u, 1);
        }
        old = __shfl_sync(0xFFFFFFFFu, old, 0);
        if (old != S - 1) return;
        if (lane == 0) p.count[u] = 0;  // nobody else touches it again in this launch
        __threadfence();
        // four (token, row) sums per lane at a time, so that the loads of a slice do not wait for one another
        const int items = p.m * 16;
        const int64_t sstride = (int64_t)p.cols * prow;
        for (int i0 = lane; i0 < items; i0 += 128) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            const float* src[4];
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const int i = min(i0 + 32 * w, items - 1), tok = i >> 4;
                src[w] = p.part + (int64_t)(p.x_f32 ? 3 * tok : tok) * prow + u * 16 + (i & 15);
            }
            for (int s = 0; s < S; s++) {
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const float* ps = src[w] + (int64_t)s * sstride;
                    // fp32 activations: columns 3t, 3t+1, 3t+2 are the hi / mid / lo parts of token t
                    v[w] += p.x_f32 ? (__ldcg(ps + 2 * prow) + __ldcg(ps + prow)) + __ldcg(ps) : __ldcg(ps);
                }
            }
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const int i = i0 + 32 * w, row = u * 16 + (i & 15);
                if (i < items && row < p.rows) p.y[(int64_t)(i >> 4) * p.ldy + p.col0 + row] = v[w];
            }
        }
    };

    // end of a unit: the members hand their sums to member 0 through shared memory (two buffers, alternating by
    // unit, one named barrier per team and unit), member 0 adds them in member order
    int parity = 0;
    auto finish_unit = [&](int u) {
        if (W > 1) {
            float4* buf = pieces + ((size_t)parity * GEMV_WARPS + warp) * 32 * NG + lane;
            if (member != 0) {
#pragma unroll
                for (int gi = 0; gi < NG; gi++) buf[gi * 32] = make_float4(acc[gi][0], acc[gi][1], acc[gi][2], acc[gi][3]);
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(W * 32) : "memory");
            if (member == 0) {
                for (int j = 1; j < W; j++) {
#pragma unroll
                    for (int gi = 0; gi < NG; gi++) {
                        const float4 v = buf[(size_t)j * 32 * NG + gi * 32];
                        acc[gi][0] += v.x;
                        acc[gi][1] += v.y;
                        acc[gi][2] += v.z;
                        acc[gi][3] += v.w;
                    }
                }
            }
            parity ^= 1;
        }
        if (member == 0) store_unit(u);
#pragma unroll
        for (int gi = 0; gi < NG; gi++) acc[gi][0] = acc[gi][1] = acc[gi][2] = acc[gi][3] = 0.f;
    };

    if (ml == 0) {  // fewer k-tiles in the slice than members: this member only keeps the team's barriers company
        for (int u = ua; u < ub; u++) finish_unit(u);
        return;
    }
    int unit = ua, kk = 0;
    for (int g0 = 0; g0 < nt; g0 += DEPTH) {
        static_for<DEPTH>([&](auto J) {
            constexpr int j = decltype(J)::value;
            if (g0 + j < nt) {
                slots[j].template compute_n<NG>(acc, xg, (uint32_t)kk * XSTEP, c32 + (uint32_t)kk * CSTEP);
                load_next(slots[j]);
                if (++kk == ml) {
                    finish_unit(unit);
                    unit++;
                    kk = 0;
                }
            }
        });
    }
    stamp(4);
}

}  // namespace wf
