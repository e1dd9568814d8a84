// One-token decode GEMV: every warp streams its own run of tiles, from global memory straight into registers.
//
// A CTA's share of a weight (a contiguous range of tiles, row-tile major / k-tile minor) is cut once more into
// sixteen contiguous runs, one per warp.  The tile layout is already in MMA fragment order -- the sixteen bytes
// a lane needs of a plane half are contiguous and a warp's load covers 512 contiguous bytes -- so a warp loads
// its tiles with plain 16-byte global loads into registers, a few tiles ahead of the one it is multiplying
// (software pipeline over DEPTH register sets).  The weights never pass through shared memory, whose bandwidth
// is left to the activation digits; measured on a ring-of-bulk-copies form of this kernel, tile loads and
// copy writes alone took 19 of the 24 shared-memory cycles a tile cost, more than the integer pipe.
// The load requests of a warp run ahead over the following weights of a multi-op program (the first tiles of
// the next projection are in flight while the grid barrier and the activation staging run).
//
// Inside a run nothing is exchanged between warps: the sums of the row-tile being walked stay in registers.
// Where a run starts or ends inside a row-tile the warp writes the piece (sixteen sums) to shared memory; once
// per weight the warps meet on an mbarrier and the first holder of every cut row-tile adds the pieces in warp
// order.  A row-tile cut by the CTA's share boundary is then finished between CTAs exactly as in the
// several-token kernel (publish / collect through tagged scratch slots, bounded waits).
#pragma once
#include <utility>

#include "wf_gemv_core.cuh"

namespace wf {

// for (j = 0 .. N-1) with j a compile-time constant in the body: f(std::integral_constant<int, j>{})
template <class F, int... I>
__device__ __forceinline__ void static_for_impl(F& f, std::integer_sequence<int, I...>) {
    (f(std::integral_constant<int, I>{}), ...);
}
template <int N, class F> __device__ __forceinline__ void static_for(F&& f) { static_for_impl(f, std::make_integer_sequence<int, N>{}); }

constexpr int WS_SLOTS = 4;         // hand-over generations (weights) whose pieces may be alive at once
constexpr int WS_TABLE_OPS = 256;   // weights of a program whose shares are kept in shared memory
// control block: abort word | failure latch | done[WS_SLOTS] | vacant[WS_SLOTS]
constexpr int WS_CTRL_BYTES = 256;
static_assert(128 + 2 * WS_SLOTS * 8 <= WS_CTRL_BYTES, "control block");

struct WsPiece {  // the sums of one cut row-tile as far as one warp's run covers it
    float v[16];
};
constexpr int WS_PIECE_BYTES = WS_SLOTS * GEMV_WARPS * 2 * (int)sizeof(WsPiece);

// Tiles a warp holds in registers.  The per-projection kernel has room for six 1.1 KB tiles; the program kernel, which
// keeps more state alive around the tile loop, spills from five on (506 against 791 tok/s at six), so it holds four.
#ifndef WS_DEPTH_SINGLE
#define WS_DEPTH_SINGLE 6
#endif
template <int QT, bool PROGRAM> struct WsGeom {
    static constexpr int DEPTH = Tile<QT>::BYTES <= 1280 ? (PROGRAM ? 4 : WS_DEPTH_SINGLE) : 2;
};

// Shared memory of the one-token kernels:
//   control | pieces | share table (32 bytes per weight) | block records and sums (32 bytes per 32 k) | digits (8 bytes per k)
inline size_t ws_smem(int kp, int table_ops) {
    size_t b = WS_CTRL_BYTES + WS_PIECE_BYTES + (size_t)table_ops * 32 + (size_t)(kp / 32) * 32 + (size_t)kp * 8 + 64;
    return (b + 127) & ~(size_t)127;
}
inline bool ws_fits(int kp, int table_ops) { return ws_smem(kp, table_ops) <= 227 * 1024; }

// How a weight of rt row-tiles x kt k-tiles is cut over the CTAs.  Stream-K (equal numbers of tiles, row-tiles
// cut wherever a share ends) balances perfectly, but every cut row-tile is finished between two CTAs through
// global memory, a chain of L2 round trips worth about WS_CUT_PENALTY_TILES tiles of streaming that the warps
// doing it pay on every weight.  Whole row-tiles per CTA avoid that at the price of an uneven split, so the
// cheaper of the two by this estimate is taken.
constexpr int WS_CUT_PENALTY_TILES = 48;
struct WsSplit {
    int ctas;     // CTAs that get work
    int aligned;  // 1: shares are whole row-tiles and chunk_q / chunk_r count row-tiles; 0: tiles
    int chunk_q, chunk_r;
};
inline WsSplit ws_split(int sm_count, int64_t rt, int64_t kt) {
    const int64_t total = rt * kt;
    const int64_t a_ctas = std::max<int64_t>(1, std::min<int64_t>(sm_count, rt));
    const int64_t a_cost = ((rt + a_ctas - 1) / a_ctas) * kt;
    const int64_t s_ctas = gemv_ctas(sm_count, total);
    const int64_t s_cost = (total + s_ctas - 1) / s_ctas + WS_CUT_PENALTY_TILES;
    WsSplit sp;
    if (a_cost <= s_cost) {
        sp.ctas = (int)a_ctas;
        sp.aligned = 1;
        sp.chunk_q = (int)(rt / a_ctas);
        sp.chunk_r = (int)(rt % a_ctas);
    } else {
        sp.ctas = (int)s_ctas;
        sp.aligned = 0;
        sp.chunk_q = (int)(total / s_ctas);
        sp.chunk_r = (int)(total % s_ctas);
    }
    return sp;
}
// CTA bx's share [t0, t1) in tiles under a split.
WF_HD void ws_cta_share(int bx, int ctas, int chunk_q, int chunk_r, int aligned, int kt, int& t0, int& t1) {
    const int u0 = bx * chunk_q + (bx < chunk_r ? bx : chunk_r);
    const int u1 = bx < ctas ? u0 + chunk_q + (bx < chunk_r ? 1 : 0) : u0;
    t0 = aligned ? u0 * kt : u0;
    t1 = aligned ? u1 * kt : u1;
}

struct WsShare {  // a CTA's share of one weight (32 bytes: the entry of the share table)
    const uint8_t* tiles;
    int t0, t1;  // tiles
    int kt;
    int flags;
    int pad[2];
};

// This warp's run [a, b) of the share [t0, t1).
__device__ __forceinline__ void ws_run(int t0, int t1, int warp, int& a, int& b) {
    const int n = t1 - t0, q = n / GEMV_WARPS, r = n - q * GEMV_WARPS;
    a = t0 + warp * q + min(warp, r);
    b = a + q + (warp < r ? 1 : 0);
}

// Where this warp's load requests stand in the program.  A warp's stream is the sequence of its runs, weight after
// weight, cut into groups of DEPTH tiles that never straddle two weights.
struct WsCursor {
    int op = -1;
    int t = 0, end = 0;
    const uint8_t* tiles = nullptr;
};
// The next group to request: address of its first tile and its number of tiles (0 once the program is exhausted).
template <int QT, int DEPTH, class ShareFn>
__device__ __forceinline__ void ws_next_group(WsCursor& c, ShareFn& share_of, int n_ops, int warp, const uint8_t*& base, int& cnt) {
    while (c.t >= c.end) {
        if (c.op + 1 >= n_ops) {
            c.op = n_ops;
            base = nullptr;
            cnt = 0;
            return;
        }
        c.op++;
        const WsShare sh = share_of(c.op);
        ws_run(sh.t0, sh.t1, warp, c.t, c.end);
        c.tiles = sh.tiles;
    }
    cnt = min(DEPTH, c.end - c.t);
    base = c.tiles + (size_t)c.t * Tile<QT>::BYTES;
    c.t += cnt;
}
// The two lane pointers a tile is loaded through (see TileRegs::load_global).
template <int QT> struct WsLanePtrs {
    const uint8_t* pc;
    const uint8_t* ps;
    __device__ __forceinline__ WsLanePtrs(const uint8_t* base, int lane)
        : pc(base + lane * 16), ps(base + TileRegs<QT>::lane_scale_offset(lane)) {}
};
// Request the first group of the stream (the weights depend on nothing, so this comes before any wait).
template <int QT, int DEPTH, class ShareFn>
__device__ __forceinline__ void ws_prime(TileRegs<QT> (&slots)[DEPTH], WsCursor& c, ShareFn& share_of, int n_ops,
                                         int warp, int lane) {
    const uint8_t* base;
    int cnt;
    ws_next_group<QT, DEPTH>(c, share_of, n_ops, warp, base, cnt);
    const WsLanePtrs<QT> lp(base, lane);
    static_for<DEPTH>([&](auto J) {
        constexpr int j = decltype(J)::value;
        if (j < cnt) slots[j].template load_global<j * Tile<QT>::BYTES>(lp.pc, lp.ps);
    });
}
// Clear the digit words once per kernel: the staging only ever writes the word of the half a lane feeds.
__device__ __forceinline__ void ws_clear_digits(uint8_t* xd, int kp, int nthreads) {
    uint4* p = reinterpret_cast<uint4*>(xd);
    for (int i = threadIdx.x; i < kp / 2; i += nthreads) p[i] = make_uint4(0u, 0u, 0u, 0u);
}

struct WsBars {  // 32-bit shared addresses
    uint32_t done, vacant;  // [WS_SLOTS]: every warp has written its pieces / is through with the weight
};
__device__ __forceinline__ WsBars ws_bars(uint8_t* smem) {
    WsBars b;
    b.done = smem_u32(smem + 128);
    b.vacant = b.done + WS_SLOTS * 8;
    return b;
}
__device__ __forceinline__ void ws_bars_init(uint8_t* smem) {
    const uint32_t done = smem_u32(smem + 128);
    for (int s = 0; s < 2 * WS_SLOTS; s++) mbar_init(done + s * 8, GEMV_WARPS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One weight, one warp: walk the run, hand the cut pieces over, finish the row-tiles this warp is first to hold.
//   slots: the register sets holding the first group of this run (requested earlier); cur: the request cursor;
//   x32 / c32 / s32: shared addresses of the staged digits, the block records and the activation sums;
//   emit_row(n, value): store output row n of this weight (called by one lane per row);
//   share_of(o): the CTA's share of weight o of the program.
template <int QT, int DEPTH, class EmitRow, class ShareFn>
__device__ __forceinline__ void ws_consume(const WsShare& sh, int chunk_q, int chunk_r, int warp, int lane,
                                           TileRegs<QT> (&slots)[DEPTH], WsCursor& cur, const WsBars& bar,
                                           WsPiece* pieces, uint32_t& seq, uint32_t x32, uint32_t c32, uint32_t s32,
                                           uint2* slots_g, int* status, uint32_t abort32, ShareFn& share_of, int n_ops,
                                           EmitRow&& emit_row) {
    using T = Tile<QT>;
    constexpr uint32_t XSTEP = (T::K / 128) * Q8_UNIT_BYTES, RSTEP = (T::K >> 5) * 16, SSTEP = (T::K >> 5) * 8;  // staged bytes per tile
    const int g = lane >> 2, q = lane & 3, kt = sh.kt;
    const uint32_t lane_is_0 = lane == 0;
    int a, b;
    ws_run(sh.t0, sh.t1, warp, a, b);
    const int len = b - a;

    const int slot = (int)(seq % WS_SLOTS);
    const uint32_t gen = seq / WS_SLOTS;
    WsPiece* mine = pieces + ((size_t)slot * GEMV_WARPS + warp) * 2;
    // the pieces of the weight that used this slot last must have been read by everybody
    if (gen > 0) mbar_wait_or_abort(bar.vacant + slot * 8, (gen - 1) & 1, abort32);

    // pieces this warp writes: row-tile and whether this warp is the first of the CTA to hold it
    int npieces = 0, rtag0 = 0, rtag1 = 0;
    bool first0 = false, first1 = false;
    if (len > 0) {
        int rt = __float2int_rz(__fdividef((float)a, (float)kt)), kk = a - rt * kt;  // a / kt without the integer division
        while (kk < 0) {  // the float quotient is off by one at most for tile counts below 2^24; loops cover the rest
            rt--;
            kk += kt;
        }
        while (kk >= kt) {
            rt++;
            kk -= kt;
        }
        bool starts_here = kk == 0;  // the row-tile being walked began inside this run
        const uint32_t x0 = x32 + lane * 32, rec0 = c32 + q * 16, sx0 = s32 + q * 8;
        Q8Addr qa;
        qa.x = x0 + (uint32_t)kk * XSTEP;
        qa.rec = rec0 + (uint32_t)kk * RSTEP;
        qa.sx = sx0 + (uint32_t)kk * SSTEP;
        Q8Digits dg;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};

        auto flush = [&](bool ends) {
            // the four lanes of a quad hold different digits / blocks of the same two rows
            acc[0] += __shfl_xor_sync(0xFFFFFFFFu, acc[0], 1);
            acc[2] += __shfl_xor_sync(0xFFFFFFFFu, acc[2], 1);
            acc[0] += __shfl_xor_sync(0xFFFFFFFFu, acc[0], 2);
            acc[2] += __shfl_xor_sync(0xFFFFFFFFu, acc[2], 2);
            if (starts_here && ends) {  // a whole row-tile inside this run: final
                if (q == 0) {
                    emit_row(rt * 16 + g, acc[0]);
                    emit_row(rt * 16 + g + 8, acc[2]);
                }
            } else {
                WsPiece* p = mine + npieces;
                if (q == 0) {
                    p->v[g] = acc[0];
                    p->v[g + 8] = acc[2];
                }
                const bool first = starts_here || warp == 0;
                if (npieces == 0) {
                    rtag0 = rt;
                    first0 = first;
                } else {
                    rtag1 = rt;
                    first1 = first;
                }
                npieces++;
            }
            acc[0] = acc[2] = 0.f;
        };

        for (int g0 = 0; g0 < len; g0 += DEPTH) {
            // the group after this one in the warp's stream (maybe of a later weight): requested slot by slot as
            // the slots of this group are used up
            const uint8_t* nbase;
            int ncnt;
            ws_next_group<QT, DEPTH>(cur, share_of, n_ops, warp, nbase, ncnt);
            const WsLanePtrs<QT> lp(nbase, lane);
            if (g0 + DEPTH <= len && kk + DEPTH <= kt && ncnt == DEPTH) {
                // a whole group inside one row-tile, a whole group to request: straight-line code, immediate offsets
                static_for<DEPTH>([&](auto J) {
                    constexpr int j = decltype(J)::value;
                    slots[j].template compute_q8<j>(acc, qa, dg);
                    slots[j].template load_global<j * T::BYTES>(lp.pc, lp.ps);
                });
                kk += DEPTH;
                qa.x += DEPTH * XSTEP;
                qa.rec += DEPTH * RSTEP;
                qa.sx += DEPTH * SSTEP;
                if (kk == kt) {
                    flush(true);
                    kk = 0;
                    rt++;
                    starts_here = true;
                    qa.x = x0;
                    qa.rec = rec0;
                    qa.sx = sx0;
                }
            } else {
                static_for<DEPTH>([&](auto J) {
                    constexpr int j = decltype(J)::value;
                    if (g0 + j < len) {
                        slots[j].template compute_q8<0>(acc, qa, dg);
                        if (++kk == kt) {
                            flush(true);
                            kk = 0;
                            rt++;
                            starts_here = true;
                            qa.x = x0;
                            qa.rec = rec0;
                            qa.sx = sx0;
                        } else {
                            qa.x += XSTEP;
                            qa.rec += RSTEP;
                            qa.sx += SSTEP;
                        }
                    }
                    if (j < ncnt) slots[j].template load_global<j * T::BYTES>(lp.pc, lp.ps);
                });
            }
        }
        if (kk != 0) flush(false);
    }

    // ---- hand-over: every warp reports, the first holder of a cut row-tile finishes it
    __syncwarp();
    mbar_arrive_if(bar.done + slot * 8, lane_is_0);
    if ((npieces > 0 && first0) || (npieces > 1 && first1)) {
        mbar_wait_or_abort(bar.done + slot * 8, gen & 1, abort32);
        const WsPiece* all = pieces + (size_t)slot * GEMV_WARPS * 2;
        const int n = sh.t1 - sh.t0, rq = n / GEMV_WARPS, rr = n - rq * GEMV_WARPS;
        for (int pi = 0; pi < npieces; pi++) {
            if (!(pi == 0 ? first0 : first1)) continue;  // an earlier warp holds this row-tile first
            const int r = pi == 0 ? rtag0 : rtag1;
            const int row_end = min((r + 1) * kt, sh.t1);
            // the following warps whose runs begin inside the row-tile hold its next pieces, each as its first piece:
            // all loads first (they do not depend on each other), then the additions in warp order
            float pc[GEMV_WARPS];
            const int li = lane & 15;
#pragma unroll
            for (int d = 1; d < GEMV_WARPS; d++) {
                const int w2 = warp + d, a2 = sh.t0 + w2 * rq + min(w2, rr);
                pc[d] = (w2 < GEMV_WARPS && a2 < row_end) ? all[w2 * 2].v[li] : 0.f;
            }
            float v[1];
            v[0] = mine[pi].v[li];
#pragma unroll
            for (int d = 1; d < GEMV_WARPS; d++) v[0] += pc[d];
            const bool starts = r * kt >= sh.t0, ends = (r + 1) * kt <= sh.t1;
            if (!starts) {
                publish_piece<16>(slots_g + (size_t)blockIdx.x * 128, v, lane, status);
            } else {
                if (!ends) collect_pieces<16>(slots_g, v, lane, (r + 1) * kt, chunk_q, chunk_r, status);
                if (lane < 16) emit_row(r * 16 + lane, v[0]);
            }
        }
    }
    __syncwarp();
    mbar_arrive_if(bar.vacant + slot * 8, lane_is_0);
    seq++;
}

}  // namespace wf
