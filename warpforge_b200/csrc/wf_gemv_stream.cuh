// One-token decode GEMV: every warp streams its own run of tiles.
//
// A CTA's share of a weight (a contiguous range of tiles, row-tile major / k-tile minor, the same
// "stream-K" cut as the several-token kernel) is cut once more into sixteen contiguous runs, one per warp.
// A warp copies its run into a ring of its own with bulk asynchronous copies it issues itself (one or two
// tiles per copy, a few copies in flight), waits on its own mbarriers and keeps the sums of the row-tile it
// is walking in registers, so inside a run nothing is exchanged between warps: no per-tile release, no
// parking of partial sums per row-tile.  The copies of a warp run ahead over the following weights of a
// multi-op program as far as its ring is deep, so HBM keeps streaming across grid barriers.
//
// Where a run starts or ends inside a row-tile the warp writes the piece (sixteen sums) to shared memory;
// once per weight the warps meet on an mbarrier and the first holder of every cut row-tile adds the pieces
// in warp order.  A row-tile cut by the CTA's share boundary is then finished between CTAs exactly as in
// the several-token kernel (publish / collect through tagged scratch slots, bounded waits).
#pragma once
#include "wf_gemv_core.cuh"

namespace wf {

constexpr int WS_MAX_STAGES = 8;  // copies in flight per warp, at most
constexpr int WS_SLOTS = 4;       // hand-over generations (weights) whose pieces may be alive at once
// control block: abort word | full[GEMV_WARPS][WS_MAX_STAGES] | done[WS_SLOTS] | vacant[WS_SLOTS]
constexpr int WS_CTRL_BYTES = 1280;
static_assert(128 + (GEMV_WARPS * WS_MAX_STAGES + 2 * WS_SLOTS) * 8 <= WS_CTRL_BYTES, "control block");

struct WsPiece {  // the sums of one cut row-tile as far as one warp's run covers it
    float v[16];
};
constexpr int WS_PIECE_BYTES = WS_SLOTS * GEMV_WARPS * 2 * (int)sizeof(WsPiece);

template <int QT> struct WsGeom {
    static constexpr int CHUNK = Tile<QT>::BYTES <= 1280 ? 2 : 1;  // tiles per bulk copy
    static constexpr uint32_t STAGE_BYTES = CHUNK * Tile<QT>::BYTES;
};

// Shared memory of the one-token kernels:
//   control | pieces | block records and sums (32 bytes per 32 k) | digits (4 bytes per k) | rings [warp][stage]
inline size_t ws_fixed_smem(int kp) {
    size_t b = WS_CTRL_BYTES + WS_PIECE_BYTES + (size_t)(kp / 32) * 32 + (size_t)kp * 4 + 64;
    return (b + 127) & ~(size_t)127;
}
inline int ws_stages(int qt, int kp, int want) {
    const size_t fixed = ws_fixed_smem(kp), limit = 227 * 1024;
    const size_t stage = (size_t)GEMV_WARPS * (tile_bytes(qt) <= 1280 ? 2 : 1) * tile_bytes(qt);
    if (fixed + 2 * stage > limit) return 0;
    return (int)std::min<size_t>((limit - fixed) / stage, (size_t)std::min(want, WS_MAX_STAGES));
}

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

struct WsShare {  // a CTA's share of one weight
    const uint8_t* tiles;
    int t0, t1;
};

struct WsStream {       // one warp's ring position; carries over from weight to weight
    int p_op = -1;      // producer: weight whose tiles are being requested
    int p_t = 0, p_end = 0;
    const uint8_t* p_tiles = nullptr;
    int p_stage = 0;
    int c_stage = 0;    // consumer
    uint32_t c_lap = 0;
    uint32_t seq = 0;   // weights handed over so far
};

// This warp's run [a, b) of the share [t0, t1).
__device__ __forceinline__ void ws_run(int t0, int t1, int warp, int& a, int& b) {
    const int n = t1 - t0, q = n / GEMV_WARPS, r = n - q * GEMV_WARPS;
    a = t0 + warp * q + min(warp, r);
    b = a + q + (warp < r ? 1 : 0);
}

// Request the next copy of this warp's stream into the stage the producer side points at (which the caller
// knows to be free).  All lanes keep the position; lane 0 issues.  Returns without a copy once the program is
// exhausted.
template <int QT, class ShareFn>
__device__ __forceinline__ void ws_issue(WsStream& ss, ShareFn& share_of, int n_ops, int warp, int lane, uint32_t ring_w,
                                         uint32_t full_w, int stages) {
    using G = WsGeom<QT>;
    while (ss.p_t >= ss.p_end) {
        if (ss.p_op + 1 >= n_ops) {
            ss.p_op = n_ops;
            return;
        }
        ss.p_op++;
        const WsShare sh = share_of(ss.p_op);
        ws_run(sh.t0, sh.t1, warp, ss.p_t, ss.p_end);
        ss.p_tiles = sh.tiles;
    }
    const int cnt = min(G::CHUNK, ss.p_end - ss.p_t);
    if (lane == 0) {
        const uint32_t bytes = (uint32_t)cnt * Tile<QT>::BYTES, bar = full_w + ss.p_stage * 8;
        mbar_expect_tx(bar, bytes);
        bulk_load(ring_w + ss.p_stage * G::STAGE_BYTES, ss.p_tiles + (size_t)ss.p_t * Tile<QT>::BYTES, bytes, bar);
    }
    ss.p_t += cnt;
    ss.p_stage = ss.p_stage + 1 == stages ? 0 : ss.p_stage + 1;
}

struct WsBars {  // 32-bit shared addresses
    uint32_t full_w;  // this warp's full[stage]
    uint32_t done, vacant;
};
__device__ __forceinline__ WsBars ws_bars(uint8_t* smem, int warp) {
    WsBars b;
    b.full_w = smem_u32(smem + 128) + warp * WS_MAX_STAGES * 8;
    b.done = smem_u32(smem + 128) + GEMV_WARPS * WS_MAX_STAGES * 8;
    b.vacant = b.done + WS_SLOTS * 8;
    return b;
}
__device__ __forceinline__ void ws_bars_init(uint8_t* smem, int stages) {
    const uint32_t full = smem_u32(smem + 128);
    for (int w = 0; w < GEMV_WARPS; w++)
        for (int s = 0; s < stages; s++) mbar_init(full + (w * WS_MAX_STAGES + s) * 8, 1);
    const uint32_t done = full + GEMV_WARPS * WS_MAX_STAGES * 8;
    for (int s = 0; s < WS_SLOTS; s++) {
        mbar_init(done + s * 8, GEMV_WARPS);
        mbar_init(done + (WS_SLOTS + s) * 8, GEMV_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One weight, one warp: walk the run, hand the cut pieces over, finish the row-tiles this warp is first to hold.
//   x32 / c32 / s32: shared addresses of the staged digits, the block records and the activation sums;
//   emit_row(n, value): store output row n of this weight (called by one lane per row);
//   share_of(o): the CTA's share of weight o of the program (the producer side runs ahead of `op`).
template <int QT, class EmitRow, class ShareFn>
__device__ __forceinline__ void ws_consume(const WsShare& sh, int kt, int chunk_q, int chunk_r, int warp, int lane,
                                           uint32_t ring_w, const WsBars& bar, WsPiece* pieces, int stages, WsStream& ss,
                                           uint32_t x32, uint32_t c32, uint32_t s32, uint2* slots, int* status,
                                           uint32_t abort32, ShareFn& share_of, int n_ops, EmitRow&& emit_row) {
    using T = Tile<QT>;
    using R = TileRegs<QT>;
    using G = WsGeom<QT>;
    constexpr uint32_t XSTEP = T::K * 4, RSTEP = (T::K >> 5) * 16, SSTEP = (T::K >> 5) * 8;  // staged bytes per tile
    const int g = lane >> 2, q = lane & 3;
    const uint32_t lane_is_0 = lane == 0;
    int a, b;
    ws_run(sh.t0, sh.t1, warp, a, b);

    const int slot = (int)(ss.seq % WS_SLOTS);
    const uint32_t gen = ss.seq / WS_SLOTS;
    WsPiece* mine = pieces + ((size_t)slot * GEMV_WARPS + warp) * 2;
    // the pieces of the weight that used this slot last must have been read by everybody
    if (gen > 0) mbar_wait_or_abort(bar.vacant + slot * 8, (gen - 1) & 1, abort32);

    // pieces this warp writes: row-tile and whether this warp is the first of the CTA to hold it
    int npieces = 0, rtag0 = 0, rtag1 = 0;
    bool first0 = false, first1 = false;
    if (a < b) {
        int rt = a / kt, kk = a - rt * kt;
        bool starts_here = kk == 0;  // the row-tile being walked began inside this run
        const uint32_t is_lo = lane < 16 ? 1u : 0u;  // this lane feeds the low k-slots of the MMAs
        const uint32_t x0 = x32 + lane * 16, rec0 = c32 + q * 16, sx0 = s32 + q * 8;
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

        for (int t = a; t < b;) {
            const int cnt = min(G::CHUNK, b - t);
            mbar_wait_or_abort(bar.full_w + ss.c_stage * 8, ss.c_lap & 1, abort32);
            const uint32_t stage32 = ring_w + ss.c_stage * G::STAGE_BYTES + lane * 16;
#pragma unroll
            for (int i = 0; i < G::CHUNK; i++) {
                if (i < cnt) {
                    R regs;
                    regs.template load<1>(stage32 + i * T::BYTES, lane);
                    if (i == cnt - 1) {  // the stage is free once its last tile sits in registers: request the next copy into it
                        __syncwarp();
                        ws_issue<QT>(ss, share_of, n_ops, warp, lane, ring_w, bar.full_w, stages);
                    }
                    regs.compute_q8(acc, qa, dg, is_lo);
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
            }
            t += cnt;
            if (++ss.c_stage == stages) {
                ss.c_stage = 0;
                ss.c_lap++;
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
            float v[1];
            v[0] = lane < 16 ? mine[pi].v[lane] : 0.f;
            // the following warps whose runs begin inside the row-tile hold its next pieces, each as its first piece
            for (int w2 = warp + 1; w2 < GEMV_WARPS; w2++) {
                const int a2 = sh.t0 + w2 * rq + min(w2, rr);
                if (a2 >= row_end || (w2 >= rr && rq == 0)) break;  // beyond the row-tile, or a warp without tiles
                if (lane < 16) v[0] += all[w2 * 2].v[lane];
            }
            const bool starts = r * kt >= sh.t0, ends = (r + 1) * kt <= sh.t1;
            if (!starts) {
                publish_piece<16>(slots + (size_t)blockIdx.x * 128, v, lane, status);
            } else {
                if (!ends) collect_pieces<16>(slots, v, lane, (r + 1) * kt, chunk_q, chunk_r, status);
                if (lane < 16) emit_row(r * 16 + lane, v[0]);
            }
        }
    }
    __syncwarp();
    mbar_arrive_if(bar.vacant + slot * 8, lane_is_0);
    ss.seq++;
}

}  // namespace wf
