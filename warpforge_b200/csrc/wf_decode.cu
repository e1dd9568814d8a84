// A decode step as ONE persistent kernel: a "program" of quantized GEMVs (the projections of
// a token, in order) run by one CTA per SM.  This removes the per-launch prologue and tail that
// dominate microsecond-scale GEMV kernels, and lets the weights of the next projection be on
// their way while the current one finishes.
//
// One token (gemv1_program_kernel): every warp streams its own run of tiles from global memory
// straight into registers (wf_gemv_stream.cuh); its load requests run ahead over the following
// projections, so the first tiles of the next projection are in flight while the grid barrier and
// the staging of the next activations run.  Projections that read the same activations (Wq / Wk /
// Wv, Wgate / Wup) are cut as one list of row-tiles.  Several tokens (gemv_program_kernel): the
// producer thread of each CTA walks the whole program and keeps a shared-memory ring of tiles full
// with bulk copies; sixteen consumer warps take their tile out of each ring stage.
//
// Projections that read an earlier projection's output are separated by a grid barrier
// (an arrival counter in global memory, bounded spins).  With row-sharded tensor parallelism
// the all-gather is fused into the GEMV epilogue: every rank stores its rows of y into the
// other ranks' landing buffers over NVLink as 8-byte {value, tag} words -- one store carries
// the data and the proof that it arrived, so no fence and no flag round trip is needed --
// and before the barrier each rank's CTAs poll their slice of the landing buffer until the
// tag of the current barrier shows, copying the values into the plain y.  No collective is
// launched.  (No multicast loads and no waits between separately launched kernels on one
// GPU are involved: each rank runs exactly one kernel on its own GPU.)  The tag is the barrier's
// number since the program was created, cut to 32 bits; a landing buffer is written again two
// dependent barriers later at the earliest, so a stale tag could only be mistaken for a current
// one after 2^32 barriers without the buffer being rewritten, which cannot happen.
//
// The arithmetic replaces the reference's per-op launches at
// warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/ops/DotGeneralKernel.java:263-283.
#include <string.h>

#include "wf_gemv_stream.cuh"

namespace wf {

constexpr int PROG_MAX_WORLD = 8;
constexpr int PROG_BARRIER_SPINS = 1 << 24;
constexpr int OP_NEW_X = 1;    // stage activations before this op (otherwise it reuses the staged ones)
constexpr int OP_DEPENDS = 2;  // the activations were produced by earlier ops: grid (and rank) barrier first

struct ProgOp {
    const uint8_t* tiles;
    const void* x;
    float* y;                  // this rank's plain fp32 output [m, n_total]
    uint2* ll[PROG_MAX_WORLD]; // every rank's landing buffer for this op [m, n_total] {value, tag}; own at [rank]
    int n_total;
    int aligned;               // one-token kernel: chunk_q / chunk_r count whole row-tiles
    int64_t ldy, col0;
    int rows, k, kt, rt;
    int chunk_q, chunk_r;      // CTA b < ctas owns tiles [b*q + min(b,r), (b+1)*q + min(b+1,r)); the others none
    int flags, ctas;
    // one-token kernel: what is fused into the staging of x and into the store of y
    int x_kind;                // XK_BF16 / XK_F32 / XK_RMSNORM_F32 / XK_SWIGLU_F32 (wf_gemv_core.cuh)
    float eps;                 // rms_norm
    const float* x_aux;        // rms_norm: gamma [k] or null; swiglu: the up projection's output [k]
    const float* residual;     // y[n] = (x . W[n]) + residual[n] (null: plain store); may be y itself
};

struct ProgSync {                     // device memory owned by the program
    unsigned long long arrive;        // CTAs arrived at grid barriers, monotonic; alone on its 128-byte line
    unsigned long long pad0[15];
    unsigned long long epoch;         // barriers completed by earlier runs
    unsigned int done_ctas;           // CTAs that left the current run
    unsigned int pad1;
};

struct ProgParams {
    const ProgOp* ops;
    int n_ops, m;
    uint2* scratch;                   // [2][ctas][128] fix-up slots, alternating by op
    int* status;
    ProgSync* sync;
    int world, rank;
    int stages, sx, kp_max;
    int n_barriers;
    unsigned long long* timing;  // optional [ctas][64]: globaltimer at op boundaries of the first ops (salt 2)
    const int2* shares;          // one-token kernel: [n_ops][ctas] tiles {t0, t1} of every CTA's share of every op
};

__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void st_slot_sys(uint2* p, uint2 v) {
    const unsigned long long w = ((unsigned long long)v.y << 32) | v.x;
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_slot_sys(const uint2* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}

// What the consumer threads of both program kernels share: the landing of the other ranks' rows, the grid
// barrier and the way out.  A wait that ran out anywhere in this CTA, or a failure another CTA or an earlier
// kernel reported through the status word, is latched in shared memory (`failed`): from then on no landing
// poll and no barrier spin is started, so that a program whose peer has gone ends within about one
// timeout instead of one timeout per projection.
struct ProgRun {
    const ProgParams& P;
    volatile int* failed;  // CTA-wide latch in shared memory
    unsigned long long epoch;
    int barriers = 0, land_from = 0;

    __device__ __forceinline__ void consumers_sync() const { asm volatile("bar.sync 1, %0;" ::"n"(GEMV_CONSUMERS) : "memory"); }
    __device__ __forceinline__ unsigned int tag() const { return (unsigned int)(epoch + (unsigned long long)barriers + 1); }

    // Wait for the other ranks' rows of ops [first, last) and copy them into y.  The CTAs split the elements;
    // each element is polled until it carries this barrier's tag.
    __device__ __forceinline__ void land(int first, int last, unsigned int want_tag) {
        if (P.world == 1 || *failed) return;
        for (int o2 = first; o2 < last; o2++) {
            const ProgOp& op2 = P.ops[o2];
            const int total = P.m * op2.n_total;
            const uint2* mine = op2.ll[P.rank];
            for (int e = (int)blockIdx.x * GEMV_CONSUMERS + threadIdx.x; e < total; e += gridDim.x * GEMV_CONSUMERS) {
                const int col = e % op2.n_total;
                if (col >= (int)op2.col0 && col < (int)op2.col0 + op2.rows) continue;  // my own rows are already in y
                uint2 v;
                int spins = 0;
                do {
                    v = ld_slot_sys(mine + e);
                    if (v.y == want_tag) break;
                    __nanosleep(20);
                } while (++spins < GEMV_FIXUP_SPINS && !*failed);
                if (v.y != want_tag) {
                    atomicOr(P.status, STATUS_PEER_WAIT_TIMEOUT);
                    *failed = 1;
                    return;
                }
                op2.y[e] = __uint_as_float(v.x);
            }
        }
    }

    // Grid barrier number `barriers` of this run; with several ranks the landing comes first, so that after the
    // barrier every rank's y holds all rows.
    __device__ __forceinline__ void grid_barrier(int o_now) {
        consumers_sync();  // every warp of this CTA has written its y values and finished its row-tiles
        const unsigned long long idx = epoch + (unsigned long long)barriers + 1;  // 1-based barrier number
        land(land_from, o_now, (unsigned int)idx);
        land_from = o_now;
        if (P.world > 1) consumers_sync();
        if (threadIdx.x == 0) {
            // a failure reported by another CTA, another rank's stalled store or an earlier kernel: stop waiting
            int st;
            asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(st) : "l"(P.status) : "memory");
            if (st != 0) *failed = 1;
            const unsigned long long want = idx * gridDim.x;
            int spins = 0;
            // one release-add (no value comes back, the poll starts at once) and acquire loads: the y rows this
            // CTA wrote before the bar.sync above are ordered before the add, the reads after the barrier after
            // the load that saw the last arrival
            asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(&P.sync->arrive), "l"(1ULL) : "memory");
            // a short pause between polls: 148 pollers reading the line back to back slow the arrivals down
            if (!*failed) {
                while (ld_acquire_gpu(&P.sync->arrive) < want && ++spins < PROG_BARRIER_SPINS) __nanosleep(50);
                if (spins >= PROG_BARRIER_SPINS) {
                    atomicOr(P.status, STATUS_PEER_WAIT_TIMEOUT);
                    *failed = 1;
                }
            }
        }
        barriers++;
        consumers_sync();
    }

    // The rows of the last ops land before the kernel ends (tag of the barrier that never comes); the last CTA
    // out advances the epoch for the next run.
    __device__ __forceinline__ void leave() {
        consumers_sync();
        land(land_from, P.n_ops, tag());
        consumers_sync();
        if (threadIdx.x == 0) {
            __threadfence();
            const unsigned int d = atomicAdd(&P.sync->done_ctas, 1u);
            if (d == gridDim.x - 1) {
                P.sync->done_ctas = 0;
                // CTAs that skipped barriers after a failure would leave `arrive` short: resynchronise it
                P.sync->arrive = (epoch + (unsigned long long)P.n_barriers + 1) * gridDim.x;
                __threadfence();
                st_release_gpu(&P.sync->epoch, epoch + (unsigned long long)P.n_barriers + 1);  // +1: the final landing's tag
            }
        }
    }
};

// The row-shard gather of the one-token kernel: one output value to every other rank's landing buffer, tagged with
// the barrier it belongs to.  Out of line: the tile loop stores rows in several places and stays small this way.
static __device__ __noinline__ void emit_to_peers(uint2* const* ll, int world, int rank, int64_t off, float v, unsigned int tag) {
    const uint2 word = make_uint2(__float_as_uint(v), tag);
    for (int r = 0; r < world; r++)
        if (r != rank) st_slot_sys(ll[r] + off, word);
}

// This CTA's share of op `o`.
__device__ __forceinline__ void prog_share(const ProgOp& op, int bx, int& t0, int& t1) {
    ws_cta_share(bx, op.ctas, op.chunk_q, op.chunk_r, op.aligned, op.kt, t0, t1);
}

// Several tokens (2..8).  Shared memory: ctrl | partial sums | cinit (kp_max) | staged x | ring.
template <int QT, int XC>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_program_kernel(const ProgParams P) {
    using T = Tile<QT>;
    using R = TileRegs<QT>;
    constexpr int NSLOT = Slots<XC>::N, ELEMS = Slots<XC>::ELEMS;
    extern __shared__ __align__(128) uint8_t smem[];
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
    const BarrierSet bar = barrier_set(smem);
    float* partial = reinterpret_cast<float*>(smem + GEMV_CTRL_BYTES);       // [NSLOT][GEMV_WARPS][ELEMS]
    float4* cinit = reinterpret_cast<float4*>(partial + NSLOT * GEMV_WARPS * ELEMS);  // [kp_max/32][4]
    uint8_t* xs = reinterpret_cast<uint8_t*>(cinit + (P.kp_max >> 5) * 4);   // [m][sx]
    uint8_t* ring = smem + (((size_t)(xs - smem) + (size_t)P.m * P.sx + 127) & ~(size_t)127);

    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    const int bx = blockIdx.x, stages = P.stages;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        reinterpret_cast<volatile int*>(smem)[1] = 0;
        barrier_set_init<XC>(bar, stages);
    }
    __syncthreads();

    if (warp == GEMV_WARPS) {
        // ------------------------------------------------ producer: the whole program, as far ahead as the ring allows
        if (lane == 0) {
            WalkState pos;
            for (int o = 0; o < P.n_ops && !*abort_flag; o++) {
                const ProgOp& op = P.ops[o];
                int t0, t1;
                prog_share(op, bx, t0, t1);
                produce_share<QT>(op.tiles, t0, t1, smem_u32(ring), bar, stages, pos, abort_flag);
            }
        }
        return;
    }

    // ---------------------------------------------------- consumers
    ProgRun run{P, reinterpret_cast<volatile int*>(smem) + 1, ld_acquire_gpu(&P.sync->epoch)};
    const uint8_t* xrow = xs + (size_t)(g < P.m ? g : P.m - 1) * P.sx;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    WalkState st;
    bool failed = false;
    const uint32_t x32 = smem_u32(xrow) + q * 16, c32 = smem_u32(cinit) + q * 16;

    int stamp_i = 0;
    auto stamp = [&]() {
        if (P.timing != nullptr && threadIdx.x == 0 && stamp_i < 64) {
            unsigned long long tm;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm));
            P.timing[(size_t)bx * 64 + stamp_i] = tm;
        }
        stamp_i++;
    };
    stamp();

    for (int o = 0; o < P.n_ops && !failed; o++) {
        const ProgOp& op = P.ops[o];
        const int flags = op.flags;
        const int kt = op.kt;
        int t0, t1;
        prog_share(op, bx, t0, t1);
        uint2* slots = P.scratch + (size_t)(o & 1) * gridDim.x * 128;

        stamp();  // op start (4 stamps per op: start, after barrier, after staging, after compute)
        if (flags & OP_NEW_X) {
            if (flags & OP_DEPENDS) run.grid_barrier(o);
            else run.consumers_sync();  // the staged activations are about to be replaced
            stamp();
            GemvParams sp{};
            sp.x = op.x;
            sp.m = P.m;
            sp.k = op.k;
            sp.ldx = op.k;
            sp.x_f32 = 0;
            sp.sx = P.sx;
            stage_x(sp, xs, reinterpret_cast<float*>(cinit), kt * T::K, R::BETA, GEMV_CONSUMERS);
            run.consumers_sync();
            stamp();
        } else {
            stamp();
            stamp();
        }

        // y goes to every rank's buffer: the row-shard gather happens here
        auto emit = [&](int rt, const float* buf) {
            for (int i = lane; i < ELEMS; i += 32) {
                const int col = i >> 4, n = rt * 16 + (i & 15);
                if (col < P.m && n < op.rows) {
                    const int64_t off = (int64_t)col * op.ldy + op.col0 + n;
                    const float v = buf[i];
                    op.y[off] = v;
                    const uint2 word = make_uint2(__float_as_uint(v), run.tag());
                    for (int r = 0; r < P.world; r++)
                        if (r != P.rank) st_slot_sys(op.ll[r] + off, word);
                }
            }
        };
        consume_share<QT, XC>(t0, t1, kt, op.chunk_q, op.chunk_r, warp, lane, smem_u32(ring), bar, partial, stages, st, x32, c32,
                              slots, P.status, smem_u32(const_cast<int*>(abort_flag)), acc, emit);
        if (*abort_flag) failed = true;
        stamp();
    }
    if (failed) {
        if (lane == 0) atomicOr(P.status, STATUS_GEMV_FIXUP_TIMEOUT);
        *run.failed = 1;
        drain_after_abort();
    }
    run.leave();
}

// One token.  Shared memory: control | pieces | share table | block records | digits (wf_gemv_stream.cuh); all 512
// threads are consumers, every warp loads its own tiles into registers and runs ahead over the following projections.
template <int QT>
__global__ void __launch_bounds__(GEMV_CONSUMERS, 1) gemv1_program_kernel(const ProgParams P) {
    using T = Tile<QT>;
    using R = TileRegs<QT>;
    extern __shared__ __align__(128) uint8_t smem[];
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
    WsPiece* pieces = reinterpret_cast<WsPiece*>(smem + WS_CTRL_BYTES);
    WsShare* table = reinterpret_cast<WsShare*>(smem + WS_CTRL_BYTES + WS_PIECE_BYTES);
    const int n_table = min(P.n_ops, WS_TABLE_OPS);
    uint8_t* recs = reinterpret_cast<uint8_t*>(table + n_table);
    uint8_t* xd = recs + (size_t)(P.kp_max >> 5) * 32;

    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int bx = blockIdx.x;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        reinterpret_cast<volatile int*>(smem)[1] = 0;
        ws_bars_init(smem);
    }
    // this CTA's share of every projection, once, into shared memory: the load requests that run ahead and the
    // consumers read it from there instead of chasing descriptors in global memory inside the tile loop
    auto share_from_global = [&](int o) {
        const ProgOp& op = P.ops[o];
        WsShare sh;
        sh.tiles = op.tiles;
        const int2 t = P.shares[(size_t)o * gridDim.x + bx];
        sh.t0 = t.x;
        sh.t1 = t.y;
        sh.kt = op.kt;
        sh.flags = op.flags;
        sh.pad[0] = sh.pad[1] = 0;
        return sh;
    };
    for (int o = threadIdx.x; o < n_table; o += GEMV_CONSUMERS) table[o] = share_from_global(o);
    ws_clear_digits(xd, P.kp_max, GEMV_CONSUMERS);
    __syncthreads();

    const WsBars bar = ws_bars(smem);
    auto share_of = [&](int o) { return o < n_table ? table[o] : share_from_global(o); };
    // the weights depend on nothing: request the first tiles of this warp's stream at once
    constexpr int DEPTH = WsGeom<QT, true>::DEPTH;
    R slots[DEPTH];
    WsCursor cur;
    ws_prime<QT, DEPTH>(slots, cur, share_of, P.n_ops, warp, lane);

    ProgRun run{P, reinterpret_cast<volatile int*>(smem) + 1, ld_acquire_gpu(&P.sync->epoch)};
    bool failed = false;
    uint32_t seq = 0;
    int stamp_i = 0;
    auto stamp = [&]() {
        if (P.timing != nullptr && threadIdx.x == 0 && stamp_i < 64) {
            unsigned long long tm;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm));
            P.timing[(size_t)bx * 64 + stamp_i] = tm;
        }
        stamp_i++;
    };
    stamp();

    for (int o = 0; o < P.n_ops && !failed; o++) {
        const ProgOp& op = P.ops[o];
        const WsShare sh = share_of(o);
        const int flags = sh.flags, kt = sh.kt;
        // what the row stores need, fetched before the tiles are walked
        float* const y = op.y;
        const float* const residual = op.residual;
        const int rows = op.rows;
        const int64_t col0 = op.col0;
        uint2* slots_g = P.scratch + (size_t)(o & 1) * gridDim.x * 128;

        stamp();  // op start (4 stamps per op: start, after barrier, after staging, after compute)
        if (flags & OP_NEW_X) {
            if (flags & OP_DEPENDS) run.grid_barrier(o);
            else run.consumers_sync();  // the staged activations are about to be replaced
            stamp();
            switch (op.x_kind) {
                case XK_F32: stage_x_q8<R::BETA_INT, XK_F32>(op.x, op.k, xd, recs, kt * T::K, GEMV_CONSUMERS); break;
                case XK_RMSNORM_F32: {
                    const float inv = cta_rms_inv(static_cast<const float*>(op.x), op.k, op.eps, reinterpret_cast<float*>(smem + 192), GEMV_CONSUMERS);
                    stage_x_q8<R::BETA_INT, XK_RMSNORM_F32>(op.x, op.k, xd, recs, kt * T::K, GEMV_CONSUMERS, op.x_aux, inv);
                    break;
                }
                case XK_SWIGLU_F32: stage_x_q8<R::BETA_INT, XK_SWIGLU_F32>(op.x, op.k, xd, recs, kt * T::K, GEMV_CONSUMERS, op.x_aux); break;
                default: stage_x_q8<R::BETA_INT, XK_BF16>(op.x, op.k, xd, recs, kt * T::K, GEMV_CONSUMERS); break;
            }
            run.consumers_sync();
            stamp();
        } else {
            stamp();
            stamp();
        }

        // y goes to every rank's buffer: the row-shard gather happens here
        auto emit_row = [&](int n, float v) {
            if (n < rows) {
                const int64_t off = col0 + n;
                if (residual != nullptr) v += __ldcg(residual + off);  // the residual add fused into the store
                y[off] = v;
                if (P.world > 1) emit_to_peers(op.ll, P.world, P.rank, off, v, run.tag());
            }
        };
        ws_consume<QT, DEPTH>(sh, op.chunk_q, op.chunk_r, warp, lane, slots, cur, bar, pieces, seq, smem_u32(xd), smem_u32(recs),
                       smem_u32(recs) + (uint32_t)((kt * T::K) >> 5) * 16, slots_g, P.status, smem_u32(const_cast<int*>(abort_flag)),
                       share_of, P.n_ops, emit_row);
        if (*abort_flag) failed = true;
        stamp();
    }
    if (failed) {
        if (lane == 0) atomicOr(P.status, STATUS_GEMV_FIXUP_TIMEOUT);
        *run.failed = 1;
    }
    run.leave();
}

// ---------------------------------------------------------------- host side
struct Program {
    uint32_t magic = 0x57465047;  // "WFPG"
    Context* ctx = nullptr;
    std::vector<Weight*> held;    // the op list points into these weights: they cannot be freed while the program lives
    int qtype = 0, n_ops = 0, m = 0, world = 1, rank = 0;
    ProgOp* d_ops = nullptr;
    ProgSync* d_sync = nullptr;
    uint2* d_scratch = nullptr;
    int2* d_shares = nullptr;
    unsigned long long* d_timing = nullptr;
    ProgParams params{};
    size_t smem = 0;
    int grid = 0;
};

static std::mutex g_prog_mu;
static std::vector<Program*> g_programs;

static Program* get_program(Context* c, int64_t h) {
    Program* p = reinterpret_cast<Program*>(h);
    std::lock_guard<std::mutex> lk(g_prog_mu);
    if (!p || std::find(g_programs.begin(), g_programs.end(), p) == g_programs.end() || p->magic != 0x57465047 || p->ctx != c)
        return nullptr;
    return p;
}

template <int QT>
static cudaError_t program_launch_one_token(const Program& pr, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv1_program_kernel<QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    // cooperative: the grid barrier needs every CTA resident at once, and a cooperative launch starts only when
    // the device can place them all (another kernel holding SMs delays the start instead of starving the barrier)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pr.grid);
    cfg.blockDim = dim3(GEMV_CONSUMERS);
    cfg.dynamicSmemBytes = pr.smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv1_program_kernel<QT>, pr.params);
}

template <int QT, int XC>
static cudaError_t program_launch(const Program& pr, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_program_kernel<QT, XC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};  // cooperative, as for the one-token kernel
    cfg.gridDim = dim3((unsigned)pr.grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = pr.smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_program_kernel<QT, XC>, pr.params);
}

}  // namespace wf

using namespace wf;

extern "C" {

int wf_program_create(int64_t ctx, int n_ops, const int64_t* weights, const int64_t* x_dev, const int64_t* y_dev, const int* flags,
                      int64_t m, int world, int rank, const int64_t* landing_dev, int64_t* program) {
    return wf_program_create_fused(ctx, n_ops, weights, x_dev, y_dev, flags, nullptr, nullptr, nullptr, nullptr, m, world, rank,
                                   landing_dev, program);
}

int wf_program_create_fused(int64_t ctx, int n_ops, const int64_t* weights, const int64_t* x_dev, const int64_t* y_dev,
                            const int* flags, const int* x_kind, const int64_t* x_aux_dev, const float* eps,
                            const int64_t* residual_dev, int64_t m, int world, int rank, const int64_t* landing_dev,
                            int64_t* program) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    if (!weights || !x_dev || !y_dev || !flags || !program || n_ops < 1) return set_error(c, WF_ERR_INVALID_ARGUMENT, "null pointer or empty program");
    *program = 0;
    if (m < 1 || m > 8) return set_error(c, WF_ERR_SHAPE, "a program takes 1..8 bf16 tokens, got %lld", (long long)m);
    if (world < 1 || world > PROG_MAX_WORLD || rank < 0 || rank >= world) return set_error(c, WF_ERR_SHARD, "rank %d outside world %d (max %d)", rank, world, PROG_MAX_WORLD);
    if (world > 1 && !landing_dev) return set_error(c, WF_ERR_INVALID_ARGUMENT, "landing buffers are required for world > 1");
    WF_CUDA(c, cudaSetDevice(c->device));

    std::vector<ProgOp> ops((size_t)n_ops);
    int qt = 0, kp_max = 0, n_barriers = 0;
    const int grid = c->sm_count;
    for (int o = 0; o < n_ops; o++) {
        Weight* w = get_weight(c, weights[o]);
        if (!w) return set_error(c, WF_ERR_INVALID_HANDLE, "op %d: bad weight handle", o);
        if (o == 0) qt = w->g.qtype;
        if (w->g.qtype != qt) return set_error(c, WF_ERR_UNSUPPORTED_TYPE, "op %d: all weights of a program must share one quantization type", o);
        if (w->total_rows != w->g.rows * world || w->row0 != w->g.rows * rank)
            return set_error(c, WF_ERR_SHARD, "op %d: weight shard does not match rank %d of %d", o, rank, world);
        const int64_t total = w->g.rt * w->g.kt;
        if (total >= (1LL << 31)) return set_error(c, WF_ERR_TOO_LARGE, "op %d: too many tiles", o);
        ProgOp& op = ops[o];
        op.tiles = w->d_tiles;
        op.x = reinterpret_cast<const void*>(x_dev[o]);
        op.y = reinterpret_cast<float*>(y_dev[o]);
        if (!op.y) return set_error(c, WF_ERR_INVALID_ARGUMENT, "op %d: null output pointer", o);
        for (int r = 0; r < world; r++) {
            op.ll[r] = world > 1 ? reinterpret_cast<uint2*>(landing_dev[(size_t)o * world + r]) : nullptr;
            if (world > 1 && !op.ll[r]) return set_error(c, WF_ERR_INVALID_ARGUMENT, "op %d: null landing buffer for rank %d", o, r);
        }
        op.n_total = (int)w->total_rows;
        if (!op.x) return set_error(c, WF_ERR_INVALID_ARGUMENT, "op %d: null activation pointer", o);
        if ((x_dev[o] & 15) || (y_dev[o] & 3))
            return set_error(c, WF_ERR_INVALID_ARGUMENT, "op %d: misaligned pointer (activations 16 bytes, output 4 bytes)", o);
        op.x_kind = x_kind ? x_kind[o] : XK_BF16;
        op.eps = eps ? eps[o] : 0.f;
        op.x_aux = x_aux_dev ? reinterpret_cast<const float*>(x_aux_dev[o]) : nullptr;
        op.residual = residual_dev ? reinterpret_cast<const float*>(residual_dev[o]) : nullptr;
        if (op.x_kind < XK_BF16 || op.x_kind > XK_SWIGLU_F32) return set_error(c, WF_ERR_INVALID_ARGUMENT, "op %d: unknown input kind %d", o, op.x_kind);
        if ((op.x_kind != XK_BF16 || op.residual) && m != 1)
            return set_error(c, WF_ERR_SHAPE, "op %d: fused inputs and residuals are for one-token programs", o);
        if (op.x_kind == XK_SWIGLU_F32 && !op.x_aux) return set_error(c, WF_ERR_INVALID_ARGUMENT, "op %d: swiglu needs the up projection's output", o);
        if ((reinterpret_cast<uintptr_t>(op.x_aux) & 15) || (reinterpret_cast<uintptr_t>(op.residual) & 3))
            return set_error(c, WF_ERR_INVALID_ARGUMENT, "op %d: misaligned pointer (gamma / up 16 bytes, residual 4 bytes)", o);
        if (op.x_kind != XK_BF16 && (w->g.k & 7)) return set_error(c, WF_ERR_SHAPE, "op %d: fp32 inputs need K a multiple of 8", o);
        op.ldy = w->total_rows;
        op.col0 = w->row0;
        op.rows = (int)w->g.rows;
        op.k = (int)w->g.k;
        op.kt = (int)w->g.kt;
        op.rt = (int)w->g.rt;
        // the split the per-projection kernel uses: same sums, same bits
        if (m == 1) {
            const WsSplit sp = ws_split(c->sm_count, w->g.rt, w->g.kt);
            op.ctas = sp.ctas;
            op.aligned = sp.aligned;
            op.chunk_q = sp.chunk_q;
            op.chunk_r = sp.chunk_r;
        } else {
            op.ctas = std::min(grid, gemv_ctas(c->sm_count, total));
            op.aligned = 0;
            op.chunk_q = (int)(total / op.ctas);
            op.chunk_r = (int)(total % op.ctas);
        }
        op.flags = (o == 0 ? (flags[o] | OP_NEW_X) : flags[o]) & (OP_NEW_X | OP_DEPENDS);
        if ((op.flags & OP_DEPENDS) && !(op.flags & OP_NEW_X)) op.flags |= OP_NEW_X;
        if (o == 0) op.flags &= ~OP_DEPENDS;  // nothing of this run precedes the first op
        if (op.flags & OP_DEPENDS) n_barriers++;
        kp_max = std::max(kp_max, op.kt * tile_k(qt));
    }
    // One token: every CTA's share of every op, as tiles.  Consecutive projections that read the same staged
    // activations (no new input between them) and have the same K are cut as ONE list of row-tiles: a CTA then has
    // work in one or two of them instead of a short run in each, and pays the per-projection hand-over once.
    std::vector<int2> shares;
    if (m == 1) {
        shares.assign((size_t)n_ops * grid, make_int2(0, 0));
        for (int i = 0; i < n_ops;) {
            int j = i + 1;
            while (j < n_ops && !(ops[j].flags & OP_NEW_X) && ops[j].kt == ops[i].kt) j++;
            if (j - i > 1) {
                int64_t rt_all = 0;
                for (int k = i; k < j; k++) rt_all += ops[k].rt;
                const int ctas = (int)std::max<int64_t>(1, std::min<int64_t>(grid, rt_all));
                const int64_t q = rt_all / ctas, r = rt_all % ctas;
                for (int cta = 0; cta < ctas; cta++) {
                    const int64_t u0 = cta * q + std::min<int64_t>(cta, r), u1 = u0 + q + (cta < r ? 1 : 0);
                    int64_t base = 0;
                    for (int k = i; k < j; k++) {
                        const int64_t lo = std::max(u0, base) - base, hi = std::min(u1, base + ops[k].rt) - base;
                        if (lo < hi) shares[(size_t)k * grid + cta] = make_int2((int)(lo * ops[k].kt), (int)(hi * ops[k].kt));
                        base += ops[k].rt;
                    }
                }
                for (int k = i; k < j; k++) {  // whole row-tiles: nothing is finished between CTAs
                    ops[k].ctas = ctas;
                    ops[k].aligned = 1;
                    ops[k].chunk_q = ops[k].chunk_r = 0;
                }
            } else {
                for (int cta = 0; cta < grid; cta++) {
                    int t0, t1;
                    ws_cta_share(cta, ops[i].ctas, ops[i].chunk_q, ops[i].chunk_r, ops[i].aligned, ops[i].kt, t0, t1);
                    shares[(size_t)i * grid + cta] = make_int2(t0, t1);
                }
            }
            i = j;
        }
    }
    // shared memory: one token -- the streaming layout (wf_gemv_stream.cuh); several -- ctrl + partial + cinit + x + ring
    const int xc = (m == 1) ? 1 : 8;
    size_t fixed, stage;
    int stages, sx = 0;
    if (xc == 1) {
        const int table_ops = std::min(n_ops, WS_TABLE_OPS);
        if (!ws_fits(kp_max, table_ops)) return set_error(c, WF_ERR_TOO_LARGE, "K=%d does not fit one SM's shared memory", kp_max);
        fixed = ws_smem(kp_max, table_ops);
        stage = 0;
        stages = 0;
    } else {
        const int nslot = Slots<8>::N, elems = 16 * xc;
        sx = kp_max * 2 + 64;
        fixed = GEMV_CTRL_BYTES + (size_t)nslot * GEMV_WARPS * elems * 4 + (size_t)(kp_max / 32) * 64 + (size_t)m * sx;
        fixed = (fixed + 127) & ~(size_t)127;
        stage = (size_t)GEMV_WARPS * tile_bytes(qt);
        if (fixed + 2 * stage > 227 * 1024) return set_error(c, WF_ERR_TOO_LARGE, "K=%d with %lld tokens does not fit one SM's shared memory", kp_max, (long long)m);
        // the ring also carries the next projections' weights across barriers: a little deeper than the single-op kernel's
        stages = (int)std::min<size_t>((227 * 1024 - fixed) / stage, GEMV_USE_STAGES + 2);
    }

    Program* pr = new Program();
    pr->ctx = c;
    for (int o = 0; o < n_ops; o++) pr->held.push_back(get_weight(c, weights[o]));
    pr->qtype = qt;
    pr->n_ops = n_ops;
    pr->m = (int)m;
    pr->world = world;
    pr->rank = rank;
    pr->grid = grid;
    pr->smem = fixed + (size_t)stages * stage;
    cudaError_t e = cudaMalloc(&pr->d_ops, sizeof(ProgOp) * (size_t)n_ops);
    if (e == cudaSuccess) e = cudaMalloc(&pr->d_sync, sizeof(ProgSync));
    if (e == cudaSuccess) e = cudaMalloc(&pr->d_scratch, (size_t)2 * grid * 128 * sizeof(uint2));
    if (e == cudaSuccess && !shares.empty()) e = cudaMalloc(&pr->d_shares, shares.size() * sizeof(int2));
    if (e == cudaSuccess && !shares.empty()) e = cudaMemcpy(pr->d_shares, shares.data(), shares.size() * sizeof(int2), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(pr->d_ops, ops.data(), sizeof(ProgOp) * (size_t)n_ops, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(pr->d_sync, 0, sizeof(ProgSync));
    if (e == cudaSuccess) e = cudaMemset(pr->d_scratch, 0, (size_t)2 * grid * 128 * sizeof(uint2));
    if (e != cudaSuccess) {
        cudaFree(pr->d_ops);
        cudaFree(pr->d_sync);
        cudaFree(pr->d_scratch);
        cudaFree(pr->d_shares);
        delete pr;
        return cuda_status(c, e, "program allocation");
    }
    ProgParams& P = pr->params;
    P.ops = pr->d_ops;
    P.n_ops = n_ops;
    P.m = (int)m;
    P.scratch = pr->d_scratch;
    P.shares = pr->d_shares;
    P.status = c->d_status;
    P.sync = pr->d_sync;
    P.world = world;
    P.rank = rank;
    P.stages = stages;
    P.sx = sx;
    P.kp_max = kp_max;
    P.n_barriers = n_barriers;
    P.timing = nullptr;
    if (c->salt >= 2) {
        if (cudaMalloc(&pr->d_timing, (size_t)grid * 64 * 8) == cudaSuccess) {
            cudaMemset(pr->d_timing, 0, (size_t)grid * 64 * 8);
            P.timing = pr->d_timing;
        }
    }
    for (Weight* w : pr->held) w->programs++;
    {
        std::lock_guard<std::mutex> g(g_prog_mu);
        g_programs.push_back(pr);
    }
    *program = reinterpret_cast<int64_t>(pr);
    return WF_OK;
}

int wf_program_run(int64_t ctx, int64_t program, int64_t stream) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    Program* pr = get_program(c, program);
    if (!pr) return WF_ERR_INVALID_HANDLE;
    WF_CUDA(c, cudaSetDevice(c->device));
    cudaStream_t s = resolve_stream(c, stream);
    const int qt = pr->qtype;
    cudaError_t e;
    if (pr->m == 1)
        e = qt == WF_QTYPE_Q4_0 ? program_launch_one_token<WF_QTYPE_Q4_0>(*pr, s) : qt == WF_QTYPE_Q4_1 ? program_launch_one_token<WF_QTYPE_Q4_1>(*pr, s) : qt == WF_QTYPE_Q8_0 ? program_launch_one_token<WF_QTYPE_Q8_0>(*pr, s) : program_launch_one_token<WF_QTYPE_Q4_K>(*pr, s);
    else
        e = qt == WF_QTYPE_Q4_0 ? program_launch<WF_QTYPE_Q4_0, 8>(*pr, s) : qt == WF_QTYPE_Q4_1 ? program_launch<WF_QTYPE_Q4_1, 8>(*pr, s) : qt == WF_QTYPE_Q8_0 ? program_launch<WF_QTYPE_Q8_0, 8>(*pr, s) : program_launch<WF_QTYPE_Q4_K, 8>(*pr, s);
    if (e != cudaSuccess) return cuda_status(c, e, "program launch");
    c->launches++;
    return WF_OK;
}

int wf_program_step_host(int64_t ctx, int64_t program, int n_in, const void* const* host_src, const int64_t* dev_dst,
                         const int64_t* bytes, void* host_out, int64_t dev_out, int64_t out_bytes, int64_t stream) {
    {
        Context* c = get_context(ctx);
        if (!c) return WF_ERR_INVALID_HANDLE;
        ScopedLock lk(c);
        if (!lk.ok) return WF_ERR_BUSY;
        if (n_in < 0 || (n_in > 0 && (!host_src || !dev_dst || !bytes)) || out_bytes < 0 || (out_bytes > 0 && (!host_out || !dev_out)))
            return set_error(c, WF_ERR_INVALID_ARGUMENT, "null pointer or negative size");
        WF_CUDA(c, cudaSetDevice(c->device));
        cudaStream_t s = resolve_stream(c, stream);
        for (int i = 0; i < n_in; i++) {
            if (!host_src[i] || !dev_dst[i] || bytes[i] < 0) return set_error(c, WF_ERR_INVALID_ARGUMENT, "input %d: null pointer or negative size", i);
            WF_CUDA(c, cudaMemcpyAsync(reinterpret_cast<void*>(dev_dst[i]), host_src[i], (size_t)bytes[i], cudaMemcpyHostToDevice, s));
        }
    }
    const int rc = wf_program_run(ctx, program, stream);
    if (rc != WF_OK) return rc;
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    cudaStream_t s = resolve_stream(c, stream);
    if (out_bytes > 0) WF_CUDA(c, cudaMemcpyAsync(host_out, reinterpret_cast<const void*>(dev_out), (size_t)out_bytes, cudaMemcpyDeviceToHost, s));
    WF_CUDA(c, cudaStreamSynchronize(s));
    return read_device_status(c);
}

int wf_program_read_timing(int64_t ctx, int64_t program, int64_t* out, int64_t n) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    Program* pr = get_program(c, program);
    if (!pr) return WF_ERR_INVALID_HANDLE;
    if (!out || n < 0 || !pr->d_timing) return set_error(c, WF_ERR_INVALID_ARGUMENT, "timing stamps are off (wf_set_salt(ctx, 2) before wf_program_create)");
    WF_CUDA(c, cudaSetDevice(c->device));
    WF_CUDA(c, cudaDeviceSynchronize());
    WF_CUDA(c, cudaMemcpy(out, pr->d_timing, (size_t)std::min<int64_t>(n, (int64_t)pr->grid * 64) * 8, cudaMemcpyDeviceToHost));
    return WF_OK;
}

int wf_program_destroy(int64_t ctx, int64_t program) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    Program* pr = get_program(c, program);
    if (!pr) return WF_ERR_INVALID_HANDLE;
    {
        std::lock_guard<std::mutex> g(g_prog_mu);
        g_programs.erase(std::find(g_programs.begin(), g_programs.end(), pr));
    }
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    cudaFree(pr->d_ops);
    cudaFree(pr->d_sync);
    cudaFree(pr->d_scratch);
    cudaFree(pr->d_shares);
    if (pr->d_timing) cudaFree(pr->d_timing);
    for (Weight* w : pr->held) w->programs--;
    pr->magic = 0;
    delete pr;
    return WF_OK;
}

// ---- peer memory: the handle a rank hands to its peers so they can store into its buffers
int wf_ipc_export(int64_t ctx, int64_t dptr, void* handle64) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    if (!dptr || !handle64) return WF_ERR_INVALID_ARGUMENT;
    WF_CUDA(c, cudaSetDevice(c->device));
    cudaIpcMemHandle_t h;
    WF_CUDA(c, cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(dptr)));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    return WF_OK;
}

int wf_ipc_import(int64_t ctx, const void* handle64, int64_t* dptr) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    if (!dptr || !handle64) return WF_ERR_INVALID_ARGUMENT;
    WF_CUDA(c, cudaSetDevice(c->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    WF_CUDA(c, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *dptr = reinterpret_cast<int64_t>(p);
    return WF_OK;
}

int wf_ipc_close(int64_t ctx, int64_t dptr) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    WF_CUDA(c, cudaSetDevice(c->device));
    WF_CUDA(c, cudaIpcCloseMemHandle(reinterpret_cast<void*>(dptr)));
    return WF_OK;
}

}  // extern "C"
