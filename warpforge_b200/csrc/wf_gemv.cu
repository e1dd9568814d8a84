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
#include "wf_gemv_core.cuh"

namespace wf {

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
    stage_x(p, xs, reinterpret_cast<float*>(cinit), kp, R::BETA, GEMV_THREADS, XC == 1);
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
    const uint32_t my_tile = smem_u32(ring) + warp * T::BYTES + lane * 16;
    const uint32_t x32 = smem_u32(xrow) + q * 16, c32 = smem_u32(cinit) + (XC == 1 ? 0 : q * 16);
    const uint32_t live = (XC == 1) ? (uint32_t)(g == 0) : 1u;
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
            regs.load(my_tile + s * STAGE_BYTES, lane);
            __syncwarp();
            mbar_arrive_if(&empty[s], lane_is_0);
            regs.template compute<XC>(acc, x32 + kbase * 2, c32 + (kbase >> 5) * cinit_block_bytes<XC>(), live);
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
