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
// parks its partial sums in shared memory and arrives on an mbarrier -- it never waits for
// the other warps -- and one warp per segment, taken in turn and one segment late, adds the
// sixteen partials in warp order (deterministic).  A row-tile cut by a chunk boundary is
// finished by the CTA that holds its beginning: the following CTAs compute their piece
// first and publish it to a scratch slot tagged valid; the owner, which reaches that
// row-tile last, adds the pieces in CTA order, clears the tags and writes y.  The owner's
// wait is bounded; on expiry it sets a status bit instead of spinning on.
//
// Replaces the fp32 batch_matmul_f32 launch of
// warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/ops/DotGeneralKernel.java:263-281
// (PTX at .../nvidia/cuda/CudaKernels.java:4423-4585) for quantized right-hand sides.
#include "wf_gemv_stream.cuh"

namespace wf {

// ---------------------------------------------------------------- the kernel
// Shared-memory map (bytes): [0,4) abort flag | [128, 128 + GEMV_CTRL_BYTES) barriers |
// partial sums [N][GEMV_WARPS][ELEMS] | cinit | staged x | ring stages (128-byte aligned).
template <int QT, int XC>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvParams p) {
    using T = Tile<QT>;
    using R = TileRegs<QT>;
    constexpr int NSLOT = Slots<XC>::N, ELEMS = Slots<XC>::ELEMS;
    extern __shared__ __align__(128) uint8_t smem[];
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
    const BarrierSet bar = barrier_set(smem);
    float* partial = reinterpret_cast<float*>(smem + GEMV_CTRL_BYTES);       // [NSLOT][GEMV_WARPS][ELEMS]
    const int kp = p.kt * T::K;
    float4* cinit = reinterpret_cast<float4*>(partial + NSLOT * GEMV_WARPS * ELEMS);  // [kp/32][4]
    uint8_t* xs = reinterpret_cast<uint8_t*>(cinit + (kp >> 5) * 4);         // [xcols][sx]
    const int xcols = p.x_f32 ? 3 * p.m : p.m;
    uint8_t* ring = smem + (((size_t)(xs - smem) + (size_t)xcols * p.sx + 127) & ~(size_t)127);

    // warp-uniform values, obtained in a way the compiler can see is uniform
    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    const int bx = blockIdx.x;
    const int t0 = bx * p.chunk_q + min(bx, p.chunk_r);
    const int t1 = t0 + p.chunk_q + (bx < p.chunk_r ? 1 : 0);
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
    // Launched with programmatic stream serialization: the next kernel of the stream may take an SM
    // as soon as this CTA has left it, and streams its weights (which no kernel writes) while
    // the rest of this grid is still running.  Everything that touches memory a previous
    // kernel may have written -- activations, y, scratch slots, status -- comes after
    // griddepcontrol.wait, which returns once the whole previous grid has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        barrier_set_init<XC>(bar, stages);
    }
    __syncthreads();

    if (warp == GEMV_WARPS) {  // producer warp: the weights do not depend on anything, start at once
        if (lane == 0) {
            WalkState pos;
            produce_share<QT>(p.tiles, t0, t1, smem_u32(ring), bar, stages, pos, abort_flag);
        }
        return;
    }

    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(0);
    // cinit entries of dead columns stay uninitialised: they only feed dead columns
    stage_x(p, xs, reinterpret_cast<float*>(cinit), kp, R::BETA, GEMV_CONSUMERS);
    asm volatile("bar.sync 1, %0;" ::"n"(GEMV_CONSUMERS) : "memory");
    stamp(1);

    // dead columns read the last live row: their results are computed and never stored
    const uint8_t* xrow = xs + (size_t)(g < xcols ? g : xcols - 1) * p.sx;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    // y of one finished row-tile, from a shared-memory buffer (element i = column * 16 + row)
    auto emit = [&](int rt, const float* buf) {
        if (!p.x_f32) {
            for (int i = lane; i < ELEMS; i += 32) {
                const int col = i >> 4, n = rt * 16 + (i & 15);
                if (col < p.m && n < p.rows) p.y[(int64_t)col * p.ldy + p.col0 + n] = buf[i];
            }
        } else {  // columns 3t, 3t+1, 3t+2 are the hi / mid / lo parts of token t
            for (int i = lane; i < 16 * p.m; i += 32) {
                const int tok = i >> 4, r = i & 15, n = rt * 16 + r;
                if (n < p.rows)
                    p.y[(int64_t)tok * p.ldy + p.col0 + n] =
                        (buf[(3 * tok + 2) * 16 + r] + buf[(3 * tok + 1) * 16 + r]) + buf[(3 * tok) * 16 + r];
            }
        }
    };

    const uint32_t x32 = smem_u32(xrow) + q * 16, c32 = smem_u32(cinit) + q * 16;
    stamp(2);
    WalkState st;
    consume_share<QT, XC>(t0, t1, p.kt, p.chunk_q, p.chunk_r, warp, lane, smem_u32(ring), bar, partial, stages, st, x32, c32,
                          p.scratch, p.status, smem_u32(const_cast<int*>(abort_flag)), acc, emit);
    stamp(4);
    if (*abort_flag) {  // a wait ran out somewhere in this CTA
        if (lane == 0) atomicOr(p.status, STATUS_GEMV_FIXUP_TIMEOUT);
        drain_after_abort();
    }
    stamp(5);
}

// ---------------------------------------------------------------- one bf16 token
// Integer MMAs on exact base-256 digits of the activations, every warp streaming its own run of tiles from
// global memory into registers (wf_gemv_stream.cuh).  512 threads, all of them consumers.
template <int QT>
__global__ void __launch_bounds__(GEMV_CONSUMERS, 1) gemv1_kernel(const GemvParams p) {
    using T = Tile<QT>;
    using R = TileRegs<QT>;
    extern __shared__ __align__(128) uint8_t smem[];
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
    WsPiece* pieces = reinterpret_cast<WsPiece*>(smem + WS_CTRL_BYTES);
    uint8_t* recs = smem + WS_CTRL_BYTES + WS_PIECE_BYTES;
    const int kp = p.kt * T::K;
    uint8_t* xd = recs + (size_t)(kp >> 5) * 32;

    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int bx = blockIdx.x;
    int t0, t1;
    ws_cta_share(bx, (int)gridDim.x, p.chunk_q, p.chunk_r, p.aligned, p.kt, t0, t1);
    auto stamp = [&](int i) {
        if (p.timing != nullptr && threadIdx.x == 0) {
            unsigned long long tm;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm));
            p.timing[(size_t)blockIdx.x * 8 + i] = tm;
        }
    };
    // Programmatic stream serialization: see gemv_kernel.  The weights depend on nothing, so every warp
    // requests the first tiles of its run before waiting for the previous grid.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const WsShare share{p.tiles, t0, t1, p.kt, 0, {0, 0}};
    auto share_of = [&](int) { return share; };
    R slots[WsGeom<QT>::DEPTH];
    WsCursor cur;
    ws_prime<QT>(slots, cur, share_of, 1, warp, lane);
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        ws_bars_init(smem);
    }
    ws_clear_digits(xd, kp, GEMV_CONSUMERS);
    __syncthreads();
    const WsBars bar = ws_bars(smem);

    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(0);
    stage_x_q8<R::BETA_INT>(p.x, p.k, xd, recs, kp, GEMV_CONSUMERS);
    __syncthreads();
    stamp(1);
    auto emit_row = [&](int n, float v) {
        if (n < p.rows) p.y[p.col0 + n] = v;
    };
    stamp(2);
    uint32_t seq = 0;
    ws_consume<QT>(share, p.chunk_q, p.chunk_r, warp, lane, slots, cur, bar, pieces, seq, smem_u32(xd), smem_u32(recs),
                   smem_u32(recs) + (uint32_t)(kp >> 5) * 16, p.scratch, p.status, smem_u32(const_cast<int*>(abort_flag)), share_of, 1,
                   emit_row);
    stamp(4);
    if (*abort_flag) {  // a wait ran out somewhere in this CTA
        if (lane == 0) atomicOr(p.status, STATUS_GEMV_FIXUP_TIMEOUT);
    }
    stamp(5);
}

// ---------------------------------------------------------------- host side
template <int XC>
static size_t gemv_fixed_smem(int kp, int xcols, int* sx_out) {
    const int sx = kp * 2 + 64;  // +64: consecutive rows start 16 banks apart
    if (sx_out) *sx_out = sx;
    size_t b = GEMV_CTRL_BYTES + (size_t)Slots<XC>::N * GEMV_WARPS * Slots<XC>::ELEMS * 4 + (size_t)(kp / 32) * 64 + (size_t)xcols * sx;
    return (b + 127) & ~(size_t)127;
}

constexpr size_t GEMV_SMEM_LIMIT = 227 * 1024;

// Ring depth that fits beside the staged activations (0 = does not fit at all).
template <int XC>
static int gemv_stages(int qt, int kp, int xcols) {
    const size_t fixed = gemv_fixed_smem<XC>(kp, xcols, nullptr), stage = (size_t)GEMV_WARPS * tile_bytes(qt);
    if (fixed + stage > GEMV_SMEM_LIMIT) return 0;
    return (int)std::min<size_t>((GEMV_SMEM_LIMIT - fixed) / stage, GEMV_USE_STAGES);
}

// Largest number of tokens one pass can take: bounded by the 8 mma columns (3 per fp32
// token) and by the shared memory the staged activations and a 2-deep ring need.
int gemv_max_tokens_per_pass(const Weight& w, int x_dtype) {
    const int kp = (int)w.g.kt * tile_k(w.g.qtype);
    const int per_tok = x_dtype == WF_DTYPE_F32 ? 3 : 1;
    int best = 0;
    for (int m = 1; m * per_tok <= GEMV_XCOLS; m++)
        if (gemv_stages<8>(w.g.qtype, kp, m * per_tok) >= 2) best = m;
    if (best == 0 && per_tok == 1 && ws_fits(kp, 0)) best = 1;  // only the one-token kernel fits
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_kernel<QT, XC>, p);
}

template <int QT>
static cudaError_t launch_one_token(const GemvParams& p, int grid, size_t smem, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv1_kernel<QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMV_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GEMV_CONSUMERS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv1_kernel<QT>, p);
}

static cudaError_t launch_qt_one_token(int qt, const GemvParams& p, int grid, size_t smem, cudaStream_t s) {
    return qt == WF_QTYPE_Q4_0   ? launch_one_token<WF_QTYPE_Q4_0>(p, grid, smem, s)
           : qt == WF_QTYPE_Q4_1 ? launch_one_token<WF_QTYPE_Q4_1>(p, grid, smem, s)
           : qt == WF_QTYPE_Q8_0 ? launch_one_token<WF_QTYPE_Q8_0>(p, grid, smem, s)
                                 : launch_one_token<WF_QTYPE_Q4_K>(p, grid, smem, s);
}

template <int XC>
static cudaError_t launch_qt(int qt, const GemvParams& p, int grid, size_t smem, cudaStream_t s) {
    return qt == WF_QTYPE_Q4_0   ? launch_one<WF_QTYPE_Q4_0, XC>(p, grid, smem, s)
           : qt == WF_QTYPE_Q4_1 ? launch_one<WF_QTYPE_Q4_1, XC>(p, grid, smem, s)
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

// One launch per pass of up to `per_pass` tokens.  `slots` are the fix-up slots to use;
// clear_slots: zero them on the stream before every launch (for slots that may hold leftovers).
static int launch_passes(Context* c, const GemvCall& call, cudaStream_t s, uint2* slots, bool clear_slots,
                         unsigned long long* timing, const char* what) {
    const Weight& w = *call.w;
    const int qt = w.g.qtype;
    const int kp = (int)w.g.kt * tile_k(qt);
    const int per_pass = gemv_max_tokens_per_pass(w, call.x_dtype);
    const int64_t total = w.g.rt * w.g.kt;
    const int grid_several = gemv_ctas(c->sm_count, total);
    const WsSplit one = ws_split(c->sm_count, w.g.rt, w.g.kt);  // the one-token kernel's cut
    const size_t esz = call.x_dtype == WF_DTYPE_F32 ? 4 : 2;
    int max_rounds = (int)((total / grid_several + 1 + GEMV_WARPS - 1) / GEMV_WARPS);
    for (int64_t m0 = 0; m0 < call.m; m0 += per_pass) {
        GemvParams p{};
        p.tiles = w.d_tiles;
        p.x = static_cast<const uint8_t*>(call.d_x) + (size_t)m0 * w.g.k * esz;
        p.y = call.d_y + m0 * call.ldy;
        p.scratch = slots;
        p.status = c->d_status;
        p.timing = timing;
        p.ldy = call.ldy;
        p.col0 = call.col0;
        p.ldx = w.g.k;
        p.rows = (int)w.g.rows;
        p.k = (int)w.g.k;
        p.kt = (int)w.g.kt;
        p.rt = (int)w.g.rt;
        p.m = (int)((call.m - m0) < per_pass ? (call.m - m0) : per_pass);
        p.x_f32 = call.x_dtype == WF_DTYPE_F32;
        const int xcols = p.x_f32 ? 3 * p.m : p.m;
        const bool one_token = xcols == 1 && ws_fits(kp, 0);
        const int grid = one_token ? one.ctas : grid_several;
        p.chunk_q = one_token ? one.chunk_q : (int)(total / grid);
        p.chunk_r = one_token ? one.chunk_r : (int)(total % grid);
        p.aligned = one_token ? one.aligned : 0;
        const size_t stage = (size_t)GEMV_WARPS * tile_bytes(qt);
        if (clear_slots) WF_CUDA(c, cudaMemsetAsync(slots, 0, (size_t)grid * 128 * sizeof(uint2), s));
        cudaError_t e;
        if (one_token) {  // one bf16 token: the integer path, every warp streaming its own run
            e = launch_qt_one_token(qt, p, grid, ws_smem(kp, 0), s);
        } else {
            p.stages = std::min(gemv_stages<8>(qt, kp, xcols), std::max(max_rounds, 1));
            e = launch_qt<8>(qt, p, grid, gemv_fixed_smem<8>(kp, xcols, &p.sx) + p.stages * stage, s);
        }
        if (e != cudaSuccess) return cuda_status(c, e, what);
        c->launches++;
    }
    return WF_OK;
}

static int check_shape(Context* c, const Weight& w, int x_dtype) {
    if (gemv_max_tokens_per_pass(w, x_dtype) < 1)
        return set_error(c, WF_ERR_TOO_LARGE, "K=%lld needs more shared memory than one SM has", (long long)w.g.k);
    if (w.g.rt * w.g.kt >= (1LL << 31)) return set_error(c, WF_ERR_TOO_LARGE, "weight has too many tiles");
    return WF_OK;
}

int gemv_launch(Context* c, const GemvCall& call, cudaStream_t s) {
    int rc = check_shape(c, *call.w, call.x_dtype);
    if (rc != WF_OK) return rc;
    if (call.w->g.rt * call.w->g.kt < 1) return WF_OK;
    rc = gemv_prepare_stream(c, s);
    if (rc != WF_OK) return rc;
    return launch_passes(c, call, s, c->gemv_scratch[s].d_slots, false, c->salt >= 2 ? c->d_timing : nullptr, "gemv launch");
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
    int rc = check_shape(c, *call.w, call.x_dtype);
    if (rc != WF_OK) return rc;
    if (c->sm_count > GEMV_NOALLOC_MAX_CTAS)
        return set_error(c, WF_ERR_TOO_LARGE, "device has %d SMs; the static fix-up array covers at most %d", c->sm_count,
                         GEMV_NOALLOC_MAX_CTAS);
    if (call.w->g.rt * call.w->g.kt < 1) return WF_OK;
    uint2* slots = nullptr;
    rc = noalloc_slots_for_current_device(c, &slots);
    if (rc != WF_OK) return rc;
    return launch_passes(c, call, s, slots, true, nullptr, "gemv launch (no-alloc)");
}

}  // namespace wf
