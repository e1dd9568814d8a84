// Decode GEMV, y[m, rows] = x[m, K] . W[rows, K]^T with W in the tiled quantized layout of wf_layout.cuh: the launch side
// and the one-token kernel.  HBM-bound: every weight byte is read exactly once, from global memory straight into
// the registers of the warp that multiplies it.
//   * one token, bf16 or fp32: gemv1_kernel below (integer MMAs on exact base-256 digits of the activations,
//     wf_gemv_stream.cuh);
//   * 2 .. 32 activation columns (bf16 tokens, or two and more fp32 tokens as three exact bf16 columns each): gemvn_kernel
//     (bf16 MMAs, k-sliced units, wf_gemv_multi.cuh); more tokens than that go through it in passes, or to the
//     tensor-core GEMM (wf_gemm.cu) where the caller routes them there.
//
// Replaces the fp32 batch_matmul_f32 launch of
// warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/ops/DotGeneralKernel.java:263-281
// (PTX at .../nvidia/cuda/CudaKernels.java:4423-4585) for quantized right-hand sides.
#include "wf_gemv_multi.cuh"

namespace wf {

// ---------------------------------------------------------------- one token
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
    constexpr int DEPTH = WsGeom<QT, false>::DEPTH;
    R slots[DEPTH];
    WsCursor cur;
    ws_prime<QT, DEPTH>(slots, cur, share_of, 1, warp, lane);
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        ws_bars_init(smem);
    }
    ws_clear_digits(xd, kp, GEMV_CONSUMERS);
    __syncthreads();
    const WsBars bar = ws_bars(smem);

    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(0);
    if (p.x_f32) stage_x_q8<R::BETA_INT, XK_F32>(p.x, p.k, xd, recs, kp, GEMV_CONSUMERS);
    else stage_x_q8<R::BETA_INT, XK_BF16>(p.x, p.k, xd, recs, kp, GEMV_CONSUMERS);
    __syncthreads();
    stamp(1);
    auto emit_row = [&](int n, float v) {
        if (n < p.rows) p.y[p.col0 + n] = v;
    };
    stamp(2);
    uint32_t seq = 0;
    ws_consume<QT, DEPTH>(share, p.chunk_q, p.chunk_r, warp, lane, slots, cur, bar, pieces, seq, smem_u32(xd), smem_u32(recs),
                   smem_u32(recs) + (uint32_t)(kp >> 5) * 16, p.scratch, p.status, smem_u32(const_cast<int*>(abort_flag)), share_of, 1,
                   emit_row);
    stamp(4);
    if (*abort_flag) {  // a wait ran out somewhere in this CTA
        if (lane == 0) atomicOr(p.status, STATUS_GEMV_FIXUP_TIMEOUT);
    }
    stamp(5);
}

// ---------------------------------------------------------------- host side
constexpr size_t GEMV_SMEM_LIMIT = 227 * 1024;

// The cut of a weight for `cols` activation columns, worked out once per weight (the search walks a few thousand
// candidates: too slow for every call of a microsecond-scale kernel).
static GemvNPlan cached_plan(int sm_count, const Weight& w, int cols, bool x_f32) {
    short* e = const_cast<Weight&>(w).split_cache[x_f32 ? 1 : 0][cols];
    if (e[0] < 0) {
        const GemvNPlan p = gemvn_plan(sm_count, w.g.qtype, w.g.rt, w.g.kt, cols, x_f32);
        e[1] = (short)p.kc;
        e[2] = (short)p.team;
        e[3] = (short)p.uses_part;
        e[0] = (short)p.slices;
    }
    GemvNPlan p;
    p.slices = e[0];
    p.kc = e[1];
    p.team = e[2];
    p.uses_part = e[3] != 0;
    return p;
}

// Activation columns one launch of the several-token kernel can take for this weight: at most 32, fewer when the
// partial sums of a k-sliced launch would not fit their buffer (very tall weights).
static int gemvn_cols_per_pass(int sm_count, const Weight& w, bool x_f32) {
    for (int cols = GEMVN_MAX_COLS; cols >= (x_f32 ? 3 : 1); cols--)
        if (cached_plan(sm_count, w, cols, x_f32).slices > 0) return cols;
    return 0;
}

// Largest number of tokens one launch can take (0: the weight does not fit any kernel).
int gemv_max_tokens_per_pass(const Weight& w, int x_dtype) {
    const bool f32 = x_dtype == WF_DTYPE_F32;
    const int cols = gemvn_cols_per_pass(w.ctx ? w.ctx->sm_count : 148, w, f32);
    const int n = f32 ? cols / 3 : cols;
    if (n == 0 && ws_fits((int)w.g.kt * tile_k(w.g.qtype), 0)) return 1;
    return n;
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

template <int QT, int NG>
static cudaError_t launch_several(const GemvNParams& p, int grid, size_t smem, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemvn_kernel<QT, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMV_SMEM_LIMIT);
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
    return cudaLaunchKernelEx(&cfg, gemvn_kernel<QT, NG>, p);
}
template <int NG>
static cudaError_t launch_qt_several(int qt, const GemvNParams& p, int grid, size_t smem, cudaStream_t s) {
    return qt == WF_QTYPE_Q4_0   ? launch_several<WF_QTYPE_Q4_0, NG>(p, grid, smem, s)
           : qt == WF_QTYPE_Q4_1 ? launch_several<WF_QTYPE_Q4_1, NG>(p, grid, smem, s)
           : qt == WF_QTYPE_Q8_0 ? launch_several<WF_QTYPE_Q8_0, NG>(p, grid, smem, s)
                                 : launch_several<WF_QTYPE_Q4_K, NG>(p, grid, smem, s);
}

// Allocates (once per stream) what the kernels of that stream exchange partial results through: the one-token
// kernel's scratch slots, the several-token kernel's partial sums and arrival counters.  Streams get their own
// so GEMVs on different streams may overlap.
int gemv_prepare_stream(Context* c, cudaStream_t s) {
    GemvScratch& sc = c->gemv_scratch[s];
    if (sc.ctas >= c->sm_count) return WF_OK;
    const int rc = refuse_allocation_while_recording(c, s, "the decode kernels' scratch");
    if (rc != WF_OK) return rc;
    if (sc.d_slots) cudaFree(sc.d_slots);
    if (sc.d_part) cudaFree(sc.d_part);
    if (sc.d_count) cudaFree(sc.d_count);
    sc.d_slots = nullptr;
    sc.d_part = nullptr;
    sc.d_count = nullptr;
    sc.ctas = 0;
    WF_CUDA(c, cudaMalloc(&sc.d_slots, (size_t)c->sm_count * 128 * sizeof(uint2)));
    WF_CUDA(c, cudaMemset(sc.d_slots, 0, (size_t)c->sm_count * 128 * sizeof(uint2)));
    WF_CUDA(c, cudaMalloc(&sc.d_part, GEMVN_PART_BYTES));
    WF_CUDA(c, cudaMalloc(&sc.d_count, (size_t)GEMVN_MAX_ROW_TILES * sizeof(int)));
    WF_CUDA(c, cudaMemset(sc.d_count, 0, (size_t)GEMVN_MAX_ROW_TILES * sizeof(int)));
    sc.ctas = c->sm_count;
    return WF_OK;
}

struct GemvBuffers {
    uint2* slots;  // one-token kernel: [ctas][128] exchange slots
    float* part;   // several tokens: GEMVN_PART_BYTES of partial sums
    int* count;    // several tokens: [GEMVN_MAX_ROW_TILES] arrival counters
};

// One launch per pass of tokens.  clear: zero the exchange slots / arrival counters on the stream before every
// launch (for buffers that may hold leftovers of a failed call).
static int launch_passes(Context* c, const GemvCall& call, cudaStream_t s, const GemvBuffers& buf, bool clear,
                         unsigned long long* timing, const char* what) {
    const Weight& w = *call.w;
    const int qt = w.g.qtype;
    const int kp = (int)w.g.kt * tile_k(qt);
    const bool f32 = call.x_dtype == WF_DTYPE_F32;
    const size_t esz = f32 ? 4 : 2;
    if (call.m == 1 && ws_fits(kp, 0)) {  // one token (bf16 or fp32): the integer path, every warp streaming its own run
        const WsSplit one = ws_split(c->sm_count, w.g.rt, w.g.kt);
        GemvParams p{};
        p.tiles = w.d_tiles;
        p.x = call.d_x;
        p.y = call.d_y;
        p.scratch = buf.slots;
        p.status = c->d_status;
        p.timing = timing;
        p.ldy = call.ldy;
        p.col0 = call.col0;
        p.ldx = w.g.k;
        p.rows = (int)w.g.rows;
        p.k = (int)w.g.k;
        p.kt = (int)w.g.kt;
        p.rt = (int)w.g.rt;
        p.m = 1;
        p.x_f32 = f32;
        p.chunk_q = one.chunk_q;
        p.chunk_r = one.chunk_r;
        p.aligned = one.aligned;
        if (clear) WF_CUDA(c, cudaMemsetAsync(buf.slots, 0, (size_t)one.ctas * 128 * sizeof(uint2), s));
        cudaError_t e = launch_qt_one_token(qt, p, one.ctas, ws_smem(kp, 0), s);
        if (e != cudaSuccess) return cuda_status(c, e, what);
        c->launches++;
        return WF_OK;
    }
    const int per_tok = f32 ? 3 : 1;
    const int per_pass = gemvn_cols_per_pass(c->sm_count, w, f32) / per_tok;
    if (per_pass < 1) return set_error(c, WF_ERR_TOO_LARGE, "weight [%lld x %lld] is beyond the decode kernels", (long long)w.g.rows, (long long)w.g.k);
    if (w.g.rt > GEMVN_MAX_ROW_TILES) return set_error(c, WF_ERR_TOO_LARGE, "%lld rows: more than %d row-tiles", (long long)w.g.rows, GEMVN_MAX_ROW_TILES);
    for (int64_t m0 = 0; m0 < call.m; m0 += per_pass) {
        GemvNParams p{};
        p.tiles = w.d_tiles;
        p.x = static_cast<const uint8_t*>(call.d_x) + (size_t)m0 * w.g.k * esz;
        p.y = call.d_y + m0 * call.ldy;
        p.part = buf.part;
        p.count = buf.count;
        p.status = c->d_status;
        p.timing = timing;
        p.ldy = call.ldy;
        p.col0 = call.col0;
        p.ldx = w.g.k;
        p.rows = (int)w.g.rows;
        p.k = (int)w.g.k;
        p.kt = (int)w.g.kt;
        p.rt = (int)w.g.rt;
        p.m = (int)std::min<int64_t>(call.m - m0, per_pass);
        p.x_f32 = f32;
        p.cols = p.m * per_tok;
        const GemvNPlan plan = cached_plan(c->sm_count, w, p.cols, f32);
        if (plan.slices < 1) return set_error(c, WF_ERR_TOO_LARGE, "no split of K=%lld fits %d activation columns", (long long)w.g.k, p.cols);
        p.slices = plan.slices;
        p.kc = plan.kc;
        p.team = plan.team;
        const int ng = p.cols <= 8 ? 1 : p.cols <= 16 ? 2 : 4;
        const size_t smem = gemvn_smem(qt, p.kc, p.cols, ng, p.team, &p.sx, &p.piece_off);
        if (clear && plan.uses_part) WF_CUDA(c, cudaMemsetAsync(buf.count, 0, (size_t)w.g.rt * sizeof(int), s));
        const cudaError_t e = ng == 1   ? launch_qt_several<1>(qt, p, c->sm_count, smem, s)
                              : ng == 2 ? launch_qt_several<2>(qt, p, c->sm_count, smem, s)
                                        : launch_qt_several<4>(qt, p, c->sm_count, smem, s);
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
    const GemvScratch& sc = c->gemv_scratch[s];
    return launch_passes(c, call, s, GemvBuffers{sc.d_slots, sc.d_part, sc.d_count}, false, c->salt >= 2 ? c->d_timing : nullptr, "gemv launch");
}

// ---------------------------------------------------------------- allocation-free variant
// What the kernels exchange partial results through lives, for wf_qlinear_noalloc, in these statically sized
// device arrays instead of memory obtained from cudaMalloc: the one-token kernel's slots (256 KiB), the
// several-token kernel's partial sums (8 MiB) and arrival counters (256 KiB).  Every GPU that loads the library
// carries them until the process exits.  One set per device is shared by all calls on that device.
constexpr int GEMV_NOALLOC_MAX_CTAS = 256;  // the kernel launches one CTA per SM
static __device__ __align__(256) uint2 g_noalloc_slots[GEMV_NOALLOC_MAX_CTAS * 128];
static __device__ __align__(256) float g_noalloc_part[GEMVN_PART_BYTES / sizeof(float)];
static __device__ __align__(256) int g_noalloc_count[GEMVN_MAX_ROW_TILES];

// In host code `g_noalloc_slots` is only a handle for the symbol, not an address the GPU can
// use; the device address is looked up once per device, with that device current.
static std::mutex g_noalloc_mu;
static GemvBuffers g_noalloc_ptr[64] = {};

static int noalloc_buffers_for_current_device(Context* c, GemvBuffers* out) {
    if (c->device < 0 || c->device >= 64) return set_error(c, WF_ERR_TOO_LARGE, "device index %d beyond 63", c->device);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[c->device].slots) {
        GemvBuffers b{};
        cudaError_t e = cudaGetSymbolAddress((void**)&b.slots, g_noalloc_slots);
        if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&b.part, g_noalloc_part);
        if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&b.count, g_noalloc_count);
        if (e != cudaSuccess) return cuda_status(c, e, "cudaGetSymbolAddress(static GEMV work arrays)");
        g_noalloc_ptr[c->device] = b;
    }
    *out = g_noalloc_ptr[c->device];
    return WF_OK;
}

// Same kernels and the same work split as gemv_launch, but nothing is allocated: slots, partial sums and
// counters come from the static arrays above; slots and counters are cleared on the stream before every launch,
// because the arrays keep whatever the previous call (possibly a failed one) left in them.
int gemv_launch_noalloc(Context* c, const GemvCall& call, cudaStream_t s) {
    int rc = check_shape(c, *call.w, call.x_dtype);
    if (rc != WF_OK) return rc;
    if (c->sm_count > GEMV_NOALLOC_MAX_CTAS)
        return set_error(c, WF_ERR_TOO_LARGE, "device has %d SMs; the static fix-up array covers at most %d", c->sm_count,
                         GEMV_NOALLOC_MAX_CTAS);
    if (call.w->g.rt * call.w->g.kt < 1) return WF_OK;
    GemvBuffers buf{};
    rc = noalloc_buffers_for_current_device(c, &buf);
    if (rc != WF_OK) return rc;
    return launch_passes(c, call, s, buf, true, nullptr, "gemv launch (no-alloc)");
}

}  // namespace wf

extern "C" int wf_plan_several_tokens(int qtype, int64_t rows, int64_t k, int cols, int x_is_f32, int sm_count, int* slices,
                                      int* k_tiles_per_slice, int* team, int* uses_partial_sums, int64_t* smem_bytes) {
    using namespace wf;
    const int qt = device_qtype(qtype);
    if (qt != WF_QTYPE_Q4_0 && qt != WF_QTYPE_Q4_1 && qt != WF_QTYPE_Q8_0 && qt != WF_QTYPE_Q4_K) return WF_ERR_UNSUPPORTED_TYPE;
    if (rows < 1 || k < 1 || cols < 1 || cols > GEMVN_MAX_COLS || sm_count < 1 || !slices || !k_tiles_per_slice || !team) return WF_ERR_INVALID_ARGUMENT;
    const int64_t rt = (rows + 15) / 16, kt = (k + tile_k(qt) - 1) / tile_k(qt);
    const GemvNPlan p = gemvn_plan(sm_count, qt, rt, kt, cols, x_is_f32 != 0);
    *slices = p.slices;
    *k_tiles_per_slice = p.kc;
    *team = p.team;
    if (uses_partial_sums) *uses_partial_sums = p.uses_part ? 1 : 0;
    const int ng = cols <= 8 ? 1 : cols <= 16 ? 2 : 4;
    if (smem_bytes) *smem_bytes = p.slices > 0 ? (int64_t)gemvn_smem(qt, p.kc, cols, ng, p.team, nullptr, nullptr) : 0;
    return WF_OK;
}
