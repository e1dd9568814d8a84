// The fp32 operations that sit between the quantized projections of a decode step: rms_norm,
// layer_norm, softmax, silu, silu(gate)*up, residual add and the embedding lookup.  They replace the
// custom_call kernels of the reference's NVIDIA backend
// (warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/ops/CudaCustomCallKernel.java:50-59,
// scalar one-thread-per-element PTX) and follow the arithmetic of its CPU backend
// (warpforge-backend-cpu/src/main/java/io/surfworks/warpforge/backend/cpu/ops/scalar/CustomCallKernel.java:
// layer_norm :109-171, softmax :173-224, silu :262-280, embedding :282-318, rms_norm :368-412):
// every product, sum and quotient of the per-element formulas is rounded separately as there
// (no fused multiply-add), exp is evaluated in double and rounded to float as `(float) Math.exp(x)`
// is, square roots likewise.  Only the row reductions differ: the CPU adds a row's terms one after
// another in fp32, here each thread adds its terms in fp32 and the partial sums are combined in
// double, so results agree to rounding of the reduction (about 1e-7 relative), not bit for bit.
//
// All of them are HBM-bound: one read and one write of the tensor.  Row operations keep the row in
// registers between the reduction and the normalisation (one CTA per row, up to 8192 columns; longer
// rows are read again from L2), element operations move 16 bytes per thread per step.
#include "wf_common.cuh"

namespace wf {

constexpr int ROW_THREADS = 256;
constexpr int ROW_VEC = 8;  // float4 per thread held in registers: rows up to 256 * 8 * 4 = 8192 columns

// `red` is private to one reduction (each call site passes its own array), so one barrier is enough
__device__ __forceinline__ double block_sum(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < ROW_THREADS / 32; w++) t += red[w];
    return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int w = 1; w < ROW_THREADS / 32; w++) t = fmaxf(t, red[w]);
    return t;
}

// (float) Math.exp(x): the exponential in double, one rounding to float.  Only the float result matters, so
// the double needs about 2^-44, not the library's last bit, and the fp64 pipe (a fraction of the fp32 rate
// on this GPU; the library exp made silu and softmax compute-bound at 45 % and 29 % of HBM speed) gets as few
// operations as possible: x = (32 k + j) ln2/32 + r with |r| <= ln2/64, exp(x) = 2^k * 2^(j/32) * exp(r);
// 2^(j/32) comes from a 32-entry table in shared memory, exp(r) - 1 = r + r^2/2 in double plus the terms
// from r^3 on, below 2^-22, in fp32; float -> double, the rounding of x * 32/ln2 to an integer, integer ->
// double and the scaling by 2^k are done on the bit patterns (conversion instructions are slower still).
// Seven fp64 operations per call.  Against (float) exp((double) x) of the host libm: 11 differences of one
// ulp in 4e8 arguments.  Outside [-104, 89] the float result is 0 or infinity whatever the double is.
__constant__ double EXP2_32[32] = {
    1.00000000000000000e+00, 1.02189714865411663e+00, 1.04427378242741375e+00, 1.06714040067682370e+00,
    1.09050773266525769e+00, 1.11438674259589243e+00, 1.13878863475669156e+00, 1.16372485877757748e+00,
    1.18920711500272103e+00, 1.21524735998046896e+00, 1.24185781207348400e+00, 1.26905095719173322e+00,
    1.29683955465100964e+00, 1.32523664315974132e+00, 1.35425554693689265e+00, 1.38390988196383202e+00,
    1.41421356237309515e+00, 1.44518080697704665e+00, 1.47682614593949935e+00, 1.50916442759342284e+00,
    1.54221082540794074e+00, 1.57598084510788650e+00, 1.61049033194925428e+00, 1.64575547815396495e+00,
    1.68179283050742900e+00, 1.71861929812247793e+00, 1.75625216037329945e+00, 1.79470907500310717e+00,
    1.83400808640934243e+00, 1.87416763411029996e+00, 1.91520656139714740e+00, 1.95714412417540018e+00};

// every thread of the CTA calls this once before the first exp_as_host
__device__ __forceinline__ void load_exp_table(double* tab) {
    if (threadIdx.x < 32) tab[threadIdx.x] = EXP2_32[threadIdx.x];
    __syncthreads();
}

__device__ __forceinline__ double widen_normal(float f) {  // (double) f for a normal (not zero, not subnormal) float
    const uint32_t b = __float_as_uint(f), em = b & 0x7FFFFFFFu;
    return __hiloint2double((int)((b & 0x80000000u) | ((em >> 3) + (896u << 20))), (int)(em << 29));
}

// EXACT: the host's (float) exp((double) x); otherwise the fp32 library exponential (2 ulp), about a third
// of the instructions: the exact form leaves silu and softmax issue-bound at about 45 % of HBM speed.
template <bool EXACT> __device__ __forceinline__ float exp_sel(float x, const double* tab);

__device__ __forceinline__ float exp_as_host(float x, const double* tab) {
    if (x != x) return x;
    if (x > 89.0f) return INFINITY;
    if (x < -104.0f) return 0.0f;
    if (fabsf(x) < 1e-8f) return 1.0f;
    const float t = __fmaf_rn(x, 46.1662413f, 12582912.f);  // 1.5 * 2^23: the integer lands in the low mantissa bits
    const int n = (int)(__float_as_uint(t) - 0x4B400000u);
    const float nf = __fsub_rn(t, 12582912.f);
    const double nd = __hiloint2double(0x43300000, n ^ 0x80000000) - 4503601774854144.0;  // 2^52 + 2^31
    double r = fma(-nd, 2.16608493924468348268e-02, widen_normal(x));  // ln2/32, 36 bits: the product is exact
    r = fma(-nd, 5.14560924465533821524e-14, r);
    float rf = __fmaf_rn(-nf, 2.1652221680e-02f, x);  // the same reduction in fp32 (11 + 24 bits) for the small terms
    rf = __fmaf_rn(-nf, 8.6277132141e-06f, rf);
    const float tail = rf * rf * rf * __fmaf_rn(rf, __fmaf_rn(rf, 8.33333333e-3f, 4.16666667e-2f), 1.66666667e-1f);
    double s = fma(0.5 * r, r, r);
    s += fabsf(tail) < 1e-30f ? 0.0 : widen_normal(tail);
    const double tj = tab[n & 31];
    const double v = fma(tj, s, tj);  // in [1, 2.05): adding k to the exponent field scales it exactly
    return (float)__hiloint2double(__double2hiint(v) + ((n >> 5) << 20), __double2loint(v));
}

template <> __device__ __forceinline__ float exp_sel<true>(float x, const double* tab) { return exp_as_host(x, tab); }
template <> __device__ __forceinline__ float exp_sel<false>(float x, const double*) { return expf(x); }

// A row held by one CTA: float4 pieces in registers when the row is 16-byte addressable and short
// enough, otherwise element loops over global memory.  `f(i, x)` visits every element.
struct RowView {
    const float* x;
    int n;
    bool vec;
    float4 r[ROW_VEC];
    __device__ RowView(const float* row, int n_) : x(row), n(n_) {
        vec = (n % 4 == 0) && n <= ROW_THREADS * ROW_VEC * 4 && (reinterpret_cast<uintptr_t>(row) % 16 == 0);
        if (vec) {
#pragma unroll
            for (int j = 0; j < ROW_VEC; j++) {
                const int i = (j * ROW_THREADS + threadIdx.x) * 4;
                r[j] = i < n ? __ldcs(reinterpret_cast<const float4*>(x + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    // x[i] <- h(x[i]) where the row is held in registers (the caller falls back to recomputing otherwise)
    template <class H> __device__ __forceinline__ void map_registers(H h) {
#pragma unroll
        for (int j = 0; j < ROW_VEC; j++)
            if ((j * ROW_THREADS + (int)threadIdx.x) * 4 < n) r[j] = make_float4(h(r[j].x), h(r[j].y), h(r[j].z), h(r[j].w));
    }
    template <class F> __device__ __forceinline__ void for_each(F f) const {
        if (vec) {
#pragma unroll
            for (int j = 0; j < ROW_VEC; j++) {
                const int i = (j * ROW_THREADS + threadIdx.x) * 4;
                if (i < n) {
                    f(i, r[j].x);
                    f(i + 1, r[j].y);
                    f(i + 2, r[j].z);
                    f(i + 3, r[j].w);
                }
            }
        } else {
            for (int i = threadIdx.x; i < n; i += ROW_THREADS) f(i, x[i]);
        }
    }
    // y[i] = g(i, x[i]); 16-byte stores on the register path
    template <class G> __device__ __forceinline__ void write(float* y, G g) const {
        if (vec && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
#pragma unroll
            for (int j = 0; j < ROW_VEC; j++) {
                const int i = (j * ROW_THREADS + threadIdx.x) * 4;
                if (i < n) __stcs(reinterpret_cast<float4*>(y + i), make_float4(g(i, r[j].x), g(i + 1, r[j].y), g(i + 2, r[j].z), g(i + 3, r[j].w)));
            }
        } else {
            for_each([&](int i, float v) { y[i] = g(i, v); });
        }
    }
};

// CustomCallKernel.java:368-412: rms = (float) sqrt(sumSq / n + eps); y = x * (1 / rms) [* gamma]
__global__ void __launch_bounds__(ROW_THREADS) rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                               float* __restrict__ y, int n, float eps) {
    __shared__ double red[ROW_THREADS / 32];
    const RowView row(x + (size_t)blockIdx.x * n, n);
    float part = 0.f;
    row.for_each([&](int, float v) { part = __fadd_rn(part, __fmul_rn(v, v)); });
    const float sum_sq = (float)block_sum((double)part, red);
    const float rms = (float)sqrt((double)__fadd_rn(__fdiv_rn(sum_sq, (float)n), eps));
    const float inv = __fdiv_rn(1.0f, rms);
    row.write(y + (size_t)blockIdx.x * n, [&](int i, float v) {
        const float t = __fmul_rn(v, inv);
        return gamma ? __fmul_rn(t, gamma[i]) : t;
    });
}

// CustomCallKernel.java:109-171: mean, then the variance of (x - mean), invStd = 1 / (float) sqrt(var + eps)
__global__ void __launch_bounds__(ROW_THREADS) layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                 const float* __restrict__ beta, float* __restrict__ y, int n,
                                                                 float eps) {
    __shared__ double red[ROW_THREADS / 32], red2[ROW_THREADS / 32];
    const RowView row(x + (size_t)blockIdx.x * n, n);
    float part = 0.f;
    row.for_each([&](int, float v) { part = __fadd_rn(part, v); });
    const float mean = __fdiv_rn((float)block_sum((double)part, red), (float)n);
    part = 0.f;
    row.for_each([&](int, float v) {
        const float d = __fsub_rn(v, mean);
        part = __fadd_rn(part, __fmul_rn(d, d));
    });
    const float var = __fdiv_rn((float)block_sum((double)part, red2), (float)n);
    const float inv = __fdiv_rn(1.0f, (float)sqrt((double)__fadd_rn(var, eps)));
    row.write(y + (size_t)blockIdx.x * n, [&](int i, float v) {
        float t = __fmul_rn(__fsub_rn(v, mean), inv);
        if (gamma) t = __fmul_rn(t, gamma[i]);
        if (beta) t = __fadd_rn(t, beta[i]);
        return t;
    });
}

// CustomCallKernel.java:173-224, over the last dimension: (float) exp(x - max) / sum
template <bool EXACT>
__global__ void __launch_bounds__(ROW_THREADS) softmax_kernel(const float* __restrict__ x, float* __restrict__ y, int n) {
    __shared__ double red[ROW_THREADS / 32];
    __shared__ float redf[ROW_THREADS / 32];
    __shared__ double tab[32];
    if (EXACT) load_exp_table(tab);
    RowView row(x + (size_t)blockIdx.x * n, n);
    float mx = -INFINITY;
    row.for_each([&](int, float v) { mx = v > mx ? v : mx; });  // `if (val > maxVal)`: a NaN never becomes the maximum
    mx = block_max(mx, redf);
    float part = 0.f;
    if (row.vec) {  // the exponentials replace the row in registers: one exp per element
        row.map_registers([&](float v) { return exp_sel<EXACT>(__fsub_rn(v, mx), tab); });
        row.for_each([&](int, float e) { part = __fadd_rn(part, e); });
        const float sum = (float)block_sum((double)part, red);
        row.write(y + (size_t)blockIdx.x * n, [&](int, float e) { return __fdiv_rn(e, sum); });
    } else {
        row.for_each([&](int, float v) { part = __fadd_rn(part, exp_sel<EXACT>(__fsub_rn(v, mx), tab)); });
        const float sum = (float)block_sum((double)part, red);
        row.write(y + (size_t)blockIdx.x * n, [&](int, float v) { return __fdiv_rn(exp_sel<EXACT>(__fsub_rn(v, mx), tab), sum); });
    }
}

// ---- element operations: 16 bytes per thread per step, grid sized to the SM count
template <bool EXACT> __device__ __forceinline__ float silu_as_host(float x, const double* tab) {  // CustomCallKernel.java:273-275
    const float sigmoid = __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_sel<EXACT>(-x, tab)));
    return __fmul_rn(x, sigmoid);
}

enum { EL_SILU = 0, EL_SWIGLU = 1, EL_ADD = 2, EL_GELU = 3 };

// CustomCallKernel.java:240-250, the tanh form, float operations in the reference's order; tanh itself in double
// (the reference calls Math.tanh on the widened float), rounded to float once.
__device__ __forceinline__ float gelu_as_host(float x) {
    const float x3 = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, x), x), x);
    const float inner = __fmul_rn(0.7978845608f, __fadd_rn(x, x3));
    const float t = (float)tanh((double)inner);
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, t));
}

template <int OP, bool EXACT> __device__ __forceinline__ float el(float a, float b, const double* tab) {
    if (OP == EL_GELU) return gelu_as_host(a);
    if (OP == EL_SILU) return silu_as_host<EXACT>(a, tab);
    if (OP == EL_SWIGLU) return __fmul_rn(silu_as_host<EXACT>(a, tab), b);
    return __fadd_rn(a, b);
}

template <int OP, bool EXACT>
__global__ void __launch_bounds__(256) elementwise_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          float* __restrict__ y, int64_t n, int vec) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, step = (int64_t)gridDim.x * blockDim.x;
    __shared__ double tab[32];
    if (OP != EL_ADD && OP != EL_GELU && EXACT) load_exp_table(tab);
    if (vec) {
        for (int64_t i = tid; i < n / 4; i += step) {
            const float4 u = __ldcs(reinterpret_cast<const float4*>(a) + i);
            const float4 v = (OP == EL_SILU || OP == EL_GELU) ? u : __ldcs(reinterpret_cast<const float4*>(b) + i);
            __stcs(reinterpret_cast<float4*>(y) + i, make_float4(el<OP, EXACT>(u.x, v.x, tab), el<OP, EXACT>(u.y, v.y, tab), el<OP, EXACT>(u.z, v.z, tab), el<OP, EXACT>(u.w, v.w, tab)));
        }
        for (int64_t i = n / 4 * 4 + tid; i < n; i += step) y[i] = el<OP, EXACT>(a[i], (OP == EL_SILU || OP == EL_GELU) ? 0.f : b[i], tab);
    } else {
        for (int64_t i = tid; i < n; i += step) y[i] = el<OP, EXACT>(a[i], (OP == EL_SILU || OP == EL_GELU) ? 0.f : b[i], tab);
    }
}

// stablehlo.dot on dense fp32 operands, C[M,N] = A[M,K] . B[K,N] (the reference's GPU kernel:
// nvidia/ops/DotKernel.java:18-154 with the naive PTX of nvidia/cuda/CudaKernels.java; CPU arithmetic
// cpu/ops/scalar/DotKernel.java:51-59).  Every output is summed by one thread over k ascending with a separate
// multiply and add, exactly the CPU loop `sum += a * b`, so the result has the CPU's bits; tiles of 64 x 64 outputs
// (4 x 4 per thread) and 16 k per step go through shared memory.  Not a hot path (the quantized linear is): plain
// fp32 arithmetic, no tensor cores, because a reordered or fused sum would not be the reference's number.
constexpr int DOT_TILE = 64, DOT_KSTEP = 16;
__global__ void __launch_bounds__(256) dot_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                                      int M, int N, int K) {
    __shared__ float as[DOT_KSTEP][DOT_TILE + 1], bs[DOT_KSTEP][DOT_TILE];
    const int tx = threadIdx.x, ty = threadIdx.y, tid = ty * 16 + tx;
    const int n0 = blockIdx.x * DOT_TILE;
    for (int m0 = blockIdx.y * DOT_TILE; m0 < M; m0 += gridDim.y * DOT_TILE) {
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
        for (int k0 = 0; k0 < K; k0 += DOT_KSTEP) {
            // A tile [64 rows][16 k] (transposed into as[k][row]) and B tile [16 k][64 cols]: 1024 elements each, 4 per thread
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int e = tid + u * 256;
                const int ar = e >> 4, ak = e & 15;
                as[ak][ar] = (m0 + ar < M && k0 + ak < K) ? a[(size_t)(m0 + ar) * K + k0 + ak] : 0.f;
                const int bk = e >> 6, bc = e & 63;
                bs[bk][bc] = (k0 + bk < K && n0 + bc < N) ? b[(size_t)(k0 + bk) * N + n0 + bc] : 0.f;
            }
            __syncthreads();
            const int kmax = min(DOT_KSTEP, K - k0);  // never add the zero padding: (-0) + (+0) would lose a sign
            for (int kk = 0; kk < kmax; kk++) {
                float av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) av[i] = as[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; j++) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int r = m0 + ty * 4 + i, col = n0 + tx * 4 + j;
                if (r < M && col < N) c[(size_t)r * N + col] = acc[i][j];
            }
    }
}

// CustomCallKernel.java:282-318: row `index` of the table per looked-up position.  The CPU throws on an
// index outside the table; here such a row is filled with zeros and the status word says so.
__global__ void __launch_bounds__(256) embedding_kernel(const int64_t* __restrict__ indices, const float* __restrict__ table,
                                                        float* __restrict__ y, int64_t count, int64_t vocab, int dim, int vec,
                                                        int* status) {
    for (int64_t r = blockIdx.x; r < count; r += gridDim.x) {
        const int64_t idx = (int64_t)(int)indices[r];  // `(int) indexData.getAtIndex(JAVA_LONG, i)`
        const bool ok = idx >= 0 && idx < vocab;
        if (!ok && threadIdx.x == 0) atomicOr(status, STATUS_BAD_INDEX);
        const float* src = table + (size_t)(ok ? idx : 0) * dim;
        float* dst = y + (size_t)r * dim;
        if (vec) {
            for (int i = threadIdx.x; i < dim / 4; i += blockDim.x)
                reinterpret_cast<float4*>(dst)[i] = ok ? __ldg(reinterpret_cast<const float4*>(src) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = ok ? src[i] : 0.f;
        }
    }
}

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }
static bool aligned4(const void* p) { return reinterpret_cast<uintptr_t>(p) % 4 == 0; }

static int element_grid(Context* c, int64_t n) {
    const int64_t want = (n / 4 + 255) / 256;
    return (int)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)c->sm_count * 8));
}

}  // namespace wf

using namespace wf;

#define GLUE_ENTER(ctxh)                                                   \
    Context* c = get_context(ctxh);                                        \
    if (!c) return WF_ERR_INVALID_HANDLE;                                  \
    ScopedLock _lk(c);                                                     \
    if (!_lk.ok) return WF_ERR_BUSY;                                       \
    WF_CUDA(c, cudaSetDevice(c->device));                                  \
    cudaStream_t s = resolve_stream(c, stream)

static int launched(Context* c, const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_status(c, e, what);
    c->launches++;
    return WF_OK;
}

static int check_rows(Context* c, const char* what, int64_t x, int64_t y, int64_t rows, int64_t n) {
    if (!x || !y) return set_error(c, WF_ERR_INVALID_ARGUMENT, "%s: null pointer", what);
    if (!aligned4(reinterpret_cast<void*>(x)) || !aligned4(reinterpret_cast<void*>(y)))
        return set_error(c, WF_ERR_INVALID_ARGUMENT, "%s: fp32 pointers must be 4-byte aligned", what);
    if (rows < 0 || n < 1 || n > (1 << 30) || rows > (1LL << 31) - 1)
        return set_error(c, WF_ERR_SHAPE, "%s: bad shape rows=%lld n=%lld", what, (long long)rows, (long long)n);
    return WF_OK;
}

extern "C" {

int wf_set_exact_exp(int64_t ctx, int on) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    c->glue_exact = on != 0;
    return WF_OK;
}

int wf_rms_norm(int64_t ctx, int64_t x_dev, int64_t gamma_dev, int64_t y_dev, int64_t rows, int64_t n, float eps, int64_t stream) {
    GLUE_ENTER(ctx);
    int rc = check_rows(c, "rms_norm", x_dev, y_dev, rows, n);
    if (rc != WF_OK || rows == 0) return rc;
    rms_norm_kernel<<<(unsigned)rows, ROW_THREADS, 0, s>>>(reinterpret_cast<const float*>(x_dev), reinterpret_cast<const float*>(gamma_dev),
                                                          reinterpret_cast<float*>(y_dev), (int)n, eps);
    return launched(c, "rms_norm");
}

int wf_layer_norm(int64_t ctx, int64_t x_dev, int64_t gamma_dev, int64_t beta_dev, int64_t y_dev, int64_t rows, int64_t n, float eps,
                  int64_t stream) {
    GLUE_ENTER(ctx);
    int rc = check_rows(c, "layer_norm", x_dev, y_dev, rows, n);
    if (rc != WF_OK || rows == 0) return rc;
    layer_norm_kernel<<<(unsigned)rows, ROW_THREADS, 0, s>>>(reinterpret_cast<const float*>(x_dev), reinterpret_cast<const float*>(gamma_dev),
                                                            reinterpret_cast<const float*>(beta_dev), reinterpret_cast<float*>(y_dev), (int)n, eps);
    return launched(c, "layer_norm");
}

int wf_softmax(int64_t ctx, int64_t x_dev, int64_t y_dev, int64_t rows, int64_t n, int64_t stream) {
    GLUE_ENTER(ctx);
    int rc = check_rows(c, "softmax", x_dev, y_dev, rows, n);
    if (rc != WF_OK || rows == 0) return rc;
    if (c->glue_exact)
        softmax_kernel<true><<<(unsigned)rows, ROW_THREADS, 0, s>>>(reinterpret_cast<const float*>(x_dev), reinterpret_cast<float*>(y_dev), (int)n);
    else
        softmax_kernel<false><<<(unsigned)rows, ROW_THREADS, 0, s>>>(reinterpret_cast<const float*>(x_dev), reinterpret_cast<float*>(y_dev), (int)n);
    return launched(c, "softmax");
}

static int elementwise(int64_t ctx, int op, const char* what, int64_t a_dev, int64_t b_dev, int64_t y_dev, int64_t count, int64_t stream) {
    GLUE_ENTER(ctx);
    const void *a = reinterpret_cast<void*>(a_dev), *b = reinterpret_cast<void*>(b_dev), *y = reinterpret_cast<void*>(y_dev);
    const bool unary = op == EL_SILU || op == EL_GELU;
    if (!a || !y || (!unary && !b)) return set_error(c, WF_ERR_INVALID_ARGUMENT, "%s: null pointer", what);
    if (!aligned4(a) || !aligned4(b) || !aligned4(y)) return set_error(c, WF_ERR_INVALID_ARGUMENT, "%s: fp32 pointers must be 4-byte aligned", what);
    if (count < 0) return set_error(c, WF_ERR_SHAPE, "%s: negative element count", what);
    if (count == 0) return WF_OK;
    const int vec = aligned16(a) && aligned16(y) && (unary || aligned16(b));
    const float *fa = static_cast<const float*>(a), *fb = static_cast<const float*>(b);
    float* fy = reinterpret_cast<float*>(y_dev);
    const int grid = element_grid(c, count);
    if (op == EL_GELU) elementwise_kernel<EL_GELU, false><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    else if (op == EL_SILU && c->glue_exact) elementwise_kernel<EL_SILU, true><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    else if (op == EL_SILU) elementwise_kernel<EL_SILU, false><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    else if (op == EL_SWIGLU && c->glue_exact) elementwise_kernel<EL_SWIGLU, true><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    else if (op == EL_SWIGLU) elementwise_kernel<EL_SWIGLU, false><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    else elementwise_kernel<EL_ADD, false><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    return launched(c, what);
}

int wf_silu(int64_t ctx, int64_t x_dev, int64_t y_dev, int64_t count, int64_t stream) {
    return elementwise(ctx, EL_SILU, "silu", x_dev, 0, y_dev, count, stream);
}

int wf_dot_f32(int64_t ctx, int64_t a_dev, int64_t b_dev, int64_t c_dev, int64_t m, int64_t n, int64_t k, int64_t stream) {
    GLUE_ENTER(ctx);
    if (m < 0 || n < 0 || k < 0 || m > (1LL << 30) || n > (1LL << 30) || k > (1LL << 30)) return set_error(c, WF_ERR_SHAPE, "dot: dimension out of range");
    if (m == 0 || n == 0) return WF_OK;
    if (!c_dev || (k > 0 && (!a_dev || !b_dev))) return set_error(c, WF_ERR_INVALID_ARGUMENT, "dot: null pointer");
    if ((a_dev | b_dev | c_dev) & 3) return set_error(c, WF_ERR_INVALID_ARGUMENT, "dot: fp32 pointers must be 4-byte aligned");
    const dim3 grid((unsigned)((n + DOT_TILE - 1) / DOT_TILE), (unsigned)std::min<int64_t>((m + DOT_TILE - 1) / DOT_TILE, 65535));
    dot_f32_kernel<<<grid, dim3(16, 16), 0, s>>>(reinterpret_cast<const float*>(a_dev), reinterpret_cast<const float*>(b_dev),
                                                 reinterpret_cast<float*>(c_dev), (int)m, (int)n, (int)k);
    return launched(c, "dot");
}

int wf_gelu(int64_t ctx, int64_t x_dev, int64_t y_dev, int64_t count, int64_t stream) {
    return elementwise(ctx, EL_GELU, "gelu", x_dev, 0, y_dev, count, stream);
}

int wf_swiglu(int64_t ctx, int64_t gate_dev, int64_t up_dev, int64_t y_dev, int64_t count, int64_t stream) {
    return elementwise(ctx, EL_SWIGLU, "swiglu", gate_dev, up_dev, y_dev, count, stream);
}

int wf_add(int64_t ctx, int64_t a_dev, int64_t b_dev, int64_t y_dev, int64_t count, int64_t stream) {
    return elementwise(ctx, EL_ADD, "add", a_dev, b_dev, y_dev, count, stream);
}

int wf_embedding(int64_t ctx, int64_t indices_dev, int64_t table_dev, int64_t y_dev, int64_t count, int64_t vocab, int64_t dim, int64_t stream) {
    GLUE_ENTER(ctx);
    if (!indices_dev || !table_dev || !y_dev) return set_error(c, WF_ERR_INVALID_ARGUMENT, "embedding: null pointer");
    if (indices_dev % 8 || table_dev % 4 || y_dev % 4) return set_error(c, WF_ERR_INVALID_ARGUMENT, "embedding: misaligned pointer");
    if (count < 0 || vocab < 1 || dim < 1 || dim > (1 << 30)) return set_error(c, WF_ERR_SHAPE, "embedding: bad shape");
    if (count == 0) return WF_OK;
    const int vec = dim % 4 == 0 && table_dev % 16 == 0 && y_dev % 16 == 0;
    const int grid = (int)std::min<int64_t>(count, (int64_t)c->sm_count * 8);
    embedding_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const int64_t*>(indices_dev), reinterpret_cast<const float*>(table_dev),
                                          reinterpret_cast<float*>(y_dev), count, vocab, (int)dim, vec, c->d_status);
    return launched(c, "embedding");
}

}  // extern "C"
