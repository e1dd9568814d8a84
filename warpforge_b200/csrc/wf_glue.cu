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

// (float) Math.exp(x): the exponential in double, one rounding to float.  Only the float result matters,
// so the double value needs far less than the library's last-bit accuracy: argument reduction by ln 2
// in two parts and the Taylor series to r^11 (|r| <= 0.347, truncation below 2^-46) leave an error of
// about 2^-46, which changes the rounded float for roughly one argument in four million.  Outside
// [-104, 89] the float result is 0 or infinity whatever the double is.
__device__ __forceinline__ float exp_as_host(float x) {
    if (x != x) return x;
    if (x > 89.0f) return INFINITY;
    if (x < -104.0f) return 0.0f;
    const double xd = (double)x;
    const double kf = rint(xd * 1.4426950408889634074);
    double r = fma(-kf, 6.93147180369123816490e-01, xd);
    r = fma(-kf, 1.90821492927058770002e-10, r);
    double p = 2.50521083854417187751e-08;  // 1/11!
    p = fma(p, r, 2.75573192239858906526e-07);
    p = fma(p, r, 2.75573192239858906526e-06);
    p = fma(p, r, 2.48015873015873015873e-05);
    p = fma(p, r, 1.98412698412698412698e-04);
    p = fma(p, r, 1.38888888888888888889e-03);
    p = fma(p, r, 8.33333333333333333333e-03);
    p = fma(p, r, 4.16666666666666666667e-02);
    p = fma(p, r, 1.66666666666666666667e-01);
    p = fma(p, r, 0.5);
    p = fma(p, r, 1.0);
    p = fma(p, r, 1.0);
    const long long bits = (long long)((int)kf + 1023) << 52;
    return (float)(p * __longlong_as_double(bits));
}

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
__global__ void __launch_bounds__(ROW_THREADS) softmax_kernel(const float* __restrict__ x, float* __restrict__ y, int n) {
    __shared__ double red[ROW_THREADS / 32];
    __shared__ float redf[ROW_THREADS / 32];
    RowView row(x + (size_t)blockIdx.x * n, n);
    float mx = -INFINITY;
    row.for_each([&](int, float v) { mx = v > mx ? v : mx; });  // `if (val > maxVal)`: a NaN never becomes the maximum
    mx = block_max(mx, redf);
    float part = 0.f;
    if (row.vec) {  // the exponentials replace the row in registers: one exp per element
        row.map_registers([&](float v) { return exp_as_host(__fsub_rn(v, mx)); });
        row.for_each([&](int, float e) { part = __fadd_rn(part, e); });
        const float sum = (float)block_sum((double)part, red);
        row.write(y + (size_t)blockIdx.x * n, [&](int, float e) { return __fdiv_rn(e, sum); });
    } else {
        row.for_each([&](int, float v) { part = __fadd_rn(part, exp_as_host(__fsub_rn(v, mx))); });
        const float sum = (float)block_sum((double)part, red);
        row.write(y + (size_t)blockIdx.x * n, [&](int, float v) { return __fdiv_rn(exp_as_host(__fsub_rn(v, mx)), sum); });
    }
}

// ---- element operations: 16 bytes per thread per step, grid sized to the SM count
__device__ __forceinline__ float silu_as_host(float x) {  // CustomCallKernel.java:273-275
    const float sigmoid = __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_as_host(-x)));
    return __fmul_rn(x, sigmoid);
}

enum { EL_SILU = 0, EL_SWIGLU = 1, EL_ADD = 2 };

template <int OP> __device__ __forceinline__ float el(float a, float b) {
    if (OP == EL_SILU) return silu_as_host(a);
    if (OP == EL_SWIGLU) return __fmul_rn(silu_as_host(a), b);
    return __fadd_rn(a, b);
}

template <int OP>
__global__ void __launch_bounds__(256) elementwise_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          float* __restrict__ y, int64_t n, int vec) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, step = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        for (int64_t i = tid; i < n / 4; i += step) {
            const float4 u = __ldcs(reinterpret_cast<const float4*>(a) + i);
            const float4 v = OP == EL_SILU ? u : __ldcs(reinterpret_cast<const float4*>(b) + i);
            __stcs(reinterpret_cast<float4*>(y) + i, make_float4(el<OP>(u.x, v.x), el<OP>(u.y, v.y), el<OP>(u.z, v.z), el<OP>(u.w, v.w)));
        }
        for (int64_t i = n / 4 * 4 + tid; i < n; i += step) y[i] = el<OP>(a[i], OP == EL_SILU ? 0.f : b[i]);
    } else {
        for (int64_t i = tid; i < n; i += step) y[i] = el<OP>(a[i], OP == EL_SILU ? 0.f : b[i]);
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
    softmax_kernel<<<(unsigned)rows, ROW_THREADS, 0, s>>>(reinterpret_cast<const float*>(x_dev), reinterpret_cast<float*>(y_dev), (int)n);
    return launched(c, "softmax");
}

static int elementwise(int64_t ctx, int op, const char* what, int64_t a_dev, int64_t b_dev, int64_t y_dev, int64_t count, int64_t stream) {
    GLUE_ENTER(ctx);
    const void *a = reinterpret_cast<void*>(a_dev), *b = reinterpret_cast<void*>(b_dev), *y = reinterpret_cast<void*>(y_dev);
    if (!a || !y || (op != EL_SILU && !b)) return set_error(c, WF_ERR_INVALID_ARGUMENT, "%s: null pointer", what);
    if (!aligned4(a) || !aligned4(b) || !aligned4(y)) return set_error(c, WF_ERR_INVALID_ARGUMENT, "%s: fp32 pointers must be 4-byte aligned", what);
    if (count < 0) return set_error(c, WF_ERR_SHAPE, "%s: negative element count", what);
    if (count == 0) return WF_OK;
    const int vec = aligned16(a) && aligned16(y) && (op == EL_SILU || aligned16(b));
    const float *fa = static_cast<const float*>(a), *fb = static_cast<const float*>(b);
    float* fy = reinterpret_cast<float*>(y_dev);
    const int grid = element_grid(c, count);
    if (op == EL_SILU) elementwise_kernel<EL_SILU><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    else if (op == EL_SWIGLU) elementwise_kernel<EL_SWIGLU><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    else elementwise_kernel<EL_ADD><<<grid, 256, 0, s>>>(fa, fb, fy, count, vec);
    return launched(c, what);
}

int wf_silu(int64_t ctx, int64_t x_dev, int64_t y_dev, int64_t count, int64_t stream) {
    return elementwise(ctx, EL_SILU, "silu", x_dev, 0, y_dev, count, stream);
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
