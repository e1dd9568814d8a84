/*
 * CPU oracle for the quantized-matmul path -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement of what WarpForge's CPU side computes when a GGUF block-quantized
 * weight is dequantized to fp32 and fed to the CPU backend's dot_general.  Only the tests,
 * the smoke check and the CPU-baseline legs of the benchmark may link or load this file;
 * the CUDA library never does.
 *
 * Reference files followed (paths inside the WarpForge project):
 *   fp16 -> fp32      warpforge-data/src/main/java/io/surfworks/warpforge/data/quant/Dequantizer.java:121-147
 *   bf16 -> fp32      .../quant/Dequantizer.java:178-182  (bits << 16)
 *   Q8_0 block        .../quant/Dequantizer.java:204-221
 *   Q4_0 block        .../quant/Dequantizer.java:251-279  (interleaved: byte i -> elements 2i, 2i+1)
 *   Q4_1 block        .../quant/Dequantizer.java:304-358
 *   dot_general       warpforge-backend-cpu/src/main/java/io/surfworks/warpforge/backend/cpu/ops/scalar/DotGeneralKernel.java:17-133
 *   dot               warpforge-backend-cpu/src/main/java/io/surfworks/warpforge/backend/cpu/ops/scalar/DotKernel.java:18-102
 *   tolerance rule    warpforge-core/src/main/java/io/surfworks/warpforge/core/testing/ToleranceConfig.java:164-182
 *
 * Q4_K has no implementation in the reference (Dequantizer.forType throws for it,
 * Dequantizer.java:58-71; only the geometry 256 elements / 144 bytes is fixed at
 * warpforge-data/.../format/GGUF.java:345-346).  wfo_dequant_q4_k restates the public GGUF
 * Q4_K super-block format; its parity is UNPINNED by the reference and is cross-checked
 * only against the third-party gguf Python package used as a black box.  The same holds for
 * Q5_0 (22 bytes / 32 elements, sized at GGUF.java:332-351, never dequantized by the reference):
 * wfo_dequant_q5_0 restates the public block format, parity UNPINNED, cross-checked against gguf.
 *
 * Java evaluates `sum += a * b` on floats as a separately rounded multiply and add, in
 * ascending k, with one accumulator.  Build with -ffp-contract=off so gcc does the same.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define WFO_Q8_0 8
#define WFO_Q4_0 2
#define WFO_Q4_1 3
#define WFO_Q4_K 14
#define WFO_Q5_0 6

static inline float bits_to_float(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* Dequantizer.java:121-147.  Subnormals are mant/1024 * 2^-14, NaN is the canonical quiet NaN. */
float wfo_half_to_float(uint16_t bits) {
    uint32_t sign = (bits >> 15) & 0x1u;
    uint32_t exp = (bits >> 10) & 0x1Fu;
    uint32_t mant = bits & 0x3FFu;
    if (exp == 0) {
        if (mant == 0) return sign ? -0.0f : 0.0f;
        float val = (float)mant / 1024.0f;
        val = (float)((double)val * 6.103515625e-05); /* Math.pow(2, -14) in double, cast back */
        return sign ? -val : val;
    }
    if (exp == 31) {
        if (mant == 0) return sign ? -INFINITY : INFINITY;
        return bits_to_float(0x7FC00000u); /* Float.NaN */
    }
    return bits_to_float((sign << 31) | ((exp + 112u) << 23) | (mant << 13));
}

/* Dequantizer.java:178-182 */
float wfo_bf16_to_float(uint16_t bits) { return bits_to_float((uint32_t)bits << 16); }

void wfo_half_to_float_array(const uint16_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = wfo_half_to_float(in[i]);
}

void wfo_bf16_to_float_array(const uint16_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = wfo_bf16_to_float(in[i]);
}

static inline uint16_t load_u16(const uint8_t* p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }

/* Dequantizer.java:204-221.  blocks = ceil(n/32); writes stop at n. */
void wfo_dequant_q8_0(const uint8_t* in, float* out, int64_t n) {
    int64_t nblocks = (n + 31) / 32, o = 0;
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t* blk = in + b * 34;
        float scale = wfo_half_to_float(load_u16(blk));
        for (int i = 0; i < 32 && o < n; i++) out[o++] = (float)(int8_t)blk[2 + i] * scale;
    }
}

/* Dequantizer.java:251-279.  Low nibble first, then high nibble of the same byte. */
void wfo_dequant_q4_0(const uint8_t* in, float* out, int64_t n) {
    int64_t nblocks = (n + 31) / 32, o = 0;
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t* blk = in + b * 18;
        float scale = wfo_half_to_float(load_u16(blk));
        for (int i = 0; i < 16 && o < n; i++) {
            uint8_t packed = blk[2 + i];
            int q0 = (packed & 0x0F) - 8;
            if (o < n) out[o++] = (float)q0 * scale;
            int q1 = ((packed >> 4) & 0x0F) - 8;
            if (o < n) out[o++] = (float)q1 * scale;
        }
    }
}

/* Dequantizer.java:304-358: scale fp16, min fp16, 16 code bytes; value = q * scale + min. */
void wfo_dequant_q4_1(const uint8_t* in, float* out, int64_t n) {
    int64_t nblocks = (n + 31) / 32, o = 0;
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t* blk = in + b * 20;
        float scale = wfo_half_to_float(load_u16(blk));
        float min = wfo_half_to_float(load_u16(blk + 2));
        for (int i = 0; i < 16 && o < n; i++) {
            uint8_t packed = blk[4 + i];
            if (o < n) out[o++] = (float)(packed & 0x0F) * scale + min;
            if (o < n) out[o++] = (float)((packed >> 4) & 0x0F) * scale + min;
        }
    }
}

/*
 * Q5_0 block, 22 bytes / 32 elements (public GGUF format; the reference only knows its size,
 * GGUF.java:332-351): [0:2) d fp16, [2:6) 32 high bits (little-endian word, bit e = element e),
 * [6:22) 16 code bytes: element i < 16 = low nibble of byte i, element i + 16 = high nibble of byte i.
 * w = d * ((nibble | bit << 4) - 16).
 */
void wfo_dequant_q5_0(const uint8_t* in, float* out, int64_t n) {
    int64_t nblocks = (n + 31) / 32;
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t* blk = in + b * 22;
        float d = wfo_half_to_float(load_u16(blk));
        uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
        for (int e = 0; e < 32; e++) {
            int64_t o = b * 32 + e;
            if (o >= n) break;
            uint8_t byte = blk[6 + (e & 15)];
            int nib = e < 16 ? (byte & 0x0F) : (byte >> 4);
            int q = (nib | (int)(((qh >> e) & 1u) << 4)) - 16;
            out[o] = (float)q * d;
        }
    }
}

/*
 * Q4_K super-block, 144 bytes / 256 elements (public GGUF format; NOT in the reference):
 *   [0:2) d fp16, [2:4) dmin fp16, [4:16) eight 6-bit scales + eight 6-bit mins, [16:144) codes.
 * Sub-block j < 4: sc = s[j] & 63, m = s[j+4] & 63;
 * j >= 4:          sc = (s[j+4] & 15) | ((s[j-4] >> 6) << 4), m = (s[j+4] >> 4) | ((s[j] >> 6) << 4).
 * Code bytes [32c, 32c+32) hold elements 64c+l in the low nibble (sub-block 2c) and
 * 64c+32+l in the high nibble (sub-block 2c+1).  w = (d*sc)*q - (dmin*m), all fp32.
 */
void wfo_q4k_scale_min(const uint8_t* s, int j, int* sc, int* m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        *m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

void wfo_dequant_q4_k(const uint8_t* in, float* out, int64_t n) {
    int64_t nblocks = (n + 255) / 256;
    float tmp[256];
    for (int64_t b = 0; b < nblocks; b++) {
        const uint8_t* blk = in + b * 144;
        float d = wfo_half_to_float(load_u16(blk));
        float dmin = wfo_half_to_float(load_u16(blk + 2));
        const uint8_t* s = blk + 4;
        const uint8_t* q = blk + 16;
        for (int c = 0; c < 4; c++) {
            int sc, m;
            wfo_q4k_scale_min(s, 2 * c, &sc, &m);
            float d1 = d * (float)sc, m1 = dmin * (float)m;
            wfo_q4k_scale_min(s, 2 * c + 1, &sc, &m);
            float d2 = d * (float)sc, m2 = dmin * (float)m;
            for (int l = 0; l < 32; l++) {
                tmp[64 * c + l] = d1 * (float)(q[32 * c + l] & 0x0F) - m1;
                tmp[64 * c + 32 + l] = d2 * (float)(q[32 * c + l] >> 4) - m2;
            }
        }
        int64_t left = n - b * 256;
        memcpy(out + b * 256, tmp, (size_t)(left < 256 ? left : 256) * sizeof(float));
    }
}

int64_t wfo_block_elems(int qtype) { return qtype == WFO_Q4_K ? 256 : 32; }

int64_t wfo_block_bytes(int qtype) {
    switch (qtype) {
        case WFO_Q8_0: return 34;
        case WFO_Q4_0: return 18;
        case WFO_Q4_1: return 20;
        case WFO_Q4_K: return 144;
        case WFO_Q5_0: return 22;
        default: return -1;
    }
}

int wfo_dequant(int qtype, const uint8_t* in, float* out, int64_t n) {
    switch (qtype) {
        case WFO_Q8_0: wfo_dequant_q8_0(in, out, n); return 0;
        case WFO_Q4_0: wfo_dequant_q4_0(in, out, n); return 0;
        case WFO_Q4_1: wfo_dequant_q4_1(in, out, n); return 0;
        case WFO_Q4_K: wfo_dequant_q4_k(in, out, n); return 0;
        case WFO_Q5_0: wfo_dequant_q5_0(in, out, n); return 0;
        default: return -1; /* Dequantizer.forType: "Dequantization not yet implemented" */
    }
}

/* DotKernel.java:51-59: [M,K] x [K,N], sum += a*b, k ascending. */
void wfo_dot_f32(const float* a, const float* b, float* c, int64_t M, int64_t K, int64_t N) {
    for (int64_t m = 0; m < M; m++)
        for (int64_t n = 0; n < N; n++) {
            float sum = 0.0f;
            for (int64_t k = 0; k < K; k++) sum += a[m * K + k] * b[k * N + n];
            c[m * N + n] = sum;
        }
}

/*
 * DotGeneralKernel.java:17-133, generic form.  Shapes are row-major; output index order is
 * batch dims, lhs free dims, rhs free dims (lines 64-82); the contraction counter advances
 * the last contracting dim fastest (lines 118-125).  Returns 0, or -1 on a rank above 8.
 */
int wfo_dot_general_f32(const float* lhs, const int64_t* lhs_shape, int lhs_rank, const float* rhs,
                        const int64_t* rhs_shape, int rhs_rank, const int64_t* lhs_batch,
                        const int64_t* rhs_batch, int n_batch, const int64_t* lhs_contract,
                        const int64_t* rhs_contract, int n_contract, float* out) {
    if (lhs_rank > 8 || rhs_rank > 8) return -1;
    int64_t lstr[8], rstr[8];
    int lfree[8], rfree[8], nlf = 0, nrf = 0;
    for (int i = lhs_rank - 1, s = 1; i >= 0; i--) { lstr[i] = s; s *= (int)lhs_shape[i]; }
    for (int i = rhs_rank - 1, s = 1; i >= 0; i--) { rstr[i] = s; s *= (int)rhs_shape[i]; }
    for (int d = 0; d < lhs_rank; d++) {
        int used = 0;
        for (int i = 0; i < n_batch; i++) used |= lhs_batch[i] == d;
        for (int i = 0; i < n_contract; i++) used |= lhs_contract[i] == d;
        if (!used) lfree[nlf++] = d;
    }
    for (int d = 0; d < rhs_rank; d++) {
        int used = 0;
        for (int i = 0; i < n_batch; i++) used |= rhs_batch[i] == d;
        for (int i = 0; i < n_contract; i++) used |= rhs_contract[i] == d;
        if (!used) rfree[nrf++] = d;
    }
    int out_rank = n_batch + nlf + nrf;
    int64_t oshape[24], total = 1, csize = 1;
    for (int i = 0; i < n_batch; i++) oshape[i] = lhs_shape[lhs_batch[i]];
    for (int i = 0; i < nlf; i++) oshape[n_batch + i] = lhs_shape[lfree[i]];
    for (int i = 0; i < nrf; i++) oshape[n_batch + nlf + i] = rhs_shape[rfree[i]];
    for (int i = 0; i < out_rank; i++) total *= oshape[i];
    for (int i = 0; i < n_contract; i++) csize *= lhs_shape[lhs_contract[i]];

    for (int64_t flat = 0; flat < total; flat++) {
        int64_t oidx[24], rem = flat;
        for (int i = out_rank - 1; i >= 0; i--) { oidx[i] = rem % oshape[i]; rem /= oshape[i]; }
        int64_t lbase = 0, rbase = 0;
        for (int i = 0; i < n_batch; i++) {
            lbase += oidx[i] * lstr[lhs_batch[i]];
            rbase += oidx[i] * rstr[rhs_batch[i]];
        }
        for (int i = 0; i < nlf; i++) lbase += oidx[n_batch + i] * lstr[lfree[i]];
        for (int i = 0; i < nrf; i++) rbase += oidx[n_batch + nlf + i] * rstr[rfree[i]];
        int64_t cidx[8] = {0};
        float sum = 0.0f;
        for (int64_t c = 0; c < csize; c++) {
            int64_t lo = lbase, ro = rbase;
            for (int i = 0; i < n_contract; i++) {
                lo += cidx[i] * lstr[lhs_contract[i]];
                ro += cidx[i] * rstr[rhs_contract[i]];
            }
            sum += lhs[lo] * rhs[ro];
            for (int i = n_contract - 1; i >= 0; i--) {
                if (++cidx[i] < lhs_shape[lhs_contract[i]]) break;
                cidx[i] = 0;
            }
        }
        out[flat] = sum;
    }
    return 0;
}

/* linear: lhs [M,K] contract 1, rhs [N,K] contract 1 -> [M,N]; same accumulate rule. */
static void linear_rows(const float* x, const float* wrow, float* y, int64_t M, int64_t N, int64_t K,
                        int64_t n) {
    for (int64_t m = 0; m < M; m++) {
        const float* xr = x + m * K;
        float sum = 0.0f;
        for (int64_t k = 0; k < K; k++) sum += xr[k] * wrow[k];
        y[m * N + n] = sum;
    }
}

/* Static split of [0, n) over nthreads pthreads; each thread runs fn(ctx, begin, end). */
typedef void (*wfo_range_fn)(void* ctx, int64_t begin, int64_t end);
typedef struct { wfo_range_fn fn; void* ctx; int64_t begin, end; } wfo_task;

static void* wfo_task_main(void* p) {
    wfo_task* t = (wfo_task*)p;
    t->fn(t->ctx, t->begin, t->end);
    return NULL;
}

static void wfo_parallel_for(int64_t n, int nthreads, wfo_range_fn fn, void* ctx) {
    int nt = nthreads > 0 ? nthreads : 1;
    if (nt > 256) nt = 256;
    if ((int64_t)nt > n) nt = n > 0 ? (int)n : 1;
    if (nt == 1) { fn(ctx, 0, n); return; }
    pthread_t th[256];
    wfo_task tasks[256];
    for (int t = 0; t < nt; t++) {
        tasks[t].fn = fn;
        tasks[t].ctx = ctx;
        tasks[t].begin = n * t / nt;
        tasks[t].end = n * (t + 1) / nt;
        if (t > 0 && pthread_create(&th[t], NULL, wfo_task_main, &tasks[t]) != 0) {
            wfo_task_main(&tasks[t]); /* could not spawn: run it here */
            tasks[t].fn = NULL;
        }
    }
    wfo_task_main(&tasks[0]);
    for (int t = 1; t < nt; t++)
        if (tasks[t].fn) pthread_join(th[t], NULL);
}

typedef struct {
    int qtype;
    const uint8_t* blocks;
    const float* w;
    const float* x;
    float* y;
    const int64_t* rows;
    int64_t M, N, K, row_bytes;
} wfo_lin_ctx;

static void linear_f32_range(void* p, int64_t b, int64_t e) {
    wfo_lin_ctx* c = (wfo_lin_ctx*)p;
    for (int64_t n = b; n < e; n++) linear_rows(c->x, c->w + n * c->K, c->y, c->M, c->N, c->K, n);
}

void wfo_linear_f32(const float* x, const float* w, float* y, int64_t M, int64_t N, int64_t K,
                    int nthreads) {
    wfo_lin_ctx c = {0, NULL, w, x, y, NULL, M, N, K, 0};
    wfo_parallel_for(N, nthreads, linear_f32_range, &c);
}

static void qlinear_range(void* p, int64_t b, int64_t e) {
    wfo_lin_ctx* c = (wfo_lin_ctx*)p;
    float* wrow = (float*)malloc((size_t)c->K * sizeof(float));
    for (int64_t i = b; i < e; i++) {
        int64_t n = c->rows ? c->rows[i] : i;
        wfo_dequant(c->qtype, c->blocks + n * c->row_bytes, wrow, c->K);
        if (c->rows) {
            for (int64_t m = 0; m < c->M; m++) {
                const float* xr = c->x + m * c->K;
                float sum = 0.0f;
                for (int64_t k = 0; k < c->K; k++) sum += xr[k] * wrow[k];
                c->y[i * c->M + m] = sum;
            }
        } else {
            linear_rows(c->x, wrow, c->y, c->M, c->N, c->K, n);
        }
    }
    free(wrow);
}

/*
 * The composed path: dequantize the weight to fp32 exactly as QuantizedTensorView.
 * dequantizeToArray would (QuantizedTensorView.java:161-166), then the sequential fp32 dot.
 * Rows are dequantized one at a time (K is a multiple of the block, so a row is a whole
 * number of blocks and per-row dequant gives the same floats as whole-tensor dequant).
 * Parallel over output rows only, never over k.  x is fp32 [M,K] (bf16 activations are
 * widened exactly by the caller).  Returns 0, -1 for an unknown type, -2 if K is ragged.
 */
int wfo_qlinear(int qtype, const uint8_t* blocks, int64_t N, int64_t K, const float* x, int64_t M,
                float* y, int nthreads) {
    int64_t be = wfo_block_elems(qtype), bb = wfo_block_bytes(qtype);
    if (bb < 0) return -1;
    if (K % be != 0) return -2;
    wfo_lin_ctx c = {qtype, blocks, NULL, x, y, NULL, M, N, K, K / be * bb};
    wfo_parallel_for(N, nthreads, qlinear_range, &c);
    return 0;
}

/* Same, for a subset of rows: y_rows[i*M + m] for row rows[i] (sampled parity at large sizes). */
int wfo_qlinear_rows(int qtype, const uint8_t* blocks, int64_t K, const float* x, int64_t M,
                     const int64_t* rows, int64_t nrows, float* y_rows, int nthreads) {
    int64_t be = wfo_block_elems(qtype), bb = wfo_block_bytes(qtype);
    if (bb < 0) return -1;
    if (K % be != 0) return -2;
    wfo_lin_ctx c = {qtype, blocks, NULL, x, y_rows, rows, M, 0, K, K / be * bb};
    wfo_parallel_for(nrows, nthreads, qlinear_range, &c);
    return 0;
}

/* ToleranceConfig.java:164-182; returns the number of elements that are NOT close. */
int64_t wfo_count_not_close(const float* expected, const float* actual, int64_t n, double atol,
                            double rtol) {
    int64_t bad = 0;
    for (int64_t i = 0; i < n; i++) {
        double e = expected[i], a = actual[i];
        if (isnan(e) && isnan(a)) continue;
        if (isnan(e) || isnan(a)) { bad++; continue; }
        if (isinf(e) && isinf(a)) { bad += e != a; continue; }
        if (isinf(e) || isinf(a)) { bad++; continue; }
        if (fabs(e - a) > atol + rtol * fabs(e)) bad++;
    }
    return bad;
}

/* ---- the fp32 operations between the projections (CPU backend CustomCallKernel.java) --------------
 * One float accumulator, elements in ascending order, every operation rounded to float as the Java
 * code's float arithmetic is; Math.exp / Math.sqrt are the double functions, cast back to float. */

/* CustomCallKernel.java:368-412.  gamma may be NULL (the optional second input). */
void wfo_rms_norm(const float* x, const float* gamma, float* y, int64_t rows, int64_t n, float eps) {
    for (int64_t b = 0; b < rows; b++) {
        const float* in = x + b * n;
        float sum_sq = 0;
        for (int64_t i = 0; i < n; i++) sum_sq += in[i] * in[i];
        float rms = (float)sqrt((double)(sum_sq / (float)n + eps));
        float inv = 1.0f / rms;
        for (int64_t i = 0; i < n; i++) {
            float v = in[i] * inv;
            if (gamma) v *= gamma[i];
            y[b * n + i] = v;
        }
    }
}

/* CustomCallKernel.java:109-171.  gamma / beta may be NULL. */
void wfo_layer_norm(const float* x, const float* gamma, const float* beta, float* y, int64_t rows, int64_t n, float eps) {
    for (int64_t b = 0; b < rows; b++) {
        const float* in = x + b * n;
        float sum = 0;
        for (int64_t i = 0; i < n; i++) sum += in[i];
        float mean = sum / (float)n;
        float var_sum = 0;
        for (int64_t i = 0; i < n; i++) {
            float d = in[i] - mean;
            var_sum += d * d;
        }
        float var = var_sum / (float)n;
        float inv = 1.0f / (float)sqrt((double)(var + eps));
        for (int64_t i = 0; i < n; i++) {
            float v = (in[i] - mean) * inv;
            if (gamma) v *= gamma[i];
            if (beta) v += beta[i];
            y[b * n + i] = v;
        }
    }
}

/* CustomCallKernel.java:173-224 with the default dimension (the last one, inner size 1). */
void wfo_softmax(const float* x, float* y, int64_t rows, int64_t n) {
    for (int64_t b = 0; b < rows; b++) {
        const float* in = x + b * n;
        float mx = -INFINITY;
        for (int64_t i = 0; i < n; i++)
            if (in[i] > mx) mx = in[i];
        float sum = 0;
        for (int64_t i = 0; i < n; i++) sum += (float)exp((double)(in[i] - mx));
        for (int64_t i = 0; i < n; i++) y[b * n + i] = (float)exp((double)(in[i] - mx)) / sum;
    }
}

/* CustomCallKernel.java:262-280 */
void wfo_silu(const float* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float sigmoid = 1.0f / (1.0f + (float)exp((double)-x[i]));
        y[i] = x[i] * sigmoid;
    }
}

/* CustomCallKernel.java:226-260, the tanh form (the only one reachable: `approximate` is fixed to "tanh"):
 * inner = 0.7978845608f * (x + 0.044715f * x * x * x) in float, left to right; 0.5f * x * (1.0f + (float) tanh(inner)). */
void wfo_gelu(const float* x, float* y, int64_t n) {
    const float SQRT_2_OVER_PI = 0.7978845608f, COEFF = 0.044715f;
    for (int64_t i = 0; i < n; i++) {
        float v = x[i];
        float inner = SQRT_2_OVER_PI * (v + COEFF * v * v * v);
        y[i] = 0.5f * v * (1.0f + (float)tanh((double)inner));
    }
}

/* silu custom_call, then stablehlo.multiply (cpu/ops/scalar/MultiplyKernel: a[i] * b[i]) */
void wfo_swiglu(const float* gate, const float* up, float* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float sigmoid = 1.0f / (1.0f + (float)exp((double)-gate[i]));
        float s = gate[i] * sigmoid;
        y[i] = s * up[i];
    }
}

/* stablehlo.add (cpu/ops/scalar/AddKernel: a[i] + b[i]) */
void wfo_add(const float* a, const float* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = a[i] + b[i];
}

/* CustomCallKernel.java:282-318; returns -1 at the first index outside the table (Java throws there). */
int wfo_embedding(const int64_t* indices, const float* table, float* y, int64_t count, int64_t vocab, int64_t dim) {
    for (int64_t i = 0; i < count; i++) {
        int64_t idx = (int64_t)(int32_t)indices[i];
        if (idx < 0 || idx >= vocab) return -1;
        memcpy(y + i * dim, table + idx * dim, (size_t)dim * sizeof(float));
    }
    return 0;
}

int wfo_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
