// Host runtime behind the C ABI: contexts, streams, memory, weight upload, the qlinear
// dispatch and error reporting.  Plays the part of CudaContext + NvidiaBackend's device
// bookkeeping (warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/
// cuda/CudaContext.java:21-657, NvidiaBackend.java:85-463), but keeps weights resident on
// the device and never synchronizes inside the hot call when it is given device pointers.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <thread>
#include <unordered_set>

#include "wf_common.cuh"

namespace wf {

static std::mutex g_registry_mu;
static std::unordered_set<Context*> g_contexts;

int set_error(Context* c, int status, const char* fmt, ...) {
    if (c) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        c->last_error = buf;
    }
    return status;
}

int cuda_status(Context* c, cudaError_t e, const char* what) {
    return set_error(c, WF_ERR_CUDA_BASE + (int)e, "%s failed: %s (%d)", what, cudaGetErrorName(e), (int)e);
}

Context* get_context(int64_t h) {
    Context* c = reinterpret_cast<Context*>(h);
    std::lock_guard<std::mutex> lk(g_registry_mu);
    if (!c || !g_contexts.count(c) || c->magic != CTX_MAGIC) return nullptr;
    return c;
}

Weight* get_weight(Context* c, int64_t h) {
    Weight* w = reinterpret_cast<Weight*>(h);
    if (!w || std::find(c->weights.begin(), c->weights.end(), w) == c->weights.end() || w->magic != WEIGHT_MAGIC)
        return nullptr;
    return w;
}

cudaStream_t resolve_stream(Context* c, int64_t stream) {
    return stream == 0 ? c->stream : reinterpret_cast<cudaStream_t>(stream);
}

int ensure_stage(Context* c, int64_t host_bytes, int64_t dev_bytes) {
    if (host_bytes > c->h_stage_bytes) {
        if (c->h_stage) cudaFreeHost(c->h_stage);
        c->h_stage = nullptr;
        c->h_stage_bytes = 0;
        WF_CUDA(c, cudaMallocHost(&c->h_stage, (size_t)host_bytes));
        c->h_stage_bytes = host_bytes;
    }
    if (dev_bytes > c->d_stage_bytes) {
        if (c->d_stage) cudaFree(c->d_stage);
        c->d_stage = nullptr;
        c->d_stage_bytes = 0;
        WF_CUDA(c, cudaMalloc(&c->d_stage, (size_t)dev_bytes));
        c->d_stage_bytes = dev_bytes;
    }
    return WF_OK;
}

// Host blocks (pageable memory, e.g. a mapped file) -> tiled device layout as a three-stage pipeline over
// chunks of whole 16-row tiles: helper threads copy chunk i+1 into one of two pinned buffers while the DMA
// of chunk i runs and the repack kernel of chunk i-1 writes its tiles.  A plain cudaMemcpyAsync from
// pageable memory stages through one driver thread and runs several times slower; the scratch on the
// device is two chunks, not a second copy of the tensor.
constexpr int64_t UPLOAD_CHUNK = 8 << 20;
constexpr int UPLOAD_THREADS = 4;

static cudaError_t upload_and_repack(Context* c, int qtype, const uint8_t* src, int64_t rows, int64_t k, int64_t row_bytes,
                                     uint8_t* d_tiles, int64_t tile_row_bytes, int q4_0_order, cudaStream_t s) {
    const int64_t chunk_rows = std::max<int64_t>(TILE_ROWS, UPLOAD_CHUNK / row_bytes / TILE_ROWS * TILE_ROWS);
    const int64_t chunk_bytes = (chunk_rows * row_bytes + 255) & ~255LL;
    const int nchunks = (int)((rows + chunk_rows - 1) / chunk_rows);
    cudaError_t e = cudaSuccess;
    if (chunk_bytes > c->upload_chunk_bytes) {
        if (c->h_upload) cudaFreeHost(c->h_upload);
        if (c->d_upload) cudaFree(c->d_upload);
        c->h_upload = c->d_upload = nullptr;
        c->upload_chunk_bytes = 0;
        e = cudaMallocHost(&c->h_upload, (size_t)(2 * chunk_bytes));
        if (e == cudaSuccess) e = cudaMalloc(&c->d_upload, (size_t)(2 * chunk_bytes));
        if (e != cudaSuccess) return e;
        c->upload_chunk_bytes = chunk_bytes;
    }
    for (int i = 0; i < 2; i++)
        if (!c->upload_done[i] && (e = cudaEventCreateWithFlags(&c->upload_done[i], cudaEventDisableTiming)) != cudaSuccess) return e;
    uint8_t* const pinned = static_cast<uint8_t*>(c->h_upload);
    auto chunk_size = [&](int i) { return std::min(chunk_rows, rows - i * chunk_rows) * row_bytes; };

    // released: chunks [0, released) may be written into their pinned buffer; filled[i]: helpers done with chunk i
    const int helpers_n = rows * row_bytes > (1 << 20) ? UPLOAD_THREADS : 0;
    std::atomic<int> released{2};
    std::atomic<bool> stop{false};
    std::vector<std::atomic<int>> filled((size_t)nchunks);
    for (auto& f : filled) f.store(0);
    std::vector<std::thread> helpers;
    for (int t = 0; t < helpers_n; t++)
        helpers.emplace_back([&, t] {
            for (int i = 0; i < nchunks; i++) {
                while (released.load(std::memory_order_acquire) <= i && !stop.load()) std::this_thread::yield();
                if (stop.load()) return;
                const int64_t n = chunk_size(i), part = (n / helpers_n + 4095) & ~4095LL;
                const int64_t lo = std::min(n, t * part), hi = std::min(n, (t + 1) * part);
                if (hi > lo) memcpy(pinned + (i & 1) * chunk_bytes + lo, src + i * chunk_rows * row_bytes + lo, (size_t)(hi - lo));
                filled[(size_t)i].fetch_add(1, std::memory_order_release);
            }
        });
    for (int i = 0; i < nchunks && e == cudaSuccess; i++) {
        const int64_t n = chunk_size(i), r0 = i * chunk_rows;
        uint8_t* h = pinned + (i & 1) * chunk_bytes;
        uint8_t* d = static_cast<uint8_t*>(c->d_upload) + (i & 1) * chunk_bytes;
        if (helpers_n == 0) {
            if (i >= 2) e = cudaEventSynchronize(c->upload_done[i & 1]);
            memcpy(h, src + r0 * row_bytes, (size_t)n);
        } else {
            while (filled[(size_t)i].load(std::memory_order_acquire) < helpers_n) std::this_thread::yield();
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(d, h, (size_t)n, cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) e = cudaEventRecord(c->upload_done[i & 1], s);
        if (e == cudaSuccess) e = launch_repack(qtype, d, d_tiles + r0 / TILE_ROWS * tile_row_bytes, n / row_bytes, k, q4_0_order, s);
        if (helpers_n && i >= 1 && e == cudaSuccess) {  // the DMA of chunk i-1 has left its pinned buffer: chunk i+1 may fill it
            e = cudaEventSynchronize(c->upload_done[(i - 1) & 1]);
            released.store(i + 2, std::memory_order_release);
        }
    }
    stop.store(e != cudaSuccess);
    for (std::thread& h : helpers) h.join();
    return e;
}

static bool qtype_supported(int qt) {
    return qt == WF_QTYPE_Q4_0 || qt == WF_QTYPE_Q4_1 || qt == WF_QTYPE_Q5_0 || qt == WF_QTYPE_Q8_0 || qt == WF_QTYPE_Q4_K;
}

}  // namespace wf

using namespace wf;

#define WF_ENTER(ctxh)                                   \
    Context* c = get_context(ctxh);                      \
    if (!c) return WF_ERR_INVALID_HANDLE;                \
    ScopedLock _lk(c);                                   \
    if (!_lk.ok) return WF_ERR_BUSY;                     \
    {                                                    \
        cudaError_t _e = cudaSetDevice(c->device);       \
        if (_e != cudaSuccess) return cuda_status(c, _e, "cudaSetDevice"); \
    }

extern "C" {

int wf_version(void) { return 100; }

int wf_device_count(int* count) {
    if (!count) return WF_ERR_INVALID_ARGUMENT;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        cudaGetLastError();
        return WF_ERR_NO_DEVICE;
    }
    *count = n;
    return WF_OK;
}

int wf_init(int device, int64_t* ctx) {
    if (!ctx) return WF_ERR_INVALID_ARGUMENT;
    *ctx = 0;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        return WF_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= n) return WF_ERR_INVALID_ARGUMENT;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return WF_ERR_NO_DEVICE;
    if (prop.major != 10) return WF_ERR_NOT_SM100;  // kernels are built for sm_100a only
    Context* c = new Context();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->cc_major = prop.major;
    c->cc_minor = prop.minor;
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&c->d_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->d_status, 0, sizeof(int));
    if (e != cudaSuccess) {
        if (c->stream) cudaStreamDestroy(c->stream);
        delete c;
        return WF_ERR_CUDA_BASE + (int)e;
    }
    {
        std::lock_guard<std::mutex> lk(g_registry_mu);
        g_contexts.insert(c);
    }
    *ctx = reinterpret_cast<int64_t>(c);
    return WF_OK;
}

int wf_destroy(int64_t ctx) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    if (!c->mu.try_lock()) return WF_ERR_BUSY;
    {
        std::lock_guard<std::mutex> lk(g_registry_mu);
        g_contexts.erase(c);
    }
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (Weight* w : c->weights) {
        cudaFree(w->d_tiles);
        w->magic = 0;
        delete w;
    }
    for (auto& kv : c->allocs) cudaFree(reinterpret_cast<void*>(kv.first));
    for (void* h : c->host_allocs) cudaFreeHost(h);
    for (auto& kv : c->gemv_scratch) {
        cudaFree(kv.second.d_slots);
        cudaFree(kv.second.d_part);
        cudaFree(kv.second.d_count);
    }
    for (cudaGraphExec_t g : c->graphs) cudaGraphExecDestroy(g);
    for (cudaEvent_t ev : c->events) cudaEventDestroy(ev);
    for (cudaStream_t s : c->streams) cudaStreamDestroy(s);
    if (c->h_stage) cudaFreeHost(c->h_stage);
    if (c->h_upload) cudaFreeHost(c->h_upload);
    if (c->d_upload) cudaFree(c->d_upload);
    for (cudaEvent_t e : c->upload_done)
        if (e) cudaEventDestroy(e);
    if (c->d_stage) cudaFree(c->d_stage);
    if (c->d_x16) cudaFree(c->d_x16);
    if (c->d_gemm_partial) cudaFree(c->d_gemm_partial);
    if (c->d_gemm_ready) cudaFree(c->d_gemm_ready);
    cudaFree(c->d_status);
    if (c->d_timing) cudaFree(c->d_timing);
    cudaStreamDestroy(c->stream);
    c->magic = 0;
    c->mu.unlock();
    delete c;
    return WF_OK;
}

int wf_device_info(int64_t ctx, int* sm_count, int* cc_major, int* cc_minor, int64_t* total_mem, int64_t* free_mem) {
    WF_ENTER(ctx);
    size_t f = 0, t = 0;
    WF_CUDA(c, cudaMemGetInfo(&f, &t));
    if (sm_count) *sm_count = c->sm_count;
    if (cc_major) *cc_major = c->cc_major;
    if (cc_minor) *cc_minor = c->cc_minor;
    if (total_mem) *total_mem = (int64_t)t;
    if (free_mem) *free_mem = (int64_t)f;
    return WF_OK;
}

int wf_stream_create(int64_t ctx, int64_t* stream) {
    WF_ENTER(ctx);
    if (!stream) return WF_ERR_INVALID_ARGUMENT;
    cudaStream_t s;
    WF_CUDA(c, cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    c->streams.push_back(s);
    *stream = reinterpret_cast<int64_t>(s);
    return WF_OK;
}

int wf_stream_destroy(int64_t ctx, int64_t stream) {
    WF_ENTER(ctx);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    auto it = std::find(c->streams.begin(), c->streams.end(), s);
    if (stream == 0 || it == c->streams.end()) return WF_ERR_INVALID_HANDLE;
    WF_CUDA(c, cudaStreamSynchronize(s));
    auto sc = c->gemv_scratch.find(s);
    if (sc != c->gemv_scratch.end()) {
        cudaFree(sc->second.d_slots);
        cudaFree(sc->second.d_part);
        cudaFree(sc->second.d_count);
        c->gemv_scratch.erase(sc);
    }
    c->streams.erase(it);
    WF_CUDA(c, cudaStreamDestroy(s));
    return WF_OK;
}

}  // extern "C"

namespace wf {
int read_device_status(Context* c) {
    int st = 0;
    WF_CUDA(c, cudaMemcpy(&st, c->d_status, sizeof st, cudaMemcpyDeviceToHost));
    if (st != 0) {
        WF_CUDA(c, cudaMemset(c->d_status, 0, sizeof st));
        if (st == STATUS_BAD_INDEX) return set_error(c, WF_ERR_INDEX, "an embedding index was outside the table (its row was written as zeros)");
        return set_error(c, WF_ERR_DEVICE_WAIT, "a device-side bounded wait expired (status bits 0x%x)", st);
    }
    return WF_OK;
}

int refuse_allocation_while_recording(Context* c, cudaStream_t s, const char* what) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
        cudaGetLastError();
        return WF_OK;
    }
    if (st == cudaStreamCaptureStatusNone) return WF_OK;
    return set_error(c, WF_ERR_RECORDING, "%s would be allocated while the stream is being recorded: run the call once before wf_graph_begin", what);
}
}  // namespace wf

extern "C" {

int wf_stream_sync(int64_t ctx, int64_t stream) {
    WF_ENTER(ctx);
    cudaStream_t s = resolve_stream(c, stream);
    WF_CUDA(c, cudaStreamSynchronize(s));
    return read_device_status(c);
}

int wf_malloc(int64_t ctx, int64_t bytes, int64_t* dptr) {
    WF_ENTER(ctx);
    if (!dptr || bytes < 0) return WF_ERR_INVALID_ARGUMENT;
    void* p = nullptr;
    WF_CUDA(c, cudaMalloc(&p, (size_t)std::max<int64_t>(bytes, 1)));
    c->allocs[reinterpret_cast<int64_t>(p)] = bytes;
    *dptr = reinterpret_cast<int64_t>(p);
    return WF_OK;
}

int wf_free(int64_t ctx, int64_t dptr) {
    WF_ENTER(ctx);
    auto it = c->allocs.find(dptr);
    if (it == c->allocs.end()) return WF_ERR_INVALID_HANDLE;
    c->allocs.erase(it);
    WF_CUDA(c, cudaFree(reinterpret_cast<void*>(dptr)));
    return WF_OK;
}

int wf_host_alloc(int64_t ctx, int64_t bytes, void** host) {
    WF_ENTER(ctx);
    if (!host || bytes < 0) return WF_ERR_INVALID_ARGUMENT;
    void* p = nullptr;
    WF_CUDA(c, cudaMallocHost(&p, (size_t)std::max<int64_t>(bytes, 1)));
    c->host_allocs.push_back(p);
    *host = p;
    return WF_OK;
}

int wf_host_free(int64_t ctx, void* host) {
    WF_ENTER(ctx);
    auto it = std::find(c->host_allocs.begin(), c->host_allocs.end(), host);
    if (it == c->host_allocs.end()) return WF_ERR_INVALID_HANDLE;
    c->host_allocs.erase(it);
    WF_CUDA(c, cudaFreeHost(host));
    return WF_OK;
}

int wf_memcpy_h2d(int64_t ctx, int64_t dst, const void* src, int64_t bytes, int64_t stream, int sync) {
    WF_ENTER(ctx);
    if (!dst || !src || bytes < 0) return WF_ERR_INVALID_ARGUMENT;
    cudaStream_t s = resolve_stream(c, stream);
    WF_CUDA(c, cudaMemcpyAsync(reinterpret_cast<void*>(dst), src, (size_t)bytes, cudaMemcpyHostToDevice, s));
    if (sync) WF_CUDA(c, cudaStreamSynchronize(s));
    return WF_OK;
}

int wf_memcpy_d2h(int64_t ctx, void* dst, int64_t src, int64_t bytes, int64_t stream, int sync) {
    WF_ENTER(ctx);
    if (!dst || !src || bytes < 0) return WF_ERR_INVALID_ARGUMENT;
    cudaStream_t s = resolve_stream(c, stream);
    WF_CUDA(c, cudaMemcpyAsync(dst, reinterpret_cast<const void*>(src), (size_t)bytes, cudaMemcpyDeviceToHost, s));
    if (sync) WF_CUDA(c, cudaStreamSynchronize(s));
    return WF_OK;
}

int wf_weight_upload(int64_t ctx, int qtype, const void* blocks, int64_t n_rows, int64_t k, int shard_rank,
                     int shard_world, int64_t* weight) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    return weight_upload(c, qtype, blocks, n_rows, k, shard_rank, shard_world, WF_Q4_0_ORDER_REFERENCE, weight);
}

}  // extern "C"

namespace wf {
int weight_upload(Context* c, int qtype, const void* blocks, int64_t n_rows, int64_t k, int shard_rank, int shard_world,
                  int q4_0_order, int64_t* weight) {
    ScopedLock lock(c);
    if (!lock.ok) return WF_ERR_BUSY;
    WF_CUDA(c, cudaSetDevice(c->device));
    if (!blocks || !weight) return set_error(c, WF_ERR_INVALID_ARGUMENT, "null pointer");
    *weight = 0;
    if (!qtype_supported(qtype))
        return set_error(c, WF_ERR_UNSUPPORTED_TYPE, "Quantized matmul not implemented for ggml type %d", qtype);
    if (n_rows <= 0 || k <= 0 || k % block_k(qtype) != 0 || k > (1 << 24) || n_rows > (1LL << 31) - 16)
        return set_error(c, WF_ERR_SHAPE, "bad shape rows=%lld k=%lld (k must be a positive multiple of %d)",
                         (long long)n_rows, (long long)k, block_k(qtype));
    if (shard_world < 1 || shard_rank < 0 || shard_rank >= shard_world)
        return set_error(c, WF_ERR_SHARD, "shard rank %d outside world %d", shard_rank, shard_world);
    if (n_rows % shard_world != 0)
        return set_error(c, WF_ERR_SHARD, "rows=%lld not divisible by world %d", (long long)n_rows, shard_world);

    const int64_t rows = n_rows / shard_world, row0 = rows * shard_rank;
    const int64_t row_bytes = k / block_k(qtype) * block_bytes(qtype);
    Weight* w = new Weight();
    w->ctx = c;
    w->g.qtype = device_qtype(qtype);  // the kernels see the device format; `qtype` is the file's
    w->file_qtype = qtype;
    w->g.rows = rows;
    w->g.k = k;
    w->g.rt = (rows + TILE_ROWS - 1) / TILE_ROWS;
    w->g.kt = (k + tile_k(w->g.qtype) - 1) / tile_k(w->g.qtype);
    w->g.rt_alloc = (w->g.rt + 7) / 8 * 8;
    w->row0 = row0;
    w->total_rows = n_rows;
    cudaError_t e = cudaMalloc(&w->d_tiles, (size_t)w->g.bytes());
    if (e == cudaSuccess) e = cudaMemsetAsync(w->d_tiles, 0, (size_t)w->g.bytes(), c->stream);
    if (e == cudaSuccess)
        e = upload_and_repack(c, qtype, static_cast<const uint8_t*>(blocks) + row0 * row_bytes, rows, k, row_bytes, w->d_tiles,
                              w->g.kt * (int64_t)tile_bytes(w->g.qtype), q4_0_order, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        if (w->d_tiles) cudaFree(w->d_tiles);
        delete w;
        return cuda_status(c, e, "weight upload");
    }
    c->launches++;
    c->weights.push_back(w);
    *weight = reinterpret_cast<int64_t>(w);
    return WF_OK;
}
}  // namespace wf

extern "C" {

int wf_weight_free(int64_t ctx, int64_t weight) {
    WF_ENTER(ctx);
    Weight* w = get_weight(c, weight);
    if (!w) return WF_ERR_INVALID_HANDLE;
    if (w->programs > 0)
        return set_error(c, WF_ERR_IN_USE, "weight is referenced by %d live program(s): destroy them first", w->programs);
    c->weights.erase(std::find(c->weights.begin(), c->weights.end(), w));
    WF_CUDA(c, cudaStreamSynchronize(c->stream));
    cudaFree(w->d_tiles);
    w->magic = 0;
    delete w;
    return WF_OK;
}

int wf_weight_info(int64_t ctx, int64_t weight, int* qtype, int64_t* rows, int64_t* k, int64_t* row0,
                   int64_t* device_bytes) {
    WF_ENTER(ctx);
    Weight* w = get_weight(c, weight);
    if (!w) return WF_ERR_INVALID_HANDLE;
    if (qtype) *qtype = w->file_qtype;
    if (rows) *rows = w->g.rows;
    if (k) *k = w->g.k;
    if (row0) *row0 = w->row0;
    if (device_bytes) *device_bytes = w->g.bytes();
    return WF_OK;
}

int wf_dequant_rows(int64_t ctx, int64_t weight, int64_t row0, int64_t nrows, float* out_host) {
    WF_ENTER(ctx);
    Weight* w = get_weight(c, weight);
    if (!w) return WF_ERR_INVALID_HANDLE;
    if (!out_host && nrows > 0) return WF_ERR_INVALID_ARGUMENT;
    if (row0 < 0 || nrows < 0 || row0 + nrows > w->g.rows)
        return set_error(c, WF_ERR_SHAPE, "rows [%lld, %lld) outside shard of %lld rows", (long long)row0,
                         (long long)(row0 + nrows), (long long)w->g.rows);
    if (nrows == 0) return WF_OK;
    const int64_t bytes = nrows * w->g.k * (int64_t)sizeof(float);
    float* d_out = nullptr;
    WF_CUDA(c, cudaMalloc(&d_out, (size_t)bytes));
    cudaError_t e = launch_dequant_rows(*w, row0, nrows, d_out, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(out_host, d_out, (size_t)bytes, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(d_out);
    if (e != cudaSuccess) return cuda_status(c, e, "dequant rows");
    c->launches++;
    return read_device_status(c);
}

int wf_qlinear(int64_t ctx, int64_t weight, const void* x, int x_dtype, int x_on_device, int64_t m, void* y,
               int y_on_device, int64_t stream) {
    WF_ENTER(ctx);
    Weight* w = get_weight(c, weight);
    if (!w) return WF_ERR_INVALID_HANDLE;
    if (x_dtype != WF_DTYPE_BF16 && x_dtype != WF_DTYPE_F32)
        return set_error(c, WF_ERR_INVALID_ARGUMENT, "x_dtype %d is neither BF16 nor F32", x_dtype);
    if (m < 0 || m > (1 << 20)) return set_error(c, WF_ERR_SHAPE, "m=%lld out of range", (long long)m);
    if (m == 0) return WF_OK;
    if (!x || !y) return set_error(c, WF_ERR_INVALID_ARGUMENT, "null pointer");
    // the kernels read activations in 16-byte pieces and write fp32: reject pointers they would fault on
    if (x_on_device && (reinterpret_cast<uintptr_t>(x) & 15))
        return set_error(c, WF_ERR_INVALID_ARGUMENT, "device activation pointer must be 16-byte aligned");
    if (y_on_device && (reinterpret_cast<uintptr_t>(y) & 3))
        return set_error(c, WF_ERR_INVALID_ARGUMENT, "device output pointer must be 4-byte aligned");
    cudaStream_t s = resolve_stream(c, stream);
    const int64_t xb = m * w->g.k * (x_dtype == WF_DTYPE_F32 ? 4 : 2), yb = m * w->g.rows * 4;
    const void* d_x = x;
    float* d_y = static_cast<float*>(y);
    if (!x_on_device || !y_on_device) {
        // host operands: pinned staging, copies on the same stream, result waited for
        const int64_t xo = 0, yo = (xb + 255) & ~255LL;
        int rc = ensure_stage(c, yo + yb, yo + yb);
        if (rc != WF_OK) return rc;
        if (!x_on_device) {
            memcpy(static_cast<uint8_t*>(c->h_stage) + xo, x, (size_t)xb);
            WF_CUDA(c, cudaMemcpyAsync(static_cast<uint8_t*>(c->d_stage) + xo, static_cast<uint8_t*>(c->h_stage) + xo,
                                       (size_t)xb, cudaMemcpyHostToDevice, s));
            d_x = static_cast<uint8_t*>(c->d_stage) + xo;
        }
        if (!y_on_device) d_y = reinterpret_cast<float*>(static_cast<uint8_t*>(c->d_stage) + yo);
    }
    GemvCall call{w, d_x, x_dtype, m, d_y, w->g.rows, 0};
    // many tokens: tensor-core GEMM; a few tokens: the HBM-bound GEMV
    int rc = gemm_supported(*w, x_dtype, m, call.d_x) ? gemm_launch(c, call, s) : gemv_launch(c, call, s);
    if (rc != WF_OK) return rc;
    if (!y_on_device) {
        const int64_t yo = (xb + 255) & ~255LL;
        WF_CUDA(c, cudaMemcpyAsync(static_cast<uint8_t*>(c->h_stage) + yo, d_y, (size_t)yb, cudaMemcpyDeviceToHost, s));
        WF_CUDA(c, cudaStreamSynchronize(s));
        memcpy(y, static_cast<uint8_t*>(c->h_stage) + yo, (size_t)yb);
        return read_device_status(c);  // the result is in the caller's hands: a wait that ran out must not pass as success
    } else if (!x_on_device) {
        WF_CUDA(c, cudaStreamSynchronize(s));  // the staging buffer is reused by the next call
        return read_device_status(c);
    }
    return WF_OK;
}

int wf_qlinear_noalloc(int64_t ctx, int64_t weight, int64_t x_dev, int x_dtype, int64_t m, int64_t y_dev, int64_t stream) {
    WF_ENTER(ctx);
    Weight* w = get_weight(c, weight);
    if (!w) return WF_ERR_INVALID_HANDLE;
    if (x_dtype != WF_DTYPE_BF16 && x_dtype != WF_DTYPE_F32)
        return set_error(c, WF_ERR_INVALID_ARGUMENT, "x_dtype %d is neither BF16 nor F32", x_dtype);
    if (m < 0 || m > (1 << 20)) return set_error(c, WF_ERR_SHAPE, "m=%lld out of range", (long long)m);
    if (m == 0) return WF_OK;
    if (!x_dev || !y_dev) return set_error(c, WF_ERR_INVALID_ARGUMENT, "null device pointer");
    if ((x_dev & 15) || (y_dev & 3))
        return set_error(c, WF_ERR_INVALID_ARGUMENT, "device pointers must be aligned (activations 16 bytes, output 4 bytes)");
    GemvCall call{w, reinterpret_cast<const void*>(x_dev), x_dtype, m, reinterpret_cast<float*>(y_dev), w->g.rows, 0};
    return gemv_launch_noalloc(c, call, resolve_stream(c, stream));
}

int wf_graph_begin(int64_t ctx, int64_t stream) {
    WF_ENTER(ctx);
    cudaStream_t s = resolve_stream(c, stream);
    int rc = gemv_prepare_stream(c, s);  // no allocation may happen while recording
    if (rc != WF_OK) return rc;
    c->capture_launches = c->launches;
    WF_CUDA(c, cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    return WF_OK;
}

int wf_graph_end(int64_t ctx, int64_t stream, int64_t* graph) {
    WF_ENTER(ctx);
    if (!graph) return WF_ERR_INVALID_ARGUMENT;
    *graph = 0;
    cudaGraph_t g = nullptr;
    WF_CUDA(c, cudaStreamEndCapture(resolve_stream(c, stream), &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_status(c, e, "cudaGraphInstantiate");
    c->graphs.push_back(exec);
    c->graph_launches[exec] = c->launches - c->capture_launches;
    c->launches = c->capture_launches;  // recorded, not yet run
    *graph = reinterpret_cast<int64_t>(exec);
    return WF_OK;
}

int wf_graph_launch(int64_t ctx, int64_t graph, int64_t stream) {
    WF_ENTER(ctx);
    cudaGraphExec_t exec = reinterpret_cast<cudaGraphExec_t>(graph);
    if (std::find(c->graphs.begin(), c->graphs.end(), exec) == c->graphs.end()) return WF_ERR_INVALID_HANDLE;
    WF_CUDA(c, cudaGraphLaunch(exec, resolve_stream(c, stream)));
    c->launches += c->graph_launches[exec];
    return WF_OK;
}

int wf_graph_destroy(int64_t ctx, int64_t graph) {
    WF_ENTER(ctx);
    cudaGraphExec_t exec = reinterpret_cast<cudaGraphExec_t>(graph);
    auto it = std::find(c->graphs.begin(), c->graphs.end(), exec);
    if (it == c->graphs.end()) return WF_ERR_INVALID_HANDLE;
    c->graphs.erase(it);
    c->graph_launches.erase(exec);
    WF_CUDA(c, cudaGraphExecDestroy(exec));
    return WF_OK;
}

const char* wf_error_string(int status) {
    switch (status) {
        case WF_OK: return "WF_OK";
        case WF_ERR_INVALID_ARGUMENT: return "WF_ERR_INVALID_ARGUMENT";
        case WF_ERR_INVALID_HANDLE: return "WF_ERR_INVALID_HANDLE";
        case WF_ERR_UNSUPPORTED_TYPE: return "WF_ERR_UNSUPPORTED_TYPE";
        case WF_ERR_SHAPE: return "WF_ERR_SHAPE";
        case WF_ERR_SHARD: return "WF_ERR_SHARD";
        case WF_ERR_BUSY: return "WF_ERR_BUSY";
        case WF_ERR_NO_DEVICE: return "WF_ERR_NO_DEVICE";
        case WF_ERR_NOT_SM100: return "WF_ERR_NOT_SM100";
        case WF_ERR_NCCL_UNAVAILABLE: return "WF_ERR_NCCL_UNAVAILABLE";
        case WF_ERR_DEVICE_WAIT: return "WF_ERR_DEVICE_WAIT";
        case WF_ERR_TOO_LARGE: return "WF_ERR_TOO_LARGE";
        case WF_ERR_GGUF: return "WF_ERR_GGUF";
        case WF_ERR_INDEX: return "WF_ERR_INDEX";
        case WF_ERR_RECORDING: return "WF_ERR_RECORDING";
        case WF_ERR_IN_USE: return "WF_ERR_IN_USE";
        default: break;
    }
    if (status >= WF_ERR_NCCL_BASE) return "WF_ERR_NCCL";
    if (status >= WF_ERR_CUDA_BASE) return cudaGetErrorName((cudaError_t)(status - WF_ERR_CUDA_BASE));
    return "WF_ERR_UNKNOWN";
}

int wf_last_error(int64_t ctx, char* buf, int64_t buf_len) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    if (!buf || buf_len <= 0) return WF_ERR_INVALID_ARGUMENT;
    snprintf(buf, (size_t)buf_len, "%s", c->last_error.c_str());
    return WF_OK;
}

int wf_event_create(int64_t ctx, int64_t* event) {
    WF_ENTER(ctx);
    if (!event) return WF_ERR_INVALID_ARGUMENT;
    cudaEvent_t ev;
    WF_CUDA(c, cudaEventCreate(&ev));
    c->events.push_back(ev);
    *event = reinterpret_cast<int64_t>(ev);
    return WF_OK;
}

int wf_event_destroy(int64_t ctx, int64_t event) {
    WF_ENTER(ctx);
    cudaEvent_t ev = reinterpret_cast<cudaEvent_t>(event);
    auto it = std::find(c->events.begin(), c->events.end(), ev);
    if (it == c->events.end()) return WF_ERR_INVALID_HANDLE;
    c->events.erase(it);
    WF_CUDA(c, cudaEventDestroy(ev));
    return WF_OK;
}

int wf_event_record(int64_t ctx, int64_t event, int64_t stream) {
    WF_ENTER(ctx);
    cudaEvent_t ev = reinterpret_cast<cudaEvent_t>(event);
    if (std::find(c->events.begin(), c->events.end(), ev) == c->events.end()) return WF_ERR_INVALID_HANDLE;
    WF_CUDA(c, cudaEventRecord(ev, resolve_stream(c, stream)));
    return WF_OK;
}

int wf_event_elapsed_ms(int64_t ctx, int64_t start, int64_t stop, float* ms) {
    WF_ENTER(ctx);
    if (!ms) return WF_ERR_INVALID_ARGUMENT;
    cudaEvent_t a = reinterpret_cast<cudaEvent_t>(start), b = reinterpret_cast<cudaEvent_t>(stop);
    if (std::find(c->events.begin(), c->events.end(), a) == c->events.end() ||
        std::find(c->events.begin(), c->events.end(), b) == c->events.end())
        return WF_ERR_INVALID_HANDLE;
    WF_CUDA(c, cudaEventSynchronize(b));
    WF_CUDA(c, cudaEventElapsedTime(ms, a, b));
    return WF_OK;
}

int wf_set_salt(int64_t ctx, int salt) {
    WF_ENTER(ctx);
    if (salt < 0 || salt > 2) return WF_ERR_INVALID_ARGUMENT;
    if (salt >= 2 && !c->d_timing) {
        WF_CUDA(c, cudaMalloc(&c->d_timing, (size_t)c->sm_count * 8 * sizeof(unsigned long long)));
        WF_CUDA(c, cudaMemset(c->d_timing, 0, (size_t)c->sm_count * 8 * sizeof(unsigned long long)));
    }
    c->salt = salt;
    return WF_OK;
}

int wf_read_timing(int64_t ctx, int64_t* out, int64_t n) {
    WF_ENTER(ctx);
    if (!out || n < 0) return WF_ERR_INVALID_ARGUMENT;
    if (!c->d_timing) return set_error(c, WF_ERR_INVALID_ARGUMENT, "timing stamps are off (wf_set_salt(ctx, 2) first)");
    const int64_t have = (int64_t)c->sm_count * 8;
    WF_CUDA(c, cudaDeviceSynchronize());
    WF_CUDA(c, cudaMemcpy(out, c->d_timing, (size_t)std::min(n, have) * sizeof(int64_t), cudaMemcpyDeviceToHost));
    return WF_OK;
}

int wf_launch_count(int64_t ctx, int64_t* launches) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    if (!launches) return WF_ERR_INVALID_ARGUMENT;
    *launches = c->launches;
    return WF_OK;
}

}  // extern "C"
