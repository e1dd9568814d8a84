// Row-sharded tensor parallelism: the all-gather behind a sharded qlinear.
// Keeps the semantics of CollectiveApi.allGather(input, output)
// (warpforge-io/src/main/java/io/surfworks/warpforge/io/collective/CollectiveApi.java:137-146;
// UCC implementation .../collective/impl/UccCollectiveImpl.java:503-543): rank r's chunk lands
// at offset r * chunk on every rank -- but on device buffers over NCCL / NVLink instead of
// host buffers over UCC / RoCE.  libnccl is resolved at run time with dlopen, the way the
// reference resolves libucc (io/collective/Collective.java:45-71), so the library loads on
// machines without NCCL and reports WF_ERR_NCCL_UNAVAILABLE only when a communicator is asked for.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "wf_common.cuh"

namespace wf {

struct NcclId { char internal[128]; };
typedef void* NcclComm;
enum { NCCL_SUCCESS = 0, NCCL_INT8 = 0, NCCL_FLOAT32 = 7 };

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

static NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {getenv("WF_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            if (!n || !*n) continue;
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) return;
#define WF_SYM(field, name) *reinterpret_cast<void**>(&api.field) = dlsym(api.handle, name)
        WF_SYM(GetUniqueId, "ncclGetUniqueId");
        WF_SYM(CommInitRank, "ncclCommInitRank");
        WF_SYM(CommDestroy, "ncclCommDestroy");
        WF_SYM(AllGather, "ncclAllGather");
        WF_SYM(GroupStart, "ncclGroupStart");
        WF_SYM(GroupEnd, "ncclGroupEnd");
        WF_SYM(GetErrorString, "ncclGetErrorString");
#undef WF_SYM
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.GroupStart && api.GroupEnd;
    });
    return api;
}

struct Comm {
    uint32_t magic = COMM_MAGIC;
    Context* ctx = nullptr;
    NcclComm comm = nullptr;
    int rank = 0, world = 1;
    float* d_tmp = nullptr;  // [world][m][rows] staging for multi-token gathers
    int64_t tmp_bytes = 0;
};

static std::mutex g_comm_mu;
static std::vector<Comm*> g_comms;

static Comm* get_comm(Context* c, int64_t h) {
    Comm* k = reinterpret_cast<Comm*>(h);
    std::lock_guard<std::mutex> lk(g_comm_mu);
    if (!k || std::find(g_comms.begin(), g_comms.end(), k) == g_comms.end() || k->magic != COMM_MAGIC || k->ctx != c)
        return nullptr;
    return k;
}

static int nccl_status(Context* c, int r, const char* what) {
    NcclApi& a = nccl();
    return set_error(c, WF_ERR_NCCL_BASE + r, "%s failed: %s (%d)", what, a.GetErrorString ? a.GetErrorString(r) : "nccl", r);
}

// [world][m][rows] -> [m][world*rows]: one strip of `rows` floats per (rank, token), copied by the CTAs of grid row
// blockIdx.y = rank * m + token (grid-stride over y for very many tokens); 16-byte pieces when the strips allow it.
__global__ void __launch_bounds__(256) unshard_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t m, int64_t rows,
                                                      int world, int vec) {
    const int64_t n = (int64_t)world * rows, strips = (int64_t)world * m;
    for (int64_t sidx = blockIdx.y; sidx < strips; sidx += gridDim.y) {
        const int64_t r = sidx / m, t = sidx - r * m;  // one division per strip, not per element
        const float* s = src + sidx * rows;
        float* d = dst + t * n + r * rows;
        if (vec) {
            for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (rows >> 2); i += (int64_t)gridDim.x * blockDim.x)
                reinterpret_cast<float4*>(d)[i] = __ldcs(reinterpret_cast<const float4*>(s) + i);
        } else {
            for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += (int64_t)gridDim.x * blockDim.x) d[i] = s[i];
        }
    }
}

}  // namespace wf

using namespace wf;

extern "C" {

int wf_comm_get_unique_id(void* id128) {
    if (!id128) return WF_ERR_INVALID_ARGUMENT;
    NcclApi& a = nccl();
    if (!a.ok) return WF_ERR_NCCL_UNAVAILABLE;
    NcclId id;
    int r = a.GetUniqueId(&id);
    if (r != NCCL_SUCCESS) return WF_ERR_NCCL_BASE + r;
    memcpy(id128, &id, sizeof id);
    return WF_OK;
}

int wf_comm_init(int64_t ctx, const void* id128, int rank, int world, int64_t* comm) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    if (!id128 || !comm) return set_error(c, WF_ERR_INVALID_ARGUMENT, "null pointer");
    *comm = 0;
    if (world < 1 || rank < 0 || rank >= world) return set_error(c, WF_ERR_SHARD, "rank %d outside world %d", rank, world);
    NcclApi& a = nccl();
    if (!a.ok) return set_error(c, WF_ERR_NCCL_UNAVAILABLE, "libnccl.so.2 could not be loaded");
    WF_CUDA(c, cudaSetDevice(c->device));
    NcclId id;
    memcpy(&id, id128, sizeof id);
    Comm* k = new Comm();
    k->ctx = c;
    k->rank = rank;
    k->world = world;
    int r = a.CommInitRank(&k->comm, world, id, rank);
    if (r != NCCL_SUCCESS) {
        delete k;
        return nccl_status(c, r, "ncclCommInitRank");
    }
    {
        std::lock_guard<std::mutex> g(g_comm_mu);
        g_comms.push_back(k);
    }
    *comm = reinterpret_cast<int64_t>(k);
    return WF_OK;
}

int wf_comm_destroy(int64_t ctx, int64_t comm) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    Comm* k = get_comm(c, comm);
    if (!k) return WF_ERR_INVALID_HANDLE;
    {
        std::lock_guard<std::mutex> g(g_comm_mu);
        g_comms.erase(std::find(g_comms.begin(), g_comms.end(), k));
    }
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    nccl().CommDestroy(k->comm);
    if (k->d_tmp) cudaFree(k->d_tmp);
    k->magic = 0;
    delete k;
    return WF_OK;
}

int wf_allgather(int64_t ctx, int64_t comm, int64_t send_dev, int64_t recv_dev, int64_t bytes_per_rank, int64_t stream) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    Comm* k = get_comm(c, comm);
    if (!k) return WF_ERR_INVALID_HANDLE;
    if (!send_dev || !recv_dev || bytes_per_rank < 0) return set_error(c, WF_ERR_INVALID_ARGUMENT, "bad all-gather arguments");
    if (bytes_per_rank == 0) return WF_OK;
    WF_CUDA(c, cudaSetDevice(c->device));
    int r = nccl().AllGather(reinterpret_cast<const void*>(send_dev), reinterpret_cast<void*>(recv_dev),
                             (size_t)bytes_per_rank, NCCL_INT8, k->comm, resolve_stream(c, stream));
    if (r != NCCL_SUCCESS) return nccl_status(c, r, "ncclAllGather");
    return WF_OK;
}

int wf_qlinear_allgather(int64_t ctx, int64_t comm, int64_t weight, const void* x_dev, int x_dtype, int64_t m,
                         void* y_full_dev, int64_t stream) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    Comm* k = get_comm(c, comm);
    Weight* w = get_weight(c, weight);
    if (!k || !w) return WF_ERR_INVALID_HANDLE;
    if (x_dtype != WF_DTYPE_BF16 && x_dtype != WF_DTYPE_F32) return set_error(c, WF_ERR_INVALID_ARGUMENT, "bad x_dtype %d", x_dtype);
    if (m < 0 || m > (1 << 20)) return set_error(c, WF_ERR_SHAPE, "m=%lld out of range", (long long)m);
    if (m == 0) return WF_OK;
    if (!x_dev || !y_full_dev) return set_error(c, WF_ERR_INVALID_ARGUMENT, "null pointer");
    if ((reinterpret_cast<uintptr_t>(x_dev) & 15) || (reinterpret_cast<uintptr_t>(y_full_dev) & 3))
        return set_error(c, WF_ERR_INVALID_ARGUMENT, "device pointers must be aligned (activations 16 bytes, output 4 bytes)");
    if (w->total_rows != w->g.rows * k->world || w->row0 != w->g.rows * k->rank)
        return set_error(c, WF_ERR_SHARD, "weight shard (row0=%lld rows=%lld of %lld) does not match rank %d of %d",
                         (long long)w->row0, (long long)w->g.rows, (long long)w->total_rows, k->rank, k->world);
    WF_CUDA(c, cudaSetDevice(c->device));
    cudaStream_t s = resolve_stream(c, stream);
    const int64_t rows = w->g.rows, n = w->total_rows;
    float* y = static_cast<float*>(y_full_dev);
    if (m == 1) {
        // one token: the rank-major gather IS the full output row; compute in place
        GemvCall call{w, x_dev, x_dtype, 1, y, n, w->row0};
        int rc = gemv_launch(c, call, s);
        if (rc != WF_OK) return rc;
        if (k->world > 1) {
            int r = nccl().AllGather(y + w->row0, y, (size_t)rows, NCCL_FLOAT32, k->comm, s);
            if (r != NCCL_SUCCESS) return nccl_status(c, r, "ncclAllGather");
        }
        return WF_OK;
    }
    const int64_t need = (int64_t)k->world * m * rows * 4 + m * rows * 4;
    if (need > k->tmp_bytes) {
        const int rc = refuse_allocation_while_recording(c, s, "the gather buffer");
        if (rc != WF_OK) return rc;
        if (k->d_tmp) cudaFree(k->d_tmp);
        k->d_tmp = nullptr;
        k->tmp_bytes = 0;
        WF_CUDA(c, cudaMalloc(&k->d_tmp, (size_t)need));
        k->tmp_bytes = need;
    }
    float* mine = k->d_tmp + (int64_t)k->world * m * rows;
    GemvCall call{w, x_dev, x_dtype, m, mine, rows, 0};
    int rc = gemm_supported(*w, x_dtype, m, call.d_x) ? gemm_launch(c, call, s) : gemv_launch(c, call, s);
    if (rc != WF_OK) return rc;
    int r = nccl().AllGather(mine, k->d_tmp, (size_t)(m * rows), NCCL_FLOAT32, k->comm, s);
    if (r != NCCL_SUCCESS) return nccl_status(c, r, "ncclAllGather");
    const int vec = (rows % 4 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0);
    const dim3 grid((unsigned)std::max<int64_t>(1, std::min<int64_t>((rows / (vec ? 4 : 1) + 255) / 256, 8)),
                    (unsigned)std::min<int64_t>((int64_t)k->world * m, 65535));
    unshard_kernel<<<grid, 256, 0, s>>>(k->d_tmp, y, m, rows, k->world, vec);
    WF_CUDA(c, cudaGetLastError());
    c->launches++;
    return WF_OK;
}

}  // extern "C"
