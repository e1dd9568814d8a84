// Row-sharded tensor parallelism: the all-gather behind a sharded qlinear.
// Keeps the semantics of CollectiveApi.allGather(input, output)
// (warpforge-io/src/main/java/io/surfworks/warpforge/io/collective/CollectiveApi.java:137-146;
// UCC implementation .../collective/impl/UccCollectiveImpl.java:503-543): rank r's chunk lands
// at offset r * chunk on every rank -- but on device buffers over NCCL / NVLink instead of
// host buffers over UCC / RoCE.  libnccl is resolved at run time with dlopen, the way the
// reference resolves libucc (io/collective/Collective.java:45-71), so the library loads on
// machines without NCCL and reports WF_ERR_NCCL_UNAVAILABLE only when a communicator is asked for.
// NCCL carries the bootstrap and the plain wf_allgather.  The gather behind wf_qlinear_allgather goes, between
// the GPUs of one node, by this file's own kernels over peer-mapped memory (plain stores and loads, bulk copies
// without multicast): gather_small_kernel for the decode kernels' outputs, gather_bulk_kernel /
// gather_large_kernel for the tensor-core kernel's; NCCL + unshard_kernel is the fallback.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "wf_common.cuh"
#include "wf_gemv_core.cuh"

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

constexpr int WF_MAX_GATHER_RANKS = 8;  // one node

struct Comm {
    uint32_t magic = COMM_MAGIC;
    Context* ctx = nullptr;
    NcclComm comm = nullptr;
    int rank = 0, world = 1;
    float* d_tmp = nullptr;  // NCCL route: [world][m][rows] gathered rank-major, then this rank's [m][rows]
    int64_t tmp_bytes = 0;
    // Gathers by this file's own kernels: every rank owns one block (landing buffer, flags, staging area) that
    // the other ranks of the node map through IPC.  land[r] is rank r's block (land[rank] the own one); all null
    // when the mappings could not be made on every rank, and the NCCL path is then the only one.
    uint2* land[WF_MAX_GATHER_RANKS] = {};
    unsigned int* d_epoch = nullptr;  // [0] small gathers done so far, [1] CTAs that finished the current one; [2], [3] the same for large ones
    int64_t stage_bytes = 0;          // size of the staging area behind the landing buffer and the flags
    bool peer_ok = false;
    bool bulk = true;  // large gathers by bulk copies through shared memory (WF_GATHER=registers: by loads into registers)
    unsigned long long wait_ns = 5000000000ull;
};

// One allocation per rank, mapped by every peer: the landing buffer of the small gathers (two halves for even /
// odd gathers, each [world][m * rows] tagged words), one page of flags, and the staging area of the large gathers.
constexpr int64_t GATHER_LAND_BYTES = 32ll << 20;
constexpr int64_t GATHER_FLAG_BYTES = 4096;  // unsigned ready[8] at 0, done[8] at 2048
constexpr int64_t GATHER_STAGE_DEFAULT = 128ll << 20;

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

struct GatherPeers {
    uint2* land[WF_MAX_GATHER_RANKS];
};

// All-gather of a small row-sharded output without a library call: y is [m][world * rows] on every rank and
// this rank's kernel has just written its own column block [rank * rows, (rank + 1) * rows).  Every element
// travels as one 8-byte word {value, tag} stored straight into each peer's landing buffer; the tag is the
// number of this gather (counted on the device, so that a replayed graph keeps counting), and a word is
// valid for its reader the moment it carries the tag -- no fence, no flag, one NVLink crossing.  Each rank
// then polls its own landing buffer and writes the peers' values into y.  Gathers alternate between the two
// halves of the landing buffer: a rank can push gather g + 2 only after it finished g + 1, which needed
// every peer's push of g + 1, which every peer issues after it finished reading g -- so a half is never
// overwritten while someone still reads it.  The waits end after `wait_ns` and set a status bit.
// Every rank runs exactly one such kernel per gather; nothing on one GPU waits for another launch of that GPU.
// At most one CTA per SM, so that all CTAs of the grid are resident: a CTA that had not started yet would not
// have pushed, and the peers' CTAs waiting for its words could keep its own peers from ever starting.
constexpr int GATHER_THREADS = 1024, GATHER_BATCH = 4;

__global__ void __launch_bounds__(GATHER_THREADS) gather_small_kernel(float* __restrict__ y, GatherPeers peers, unsigned int* epoch, int* status,
                                                                      int m, int rows, int world, int rank, int64_t half_words,
                                                                      unsigned long long wait_ns) {
    const unsigned int e = *reinterpret_cast<volatile unsigned int*>(epoch);
    const unsigned int tag = e + 1u ? e + 1u : 1u;
    const int64_t n = (int64_t)world * rows;
    const int total = m * rows;
    const int64_t half = (int64_t)(e & 1u) * half_words;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
    // push: my block of y to every peer.  A thread has GATHER_BATCH loads in flight before its first store:
    // with one, every round of the loop would cost a trip to L2.
    for (int base = tid; base < total; base += nthreads * GATHER_BATCH) {
        float v[GATHER_BATCH];
#pragma unroll
        for (int u = 0; u < GATHER_BATCH; u++) {
            const int i = base + u * nthreads;
            if (i < total) {
                const int t = i / rows, j = i - t * rows;
                v[u] = y[t * n + (int64_t)rank * rows + j];
            }
        }
#pragma unroll
        for (int u = 0; u < GATHER_BATCH; u++) {
            const int i = base + u * nthreads;
            if (i < total) {
                const unsigned long long word = ((unsigned long long)tag << 32) | __float_as_uint(v[u]);
                const int64_t at = half + (int64_t)rank * total + i;
                for (int d = 1; d < world; d++) {
                    const int r = rank + d < world ? rank + d : rank + d - world;  // spread the first stores over the links
                    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(peers.land[r] + at), "l"(word) : "memory");
                }
            }
        }
    }
    // pull: the peers' blocks out of my landing buffer, GATHER_BATCH words polled at a time
    const uint2* mine = peers.land[rank] + half;
    unsigned long long t0 = 0;
    bool gave_up = false;
    const int others = (world - 1) * total;
    for (int base = tid; base < others && !gave_up; base += nthreads * GATHER_BATCH) {
        const uint2* p[GATHER_BATCH];
        float* out[GATHER_BATCH];
        unsigned long long w[GATHER_BATCH];
#pragma unroll
        for (int u = 0; u < GATHER_BATCH; u++) {
            const int q = base + u * nthreads;
            p[u] = nullptr;
            if (q < others) {
                int r = q / total;
                const int i = q - r * total;
                r += r >= rank;
                const int t = i / rows, j = i - t * rows;
                p[u] = mine + (int64_t)r * total + i;
                out[u] = y + t * n + (int64_t)r * rows + j;
            }
        }
        for (;;) {
            bool all = true;
#pragma unroll
            for (int u = 0; u < GATHER_BATCH; u++)
                if (p[u]) asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w[u]) : "l"(p[u]) : "memory");
#pragma unroll
            for (int u = 0; u < GATHER_BATCH; u++) {
                if (p[u] && (unsigned int)(w[u] >> 32) == tag) {
                    *out[u] = __uint_as_float((unsigned int)w[u]);
                    p[u] = nullptr;
                }
                all = all && !p[u];
            }
            if (all) break;
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (!t0) t0 = now;
            if (now - t0 > wait_ns || (*reinterpret_cast<volatile int*>(status) & STATUS_PEER_WAIT_TIMEOUT)) {
                gave_up = true;
                break;
            }
            __nanosleep(40);
        }
        if (gave_up) atomicOr(status, STATUS_PEER_WAIT_TIMEOUT);
    }
    // the last CTA out counts the gather
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(epoch + 1, 1u) == gridDim.x - 1) {
            epoch[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(epoch) = e + 1u;
        }
    }
}

__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int* gather_flags(uint2* base, int which) {
    return reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(base) + GATHER_LAND_BYTES) + which * 512;
}
__device__ __forceinline__ float* gather_stage(uint2* base) {
    return reinterpret_cast<float*>(reinterpret_cast<char*>(base) + GATHER_LAND_BYTES + GATHER_FLAG_BYTES);
}

// Large gathers (the prefill): every rank's kernel writes its [m][rows] block into its OWN staging area, the
// ranks tell each other "ready", and each rank reads the peers' blocks over NVLink straight into the
// token-major rows of its y -- one crossing, no rank-major intermediate and no second pass over HBM.
// Before a rank overwrites its staging area for the next gather, every peer must have finished reading the
// previous one: each rank's last CTA tells the peers "done", and this kernel, launched before the producer of
// the next block, waits for those flags.  It waits for kernels of other GPUs only.
__global__ void gather_wait_done_kernel(GatherPeers peers, const unsigned int* epoch, int* status, int world, int rank,
                                        unsigned long long wait_ns) {
    const unsigned int e = *reinterpret_cast<const volatile unsigned int*>(epoch + 2);
    const int r = threadIdx.x;
    if (e == 0 || r >= world || r == rank) return;
    const unsigned int* done = gather_flags(peers.land[rank], 1) + r;
    unsigned long long t0 = 0;
    while ((int)(ld_acquire_sys_u32(done) - e) < 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (!t0) t0 = now;
        if (now - t0 > wait_ns || (*reinterpret_cast<volatile int*>(status) & STATUS_PEER_WAIT_TIMEOUT)) {
            atomicOr(status, STATUS_PEER_WAIT_TIMEOUT);
            return;
        }
        __nanosleep(100);
    }
}

__global__ void __launch_bounds__(GATHER_THREADS) gather_large_kernel(float* __restrict__ y, GatherPeers peers, unsigned int* epoch, int* status,
                                                                      int64_t m, int rows, int world, int rank, int vec,
                                                                      unsigned long long wait_ns) {
    __shared__ int failed;
    const unsigned int e = *reinterpret_cast<volatile unsigned int*>(epoch + 2);
    const unsigned int tag = e + 1u;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    // my block is complete (the kernel that wrote it ended before this one started): tell the peers
    if (blockIdx.x == 0 && (int)threadIdx.x < world && (int)threadIdx.x != rank) {
        __threadfence_system();
        st_release_sys_u32(gather_flags(peers.land[threadIdx.x], 0) + rank, tag);
    }
    if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
        const unsigned int* ready = gather_flags(peers.land[rank], 0) + threadIdx.x;
        unsigned long long t0 = 0;
        while ((int)(ld_acquire_sys_u32(ready) - tag) < 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (!t0) t0 = now;
            if (now - t0 > wait_ns || (*reinterpret_cast<volatile int*>(status) & STATUS_PEER_WAIT_TIMEOUT)) {
                failed = 1;
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (failed) {
        if (threadIdx.x == 0) atomicOr(status, STATUS_PEER_WAIT_TIMEOUT);
    } else {
        // strips of `rows` floats: strip c belongs to token c / world and to the rank (c % world + rank) % world, so
        // that the CTAs of all ranks read from all peers at once
        const int64_t n = (int64_t)world * rows;
        const int per = vec ? rows >> 2 : rows;  // pieces per strip
        const int64_t pieces = (int64_t)world * m * per;
        const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (int64_t)gridDim.x * blockDim.x;
        for (int64_t base = tid; base < pieces; base += nthreads * GATHER_BATCH) {
            uint4 v[GATHER_BATCH];
            float* out[GATHER_BATCH];
#pragma unroll
            for (int u = 0; u < GATHER_BATCH; u++) {
                const int64_t q = base + u * nthreads;
                out[u] = nullptr;
                if (q < pieces) {
                    const int64_t c = q / per;
                    const int i = (int)(q - c * per);
                    const int64_t t = c / world;
                    int r = (int)(c - t * world) + rank;
                    r -= r >= world ? world : 0;
                    const float* src = gather_stage(peers.land[r]) + t * rows;
                    out[u] = y + t * n + (int64_t)r * rows;
                    if (vec) {
                        asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                                     : "l"(reinterpret_cast<const uint4*>(src) + i)
                                     : "memory");
                        out[u] += 4 * i;
                    } else {
                        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v[u].x) : "l"(src + i) : "memory");
                        out[u] += i;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < GATHER_BATCH; u++) {
                if (out[u]) {
                    if (vec) __stcs(reinterpret_cast<uint4*>(out[u]), v[u]);
                    else *out[u] = __uint_as_float(v[u].x);
                }
            }
        }
    }
    // the last CTA out counts the gather and tells the peers that this rank no longer reads their blocks
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        failed = atomicAdd(epoch + 3, 1u) == gridDim.x - 1 ? 2 : 0;
    }
    __syncthreads();
    if (failed == 2) {
        if (threadIdx.x == 0) {
            epoch[3] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(epoch + 2) = tag;
        }
        if ((int)threadIdx.x < world && (int)threadIdx.x != rank)
            st_release_sys_u32(gather_flags(peers.land[threadIdx.x], 1) + rank, tag);
    }
}

// The same gather with the copy engine of the SM instead of registers: one thread per CTA walks its pieces
// (<= 16 KB of a strip each), bulk-loads them from the owner's staging area into a ring of shared-memory
// buffers and bulk-stores them into y.  Eight loads of 16 KB are in flight per SM -- far more than registers
// hold, which is what reads over NVLink need -- and no data passes through a register.  Strips must be
// multiples of 16 bytes at 16-byte aligned addresses and at least GB_MIN_STRIP long; other shapes take
// gather_large_kernel.
constexpr int GB_PIECE = 16384, GB_BUFS = 12, GB_LAG = 4;
constexpr int GB_SMEM = GB_BUFS * GB_PIECE + GB_BUFS * 8 + 16;
constexpr int GB_MIN_STRIP = 8192;  // shorter strips: one bulk copy per strip costs more than it moves (measured at 512 bytes: 3 x slower)

__global__ void __launch_bounds__(32) gather_bulk_kernel(float* __restrict__ y, GatherPeers peers, unsigned int* epoch, int* status, int64_t m,
                                                         int rows, int world, int rank, unsigned long long wait_ns) {
    extern __shared__ __align__(128) uint8_t gb_smem[];
    const uint32_t buf0 = smem_u32(gb_smem), bar0 = buf0 + GB_BUFS * GB_PIECE, abort32 = bar0 + GB_BUFS * 8;
    const int lane = threadIdx.x;
    const unsigned int e = *reinterpret_cast<volatile unsigned int*>(epoch + 2);
    const unsigned int tag = e + 1u;
    if (lane == 0) {
        for (int b = 0; b < GB_BUFS; b++) mbar_init(bar0 + b * 8, 1);
        *reinterpret_cast<volatile int*>(gb_smem + GB_BUFS * GB_PIECE + GB_BUFS * 8) = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    bool failed = false;
    if (lane < world && lane != rank) {
        if (blockIdx.x == 0) {
            __threadfence_system();
            st_release_sys_u32(gather_flags(peers.land[lane], 0) + rank, tag);
        }
        const unsigned int* ready = gather_flags(peers.land[rank], 0) + lane;
        unsigned long long t0 = 0;
        while ((int)(ld_acquire_sys_u32(ready) - tag) < 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (!t0) t0 = now;
            if (now - t0 > wait_ns || (*reinterpret_cast<volatile int*>(status) & STATUS_PEER_WAIT_TIMEOUT)) {
                failed = true;
                break;
            }
            __nanosleep(100);
        }
    }
    failed = __any_sync(0xFFFFFFFFu, failed);
    if (failed) {
        if (lane == 0) atomicOr(status, STATUS_PEER_WAIT_TIMEOUT);
    } else if (lane == 0) {
        asm volatile("fence.proxy.async;" ::: "memory");  // what the flags ordered is read by the copy engine from here on
        const int64_t n = (int64_t)world * rows;
        const int strip_bytes = rows * 4, pps = (strip_bytes + GB_PIECE - 1) / GB_PIECE;
        const int64_t total = (int64_t)world * m * pps;
        const int64_t count = blockIdx.x < total ? (total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        auto locate = [&](int64_t sq, const char*& src, char*& dst, uint32_t& bytes) {
            const int64_t q = blockIdx.x + sq * gridDim.x;
            const int64_t c = q / pps;
            const int off = (int)(q - c * pps) * GB_PIECE;
            const int64_t t = c / world;
            int r = (int)(c - t * world) + rank;  // the CTAs of all ranks read from all peers at once
            r -= r >= world ? world : 0;
            bytes = (uint32_t)min(GB_PIECE, strip_bytes - off);
            src = reinterpret_cast<const char*>(gather_stage(peers.land[r]) + t * rows) + off;
            dst = reinterpret_cast<char*>(y + t * n + (int64_t)r * rows) + off;
        };
        auto issue = [&](int64_t sq) {
            const char* src;
            char* dst;
            uint32_t bytes;
            locate(sq, src, dst, bytes);
            const int b = (int)(sq % GB_BUFS);
            mbar_expect_tx(bar0 + b * 8, bytes);
            bulk_load(buf0 + b * GB_PIECE, src, bytes, bar0 + b * 8);
        };
        for (int64_t sq = 0; sq < count && sq < GB_BUFS - GB_LAG; sq++) issue(sq);
        bool aborted = false;
        for (int64_t sq = 0; sq < count; sq++) {
            const int b = (int)(sq % GB_BUFS);
            mbar_wait_or_abort(bar0 + b * 8, (uint32_t)((sq / GB_BUFS) & 1), abort32);
            if (*reinterpret_cast<volatile int*>(gb_smem + GB_BUFS * GB_PIECE + GB_BUFS * 8)) {
                aborted = true;
                break;
            }
            const char* src;
            char* dst;
            uint32_t bytes;
            locate(sq, src, dst, bytes);
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(buf0 + b * GB_PIECE), "r"(bytes)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            const int64_t nxt = sq + GB_BUFS - GB_LAG;
            if (nxt < count) {
                // the buffer of piece nxt last held piece sq - GB_LAG: its store must have read it out
                asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(GB_LAG) : "memory");
                issue(nxt);
            }
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (aborted) {
            atomicOr(status, STATUS_GEMV_FIXUP_TIMEOUT);
            drain_after_abort();
        }
    }
    __syncwarp();
    // the last CTA out counts the gather and tells the peers that this rank no longer reads their blocks
    int last = 0;
    if (lane == 0) {
        __threadfence();
        last = atomicAdd(epoch + 3, 1u) == gridDim.x - 1;
        if (last) {
            epoch[3] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(epoch + 2) = tag;
        }
    }
    last = __shfl_sync(0xFFFFFFFFu, last, 0);
    if (last && lane < world && lane != rank) st_release_sys_u32(gather_flags(peers.land[lane], 1) + rank, tag);
}

// Maps every rank's landing buffer into this process.  All ranks agree on the outcome (a second gather of
// one flag per rank), because a rank that took the peer-store path alone would wait for stores nobody sends.
static void setup_peer_landing(Context* c, Comm* k) {
    NcclApi& a = nccl();
    if (k->world < 2 || k->world > WF_MAX_GATHER_RANKS) return;
    const char* off = getenv("WF_GATHER");
    const bool want = !(off && !strcmp(off, "nccl"));
    if (const char* ms = getenv("WF_GATHER_WAIT_MS")) {
        const long long v = atoll(ms);
        if (v > 0) k->wait_ns = (unsigned long long)v * 1000000ull;
    }
    bool ok = want;
    uint2* own = nullptr;
    char* d_x = nullptr;  // [world][64] handles, then [world] flags
    cudaIpcMemHandle_t h[WF_MAX_GATHER_RANKS];
    memset(h, 0, sizeof h);
    int64_t stage = GATHER_STAGE_DEFAULT;
    if (const char* mb = getenv("WF_GATHER_STAGE_MB")) {
        const long long v = atoll(mb);
        if (v >= 0 && v <= 65536) stage = v << 20;
    }
    ok = ok && cudaMalloc(&own, (size_t)(GATHER_LAND_BYTES + GATHER_FLAG_BYTES + stage)) == cudaSuccess;
    ok = ok && cudaMemset(own, 0, (size_t)(GATHER_LAND_BYTES + GATHER_FLAG_BYTES)) == cudaSuccess;
    ok = ok && cudaMalloc(&k->d_epoch, 4 * sizeof(unsigned int)) == cudaSuccess;
    ok = ok && cudaMemset(k->d_epoch, 0, 4 * sizeof(unsigned int)) == cudaSuccess;
    k->stage_bytes = stage;
    ok = ok && cudaIpcGetMemHandle(&h[k->rank], own) == cudaSuccess;
    cudaGetLastError();
    // the two exchanges run on every rank whatever happened above, so that no rank waits alone
    if (cudaMalloc(&d_x, (size_t)k->world * 64 + (size_t)k->world * 4) != cudaSuccess) {
        cudaGetLastError();
        if (own) cudaFree(own);
        if (k->d_epoch) cudaFree(k->d_epoch);
        k->d_epoch = nullptr;
        return;  // the exchanges below cannot run; peers time out of their NCCL call the way they would for a lost rank
    }
    cudaStream_t s = c->stream;
    cudaMemcpyAsync(d_x + (size_t)k->rank * 64, &h[k->rank], 64, cudaMemcpyHostToDevice, s);
    bool exchanged = a.AllGather(d_x + (size_t)k->rank * 64, d_x, 64, NCCL_INT8, k->comm, s) == NCCL_SUCCESS;
    cudaMemcpyAsync(h, d_x, (size_t)k->world * 64, cudaMemcpyDeviceToHost, s);
    exchanged = exchanged && cudaStreamSynchronize(s) == cudaSuccess;
    ok = ok && exchanged;
    if (ok) {
        for (int r = 0; r < k->world && ok; r++) {
            if (r == k->rank) {
                k->land[r] = own;
                continue;
            }
            void* p = nullptr;
            ok = cudaIpcOpenMemHandle(&p, h[r], cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
            k->land[r] = static_cast<uint2*>(p);
        }
        cudaGetLastError();
    }
    int flags[WF_MAX_GATHER_RANKS] = {};
    int* d_f = reinterpret_cast<int*>(d_x + (size_t)k->world * 64);
    // the flag carries the size of the staging area: ranks that disagreed on it would route the same gather differently
    const int mine = ok ? (int)(stage >> 20) + 1 : 0;
    flags[k->rank] = mine;
    cudaMemcpyAsync(d_f + k->rank, &flags[k->rank], 4, cudaMemcpyHostToDevice, s);
    bool agreed = a.AllGather(d_f + k->rank, d_f, 4, NCCL_INT8, k->comm, s) == NCCL_SUCCESS;
    cudaMemcpyAsync(flags, d_f, (size_t)k->world * 4, cudaMemcpyDeviceToHost, s);
    agreed = agreed && cudaStreamSynchronize(s) == cudaSuccess;
    for (int r = 0; r < k->world; r++) agreed = agreed && mine != 0 && flags[r] == mine;
    cudaFree(d_x);
    if (!agreed) {
        for (int r = 0; r < k->world; r++) {
            if (r != k->rank && k->land[r]) cudaIpcCloseMemHandle(k->land[r]);
            k->land[r] = nullptr;
        }
        if (own) cudaFree(own);
        if (k->d_epoch) cudaFree(k->d_epoch);
        k->d_epoch = nullptr;
        cudaGetLastError();
        return;
    }
    k->peer_ok = true;
    k->bulk = !(off && !strcmp(off, "registers")) &&
              cudaFuncSetAttribute(gather_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_SMEM) == cudaSuccess;
    cudaGetLastError();
}

static void release_peer_landing(Comm* k) {
    for (int r = 0; r < k->world && r < WF_MAX_GATHER_RANKS; r++) {
        if (!k->land[r]) continue;
        if (r == k->rank) cudaFree(k->land[r]);
        else cudaIpcCloseMemHandle(k->land[r]);
        k->land[r] = nullptr;
    }
    if (k->d_epoch) cudaFree(k->d_epoch);
    k->d_epoch = nullptr;
    k->peer_ok = false;
}

// True when this gather goes by peer stores: the mappings exist, the decode kernels produce the output (they
// write a column block of a wider matrix in place) and both halves of the landing buffer hold it.
static bool gather_by_peer_stores(const Comm* k, const Weight& w, int x_dtype, int64_t m, const void* x) {
    if (!k->peer_ok || k->world < 2) return false;
    if (gemm_supported(w, x_dtype, m, x)) return false;
    const int64_t words = (int64_t)k->world * m * w.g.rows;
    return words < (1ll << 31) && 2 * words * (int64_t)sizeof(uint2) <= GATHER_LAND_BYTES;
}

// True when a gather that is not small goes through the staging areas: every rank's block fits its own.
static bool gather_by_peer_loads(const Comm* k, int64_t m, int64_t rows) {
    return k->peer_ok && k->world > 1 && m * rows * 4 <= k->stage_bytes && (int64_t)k->world * m * rows < (1ll << 40);
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
    setup_peer_landing(c, k);
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
    if (k->peer_ok) {
        // The peers may still be reading this rank's block of the last large gather: wait for their "done".  A peer
        // that has gone lets this wait run out; that is no failure of any call of this context, so the status word
        // is put back afterwards.
        int before = 0;
        cudaMemcpy(&before, c->d_status, sizeof before, cudaMemcpyDeviceToHost);
        GatherPeers peers;
        for (int r = 0; r < WF_MAX_GATHER_RANKS; r++) peers.land[r] = k->land[r];
        gather_wait_done_kernel<<<1, 32, 0, c->stream>>>(peers, k->d_epoch, c->d_status, k->world, k->rank, k->wait_ns);
        cudaDeviceSynchronize();
        cudaMemcpy(c->d_status, &before, sizeof before, cudaMemcpyHostToDevice);
    }
    release_peer_landing(k);
    nccl().CommDestroy(k->comm);
    if (k->d_tmp) cudaFree(k->d_tmp);
    k->magic = 0;
    delete k;
    return WF_OK;
}

int wf_comm_info(int64_t ctx, int64_t comm, int* rank, int* world, int* peer_stores) {
    Context* c = get_context(ctx);
    if (!c) return WF_ERR_INVALID_HANDLE;
    ScopedLock lk(c);
    if (!lk.ok) return WF_ERR_BUSY;
    Comm* k = get_comm(c, comm);
    if (!k) return WF_ERR_INVALID_HANDLE;
    if (rank) *rank = k->rank;
    if (world) *world = k->world;
    if (peer_stores) *peer_stores = k->peer_ok ? 1 : 0;
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
    if (gather_by_peer_stores(k, *w, x_dtype, m, x_dev)) {
        // every rank computes its column block of y in place, then one kernel exchanges the blocks
        GemvCall call{w, x_dev, x_dtype, m, y, n, w->row0};
        int rc = gemv_launch(c, call, s);
        if (rc != WF_OK) return rc;
        GatherPeers peers;
        for (int r = 0; r < WF_MAX_GATHER_RANKS; r++) peers.land[r] = k->land[r];
        const int64_t total = m * rows;
        const int ctas = (int)std::max<int64_t>(1, std::min<int64_t>((total * (k->world - 1) + GATHER_THREADS - 1) / GATHER_THREADS, c->sm_count));
        gather_small_kernel<<<ctas, GATHER_THREADS, 0, s>>>(y, peers, k->d_epoch, c->d_status, (int)m, (int)rows, k->world, k->rank,
                                                            GATHER_LAND_BYTES / 2 / (int64_t)sizeof(uint2), k->wait_ns);
        WF_CUDA(c, cudaGetLastError());
        c->launches++;
        return WF_OK;
    }
    if (gather_by_peer_loads(k, m, rows)) {
        GatherPeers peers;
        for (int r = 0; r < WF_MAX_GATHER_RANKS; r++) peers.land[r] = k->land[r];
        gather_wait_done_kernel<<<1, 32, 0, s>>>(peers, k->d_epoch, c->d_status, k->world, k->rank, k->wait_ns);
        WF_CUDA(c, cudaGetLastError());
        float* mine = reinterpret_cast<float*>(reinterpret_cast<char*>(k->land[k->rank]) + GATHER_LAND_BYTES + GATHER_FLAG_BYTES);
        GemvCall call{w, x_dev, x_dtype, m, mine, rows, 0};
        int rc = gemm_supported(*w, x_dtype, m, call.d_x) ? gemm_launch(c, call, s) : gemv_launch(c, call, s);
        if (rc != WF_OK) return rc;
        const int vec = (rows % 4 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0);
        const int64_t pieces = (int64_t)k->world * m * (vec ? rows / 4 : rows);
        const int ctas = (int)std::max<int64_t>(1, std::min<int64_t>((pieces + GATHER_THREADS - 1) / GATHER_THREADS, c->sm_count));
        if (vec && k->bulk && rows * 4 >= GB_MIN_STRIP) {
            const int64_t total = (int64_t)k->world * m * ((rows * 4 + GB_PIECE - 1) / GB_PIECE);
            const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(total, c->sm_count));
            gather_bulk_kernel<<<grid, 32, GB_SMEM, s>>>(y, peers, k->d_epoch, c->d_status, m, (int)rows, k->world, k->rank, k->wait_ns);
        } else {
            gather_large_kernel<<<ctas, GATHER_THREADS, 0, s>>>(y, peers, k->d_epoch, c->d_status, m, (int)rows, k->world, k->rank, vec, k->wait_ns);
        }
        WF_CUDA(c, cudaGetLastError());
        c->launches += 2;
        return WF_OK;
    }
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
