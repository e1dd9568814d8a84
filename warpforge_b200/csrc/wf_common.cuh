// Internal declarations shared by the translation units of libwfb200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/wfb200.h"
#include "wf_layout.cuh"

namespace wf {

constexpr uint32_t CTX_MAGIC = 0x57464358;     // "WFCX"
constexpr uint32_t WEIGHT_MAGIC = 0x57465754;  // "WFWT"
constexpr uint32_t COMM_MAGIC = 0x5746434D;    // "WFCM"

// Device-side status bits, OR-ed into Context::d_status by kernels that give up a wait.
constexpr int STATUS_GEMV_FIXUP_TIMEOUT = 1;
constexpr int STATUS_GEMM_PIPE_TIMEOUT = 2;
constexpr int STATUS_PEER_WAIT_TIMEOUT = 4;
constexpr int STATUS_BAD_INDEX = 8;  // an embedding index outside the table

struct Context;

struct Weight {
    uint32_t magic = WEIGHT_MAGIC;
    Context* ctx = nullptr;
    WeightGeom g{};          // g.qtype is the DEVICE format (device_qtype of the file's type)
    int file_qtype = 0;      // ggml type of the blocks that were uploaded
    int64_t row0 = 0;        // first global row of this shard
    int64_t total_rows = 0;  // rows of the unsharded tensor
    uint8_t* d_tiles = nullptr;
    int programs = 0;        // live programs whose op lists point at d_tiles
    // how the several-token decode kernel cuts this weight, per activation dtype (bf16 / fp32) and column count:
    // {slices, k-tiles per slice, team size, uses partial sums}, slices = -1 until first asked for (0: no cut fits)
    short split_cache[2][33][4];
    Weight() {
        for (auto& a : split_cache)
            for (auto& b : a) b[0] = -1;
    }
};

// Scratch for the GEMV fix-up between CTAs, one per stream that launches GEMVs.
struct GemvScratch {
    uint2* d_slots = nullptr;  // [ctas][128] {value bits, tag}
    float* d_part = nullptr;   // several-token kernel: partial sums of k-sliced launches
    int* d_count = nullptr;    // several-token kernel: arrival counters per row-tile
    int ctas = 0;
};

struct Context {
    uint32_t magic = CTX_MAGIC;
    int device = 0;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    cudaStream_t stream = nullptr;  // the context's own compute stream
    int* d_status = nullptr;
    int salt = 0;                            // instrumentation level, 2 = kernel timing stamps
    unsigned long long* d_timing = nullptr;  // [sm_count][8]
    std::mutex mu;  // guards against concurrent use (try_lock -> WF_ERR_BUSY)
    std::string last_error;
    std::vector<cudaStream_t> streams;
    std::vector<cudaEvent_t> events;
    std::vector<cudaGraphExec_t> graphs;
    int64_t capture_launches = 0;  // product kernels recorded by the capture in progress
    std::unordered_map<cudaGraphExec_t, int64_t> graph_launches;
    std::unordered_map<int64_t, int64_t> allocs;  // device ptr -> bytes
    std::vector<void*> host_allocs;
    std::vector<Weight*> weights;
    std::unordered_map<cudaStream_t, GemvScratch> gemv_scratch;
    // pinned staging for host-pointer calls
    void* h_stage = nullptr;
    int64_t h_stage_bytes = 0;
    void* d_stage = nullptr;
    int64_t d_stage_bytes = 0;
    void* h_upload = nullptr;  // two pinned chunks the weight upload streams a host tensor through
    void* d_upload = nullptr;  // their landing place on the device, read by the repack kernel
    int64_t upload_chunk_bytes = 0;
    cudaEvent_t upload_done[2] = {nullptr, nullptr};
    void* d_x16 = nullptr;  // fp16 copy of the activations for the tensor-core GEMM
    int64_t x16_bytes = 0;
    float* d_gemm_partial = nullptr;       // [sm_count][512][128] pieces of tiles cut by a share boundary
    unsigned int* d_gemm_ready = nullptr;  // [sm_count][4] generation whose piece is complete, per 32-row quarter; then {generation, CTAs out}
    int64_t launches = 0;
    bool glue_exact = false;  // silu / softmax evaluate exp as the host does (double, one rounding) instead of expf
    int gemv_ctas_per_sm[3] = {0, 0, 0};
};

int set_error(Context* c, int status, const char* fmt, ...);
int cuda_status(Context* c, cudaError_t e, const char* what);
// Reads and clears the device status word after the stream has been waited for: WF_OK, or the failure a
// kernel recorded there (a bounded wait that ran out, an index outside a table).
int read_device_status(Context* c);
// WF_OK, or WF_ERR_RECORDING when `s` is being recorded into a graph: the caller is about to allocate (or
// grow) `what`, which a recording must not do -- recorded nodes would keep pointing at memory a later call
// frees.  Running the same call once before wf_graph_begin sizes everything.
int refuse_allocation_while_recording(Context* c, cudaStream_t s, const char* what);
Context* get_context(int64_t h);
Weight* get_weight(Context* c, int64_t h);
cudaStream_t resolve_stream(Context* c, int64_t stream);
int ensure_stage(Context* c, int64_t host_bytes, int64_t dev_bytes);
// validated shard upload + repack shared by wf_weight_upload and wf_gguf_upload; takes the context lock
int weight_upload(Context* c, int qtype, const void* blocks, int64_t n_rows, int64_t k, int shard_rank, int shard_world,
                  int q4_0_order, int64_t* weight);

// wf_repack.cu
cudaError_t launch_repack(int qtype, const uint8_t* d_raw, uint8_t* d_tiles, int64_t rows, int64_t k,
                          int q4_0_order, cudaStream_t s);
cudaError_t launch_dequant_rows(const Weight& w, int64_t row0, int64_t nrows, float* d_out, cudaStream_t s);

// wf_gemv.cu
struct GemvCall {
    const Weight* w;
    const void* d_x;  // [m, k] bf16 or fp32
    int x_dtype;
    int64_t m;       // tokens, any value >= 1 (chunked internally)
    float* d_y;      // y[token * ldy + col0 + row]
    int64_t ldy;
    int64_t col0;
};
int gemv_launch(Context* c, const GemvCall& call, cudaStream_t s);
int gemv_max_tokens_per_pass(const Weight& w, int x_dtype);
int gemv_prepare_stream(Context* c, cudaStream_t s);
int gemv_launch_noalloc(Context* c, const GemvCall& call, cudaStream_t s);

// wf_gemm.cu
bool gemm_supported(const Weight& w, int x_dtype, int64_t m, const void* d_x);
int gemm_launch(Context* c, const GemvCall& call, cudaStream_t s);

struct ScopedLock {
    Context* c;
    bool ok;
    explicit ScopedLock(Context* ctx) : c(ctx), ok(ctx && ctx->mu.try_lock()) {}
    ~ScopedLock() {
        if (ok) c->mu.unlock();
    }
};

}  // namespace wf

#define WF_CUDA(c, call)                                         \
    do {                                                         \
        cudaError_t _e = (call);                                 \
        if (_e != cudaSuccess) return wf::cuda_status(c, _e, #call); \
    } while (0)
