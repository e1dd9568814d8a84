/*
 * wfb200 -- C ABI of the B200-native quantized dot_general / linear library.
 *
 * This is the boundary a WarpForge NVIDIA backend binds with Panama FFM, the same way its
 * CudaRuntime binds libcuda and its CublasRuntime binds libcublas
 * (warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/cuda/CudaRuntime.java:64-130,
 *  .../nvidia/cublas/CublasRuntime.java:116-135): every function returns an int status
 * (0 = success), handles / device pointers / streams are 64-bit integers (JAVA_LONG),
 * host buffers and out-parameters are plain addresses (ADDRESS), there are no structs by
 * value and no callbacks.  Negative codes are argument / state errors found before any GPU
 * work (the reference throws IllegalArgumentException / UnsupportedOperationException at
 * .../nvidia/ops/DotGeneralKernel.java:54-62,80-81,183-186,221-225); positive codes carry
 * a CUDA (1000 + cudaError) or NCCL (2000 + ncclResult) status, mirroring
 * CudaRuntime.checkError (CudaRuntime.java:615-633).
 *
 * All compute runs in hand-written sm_100a kernels.  There is no CPU fallback: without a
 * usable device wf_init fails and nothing else can be called.
 */
#ifndef WFB200_H
#define WFB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---------------------------------------------------------------- */
#define WF_OK 0
#define WF_ERR_INVALID_ARGUMENT (-1) /* null pointer, negative size, bad enum            */
#define WF_ERR_INVALID_HANDLE (-2)   /* unknown, destroyed or foreign handle             */
#define WF_ERR_UNSUPPORTED_TYPE (-3) /* qtype with no kernel (Dequantizer.java:58-71)    */
#define WF_ERR_SHAPE (-4)            /* K not a multiple of the block, M/N/K out of range */
#define WF_ERR_SHARD (-5)            /* rank >= world, rows not divisible                */
#define WF_ERR_BUSY (-6)             /* context used from two threads at once            */
#define WF_ERR_NO_DEVICE (-7)        /* no CUDA device / driver                          */
#define WF_ERR_NOT_SM100 (-8)        /* device is not compute capability 10.x            */
#define WF_ERR_NCCL_UNAVAILABLE (-9) /* libnccl could not be loaded                      */
#define WF_ERR_DEVICE_WAIT (-10)     /* a bounded device-side wait ran out (see wf_stream_sync) */
#define WF_ERR_TOO_LARGE (-11)       /* request exceeds a fixed capacity                 */
#define WF_ERR_GGUF (-12)            /* not a GGUF file, unsupported version or type, truncated */
#define WF_ERR_INDEX (-13)           /* an embedding index outside the table (reported by wf_stream_sync) */
#define WF_ERR_RECORDING (-14)       /* the call would allocate device memory while its stream is being recorded into a graph */
#define WF_ERR_IN_USE (-15)          /* the object is still referenced (a weight held by a live program)   */
#define WF_ERR_CUDA_BASE 1000
#define WF_ERR_NCCL_BASE 2000

/* ---- enums (ggml type ids, as in GGUF.java:294-305) ------------------------------- */
#define WF_QTYPE_Q4_0 2
#define WF_QTYPE_Q4_1 3
#define WF_QTYPE_Q5_0 6 /* GGUF.java:332-351 knows its size only; held on the device in the Q8_0 layout */
#define WF_QTYPE_Q8_0 8
#define WF_QTYPE_Q4_K 14

#define WF_DTYPE_F32 0
#define WF_DTYPE_BF16 1

/* GEMM operand precision for the tensor-core (prefill) path. */
#define WF_GEMM_AUTO 0

/* ---- library / context -------------------------------------------------------------
 * Replaces CudaContext.create / close (nvidia/cuda/CudaContext.java:41-52, 624-657) and
 * NvidiaBackend's device bookkeeping (nvidia/NvidiaBackend.java:85-138, 459-463).
 * A context owns one device, one non-blocking compute stream, and every allocation made
 * through it.  It is not re-entrant: concurrent calls on one context return WF_ERR_BUSY.
 * wf_destroy frees everything; a second wf_destroy returns WF_ERR_INVALID_HANDLE. */
int wf_version(void);
int wf_device_count(int* count);
int wf_init(int device, int64_t* ctx);
int wf_destroy(int64_t ctx);
int wf_device_info(int64_t ctx, int* sm_count, int* cc_major, int* cc_minor, int64_t* total_mem,
                   int64_t* free_mem);

/* Replaces GpuBackend.createStream / destroyStream / synchronizeStream
 * (warpforge-core/src/main/java/io/surfworks/warpforge/core/backend/GpuBackend.java:100-130).
 * stream 0 everywhere below means the context's own compute stream.  wf_stream_sync also
 * reports WF_ERR_DEVICE_WAIT if a kernel gave up a bounded wait since the last sync. */
int wf_stream_create(int64_t ctx, int64_t* stream);
int wf_stream_destroy(int64_t ctx, int64_t stream);
int wf_stream_sync(int64_t ctx, int64_t stream);

/* Replaces CudaContext.allocate / free / copyToDevice / copyToHost
 * (nvidia/cuda/CudaContext.java:80-150) and GpuBackend.allocateDevice / allocatePinned.
 * Copies are asynchronous on `stream` and need a wf_stream_sync before the host buffer is
 * reused, unless `sync` is non-zero. */
int wf_malloc(int64_t ctx, int64_t bytes, int64_t* dptr);
int wf_free(int64_t ctx, int64_t dptr);
int wf_host_alloc(int64_t ctx, int64_t bytes, void** host);
int wf_host_free(int64_t ctx, void* host);
int wf_memcpy_h2d(int64_t ctx, int64_t dst, const void* src, int64_t bytes, int64_t stream, int sync);
int wf_memcpy_d2h(int64_t ctx, void* dst, int64_t src, int64_t bytes, int64_t stream, int sync);

/* ---- quantized weights -------------------------------------------------------------
 * Takes the raw GGUF blocks of one [n_rows x k] tensor (blocks run along k inside a row,
 * exactly the bytes GGUF.tensor(name) returns, GGUF.java:221-225, sized by
 * GGUF.java:332-351) and keeps the row shard [rank*n_rows/world, (rank+1)*n_rows/world) on
 * the device in the library's tiled layout.  The reference has no counterpart: it would
 * dequantize to fp32 on the host (QuantizedTensorView.dequantizeToArray,
 * warpforge-data/.../quant/QuantizedTensorView.java:161-166) and upload 4 bytes per weight.
 * `blocks` points at the FULL tensor; only the shard is copied.  wf_weight_free returns
 * WF_ERR_IN_USE while a live program (wf_program_create) holds the weight. */
int wf_weight_upload(int64_t ctx, int qtype, const void* blocks, int64_t n_rows, int64_t k, int shard_rank,
                     int shard_world, int64_t* weight);
int wf_weight_free(int64_t ctx, int64_t weight);
/* rows = rows held by this shard, row0 = first global row of the shard. */
int wf_weight_info(int64_t ctx, int64_t weight, int* qtype, int64_t* rows, int64_t* k, int64_t* row0,
                   int64_t* device_bytes);

/* ---- GGUF files ---------------------------------------------------------------------
 * Replaces GGUF.open / tensorInfo / tensor / metadata / close for the weights of this path
 * (warpforge-data/src/main/java/io/surfworks/warpforge/data/format/GGUF.java:96-176 open and
 * header parse, :206-225 tensor lookup and data slice, :294-351 ggml type numbers and block
 * sizes, :357-470 value decoding).  The file is memory-mapped read-only and stays mapped
 * until wf_gguf_close; handles are process-wide and need no device, so a file can be
 * inspected without a context.  Failures the reference reports as exceptions come back as
 * WF_ERR_GGUF with the reference's message in `err` ("Invalid GGUF magic: ...", "File too
 * small to be a GGUF file: ...", "Unsupported GGUF version: ...", "Unknown GGML type: ...");
 * a name that is not in the file is WF_ERR_INVALID_ARGUMENT ("No tensor named: ...").
 * Dimensions are in file order: dims[0] varies fastest, so a linear weight [n_rows, k] is
 * stored as {k, n_rows}; unused entries of dims8 are 1.  `offset` is relative to the data
 * section, whose start wf_gguf_info reports (header end rounded up to general.alignment,
 * default 32).  Metadata values are rendered as text (numbers in decimal, booleans as
 * true/false, arrays as their first elements in brackets). */
int wf_gguf_open(const char* path, int64_t* gguf, char* err, int64_t err_len);
int wf_gguf_close(int64_t gguf);
int wf_gguf_info(int64_t gguf, int* version, int64_t* tensor_count, int64_t* metadata_count, int64_t* data_offset,
                 int* alignment, int64_t* file_size);
int wf_gguf_tensor_name(int64_t gguf, int64_t index, char* buf, int64_t n);
int wf_gguf_tensor_info(int64_t gguf, const char* name, int* ggml_type, int* n_dims, int64_t* dims8, int64_t* offset,
                        int64_t* size);
int wf_gguf_tensor_data(int64_t gguf, const char* name, const void** data, int64_t* size);
int wf_gguf_metadata(int64_t gguf, int64_t index, char* key, int64_t key_len, char* value, int64_t value_len);

/* wf_weight_upload straight from the mapping: the 2-D tensor `name` ({k, n_rows} in the
 * file) becomes a device-resident row shard without the bytes passing through the caller.
 * q4_0_order says how the 16 quant bytes of a Q4_0 or Q4_1 block map to its 32 elements:
 * WF_Q4_0_ORDER_REFERENCE is the order Dequantizer.java:251-279 reads (byte i holds
 * elements 2i and 2i+1), WF_Q4_0_ORDER_GGML the order ggml writes (byte i holds elements i
 * and i+16).  The device layout is the same either way, so the choice costs nothing at
 * run time; it is ignored for the other types. */
#define WF_Q4_0_ORDER_REFERENCE 0
#define WF_Q4_0_ORDER_GGML 1
int wf_gguf_upload(int64_t ctx, int64_t gguf, const char* name, int shard_rank, int shard_world, int q4_0_order,
                   int64_t* weight);

/* Replaces Dequantizer.dequantize(MemorySegment, float[], int)
 * (warpforge-data/.../quant/Dequantizer.java:204-221 Q8_0, :251-279 Q4_0; Q4_K per the GGUF
 * block format): fp32 values of shard rows [row0, row0+nrows), bit-identical to the CPU
 * result, written to host memory. */
int wf_dequant_rows(int64_t ctx, int64_t weight, int64_t row0, int64_t nrows, float* out_host);

/* ---- the fp32 operations between the projections of a decode step ---------------------
 * Replace the custom_call kernels of CudaCustomCallKernel.execute
 * (nvidia/ops/CudaCustomCallKernel.java:50-59: "rms_norm", "layer_norm", "softmax", "silu",
 * "embedding") with the arithmetic of the CPU backend's CustomCallKernel
 * (warpforge-backend-cpu/.../ops/scalar/CustomCallKernel.java: layer_norm :109-171,
 * softmax :173-224, silu :262-280, embedding :282-318, rms_norm :368-412).  All pointers are
 * device pointers to contiguous fp32 (indices: int64), the calls only enqueue on `stream`.
 * Row operations work on [rows, n] and normalise the last dimension, as the reference does;
 * gamma / beta may be 0 (not given), as the optional inputs of the reference are.  The
 * reference takes eps = 1e-5 always (it does not parse the op's attributes); pass that for
 * parity.  wf_swiglu is silu(gate) * up (the silu custom_call followed by stablehlo.multiply),
 * wf_add the residual stablehlo.add.  In-place use (y == x) is allowed for all but
 * wf_embedding.  An embedding index outside [0, vocab) writes a row of zeros and makes the
 * next wf_stream_sync return WF_ERR_INDEX (the CPU backend throws there).
 * wf_set_exact_exp(ctx, 1) makes wf_silu / wf_swiglu / wf_softmax evaluate the exponential
 * as the CPU backend does, (float) Math.exp(x): the result then equals the CPU's bit for bit
 * (silu, swiglu) at about half the speed; the default is the fp32 exponential (2 ulp), which
 * keeps these operations memory-bound. */
int wf_set_exact_exp(int64_t ctx, int on);
int wf_rms_norm(int64_t ctx, int64_t x_dev, int64_t gamma_dev, int64_t y_dev, int64_t rows, int64_t n, float eps,
                int64_t stream);
int wf_layer_norm(int64_t ctx, int64_t x_dev, int64_t gamma_dev, int64_t beta_dev, int64_t y_dev, int64_t rows,
                  int64_t n, float eps, int64_t stream);
int wf_softmax(int64_t ctx, int64_t x_dev, int64_t y_dev, int64_t rows, int64_t n, int64_t stream);
int wf_silu(int64_t ctx, int64_t x_dev, int64_t y_dev, int64_t count, int64_t stream);
/* stablehlo.dot on dense fp32 device operands: C[m,n] = A[m,k] . B[k,n], row-major (nvidia/ops/DotKernel.java:18-154;
 * CPU arithmetic cpu/ops/scalar/DotKernel.java:51-59).  Each output is summed over k ascending with a separate
 * multiply and add, as the CPU kernel does, so the bits are the CPU's.  A vector operand is a matrix with m = 1 or n = 1. */
int wf_dot_f32(int64_t ctx, int64_t a_dev, int64_t b_dev, int64_t c_dev, int64_t m, int64_t n, int64_t k, int64_t stream);
/* gelu, tanh form: 0.5 x (1 + tanh(0.7978845608 (x + 0.044715 x^3))), cpu/ops/scalar/CustomCallKernel.java:226-260. */
int wf_gelu(int64_t ctx, int64_t x_dev, int64_t y_dev, int64_t count, int64_t stream);
int wf_swiglu(int64_t ctx, int64_t gate_dev, int64_t up_dev, int64_t y_dev, int64_t count, int64_t stream);
int wf_add(int64_t ctx, int64_t a_dev, int64_t b_dev, int64_t y_dev, int64_t count, int64_t stream);
int wf_embedding(int64_t ctx, int64_t indices_dev, int64_t table_dev, int64_t y_dev, int64_t count, int64_t vocab,
                 int64_t dim, int64_t stream);

/* ---- the op -------------------------------------------------------------------------
 * Replaces DotGeneralKernel.execute for `linear`: lhs [m,k] contracting dim 1, rhs [n,k]
 * contracting dim 1 (nvidia/ops/DotGeneralKernel.java:169-298 with transposeB, CPU rule at
 * warpforge-backend-cpu/.../ops/scalar/DotGeneralKernel.java:85-128), with rhs a quantized
 * weight handle.  y[m, rows] = x[m, k] . W[rows, k]^T, fp32 accumulation, fp32 output.
 * x_dtype is WF_DTYPE_BF16 or WF_DTYPE_F32.  x / y are device pointers (x_on_device /
 * y_on_device non-zero) or host pointers; host buffers are staged through pinned memory
 * and the call returns after the result is in `y`.  With device pointers the call only
 * enqueues work on `stream`; with a host pointer it waits for the result and reports a bounded
 * device-side wait that ran out as WF_ERR_DEVICE_WAIT, like wf_stream_sync.  Up to 32 bf16 tokens
 * (10 fp32 tokens) per launch run on the memory-bound decode kernels; more bf16 tokens run on the
 * tensor-core GEMM, whose activation copy and tile-piece scratch belong to the context: many-token
 * calls of one context must not overlap on different streams. */
int wf_qlinear(int64_t ctx, int64_t weight, const void* x, int x_dtype, int x_on_device, int64_t m, void* y,
               int y_on_device, int64_t stream);

/* Same op followed by the gather of the row shards: every rank passes its own shard handle and
 * receives the full y[m, n_total] (columns [r * rows, (r + 1) * rows) of every token are rank r's),
 * the result of CollectiveApi.allGather on the shards' outputs.  Device pointers only; the call
 * enqueues on `stream`.  A collective: every rank of the communicator makes the same calls in the
 * same order.  How the rows travel is described at wf_comm_info; a peer that does not arrive within
 * the wait limit shows as WF_ERR_DEVICE_WAIT at the next synchronisation.  The gathers of one communicator
 * are numbered on the device in the order they execute: issue them on one stream (or on streams ordered by
 * events), never on two streams that may run concurrently. */
int wf_qlinear_allgather(int64_t ctx, int64_t comm, int64_t weight, const void* x_dev, int x_dtype, int64_t m,
                         void* y_full_dev, int64_t stream);

/* wf_qlinear for hosts that must not allocate device memory once they are running.  (No
 * counterpart in the reference: its kernels allocate and free on every call,
 * nvidia/ops/DotGeneralKernel.java:238-296.)  Think of an embedding application that handed
 * all device memory to its own arena at start-up, or a serving loop with a "no allocation
 * after warm-up" rule: there a cudaMalloc can fail for lack of memory, or stall the whole
 * device while it synchronizes.  wf_qlinear obtains a small per-stream work area from
 * cudaMalloc the first time a stream is used; this variant never calls cudaMalloc, cudaFree
 * or any allocating routine.  Its work area (the slots through which thread blocks hand
 * partial rows to each other) is a fixed 256 KiB array compiled into the library, present
 * on every GPU that loads it until the process ends.
 *   - x and y are DEVICE pointers (x: [m, k] bf16 or fp32, y: [m, rows] fp32); the call only
 *     enqueues work on `stream`.
 *   - Limit: the device may have at most 256 SMs (one slot set per SM); beyond that, and for
 *     a K that does not fit one SM's shared memory, the call returns WF_ERR_TOO_LARGE.
 *   - The first call on each device looks up the array's device address (and the first use
 *     of a kernel variant sets a function attribute); make that first call before starting
 *     any stream capture.
 *   - All calls on one device share the one array and it keeps what the last call left in
 *     it, so every call first clears the part it uses, on `stream`.  Two calls that can run
 *     at the same time on the GPU (different streams, or two contexts on one device) would
 *     use the same slots and corrupt each other: issue them on one stream, or order them. */
int wf_qlinear_noalloc(int64_t ctx, int64_t weight, int64_t x_dev, int x_dtype, int64_t m, int64_t y_dev,
                       int64_t stream);

/* ---- collectives --------------------------------------------------------------------
 * Replaces CollectiveApi.allGather(Tensor input, Tensor output)
 * (warpforge-io/src/main/java/io/surfworks/warpforge/io/collective/CollectiveApi.java:137-146,
 * UCC implementation at .../collective/impl/UccCollectiveImpl.java:503-543): rank r's
 * `bytes_per_rank` land at recv + r*bytes_per_rank on every rank.  Transport is NCCL over
 * NVLink on device buffers.  Bootstrap mirrors CollectiveConfig(worldSize, rank, ...)
 * (.../collective/CollectiveConfig.java:15-40): rank 0 creates a 128-byte id and the
 * caller distributes it out of band. */
int wf_comm_get_unique_id(void* id128);
int wf_comm_init(int64_t ctx, const void* id128, int rank, int world, int64_t* comm);
int wf_comm_destroy(int64_t ctx, int64_t comm);
/* rank, world and whether the ranks could map each other's landing buffers (cudaIpc, one node): with
 * peer_stores == 1, wf_qlinear_allgather of up to 32 tokens (outputs of at most 2 M floats over all ranks)
 * exchanges the row blocks by one kernel of 8-byte {value, tag} stores into the peers' memory instead of an
 * NCCL all-gather plus a copy; larger outputs and the tensor-core path keep NCCL.  A rank waits at most
 * WF_GATHER_WAIT_MS (environment, default 5000) for its peers' stores, then sets the peer-wait status.
 * WF_GATHER=nccl in the environment at wf_comm_init keeps every gather on NCCL.  The mapped block costs each rank
 * 32 MB + WF_GATHER_STAGE_MB (environment, default 128, the same on every rank) of device memory; blocks of more
 * tokens than the staging area holds (m * rows * 4 bytes per rank) go by NCCL.  Any pointer may be null. */
int wf_comm_info(int64_t ctx, int64_t comm, int* rank, int* world, int* peer_stores);
int wf_allgather(int64_t ctx, int64_t comm, int64_t send_dev, int64_t recv_dev, int64_t bytes_per_rank,
                 int64_t stream);

/* ---- decode programs ----------------------------------------------------------------
 * A decode step is a fixed list of quantized projections.  The reference would run it as
 * one Backend.execute per op from GraphExecutor's loop (warpforge-core/.../graph/GraphExecutor.java:75-104),
 * each with its own launch and synchronisation; a program runs the whole list as ONE
 * persistent kernel per GPU, streaming the weights of consecutive ops back to back.
 *   weights[n_ops]           weight handles, all of one quantization type
 *   x_dev[n_ops]             bf16 activations [m, k] each op reads (device pointers)
 *   y_dev[n_ops]             this rank's fp32 output buffer [m, n_total] of each op; after the run it
 *                            holds ALL rows (own shard computed here, the others gathered)
 *   flags[n_ops]             WF_OP_NEW_X: stage x before this op (else it reuses the previous op's);
 *                            WF_OP_DEPENDS: x was produced by earlier ops of the program, so all CTAs
 *                            (and all ranks' rows) must be complete first
 *   landing_dev[n_ops*world] world > 1: for op o and rank r the address, valid on THIS device, of rank
 *                            r's landing buffer for that op (8 * m * n_total bytes, zeroed once; own at
 *                            r == rank, peers' through wf_ipc_import).  Ranks store their rows into each
 *                            other's landing buffers from inside the GEMV epilogue -- the all-gather of
 *                            CollectiveApi.allGather without a collective call.  A landing buffer may
 *                            be shared by ops at least two WF_OP_DEPENDS apart.
 * m is 1..8 tokens.  Waits inside the kernel are bounded (WF_ERR_DEVICE_WAIT at the next sync). */
#define WF_OP_NEW_X 1
#define WF_OP_DEPENDS 2
int wf_program_create(int64_t ctx, int n_ops, const int64_t* weights, const int64_t* x_dev, const int64_t* y_dev,
                      const int* flags, int64_t m, int world, int rank, const int64_t* landing_dev, int64_t* program);
/* The same with the fp32 operations that sit between a decoder layer's projections fused into the one-token
 * kernel (m = 1), so that a projection reads the previous ones' fp32 outputs directly and no kernel runs in
 * between (the reference runs each as its own custom_call / elementwise op with an allocation, two copies and a
 * synchronisation: nvidia/ops/CudaCustomCallKernel.java:50-59, CPU arithmetic at
 * cpu/ops/scalar/CustomCallKernel.java:173-224 (rms_norm), :262-280 (silu), MultiplyKernel, AddKernel).
 * Per op o (each array may be NULL = all zero):
 *   x_kind[o]  WF_X_BF16 (0): x_dev[o] is a bf16 row, as in wf_program_create;  WF_X_F32 (1): an fp32 row;
 *              WF_X_RMSNORM_F32 (2): x = rms_norm(x_dev[o] fp32, gamma = x_aux_dev[o] fp32 or 0, eps[o]);
 *              WF_X_SWIGLU_F32 (3): x = silu(x_dev[o]) * x_aux_dev[o], both fp32 rows of length k.
 *              Only the op that stages new activations (WF_OP_NEW_X) is looked at.
 *   residual_dev[o]  0, or an fp32 row [n_total] added to the result before it is stored (and before it is sent
 *              to the other ranks); may be y_dev[o] itself (h += W x). */
#define WF_X_BF16 0
#define WF_X_F32 1
#define WF_X_RMSNORM_F32 2
#define WF_X_SWIGLU_F32 3
int wf_program_create_fused(int64_t ctx, int n_ops, const int64_t* weights, const int64_t* x_dev, const int64_t* y_dev,
                            const int* flags, const int* x_kind, const int64_t* x_aux_dev, const float* eps,
                            const int64_t* residual_dev, int64_t m, int world, int rank, const int64_t* landing_dev,
                            int64_t* program);
int wf_program_run(int64_t ctx, int64_t program, int64_t stream);
/* One token end to end in one call: copy n_in activation buffers from (pinned) host memory to their device
 * buffers, run the program, copy out_bytes of a result back to host memory, wait, and report a device-side wait
 * that ran out (WF_ERR_DEVICE_WAIT) -- what a per-token loop of the reference does with copyToDevice / execute /
 * copyToHost / synchronize (nvidia/ops/DotGeneralKernel.java:169-298), without the allocations. */
int wf_program_step_host(int64_t ctx, int64_t program, int n_in, const void* const* host_src, const int64_t* dev_dst,
                         const int64_t* bytes, void* host_out, int64_t dev_out, int64_t out_bytes, int64_t stream);
int wf_program_destroy(int64_t ctx, int64_t program);
/* With wf_set_salt(ctx, 2) before wf_program_create: [sm_count][64] globaltimer stamps of the first ops
 * (kernel start, then per op: start, after barrier, after staging, after compute). */
int wf_program_read_timing(int64_t ctx, int64_t program, int64_t* out, int64_t n);
/* Peer access to a wf_malloc'ed buffer of another process on the same node (the role
 * GpuBackend.registerForRdma plays for the reference's host-memory collectives,
 * nvidia/NvidiaBackend.java:244-259): a 64-byte handle to hand to the peers out of band. */
int wf_ipc_export(int64_t ctx, int64_t dptr, void* handle64);
int wf_ipc_import(int64_t ctx, const void* handle64, int64_t* dptr);
int wf_ipc_close(int64_t ctx, int64_t dptr);

/* ---- launch management -------------------------------------------------------------
 * The reference launches every kernel with cuLaunchKernel on stream 0 and synchronizes the
 * context after each op (nvidia/cuda/CudaContext.java:273-321, nvidia/ops/DotGeneralKernel.java:283).
 * A decode step is hundreds of microsecond-scale kernels, so the backend instead records a
 * sequence of device-pointer calls (wf_qlinear, wf_qlinear_allgather, wf_allgather, copies)
 * issued on `stream` between begin and end into a CUDA graph and replays it with one launch.
 * Only calls with device pointers may be recorded.  Nothing is allocated while a stream is being
 * recorded: wf_graph_begin sizes the decode kernels' scratch, and a recorded call that would have to
 * allocate or grow another buffer (the GEMM's activation copy and piece buffers, the gather buffer of
 * wf_qlinear_allgather) returns WF_ERR_RECORDING and records nothing -- issue the same call once
 * before wf_graph_begin. */
int wf_graph_begin(int64_t ctx, int64_t stream);
int wf_graph_end(int64_t ctx, int64_t stream, int64_t* graph);
int wf_graph_launch(int64_t ctx, int64_t graph, int64_t stream);
int wf_graph_destroy(int64_t ctx, int64_t graph);

/* ---- errors -------------------------------------------------------------------------
 * Replaces CudaRuntime.getErrorName / checkError message formatting. */
const char* wf_error_string(int status);
int wf_last_error(int64_t ctx, char* buf, int64_t buf_len);

/* ---- measurement helpers (used by the benchmark; CudaContext.java:519-613 has the
 * reference's CUDA-event helpers) -------------------------------------------------- */
int wf_event_create(int64_t ctx, int64_t* event);
int wf_event_destroy(int64_t ctx, int64_t event);
int wf_event_record(int64_t ctx, int64_t event, int64_t stream);
int wf_event_elapsed_ms(int64_t ctx, int64_t start, int64_t stop, float* ms);
/* Instrumentation level, the `salt` every reference kernel class is constructed with
 * (nvidia/ops/DotGeneralKernel.java:40-43; SALT_TIMING at nvidia/cuda/CudaKernels.java:31-37).
 * 0 = none; 2 = GEMV kernels record per-CTA globaltimer stamps (start, activations staged,
 * loop entered, first tile landed, loop done, end) that wf_read_timing copies out as
 * [sm_count][8] int64 nanoseconds after synchronizing the device. */
int wf_set_salt(int64_t ctx, int salt);
int wf_read_timing(int64_t ctx, int64_t* out, int64_t n);
/* Number of kernel launches this context has issued (product kernels only). */
int wf_launch_count(int64_t ctx, int64_t* launches);
/* How the several-token decode kernel would cut a [rows x k] weight of type qtype for `cols` activation columns
 * (1..32; an fp32 token counts three) on a device with sm_count SMs: k-slices, k-tiles per slice, warps per team,
 * whether partial sums are used, shared-memory bytes.  Needs no device (host arithmetic only); slices = 0 means
 * no cut fits and the call is run in several launches of fewer columns. */
int wf_plan_several_tokens(int qtype, int64_t rows, int64_t k, int cols, int x_is_f32, int sm_count, int* slices,
                           int* k_tiles_per_slice, int* team, int* uses_partial_sums, int64_t* smem_bytes);

#ifdef __cplusplus
}
#endif
#endif /* WFB200_H */
