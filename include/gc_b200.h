/*
 * gc_b200.h — C ABI of the B200 (sm_100a) execution backend for Intel Graph
 * Compiler's matmul / MLP / attention partitions.
 *
 * Two groups of entry points live in libGcDnnlApi.so:
 *   1. the oneDNN-graph backend API of the reference (dnnl_graph_compiler.h in
 *      this directory) — create / compile / execute on JSON partitions;
 *   2. the entry points below: the runtime symbols the reference's JIT-ed code
 *      calls (dnnl_brgemm_*), and direct launchers for the kernels that replace
 *      its deep-tiled matmul pipeline, for callers that already hold device
 *      buffers (benchmark harnesses, a framework's own executor).
 *
 * All pointers are plain device pointers unless stated otherwise; `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).  Every
 * function returns 0 on success or a gcb200_status; the message of the last
 * failure on the calling thread is available from gcb200_last_error().
 * Nothing here falls back to the CPU: without a usable sm_100 device every
 * launcher fails with GCB200_NO_DEVICE.
 */
#ifndef GC_B200_H
#define GC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  GCB200_OK = 0,
  GCB200_INVALID_ARGUMENT = 1,
  GCB200_UNIMPLEMENTED = 2,
  GCB200_NO_DEVICE = 3,
  GCB200_CUDA_ERROR = 4,
  GCB200_DEVICE_TIMEOUT = 5 /* a bounded wait inside a kernel ran out; see gcb200_device_error */
} gcb200_status;

const char *gcb200_last_error(void);

/* Reads and clears the device-side error word (0 = none; otherwise the code of
 * the bounded wait that gave up).  Synchronises `stream`. */
int gcb200_device_error(void *stream, int *code);

/* Kernel launches this library has issued since it was loaded (all launchers,
 * all threads).  Benchmarks difference it around a timed region. */
int gcb200_launch_count(uint64_t *count);

/* Number of SMs of the current device (persistent grids are sized from it). */
int gcb200_sm_count(int *count);

/* ---------------------------------------------------------------------------
 * bf16 matmul with fused post-ops.
 * Replaces: onednn_graph.matmul lowered by MatMulOpLowering
 * (lib/gc/Transforms/OneDNNGraphToLinalg.cpp:421-499), deep-tiled by
 * DeepTileMatmul (lib/gc/Transforms/DeepTileContractionOp.cpp:958-1014) into
 * brgemm calls (lib/gc/ExecutionEngine/CPURuntime/Microkernel/BrgemmOnednn.cpp:
 * 145-168) with the bias add and ReLU fused by IterativeTilingAndFusion.cpp:743-828.
 *
 *   Y = act( bf16( bf16(op(A) . op(B)) + bias ) )      f32 accumulation
 * A: [M,K] (or [K,M] when transpose_a); B: [K,N] (or [N,K] when transpose_b);
 * bias: [N] bf16 or NULL; Y: [M,N] bf16, all row-major and contiguous.
 */
int gcb200_matmul_bf16(const void *A, const void *B, const void *bias, void *Y, int64_t M, int64_t N, int64_t K,
                       int transpose_a, int transpose_b, int relu, void *stream);

/* Same contraction, raw f32 accumulators out (no rounding, no post-op): the
 * K-split form of the reference, where partial sums stay f32 until they are
 * reduced (DeepTileContractionOp.cpp:446-471, 988-996).  Used by row-parallel
 * layers whose partial sums are reduced across GPUs. */
int gcb200_matmul_bf16_f32out(const void *A, const void *B, float *Y, int64_t M, int64_t N, int64_t K,
                              int transpose_a, int transpose_b, void *stream);

/* Row-parallel layer across GPUs, compute and exchange in one kernel: the f32 partial sums
 * A.B of this rank are written by the GEMM epilogue, tile by tile, into plane `my_plane` of EVERY
 * buffer in peer_bufs[0..n_peers) — device pointers to [planes][M][N] f32 buffers, one per rank,
 * peer-mapped (e.g. symmetric memory), this rank's own included.  Plain stores over NVLink, no
 * loads from a peer.  After a cross-rank barrier every rank holds all partial planes and finishes with
 * gcb200_reduce_bias_act_bf16 (planes summed in rank order, so every rank gets identical bits).
 * The across-device form of the reference's K-split (DeepTileContractionOp.cpp:446-471). */
int gcb200_matmul_bf16_f32out_push(const void *A, const void *B, void *const *peer_bufs, int n_peers, int my_plane,
                                   int64_t M, int64_t N, int64_t K, void *stream);

/* The same layer with the exchange shaped as reduce-scatter + all-gather (an all-reduce's traffic instead
 * of g copies of every partial sum): row block d of the f32 partial sums, rows [d M/g, (d+1) M/g), is stored
 * by the GEMM epilogue into plane `my_plane` of peer d's buffer [g][M/g][N] f32 only.  After a barrier rank d
 * calls gcb200_reduce_slice_broadcast_bf16 on its own buffer: planes summed in rank order, bias, ReLU, one
 * cast, and the bf16 rows are stored at row `row0` = d M/g of EVERY rank's [M,N] result buffer
 * (peer_out[0..n_peers)); after a second barrier every rank holds the whole layer output, bit-identical. */
int gcb200_matmul_bf16_f32out_scatter(const void *A, const void *B, void *const *peer_bufs, int n_peers, int my_plane,
                                      int64_t M, int64_t N, int64_t K, void *stream);
int gcb200_reduce_slice_broadcast_bf16(const float *parts, int nparts, int64_t rows, int64_t N, const void *bias,
                                       void *const *peer_out, int n_peers, int64_t row0, int relu, void *stream);

/* Column-sharded GEMM across GPUs with the all-gather of C done by the GEMM epilogue: this rank computes
 * its column block  act(bf16(bf16(A . B_block) + bias_block))  ([M, N] with N = columns of the block) and
 * stores every finished 16-byte chunk straight into EVERY rank's full result: peer_C[d] is the address of
 * element (0, first column of this rank's block) inside rank d's [M, ldc] bf16 buffer (peer-mapped, this
 * rank's own included).  Plain NVLink stores, no loads from a peer; after one cross-rank barrier every rank
 * holds the whole C.  The across-device form of the reference's N split (NThreads,
 * DeepTileContractionOp.cpp:562-601).  N must be a multiple of 8, ldc of 8 (no such limit for M <= 64, where
 * the weight-stationary kernel stores single elements). */
int gcb200_matmul_bf16_allgather(const void *A, const void *B, const void *bias, void *const *peer_C, int n_peers,
                                 int64_t M, int64_t N, int64_t K, int64_t ldc, int transpose_a, int transpose_b, int relu,
                                 void *stream);
/* The u8 x s8 counterpart: out = float(acc - comp[n]) * scale[n] + bias[n] stored as f32 into every rank's
 * [M, ldc] buffer at peer_C[d]; scales, bias and zero-point compensation are those of the column block. */
int gcb200_matmul_u8s8_allgather(const void *A, const void *W, const float *scale, const float *bias, const int32_t *comp,
                                 void *const *peer_C, int n_peers, int64_t M, int64_t N, int64_t K, int64_t ldc,
                                 int transpose_b, void *stream);

/* The same three peer-store forms with ONE NVLink multicast address instead of a list of peer addresses:
 * `mc_buf` / `mc_C` is the multicast mapping of a buffer that every rank has bound to the same multicast
 * object (e.g. the multicast pointer of a torch symmetric-memory allocation), so each finished 16-byte chunk
 * leaves this GPU once (`multimem.st`) and the NVSwitch writes it into every rank's copy, this rank's own
 * included — 1/(g-1) of the NVLink traffic of the address-list forms.  Row-major kernel only (M > 64).
 * mc_C points at this rank's column block inside the multicast mapping of the full [M, ldc] result. */
int gcb200_matmul_bf16_f32out_push_mc(const void *A, const void *B, void *mc_buf, int my_plane, int64_t M, int64_t N,
                                      int64_t K, void *stream);
int gcb200_matmul_bf16_allgather_mc(const void *A, const void *B, const void *bias, void *mc_C, int64_t M, int64_t N,
                                    int64_t K, int64_t ldc, int transpose_a, int transpose_b, int relu, void *stream);
int gcb200_matmul_u8s8_allgather_mc(const void *A, const void *W, const float *scale, const float *bias, const int32_t *comp,
                                    void *mc_C, int64_t M, int64_t N, int64_t K, int64_t ldc, int transpose_b, void *stream);

/* Sum `nparts` f32 planes [M,N] (`plane_stride` elements apart) in plane order,
 * then apply the bf16 epilogue bf16(bf16(sum)+bias), ReLU.  The reduce + cast
 * step of the K-split form (DeepTileContractionOp.cpp:446-471). */
int gcb200_reduce_bias_act_bf16(const float *parts, int nparts, int64_t plane_stride, const void *bias, void *Y,
                                int64_t M, int64_t N, int relu, void *stream);

/* ---------------------------------------------------------------------------
 * u8 x s8 -> s32 matmul with zero-point compensation and per-channel dequant.
 * Replaces: the int8 brgemm path (BrgemmNaive.cpp:102-140 semantics; dtype
 * pairs lib/gc/Dialect/Microkernel/MicrokernelOps.cpp:556-570) with the
 * compensation of legacy/core/src/ops/matmul_core.cpp:655-700.
 *
 *   acc = A_u8 . W_s8  (exact s32);  comp[n] = zp_a * sum_k W[k,n]
 *   out = float(acc - comp[n]) * scale[n] + bias[n]
 * A: [M,K] u8; W: [K,N] s8 (or [N,K] when transpose_b: the K-contiguous form the
 * tensor core reads fastest for 8-bit operands); scale, bias: [N] f32 (bias may be NULL); comp: [N]
 * s32 as produced by gcb200_colsum_s8 (NULL = no compensation); out: [M,N] f32;
 * acc_out: optional [M,N] s32 receiving the raw accumulators (bit-exact check).
 */
int gcb200_matmul_u8s8(const void *A, const void *W, const float *scale, const float *bias, const int32_t *comp,
                       float *out, int32_t *acc_out, int64_t M, int64_t N, int64_t K, int transpose_b, void *stream);
int gcb200_colsum_s8(const void *W, int32_t *comp, int64_t K, int64_t N, int32_t zp_a, void *stream);

/* ---------------------------------------------------------------------------
 * Exact-order f32 matmul (+bias, ReLU) for f32 graphs — the form the reference's
 * C-API test exercises (test/dnnl/TestApiOps.cpp:69-119).  CUDA cores, k
 * ascending, separate multiply and add. */
int gcb200_matmul_f32(const float *A, const float *B, const float *bias, float *Y, int64_t M, int64_t N, int64_t K,
                      int transpose_a, int transpose_b, int relu, void *stream);

/* ---------------------------------------------------------------------------
 * Tile selection (the GPU counterpart of MatmulConfig, include/gc/Analysis/
 * MatmulConfigAnalysis.h:25-34, chosen by MatmulConfigAnalysis.cpp:435-552).
 * Pure host logic; needs no device. */
typedef struct {
  int swapped, bn, splits, stages, group_m, grid;
  int pair; /* 1: CTA-pair kernel (tcgen05 cta_group::2), 256 x bn tiles on two SMs */
  int kpb;  /* K blocks of 128 bytes per pipeline stage (0 or 1: one) */
} gcb200_matmul_config;
int gcb200_select_matmul_config(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count,
                                gcb200_matmul_config *cfg);

/* Measured configurations.  A configuration recorded for a shape (found by timing candidates on the
 * device, see gc_b200/tune.py) takes precedence over the model in gcb200_select_matmul_config and in every
 * matmul launch of that exact shape; the cache is a text file (one "M N K dtype_bytes out_bytes : swapped bn
 * splits stages group_m grid pair kpb" line per shape), read once from the path in GC_B200_TUNE_CACHE and
 * loadable / savable explicitly.  The reference's counterpart is the per-op override attribute set of
 * MatmulConfigAnalysis.cpp:368-401.  Host logic; needs no device. */
int gcb200_tune_cache_put(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, const gcb200_matmul_config *cfg);
int gcb200_tune_cache_get(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, gcb200_matmul_config *cfg, int *found);
int gcb200_tune_cache_load(const char *path, int *entries_read);
int gcb200_tune_cache_save(const char *path, int *entries_written);
int gcb200_tune_cache_erase(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes);
int gcb200_tune_cache_clear(void);
/* The model's own choice, ignoring recorded configurations (what a tuner compares against). */
int gcb200_model_matmul_config(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count,
                               gcb200_matmul_config *cfg);

/* bf16 matmul with an explicit tile configuration (tuning, tests). */
int gcb200_matmul_bf16_cfg(const void *A, const void *B, const void *bias, void *Y, int64_t M, int64_t N, int64_t K,
                           int transpose_a, int transpose_b, int relu, const gcb200_matmul_config *cfg, void *stream);

/* ---------------------------------------------------------------------------
 * Fused attention (extension: the reference has softmax and matmul pieces but no
 * fused pattern — lib/gc/Transforms/DecomposeAggregatedOps.cpp:24-38 defines the
 * softmax it would use).  O = softmax(Q K^T * scale [+ causal mask]) V, softmax
 * in f32; Q, K, V, O: [batch*heads][seq][head_dim] bf16, contiguous. */
int gcb200_attention_bf16(const void *Q, const void *K, const void *V, void *O, int64_t batch_heads, int64_t seq,
                          int64_t head_dim, float scale, int causal, void *stream);

/* ---------------------------------------------------------------------------
 * Additions around the dnnl_graph_compiler_* API (declared in
 * dnnl_graph_compiler.h; tensor struct repeated here as an opaque pointer to
 * keep this header standalone).
 *
 * gcb200_execute_on_stream: like dnnl_graph_compiler_execute
 * (src/dnnl/dnnl_graph_compiler.cpp:214-226) but enqueues on the caller's stream
 * and returns without synchronising when every tensor is a device pointer.
 * gcb200_plan_dump: text form of the compiled launch plan (steps, fused post-ops,
 * arena offsets) — the counterpart of the reference's --ir_printing
 * (python/gc_mlir/graph_compiler.py:30-34).  Needs no device.
 * gcb200_plan_arena: the workspace planner by itself (role of
 * lib/gc/Transforms/StaticMemoryPlanning.cpp:628-652). */
struct dnnl_graph_compiler_executable;
struct dnnl_graph_compiler_tensor;
int gcb200_execute_on_stream(const struct dnnl_graph_compiler_executable *exe, struct dnnl_graph_compiler_tensor *inputs,
                             struct dnnl_graph_compiler_tensor *outputs, void *stream);
int gcb200_plan_dump(const struct dnnl_graph_compiler_executable *exe, char *buf, size_t cap, size_t *needed);
int gcb200_plan_arena(const int64_t *bytes, const int *first, const int *last, int n, int64_t align, int64_t *offsets,
                      int64_t *total);
/* Observability, in the reference's terms.  GC_DEBUG=<extended regex over source file paths> enables the
 * "[DEBUG] [file:line] ..." lines of the matching files on stdout, errors always go to stderr as "[ERROR] ..."
 * (include/gc/Utils/Log.h:43-66).  GC_B200_VERBOSE=1 prints, per compiled partition, what
 * gcb200_describe_launches returns: one line per step with the kernel and, for matmuls, tile, K split, pipeline
 * depth and grid as chosen for `sm_count` SMs (the reference prints its choice under LLVM_DEBUG,
 * lib/gc/Analysis/MatmulConfigAnalysis.cpp:544-546).  Needs no device. */
int gcb200_describe_launches(const struct dnnl_graph_compiler_executable *exe, int sm_count, char *buf, size_t cap, size_t *needed);
/* Debug guard bands.  With GC_B200_GUARD=<bytes> in the environment when a partition is COMPILED, every slice of its
 * workspace arena is planned with that many bytes (rounded up to 256) of canary before and after it; every
 * synchronous execute then checks the bands and fails with dnnl_runtime_error naming the tensor whose band was
 * overwritten (the reference's debug memory pool keeps such a canary per allocation,
 * lib/gc/ExecutionEngine/CPURuntime/MemoryPool.cpp:55-60, :213-217).  gcb200_guard_check runs the check on demand
 * (synchronises the device); gcb200_guard_selftest damages one band from the host, the way a stray store would,
 * so that the detection itself can be tested without any out-of-bounds access on the GPU. */
int gcb200_guard_check(const struct dnnl_graph_compiler_executable *exe, int *damaged_bands);
int gcb200_guard_selftest(const struct dnnl_graph_compiler_executable *exe);
/* The planner on a raw trace, with the reference's interface (memoryplan::scheduleMemoryAllocations,
 * include/gc/Transforms/StaticMemoryPlanning.h:57-62): trace i allocates trace_size[i] elements for buffer
 * trace_buffer[i], or releases it when the size is 0; hint i says buffer hint_buffer[i] may take over
 * hint_candidate[i] in place (hint_kind 0: only at its start, 1: anywhere inside; order matters).
 * Out: (buffer, offset) pairs for every buffer, the total size, and (buffer, reused buffer) pairs.
 * n_out / n_sel: capacity in, count out.  Needs no device. */
int gcb200_schedule_memory(const uint64_t *trace_buffer, const uint64_t *trace_size, int n_traces, uint64_t alignment,
                           int hot_first, const uint64_t *hint_buffer, const uint64_t *hint_candidate,
                           const int *hint_kind, int n_hints, uint64_t *out_buffer, uint64_t *out_offset, int *n_out,
                           uint64_t *total, uint64_t *sel_buffer, uint64_t *sel_reused, int *n_sel);

/* ---------------------------------------------------------------------------
 * Tensor-parallel MLP across the GPUs of one node: one process per GPU, each calling these with the same shapes.
 * The across-device form of the reference's N and K thread splits (NThreads / KThreads,
 * lib/gc/Transforms/DeepTileContractionOp.cpp:562-601; f32 partial sums reduced, then cast: :446-471, :988-996),
 * behind the same call shape as dnnl_graph_compiler_execute (src/dnnl/dnnl_graph_compiler.cpp:214-226): build once,
 * then one call per step.
 *
 * Layers 0, 2, ... are column-parallel (this rank's weight shard is [hidden[i], hidden[i+1] / world], its bias shard
 * [hidden[i+1] / world]); layers 1, 3, ... are row-parallel (shard [hidden[i] / world, hidden[i+1]], whole bias).
 * The f32 partial sums of a row-parallel layer leave the GEMM epilogue row block by row block for the rank that
 * owns the rows; the owner reduces in rank order, applies bias / ReLU, casts once and stores the bf16 rows into every
 * rank's activation buffer.  Hand-offs between GPUs are counters in device memory that this library's own kernels add to and
 * wait on (bounded; a wait that runs out sets the device error word): no other library's kernel and no host round
 * trip sits between the layers.  Every rank ends a step with the same bits.
 *
 * The caller provides the memory every rank can address (e.g. torch symmetric memory), as tables indexed by rank,
 * this rank's own entry included:
 *   recv[s][r]   f32  [recv_planes][batch / world][max row-parallel width]   partial sums, s = 0, 1 (consecutive exchanges alternate)
 *   act[s][r]    bf16 [batch][max row-parallel width]                  reduced activations / the result
 *   signals[r]   uint32[16], zeroed once before the first step (all ranks, then a barrier)
 *   x_in[r]      bf16 [batch][hidden[0]]  (optional; needed by gcb200_tp_mlp_execute)
 * batch must be a multiple of 128 and of 32 x world; every width a multiple of 8 x world.
 *
 * gcb200_tp_mlp_create     host only (no device needed): checks, fixes the tile configuration of the row-parallel layers.
 * gcb200_tp_mlp_describe   text form of the step: layers, counters, arrivals expected per step.
 * gcb200_tp_mlp_step       enqueues one step on `stream` for a device-resident input x [batch, hidden[0]] (the same
 *                          values on every rank); *result = this rank's copy of the [batch, hidden[layers]] output, valid
 *                          once the stream has run and until the step after the next.  The second call with the same
 *                          x captures the step into a CUDA graph; later calls replay it.
 * gcb200_tp_mlp_execute    the synchronous host-buffer form: this rank copies ITS row block of x_host (every rank
 *                          passes the same full array) to the device, the blocks are exchanged over NVLink, the
 *                          step runs, the whole result is copied to y_host (may be NULL on ranks that do not want
 *                          it), and the call returns when all of it has finished.
 * All ranks must issue the same sequence of steps; a rank that stops stepping makes the others' waits run out
 * (GCB200_DEVICE_TIMEOUT from gcb200_device_error, GCB200_CUDA_ERROR from gcb200_tp_mlp_execute). */
typedef struct gcb200_tp_mlp gcb200_tp_mlp;
typedef struct {
  int world, rank;
  int64_t batch;
  int layers;                    /* even, 2..12 */
  const int64_t *hidden;         /* layers + 1 full widths */
  const void *const *weights;    /* layers shards, bf16, device */
  const void *const *biases;     /* layers entries, bf16, device; NULL = no bias */
  int relu;
  void *const *recv[2];
  void *const *act[2];
  void *const *signals;
  void *const *x_in;             /* may be NULL */
  int recv_planes;               /* planes of [batch / world][width] f32 each recv buffer holds; 0 = world.  With 2 x world
                                    a rank whose share of K is long splits it once more (one plane per rank and split) */
} gcb200_tp_mlp_desc;
int gcb200_tp_mlp_create(const gcb200_tp_mlp_desc *desc, gcb200_tp_mlp **plan);
int gcb200_tp_mlp_destroy(gcb200_tp_mlp *plan);
int gcb200_tp_mlp_describe(const gcb200_tp_mlp *plan, int sm_count, char *buf, size_t cap, size_t *needed);
int gcb200_tp_mlp_step(gcb200_tp_mlp *plan, const void *x, void *stream, void **result);
int gcb200_tp_mlp_execute(gcb200_tp_mlp *plan, const void *x_host, void *y_host);
/* One step launched eagerly with a CUDA event behind every launch; writes one line per kernel ("<microseconds> us
 * <what>": the time from the end of the launch before to the end of this one, waits for other ranks included) and
 * the total.  Synchronises `stream`.  Every rank must call it (it is a step like any other). */
int gcb200_tp_mlp_timeline(gcb200_tp_mlp *plan, const void *x, void *stream, char *buf, size_t cap, size_t *needed);
/* Device-side time stamps of the plan's most recent step, written by the kernels themselves (so a replayed CUDA graph can
 * be read, which events cannot see into): one line per kernel with four times in microseconds after the step's first
 * kernel started - launched, released by the kernel ahead in the stream, cross-GPU wait over, last CTA done.  Only for a
 * plan whose first step ran with GC_B200_TP_TRACE=1 in the environment (an error otherwise).  Synchronises the device. */
int gcb200_tp_mlp_trace(gcb200_tp_mlp *plan, char *buf, size_t cap, size_t *needed);

/* Failure-path self-test: launches a kernel that waits (for at most `limit_cycles` SM clock cycles, which must not
 * exceed the library's own limit) on a counter nothing ever adds to, gives up, records code 7 in the device error
 * word and returns through its normal exit - the path every bounded wait of the kernels above takes when a peer or
 * a copy never answers.  The reference maps such a run-time failure to dnnl_runtime_error
 * (src/dnnl/dnnl_graph_compiler.cpp:217-225); the next dnnl_graph_compiler_execute on this device does the same once,
 * clears the word and later calls succeed.  Nothing faults, traps or hangs. */
int gcb200_wait_selftest(long long limit_cycles, void *stream);

/* ---------------------------------------------------------------------------
 * Split-K bf16 matmul that allocates nothing.  No counterpart in the reference
 * (its runtime allocates freely from FILO pools); added for hosts that cannot
 * let a library call cudaMalloc once they are running — a server that has given
 * all device memory to its own pool, a latency-critical thread that must not
 * take the driver's allocation lock, a runtime with a fixed memory budget.
 *
 *   Y = act( bf16( bf16(A . B) + bias ) ),  A [M,K], B [K,N], bias [N] or NULL, Y [M,N], bf16
 *
 * The f32 partial-sum planes (splits * M * N * 4 bytes) live in a 16 MiB array
 * that is part of the loaded module: every GPU that loads the library holds it
 * until exit.  Larger requests fail with GCB200_INVALID_ARGUMENT and a message
 * naming both sizes.  `splits` <= 0 lets the library choose (at least 2).
 * The array is shared by all calls and keeps the previous call's contents;
 * nothing in it needs clearing, since each split writes its plane in full before
 * the reduction reads it.  Calls that overlap on the GPU race on it: serialise
 * calls per device.  The first call on a device resolves the array's device
 * address and sets the kernel's shared-memory limit; issue it before starting
 * any stream capture.  Neither this function nor gcb200_static_error calls
 * cudaMalloc, cudaFree or any allocating routine.
 * gcb200_static_error reads (and clears when non-zero) the module-resident word
 * in which these kernels record a bounded wait that gave up. */
int gcb200_matmul_bf16_splitk_static(const void *A, const void *B, const void *bias, void *Y, int64_t M, int64_t N,
                                     int64_t K, int splits, int relu, void *stream);
int gcb200_static_error(void *stream, int *code);

/* ---------------------------------------------------------------------------
 * Microkernel runtime ABI of the reference
 * (include/gc/ExecutionEngine/CPURuntime/Microkernel/BrgemmInterface.h:31-63):
 * same names, argument meaning and units (elements); A, B, C are DEVICE
 * pointers here.  dtype codes are dnnl_data_type_t (bf16 = 2, f32 = 3, s8 = 5,
 * u8 = 6).  B is plain [K][LDB] for f32 and VNNI-packed for bf16
 * ([K/2][LDB][2]) and int8 ([K/4][LDB][4]), as in BrgemmNaive.cpp:71-140.
 * Calls are enqueued on the legacy default stream. */
int64_t dnnl_brgemm_dispatch(int64_t M, int64_t N, int64_t K, int64_t LDA, int64_t LDB, int64_t LDC, int64_t stride_a,
                             int64_t stride_b, float beta, int64_t dtypeA, int64_t dtypeB);
void dnnl_brgemm_tileconfig(int64_t kernel);
void dnnl_brgemm_tilerelease(void);
void dnnl_brgemm_execute(int64_t kernel, void *A, uint64_t A_offset, void *B, uint64_t B_offset, void *C,
                         uint64_t C_offset, int num);

#ifdef __cplusplus
}
#endif
#endif /* GC_B200_H */
