/*
 * dnnl_graph_compiler.h — the oneDNN-graph backend C API of Intel Graph Compiler,
 * re-created for the B200 backend.
 *
 * The reference implements these six entry points in src/dnnl/dnnl_graph_compiler.cpp
 * but takes their declarations from a header of a oneDNN fork
 * ("graph/backend/elyzor/include/dnnl_graph_compiler.h", included at
 * src/dnnl/dnnl_graph_compiler.cpp:35; fork fetched by cmake/onednn.cmake:5-9,
 * branch "dev", no commit pin), which is not part of the reference tree.  The
 * struct layouts below are the ones its call sites prove:
 *   - designated initialisers  {.num_threads = 4}                 test/dnnl/TestApiBasic.cpp:28
 *                              {.id, .ndims, .dims, .data}        test/dnnl/TestApiBasic.cpp:43-45
 *   - field uses  tensor->id / ndims / dims / data                src/dnnl/dnnl_graph_compiler.cpp:76,113-126
 *                 ctx->num_threads                                src/dnnl/dnnl_graph_compiler.cpp:174
 *                 v->api_version.{major,minor,patch,hash}         test/dnnl/TestApiBasic.cpp:60-79
 * Integer widths of num_threads / ndims / version numbers are inferred
 * (uint32_t / uint8_t / uint8_t: the version test compares against
 * std::numeric_limits<uint8_t>::max()).
 *
 * A maintainer switching the oneDNN graph backend to this library links
 * libGcDnnlApi.so built from this repository instead of the reference's
 * GcDnnlApi target; no call site changes.
 *
 * Differences in behaviour, all additive:
 *   - tensor `data` may be a HOST pointer (as in the reference; copied to and from
 *     the device by the call) or a DEVICE pointer (used in place, zero copy; the
 *     call first waits for all work previously queued on the device, on any stream);
 *   - the JSON may carry op kinds which the reference's front end cannot express:
 *     `QuantizedMatMul` (src u8 [M,K], weights s8 [K,N], scales f32 [N], optional bias
 *     f32 [N]; attr `src_zp` s64, optional `relu`; dst f32 [M,N] =
 *     float(acc - src_zp * colsum(W)) * scale + bias, optionally the raw s32 sums as a
 *     second output), `SDPA` (Q, K, V bf16 [B,H,S,128]; attrs `scale` f32, `causal`
 *     bool; O bf16), and `StaticReshape`, `Exp`, `Negate`;
 *   - `engine_kind` "gpu" is accepted besides "cpu".
 */
#ifndef DNNL_GRAPH_COMPILER_H
#define DNNL_GRAPH_COMPILER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* oneDNN status codes (oneapi/dnnl/dnnl_common_types.h); defined here only when
 * that header has not been included. */
#ifndef ONEAPI_DNNL_DNNL_COMMON_TYPES_H
typedef enum {
  dnnl_success = 0,
  dnnl_out_of_memory = 1,
  dnnl_invalid_arguments = 2,
  dnnl_unimplemented = 3,
  dnnl_last_impl_reached = 4,
  dnnl_runtime_error = 5,
  dnnl_not_required = 6,
  dnnl_invalid_graph = 7,
  dnnl_invalid_graph_op = 8,
  dnnl_invalid_shape = 9,
  dnnl_invalid_data_type = 10
} dnnl_status_t;
#define DNNL_MAX_NDIMS 12
#endif

#define DNNL_GC_API_V_MAJOR 0
#define DNNL_GC_API_V_MINOR 1
#define DNNL_GC_API_V_PATCH 0
#define DNNL_GC_API_V_HASH "N/A"

struct dnnl_graph_compiler;            /* opaque */
struct dnnl_graph_compiler_executable; /* opaque */

struct dnnl_graph_compiler_context {
  uint32_t num_threads; /* accepted for compatibility; the GPU backend ignores it */
};

struct dnnl_graph_compiler_tensor {
  size_t id;     /* logical tensor id of the JSON graph */
  uint8_t ndims;
  int64_t *dims;
  void *data;    /* host or device pointer */
};

struct dnnl_graph_compiler_version {
  struct {
    uint8_t major, minor, patch;
    const char *hash;
  } api_version, gc_version;
};

/* src/dnnl/dnnl_graph_compiler.cpp:157-167 */
const struct dnnl_graph_compiler_version *dnnl_graph_compiler_get_version(void);

/* src/dnnl/dnnl_graph_compiler.cpp:169-183 — ctx may be NULL. */
dnnl_status_t dnnl_graph_compiler_create(const struct dnnl_graph_compiler_context *ctx,
                                         const struct dnnl_graph_compiler **gc);

/* src/dnnl/dnnl_graph_compiler.cpp:185-188 */
void dnnl_graph_compiler_destroy(const struct dnnl_graph_compiler *gc);

/* src/dnnl/dnnl_graph_compiler.cpp:190-207 — parse the JSON partition, plan the
 * launch list and the workspace arena.  Malformed graph -> dnnl_invalid_graph;
 * unsupported op kind / dtype / engine / fpmath / layout -> dnnl_unimplemented. */
dnnl_status_t dnnl_graph_compiler_compile(const struct dnnl_graph_compiler *gc, const char *graph_json,
                                          const struct dnnl_graph_compiler_executable **exe);

/* src/dnnl/dnnl_graph_compiler.cpp:209-212 */
void dnnl_graph_compiler_destroy_executable(const struct dnnl_graph_compiler_executable *exe);

/* src/dnnl/dnnl_graph_compiler.cpp:214-226 — tensors are matched to the
 * partition's arguments by id; order may differ.  Returns after the results are
 * in `outputs` (host pointers) or enqueued-and-synchronised (device pointers). */
dnnl_status_t dnnl_graph_compiler_execute(const struct dnnl_graph_compiler_executable *exe,
                                          struct dnnl_graph_compiler_tensor *inputs,
                                          struct dnnl_graph_compiler_tensor *outputs);

#ifdef __cplusplus
}
#endif
#endif /* DNNL_GRAPH_COMPILER_H */
