// Internal C++ interface of the CUDA runtime: per-device state (error word,
// workspace arena, SM count), tensor-map construction and the typed launchers
// the C ABI (include/gc_b200.h) and the graph executor call.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"

namespace gcb {

struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

#define GCB_CUDA(expr)                                                                           \
  do {                                                                                           \
    cudaError_t _e = (expr);                                                                     \
    if (_e != cudaSuccess)                                                                       \
      throw ::gcb::CudaError(std::string(#expr) + ": " + cudaGetErrorString(_e));                \
  } while (0)

// Per-device singleton.  Created on first use with that device current.
struct DeviceState {
  int device = -1;
  int sm_count = 0;
  int *d_error = nullptr;          // device word written by kernels on a bounded-wait time-out
  int *d_zero = nullptr;           // device word that stays zero (the wait self-test waits on it)
  // Split-K partial planes of the direct launchers (executables bring their own scratch).  ONE block per
  // device, shared by every stream and thread: launches that may split K and overlap on the GPU must be
  // serialised by the caller.  Growing it never frees the old block (see ensure_workspace).
  void *workspace = nullptr;
  size_t workspace_bytes = 0;
  unsigned long long workspace_generation = 0;   // bumped whenever a larger block replaces the workspace
  void *ensure_workspace(size_t bytes); // thread-safe; grows by allocating a larger block
};
DeviceState &device_state();       // throws CudaError when no usable device / driver

enum class ElemType : int { BF16 = 0, U8 = 1, S8 = 2, F32 = 3, S32 = 4 };

// 2-D row-major tensor map: `inner` contiguous elements per row, `outer` rows,
// `row_stride_bytes` between rows; 128-byte swizzle.
CUtensorMap make_tmap_2d(ElemType t, const void *ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                         uint32_t box_inner, uint32_t box_outer);

// --------------------------------------------------------------------------- tile selection
// The GPU counterpart of the reference's MatmulConfig (include/gc/Analysis/
// MatmulConfigAnalysis.h:25-34): instead of thread counts and cache-level
// block sizes it picks the MMA tile, operand orientation, split-K factor,
// pipeline depth and rasterisation group for one matmul shape.
struct MatmulConfig {
  int swapped;   // 1: weights take the MMA M side (small-batch / decode shapes)
  int bn;        // MMA N per tile
  int splits;    // split-K factor
  int stages;    // shared-memory pipeline depth
  int group_m;   // rasterisation group
  int grid;      // CTAs launched (persistent)
  int pair;      // 1: CTA-pair kernel (256 x bn tiles, two SMs per tile)
  int kpb;       // K blocks of 128 bytes per pipeline stage (0 or 1: one)
};
// dtype_bytes: 2 (bf16) or 1 (int8).  out_bytes: bytes per output element written by the GEMM kernel.
// max_splits < 8 restricts the K split (1: none - launches whose partial sums leave through peer stores); such a
// request is answered by the model alone.
MatmulConfig select_matmul_config(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count, int max_splits = 8);
// The fitted time model alone (select_matmul_config consults the measured configurations of tune_cache.h first).
MatmulConfig model_matmul_config(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count, int max_splits = 8);
// Bytes of f32 / s32 split-K partial planes the selected configuration of this shape needs (0: no split).
size_t matmul_scratch_bytes(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count);
// Whether the TMA path can take this operand layout (16-byte aligned base and row pitch).
bool tma_compatible(const void *ptr, int64_t row_elems, int elem_bytes);

// Shared-memory stage geometry and tensor map of one GEMM operand tile (`tile_mn` rows of the MMA
// M or N side; K contiguous in memory unless mn_major).
OperandGeom operand_geom(bool mn_major, int tile_mn, int elem_bytes, int kpb = 1);
// (sets g.one_load when the operand can be fetched with a single 3-D copy per stage)
CUtensorMap operand_tmap(OperandGeom &g, ElemType t, int elem_bytes, const void *ptr, int64_t mn_total,
                         int64_t k_total, int tile_mn, int kpb = 1);
CUtensorMap make_tmap_3d(ElemType t, const void *ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                         uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2);

// --------------------------------------------------------------------------- launchers
struct MatmulArgs {
  const void *A = nullptr;      // [M,K] row-major, or [K,M] when trans_a
  const void *B = nullptr;      // [K,N] row-major, or [N,K] when trans_b
  int64_t M = 0, N = 0, K = 0;
  int trans_a = 0, trans_b = 0;
  int int8 = 0;                 // 0: bf16 x bf16 -> f32;  1: u8 x s8 -> s32
  int out_kind = OUT_BF16;
  void *out = nullptr;
  int64_t ld_out = 0;           // 0 -> N
  int bias_kind = BIAS_NONE;
  const void *bias = nullptr;
  const float *scale = nullptr;
  const int32_t *comp = nullptr;
  int32_t *acc_dump = nullptr;
  int relu = 0;
  int n_peers = 0;              // > 0: push the f32 result into plane `peer_plane` of each peer buffer
  int peer_plane = 0;
  int peer_rows = 0;            // > 0: rows are scattered to their owner (row / peer_rows) instead of sent to every peer
  int peer_splits = 1;          // row scatter only: K splits of this launch, each with its own plane at the owner
                                // (plane = peer_plane * peer_splits + split; the owner's buffer holds n_peers * peer_splits planes)
  void *const *peer_out = nullptr;
  int peer_multicast = 0;       // 1: n_peers == 1 and peer_out[0] is an NVLink multicast address of all ranks' buffers
  const MatmulConfig *force = nullptr; // optional override
  void *scratch = nullptr;      // optional caller-provided split-K scratch (else the device workspace)
  size_t scratch_bytes = 0;
  // cross-GPU hand-off (see GemmParams): counters to add to after the row scatter, counter to wait for before loading
  uint32_t *const *signal_peer = nullptr;   // [n_peers], with peer_rows > 0 (rows per peer a multiple of 32)
  const uint32_t *wait_counter = nullptr;
  const uint32_t *epoch = nullptr;          // required with wait_counter
  uint32_t wait_per_step = 0;
  int *arrivals_per_peer = nullptr;         // out: counter increments each peer receives from this launch
  unsigned long long *trace = nullptr;      // optional device time stamps of this launch (four words, see sm100_ptx.cuh)
};
void matmul_tc(const MatmulArgs &a, cudaStream_t stream);

// reduce `nparts` f32 planes [M,N] (stride `plane` elements) then the bf16 epilogue
void reduce_epilogue_bf16(const float *parts, int nparts, int64_t plane, const void *bias_bf16, void *out_bf16,
                          int64_t M, int64_t N, int relu, cudaStream_t stream);
void reduce_planes(const void *parts, int nparts, int64_t plane, void *out, int64_t M, int64_t N, int out_kind,
                   int bias_kind, const void *bias, const float *scale, const int32_t *comp, int32_t *acc_dump,
                   int relu, cudaStream_t stream);
// comp[n] = zp * sum_k W[k,n]   (W s8 [K,N] row-major)
void colsum_s8(const int8_t *W, int32_t *comp, int64_t K, int64_t N, int32_t zp, cudaStream_t stream);

// Exact-order f32 SIMT matmul (k ascending, separate multiply and add) for f32
// graphs and for operand layouts TMA cannot address.  in_kind: 0 f32, 1 bf16.
void matmul_simt(const void *A, const void *B, const void *bias, void *out, int64_t M, int64_t N, int64_t K,
                 int trans_a, int trans_b, int in_kind, int relu, cudaStream_t stream);

int read_device_error(cudaStream_t stream); // synchronises the stream; returns and clears the error word

// Kernel launches issued by this library since load (every launcher counts its own).
// Sum `nparts` f32 planes of a [rows, N] slice in plane order, bias + ReLU + cast, and store the bf16 slice
// at row `row0` of the [*, N] result buffer of EVERY peer (plain stores; the all-gather half of an all-reduce).
void reduce_slice_broadcast_bf16(const float *parts, int nparts, int64_t rows, int64_t N, const void *bias_bf16,
                                 void *const *peer_out, int n_peers, int64_t row0, int relu, cudaStream_t stream);
void count_launch(int n = 1);
unsigned long long launch_count();

} // namespace gcb
