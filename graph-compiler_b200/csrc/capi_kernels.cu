// extern "C" launchers declared in include/gc_b200.h, and the device-pointer
// implementation of the reference's microkernel runtime ABI (dnnl_brgemm_*).
#include <mutex>
#include <type_traits>
#include <shared_mutex>
#include <string>
#include <vector>

#include "../../include/gc_b200.h"
#include "runtime.h"
#include "tune_cache.h"
#include "sm100_ptx.cuh"

#define GCB_EXPORT extern "C" __attribute__((visibility("default")))

namespace gcb {

thread_local std::string g_last_error;

int guard_status(const std::exception_ptr &ep) {
  try {
    std::rethrow_exception(ep);
  } catch (const CudaError &e) {
    g_last_error = e.what();
    return g_last_error.rfind("no CUDA device", 0) == 0 || g_last_error.rfind("this library is built", 0) == 0
               ? GCB200_NO_DEVICE
               : GCB200_CUDA_ERROR;
  } catch (const std::invalid_argument &e) {
    g_last_error = e.what();
    return GCB200_INVALID_ARGUMENT;
  } catch (const std::logic_error &e) {
    g_last_error = e.what();
    return GCB200_UNIMPLEMENTED;
  } catch (const std::exception &e) {
    g_last_error = e.what();
    return GCB200_CUDA_ERROR;
  }
}

template <class F> static int guarded(F &&f) {
  try {
    f();
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}

static void require(bool ok, const char *msg) {
  if (!ok) throw std::invalid_argument(msg);
}

// bf16 matmul: tensor-core path when TMA can address both operands, else the
// exact-order SIMT kernel (same numerics, no alignment demands).
static void matmul_bf16_any(const void *A, const void *B, const void *bias, void *Y, int64_t M, int64_t N, int64_t K,
                            int ta, int tb, int relu, const MatmulConfig *force, cudaStream_t s) {
  require(A && B && Y, "null tensor pointer");
  require(M > 0 && N > 0 && K > 0, "matmul dimensions must be positive");
  const bool ok = tma_compatible(A, ta ? M : K, 2) && tma_compatible(B, tb ? K : N, 2);
  if (!ok) {
    matmul_simt(A, B, bias, Y, M, N, K, ta, tb, 1, relu, s);
    return;
  }
  MatmulArgs a;
  a.A = A; a.B = B; a.M = M; a.N = N; a.K = K; a.trans_a = ta; a.trans_b = tb;
  a.out_kind = OUT_BF16; a.out = Y;
  a.bias_kind = bias ? BIAS_BF16 : BIAS_NONE; a.bias = bias; a.relu = relu;
  a.force = force;
  matmul_tc(a, s);
}

} // namespace gcb

using namespace gcb;

GCB_EXPORT const char *gcb200_last_error(void) { return g_last_error.c_str(); }

GCB_EXPORT int gcb200_device_error(void *stream, int *code) {
  return guarded([&] {
    require(code != nullptr, "code is null");
    *code = read_device_error(static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_launch_count(uint64_t *count) {
  if (!count) return GCB200_INVALID_ARGUMENT;
  *count = launch_count();
  return GCB200_OK;
}

GCB_EXPORT int gcb200_sm_count(int *count) {
  return guarded([&] {
    require(count != nullptr, "count is null");
    *count = device_state().sm_count;
  });
}

GCB_EXPORT int gcb200_matmul_bf16(const void *A, const void *B, const void *bias, void *Y, int64_t M, int64_t N,
                                  int64_t K, int transpose_a, int transpose_b, int relu, void *stream) {
  return guarded([&] {
    matmul_bf16_any(A, B, bias, Y, M, N, K, transpose_a, transpose_b, relu, nullptr, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_bf16_cfg(const void *A, const void *B, const void *bias, void *Y, int64_t M, int64_t N,
                                      int64_t K, int transpose_a, int transpose_b, int relu,
                                      const gcb200_matmul_config *cfg, void *stream) {
  return guarded([&] {
    require(cfg != nullptr, "cfg is null");
    require(cfg->bn >= 16 && cfg->bn <= 256 && cfg->bn % 16 == 0, "bn must be a multiple of 16 in [16,256]");
    require(cfg->swapped || cfg->bn >= 64, "row-major tiles need bn >= 64");
    require(!cfg->pair || (!cfg->swapped && cfg->bn % 32 == 0), "the CTA-pair kernel needs bn a multiple of 32 (each CTA stages half the columns) and the row-major orientation");
    require(cfg->stages >= 2 && cfg->stages <= 8, "stages must be in [2,8]");
    require(cfg->splits >= 1 && cfg->group_m >= 1, "splits and group_m must be positive");
    MatmulConfig c{cfg->swapped, cfg->bn, cfg->splits, cfg->stages, cfg->group_m, cfg->grid, cfg->pair, cfg->kpb};
    const int kb = int((K + 63) / 64);
    const int per = (kb + c.splits - 1) / c.splits;
    c.splits = (kb + per - 1) / per;
    matmul_bf16_any(A, B, bias, Y, M, N, K, transpose_a, transpose_b, relu, &c, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_bf16_f32out(const void *A, const void *B, float *Y, int64_t M, int64_t N, int64_t K,
                                         int transpose_a, int transpose_b, void *stream) {
  return guarded([&] {
    require(A && B && Y, "null tensor pointer");
    require(M > 0 && N > 0 && K > 0, "matmul dimensions must be positive");
    if (!(tma_compatible(A, transpose_a ? M : K, 2) && tma_compatible(B, transpose_b ? K : N, 2)))
      throw std::logic_error("f32-out matmul needs 16-byte aligned operand rows");
    MatmulArgs a;
    a.A = A; a.B = B; a.M = M; a.N = N; a.K = K; a.trans_a = transpose_a; a.trans_b = transpose_b;
    a.out_kind = OUT_F32; a.out = Y;
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_bf16_f32out_push(const void *A, const void *B, void *const *peer_bufs, int n_peers, int my_plane,
                                              int64_t M, int64_t N, int64_t K, void *stream) {
  return guarded([&] {
    require(A && B && peer_bufs && n_peers >= 1 && n_peers <= 8 && my_plane >= 0, "bad arguments");
    require(M > 0 && N > 0 && K > 0, "matmul dimensions must be positive");
    for (int d = 0; d < n_peers; ++d) require(peer_bufs[d] && (reinterpret_cast<uintptr_t>(peer_bufs[d]) & 15) == 0, "peer buffers must be 16-byte aligned");
    if (!(tma_compatible(A, K, 2) && tma_compatible(B, N, 2))) throw std::logic_error("push matmul needs 16-byte aligned operand rows");
    MatmulArgs a;
    a.A = A; a.B = B; a.M = M; a.N = N; a.K = K;
    a.out_kind = OUT_F32; a.out = peer_bufs[0];
    a.n_peers = n_peers; a.peer_plane = my_plane; a.peer_out = peer_bufs;
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

// The three peer-store forms with ONE multicast address instead of a list of peer addresses (see the header).
GCB_EXPORT int gcb200_matmul_bf16_f32out_push_mc(const void *A, const void *B, void *mc_buf, int my_plane, int64_t M, int64_t N,
                                                 int64_t K, void *stream) {
  return guarded([&] {
    require(A && B && mc_buf && my_plane >= 0 && (reinterpret_cast<uintptr_t>(mc_buf) & 15) == 0, "bad arguments");
    require(M > 64 && N > 0 && K > 0, "multicast push needs M > 64 and positive N, K");
    if (!(tma_compatible(A, K, 2) && tma_compatible(B, N, 2))) throw std::logic_error("push matmul needs 16-byte aligned operand rows");
    void *const one[1] = {mc_buf};
    MatmulArgs a;
    a.A = A; a.B = B; a.M = M; a.N = N; a.K = K;
    a.out_kind = OUT_F32; a.out = mc_buf;
    a.n_peers = 1; a.peer_plane = my_plane; a.peer_out = one; a.peer_multicast = 1;
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_bf16_allgather_mc(const void *A, const void *B, const void *bias, void *mc_C, int64_t M, int64_t N,
                                               int64_t K, int64_t ldc, int transpose_a, int transpose_b, int relu, void *stream) {
  return guarded([&] {
    require(A && B && mc_C && (reinterpret_cast<uintptr_t>(mc_C) & 15) == 0, "bad arguments");
    require(M > 64 && N > 0 && K > 0 && ldc >= N, "multicast all-gather matmul needs M > 64, positive N, K and ldc >= N");
    if (!(tma_compatible(A, transpose_a ? M : K, 2) && tma_compatible(B, transpose_b ? K : N, 2)))
      throw std::logic_error("all-gather matmul needs 16-byte aligned operand rows");
    void *const one[1] = {mc_C};
    MatmulArgs a;
    a.A = A; a.B = B; a.M = M; a.N = N; a.K = K; a.trans_a = transpose_a; a.trans_b = transpose_b;
    a.out_kind = OUT_BF16; a.out = mc_C; a.ld_out = ldc;
    a.bias_kind = bias ? BIAS_BF16 : BIAS_NONE; a.bias = bias; a.relu = relu;
    a.n_peers = 1; a.peer_out = one; a.peer_multicast = 1;
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_u8s8_allgather_mc(const void *A, const void *W, const float *scale, const float *bias,
                                               const int32_t *comp, void *mc_C, int64_t M, int64_t N, int64_t K, int64_t ldc,
                                               int transpose_b, void *stream) {
  return guarded([&] {
    require(A && W && scale && mc_C && (reinterpret_cast<uintptr_t>(mc_C) & 15) == 0, "bad arguments");
    require(M > 64 && N > 0 && K > 0 && ldc >= N, "multicast all-gather matmul needs M > 64, positive N, K and ldc >= N");
    if (!(tma_compatible(A, K, 1) && tma_compatible(W, transpose_b ? K : N, 1)))
      throw std::logic_error("int8 matmul needs K and N to be multiples of 16 and 16-byte aligned bases");
    void *const one[1] = {mc_C};
    MatmulArgs a;
    a.A = A; a.B = W; a.M = M; a.N = N; a.K = K; a.int8 = 1; a.trans_b = transpose_b;
    a.out_kind = OUT_DEQUANT_F32; a.out = mc_C; a.ld_out = ldc; a.scale = scale; a.comp = comp;
    a.bias_kind = bias ? BIAS_F32 : BIAS_NONE; a.bias = bias;
    a.n_peers = 1; a.peer_out = one; a.peer_multicast = 1;
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_bf16_f32out_scatter(const void *A, const void *B, void *const *peer_bufs, int n_peers, int my_plane,
                                                 int64_t M, int64_t N, int64_t K, void *stream) {
  return guarded([&] {
    require(A && B && peer_bufs && n_peers >= 1 && n_peers <= 8 && my_plane >= 0, "bad arguments");
    require(M > 0 && N > 0 && K > 0 && M % n_peers == 0, "M must be a positive multiple of the number of peers");
    for (int d = 0; d < n_peers; ++d) require(peer_bufs[d] && (reinterpret_cast<uintptr_t>(peer_bufs[d]) & 15) == 0, "peer buffers must be 16-byte aligned");
    if (!(tma_compatible(A, K, 2) && tma_compatible(B, N, 2))) throw std::logic_error("scatter matmul needs 16-byte aligned operand rows");
    MatmulArgs a;
    a.A = A; a.B = B; a.M = M; a.N = N; a.K = K;
    a.out_kind = OUT_F32; a.out = peer_bufs[0];
    a.n_peers = n_peers; a.peer_plane = my_plane; a.peer_out = peer_bufs; a.peer_rows = int(M / n_peers);
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_reduce_slice_broadcast_bf16(const float *parts, int nparts, int64_t rows, int64_t N, const void *bias,
                                                  void *const *peer_out, int n_peers, int64_t row0, int relu, void *stream) {
  return guarded([&] {
    require(parts && peer_out, "bad arguments");
    reduce_slice_broadcast_bf16(parts, nparts, rows, N, bias, peer_out, n_peers, row0, relu, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_reduce_bias_act_bf16(const float *parts, int nparts, int64_t plane_stride, const void *bias,
                                           void *Y, int64_t M, int64_t N, int relu, void *stream) {
  return guarded([&] {
    require(parts && Y && nparts >= 1, "bad arguments");
    reduce_epilogue_bf16(parts, nparts, plane_stride, bias, Y, M, N, relu, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_u8s8(const void *A, const void *W, const float *scale, const float *bias,
                                  const int32_t *comp, float *out, int32_t *acc_out, int64_t M, int64_t N, int64_t K,
                                  int transpose_b, void *stream) {
  return guarded([&] {
    require(A && W && (out || acc_out), "null tensor pointer");
    require(!out || scale, "dequantised output needs scales");
    require(M > 0 && N > 0 && K > 0, "matmul dimensions must be positive");
    if (!(tma_compatible(A, K, 1) && tma_compatible(W, transpose_b ? K : N, 1)))
      throw std::logic_error("int8 matmul needs K and N to be multiples of 16 and 16-byte aligned bases");
    MatmulArgs a;
    a.A = A; a.B = W; a.M = M; a.N = N; a.K = K; a.int8 = 1; a.trans_b = transpose_b;
    if (out) {
      a.out_kind = OUT_DEQUANT_F32; a.out = out; a.scale = scale; a.comp = comp;
      a.bias_kind = bias ? BIAS_F32 : BIAS_NONE; a.bias = bias; a.acc_dump = acc_out;
    } else {
      a.out_kind = OUT_S32; a.out = acc_out;
    }
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_bf16_allgather(const void *A, const void *B, const void *bias, void *const *peer_C, int n_peers,
                                            int64_t M, int64_t N, int64_t K, int64_t ldc, int transpose_a, int transpose_b,
                                            int relu, void *stream) {
  return guarded([&] {
    require(A && B && peer_C && n_peers >= 1 && n_peers <= 8, "bad arguments");
    require(M > 0 && N > 0 && K > 0 && ldc >= N, "all-gather matmul needs positive M, N, K and ldc >= N");
    for (int d = 0; d < n_peers; ++d) require(peer_C[d] && (reinterpret_cast<uintptr_t>(peer_C[d]) & 15) == 0, "peer buffers must be 16-byte aligned");
    if (!(tma_compatible(A, transpose_a ? M : K, 2) && tma_compatible(B, transpose_b ? K : N, 2)))
      throw std::logic_error("all-gather matmul needs 16-byte aligned operand rows");
    MatmulArgs a;
    a.A = A; a.B = B; a.M = M; a.N = N; a.K = K; a.trans_a = transpose_a; a.trans_b = transpose_b;
    a.out_kind = OUT_BF16; a.out = peer_C[0]; a.ld_out = ldc;
    a.bias_kind = bias ? BIAS_BF16 : BIAS_NONE; a.bias = bias; a.relu = relu;
    a.n_peers = n_peers; a.peer_out = peer_C;
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_u8s8_allgather(const void *A, const void *W, const float *scale, const float *bias,
                                            const int32_t *comp, void *const *peer_C, int n_peers, int64_t M, int64_t N,
                                            int64_t K, int64_t ldc, int transpose_b, void *stream) {
  return guarded([&] {
    require(A && W && scale && peer_C && n_peers >= 1 && n_peers <= 8, "bad arguments");
    require(M > 0 && N > 0 && K > 0 && ldc >= N, "all-gather matmul needs positive M, N, K and ldc >= N");
    for (int d = 0; d < n_peers; ++d) require(peer_C[d] && (reinterpret_cast<uintptr_t>(peer_C[d]) & 15) == 0, "peer buffers must be 16-byte aligned");
    if (!(tma_compatible(A, K, 1) && tma_compatible(W, transpose_b ? K : N, 1)))
      throw std::logic_error("int8 matmul needs K and N to be multiples of 16 and 16-byte aligned bases");
    MatmulArgs a;
    a.A = A; a.B = W; a.M = M; a.N = N; a.K = K; a.int8 = 1; a.trans_b = transpose_b;
    a.out_kind = OUT_DEQUANT_F32; a.out = peer_C[0]; a.ld_out = ldc; a.scale = scale; a.comp = comp;
    a.bias_kind = bias ? BIAS_F32 : BIAS_NONE; a.bias = bias;
    a.n_peers = n_peers; a.peer_out = peer_C;
    matmul_tc(a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_colsum_s8(const void *W, int32_t *comp, int64_t K, int64_t N, int32_t zp_a, void *stream) {
  return guarded([&] {
    require(W && comp && K > 0 && N > 0, "bad arguments");
    device_state();
    colsum_s8(static_cast<const int8_t *>(W), comp, K, N, zp_a, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_matmul_f32(const float *A, const float *B, const float *bias, float *Y, int64_t M, int64_t N,
                                 int64_t K, int transpose_a, int transpose_b, int relu, void *stream) {
  return guarded([&] {
    require(A && B && Y && M > 0 && N > 0 && K > 0, "bad arguments");
    matmul_simt(A, B, bias, Y, M, N, K, transpose_a, transpose_b, 0, relu, static_cast<cudaStream_t>(stream));
  });
}

GCB_EXPORT int gcb200_select_matmul_config(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes,
                                           int sm_count, gcb200_matmul_config *cfg) {
  return guarded([&] {
    require(cfg && M > 0 && N > 0 && K > 0 && sm_count > 0, "bad arguments");
    require(dtype_bytes == 1 || dtype_bytes == 2, "dtype_bytes must be 1 or 2");
    MatmulConfig c = select_matmul_config(M, N, K, dtype_bytes, out_bytes, sm_count);
    *cfg = gcb200_matmul_config{c.swapped, c.bn, c.splits, c.stages, c.group_m, c.grid, c.pair, c.kpb};
  });
}

GCB_EXPORT int gcb200_model_matmul_config(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count,
                                          gcb200_matmul_config *cfg) {
  return guarded([&] {
    require(cfg && M > 0 && N > 0 && K > 0 && sm_count > 0, "bad arguments");
    require(dtype_bytes == 1 || dtype_bytes == 2, "dtype_bytes must be 1 or 2");
    MatmulConfig c = model_matmul_config(M, N, K, dtype_bytes, out_bytes, sm_count);
    *cfg = gcb200_matmul_config{c.swapped, c.bn, c.splits, c.stages, c.group_m, c.grid, c.pair, c.kpb};
  });
}

GCB_EXPORT int gcb200_tune_cache_put(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes,
                                     const gcb200_matmul_config *cfg) {
  return guarded([&] {
    require(cfg, "bad arguments");
    tune::put(tune::Key{M, N, K, dtype_bytes, out_bytes},
              MatmulConfig{cfg->swapped, cfg->bn, cfg->splits, cfg->stages, cfg->group_m, cfg->grid, cfg->pair, cfg->kpb});
  });
}

GCB_EXPORT int gcb200_tune_cache_get(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, gcb200_matmul_config *cfg,
                                     int *found) {
  return guarded([&] {
    require(cfg && found, "bad arguments");
    MatmulConfig c{};
    *found = tune::lookup(tune::Key{M, N, K, dtype_bytes, out_bytes}, &c) ? 1 : 0;
    if (*found) *cfg = gcb200_matmul_config{c.swapped, c.bn, c.splits, c.stages, c.group_m, c.grid, c.pair, c.kpb};
  });
}

GCB_EXPORT int gcb200_tune_cache_load(const char *path, int *entries_read) {
  return guarded([&] {
    require(path, "bad arguments");
    const int n = tune::load(path);
    if (entries_read) *entries_read = n;
  });
}

GCB_EXPORT int gcb200_tune_cache_save(const char *path, int *entries_written) {
  return guarded([&] {
    require(path, "bad arguments");
    const int n = tune::save(path);
    if (entries_written) *entries_written = n;
  });
}

GCB_EXPORT int gcb200_tune_cache_erase(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes) {
  return guarded([&] { tune::erase(tune::Key{M, N, K, dtype_bytes, out_bytes}); });
}

GCB_EXPORT int gcb200_tune_cache_clear(void) {
  return guarded([&] { tune::clear(); });
}

// ----------------------------------------------------------------------------- brgemm runtime ABI
namespace {

struct BrgemmDesc {
  int64_t M, N, K, LDA, LDB, LDC, stride_a, stride_b;
  float beta;
  int64_t dtA, dtB;
};
std::shared_mutex g_brgemm_lock;
std::vector<BrgemmDesc> g_brgemm;

enum : int64_t { DT_BF16 = 2, DT_F32 = 3, DT_S8 = 5, DT_U8 = 6 };

// One thread per C element; batch ascending then k ascending, separate multiply
// and add — the accumulation chain of BrgemmNaive.cpp:46-140, so f32 results are
// bit-identical to the reference's naive kernel.
template <typename TA, typename TB, typename TC, int VNNI>
__global__ void brgemm_kernel(BrgemmDesc d, const TA *A, const TB *B, TC *C, int num) {
  const int64_t n = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  const int64_t m = blockIdx.y * int64_t(blockDim.y) + threadIdx.y;
  if (m >= d.M || n >= d.N) return;
  // beta == 0 clears a dense M*N block at C (BrgemmNaive.cpp:36-44) — with LDC == N this is the tile itself
  TC acc = (d.beta == 0.0f) ? TC(0) : C[m * d.LDC + n];
  for (int b = 0; b < num; ++b) {
    const TA *a = A + b * d.stride_a + m * d.LDA;
    const TB *bb = B + b * d.stride_b;
    for (int64_t k = 0; k < d.K; ++k) {
      const int64_t kv = k - k % VNNI;
      const TB bv = bb[kv * d.LDB + VNNI * n + (k % VNNI)];
      if constexpr (sizeof(TC) == 4 && std::is_same<TC, float>::value) {
        float af, bf;
        if constexpr (sizeof(TA) == 2) { af = bf16_bits_to_f32(a[k]); bf = bf16_bits_to_f32(bv); }
        else { af = a[k]; bf = bv; }
        acc = __fadd_rn(acc, __fmul_rn(af, bf));
      } else {
        acc += int32_t(a[k]) * int32_t(bv);
      }
    }
  }
  C[m * d.LDC + n] = acc;
}

template <typename TA, typename TB, typename TC, int VNNI>
void launch_brgemm(const BrgemmDesc &d, void *A, uint64_t Ao, void *B, uint64_t Bo, void *C, uint64_t Co, int num) {
  dim3 block(32, 8), grid(unsigned((d.N + 31) / 32), unsigned((d.M + 7) / 8));
  brgemm_kernel<TA, TB, TC, VNNI><<<grid, block>>>(d, static_cast<const TA *>(A) + Ao, static_cast<const TB *>(B) + Bo,
                                                   static_cast<TC *>(C) + Co, num);
}

} // namespace

GCB_EXPORT int64_t dnnl_brgemm_dispatch(int64_t M, int64_t N, int64_t K, int64_t LDA, int64_t LDB, int64_t LDC,
                                        int64_t stride_a, int64_t stride_b, float beta, int64_t dtypeA,
                                        int64_t dtypeB) {
  std::unique_lock<std::shared_mutex> g(g_brgemm_lock);
  g_brgemm.push_back(BrgemmDesc{M, N, K, LDA, LDB, LDC, stride_a, stride_b, beta, dtypeA, dtypeB});
  return int64_t(g_brgemm.size()) - 1;
}

GCB_EXPORT void dnnl_brgemm_tileconfig(int64_t) {}
GCB_EXPORT void dnnl_brgemm_tilerelease(void) {}

GCB_EXPORT void dnnl_brgemm_execute(int64_t kernel, void *A, uint64_t A_offset, void *B, uint64_t B_offset, void *C,
                                    uint64_t C_offset, int num) {
  BrgemmDesc d;
  {
    std::shared_lock<std::shared_mutex> g(g_brgemm_lock);
    if (kernel < 0 || kernel >= int64_t(g_brgemm.size())) {
      g_last_error = "dnnl_brgemm_execute: invalid kernel handle";
      return;
    }
    d = g_brgemm[size_t(kernel)];
  }
  int rc = guarded([&] {
    device_state();
    if (d.dtA == DT_F32 && d.dtB == DT_F32) launch_brgemm<float, float, float, 1>(d, A, A_offset, B, B_offset, C, C_offset, num);
    else if (d.dtA == DT_BF16 && d.dtB == DT_BF16) launch_brgemm<uint16_t, uint16_t, float, 2>(d, A, A_offset, B, B_offset, C, C_offset, num);
    else if (d.dtA == DT_U8 && d.dtB == DT_S8) launch_brgemm<uint8_t, int8_t, int32_t, 4>(d, A, A_offset, B, B_offset, C, C_offset, num);
    else if (d.dtA == DT_S8 && d.dtB == DT_S8) launch_brgemm<int8_t, int8_t, int32_t, 4>(d, A, A_offset, B, B_offset, C, C_offset, num);
    else if (d.dtA == DT_S8 && d.dtB == DT_U8) launch_brgemm<int8_t, uint8_t, int32_t, 4>(d, A, A_offset, B, B_offset, C, C_offset, num);
    else if (d.dtA == DT_U8 && d.dtB == DT_U8) launch_brgemm<uint8_t, uint8_t, int32_t, 4>(d, A, A_offset, B, B_offset, C, C_offset, num);
    else throw std::logic_error("dnnl_brgemm_execute: unsupported dtype pair");
    GCB_CUDA(cudaGetLastError());
    count_launch();
  });
  (void)rc;
}

#include "attention.h"
GCB_EXPORT int gcb200_attention_bf16(const void *Q, const void *K, const void *V, void *O, int64_t batch_heads,
                                     int64_t seq, int64_t head_dim, float scale, int causal, void *stream) {
  return guarded([&] {
    require(Q && K && V && O && batch_heads > 0 && seq > 0 && head_dim > 0, "bad arguments");
    device_state();
    attention_bf16(Q, K, V, O, batch_heads, seq, head_dim, scale, causal, static_cast<cudaStream_t>(stream));
  });
}
