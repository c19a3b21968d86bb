// CPU oracle for the matmul / MLP / attention path of Intel Graph Compiler.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain scalar C++, the
// arithmetic that the reference CPU pipeline performs for the partitions the
// CUDA backend accelerates.  It is the checker for the parity tests, the
// smoke test and the CPU-baseline leg of the benchmark; nothing in the product
// library links, loads or calls it.
//
// Pinning: every function below is checked (tests/test_oracle_*.py) against
//   * the reference's own naive brgemm, lib/gc/ExecutionEngine/CPURuntime/
//     Microkernel/BrgemmNaive.cpp, compiled unmodified into oracle/_ref/
//     (f32, bf16-VNNI and the four int8 combinations, beta 0 and 1);
//   * the closed-form tiles of test/mlir/test/gc/cpu-runner/brgemm-*.mlir;
//   * the triple-loop expectation of test/dnnl/TestApiOps.cpp:69-119.
// Per-channel int8 dequantisation and attention have no test in the reference:
// for those two functions parity is UNPINNED beyond the s32 accumulator and the
// softmax definition respectively.
//
// Build: see oracle/Makefile (g++ -O3 -mavx2 -ffp-contract=off -fopenmp).
// -ffp-contract=off matters: the reference computes mul then add in f32.

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define GCO_API extern "C" __attribute__((visibility("default")))

namespace {

// dnnl_data_type_t codes used at the brgemm ABI
// (include/gc/ExecutionEngine/CPURuntime/Microkernel/BrgemmInterface.h:31-63).
enum : int64_t { DT_F16 = 1, DT_BF16 = 2, DT_F32 = 3, DT_S32 = 4, DT_S8 = 5, DT_U8 = 6 };

inline float bf16_to_f32(uint16_t v) {
  // BrgemmInterface.h:72-76 — widening is a 16-bit shift.
  uint32_t u = uint32_t(v) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

inline uint16_t f32_to_bf16(float f) {
  // BrgemmInterface.h:83-92 — round to nearest even, NaN -> 0x7FC0.
  if (std::isnan(f)) return 0x7FC0;
  uint32_t u;
  std::memcpy(&u, &f, 4);
  uint32_t bias = ((u >> 16) & 1u) + 0x7FFFu;
  return uint16_t((u + bias) >> 16);
}

inline bool is_int8(int64_t dt) { return dt == DT_S8 || dt == DT_U8; }

template <typename TA, typename TB>
void brgemm_int8(int64_t M, int64_t N, int64_t K, int64_t LDA, int64_t LDB, int64_t LDC,
                 int64_t sa, int64_t sb, const TA *A, const TB *B, int32_t *C, int num) {
  // BrgemmNaive.cpp:102-140 — B is VNNI [K/4][N][4]; a K tail shorter than 4
  // reads only the existing slots.
  for (int b = 0; b < num; ++b) {
    for (int64_t m = 0; m < M; ++m)
      for (int64_t n = 0; n < N; ++n) {
        int32_t acc = C[m * LDC + n];
        for (int64_t k = 0; k < K; ++k) {
          int64_t k4 = k & ~int64_t(3), r = k & 3;
          acc += int32_t(A[m * LDA + k]) * int32_t(B[k4 * LDB + 4 * n + r]);
        }
        C[m * LDC + n] = acc;
      }
    A += sa;
    B += sb;
  }
}

} // namespace

// ---------------------------------------------------------------------------
// scalar conversions (exposed so that tests can pin them)
// ---------------------------------------------------------------------------
GCO_API uint16_t gco_f32_to_bf16(float f) { return f32_to_bf16(f); }
GCO_API float gco_bf16_to_f32(uint16_t v) { return bf16_to_f32(v); }

GCO_API void gco_f32_to_bf16_array(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}
GCO_API void gco_bf16_to_f32_array(const uint16_t *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

// ---------------------------------------------------------------------------
// brgemm microkernel, restated.  Follows BrgemmNaive.cpp:46-140,158-209:
//   if beta == 0: C = 0;  for b < num: C[m,n] += sum_k A_b[m,k] * B_b[k,n]
// Units are elements.  f32: B plain [K][LDB].  bf16: B VNNI [K/2][LDB][2].
// int8: B VNNI [K/4][LDB][4].  Accumulation order per element: batch
// ascending, k ascending — the same as the reference.
// ---------------------------------------------------------------------------
GCO_API int gco_brgemm(int64_t M, int64_t N, int64_t K, int64_t LDA, int64_t LDB, int64_t LDC,
                       int64_t stride_a, int64_t stride_b, float beta, int64_t dtA, int64_t dtB,
                       const void *A, uint64_t A_off, const void *B, uint64_t B_off, void *C,
                       uint64_t C_off, int num) {
  const bool i8 = is_int8(dtA) && is_int8(dtB);
  const bool fl = (dtA == DT_F32 && dtB == DT_F32) || (dtA == DT_BF16 && dtB == DT_BF16);
  if (!i8 && !fl) return -1;
  if (beta == 0.0f) {
    // BrgemmNaive.cpp:36-44,169-180: a dense M*N block is cleared, not an
    // LDC-strided one.
    if (i8) {
      int32_t *c = (int32_t *)C + C_off;
      for (int64_t i = 0; i < M * N; ++i) c[i] = 0;
    } else {
      float *c = (float *)C + C_off;
      for (int64_t i = 0; i < M * N; ++i) c[i] = 0.f;
    }
  }
  if (dtA == DT_F32) {
    const float *a = (const float *)A + A_off, *b = (const float *)B + B_off;
    float *c = (float *)C + C_off;
    for (int i = 0; i < num; ++i) {
      for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
          float acc = c[m * LDC + n];
          for (int64_t k = 0; k < K; ++k) acc += a[m * LDA + k] * b[k * LDB + n];
          c[m * LDC + n] = acc;
        }
      a += stride_a;
      b += stride_b;
    }
  } else if (dtA == DT_BF16) {
    const uint16_t *a = (const uint16_t *)A + A_off, *b = (const uint16_t *)B + B_off;
    float *c = (float *)C + C_off;
    for (int i = 0; i < num; ++i) {
      for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
          float acc = c[m * LDC + n];
          for (int64_t k = 0; k < K; ++k) {
            int64_t k2 = k & ~int64_t(1), r = k & 1;
            acc += bf16_to_f32(a[m * LDA + k]) * bf16_to_f32(b[k2 * LDB + 2 * n + r]);
          }
          c[m * LDC + n] = acc;
        }
      a += stride_a;
      b += stride_b;
    }
  } else {
    int32_t *c = (int32_t *)C + C_off;
    if (dtA == DT_U8 && dtB == DT_S8)
      brgemm_int8(M, N, K, LDA, LDB, LDC, stride_a, stride_b, (const uint8_t *)A + A_off,
                  (const int8_t *)B + B_off, c, num);
    else if (dtA == DT_S8 && dtB == DT_S8)
      brgemm_int8(M, N, K, LDA, LDB, LDC, stride_a, stride_b, (const int8_t *)A + A_off,
                  (const int8_t *)B + B_off, c, num);
    else if (dtA == DT_S8 && dtB == DT_U8)
      brgemm_int8(M, N, K, LDA, LDB, LDC, stride_a, stride_b, (const int8_t *)A + A_off,
                  (const uint8_t *)B + B_off, c, num);
    else
      brgemm_int8(M, N, K, LDA, LDB, LDC, stride_a, stride_b, (const uint8_t *)A + A_off,
                  (const uint8_t *)B + B_off, c, num);
  }
  return 0;
}

// Pack a row-major [K][N] matrix into the VNNI layout [ceil(K/v)][N][v] that
// the bf16 (v=2) and int8 (v=4) microkernels read
// (lib/gc/Dialect/Linalgx/Utils.cpp:317-324).  Padding slots are zero.
GCO_API void gco_pack_vnni(const void *src, void *dst, int64_t K, int64_t N, int64_t ld_src,
                           int elem_size, int v) {
  const uint8_t *s = (const uint8_t *)src;
  uint8_t *d = (uint8_t *)dst;
  int64_t Kp = (K + v - 1) / v;
  std::memset(d, 0, size_t(Kp) * N * v * elem_size);
  for (int64_t k = 0; k < K; ++k)
    for (int64_t n = 0; n < N; ++n)
      std::memcpy(d + ((k / v) * N * v + n * v + (k % v)) * elem_size, s + (k * ld_src + n) * elem_size,
                  elem_size);
}

// ---------------------------------------------------------------------------
// Deep-tiled matmul, restated.  lib/gc/Transforms/DeepTileContractionOp.cpp:
// the (M,N) output is cut into innermost blocks (32 when the dimension is a
// multiple of 32, else the whole dimension — MatmulConfigAnalysis.cpp:465-468);
// for every output block the K blocks are visited in ascending order
// (:603-638), each visit is one brgemm call that accumulates in f32 (:152-235),
// the first visit starts from zero (:900-946).  The (m,k,n) loop order below
// gives every output element exactly that k-ascending accumulation chain while
// letting the compiler vectorise over n.
// ---------------------------------------------------------------------------
static void acc_f32_from_bf16(const uint16_t *A, const uint16_t *B, float *acc, int64_t M, int64_t N,
                              int64_t K, int transA, int transB) {
  // A: [M,K] (or [K,M] when transA); B: [K,N] (or [N,K] when transB)
  // (lib/gc/Transforms/OneDNNGraphToLinalg.cpp:421-480: transposes are part of
  // the matmul op, not separate copies with extra rounding).
  std::vector<float> Bf(size_t(K) * N);
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < K; ++k)
    for (int64_t n = 0; n < N; ++n)
      Bf[k * N + n] = bf16_to_f32(transB ? B[n * K + k] : B[k * N + n]);
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float *c = acc + m * N;
    for (int64_t n = 0; n < N; ++n) c[n] = 0.f;
    for (int64_t k = 0; k < K; ++k) {
      float a = bf16_to_f32(transA ? A[k * M + m] : A[m * K + k]);
      const float *b = Bf.data() + k * N;
      for (int64_t n = 0; n < N; ++n) c[n] += a * b[n];
    }
  }
}

// One bf16 linear layer: Y = act(bf16(bf16(A.W) + bias)).
//   acc  : f32 accumulate of exact bf16 products, k ascending
//   y0   : single RNE cast at the last K block (DeepTileContractionOp.cpp:872-889)
//   y1   : bias add is a bf16 linalg.add that the pipeline evaluates as
//          extf, addf(f32), truncf (lib/gc/Transforms/Pipeline.cpp:81-90)
//   relu : linalg.max(x, 0) (OneDNNGraphToLinalg.cpp:355-358)
// acc_out (optional) receives the f32 accumulators.
GCO_API void gco_linear_bf16(const uint16_t *A, const uint16_t *W, const uint16_t *bias, uint16_t *Y,
                             int64_t M, int64_t N, int64_t K, int transA, int transB, int relu,
                             float *acc_out) {
  std::vector<float> tmp;
  float *acc = acc_out;
  if (!acc) {
    tmp.resize(size_t(M) * N);
    acc = tmp.data();
  }
  acc_f32_from_bf16(A, W, acc, M, N, K, transA, transB);
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      uint16_t y = f32_to_bf16(acc[m * N + n]);
      if (bias) y = f32_to_bf16(bf16_to_f32(y) + bf16_to_f32(bias[n]));
      if (relu) {
        float f = bf16_to_f32(y);
        // arith.maximumf(x, 0): NaN propagates, -0 -> +0
        if (!(f != f)) y = f > 0.f ? y : uint16_t(0);
      }
      Y[m * N + n] = y;
    }
}

// Epilogue alone, applied to f32 sums that were reduced elsewhere (the
// K-split rule of DeepTileContractionOp.cpp:446-471,988-996: partial sums stay
// f32, are added, and only then cast).  parts = [nparts][M*N].
GCO_API void gco_reduce_epilogue_bf16(const float *parts, int nparts, const uint16_t *bias, uint16_t *Y,
                                      int64_t M, int64_t N, int relu) {
  for (int64_t i = 0; i < M * N; ++i) {
    float s = parts[i];
    for (int p = 1; p < nparts; ++p) s += parts[size_t(p) * M * N + i];
    uint16_t y = f32_to_bf16(s);
    if (bias) y = f32_to_bf16(bf16_to_f32(y) + bf16_to_f32(bias[i % N]));
    if (relu) {
      float f = bf16_to_f32(y);
      if (!(f != f)) y = f > 0.f ? y : uint16_t(0);
    }
    Y[i] = y;
  }
}

// f32 matmul (+bias) — the form test/dnnl/TestApiOps.cpp:69-119 exercises.
// Accumulation starts from zero, k ascending; bias is added afterwards as a
// separate linalg.add (OneDNNGraphToLinalg.cpp:484-494).
GCO_API void gco_matmul_f32(const float *A, const float *B, const float *bias, float *Y, int64_t M,
                            int64_t N, int64_t K, int transA, int transB, int relu) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float *c = Y + m * N;
    for (int64_t n = 0; n < N; ++n) c[n] = 0.f;
    for (int64_t k = 0; k < K; ++k) {
      float a = transA ? A[k * M + m] : A[m * K + k];
      if (!transB) {
        const float *b = B + k * N;
        for (int64_t n = 0; n < N; ++n) c[n] += a * b[n];
      } else {
        for (int64_t n = 0; n < N; ++n) c[n] += a * B[n * K + k];
      }
    }
    for (int64_t n = 0; n < N; ++n) {
      float v = c[n];
      if (bias) v = v + bias[n];
      if (relu) v = (v != v) ? v : (v > 0.f ? v : 0.f);
      c[n] = v;
    }
  }
}

// u8 x s8 -> s32 linear with zero-point compensation and per-channel dequant.
//   acc[m,n]  = sum_k int32(A[m,k]) * int32(W[k,n])        (BrgemmNaive.cpp:102-140; exact)
//   comp[n]   = zp_a * sum_k int32(W[k,n])                  (legacy/core/src/ops/matmul_core.cpp:655-700)
//   out[m,n]  = float(acc - comp) * scale[n] + bias[n]      (one fmul, one fadd; UNPINNED: no reference test)
// Either output pointer may be null.
GCO_API void gco_linear_u8s8(const uint8_t *A, const int8_t *W, const float *scale, const float *bias,
                             int32_t zp_a, int64_t M, int64_t N, int64_t K, int32_t *acc_out,
                             float *out) {
  std::vector<int32_t> comp(N, 0);
  for (int64_t k = 0; k < K; ++k)
    for (int64_t n = 0; n < N; ++n) comp[n] += int32_t(W[k * N + n]);
  for (int64_t n = 0; n < N; ++n) comp[n] *= zp_a;
  std::vector<int16_t> W16(size_t(K) * N);
  for (size_t i = 0; i < W16.size(); ++i) W16[i] = W[i];
#pragma omp parallel
  {
    std::vector<int32_t> row(N);
#pragma omp for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
      for (int64_t n = 0; n < N; ++n) row[n] = 0;
      for (int64_t k = 0; k < K; ++k) {
        int32_t a = A[m * K + k];
        const int16_t *w = W16.data() + k * N;
        for (int64_t n = 0; n < N; ++n) row[n] += a * int32_t(w[n]);
      }
      if (acc_out)
        for (int64_t n = 0; n < N; ++n) acc_out[m * N + n] = row[n];
      if (out)
        for (int64_t n = 0; n < N; ++n) {
          float v = float(row[n] - comp[n]) * scale[n];
          out[m * N + n] = bias ? v + bias[n] : v;
        }
    }
  }
}

// Row softmax in f32: max, sub, exp, sum, div
// (lib/gc/Transforms/DecomposeAggregatedOps.cpp:24-38; benchgc
// test/benchgc/src/benchgc/linalg/softmax.py:27-31).
GCO_API void gco_softmax_f32(const float *X, float *Y, int64_t rows, int64_t cols) {
  for (int64_t r = 0; r < rows; ++r) {
    const float *x = X + r * cols;
    float *y = Y + r * cols;
    float mx = -std::numeric_limits<float>::infinity();
    for (int64_t c = 0; c < cols; ++c) mx = x[c] > mx ? x[c] : mx;
    float s = 0.f;
    for (int64_t c = 0; c < cols; ++c) {
      y[c] = std::exp(x[c] - mx);
      s += y[c];
    }
    for (int64_t c = 0; c < cols; ++c) y[c] = y[c] / s;
  }
}

// Attention, restated from the pieces the reference has (batch matmul with f32
// accumulate + the softmax above); the reference has no fused pattern and no
// test for it, so parity for this function is UNPINNED.
//   S = (Q K^T) * scale  (f32), causal: S[i,j] = -inf for j > i
//   P = softmax(S) (f32);  O = bf16(P V)  (f32 accumulate, one RNE cast)
// Q,K,V,O: [BH][S][D] bf16, contiguous.
GCO_API void gco_attention_bf16(const uint16_t *Q, const uint16_t *K, const uint16_t *V, uint16_t *O,
                                int64_t BH, int64_t S, int64_t D, float scale, int causal) {
#pragma omp parallel
  {
    std::vector<float> s(S), kf(size_t(S) * D), vf(size_t(S) * D), o(D);
#pragma omp for schedule(dynamic, 1)
    for (int64_t bh = 0; bh < BH; ++bh) {
      const uint16_t *q = Q + bh * S * D, *k = K + bh * S * D, *v = V + bh * S * D;
      for (int64_t i = 0; i < S * D; ++i) {
        kf[i] = bf16_to_f32(k[i]);
        vf[i] = bf16_to_f32(v[i]);
      }
      for (int64_t i = 0; i < S; ++i) {
        int64_t jmax = causal ? i + 1 : S;
        float mx = -std::numeric_limits<float>::infinity();
        for (int64_t j = 0; j < jmax; ++j) {
          float acc = 0.f;
          for (int64_t d = 0; d < D; ++d) acc += bf16_to_f32(q[i * D + d]) * kf[j * D + d];
          s[j] = acc * scale;
          mx = s[j] > mx ? s[j] : mx;
        }
        float sum = 0.f;
        for (int64_t j = 0; j < jmax; ++j) {
          s[j] = std::exp(s[j] - mx);
          sum += s[j];
        }
        for (int64_t d = 0; d < D; ++d) o[d] = 0.f;
        for (int64_t j = 0; j < jmax; ++j) {
          float p = s[j] / sum;
          for (int64_t d = 0; d < D; ++d) o[d] += p * vf[j * D + d];
        }
        for (int64_t d = 0; d < D; ++d) O[bh * S * D + i * D + d] = f32_to_bf16(o[d]);
      }
    }
  }
}

GCO_API int gco_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
GCO_API void gco_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

// ---------------------------------------------------------------------------
// The same linear layers, but computed by driving a brgemm microkernel through
// its runtime ABI (dnnl_brgemm_dispatch / dnnl_brgemm_execute), the way the
// JIT-ed code of the reference does (call stack: DeepTileContractionOp.cpp:603-638
// -> ConvertMicrokernelToDnnlFunc.cpp:58-116 -> BrgemmOnednn.cpp:145-168).
// `dispatch` and `execute` are function pointers so that the caller can plug in
// the reference's own BrgemmNaive.cpp (oracle/_ref) — then the arithmetic is
// the reference's, only the loop nest around it is restated.
//
// Weights are packed once into block-VNNI form [N/nb][K/kb][kb/v][nb][v], the
// layout of the reference's packed-matmul generics (Linalgx/Utils.cpp:335-371);
// per output block one call runs the whole K reduction with beta = 0
// (zero-fill fused into the first call, ConvertLinalgToMicrokernel.cpp:335-350).
// ---------------------------------------------------------------------------
typedef int64_t (*gco_dispatch_fn)(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                                   float, int64_t, int64_t);
typedef void (*gco_execute_fn)(int64_t, void *, uint64_t, void *, uint64_t, void *, uint64_t, int);

static int64_t pick_block(int64_t dim) { return dim % 32 == 0 ? 32 : dim; }

template <typename TB>
static void pack_block_vnni(const TB *W, TB *P, int64_t K, int64_t N, int64_t kb, int64_t nb, int v) {
  // P[(n/nb)][(k/kb)][(k%kb)/v][n%nb][k%v]; kb is padded up to a multiple of v per block
  int64_t kbp = (kb + v - 1) / v * v;
  std::memset(P, 0, sizeof(TB) * size_t(N / nb) * (K / kb) * kbp * nb);
  for (int64_t k = 0; k < K; ++k)
    for (int64_t n = 0; n < N; ++n) {
      int64_t bn = n / nb, bk = k / kb, kk = k % kb, nn = n % nb;
      size_t off = ((size_t(bn) * (K / kb) + bk) * kbp * nb) + size_t(kk / v) * nb * v + nn * v + kk % v;
      P[off] = W[k * N + n];
    }
}

GCO_API int gco_linear_bf16_brgemm_nest(gco_dispatch_fn dispatch, gco_execute_fn execute, const uint16_t *A,
                                        const uint16_t *W, const uint16_t *bias, uint16_t *Y, int64_t M,
                                        int64_t N, int64_t K, int relu, float *acc_out) {
  const int64_t mb = pick_block(M), nb = pick_block(N), kb = pick_block(K);
  const int64_t kbp = (kb + 1) / 2 * 2;
  std::vector<uint16_t> P(size_t(N / nb) * (K / kb) * kbp * nb);
  pack_block_vnni(W, P.data(), K, N, kb, nb, 2);
  // A tile (i, kblk) starts at A[i*mb*K + kblk*kb]: LDA = K, batch stride = kb.
  int64_t h = dispatch(mb, nb, kb, K, nb, nb, kb, kbp * nb, 0.0f, DT_BF16, DT_BF16);
  if (h < 0) return -1;
#pragma omp parallel
  {
    std::vector<float> c(size_t(mb) * nb);
#pragma omp for collapse(2) schedule(static)
    for (int64_t i = 0; i < M / mb; ++i)
      for (int64_t j = 0; j < N / nb; ++j) {
        execute(h, (void *)A, uint64_t(i * mb * K), (void *)P.data(), uint64_t(size_t(j) * (K / kb) * kbp * nb),
                c.data(), 0, int(K / kb));
        for (int64_t m = 0; m < mb; ++m)
          for (int64_t n = 0; n < nb; ++n) {
            float a = c[m * nb + n];
            int64_t gm = i * mb + m, gn = j * nb + n;
            if (acc_out) acc_out[gm * N + gn] = a;
            uint16_t y = f32_to_bf16(a);
            if (bias) y = f32_to_bf16(bf16_to_f32(y) + bf16_to_f32(bias[gn]));
            if (relu) {
              float f = bf16_to_f32(y);
              if (!(f != f)) y = f > 0.f ? y : uint16_t(0);
            }
            Y[gm * N + gn] = y;
          }
      }
  }
  return 0;
}

GCO_API int gco_linear_u8s8_brgemm_nest(gco_dispatch_fn dispatch, gco_execute_fn execute, const uint8_t *A,
                                        const int8_t *W, int64_t M, int64_t N, int64_t K, int32_t *acc_out) {
  const int64_t mb = pick_block(M), nb = pick_block(N), kb = pick_block(K);
  const int64_t kbp = (kb + 3) / 4 * 4;
  std::vector<int8_t> P(size_t(N / nb) * (K / kb) * kbp * nb);
  pack_block_vnni(W, P.data(), K, N, kb, nb, 4);
  int64_t h = dispatch(mb, nb, kb, K, nb, nb, kb, kbp * nb, 0.0f, DT_U8, DT_S8);
  if (h < 0) return -1;
#pragma omp parallel
  {
    std::vector<int32_t> c(size_t(mb) * nb);
#pragma omp for collapse(2) schedule(static)
    for (int64_t i = 0; i < M / mb; ++i)
      for (int64_t j = 0; j < N / nb; ++j) {
        execute(h, (void *)A, uint64_t(i * mb * K), (void *)P.data(), uint64_t(size_t(j) * (K / kb) * kbp * nb),
                c.data(), 0, int(K / kb));
        for (int64_t m = 0; m < mb; ++m)
          for (int64_t n = 0; n < nb; ++n) acc_out[(i * mb + m) * N + j * nb + n] = c[m * nb + n];
      }
  }
  return 0;
}

// Adaptors that give the restated gco_brgemm the same two-call ABI.
namespace {
struct Params { int64_t M, N, K, LDA, LDB, LDC, sa, sb; float beta; int64_t dtA, dtB; };
std::vector<Params> g_params;
}
GCO_API int64_t gco_brgemm_dispatch(int64_t M, int64_t N, int64_t K, int64_t LDA, int64_t LDB, int64_t LDC,
                                    int64_t sa, int64_t sb, float beta, int64_t dtA, int64_t dtB) {
  int64_t id;
#pragma omp critical(gco_dispatch)
  {
    g_params.push_back({M, N, K, LDA, LDB, LDC, sa, sb, beta, dtA, dtB});
    id = int64_t(g_params.size()) - 1;
  }
  return id;
}
GCO_API void gco_brgemm_execute(int64_t h, void *A, uint64_t Aoff, void *B, uint64_t Boff, void *C,
                                uint64_t Coff, int num) {
  Params p;
#pragma omp critical(gco_dispatch)
  p = g_params[size_t(h)];
  gco_brgemm(p.M, p.N, p.K, p.LDA, p.LDB, p.LDC, p.sa, p.sb, p.beta, p.dtA, p.dtB, A, Aoff, B, Boff, C, Coff, num);
}
