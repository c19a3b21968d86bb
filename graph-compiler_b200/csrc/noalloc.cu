// gcb200_matmul_bf16_splitk_static: the split-K bf16 matmul for callers that may not allocate.
//
// Some hosts of this library run where device allocation is off the table: a serving loop that
// has handed every byte of HBM to its own pool allocator and treats any later cudaMalloc as a bug
// (it can fail, or fragment the pool, at an arbitrary point of a long-running process), a real-time
// thread that must not take the driver's allocation lock, or an embedding runtime that was given a
// fixed memory budget at start-up.  The ordinary split-K path takes its partial-sum planes from a
// workspace that grows on demand with cudaMalloc, and the library's per-device state allocates its
// error word the first time any launcher runs.  This entry point does neither: the partial sums
// live in a fixed array that is part of the loaded module, and so does the word the kernels use to
// report a bounded wait that ran out.
//
// Cost and limits: every GPU that loads the library holds kStaticScratchBytes (16 MiB) for this
// array until the process exits, whether or not the entry point is ever called.  A call needs
// splits * M * N * 4 bytes of it and is rejected when that exceeds the array.  All calls share the
// one array and it keeps whatever the last call left in it; nothing in it has to start at zero,
// because every split writes its whole plane before the reduction reads it.  Two calls whose
// kernels overlap on the GPU (different streams, or threads) would write the same planes: callers
// must serialise calls to this entry point per device.
//
// The first call on a device looks up the device address of the array (cudaGetSymbolAddress, with
// that device current) and configures the kernel's shared-memory limit; make that first call
// before any stream capture begins.
#include <algorithm>
#include <cstdint>
#include <exception>
#include <mutex>
#include <stdexcept>
#include <string>

#include "../../include/gc_b200.h"
#include "runtime.h"
#include "sm100_ptx.cuh"

#define GCB_EXPORT extern "C" __attribute__((visibility("default")))

namespace gcb {
extern thread_local std::string g_last_error;

namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;

// Part of the module image: present in every context that loads the library.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ int g_static_error;

struct StaticState {
  bool ready = false;
  void *scratch = nullptr;  // DEVICE address of g_static_scratch on this device
  int *error = nullptr;     // DEVICE address of g_static_error
  int sm_count = 0;
};
std::mutex g_static_mutex;
StaticState g_static[64];

// In host code `g_static_scratch` names a host-side shadow of the symbol, not device memory; the
// address a kernel may dereference has to come from cudaGetSymbolAddress, per device.
StaticState &static_state() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) throw CudaError(std::string("no CUDA device: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) throw CudaError("device ordinal out of range");
  std::lock_guard<std::mutex> g(g_static_mutex);
  StaticState &s = g_static[dev];
  if (!s.ready) {
    int major = 0;
    GCB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) throw CudaError("this library is built for sm_100a only");
    GCB_CUDA(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev));
    void *p = nullptr, *q = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) throw CudaError(std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
    e = cudaGetSymbolAddress(&q, g_static_error);
    if (e != cudaSuccess) throw CudaError(std::string("cudaGetSymbolAddress(error word): ") + cudaGetErrorString(e));
    s.scratch = p;
    s.error = static_cast<int *>(q);
    s.ready = true;
  }
  return s;
}

// Sum the split planes in plane order, then bf16(bf16(sum) + bias), ReLU — the same arithmetic and
// the same order as the ordinary path's reduction.  Device code may name the array directly.
__global__ void static_reduce_kernel(int splits, long long M, long long N, const uint16_t *bias, uint16_t *out,
                                     int relu) {
  const float *planes = reinterpret_cast<const float *>(g_static_scratch);
  const long long total = M * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float s = planes[i];
    for (int k = 1; k < splits; ++k) s = __fadd_rn(s, planes[(long long)k * total + i]);
    uint32_t y = f32_to_bf16_bits(s);
    if (bias) y = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(y), bf16_bits_to_f32(bias[i % N])));
    if (relu) {
      const float f = bf16_bits_to_f32(y);
      y = (f != f) ? y : (f > 0.f ? y : 0u);
    }
    out[i] = uint16_t(y);
  }
}

// The same reduction four columns at a time with 16-byte loads (N is a multiple of 8 here, so rows and planes
// keep float4 alignment): same additions in the same order, same two roundings, packed conversions.
__global__ void __launch_bounds__(256)
static_reduce_x4_kernel(int splits, long long total4, int n4, const uint2 *bias, uint2 *out, int relu) {
  const float4 *planes = reinterpret_cast<const float4 *>(g_static_scratch);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
    float4 s = planes[i];
    for (int k = 1; k < splits; ++k) {
      const float4 t = planes[(long long)k * total4 + i];
      s.x = __fadd_rn(s.x, t.x); s.y = __fadd_rn(s.y, t.y); s.z = __fadd_rn(s.z, t.z); s.w = __fadd_rn(s.w, t.w);
    }
    uint32_t lo = pack_bf16x2_rn(s.x, s.y), hi = pack_bf16x2_rn(s.z, s.w);
    if (bias) {
      const uint2 b = bias[int(i % n4)];
      lo = pack_bf16x2_rn(__fadd_rn(__uint_as_float(lo << 16), __uint_as_float(b.x << 16)),
                          __fadd_rn(__uint_as_float(lo & 0xFFFF0000u), __uint_as_float(b.x & 0xFFFF0000u)));
      hi = pack_bf16x2_rn(__fadd_rn(__uint_as_float(hi << 16), __uint_as_float(b.y << 16)),
                          __fadd_rn(__uint_as_float(hi & 0xFFFF0000u), __uint_as_float(b.y & 0xFFFF0000u)));
    }
    if (relu) { lo = bf16x2_relu(lo); hi = bf16x2_relu(hi); }
    out[i] = make_uint2(bf16x2_fix_nan(lo), bf16x2_fix_nan(hi));
  }
}

} // namespace

int guard_status(const std::exception_ptr &ep);   // capi_kernels.cu: exception -> gcb200_status, message kept
} // namespace gcb

using namespace gcb;

GCB_EXPORT int gcb200_matmul_bf16_splitk_static(const void *A, const void *B, const void *bias, void *Y, int64_t M,
                                                int64_t N, int64_t K, int splits, int relu, void *stream_) {
  try {
    if (!A || !B || !Y || M <= 0 || N <= 0 || K <= 0) throw std::invalid_argument("bad arguments");
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) throw std::invalid_argument("M, N and K must fit 31 bits");
    if (!(tma_compatible(A, K, 2) && tma_compatible(B, N, 2)))
      throw std::invalid_argument("operands need 16-byte aligned bases and row pitches (K and N multiples of 8)");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    StaticState &st = static_state();

    MatmulConfig cfg = select_matmul_config(M, N, K, 2, 4, st.sm_count);
    cfg.pair = 0;   // this entry point drives the one-CTA kernel
    const int k_blocks = int((K + 63) / 64);
    int want = splits > 0 ? splits : std::max(2, cfg.splits);
    want = std::max(1, std::min(want, k_blocks));
    const int per = (k_blocks + want - 1) / want;
    cfg.splits = (k_blocks + per - 1) / per;     // every split owns at least one K block
    // compare by division: the product itself can wrap for absurd sizes and then pass a plain comparison
    const size_t plane_elems_max = kStaticScratchBytes / 4 / size_t(cfg.splits);
    if (size_t(M) > plane_elems_max / size_t(N))
      throw std::invalid_argument("splits * M * N * 4 = " + std::to_string(cfg.splits) + " * " + std::to_string(M) + " * " +
                                  std::to_string(N) + " * 4 bytes exceeds the static scratch of " +
                                  std::to_string(kStaticScratchBytes) + " bytes");

    GemmParams p{};
    p.K = int(K);
    p.bk_elems = 64;
    p.k_blocks = k_blocks;
    p.splits = cfg.splits;
    p.stages = cfg.stages;
    p.kpb = 1;
    p.group_m = cfg.group_m;
    p.BN = cfg.bn;
    p.out_rows = int(M);
    p.out_cols = int(N);
    p.error = st.error;
    const void *pa = cfg.swapped ? B : A, *pb = cfg.swapped ? A : B;
    const bool a_mn = cfg.swapped, b_mn = !cfg.swapped;   // weights [K,N] are MN-major, activations [M,K] K-major
    const int64_t mn_a = cfg.swapped ? N : M, mn_b = cfg.swapped ? M : N;
    p.Mm = int(mn_a);
    p.Nm = int(mn_b);
    p.tiles_m = int((mn_a + 127) / 128);
    p.tiles_n = int((mn_b + p.BN - 1) / p.BN);
    p.a = operand_geom(a_mn, 128, 2);
    p.b = operand_geom(b_mn, p.BN, 2);
    p.idesc = umma_instr_desc(1u, 1u, 1u, a_mn ? 1u : 0u, b_mn ? 1u : 0u, 128u, uint32_t(p.BN));
    uint32_t cols = 32;
    while (cols < uint32_t(2 * p.BN)) cols <<= 1;
    p.tmem_cols = cols;
    p.out_kind = OUT_F32;       // raw f32 partial sums, one plane per split
    p.out = st.scratch;
    p.ld_out = N;
    p.split_stride = M * N;
    p.bias_kind = BIAS_NONE;
    const CUtensorMap tmA = operand_tmap(p.a, ElemType::BF16, 2, pa, mn_a, K, 128);
    const CUtensorMap tmB = operand_tmap(p.b, ElemType::BF16, 2, pb, mn_b, K, p.BN);
    const int units = p.tiles_m * p.tiles_n * p.splits;
    const int grid = std::max(1, std::min(units, st.sm_count));
    const size_t smem = gemm_smem_bytes(p);
    if (smem > 232448) throw std::invalid_argument("tile configuration exceeds shared memory");
    cudaError_t e = cfg.swapped ? launch_gemm_kernel<0, true>(tmA, tmB, p, grid, smem, stream)
                                : launch_gemm_kernel<0, false>(tmA, tmB, p, grid, smem, stream);
    if (e != cudaSuccess) throw CudaError(std::string("gemm launch: ") + cudaGetErrorString(e));
    count_launch();
    const long long total = M * N;
    auto al8 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 7) == 0; };
    if (N % 4 == 0 && al8(Y) && (!bias || al8(bias))) {
      const long long total4 = total / 4;
      const int blocks = int(std::min<long long>((total4 + 255) / 256, (long long)st.sm_count * 8));
      static_reduce_x4_kernel<<<std::max(blocks, 1), 256, 0, stream>>>(cfg.splits, total4, int(N / 4), static_cast<const uint2 *>(bias),
                                                                      static_cast<uint2 *>(Y), relu);
    } else {
      const int blocks = int(std::min<long long>((total + 255) / 256, (long long)st.sm_count * 8));
      static_reduce_kernel<<<blocks, 256, 0, stream>>>(cfg.splits, M, N, static_cast<const uint16_t *>(bias),
                                                       static_cast<uint16_t *>(Y), relu);
    }
    GCB_CUDA(cudaGetLastError());
    count_launch();
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());   // same status classes as every other entry point
  }
}

GCB_EXPORT int gcb200_static_error(void *stream, int *code) {
  try {
    if (!code) throw std::invalid_argument("code is null");
    StaticState &st = static_state();
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    GCB_CUDA(cudaMemcpyAsync(code, st.error, sizeof(int), cudaMemcpyDeviceToHost, s));
    GCB_CUDA(cudaStreamSynchronize(s));
    if (*code != 0) GCB_CUDA(cudaMemsetAsync(st.error, 0, sizeof(int), s));
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}
