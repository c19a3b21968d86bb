// The oneDNN-graph backend C API (include/dnnl_graph_compiler.h) on top of the
// CUDA runtime: compile = read the JSON partition + build the launch plan;
// execute = marshal tensors by id, stage host buffers, run the plan's steps on
// the executable's stream inside its pre-planned workspace arena.
//
// Reference counterparts: src/dnnl/dnnl_graph_compiler.cpp:45-226 (executable,
// argument marshalling, status mapping) and lib/gc/ExecutionEngine/Driver/
// Driver.cpp:60-89 (the JIT engine this replaces).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <sstream>
#include <string>
#include <vector>

#include <cuda_fp16.h>

#include "../../include/dnnl_graph_compiler.h"
#include "../../include/gc_b200.h"
#include "attention.h"
#include "graph.h"
#include "log.h"
#include "memplan.h"
#include "runtime.h"
#include "sm100_ptx.cuh"

#define GCB_EXPORT extern "C" __attribute__((visibility("default")))

namespace gcb {

extern thread_local std::string g_last_error;

// ----------------------------------------------------------------------------- elementwise kernels
constexpr int kMaxRank = 12; // DNNL_MAX_NDIMS

struct EwParams {
  int rank;
  long long total;
  long long dims[kMaxRank];   // output dims
  long long sa[kMaxRank];     // element strides of operand a per output dim (0 = broadcast)
  long long sb[kMaxRank];
  int fn;                     // binary: 0 add 1 sub 2 mul 3 div; unary: 0 relu 1 sigmoid 2 pow 3 cast 4 exp 5 negate
  float beta;
  int dt_a, dt_b, dt_o;       // 0 f32, 1 bf16, 2 f16
  // how an operand's offset follows from the flat output index i without walking the dims:
  // 0 general (walk), 1 same layout (i), 2 one value (0), 3 a row vector broadcast over rows (i % c),
  // 4 one value per row (i / c), c = the innermost output dim
  int mode_a, mode_b;
  unsigned inner;
};

__device__ __forceinline__ long long ew_offset(const EwParams &p, long long i, int mode, const long long *stride) {
  switch (mode) {
  case 1: return i;
  case 2: return 0;
  case 3: return (long long)(unsigned(i) % p.inner);
  case 4: return (long long)(unsigned(i) / p.inner);
  default: {
    long long r = i, o = 0;
    for (int d = p.rank - 1; d >= 0; --d) {
      const long long c = r % p.dims[d];
      r /= p.dims[d];
      o += c * stride[d];
    }
    return o;
  }
  }
}

__device__ __forceinline__ float ew_load(const void *p, long long i, int dt) {
  if (dt == 0) return reinterpret_cast<const float *>(p)[i];
  if (dt == 1) return bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p)[i]);
  return __half2float(reinterpret_cast<const __half *>(p)[i]);
}
// Every bf16/f16 op rounds once on store: the reference evaluates low-precision
// elementwise ops as extf -> f32 op -> truncf (lib/gc/Transforms/Pipeline.cpp:81-90).
__device__ __forceinline__ void ew_store(void *p, long long i, int dt, float v) {
  if (dt == 0) reinterpret_cast<float *>(p)[i] = v;
  else if (dt == 1) reinterpret_cast<uint16_t *>(p)[i] = uint16_t(f32_to_bf16_bits(v));
  else reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
}

__global__ void binary_kernel(EwParams p, const void *a, const void *b, void *o) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.total; i += (long long)gridDim.x * blockDim.x) {
    const long long oa = ew_offset(p, i, p.mode_a, p.sa), ob = ew_offset(p, i, p.mode_b, p.sb);
    const float x = ew_load(a, oa, p.dt_a), y = ew_load(b, ob, p.dt_b);
    float v;
    switch (p.fn) {
    case 0: v = __fadd_rn(x, y); break;
    case 1: v = __fsub_rn(x, y); break;
    case 2: v = __fmul_rn(x, y); break;
    default: v = __fdiv_rn(x, y); break;
    }
    ew_store(o, i, p.dt_o, v);
  }
}

__global__ void unary_kernel(EwParams p, const void *a, void *o) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.total; i += (long long)gridDim.x * blockDim.x) {
    const long long oa = ew_offset(p, i, p.mode_a, p.sa);
    const float x = ew_load(a, oa, p.dt_a);
    float v;
    switch (p.fn) {
    case 0: v = (x != x) ? x : (x > 0.f ? x : 0.f); break;       // max(x, 0), NaN propagates
    case 1: v = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-x))); break; // 1 / (1 + exp(-x))
    case 2:
      if (p.beta == 2.f) v = __fmul_rn(x, x);
      else if (p.beta == 1.f) v = x;
      else if (p.beta == 0.5f) v = sqrtf(x);
      else if (p.beta == 3.f) v = __fmul_rn(__fmul_rn(x, x), x);
      else v = powf(x, p.beta);
      break;
    case 4: v = expf(x); break;
    case 5: v = -x; break;
    default: v = x; break;
    }
    ew_store(o, i, p.dt_o, v);
  }
}

// acc[m, n] -= comp[n]: the zero-point term of a u8 x s8 product whose accumulators are the result themselves
__global__ void sub_comp_kernel(int32_t *acc, const int32_t *comp, long long total, int N) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    acc[i] -= comp[int(i % N)];
}

struct ReduceParams {
  int rank;
  long long out_total, red_total;
  long long kdims[kMaxRank], kstr[kMaxRank]; // kept dims (output iteration) and their input strides
  int nk;
  long long rdims[kMaxRank], rstr[kMaxRank]; // reduced dims, row-major order, input strides
  int nr;
  int mean;
  int dt_a, dt_o;
  int contiguous;   // the reduced elements of one output are consecutive in memory (innermost dims reduced)
};

// One thread per output element; the reduced indices are visited in ascending
// row-major order, the order of the reference's linalg.reduce loops.
__global__ void reduce_kernel(ReduceParams p, const void *a, void *o) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.out_total; i += (long long)gridDim.x * blockDim.x) {
    long long r = i, base = 0;
    for (int d = p.nk - 1; d >= 0; --d) {
      base += (r % p.kdims[d]) * p.kstr[d];
      r /= p.kdims[d];
    }
    float s = 0.f;
    for (long long j = 0; j < p.red_total; ++j) {
      long long q = j, off = base;
      for (int d = p.nr - 1; d >= 0; --d) {
        off += (q % p.rdims[d]) * p.rstr[d];
        q /= p.rdims[d];
      }
      s = __fadd_rn(s, ew_load(a, off, p.dt_a));
    }
    if (p.mean) s = __fdiv_rn(s, float(p.red_total));
    ew_store(o, i, p.dt_o, s);
  }
}

// Long reductions (e.g. the 4096-wide mean of an RMSNorm): one block per output element.  Thread t sums
// elements t, t + 256, ... in ascending order, then the 256 partial sums are combined in a fixed tree,
// so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) reduce_block_kernel(ReduceParams p, const void *a, void *o) {
  __shared__ float part[256];
  for (long long i = blockIdx.x; i < p.out_total; i += gridDim.x) {
    long long r = i, base = 0;
    for (int d = p.nk - 1; d >= 0; --d) {
      base += (r % p.kdims[d]) * p.kstr[d];
      r /= p.kdims[d];
    }
    float s = 0.f;
    if (p.contiguous) {
#pragma unroll 4
      for (long long j = threadIdx.x; j < p.red_total; j += 256) s = __fadd_rn(s, ew_load(a, base + j, p.dt_a));
    } else {
      for (long long j = threadIdx.x; j < p.red_total; j += 256) {
        long long q = j, off = base;
        for (int d = p.nr - 1; d >= 0; --d) {
          off += (q % p.rdims[d]) * p.rstr[d];
          q /= p.rdims[d];
        }
        s = __fadd_rn(s, ew_load(a, off, p.dt_a));
      }
    }
    part[threadIdx.x] = s;
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
      if (int(threadIdx.x) < w) part[threadIdx.x] = __fadd_rn(part[threadIdx.x], part[threadIdx.x + w]);
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      float t = part[0];
      if (p.mean) t = __fdiv_rn(t, float(p.red_total));
      ew_store(o, i, p.dt_o, t);
    }
    __syncthreads();
  }
}

static int ew_dtype(DType t) {
  switch (t) {
  case DType::F32: return 0;
  case DType::BF16: return 1;
  case DType::F16: return 2;
  default: throw std::logic_error(std::string("elementwise op on dtype ") + dtype_name(t));
  }
}

static std::vector<int64_t> dense_strides(const std::vector<int64_t> &shape) {
  std::vector<int64_t> s(shape.size(), 1);
  for (int d = int(shape.size()) - 2; d >= 0; --d) s[d] = s[d + 1] * shape[d + 1];
  return s;
}
static std::vector<int64_t> strides_of(const LogicalTensor &t) {
  if (t.strided && t.stride.size() == t.shape.size()) return t.stride;
  return dense_strides(t.shape);
}
static bool is_dense(const LogicalTensor &t) { return strides_of(t) == dense_strides(t.shape); }
// elements spanned in memory by a (possibly strided) tensor
static size_t span_elems(const LogicalTensor &t) {
  if (t.numel() == 0) return 0;
  const auto s = strides_of(t);
  int64_t span = 1;
  for (size_t d = 0; d < t.shape.size(); ++d) span += (t.shape[d] - 1) * s[d];
  return size_t(span);
}

// ----------------------------------------------------------------------------- executable
struct DeviceBuffer {
  void *ptr = nullptr;
  size_t bytes = 0;
  const void *cached_host = nullptr; // constant tensors: host address whose contents are resident
  void reserve(size_t n) {
    if (n <= bytes) return;
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    bytes = 0;
    GCB_CUDA(cudaMalloc(&ptr, n));
    bytes = n;
  }
  ~DeviceBuffer() {
    if (ptr) cudaFree(ptr);
  }
};

} // namespace gcb

using namespace gcb;

struct dnnl_graph_compiler {
  uint32_t num_threads = 0;
};

struct dnnl_graph_compiler_executable {
  Plan plan;
  // device state is created on first execute so that compile needs no GPU
  mutable std::mutex mu;
  mutable bool ready = false;
  mutable int device = -1;
  mutable cudaStream_t stream = nullptr;
  mutable cudaStream_t copy_in = nullptr, copy_out = nullptr;   // host copies that overlap the first / last matmul
  mutable cudaEvent_t ev_in[4] = {}, ev_out[4] = {};
  mutable int *host_code = nullptr;                             // pinned: the device error word after a call
  // Replay of the launch list as a CUDA graph when a call repeats an earlier call's device addresses:
  // the first call runs eagerly (it also sizes the workspaces), the second is captured, later ones replay.
  struct GraphEntry {
    std::vector<const void *> key;
    cudaGraphExec_t exec = nullptr;
    unsigned long long ws_generation = 0, kernels = 0, last_use = 0;
    bool unusable = false;
  };
  mutable std::vector<GraphEntry> graphs;
  mutable unsigned long long graph_clock = 0;
  mutable DeviceBuffer arena;
  mutable std::vector<DeviceBuffer> in_stage, out_stage;
  mutable std::vector<char> comp_ready; // per QMATMUL scratch: column sums computed for a cached constant weight
  static constexpr int kCanary = 0xA5;
  mutable DeviceBuffer splitk;          // split-K partial planes of this executable's matmul steps (they run one after
                                        // another on one stream, so one block sized for the largest request serves all)

  explicit dnnl_graph_compiler_executable(const std::string &json) : plan(build_plan(read_partition(json))) {}
  ~dnnl_graph_compiler_executable() {
    if (stream) cudaStreamDestroy(stream);
    if (copy_in) cudaStreamDestroy(copy_in);
    if (copy_out) cudaStreamDestroy(copy_out);
    for (int i = 0; i < 4; ++i) {
      if (ev_in[i]) cudaEventDestroy(ev_in[i]);
      if (ev_out[i]) cudaEventDestroy(ev_out[i]);
    }
    if (host_code) cudaFreeHost(host_code);
    for (GraphEntry &g : graphs)
      if (g.exec) cudaGraphExecDestroy(g.exec);
  }

  void prepare() const {
    if (ready) return;
    DeviceState &d = device_state();
    device = d.device;
    GCB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    GCB_CUDA(cudaStreamCreateWithFlags(&copy_in, cudaStreamNonBlocking));
    GCB_CUDA(cudaStreamCreateWithFlags(&copy_out, cudaStreamNonBlocking));
    for (int i = 0; i < 4; ++i) {
      GCB_CUDA(cudaEventCreateWithFlags(&ev_in[i], cudaEventDisableTiming));
      GCB_CUDA(cudaEventCreateWithFlags(&ev_out[i], cudaEventDisableTiming));
    }
    GCB_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&host_code), sizeof(int), cudaHostAllocDefault));
    if (plan.arena_bytes) arena.reserve(plan.arena_bytes);
    if (plan.guard_bytes && plan.arena_bytes) GCB_CUDA(cudaMemset(arena.ptr, kCanary, plan.arena_bytes));
    gcLogD("executable prepared on device ", device, ": arena ", plan.arena_bytes, " bytes, ", plan.steps.size(), " steps, guard bands ",
           plan.guard_bytes, " bytes");
    in_stage.resize(plan.part.input_ids.size());
    out_stage.resize(plan.part.output_ids.size());
    comp_ready.assign(plan.scratch.size(), 0);
    {
      // split-K scratch of every matmul step, as the selector sees the shapes on this device (whole step and,
      // where the step may run as row blocks, one block); a configuration recorded later that needs more
      // falls back to the per-device workspace inside matmul_tc
      size_t need = 0;
      for (const Step &st : plan.steps) {
        if (st.kind != StepKind::MATMUL && st.kind != StepKind::QMATMUL) continue;
        const bool q = st.kind == StepKind::QMATMUL;
        if (!q && plan.part.tensors.at(st.in[0]).dtype != DType::BF16) continue;
        need = std::max(need, matmul_scratch_bytes(st.M, st.N, st.K, q ? 1 : 2, q ? 4 : 2, d.sm_count));
        if (!q && rows_chunkable(st))
          need = std::max(need, matmul_scratch_bytes(st.M / kRowChunks, st.N, st.K, 2, 2, d.sm_count));
      }
      if (need) splitk.reserve(need);
    }
    ready = true;
  }

  static dnnl_graph_compiler_tensor *find(dnnl_graph_compiler_tensor *ts, size_t n, size_t i, size_t id) {
    if (ts[i].id == id) return &ts[i];
    for (size_t j = 0; j < n; ++j)   // the order may differ from the argument order
      if (ts[j].id == id) return &ts[j];
    throw std::invalid_argument("Tensor not found");
  }

  static bool on_device(const void *p) {
    cudaPointerAttributes at;
    cudaError_t e = cudaPointerGetAttributes(&at, p);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
  }

  void check_dims(const dnnl_graph_compiler_tensor *t, const LogicalTensor &lt) const {
    if (t->ndims > DNNL_MAX_NDIMS) throw std::invalid_argument("Number of dimensions > DNNL_MAX_NDIMS");
    int64_t n = 1;
    for (int d = 0; d < t->ndims; ++d) n *= t->dims[d];
    if (n != lt.numel()) throw std::invalid_argument("Tensor " + std::to_string(lt.id) + " does not have the compiled shape");
    if (!t->data && n) throw std::invalid_argument("Tensor " + std::to_string(lt.id) + " has no data");
  }

  // A bf16 tensor-core MatMul whose rows can be computed in independent chunks: used to overlap the
  // host copy of its A operand (first step) or of its result (last step) with the other chunk's math.
  // Two chunks of >= 256 rows: each chunk still fills the SMs and re-reads the weights only once more.
  static constexpr int kRowChunks = 2;
  bool rows_chunkable(const Step &st) const {
    const Partition &p = plan.part;
    if (st.kind != StepKind::MATMUL || st.trans_a) return false;
    const LogicalTensor &A = p.tensors.at(st.in[0]);
    if (A.dtype != DType::BF16 || !is_dense(A) || !is_dense(p.tensors.at(st.in[1]))) return false;
    if (st.M < 512 || st.M % (128 * kRowChunks)) return false;
    return (st.K % 8) == 0 && (st.N % 8) == 0;
  }
  void matmul_rows(const Step &st, const void *a, const void *b, const void *bias, void *out, int64_t r0, int64_t rows,
                   cudaStream_t s) const {
    MatmulArgs m;
    m.A = static_cast<const uint8_t *>(a) + size_t(r0) * size_t(st.K) * 2;
    m.B = b; m.M = rows; m.N = st.N; m.K = st.K; m.trans_a = 0; m.trans_b = st.trans_b;
    m.out_kind = OUT_BF16; m.out = static_cast<uint8_t *>(out) + size_t(r0) * size_t(st.N) * 2;
    m.bias_kind = bias ? BIAS_BF16 : BIAS_NONE; m.bias = bias; m.relu = st.relu;
    m.scratch = splitk.ptr; m.scratch_bytes = splitk.bytes;
    matmul_tc(m, s);
  }

  // Debug mode: every guard band must still hold the canary.  Returns the number of damaged bands and describes
  // the first one; reads the bands back to the host (slow, debug only).  The stream must be idle.
  int check_guards(std::string *what) const {
    if (!plan.guard_bytes || !arena.ptr) return 0;
    std::vector<unsigned char> h(plan.guard_bytes);
    int bad = 0;
    for (const auto &band : plan.guards) {
      GCB_CUDA(cudaMemcpy(h.data(), static_cast<const uint8_t *>(arena.ptr) + band.first, plan.guard_bytes, cudaMemcpyDeviceToHost));
      size_t first_bad = plan.guard_bytes;
      for (size_t i = 0; i < plan.guard_bytes; ++i)
        if (h[i] != kCanary) { first_bad = i; break; }
      if (first_bad == plan.guard_bytes) continue;
      if (bad++ == 0 && what)
        *what = "guard band at arena offset " + std::to_string(band.first) + " (" +
                (band.second == ~size_t(0) ? std::string("scratch slot") : "tensor " + std::to_string(band.second)) +
                ") overwritten at byte " + std::to_string(first_bad);
    }
    return bad;
  }

  // One line per step with the kernel and, for matmuls, the tile configuration the selector gives for `sm_count` SMs.
  std::string describe_launches(int sm_count) const {
    std::ostringstream os;
    for (size_t i = 0; i < plan.steps.size(); ++i) {
      const Step &st = plan.steps[i];
      os << "  step " << i << " " << st.op << ": ";
      if (st.kind == StepKind::MATMUL || st.kind == StepKind::QMATMUL) {
        const bool q = st.kind == StepKind::QMATMUL;
        const bool bf16 = q || plan.part.tensors.at(st.in[0]).dtype == DType::BF16;
        const bool tma = ((st.trans_a ? st.M : st.K) * (q ? 1 : 2)) % 16 == 0 && ((st.trans_b ? st.K : st.N) * (q ? 1 : 2)) % 16 == 0;
        if (!bf16 || !tma) {
          os << "matmul_simt_kernel (exact-order f32) " << st.M << "x" << st.N << "x" << st.K << "\n";
          continue;
        }
        const MatmulConfig c = select_matmul_config(st.M, st.N, st.K, q ? 1 : 2, q ? 4 : 2, sm_count);
        os << "gemm_kernel<" << (q ? "u8 x s8" : "bf16") << (c.swapped ? ", weights on the MMA M side" : "") << "> " << st.M << "x" << st.N
           << "x" << st.K << " tile 128x" << c.bn << " splits " << c.splits << " stages " << c.stages << " K blocks/stage "
           << std::max(1, c.kpb) << " grid " << c.grid << (c.splits > 1 ? " + reduce_planes" : "") << (q ? " + colsum_s8" : "") << "\n";
      } else if (st.kind == StepKind::SDPA) {
        os << "attention_kernel B*H=" << st.batch * st.heads << " S=" << st.seq << " D=" << st.dim << " causal=" << st.causal << "\n";
      } else {
        os << (st.kind == StepKind::REDUCE ? "reduce kernel" : st.kind == StepKind::BINARY ? "binary_kernel"
               : st.kind == StepKind::COPY ? "device-to-device copy" : "unary_kernel") << "\n";
      }
    }
    return os.str();
  }

  // own_stream: run on the executable's private stream (the synchronous C API); otherwise on
  // `user_stream`, where a null handle means the legacy default stream, as everywhere in CUDA.
  void execute(dnnl_graph_compiler_tensor *inputs, dnnl_graph_compiler_tensor *outputs, cudaStream_t user_stream,
               bool own_stream, bool sync) const {
    std::lock_guard<std::mutex> g(mu);
    prepare();
    {
      // streams, arena and staging buffers belong to the device that was current at the first call
      int cur = -1;
      GCB_CUDA(cudaGetDevice(&cur));
      if (cur != device)
        throw std::runtime_error("this executable is bound to CUDA device " + std::to_string(device) + " (current at its first execute); the current device is " +
                                 std::to_string(cur));
    }
    cudaStream_t s = own_stream ? stream : user_stream;
    const Partition &p = plan.part;
    const size_t ni = p.input_ids.size(), no = p.output_ids.size();
    std::vector<void *> in_ptr(ni), out_ptr(no), out_host(no, nullptr);
    // host copies overlapped with the first / last step (synchronous API only)
    const Step *first = plan.steps.empty() ? nullptr : &plan.steps.front();
    const Step *last = plan.steps.empty() ? nullptr : &plan.steps.back();
    long piped_in = -1, piped_out = -1;   // argument index whose copy is chunked
    const void *piped_in_host = nullptr;
    if (own_stream && first && rows_chunkable(*first)) {
      const TensorSlot &sl = plan.slots.at(first->in[0]);
      if (sl.where == TensorSlot::INPUT && !p.tensors.at(first->in[0]).constant) piped_in = long(sl.index);
    }
    if (own_stream && last && rows_chunkable(*last)) {
      const TensorSlot &sl = plan.slots.at(last->out[0]);
      if (sl.where == TensorSlot::OUTPUT) piped_out = long(sl.index);
    }
    for (size_t i = 0; i < ni; ++i) {
      const LogicalTensor &lt = p.tensors.at(p.input_ids[i]);
      dnnl_graph_compiler_tensor *t = find(inputs, ni, i, lt.id);
      check_dims(t, lt);
      const size_t bytes = span_elems(lt) * dtype_bytes(lt.dtype);
      if (on_device(t->data)) {
        in_ptr[i] = t->data;
        if (long(i) == piped_in) piped_in = -1;
      } else if (long(i) == piped_in) {
        in_stage[i].reserve(bytes);
        in_ptr[i] = in_stage[i].ptr;
        piped_in_host = t->data;
      } else {
        DeviceBuffer &b = in_stage[i];
        // GC_B200_CONST_CACHE=0: re-read constant tensors on every call, as the reference does (for callers that
        // rewrite a weight buffer in place)
        static const bool const_cache = [] { const char *e = std::getenv("GC_B200_CONST_CACHE"); return !(e && e[0] == '0'); }();
        const bool resident = const_cache && lt.constant && b.cached_host == t->data && b.bytes >= bytes;
        if (!resident) {
          b.reserve(bytes);
          GCB_CUDA(cudaMemcpyAsync(b.ptr, t->data, bytes, cudaMemcpyHostToDevice, s));
          b.cached_host = (const_cache && lt.constant) ? t->data : nullptr;
          // column sums depend on the weights alone: only those computed from THIS argument are stale now
          for (const Step &qs : plan.steps)
            if (qs.kind == StepKind::QMATMUL && qs.scratch_slot >= 0) {
              const TensorSlot &ws = plan.slots.at(qs.in[1]);
              if (ws.where == TensorSlot::INPUT && size_t(ws.index) == i) comp_ready[size_t(qs.scratch_slot)] = 0;
            }
        }
        in_ptr[i] = b.ptr;
      }
    }
    for (size_t i = 0; i < no; ++i) {
      const LogicalTensor &lt = p.tensors.at(p.output_ids[i]);
      dnnl_graph_compiler_tensor *t = find(outputs, no, i, lt.id);
      check_dims(t, lt);
      const size_t bytes = size_t(lt.numel()) * dtype_bytes(lt.dtype);
      if (on_device(t->data)) {
        out_ptr[i] = t->data;
        if (long(i) == piped_out) piped_out = -1;
      } else {
        out_stage[i].reserve(bytes);
        out_ptr[i] = out_stage[i].ptr;
        out_host[i] = t->data;
      }
    }
    // The synchronous API runs on the executable's private stream.  Device tensors may still be
    // being produced (or their memory still be in use) by work the caller queued on other streams;
    // order this call after all of it.
    if (own_stream) {
      bool any_dev = false;
      for (size_t i = 0; i < ni; ++i) any_dev |= (in_ptr[i] != in_stage[i].ptr);
      for (size_t i = 0; i < no; ++i) any_dev |= (out_host[i] == nullptr);
      if (any_dev) GCB_CUDA(cudaDeviceSynchronize());
    }
    auto addr = [&](size_t id) -> void * {
      const TensorSlot &sl = plan.slots.at(id);
      if (sl.where == TensorSlot::INPUT) return in_ptr[sl.index];
      if (sl.where == TensorSlot::OUTPUT) return out_ptr[sl.index];
      return static_cast<uint8_t *>(arena.ptr) + sl.offset;
    };
    // the chunked form goes straight to the tensor-core kernel: its operands must be addressable by TMA
    auto tc_ok = [&](const Step &st) {
      return tma_compatible(addr(st.in[0]), st.K, 2) && tma_compatible(addr(st.in[1]), st.trans_b ? st.K : st.N, 2) &&
             tma_compatible(addr(st.out[0]), st.N, 2);
    };
    if (piped_in >= 0 && !tc_ok(*first)) {
      const LogicalTensor &lt = p.tensors.at(first->in[0]);
      GCB_CUDA(cudaMemcpyAsync(in_ptr[size_t(piped_in)], piped_in_host, span_elems(lt) * dtype_bytes(lt.dtype),
                               cudaMemcpyHostToDevice, s));
      piped_in = -1;
    }
    if (piped_out >= 0 && !tc_ok(*last)) piped_out = -1;
    // ---- every tensor in device memory: the launch list does not depend on anything but the addresses
    bool all_dev = true;
    for (size_t i = 0; i < ni; ++i) all_dev &= (in_ptr[i] != in_stage[i].ptr || in_stage[i].ptr == nullptr);
    for (size_t i = 0; i < no; ++i) all_dev &= (out_host[i] == nullptr);
    static const bool graphs_on = [] { const char *e = std::getenv("GC_B200_GRAPHS"); return !(e && e[0] == '0'); }();
    bool replayed = false;
    if (all_dev && graphs_on && plan.steps.size() > 1) {
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(s, &cs) != cudaSuccess) { cudaGetLastError(); cs = cudaStreamCaptureStatusActive; }
      if (cs == cudaStreamCaptureStatusNone) {
        std::vector<const void *> key(in_ptr.begin(), in_ptr.end());
        key.insert(key.end(), out_ptr.begin(), out_ptr.end());
        GraphEntry *ge = nullptr;
        for (GraphEntry &g : graphs)
          if (g.key == key) ge = &g;
        const unsigned long long gen = device_state().workspace_generation;
        if (ge && ge->exec && ge->ws_generation != gen) {   // a workspace moved: the captured addresses are stale
          cudaGraphExecDestroy(ge->exec);
          ge->exec = nullptr;
        }
        if (!ge) {
          // first sight of these addresses: remember them, run eagerly below
          if (graphs.size() >= 4) {
            size_t victim = 0;
            for (size_t i = 1; i < graphs.size(); ++i)
              if (graphs[i].last_use < graphs[victim].last_use) victim = i;
            if (graphs[victim].exec) cudaGraphExecDestroy(graphs[victim].exec);
            graphs.erase(graphs.begin() + long(victim));
          }
          graphs.push_back(GraphEntry{});
          graphs.back().key = key;
          graphs.back().last_use = ++graph_clock;
        } else if (!ge->unusable) {
          ge->last_use = ++graph_clock;
          if (!ge->exec) {
            const unsigned long long l0 = launch_count();
            cudaGraph_t g = nullptr;
            bool ok = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
            if (ok) {
              try {
                for (const Step &st : plan.steps) run_step(st, addr, in_ptr, s);
              } catch (...) {
                ok = false;
              }
              if (cudaStreamEndCapture(s, &g) != cudaSuccess || !g) ok = false;
            }
            if (ok && cudaGraphInstantiate(&ge->exec, g, 0) != cudaSuccess) ok = false;
            if (g) cudaGraphDestroy(g);
            if (!ok) {
              cudaGetLastError();
              if (ge->exec) cudaGraphExecDestroy(ge->exec);
              ge->exec = nullptr;
              ge->unusable = true;   // fall back to eager launches for these addresses
              count_launch(-int(launch_count() - l0));
            } else {
              ge->kernels = launch_count() - l0;
              ge->ws_generation = gen;
              count_launch(-int(ge->kernels));   // counted when launched, below
            }
          }
          if (ge->exec) {
            GCB_CUDA(cudaGraphLaunch(ge->exec, s));
            count_launch(int(ge->kernels));
            replayed = true;
          }
        }
      }
    }
    for (size_t k = 0; k < plan.steps.size() && !replayed; ++k) {
      const Step &st = plan.steps[k];
      const bool chunk_in = (k == 0 && piped_in >= 0), chunk_out = (k + 1 == plan.steps.size() && piped_out >= 0);
      if (!chunk_in && !chunk_out) {
        run_step(st, addr, in_ptr, s);
        continue;
      }
      // the step runs as kRowChunks row blocks: block c starts when its rows of A have arrived, and its
      // rows of the result start their way back to the host while block c + 1 computes
      const void *a = addr(st.in[0]), *b = addr(st.in[1]);
      const void *bias = st.has_bias ? addr(st.in[2]) : nullptr;
      void *out = addr(st.out[0]);
      const int64_t rows = st.M / kRowChunks;
      const size_t in_chunk = size_t(rows) * size_t(st.K) * 2, out_chunk = size_t(rows) * size_t(st.N) * 2;
      if (chunk_in)
        for (int c = 0; c < kRowChunks; ++c) {
          GCB_CUDA(cudaMemcpyAsync(static_cast<uint8_t *>(in_ptr[size_t(piped_in)]) + c * in_chunk,
                                   static_cast<const uint8_t *>(piped_in_host) + c * in_chunk, in_chunk, cudaMemcpyHostToDevice,
                                   copy_in));
          GCB_CUDA(cudaEventRecord(ev_in[c], copy_in));
        }
      for (int c = 0; c < kRowChunks; ++c) {
        if (chunk_in) GCB_CUDA(cudaStreamWaitEvent(s, ev_in[c], 0));
        matmul_rows(st, a, b, bias, out, c * rows, rows, s);
        if (chunk_out) {
          GCB_CUDA(cudaEventRecord(ev_out[c], s));
          GCB_CUDA(cudaStreamWaitEvent(copy_out, ev_out[c], 0));
          GCB_CUDA(cudaMemcpyAsync(static_cast<uint8_t *>(out_host[size_t(piped_out)]) + c * out_chunk,
                                   static_cast<const uint8_t *>(out) + c * out_chunk, out_chunk, cudaMemcpyDeviceToHost, copy_out));
        }
      }
    }
    for (size_t i = 0; i < no; ++i)
      if (out_host[i] && long(i) != piped_out) {
        const LogicalTensor &lt = p.tensors.at(p.output_ids[i]);
        GCB_CUDA(cudaMemcpyAsync(out_host[i], out_ptr[i], size_t(lt.numel()) * dtype_bytes(lt.dtype), cudaMemcpyDeviceToHost, s));
      }
    bool any_host = false;
    for (void *h : out_host) any_host |= (h != nullptr);
    if (sync || any_host) {
      // the error word travels behind the results on the same stream: one wait covers both
      GCB_CUDA(cudaMemcpyAsync(host_code, device_state().d_error, sizeof(int), cudaMemcpyDeviceToHost, s));
      GCB_CUDA(cudaStreamSynchronize(s));
      if (piped_out >= 0) GCB_CUDA(cudaStreamSynchronize(copy_out));
      const int code = *host_code;
      if (code) {
        GCB_CUDA(cudaMemset(device_state().d_error, 0, sizeof(int)));
        gcLogE("device error word = ", code, " after execute");
        throw std::runtime_error("a kernel gave up a bounded wait (code " + std::to_string(code) + ")");
      }
      if (plan.guard_bytes) {
        std::string what;
        const int bad = check_guards(&what);
        if (bad) {
          GCB_CUDA(cudaMemset(arena.ptr, kCanary, plan.arena_bytes));   // re-arm: temporaries are rewritten by every call
          gcLogE(bad, " guard band(s) damaged: ", what);
          throw std::runtime_error(what);
        }
      }
    }
  }

  template <class Addr>
  void run_step(const Step &st, Addr &addr, const std::vector<void *> &in_ptr, cudaStream_t s) const {
    const Partition &p = plan.part;
    switch (st.kind) {
    case StepKind::MATMUL: {
      const LogicalTensor &A = p.tensors.at(st.in[0]);
      if (!is_dense(A) || !is_dense(p.tensors.at(st.in[1]))) throw std::logic_error("MatMul operands must be dense row-major");
      const void *bias = st.has_bias ? addr(st.in[2]) : nullptr;
      if (A.dtype == DType::BF16) {
        const void *a = addr(st.in[0]), *b = addr(st.in[1]);
        if (tma_compatible(a, st.trans_a ? st.M : st.K, 2) && tma_compatible(b, st.trans_b ? st.K : st.N, 2)) {
          MatmulArgs m;
          m.A = a; m.B = b; m.M = st.M; m.N = st.N; m.K = st.K; m.trans_a = st.trans_a; m.trans_b = st.trans_b;
          m.out_kind = OUT_BF16; m.out = addr(st.out[0]);
          m.bias_kind = bias ? BIAS_BF16 : BIAS_NONE; m.bias = bias; m.relu = st.relu;
          m.scratch = splitk.ptr; m.scratch_bytes = splitk.bytes;
          matmul_tc(m, s);
        } else {
          matmul_simt(a, b, bias, addr(st.out[0]), st.M, st.N, st.K, st.trans_a, st.trans_b, 1, st.relu, s);
        }
      } else {
        matmul_simt(addr(st.in[0]), addr(st.in[1]), bias, addr(st.out[0]), st.M, st.N, st.K, st.trans_a, st.trans_b, 0,
                    st.relu, s);
      }
      break;
    }
    case StepKind::QMATMUL: {
      const TensorSlot &sc = plan.scratch[size_t(st.scratch_slot)];
      int32_t *comp = reinterpret_cast<int32_t *>(static_cast<uint8_t *>(arena.ptr) + sc.offset);
      // the column sums depend on the weights only: recompute unless the weights are a cached constant
      const TensorSlot &wslot = plan.slots.at(st.in[1]);
      const bool w_const = wslot.where == TensorSlot::INPUT && p.tensors.at(st.in[1]).constant &&
                           in_stage[wslot.index].cached_host != nullptr;
      if (!(w_const && comp_ready[size_t(st.scratch_slot)])) {
        colsum_s8(static_cast<const int8_t *>(addr(st.in[1])), comp, st.K, st.N, int32_t(st.zp_a), s);
        comp_ready[size_t(st.scratch_slot)] = w_const ? 1 : 0;
      }
      MatmulArgs m;
      m.A = addr(st.in[0]); m.B = addr(st.in[1]); m.M = st.M; m.N = st.N; m.K = st.K; m.int8 = 1;
      if (st.raw_acc) {
        // accumulators only: the raw s32 sums, then the zero-point term taken off per column
        m.out_kind = OUT_S32; m.out = addr(st.out[0]);
        if (!(tma_compatible(m.A, st.K, 1) && tma_compatible(m.B, st.N, 1)))
          throw std::logic_error("QuantizedMatMul needs K and N to be multiples of 16");
        m.scratch = splitk.ptr; m.scratch_bytes = splitk.bytes;
        matmul_tc(m, s);
        if (st.zp_a != 0) {
          const long long total = (long long)st.M * st.N;
          sub_comp_kernel<<<int(std::min<long long>((total + 255) / 256, 148LL * 16)), 256, 0, s>>>(static_cast<int32_t *>(addr(st.out[0])), comp, total, int(st.N));
          GCB_CUDA(cudaGetLastError());
          count_launch();
        }
        break;
      }
      m.out_kind = OUT_DEQUANT_F32; m.out = addr(st.out[0]);
      m.scale = static_cast<const float *>(addr(st.in[2]));
      m.comp = comp;
      m.bias_kind = st.has_bias ? BIAS_F32 : BIAS_NONE;
      m.bias = st.has_bias ? addr(st.in[3]) : nullptr;
      m.acc_dump = st.out.size() > 1 ? static_cast<int32_t *>(addr(st.out[1])) : nullptr;
      m.relu = st.relu;
      if (!(tma_compatible(m.A, st.K, 1) && tma_compatible(m.B, st.N, 1)))
        throw std::logic_error("QuantizedMatMul needs K and N to be multiples of 16");
      m.scratch = splitk.ptr; m.scratch_bytes = splitk.bytes;
      matmul_tc(m, s);
      break;
    }
    case StepKind::SDPA: {
      attention_bf16(addr(st.in[0]), addr(st.in[1]), addr(st.in[2]), addr(st.out[0]), st.batch * st.heads, st.seq, st.dim,
                     st.scale, st.causal ? 1 : 0, s);
      break;
    }
    case StepKind::BINARY:
    case StepKind::UNARY: {
      const LogicalTensor &O = p.tensors.at(st.out[0]);
      EwParams e{};
      e.rank = int(O.shape.size());
      if (e.rank > kMaxRank) throw std::invalid_argument("Number of dimensions > DNNL_MAX_NDIMS");
      e.total = O.numel();
      e.fn = st.fn;
      e.beta = st.beta;
      e.dt_o = ew_dtype(O.dtype);
      for (int d = 0; d < e.rank; ++d) e.dims[d] = O.shape[size_t(d)];
      auto fill = [&](const LogicalTensor &T, long long *dst) {
        const auto str = strides_of(T);
        const int off = e.rank - int(T.shape.size());
        if (off < 0) throw std::invalid_argument("operand rank exceeds result rank");
        for (int d = 0; d < e.rank; ++d) dst[d] = 0;
        for (size_t d = 0; d < T.shape.size(); ++d) {
          if (T.shape[d] == O.shape[d + off]) dst[d + off] = T.shape[d] == 1 ? 0 : str[d];
          else if (T.shape[d] == 1) dst[d + off] = 0;
          else throw std::invalid_argument("shapes are not broadcastable");
        }
      };
      // offset shortcuts (only when the flat index fits 32 bits)
      auto classify = [&](const long long *str) {
        if (e.total >= (1ll << 31) || e.rank == 0) return 0;
        const auto dense = dense_strides(O.shape);
        bool same = true, none = true, row_vec = true, row_val = true;
        for (int d = 0; d < e.rank; ++d) {
          if (e.dims[d] == 1) continue;
          const bool last = (d == e.rank - 1);
          same &= (str[d] == dense[size_t(d)]);
          none &= (str[d] == 0);
          row_vec &= last ? (str[d] == 1) : (str[d] == 0);
          row_val &= last ? (str[d] == 0) : (str[d] * e.dims[e.rank - 1] == dense[size_t(d)]);
        }
        return same ? 1 : none ? 2 : row_vec ? 3 : row_val ? 4 : 0;
      };
      e.inner = unsigned(e.rank ? e.dims[e.rank - 1] : 1);
      const LogicalTensor &A = p.tensors.at(st.in[0]);
      fill(A, e.sa);
      e.mode_a = classify(e.sa);
      e.dt_a = ew_dtype(A.dtype);
      const int threads = 256;
      const int blocks = int(std::min<long long>((e.total + threads - 1) / threads, 148LL * 16));
      if (e.total == 0) break;
      if (st.kind == StepKind::BINARY) {
        const LogicalTensor &B = p.tensors.at(st.in[1]);
        fill(B, e.sb);
        e.mode_b = classify(e.sb);
        e.dt_b = ew_dtype(B.dtype);
        binary_kernel<<<blocks, threads, 0, s>>>(e, addr(st.in[0]), addr(st.in[1]), addr(st.out[0]));
      } else {
        unary_kernel<<<blocks, threads, 0, s>>>(e, addr(st.in[0]), addr(st.out[0]));
      }
      GCB_CUDA(cudaGetLastError());
      count_launch();
      break;
    }
    case StepKind::REDUCE: {
      const LogicalTensor &A = p.tensors.at(st.in[0]);
      const LogicalTensor &O = p.tensors.at(st.out[0]);
      ReduceParams r{};
      const auto str = strides_of(A);
      r.rank = int(A.shape.size());
      if (r.rank > kMaxRank) throw std::invalid_argument("Number of dimensions > DNNL_MAX_NDIMS");
      r.out_total = 1;
      r.red_total = 1;
      for (int d = 0; d < r.rank; ++d) {
        const bool red = std::find(st.axes.begin(), st.axes.end(), int64_t(d)) != st.axes.end();
        if (red) { r.rdims[r.nr] = A.shape[size_t(d)]; r.rstr[r.nr++] = str[size_t(d)]; r.red_total *= A.shape[size_t(d)]; }
        else { r.kdims[r.nk] = A.shape[size_t(d)]; r.kstr[r.nk++] = str[size_t(d)]; r.out_total *= A.shape[size_t(d)]; }
      }
      if (r.out_total != O.numel()) throw std::invalid_argument("reduce output shape does not match");
      r.mean = st.mean ? 1 : 0;
      {
        // reduced dims innermost and dense: element j of the reduction sits j elements after the first
        long long expect = 1;
        bool ok = r.nr > 0;
        for (int d = r.nr - 1; d >= 0 && ok; --d) {
          ok = (r.rstr[d] == expect);
          expect *= r.rdims[d];
        }
        r.contiguous = ok ? 1 : 0;
      }
      r.dt_a = ew_dtype(A.dtype);
      r.dt_o = ew_dtype(O.dtype);
      if (r.red_total >= 512 && r.out_total > 0) {
        const int blocks = int(std::min<long long>(r.out_total, 148LL * 8));
        reduce_block_kernel<<<blocks, 256, 0, s>>>(r, addr(st.in[0]), addr(st.out[0]));
      } else {
        const int threads = 128;
        const int blocks = int(std::min<long long>((r.out_total + threads - 1) / threads, 148LL * 16));
        reduce_kernel<<<std::max(blocks, 1), threads, 0, s>>>(r, addr(st.in[0]), addr(st.out[0]));
      }
      GCB_CUDA(cudaGetLastError());
      count_launch();
      break;
    }
    case StepKind::COPY: {
      const LogicalTensor &A = p.tensors.at(st.in[0]);
      if (!is_dense(A)) throw std::logic_error("StaticReshape of a strided tensor");
      const size_t bytes = size_t(A.numel()) * dtype_bytes(A.dtype);
      if (bytes) GCB_CUDA(cudaMemcpyAsync(addr(st.out[0]), addr(st.in[0]), bytes, cudaMemcpyDeviceToDevice, s));
      break;
    }
    default: throw std::logic_error("unsupported step");
    }
    (void)in_ptr;
  }
};

// ----------------------------------------------------------------------------- C API
#ifndef GCB_VERSION_MAJOR
#define GCB_VERSION_MAJOR 0
#define GCB_VERSION_MINOR 1
#define GCB_VERSION_PATCH 0
#endif

GCB_EXPORT const dnnl_graph_compiler_version *dnnl_graph_compiler_get_version(void) {
  static const dnnl_graph_compiler_version ver = {
      {DNNL_GC_API_V_MAJOR, DNNL_GC_API_V_MINOR, DNNL_GC_API_V_PATCH, DNNL_GC_API_V_HASH},
      {GCB_VERSION_MAJOR, GCB_VERSION_MINOR, GCB_VERSION_PATCH, "b200"}};
  return &ver;
}

GCB_EXPORT dnnl_status_t dnnl_graph_compiler_create(const dnnl_graph_compiler_context *ctx, const dnnl_graph_compiler **gc) {
  try {
    auto *g = new dnnl_graph_compiler();
    g->num_threads = ctx ? ctx->num_threads : 0;
    *gc = g;
    return dnnl_success;
  } catch (const std::bad_alloc &) {
    return dnnl_out_of_memory;
  } catch (...) {
    return dnnl_runtime_error;
  }
}

GCB_EXPORT void dnnl_graph_compiler_destroy(const dnnl_graph_compiler *gc) { delete gc; }

GCB_EXPORT dnnl_status_t dnnl_graph_compiler_compile(const dnnl_graph_compiler *gc, const char *graph_json,
                                                     const dnnl_graph_compiler_executable **exe) {
  (void)gc;
  try {
    if (!graph_json || !exe) throw std::invalid_argument("null argument");
    auto *e = new dnnl_graph_compiler_executable(std::string(graph_json));
    *exe = e;
    gcLogD("compiled a partition of ", e->plan.part.ops.size(), " ops into ", e->plan.steps.size(), " steps");
    if (gcb::logging::verbose()) std::cout << "[gc_b200] launch plan\n" << e->describe_launches(148) << std::flush;
    return dnnl_success;
  } catch (const std::invalid_argument &e) {
    g_last_error = e.what();
    return dnnl_invalid_graph;
  } catch (const std::logic_error &e) {
    g_last_error = e.what();
    return dnnl_unimplemented;
  } catch (const std::bad_alloc &) {
    return dnnl_out_of_memory;
  } catch (const std::exception &e) {
    g_last_error = e.what();
    return dnnl_runtime_error;
  } catch (...) {
    return dnnl_runtime_error;
  }
}

GCB_EXPORT void dnnl_graph_compiler_destroy_executable(const dnnl_graph_compiler_executable *exe) { delete exe; }

static dnnl_status_t execute_impl(const dnnl_graph_compiler_executable *exe, dnnl_graph_compiler_tensor *inputs,
                                  dnnl_graph_compiler_tensor *outputs, cudaStream_t stream, bool own_stream, bool sync) {
  try {
    if (!exe) throw std::invalid_argument("null executable");
    exe->execute(inputs, outputs, stream, own_stream, sync);
    return dnnl_success;
  } catch (const std::bad_alloc &) {
    return dnnl_out_of_memory;
  } catch (const std::exception &e) {
    g_last_error = e.what();
    gcLogE("execute failed: ", e.what());
    return dnnl_runtime_error; // the reference maps every execute failure to runtime_error (:217-225)
  } catch (...) {
    return dnnl_runtime_error;
  }
}

GCB_EXPORT dnnl_status_t dnnl_graph_compiler_execute(const dnnl_graph_compiler_executable *exe,
                                                     dnnl_graph_compiler_tensor *inputs,
                                                     dnnl_graph_compiler_tensor *outputs) {
  return execute_impl(exe, inputs, outputs, nullptr, true, true);
}

// --- additions declared in include/gc_b200.h ---------------------------------------------------
GCB_EXPORT int gcb200_execute_on_stream(const dnnl_graph_compiler_executable *exe, dnnl_graph_compiler_tensor *inputs,
                                        dnnl_graph_compiler_tensor *outputs, void *stream) {
  return int(execute_impl(exe, inputs, outputs, static_cast<cudaStream_t>(stream), false, false));
}

GCB_EXPORT int gcb200_plan_dump(const dnnl_graph_compiler_executable *exe, char *buf, size_t cap, size_t *needed) {
  if (!exe) return GCB200_INVALID_ARGUMENT;
  const std::string s = exe->plan.dump();
  if (needed) *needed = s.size() + 1;
  if (buf && cap) {
    const size_t n = std::min(cap - 1, s.size());
    std::memcpy(buf, s.data(), n);
    buf[n] = '\0';
  }
  return GCB200_OK;
}

GCB_EXPORT int gcb200_describe_launches(const dnnl_graph_compiler_executable *exe, int sm_count, char *buf, size_t cap, size_t *needed) {
  if (!exe) return GCB200_INVALID_ARGUMENT;
  const std::string s = exe->describe_launches(sm_count > 0 ? sm_count : 148);
  if (needed) *needed = s.size() + 1;
  if (buf && cap) {
    const size_t n = std::min(cap - 1, s.size());
    std::memcpy(buf, s.data(), n);
    buf[n] = '\0';
  }
  return GCB200_OK;
}

GCB_EXPORT int gcb200_guard_check(const dnnl_graph_compiler_executable *exe, int *damaged) {
  if (!exe || !damaged) return GCB200_INVALID_ARGUMENT;
  try {
    std::lock_guard<std::mutex> g(exe->mu);
    if (exe->ready) GCB_CUDA(cudaDeviceSynchronize());
    std::string what;
    *damaged = exe->check_guards(&what);
    if (*damaged) g_last_error = what;
    return GCB200_OK;
  } catch (const std::exception &e) {
    g_last_error = e.what();
    return GCB200_CUDA_ERROR;
  }
}

GCB_EXPORT int gcb200_guard_selftest(const dnnl_graph_compiler_executable *exe) {
  if (!exe) return GCB200_INVALID_ARGUMENT;
  try {
    std::lock_guard<std::mutex> g(exe->mu);
    if (!exe->plan.guard_bytes || exe->plan.guards.empty()) throw std::invalid_argument("the partition was not compiled with GC_B200_GUARD");
    exe->prepare();
    // what an out-of-bounds store of a kernel would do: one byte of the first band loses its canary
    GCB_CUDA(cudaMemset(static_cast<uint8_t *>(exe->arena.ptr) + exe->plan.guards.front().first + 3, 0, 1));
    return GCB200_OK;
  } catch (const std::invalid_argument &e) {
    g_last_error = e.what();
    return GCB200_INVALID_ARGUMENT;
  } catch (const std::exception &e) {
    g_last_error = e.what();
    return GCB200_CUDA_ERROR;
  }
}

GCB_EXPORT int gcb200_schedule_memory(const uint64_t *trace_buffer, const uint64_t *trace_size, int n_traces,
                                      uint64_t alignment, int hot_first, const uint64_t *hint_buffer,
                                      const uint64_t *hint_candidate, const int *hint_kind, int n_hints,
                                      uint64_t *out_buffer, uint64_t *out_offset, int *n_out, uint64_t *total,
                                      uint64_t *sel_buffer, uint64_t *sel_reused, int *n_sel) {
  if (n_traces < 0 || n_hints < 0 || !n_out || !total || !n_sel) return GCB200_INVALID_ARGUMENT;
  try {
    std::vector<memplan::Trace> tr;
    for (int i = 0; i < n_traces; ++i) tr.push_back(memplan::Trace{trace_buffer[i], size_t(trace_size[i])});
    memplan::InplaceHints hints;
    for (int i = 0; i < n_hints; ++i)
      hints[hint_buffer[i]].emplace_back(hint_candidate[i], hint_kind[i] ? memplan::InplaceKind::Free : memplan::InplaceKind::ZeroOffset);
    std::unordered_map<uint64_t, size_t> off;
    std::unordered_map<uint64_t, std::vector<uint64_t>> reused;
    *total = memplan::schedule(tr, size_t(alignment), hot_first != 0, hints, off, reused);
    int k = 0;
    for (auto &kv : off) {
      if (k < *n_out && out_buffer && out_offset) { out_buffer[k] = kv.first; out_offset[k] = kv.second; }
      ++k;
    }
    const bool fits = k <= *n_out;
    *n_out = k;
    int m = 0;
    for (auto &kv : reused)
      for (uint64_t r : kv.second) {
        if (m < *n_sel && sel_buffer && sel_reused) { sel_buffer[m] = kv.first; sel_reused[m] = r; }
        ++m;
      }
    const bool fits2 = m <= *n_sel;
    *n_sel = m;
    return (fits && fits2) ? GCB200_OK : GCB200_INVALID_ARGUMENT;
  } catch (const std::exception &e) {
    g_last_error = e.what();
    return GCB200_INVALID_ARGUMENT;
  }
}

GCB_EXPORT int gcb200_plan_arena(const int64_t *bytes, const int *first, const int *last, int n, int64_t align,
                                 int64_t *offsets, int64_t *total) {
  if (n < 0 || align <= 0 || !offsets || !total) return GCB200_INVALID_ARGUMENT;
  std::vector<BufferLife> b;
  for (int i = 0; i < n; ++i) b.push_back(BufferLife{size_t(bytes[i]), first[i], last[i]});
  std::vector<size_t> off;
  *total = int64_t(plan_arena(b, size_t(align), off));
  for (int i = 0; i < n; ++i) offsets[i] = int64_t(off[size_t(i)]);
  return GCB200_OK;
}
