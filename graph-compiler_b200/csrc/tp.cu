// Tensor-parallel MLP step across the GPUs of one node, behind the C ABI (gcb200_tp_mlp_*).
//
// The reference splits one matmul over threads along N and along K (NThreads / KThreads,
// lib/gc/Transforms/DeepTileContractionOp.cpp:562-601); a K split produces f32 partial sums that are
// reduced and only then cast (:446-471, :988-996).  Here the threads are GPUs, one process each:
//   layer 2i    (column-parallel) rank r owns W[:, r-th block]; bias and ReLU stay local;
//   layer 2i+1  (row-parallel)    rank r owns W[r-th block, :] and produces f32 partial sums of the whole
//               [M, N] result.  The GEMM epilogue stores row block d of them straight into rank d's receive
//               buffer (reduce-scatter by rows, plain NVLink stores that overlap the tiles still being
//               computed); rank d sums the g blocks in rank order, applies bias / ReLU, casts once and stores the
//               bf16 rows into EVERY rank's activation buffer (all-gather by peer stores).
// No kernel of another library and no host round trip sits between the layers: every hand-off is a monotonic
// counter in the consumer's own memory that the producers add to after a system-scope fence
// (sm100_ptx.cuh: red_release_sys_add_u32 / wait_counter_reached).  Per exchange x:
//   part_landed[x]  at the owner: + 1 per epilogue warp, tile and rank once its 32 rows are stored;
//                   the owner's reduction waits for (step + 1) * g * tiles_n * rows/32;
//   rows_landed[x]  at every rank: + 1 per CTA of every owner's reduction once its rows are stored;
//                   the next layer's operand producers (or the end-of-step kernel) wait for (step + 1) * g * CTAs.
// Counters are never reset; `step` is a device word that the last kernel of a step increments, so a captured
// CUDA graph of the step can be replayed unchanged.  Every wait is bounded and reports through the error word.
//
// Buffer reuse is safe without further synchronisation: a rank can be at most one exchange ahead of a peer,
// because each of its layers needs rows from that peer's previous reduction; receive and activation buffers
// alternate between consecutive exchanges.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/gc_b200.h"
#include "runtime.h"
#include "sm100_ptx.cuh"

#define GCB_EXPORT extern "C" __attribute__((visibility("default")))

namespace gcb {
int guard_status(const std::exception_ptr &ep);

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxExchanges = 6;
// counter slots (uint32 index) inside a rank's signal block
// (SIG_XSTEP counts only the steps whose input was fanned out by tp_scatter_rows_kernel: SIG_X_LANDED grows only in those)
enum : int { SIG_STEP = 0, SIG_X_LANDED = 1, SIG_PART0 = 2, SIG_ROWS0 = 2 + kMaxExchanges, SIG_XSTEP = 2 + 2 * kMaxExchanges,
             SIG_WORDS = 3 + 2 * kMaxExchanges };

struct PeerRows {
  uint2 *out[kMaxRanks];
  uint32_t *landed[kMaxRanks];
};
struct PeerCopy {
  uint4 *dst[kMaxRanks];
  uint32_t *landed[kMaxRanks];
};

// Rank d's half of an exchange: wait until every rank's partial sums of rows [d R, (d+1) R) have landed here, sum
// the planes in rank order (every row is reduced exactly once, so all ranks end with identical bits), one cast,
// bias, second cast, ReLU (the reference's epilogue order), store the bf16 rows into every rank's activation
// buffer, then count this CTA in at every rank.
__global__ void __launch_bounds__(1024)
tp_reduce_bcast_kernel(const float4 *parts, int nparts, long long plane4, long long total4, int n4, const uint2 *bias, int relu,
                       PeerRows peers, int n_peers, long long dst4, const uint32_t *part_landed, uint32_t per_step,
                       const uint32_t *step, int *error, unsigned long long *trace) {
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_store(trace, 0);
  pdl_launch_dependents();
  pdl_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_store(trace, 1);
  __shared__ int ok;
  if (threadIdx.x == 0) {
    const uint32_t target = (*reinterpret_cast<const volatile uint32_t *>(step) + 1u) * per_step;
    ok = wait_counter_reached(part_landed, target, 4 * WAIT_LIMIT_CYCLES) ? 1 : 0;
    if (!ok) atomicExch(error, ERR_WAIT_PEER);
    trace_max(trace, 2);
  }
  __syncthreads();
  if (ok) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
      // planes are read four at a time (all four loads in flight before the first add: the additions stay in plane
      // order, the load latencies overlap); written by other GPUs, so read through L2
      float4 s = __ldcg(parts + i);
      for (int k = 1; k < nparts; k += 4) {
        float4 t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (k + u < nparts) t[u] = __ldcg(parts + (long long)(k + u) * plane4 + i);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (k + u < nparts) {
            s.x = __fadd_rn(s.x, t[u].x); s.y = __fadd_rn(s.y, t[u].y); s.z = __fadd_rn(s.z, t[u].z); s.w = __fadd_rn(s.w, t[u].w);
          }
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
      const uint2 v = make_uint2(bf16x2_fix_nan(lo), bf16x2_fix_nan(hi));
      for (int d = 0; d < n_peers; ++d) peers.out[d][dst4 + i] = v;
    }
  }
  // counted in even after a time-out, so that the other ranks' waits end (the error word tells the host)
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();   // ONE system-scope fence per CTA publishes the whole CTA's stores (cumulative over the barrier)
    for (int d = 0; d < n_peers; ++d) red_relaxed_sys_add_u32(peers.landed[d], 1u);
    trace_max(trace, 3);
  }
}

// Last kernel of a step: the result is complete on this rank once every owner's rows have landed; then the step
// word moves on (plain store: the kernels of the next step come later in the same stream).
__global__ void tp_step_end_kernel(const uint32_t *rows_landed, uint32_t per_step, uint32_t *step, uint32_t *xstep, int *error,
                                   unsigned long long *trace) {
  if (threadIdx.x == 0) trace_store(trace, 0);
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    trace_store(trace, 1);
    const uint32_t n = *reinterpret_cast<volatile uint32_t *>(step);
    if (!wait_counter_reached(rows_landed, (n + 1u) * per_step, 4 * WAIT_LIMIT_CYCLES)) atomicExch(error, ERR_WAIT_PEER);
    trace_max(trace, 2);
    *reinterpret_cast<volatile uint32_t *>(step) = n + 1u;
    if (xstep) *reinterpret_cast<volatile uint32_t *>(xstep) = *reinterpret_cast<volatile uint32_t *>(xstep) + 1u;
    trace_max(trace, 3);
  }
}

// Input fan-out: every rank has copied only ITS row block of the activations from the host; this kernel stores
// the block into every other rank's input buffer over NVLink and counts the CTA in at every rank (itself included).
__global__ void __launch_bounds__(256)
tp_scatter_rows_kernel(const uint4 *src, long long n16, PeerCopy peers, int n_peers, int self) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int d = 0; d < n_peers; ++d)
      if (d != self) peers.dst[d][i] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    for (int d = 0; d < n_peers; ++d) red_relaxed_sys_add_u32(peers.landed[d], 1u);
  }
}

// Wait self-test (failure path): a kernel that waits, with a caller-given short limit, on a counter nobody adds
// to, gives up, records ERR_SELFTEST and returns normally.
__global__ void wait_selftest_kernel(const uint32_t *never, long long limit_cycles, int *error) {
  if (threadIdx.x == 0 && !wait_counter_reached(never, 1u, limit_cycles)) atomicExch(error, ERR_SELFTEST);
}

template <typename... KArgs, typename... Args>
void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  GCB_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
  count_launch();
}

int reduce_blocks(int64_t rows, int64_t N) {
  // a function of the shape alone: every rank must expect the same number of arrivals
  // (CTAs of 1024 threads, at most 148: every CTA ends with one system-scope fence, so few large CTAs beat many small ones)
  const long long total4 = rows * N / 4;
  return int(std::max<long long>(1, std::min<long long>((total4 + 1023) / 1024, 148)));
}

} // namespace
} // namespace gcb

using namespace gcb;

struct gcb200_tp_mlp {
  int world = 1, rank = 0, layers = 0, relu = 1;
  int64_t M = 0;
  std::vector<int64_t> hidden;
  std::vector<const void *> W, B;
  std::vector<void *> recv[2], act[2], x_in;
  int recv_planes = 0;   // f32 planes of [rows, width] each receive buffer holds (at least `world`)
  std::vector<uint32_t *> sig;
  // local state, created by the first step (create itself needs no device)
  std::mutex mu;
  bool ready = false;
  int device = -1;
  std::vector<void *> col_out;   // outputs of the column-parallel layers [M, N / world] bf16
  void *splitk = nullptr;
  size_t splitk_bytes = 0;
  cudaStream_t stream = nullptr; // host-buffer path
  int *host_code = nullptr;
  // optional timeline of one eagerly launched step: an event after every launch (see gcb200_tp_mlp_timeline)
  std::vector<cudaEvent_t> marks;
  std::vector<std::string> mark_names;
  size_t marks_used = 0;
  bool timeline = false;
  // optional device-side time stamps (GC_B200_TP_TRACE=1 when the plan takes its first step): four words per kernel of a
  // step, written by the kernels themselves, so that a replayed graph can be read as well (see gcb200_tp_mlp_trace)
  unsigned long long *trace = nullptr;
  std::vector<std::string> trace_names;
  std::vector<MatmulConfig> row_cfg;   // configuration of every row-parallel layer (fixes the arrival counts)
  std::vector<int> row_arrivals;
  struct Graph {
    const void *a = nullptr, *b = nullptr;
    int mode = 0;
    cudaGraphExec_t exec = nullptr;
    unsigned long long kernels = 0;
    bool seen_once = false, unusable = false;
  };
  std::vector<Graph> graphs;

  int64_t rows() const { return M / world; }
  int exchanges() const { return layers / 2; }
  uint32_t *counter(int rank_, int word) const { return sig[size_t(rank_)] + word; }

  void mark(const char *name, cudaStream_t s) {
    if (!timeline) return;
    if (marks_used == marks.size()) {
      cudaEvent_t e = nullptr;
      GCB_CUDA(cudaEventCreate(&e));
      marks.push_back(e);
      mark_names.emplace_back();
    }
    mark_names[marks_used] = name;
    GCB_CUDA(cudaEventRecord(marks[marks_used++], s));
  }

  ~gcb200_tp_mlp() {
    for (cudaEvent_t e : marks) cudaEventDestroy(e);
    for (Graph &g : graphs)
      if (g.exec) cudaGraphExecDestroy(g.exec);
    for (void *p : col_out)
      if (p) cudaFree(p);
    if (splitk) cudaFree(splitk);
    if (trace) cudaFree(trace);
    if (stream) cudaStreamDestroy(stream);
    if (host_code) cudaFreeHost(host_code);
  }

  void plan_row_layers(int sm_count) {
    row_cfg.clear();
    row_arrivals.clear();
    for (int x = 0; x < exchanges(); ++x) {
      const int64_t N = hidden[size_t(2 * x + 2)], K = hidden[size_t(2 * x + 1)] / world;
      // The K split of these layers is first of all the split across ranks.  Where a rank's share of K is still long
      // and 256 x 256 tiles leave SMs idle, the rank splits its share once more: every (rank, split) owns a plane at
      // the row owner (twice the partial-sum bytes over NVLink, so only while the GEMM is long enough to hide them).
      MatmulConfig c = select_matmul_config(M, N, K, 2, 4, sm_count, /*max_splits=*/1);
      if (c.swapped) throw std::logic_error("tensor-parallel layers need a batch of more than 64 rows");
      c.splits = 1;
      c.pair = 0;
      const int k_blocks = int((K + 63) / 64);
      // Measured per rank shape (512 x 4096 x K, single launches): K = 8192: pairs with the extra split 43.7 us against
      // 47.7 us for 128-wide one-CTA tiles; K = 4096: 31.4 against 29.8 us; K = 2048: 128-wide one-CTA tiles win (21.3 us).
      const int pair_tiles = int(M / 256) * int(N / 256);
      if (M % 256 == 0 && N % 256 == 0 && M <= 1024 && k_blocks >= 128 && recv_planes >= 2 * world && 4 * pair_tiles <= sm_count) {
        c.pair = 1;
        c.bn = 256;
        c.kpb = 1;
        c.stages = 6;
        c.splits = 2;
      }
      const int tiles_n = int((N + c.bn - 1) / c.bn);
      c.grid = std::min(int((M + 127) / 128) * tiles_n * c.splits, sm_count);
      row_cfg.push_back(c);
      row_arrivals.push_back(tiles_n * int(rows() / 32) * c.splits);
    }
  }

  void prepare() {
    if (ready) return;
    DeviceState &d = device_state();
    device = d.device;
    plan_row_layers(d.sm_count);
    size_t need = 0;
    for (int x = 0; x < exchanges(); ++x) {
      const int64_t n = hidden[size_t(2 * x + 1)] / world;
      void *p = nullptr;
      GCB_CUDA(cudaMalloc(&p, size_t(M) * size_t(n) * 2));
      col_out.push_back(p);
      need = std::max(need, matmul_scratch_bytes(M, n, hidden[size_t(2 * x)], 2, 2, d.sm_count));
    }
    if (need) {
      GCB_CUDA(cudaMalloc(&splitk, need));
      splitk_bytes = need;
    }
    if (const char *e = std::getenv("GC_B200_TP_TRACE"); e && e[0] == '1') {
      const size_t words = size_t(4) * size_t(3 * exchanges() + 1);
      GCB_CUDA(cudaMalloc(reinterpret_cast<void **>(&trace), words * sizeof(unsigned long long)));
      GCB_CUDA(cudaMemset(trace, 0, words * sizeof(unsigned long long)));
    }
    GCB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    GCB_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&host_code), sizeof(int), cudaHostAllocDefault));
    *host_code = 0;
    ready = true;
  }

  // the kernels of one step; x: this rank's full [M, hidden[0]] input in device memory
  void enqueue_step(const void *x, bool x_scattered, cudaStream_t s) {
    DeviceState &d = device_state();
    const uint32_t *step_word = counter(rank, SIG_STEP);
    const void *h = x;
    marks_used = 0;
    mark("start", s);
    trace_names.clear();
    auto slot = [&](const std::string &name) -> unsigned long long * {
      if (!trace) return nullptr;
      trace_names.push_back(name);
      return trace + 4 * (trace_names.size() - 1);
    };
    for (int e = 0; e < exchanges(); ++e) {
      const int64_t Kc = hidden[size_t(2 * e)], Nc = hidden[size_t(2 * e + 1)] / world, Nr = hidden[size_t(2 * e + 2)];
      {   // column-parallel layer: local bias / ReLU; its input rows come from the other ranks (except the first layer's)
        MatmulArgs m;
        m.A = h; m.B = W[size_t(2 * e)]; m.M = M; m.N = Nc; m.K = Kc;
        m.out_kind = OUT_BF16; m.out = col_out[size_t(e)];
        m.bias_kind = B[size_t(2 * e)] ? BIAS_BF16 : BIAS_NONE; m.bias = B[size_t(2 * e)]; m.relu = relu;
        m.scratch = splitk; m.scratch_bytes = splitk_bytes;
        if (e > 0) {
          m.wait_counter = counter(rank, SIG_ROWS0 + e - 1);
          m.wait_per_step = uint32_t(world * reduce_blocks(rows(), hidden[size_t(2 * e)]));
          m.epoch = step_word;
        } else if (x_scattered) {
          m.wait_counter = counter(rank, SIG_X_LANDED);
          m.wait_per_step = uint32_t(world * scatter_blocks());
          m.epoch = counter(rank, SIG_XSTEP);
        }
        m.trace = slot("column-parallel gemm " + std::to_string(2 * e));
        matmul_tc(m, s);
        mark("column-parallel gemm (+ wait for the previous exchange's rows)", s);
      }
      {   // row-parallel layer: f32 partial sums scattered by rows from the GEMM epilogue, counted in at the owner
        void *bufs[kMaxRanks];
        uint32_t *sigs[kMaxRanks];
        for (int r = 0; r < world; ++r) { bufs[r] = recv[e & 1][size_t(r)]; sigs[r] = counter(r, SIG_PART0 + e); }
        MatmulArgs m;
        m.A = col_out[size_t(e)]; m.B = W[size_t(2 * e + 1)]; m.M = M; m.N = Nr; m.K = Nc;
        m.out_kind = OUT_F32; m.out = bufs[0];
        m.n_peers = world; m.peer_plane = rank; m.peer_out = bufs; m.peer_rows = int(rows());
        m.signal_peer = sigs;
        m.force = &row_cfg[size_t(e)];
        m.peer_splits = row_cfg[size_t(e)].splits;
        int arrivals = 0;
        m.arrivals_per_peer = &arrivals;
        m.trace = slot("row-parallel gemm " + std::to_string(2 * e + 1) + " + row scatter");
        matmul_tc(m, s);
        if (arrivals != row_arrivals[size_t(e)]) throw std::logic_error("row-parallel layer ran with an unplanned tile configuration");
        mark("row-parallel gemm + row scatter to the owners", s);
      }
      {   // this rank's rows: reduce, epilogue, all-gather by peer stores
        PeerRows pr{};
        for (int r = 0; r < world; ++r) {
          pr.out[r] = reinterpret_cast<uint2 *>(act[e & 1][size_t(r)]);
          pr.landed[r] = counter(r, SIG_ROWS0 + e);
        }
        const long long total4 = rows() * Nr / 4;
        launch_pdl(tp_reduce_bcast_kernel, dim3(unsigned(reduce_blocks(rows(), Nr))), dim3(1024), s,
                   reinterpret_cast<const float4 *>(recv[e & 1][size_t(rank)]), world * row_cfg[size_t(e)].splits, total4, total4, int(Nr / 4),
                   reinterpret_cast<const uint2 *>(B[size_t(2 * e + 1)]), relu, pr, world, (long long)(rank * total4),
                   reinterpret_cast<const uint32_t *>(counter(rank, SIG_PART0 + e)), uint32_t(world * row_arrivals[size_t(e)]), step_word,
                   d.d_error, slot("reduce " + std::to_string(e) + " + all-gather stores"));
        mark("wait for all ranks' partial sums + reduce + all-gather stores", s);
      }
      h = act[e & 1][size_t(rank)];
    }
    const int last = exchanges() - 1;
    launch_pdl(tp_step_end_kernel, dim3(1), dim3(32), s, reinterpret_cast<const uint32_t *>(counter(rank, SIG_ROWS0 + last)),
               uint32_t(world * reduce_blocks(rows(), hidden.back())), counter(rank, SIG_STEP),
               x_scattered ? counter(rank, SIG_XSTEP) : static_cast<uint32_t *>(nullptr), d.d_error, slot("end of step"));
    mark("wait for every owner's rows (end of step)", s);
  }

  int scatter_blocks() const {
    const long long n16 = rows() * hidden[0] * 2 / 16;
    return int(std::max<long long>(1, std::min<long long>((n16 + 255) / 256, 296)));
  }
  void enqueue_scatter(cudaStream_t s) {
    PeerCopy pc{};
    const size_t off = size_t(rank) * size_t(rows()) * size_t(hidden[0]) * 2;
    for (int r = 0; r < world; ++r) {
      pc.dst[r] = reinterpret_cast<uint4 *>(static_cast<uint8_t *>(x_in[size_t(r)]) + off);
      pc.landed[r] = counter(r, SIG_X_LANDED);
    }
    launch_pdl(tp_scatter_rows_kernel, dim3(unsigned(scatter_blocks())), dim3(256), s,
               reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(x_in[size_t(rank)]) + off),
               (long long)(rows() * hidden[0] * 2 / 16), pc, world, rank);
  }

  void *result() const { return act[(exchanges() - 1) & 1][size_t(rank)]; }

  // Runs `body` (which enqueues on `s`) eagerly the first time a key is seen, captures it into a CUDA graph the
  // second time and replays the graph from then on: a step is 3 launches per layer pair whose host cost would
  // otherwise exceed their device time.
  // `body(stream)` enqueues on the stream it is given.  The capture runs on the plan's own stream (the legacy default
  // stream cannot be captured, and a caller's stream is left alone); the finished graph is launched on `s`.
  template <class F> void run_cached(const void *a, const void *b, int mode, cudaStream_t s, F &&body) {
    static const bool graphs_on = [] { const char *e = std::getenv("GC_B200_TP_GRAPH"); return !(e && e[0] == '0'); }();
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (s != nullptr && cudaStreamIsCapturing(s, &cs) != cudaSuccess) { cudaGetLastError(); cs = cudaStreamCaptureStatusActive; }
    if (!graphs_on || cs != cudaStreamCaptureStatusNone) { body(s); return; }
    Graph *g = nullptr;
    for (Graph &c : graphs)
      if (c.a == a && c.b == b && c.mode == mode) g = &c;
    if (!g) {
      if (graphs.size() >= 8) {
        if (graphs.front().exec) cudaGraphExecDestroy(graphs.front().exec);
        graphs.erase(graphs.begin());
      }
      graphs.push_back(Graph{});
      g = &graphs.back();
      g->a = a; g->b = b; g->mode = mode;
    }
    if (g->unusable || !g->seen_once) {
      g->seen_once = true;
      body(s);
      return;
    }
    if (!g->exec) {
      const unsigned long long l0 = launch_count();
      cudaGraph_t graph = nullptr;
      cudaStream_t cap = stream;
      bool ok = cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
      if (ok) {
        try { body(cap); } catch (...) { ok = false; }
        if (cudaStreamEndCapture(cap, &graph) != cudaSuccess || !graph) ok = false;
      }
      if (ok && cudaGraphInstantiate(&g->exec, graph, 0) != cudaSuccess) ok = false;
      if (graph) cudaGraphDestroy(graph);
      const unsigned long long n = launch_count() - l0;
      count_launch(-int(n));   // captured, not launched
      if (!ok) {
        cudaGetLastError();
        if (g->exec) cudaGraphExecDestroy(g->exec);
        g->exec = nullptr;
        g->unusable = true;
        body(s);
        return;
      }
      g->kernels = n;
    }
    GCB_CUDA(cudaGraphLaunch(g->exec, s));
    count_launch(int(g->kernels));
  }
};

GCB_EXPORT int gcb200_tp_mlp_create(const gcb200_tp_mlp_desc *d, gcb200_tp_mlp **out) {
  try {
    if (!d || !out) throw std::invalid_argument("null argument");
    if (d->world < 1 || d->world > kMaxRanks || d->rank < 0 || d->rank >= d->world) throw std::invalid_argument("rank / world out of range (1..8 ranks)");
    if (d->layers < 2 || d->layers % 2 || d->layers / 2 > kMaxExchanges)
      throw std::invalid_argument("a tensor-parallel MLP has an even number of layers (column- then row-parallel), at most 12");
    if (!d->hidden || !d->weights || !d->biases || !d->signals) throw std::invalid_argument("null table");
    if (d->batch <= 0 || d->batch % (32 * d->world) || d->batch % 128)
      throw std::invalid_argument("the batch must be a multiple of 128 and of 32 x the number of ranks (every epilogue warp's rows have one owner)");
    auto t = std::make_unique<gcb200_tp_mlp>();
    t->world = d->world; t->rank = d->rank; t->layers = d->layers; t->relu = d->relu ? 1 : 0; t->M = d->batch;
    t->recv_planes = d->recv_planes > 0 ? d->recv_planes : d->world;
    if (t->recv_planes < d->world) throw std::invalid_argument("the receive buffers must hold at least one plane per rank");
    for (int i = 0; i <= d->layers; ++i) {
      const int64_t h = d->hidden[i];
      if (h <= 0 || h % (8 * d->world)) throw std::invalid_argument("every layer width must be a positive multiple of 8 x the number of ranks");
      t->hidden.push_back(h);
    }
    for (int i = 0; i < d->layers; ++i) {
      if (!d->weights[i]) throw std::invalid_argument("null weight shard");
      t->W.push_back(d->weights[i]);
      t->B.push_back(d->biases[i]);
      if (d->biases[i] && (reinterpret_cast<uintptr_t>(d->biases[i]) & 7)) throw std::invalid_argument("bias vectors must be 8-byte aligned");
    }
    for (int s = 0; s < 2; ++s) {
      if (!d->recv[s] || !d->act[s]) throw std::invalid_argument("null buffer table");
      for (int r = 0; r < d->world; ++r) {
        if (!d->recv[s][r] || !d->act[s][r] || (reinterpret_cast<uintptr_t>(d->recv[s][r]) & 15) || (reinterpret_cast<uintptr_t>(d->act[s][r]) & 15))
          throw std::invalid_argument("receive and activation buffers must be non-null and 16-byte aligned");
        t->recv[s].push_back(d->recv[s][r]);
        t->act[s].push_back(d->act[s][r]);
      }
    }
    for (int r = 0; r < d->world; ++r) {
      if (!d->signals[r] || (reinterpret_cast<uintptr_t>(d->signals[r]) & 3)) throw std::invalid_argument("null or misaligned counter block");
      t->sig.push_back(static_cast<uint32_t *>(d->signals[r]));
      if (d->x_in) {
        if (!d->x_in[r] || (reinterpret_cast<uintptr_t>(d->x_in[r]) & 15)) throw std::invalid_argument("input buffers must be non-null and 16-byte aligned");
        t->x_in.push_back(d->x_in[r]);
      }
    }
    t->plan_row_layers(148);   // validates the shapes without a device; redone for the real device by the first step
    *out = t.release();
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}

GCB_EXPORT int gcb200_tp_mlp_destroy(gcb200_tp_mlp *t) {
  delete t;
  return GCB200_OK;
}

GCB_EXPORT int gcb200_tp_mlp_describe(const gcb200_tp_mlp *t, int sm_count, char *buf, size_t cap, size_t *needed) {
  try {
    if (!t) throw std::invalid_argument("null plan");
    gcb200_tp_mlp &m = *const_cast<gcb200_tp_mlp *>(t);
    std::lock_guard<std::mutex> g(m.mu);
    if (!m.ready) m.plan_row_layers(sm_count > 0 ? sm_count : 148);
    std::ostringstream os;
    os << "tp" << m.world << " rank " << m.rank << " batch " << m.M << " rows/rank " << m.rows() << " counter words " << int(SIG_WORDS) << "\n";
    for (int e = 0; e < m.exchanges(); ++e) {
      const int64_t Kc = m.hidden[size_t(2 * e)], Nc = m.hidden[size_t(2 * e + 1)] / m.world, Nr = m.hidden[size_t(2 * e + 2)];
      os << "layer " << 2 * e << ": column-parallel " << m.M << "x" << Nc << "x" << Kc;
      if (e > 0) os << " waits rows_landed[" << e - 1 << "] += " << m.world * reduce_blocks(m.rows(), m.hidden[size_t(2 * e)]) << " per step";
      os << "\nlayer " << 2 * e + 1 << ": row-parallel " << m.M << "x" << Nr << "x" << Nc << " bn " << m.row_cfg[size_t(e)].bn
         << (m.row_cfg[size_t(e)].pair ? " on CTA pairs" : "") << " K splits " << m.row_cfg[size_t(e)].splits << " -> part_landed[" << e
         << "] += " << m.row_arrivals[size_t(e)] << " per rank\n";
      os << "reduce " << e << ": rows " << m.rank * m.rows() << ".." << (m.rank + 1) * m.rows() << " waits part_landed[" << e
         << "] += " << m.world * m.row_arrivals[size_t(e)] << " per step, " << reduce_blocks(m.rows(), Nr) << " CTAs -> rows_landed[" << e
         << "] at every rank, buffers slot " << (e & 1) << "\n";
    }
    const std::string s = os.str();
    if (needed) *needed = s.size() + 1;
    if (buf && cap) {
      const size_t n = std::min(cap - 1, s.size());
      std::memcpy(buf, s.data(), n);
      buf[n] = '\0';
    }
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}

GCB_EXPORT int gcb200_tp_mlp_step(gcb200_tp_mlp *t, const void *x, void *stream_, void **result) {
  try {
    if (!t || !x) throw std::invalid_argument("null argument");
    if (!tma_compatible(x, t->hidden[0], 2)) throw std::invalid_argument("the input must be 16-byte aligned");
    std::lock_guard<std::mutex> g(t->mu);
    t->prepare();
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    t->run_cached(x, nullptr, 0, s, [&](cudaStream_t q) { t->enqueue_step(x, false, q); });
    if (result) *result = t->result();
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}

GCB_EXPORT int gcb200_tp_mlp_execute(gcb200_tp_mlp *t, const void *x_host, void *y_host) {
  try {
    if (!t || !x_host) throw std::invalid_argument("null argument");
    if (t->x_in.empty()) throw std::invalid_argument("the plan was created without input buffers (x_in)");
    std::lock_guard<std::mutex> g(t->mu);
    t->prepare();
    cudaStream_t s = t->stream;
    DeviceState &d = device_state();
    const size_t slice = size_t(t->rows()) * size_t(t->hidden[0]) * 2, off = size_t(t->rank) * slice;
    const size_t out_bytes = size_t(t->M) * size_t(t->hidden.back()) * 2;
    t->run_cached(x_host, y_host, 1, s, [&](cudaStream_t q) {
      // this rank brings only its row block over its own PCIe link; the other blocks arrive over NVLink
      GCB_CUDA(cudaMemcpyAsync(static_cast<uint8_t *>(t->x_in[size_t(t->rank)]) + off, static_cast<const uint8_t *>(x_host) + off, slice,
                               cudaMemcpyHostToDevice, q));
      t->enqueue_scatter(q);
      t->enqueue_step(t->x_in[size_t(t->rank)], true, q);
      if (y_host) GCB_CUDA(cudaMemcpyAsync(y_host, t->result(), out_bytes, cudaMemcpyDeviceToHost, q));
      GCB_CUDA(cudaMemcpyAsync(t->host_code, d.d_error, sizeof(int), cudaMemcpyDeviceToHost, q));
    });
    GCB_CUDA(cudaStreamSynchronize(s));
    const int code = *t->host_code;
    if (code) {
      GCB_CUDA(cudaMemset(d.d_error, 0, sizeof(int)));
      *t->host_code = 0;
      throw CudaError("a kernel gave up a bounded wait (code " + std::to_string(code) + ")");
    }
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}

GCB_EXPORT int gcb200_tp_mlp_timeline(gcb200_tp_mlp *t, const void *x, void *stream_, char *buf, size_t cap, size_t *needed) {
  try {
    if (!t || !x) throw std::invalid_argument("null argument");
    std::lock_guard<std::mutex> g(t->mu);
    t->prepare();
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    t->timeline = true;
    try {
      t->enqueue_step(x, false, s);   // eager launches with an event behind each
    } catch (...) {
      t->timeline = false;
      throw;
    }
    t->timeline = false;
    GCB_CUDA(cudaStreamSynchronize(s));
    std::ostringstream os;
    for (size_t i = 1; i < t->marks_used; ++i) {
      float ms = 0.f;
      GCB_CUDA(cudaEventElapsedTime(&ms, t->marks[i - 1], t->marks[i]));
      os << ms * 1e3f << " us  " << t->mark_names[i] << "\n";
    }
    float total = 0.f;
    if (t->marks_used > 1) GCB_CUDA(cudaEventElapsedTime(&total, t->marks[0], t->marks[t->marks_used - 1]));
    os << total * 1e3f << " us  whole step (eager launches; a replayed graph has no launch gaps)\n";
    const std::string str = os.str();
    if (needed) *needed = str.size() + 1;
    if (buf && cap) {
      const size_t n = std::min(cap - 1, str.size());
      std::memcpy(buf, str.data(), n);
      buf[n] = '\0';
    }
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}

GCB_EXPORT int gcb200_tp_mlp_trace(gcb200_tp_mlp *t, char *buf, size_t cap, size_t *needed) {
  try {
    if (!t) throw std::invalid_argument("null plan");
    std::lock_guard<std::mutex> g(t->mu);
    if (!t->ready || !t->trace || t->trace_names.empty())
      throw std::invalid_argument("no time stamps: set GC_B200_TP_TRACE=1 before the plan's first step, and take a step");
    GCB_CUDA(cudaDeviceSynchronize());
    std::vector<unsigned long long> w(4 * t->trace_names.size());
    GCB_CUDA(cudaMemcpy(w.data(), t->trace, w.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    std::ostringstream os;
    os << "us after the first kernel of the step started: launched, released by the kernel ahead, cross-GPU wait over, last CTA done\n";
    const unsigned long long t0 = w[0];
    auto us = [&](unsigned long long v) { return v ? double((long long)(v - t0)) * 1e-3 : -1.0; };
    char line[256];
    for (size_t k = 0; k < t->trace_names.size(); ++k) {
      std::snprintf(line, sizeof line, "%8.1f %8.1f %8.1f %8.1f  %s\n", us(w[4 * k]), us(w[4 * k + 1]), us(w[4 * k + 2]), us(w[4 * k + 3]),
                    t->trace_names[k].c_str());
      os << line;
    }
    const std::string str = os.str();
    if (needed) *needed = str.size() + 1;
    if (buf && cap) {
      const size_t n = std::min(cap - 1, str.size());
      std::memcpy(buf, str.data(), n);
      buf[n] = '\0';
    }
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}

GCB_EXPORT int gcb200_wait_selftest(long long limit_cycles, void *stream_) {
  try {
    if (limit_cycles <= 0 || limit_cycles > WAIT_LIMIT_CYCLES) throw std::invalid_argument("the limit must be positive and at most the library's own wait limit");
    DeviceState &d = device_state();
    // the counter nobody adds to: the step word's neighbour in a zeroed scratch word of the device state
    wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(reinterpret_cast<const uint32_t *>(d.d_zero), limit_cycles, d.d_error);
    GCB_CUDA(cudaGetLastError());
    count_launch();
    return GCB200_OK;
  } catch (...) {
    return guard_status(std::current_exception());
  }
}
