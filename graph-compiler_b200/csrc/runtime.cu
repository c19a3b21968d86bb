// CUDA runtime: device state, tensor maps, tile selection, matmul launch
// planning and the small helper kernels (split-K reduction + epilogue, int8
// column sums, exact-order SIMT matmul).
#include "runtime.h"
#include "tune_cache.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "sm100_ptx.cuh"

namespace gcb {

// ----------------------------------------------------------------------------- device state
static std::atomic<unsigned long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

static std::mutex g_dev_mutex;
static DeviceState g_devs[64];

DeviceState &device_state() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) throw CudaError(std::string("no CUDA device: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) throw CudaError("device ordinal out of range");
  std::lock_guard<std::mutex> g(g_dev_mutex);
  DeviceState &d = g_devs[dev];
  if (d.device < 0) {
    cudaDeviceProp prop;
    GCB_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      throw CudaError("this library is built for sm_100a only; device is sm_" + std::to_string(prop.major) +
                      std::to_string(prop.minor));
    d.sm_count = prop.multiProcessorCount;
    GCB_CUDA(cudaMalloc(&d.d_error, 64));
    GCB_CUDA(cudaMemset(d.d_error, 0, 64));
    d.d_zero = d.d_error + 8;
    d.device = dev;
  }
  return d;
}

void *DeviceState::ensure_workspace(size_t bytes) {
  std::lock_guard<std::mutex> g(g_dev_mutex);
  if (bytes <= workspace_bytes) return workspace;
  // Grow by allocating a larger block and keeping the old one until the process exits: launches already
  // queued (or captured in a graph) on another stream or by another thread keep a valid address, and
  // nothing here synchronises the device or frees memory under a caller's feet.  Sizes at least double,
  // so the retired blocks add up to less than the live one.
  const size_t want = std::max({bytes, workspace_bytes * 2, size_t(64) << 20});
  void *fresh = nullptr;
  GCB_CUDA(cudaMalloc(&fresh, want));
  workspace = fresh;   // the previous block is retired, not freed
  workspace_bytes = want;
  ++workspace_generation;
  return workspace;
}

int read_device_error(cudaStream_t stream) {
  DeviceState &d = device_state();
  int h = 0;
  GCB_CUDA(cudaMemcpyAsync(&h, d.d_error, sizeof(int), cudaMemcpyDeviceToHost, stream));
  GCB_CUDA(cudaStreamSynchronize(stream));
  if (h != 0) GCB_CUDA(cudaMemsetAsync(d.d_error, 0, sizeof(int), stream));
  return h;
}

// ----------------------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  if (!fn) throw CudaError("cuTensorMapEncodeTiled is not available from the driver");
  return fn;
}

CUtensorMap make_tmap_2d(ElemType t, const void *ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                         uint32_t box_inner, uint32_t box_outer) {
  CUtensorMap m;
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  switch (t) {
  case ElemType::BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
  case ElemType::U8:
  case ElemType::S8: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
  case ElemType::F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
  case ElemType::S32: dt = CU_TENSOR_MAP_DATA_TYPE_INT32; break;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_fn()(&m, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw CudaError("cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)));
  return m;
}

CUtensorMap make_tmap_3d(ElemType t, const void *ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                         uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2) {
  CUtensorMap m;
  CUtensorMapDataType dt = (t == ElemType::BF16)  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : (t == ElemType::F32) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : (t == ElemType::S32) ? CU_TENSOR_MAP_DATA_TYPE_INT32
                                                  : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode_fn()(&m, dt, 3, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw CudaError("cuTensorMapEncodeTiled (3-D) failed with CUresult " + std::to_string(int(r)));
  return m;
}

bool tma_compatible(const void *ptr, int64_t row_elems, int elem_bytes) {
  return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && ((row_elems * elem_bytes) & 15) == 0;
}

// ----------------------------------------------------------------------------- tile selection
static int ceil_div(int64_t a, int64_t b) { return int((a + b - 1) / b); }

MatmulConfig select_matmul_config(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count, int max_splits) {
  if (max_splits >= 1 && max_splits < 8) return model_matmul_config(M, N, K, dtype_bytes, out_bytes, sm_count, max_splits);
  // a configuration measured for exactly this shape beats the model; an explicit GC_B200_TILE beats both
  MatmulConfig c{};
  if (!std::getenv("GC_B200_TILE") && tune::lookup(tune::Key{M, N, K, dtype_bytes, out_bytes}, &c) && (!c.swapped || M <= 64)) {
    if (c.grid <= 0 || c.grid > sm_count) c.grid = sm_count;
    return c;
  }
  return model_matmul_config(M, N, K, dtype_bytes, out_bytes, sm_count);
}

MatmulConfig model_matmul_config(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count, int max_splits) {
  MatmulConfig c{};
  const int bk = 128 / dtype_bytes;
  const int k_blocks = ceil_div(K, bk);
  const int out_gran = out_bytes == 2 ? 64 : 32; // epilogue works in 128-byte row slabs
  c.swapped = (M <= 64 && N >= 128) ? 1 : 0;
  int tiles;
  if (c.swapped) {
    c.bn = std::max(16, ceil_div(M, 16) * 16);
    tiles = ceil_div(N, 128);
  } else {
    // Time model fitted to measurements on B200 (microseconds): a CTA spends c per 128-byte K block —
    // dominated by the per-stage hand-shake, so it shrinks little with the tile and a lot when a
    // stage carries two K blocks (possible while three stages still fit: bn <= 128) — plus a fixed
    // cost per tile; a split-K run adds the traffic of its partial planes and a second launch.
    //   measured per K block at 8192^3 / 16384^3: bn 256: 0.42;  bn 128: 0.38 (one block per stage),
    //   0.277 (two);  bn 64: 0.29 (one)
    const int cand[4] = {256, 192, 128, 64};
    const int split_cand[6] = {1, 2, 3, 4, 6, 8};
    double best_t = 1e30;
    int best_bn = 256, best_sp = 1, best_kpb = 1;
    for (int bn : cand) {
      if (bn % out_gran) continue;
      int bn_eff = bn;
      if (N < bn) bn_eff = std::max(out_gran, ceil_div(N, out_gran) * out_gran);
      const int kpb = (bn_eff <= 128 && k_blocks >= 4) ? 2 : 1;
      const double c_kb = bn_eff >= 256 ? 0.42 : bn_eff >= 192 ? 0.40 : bn_eff >= 128 ? (kpb == 2 ? 0.277 : 0.38)
                                                                                      : (kpb == 2 ? 0.21 : 0.29) * std::max(0.6, bn_eff / 64.0);
      const int t = ceil_div(M, 128) * ceil_div(N, bn_eff);
      for (int sp : split_cand) {
        if (sp > max_splits) continue;
        if (sp > 1 && (k_blocks < 16 * sp || t >= sm_count)) continue;
        const int kbs = ceil_div(k_blocks, sp);
        if (sp > 1 && kbs % kpb) continue;   // a stage must not straddle two splits
        const int waves = ceil_div(t * sp, sm_count);
        double us = waves * (kbs * c_kb + 3.0);
        // partial planes written and read back (f32), the result written, one more launch:
        // measured 13 us for 2 planes of 512 x 4096
        if (sp > 1) us += 3.0 + (2.0 * sp * double(M) * double(N) * 4.0 + double(M) * double(N) * out_bytes) / 3.5e6;
        if (us < best_t - 1e-9) { best_t = us; best_bn = bn_eff; best_sp = sp; best_kpb = kpb; }
      }
    }
    // int8, less than one wave of 256-wide tiles: 128-wide tiles with two K blocks per stage give twice the
    // tiles (every SM works, the tail wave is short) at the same hand-shakes per byte.  Measured with the
    // tuner at 1024 x 4096 x 4096 with operands coming from HBM: 30.8 us against 37.0 us; the model's
    // constants, fitted on bf16 shapes, rank the two the other way round.  At 8192^3 256-wide tiles stay ahead.
    if (dtype_bytes == 1 && best_bn == 256 && best_sp == 1 && k_blocks >= 4 && N % 128 == 0 &&
        ceil_div(M, 128) * ceil_div(N, 256) <= sm_count) {
      best_bn = 128;
      best_kpb = 2;
    }
    c.bn = best_bn;
    c.splits = best_sp;
    c.kpb = best_kpb;
    tiles = ceil_div(M, 128) * ceil_div(N, c.bn);
  }
  if (c.swapped) {
    // decode shapes stream the weights once (measured at M=16, K=8192, N=28672: 5.5 TB/s with two K
    // blocks per stage and no split, 4.8 with one): split K only when there are fewer tiles than SMs
    c.kpb = k_blocks >= 4 ? 2 : 1;
    c.splits = 1;
    if (tiles < sm_count && k_blocks >= 32) {
      int sp = std::max(1, std::min({(sm_count + tiles - 1) / tiles, k_blocks / 16, 32}));
      while (sp > 1 && ceil_div(k_blocks, sp) % c.kpb) --sp;
      c.splits = sp;
    }
  }
  // every split must own at least one K block
  {
    const int per = ceil_div(k_blocks, c.splits);
    c.splits = ceil_div(k_blocks, per);
  }
  const size_t a_bytes = 128 * 128;
  size_t b_bytes;
  {
    // worst case over orientations: MN-major operands are staged in full 128-byte boxes
    const int box_mn = 128 / dtype_bytes;
    const size_t mn = size_t(ceil_div(c.bn, box_mn)) * size_t(bk) * 128;
    const size_t km = size_t(c.bn) * 128;
    b_bytes = std::max(mn, km);
  }
  const size_t budget = 232448 - 1024 - 4 * 8192 - 256;
  const int kpb_eff = std::max(1, c.kpb);
  c.stages = int(std::min<size_t>(8, budget / ((a_bytes + b_bytes) * size_t(kpb_eff))));
  c.stages = std::max(2, std::min(c.stages, std::max(2, ceil_div(k_blocks, kpb_eff))));
  // Rasterisation: 8 tile rows per column sweep; with very long K (measured at 16384^3: 6.34 ms against 6.92 ms) four,
  // so that fewer CTAs walk the same weight columns and drift apart in L2.
  c.group_m = (k_blocks >= 256 && tiles >= 8 * sm_count) ? 4 : 8;
  // CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles on two SMs, half the weight bytes per SM): measured faster where
  // a few hundred activation rows meet a large streamed weight matrix (512 x 16384 x 4096: 64.7 against 73.0 us;
  // 512 x 4096 x 16384 split in two: 64.3 against 68.6 us), slower on large square shapes (4096^3: 109.5 against 103.1 us).
  c.pair = (!c.swapped && dtype_bytes == 2 && c.bn == 256 && c.kpb <= 1 && M % 256 == 0 && M <= 1024 && N >= 2048 && N % 256 == 0 &&
            k_blocks / std::max(1, c.splits) >= 16) ? 1 : 0;
  // u8 x s8 on several waves of tiles: pairs measured 8192^3 393.5 against 418.6 us, 4096^3 68.5 against 70.5 us
  // (1024 x 4096 x 4096, a single wave: 31.7 against 31.9 us - left on one CTA per tile)
  if (!c.swapped && dtype_bytes == 1 && c.bn == 256 && c.kpb <= 1 && c.splits == 1 && M % 256 == 0 && N % 256 == 0 &&
      tiles >= 2 * sm_count && k_blocks >= 16)
    c.pair = 1;
  c.grid = std::min(tiles * c.splits, sm_count);
  if (const char *ov = std::getenv("GC_B200_TILE")) {
    // "bn,splits,stages,group_m" — any field may be 0 to keep the heuristic's choice
    int bn = 0, sp = 0, st = 0, gm = 0, pr = -1, kp = 0;
    if (std::sscanf(ov, "%d,%d,%d,%d,%d,%d", &bn, &sp, &st, &gm, &pr, &kp) >= 1) {
      if (pr >= 0) c.pair = pr;
      if (kp > 0) c.kpb = kp;
      if (bn > 0 && !c.swapped) c.bn = bn;
      if (sp > 0) { const int per = ceil_div(k_blocks, sp); c.splits = ceil_div(k_blocks, per); }
      if (st > 0) c.stages = std::min(st, c.stages);
      if (gm > 0) c.group_m = gm;
      const int t2 = c.swapped ? ceil_div(N, 128) : ceil_div(M, 128) * ceil_div(N, c.bn);
      c.grid = std::min(t2 * c.splits, sm_count);
    }
  }
  return c;
}

size_t matmul_scratch_bytes(int64_t M, int64_t N, int64_t K, int dtype_bytes, int out_bytes, int sm_count) {
  const MatmulConfig c = select_matmul_config(M, N, K, dtype_bytes, out_bytes, sm_count);
  return c.splits > 1 ? size_t(c.splits) * size_t(M) * size_t(N) * 4 : 0;
}

// ----------------------------------------------------------------------------- matmul planning
OperandGeom operand_geom(bool mn_major, int tile_mn, int elem_bytes, int kpb) {
  OperandGeom g{};
  const uint32_t bk = 128 / elem_bytes;  // K elements per 128-byte K block
  g.mn_major = mn_major ? 1u : 0u;
  if (!mn_major) {
    // [K block][MN row][128 B]: each K block is its own swizzled [tile_mn x 128 B] tile
    g.boxes = uint32_t(kpb);
    g.box_bytes = uint32_t(tile_mn) * 128u;
    g.box_mn = uint32_t(tile_mn);
    g.lbo = 16;
    g.sbo = 1024;
    g.kstep = 32;
    g.sub_step = g.box_bytes;
    g.bytes = g.boxes * g.box_bytes;
    g.one_load = kpb == 1 ? 1u : 0u;
  } else {
    // [MN group][K row][128 B]: the K blocks of a stage are consecutive rows of every group
    g.box_mn = 128 / elem_bytes;
    g.boxes = (uint32_t(tile_mn) + g.box_mn - 1) / g.box_mn;
    g.box_bytes = bk * uint32_t(kpb) * 128u;
    g.lbo = g.box_bytes;
    g.sbo = 1024;
    g.kstep = (32u / elem_bytes) * 128u;
    g.sub_step = bk * 128u;
    g.bytes = g.boxes * g.box_bytes;
  }
  return g;
}

CUtensorMap operand_tmap(OperandGeom &g, ElemType t, int elem_bytes, const void *ptr, int64_t mn_total,
                                int64_t k_total, int tile_mn, int kpb) {
  const uint32_t bk = 128 / elem_bytes;
  if (g.mn_major && elem_bytes == 2 && mn_total % int64_t(g.box_mn) == 0 && tile_mn % int(g.box_mn) == 0) {
    // memory [k_total][mn_total] seen as [group][k][128 bytes]: one copy brings all 64-wide (128-byte)
    // groups of the tile, landing as consecutive [rows x 128 B] blocks — the layout the MMA reads.
    // Only when MN is a whole number of groups: a partial last group would make the copy read past
    // the end of the last row; and only when the tile is a whole number of groups wide, so that every
    // tile starts on a group boundary (tiles of 16 x odd columns take one 2-D copy per group instead).  16-bit operands only: the same 3-D form on 8-bit operands returned
    // wrong data for the second group at small N on B200, so those keep one 2-D copy per group.
    g.one_load = 1;
    return make_tmap_3d(t, ptr, g.box_mn, uint64_t(k_total), uint64_t(mn_total) / g.box_mn,
                        uint64_t(mn_total) * elem_bytes, 128, g.box_mn, bk * uint32_t(kpb), g.boxes);
  }
  if (!g.mn_major) {  // memory [mn_total][k_total], K contiguous
    if (kpb > 1 && elem_bytes == 2 && k_total % int64_t(bk) == 0) {
      // [K block][mn][128 bytes]: one copy brings the stage's K blocks as consecutive swizzled tiles.
      // Only when K is a whole number of blocks (a partial block would read into the next row).
      g.one_load = 1;
      g.k3d = 1;
      return make_tmap_3d(t, ptr, bk, uint64_t(mn_total), uint64_t(k_total) / bk, uint64_t(k_total) * elem_bytes, 128, bk,
                          uint32_t(tile_mn), uint32_t(kpb));
    }
    return make_tmap_2d(t, ptr, uint64_t(k_total), uint64_t(mn_total), uint64_t(k_total) * elem_bytes, bk,
                        uint32_t(tile_mn));
  }
  // memory [k_total][mn_total], MN contiguous
  return make_tmap_2d(t, ptr, uint64_t(mn_total), uint64_t(k_total), uint64_t(mn_total) * elem_bytes, g.box_mn,
                      bk * uint32_t(kpb));
}

void matmul_tc(const MatmulArgs &a, cudaStream_t stream) {
  DeviceState &dev = device_state();
  const int eb = a.int8 ? 1 : 2;
  const int out_bytes = a.out_kind == OUT_BF16 ? 2 : 4;
  // partial sums that leave through peer stores are not split along K here: choose the tile knowing that
  const int max_splits = (a.n_peers > 0) ? 1 : 8;
  MatmulConfig cfg = a.force ? *a.force : select_matmul_config(a.M, a.N, a.K, eb, out_bytes, dev.sm_count, max_splits);
  const int64_t ld_out = a.ld_out ? a.ld_out : a.N;

  GemmParams p{};
  p.K = int(a.K);
  p.bk_elems = 128 / eb;
  p.k_blocks = ceil_div(a.K, p.bk_elems);
  p.splits = cfg.splits;
  p.stages = cfg.stages;
  p.group_m = cfg.group_m;
  p.BN = cfg.bn;
  p.out_rows = int(a.M);
  p.out_cols = int(a.N);
  p.error = dev.d_error;
  p.trace = a.trace;

  // operand roles in MMA orientation
  const void *pa, *pb;
  bool a_mn, b_mn;
  int64_t mn_a, mn_b;
  ElemType ta, tb;
  uint32_t fa, fb;
  if (!cfg.swapped) {
    pa = a.A; a_mn = a.trans_a != 0; mn_a = a.M;
    pb = a.B; b_mn = a.trans_b == 0; mn_b = a.N;
    ta = a.int8 ? ElemType::U8 : ElemType::BF16; tb = a.int8 ? ElemType::S8 : ElemType::BF16;
    fa = a.int8 ? 0u : 1u; fb = 1u;
  } else {
    pa = a.B; a_mn = a.trans_b == 0; mn_a = a.N;
    pb = a.A; b_mn = a.trans_a != 0; mn_b = a.M;
    ta = a.int8 ? ElemType::S8 : ElemType::BF16; tb = a.int8 ? ElemType::U8 : ElemType::BF16;
    fa = 1u; fb = a.int8 ? 0u : 1u;
  }
  // the pair kernel splits the B tile in halves of bn/2 columns; 8-bit MN-major operands are fetched
  // in 128-column groups, so their half must be 128 wide
  const bool pair = cfg.pair && !cfg.swapped && !(a.int8 && cfg.bn != 256);
  p.Mm = int(mn_a);
  p.Nm = int(mn_b);
  p.tiles_m = ceil_div(mn_a, pair ? 256 : 128);
  p.tiles_n = ceil_div(mn_b, p.BN);
  // K blocks per stage: only the one-CTA kernel, and with split-K only when every split is a whole
  // number of stages (a stage must not straddle two splits)
  int kpb = (pair || cfg.kpb < 1) ? 1 : cfg.kpb;
  {
    const int per = ceil_div(p.k_blocks, p.splits);
    if (p.splits > 1 && per % kpb) kpb = 1;
    if (kpb > p.k_blocks) kpb = 1;
  }
  p.kpb = kpb;
  p.a = operand_geom(a_mn, 128, eb, kpb);
  p.b = operand_geom(b_mn, pair ? p.BN / 2 : p.BN, eb, kpb);
  p.idesc = umma_instr_desc(a.int8 ? 2u : 1u, fa, fb, a_mn ? 1u : 0u, b_mn ? 1u : 0u, pair ? 256u : 128u, uint32_t(p.BN));
  uint32_t cols = 32;
  while (cols < uint32_t(2 * p.BN)) cols <<= 1;
  p.tmem_cols = cols;

  const CUtensorMap tmA = operand_tmap(p.a, ta, eb, pa, mn_a, a.K, 128, kpb);
  const CUtensorMap tmB = operand_tmap(p.b, tb, eb, pb, mn_b, a.K, pair ? p.BN / 2 : p.BN, kpb);

  if (a.n_peers > 0) {
    // f32 partial planes ([planes][M][N], pitch N) or finished results (bf16 / dequantised f32 with their
    // post-ops, any 16-byte aligned pitch): every store is a full 16-byte chunk
    const int per16 = a.out_kind == OUT_BF16 ? 8 : 4;
    const size_t pitch_b = size_t(a.ld_out ? a.ld_out : a.N) * (a.out_kind == OUT_BF16 ? 2 : 4);
    // (the weight-stationary form stores single elements and has no such constraint; it takes finished results only)
    if ((a.out_kind != OUT_F32 && a.out_kind != OUT_BF16 && a.out_kind != OUT_DEQUANT_F32) || a.n_peers > 8 || a.acc_dump ||
        (cfg.swapped ? a.out_kind == OUT_F32 : ((a.N % per16) != 0 || (pitch_b % 16) != 0)))
      throw std::invalid_argument("peer stores need whole 16-byte chunks per row and at most 8 peers");
    if (a.out_kind != OUT_F32 && (a.peer_plane != 0 || a.peer_rows != 0))
      throw std::invalid_argument("planes and row scatter exist for f32 partial sums only");
    // no K split, except for the row scatter when the caller has sized the owners' buffers for one plane per split
    const int keep = (a.peer_rows > 0 && a.force && a.peer_splits == cfg.splits) ? cfg.splits : 1;
    cfg.splits = keep;
    p.splits = keep;
    if (a.peer_rows > 0 && (a.peer_rows * a.n_peers != a.M)) throw std::invalid_argument("row scatter needs M = peers x rows per peer");
    if (a.peer_multicast && (a.n_peers != 1 || a.peer_rows != 0 || cfg.swapped))
      throw std::invalid_argument("multicast stores take one address, every rank receives everything, row-major form only");
    p.peer_multicast = a.peer_multicast;
    p.n_peers = a.n_peers;
    p.peer_plane = a.peer_plane;
    p.peer_rows = a.peer_rows;
    for (int d = 0; d < a.n_peers; ++d) p.peer_out[d] = a.peer_out[d];
    if (a.signal_peer) {
      // one increment per epilogue warp (32 rows) and tile: a warp's rows must all belong to one owner
      if (a.peer_rows <= 0 || a.peer_rows % 32 || cfg.swapped || a.M % 128)
        throw std::invalid_argument("counted row scatter needs rows per peer that are a multiple of 32, M a multiple of 128 and the row-major kernel");
      for (int d = 0; d < a.n_peers; ++d) {
        if (!a.signal_peer[d]) throw std::invalid_argument("null peer counter");
        p.signal_peer[d] = a.signal_peer[d];
      }
      if (a.arrivals_per_peer) *a.arrivals_per_peer = p.tiles_n * (a.peer_rows / 32) * p.splits;
    }
  }
  if (a.wait_counter) {
    if (!a.epoch) throw std::invalid_argument("a counter wait needs the step counter");
    p.wait_counter = a.wait_counter;
    p.epoch = a.epoch;
    p.wait_per_step = a.wait_per_step;
  }
  const bool split = cfg.splits > 1 && a.n_peers == 0;   // (with peers the planes live at the owners)
  void *planes = nullptr;
  if (split) {
    const size_t need = size_t(cfg.splits) * size_t(a.M) * size_t(a.N) * 4;
    // the caller's scratch (an executable's own, sized when it was prepared) when it is large enough; the
    // per-device workspace otherwise (direct launchers, or a configuration recorded after the executable was prepared)
    if (a.scratch && a.scratch_bytes >= need) planes = a.scratch;
    else planes = dev.ensure_workspace(need);
    p.out_kind = a.int8 ? OUT_S32 : OUT_F32;
    p.out = planes;
    p.ld_out = a.N;
    p.split_stride = a.M * a.N;
    p.bias_kind = BIAS_NONE;
    p.relu = 0;
  } else {
    p.out_kind = a.out_kind;
    p.out = a.out;
    p.ld_out = ld_out;
    p.split_stride = 0;
    p.bias_kind = a.bias_kind;
    p.bias = a.bias;
    p.scale = a.scale;
    p.comp = a.comp;
    p.acc_dump = a.acc_dump;
    p.ld_dump = a.N;
    p.relu = a.relu;
  }
  // TMA-store epilogue: bf16 outputs (bias / ReLU applied in registers) and raw f32 / s32 planes, when the
  // copy engine can address the output (16-byte aligned base and row pitch)
  if (!cfg.swapped && a.n_peers == 0 && p.acc_dump == nullptr) {
    const int esz = p.out_kind == OUT_BF16 ? 2 : 4;
    const bool plain = p.out_kind == OUT_BF16          ? (p.bias_kind == BIAS_NONE || p.bias_kind == BIAS_BF16)
                       : p.out_kind == OUT_DEQUANT_F32 ? (p.bias_kind == BIAS_NONE || p.bias_kind == BIAS_F32)
                                                       : ((p.out_kind == OUT_F32 || p.out_kind == OUT_S32) && p.bias_kind == BIAS_NONE && !p.relu);
    if (plain && tma_compatible(p.out, p.ld_out, esz) && (!split || (size_t(p.split_stride) * esz) % 16 == 0)) {
      const ElemType ct = p.out_kind == OUT_BF16 ? ElemType::BF16 : (p.out_kind == OUT_S32 ? ElemType::S32 : ElemType::F32);
      p.tmC = make_tmap_3d(ct, p.out, uint64_t(a.N), uint64_t(a.M), uint64_t(std::max(1, p.splits)), uint64_t(p.ld_out) * esz,
                           split ? uint64_t(p.split_stride) * esz : uint64_t(a.M) * uint64_t(p.ld_out) * esz, 128 / esz, 32, 1);
      p.tma_store = 1;
    }
  }
  // Row scatter of f32 partial sums: through the copy engine as well, one tensor map per owner (tile widths that are
  // whole 32-column slabs; GC_B200_PEER_TMA=0 keeps the register-store form)
  if (!cfg.swapped && a.n_peers > 0 && a.peer_rows > 0 && a.peer_rows % 32 == 0 && a.out_kind == OUT_F32 && !a.peer_multicast &&
      p.BN % 32 == 0 && a.N % 4 == 0) {
    static const bool on = [] { const char *e = std::getenv("GC_B200_PEER_TMA"); return !(e && e[0] == '0'); }();
    bool ok = on;
    for (int d = 0; d < a.n_peers && ok; ++d) ok = tma_compatible(a.peer_out[d], a.N, 4);
    if (ok) {
      const uint64_t planes = uint64_t(a.n_peers) * uint64_t(p.splits);
      for (int d = 0; d < a.n_peers; ++d)
        p.tmPeer[d] = make_tmap_3d(ElemType::F32, a.peer_out[d], uint64_t(a.N), uint64_t(a.peer_rows), planes, uint64_t(a.N) * 4,
                                   uint64_t(a.peer_rows) * uint64_t(a.N) * 4, 32, 32, 1);
      p.tma_store = 1;
      p.tma_peer = 1;
    }
  }
  // All-gather of C through the copy engine: every finished slab is stored once per rank from shared memory (one
  // cp.async.bulk.tensor store per rank and slab instead of a loop of 16-byte stores per thread and rank)
  if (!cfg.swapped && a.n_peers > 0 && a.peer_rows == 0 && !a.peer_multicast && p.acc_dump == nullptr && p.splits == 1 &&
      (a.out_kind == OUT_BF16 || a.out_kind == OUT_DEQUANT_F32)) {
    static const bool on = [] { const char *e = std::getenv("GC_B200_PEER_TMA"); return !(e && e[0] == '0'); }();
    const int esz = a.out_kind == OUT_BF16 ? 2 : 4;
    const bool plain = a.out_kind == OUT_BF16 ? (a.bias_kind == BIAS_NONE || a.bias_kind == BIAS_BF16) : (a.bias_kind == BIAS_NONE || a.bias_kind == BIAS_F32);
    bool ok = on && plain && p.BN % (128 / esz) == 0;
    for (int d = 0; d < a.n_peers && ok; ++d) ok = tma_compatible(a.peer_out[d], ld_out, esz);
    if (ok) {
      const ElemType ct = a.out_kind == OUT_BF16 ? ElemType::BF16 : ElemType::F32;
      for (int d = 0; d < a.n_peers; ++d)
        p.tmPeer[d] = make_tmap_3d(ct, a.peer_out[d], uint64_t(a.N), uint64_t(a.M), 1, uint64_t(ld_out) * esz,
                                   uint64_t(a.M) * uint64_t(ld_out) * esz, 128 / esz, 32, 1);
      p.tma_store = 1;
      p.tma_peer = 2;
    }
  }
  const int units = p.tiles_m * p.tiles_n * p.splits;
  cudaError_t e;
  if (pair) {
    // stages are sized for the half B tile: recompute against the shared-memory budget
    const size_t budget = 232448 - 1024 - 4 * 8192 - 256;
    p.stages = int(std::max<size_t>(2, std::min<size_t>({size_t(8), budget / (p.a.bytes + p.b.bytes), size_t(std::max(2, p.k_blocks))})));
    if (a.force && a.force->stages >= 2) p.stages = std::min(p.stages, a.force->stages);
    const int grid = std::max(2, std::min(2 * units, dev.sm_count & ~1));
    const size_t smem = gemm_pair_smem_bytes(p);
    if (smem > 232448) throw std::invalid_argument("matmul tile configuration exceeds shared memory");
    e = a.int8 ? launch_gemm_pair_kernel<1>(tmA, tmB, p, grid, smem, stream)
               : launch_gemm_pair_kernel<0>(tmA, tmB, p, grid, smem, stream);
  } else {
    const int grid = std::max(1, std::min(units, cfg.grid > 0 ? cfg.grid : dev.sm_count));
    {
      const size_t budget = 232448 - 1024 - 4 * 8192 - 256;
      const int fit = int(budget / (p.a.bytes + p.b.bytes));
      if (fit < 2) throw std::invalid_argument("matmul stage does not fit twice in shared memory");
      p.stages = std::max(2, std::min({p.stages, fit, std::max(2, ceil_div(p.k_blocks, kpb))}));
      if (kpb > 1) p.stages = std::min(8, fit);
    }
    const size_t smem = gemm_smem_bytes(p);
    if (smem > 232448) throw std::invalid_argument("matmul tile configuration exceeds shared memory");
    if (!a.int8) e = cfg.swapped ? launch_gemm_kernel<0, true>(tmA, tmB, p, grid, smem, stream)
                                 : launch_gemm_kernel<0, false>(tmA, tmB, p, grid, smem, stream);
    else         e = cfg.swapped ? launch_gemm_kernel<1, true>(tmA, tmB, p, grid, smem, stream)
                                 : launch_gemm_kernel<1, false>(tmA, tmB, p, grid, smem, stream);
  }
  if (e != cudaSuccess) throw CudaError(std::string("gemm launch: ") + cudaGetErrorString(e));
  count_launch();
  if (split) {
    if (ld_out != a.N) throw std::invalid_argument("split-K with a strided output is not supported");
    reduce_planes(planes, cfg.splits, a.M * a.N, a.out, a.M, a.N, a.out_kind, a.bias_kind, a.bias, a.scale, a.comp,
                  a.acc_dump, a.relu, stream);
  }
}

// ----------------------------------------------------------------------------- helper kernels
// Sum split-K planes in split order (deterministic) and apply the epilogue.
template <bool INT>
__global__ void reduce_planes_kernel(const void *parts, int nparts, long long plane, void *out, long long M,
                                     long long N, int out_kind, int bias_kind, const void *bias, const float *scale,
                                     const int32_t *comp, int32_t *acc_dump, int relu) {
  const long long total = M * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int col = int(i % N);
    if (INT) {
      const int32_t *p = reinterpret_cast<const int32_t *>(parts);
      int32_t s = p[i];
      for (int k = 1; k < nparts; ++k) s += p[(long long)k * plane + i];
      if (acc_dump) acc_dump[i] = s;
      if (out_kind == OUT_S32) {
        reinterpret_cast<int32_t *>(out)[i] = s;
      } else {
        float f = __fmul_rn(float(s - (comp ? comp[col] : 0)), scale[col]);
        if (bias_kind == BIAS_F32) f = __fadd_rn(f, reinterpret_cast<const float *>(bias)[col]);
        if (relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
        reinterpret_cast<float *>(out)[i] = f;
      }
    } else {
      const float *p = reinterpret_cast<const float *>(parts);
      float s = p[i];
      for (int k = 1; k < nparts; ++k) s = __fadd_rn(s, p[(long long)k * plane + i]);
      if (out_kind == OUT_F32) {
        if (bias_kind == BIAS_F32) s = __fadd_rn(s, reinterpret_cast<const float *>(bias)[col]);
        if (relu) s = (s != s) ? s : (s > 0.f ? s : 0.f);
        reinterpret_cast<float *>(out)[i] = s;
      } else {
        uint32_t y = f32_to_bf16_bits(s);
        if (bias_kind == BIAS_BF16) {
          const uint32_t b = reinterpret_cast<const uint16_t *>(bias)[col];
          y = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(y), bf16_bits_to_f32(b)));
        }
        if (relu) { const float f = bf16_bits_to_f32(y); y = (f != f) ? y : (f > 0.f ? y : 0u); }
        reinterpret_cast<uint16_t *>(out)[i] = uint16_t(y);
      }
    }
  }
}

// The common case, f32 planes -> bf16 (+bias, ReLU), four columns per thread with 16-byte loads.  Same
// arithmetic as the scalar kernel: planes added in split order, one rounding, bias in f32, second rounding.
__global__ void __launch_bounds__(256)
reduce_planes_bf16x4_kernel(const float4 *parts, int nparts, long long plane4, uint2 *out, long long total4, int n4,
                            const uint2 *bias, int relu) {
  pdl_launch_dependents();
  pdl_wait();   // the planes come from the kernel ahead in the stream
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
    // four planes' loads in flight before the first add (additions stay in split order)
    float4 s = parts[i];
    for (int k = 1; k < nparts; k += 4) {
      float4 t[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (k + u < nparts) t[u] = parts[(long long)(k + u) * plane4 + i];
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
    out[i] = make_uint2(bf16x2_fix_nan(lo), bf16x2_fix_nan(hi));
  }
}

struct PeerPtrs { uint2 *p[8]; };
// The reduction of one rank's row slice, stored into every peer's result buffer (see runtime.h).
__global__ void __launch_bounds__(256)
reduce_slice_bcast_kernel(const float4 *parts, int nparts, long long plane4, long long total4, int n4, const uint2 *bias,
                          int relu, PeerPtrs out, int n_peers, long long dst4) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
    float4 s = parts[i];
    for (int k = 1; k < nparts; ++k) {
      const float4 t = parts[(long long)k * plane4 + i];
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
    const uint2 v = make_uint2(bf16x2_fix_nan(lo), bf16x2_fix_nan(hi));
    for (int d = 0; d < n_peers; ++d) out.p[d][dst4 + i] = v;
  }
}

void reduce_slice_broadcast_bf16(const float *parts, int nparts, int64_t rows, int64_t N, const void *bias_bf16,
                                 void *const *peer_out, int n_peers, int64_t row0, int relu, cudaStream_t stream) {
  DeviceState &dev = device_state();
  auto al = [](const void *q, size_t a) { return (reinterpret_cast<uintptr_t>(q) & (a - 1)) == 0; };
  if (nparts < 1 || n_peers < 1 || n_peers > 8 || rows <= 0 || N <= 0 || N % 4 || !al(parts, 16) || (bias_bf16 && !al(bias_bf16, 8)))
    throw std::invalid_argument("reduce_slice_broadcast: N must be a multiple of 4, planes 16-byte and bias 8-byte aligned, 1..8 peers");
  PeerPtrs pp{};
  for (int d = 0; d < n_peers; ++d) {
    if (!peer_out[d] || !al(peer_out[d], 8)) throw std::invalid_argument("reduce_slice_broadcast: peer buffers must be 8-byte aligned");
    pp.p[d] = reinterpret_cast<uint2 *>(peer_out[d]);
  }
  const long long total4 = rows * N / 4;
  const int threads = 256;
  const int blocks = int(std::min<long long>((total4 + threads - 1) / threads, (long long)dev.sm_count * 8));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(std::max(blocks, 1)));
  cfg.blockDim = dim3(threads);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  GCB_CUDA(cudaLaunchKernelEx(&cfg, reduce_slice_bcast_kernel, reinterpret_cast<const float4 *>(parts), nparts, (long long)(rows * N / 4),
                              total4, int(N / 4), reinterpret_cast<const uint2 *>(bias_bf16), relu, pp, n_peers,
                              (long long)(row0 * N / 4)));
  count_launch();
}

void reduce_planes(const void *parts, int nparts, int64_t plane, void *out, int64_t M, int64_t N, int out_kind,
                   int bias_kind, const void *bias, const float *scale, const int32_t *comp, int32_t *acc_dump,
                   int relu, cudaStream_t stream) {
  DeviceState &dev = device_state();
  const long long total = M * N;
  const int threads = 256;
  const int blocks = int(std::min<long long>((total + threads - 1) / threads, (long long)dev.sm_count * 8));
  const bool is_int = (out_kind == OUT_S32 || out_kind == OUT_DEQUANT_F32);
  auto al = [](const void *q, size_t a) { return (reinterpret_cast<uintptr_t>(q) & (a - 1)) == 0; };
  if (!is_int && out_kind == OUT_BF16 && (bias_kind == BIAS_NONE || bias_kind == BIAS_BF16) && N % 4 == 0 && plane % 4 == 0 &&
      al(parts, 16) && al(out, 8) && (bias_kind == BIAS_NONE || al(bias, 8)) && N / 4 < (1 << 30)) {
    const long long total4 = total / 4;
    const int blocks4 = int(std::min<long long>((total4 + threads - 1) / threads, (long long)dev.sm_count * 8));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(std::max(blocks4, 1)));
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    GCB_CUDA(cudaLaunchKernelEx(&cfg, reduce_planes_bf16x4_kernel, reinterpret_cast<const float4 *>(parts), nparts,
                                (long long)(plane / 4), reinterpret_cast<uint2 *>(out), total4, int(N / 4),
                                bias_kind == BIAS_BF16 ? reinterpret_cast<const uint2 *>(bias) : nullptr, relu));
    count_launch();
    return;
  }
  if (is_int)
    reduce_planes_kernel<true><<<blocks, threads, 0, stream>>>(parts, nparts, plane, out, M, N, out_kind, bias_kind,
                                                              bias, scale, comp, acc_dump, relu);
  else
    reduce_planes_kernel<false><<<blocks, threads, 0, stream>>>(parts, nparts, plane, out, M, N, out_kind, bias_kind,
                                                               bias, scale, comp, acc_dump, relu);
  GCB_CUDA(cudaGetLastError());
  count_launch();
}

void reduce_epilogue_bf16(const float *parts, int nparts, int64_t plane, const void *bias_bf16, void *out_bf16,
                          int64_t M, int64_t N, int relu, cudaStream_t stream) {
  reduce_planes(parts, nparts, plane, out_bf16, M, N, OUT_BF16, bias_bf16 ? BIAS_BF16 : BIAS_NONE, bias_bf16, nullptr,
                nullptr, nullptr, relu, stream);
}

// comp[n] = zp * sum_k W[k][n].  One thread per column, rows strided over
// blockIdx.y with an exact integer atomic combine.
__global__ void colsum_s8_kernel(const int8_t *W, int32_t *comp, long long K, long long N, int32_t zp) {
  const long long n = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (n >= N) return;
  int32_t s = 0;
  for (long long k = blockIdx.y; k < K; k += gridDim.y) s += int32_t(W[k * N + n]);
  atomicAdd(&comp[n], s * zp);
}

void colsum_s8(const int8_t *W, int32_t *comp, int64_t K, int64_t N, int32_t zp, cudaStream_t stream) {
  GCB_CUDA(cudaMemsetAsync(comp, 0, size_t(N) * 4, stream));
  dim3 grid(unsigned((N + 255) / 256), unsigned(std::min<int64_t>(K, 64)));
  colsum_s8_kernel<<<grid, 256, 0, stream>>>(W, comp, K, N, zp);
  GCB_CUDA(cudaGetLastError());
  count_launch();
}

// Exact-order SIMT matmul: every output element accumulates k ascending with a
// separate multiply and add, the arithmetic of the reference's scalar loops
// (BrgemmNaive.cpp:46-99).  64x64 output tile, 16-deep K slabs in shared memory.
template <int IN_KIND>
__global__ void __launch_bounds__(256) matmul_simt_kernel(const void *Ap, const void *Bp, const void *biasp, void *outp,
                                                         int M, int N, int K, int ta, int tb, int relu) {
  __shared__ float As[16][65];
  __shared__ float Bs[16][65];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  auto ld = [&](const void *base, long long idx) -> float {
    if (IN_KIND == 0) return reinterpret_cast<const float *>(base)[idx];
    return bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(base)[idx]);
  };
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int e = threadIdx.x; e < 16 * 64; e += 256) {
      const int kk = e / 64, mm = e % 64;
      const int k = k0 + kk;
      float av = 0.f, bv = 0.f;
      if (k < K && m0 + mm < M) av = ta ? ld(Ap, (long long)k * M + (m0 + mm)) : ld(Ap, (long long)(m0 + mm) * K + k);
      if (k < K && n0 + mm < N) bv = tb ? ld(Bp, (long long)(n0 + mm) * K + k) : ld(Bp, (long long)k * N + (n0 + mm));
      As[kk][mm] = av;
      Bs[kk][mm] = bv;
    }
    __syncthreads();
    const int klim = min(16, K - k0);
    for (int kk = 0; kk < klim; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m >= M || n >= N) continue;
      if (IN_KIND == 0) {
        float v = acc[i][j];
        if (biasp) v = __fadd_rn(v, reinterpret_cast<const float *>(biasp)[n]);
        if (relu) v = (v != v) ? v : (v > 0.f ? v : 0.f);
        reinterpret_cast<float *>(outp)[(long long)m * N + n] = v;
      } else {
        uint32_t y = f32_to_bf16_bits(acc[i][j]);
        if (biasp)
          y = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(y), bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(biasp)[n])));
        if (relu) { const float f = bf16_bits_to_f32(y); y = (f != f) ? y : (f > 0.f ? y : 0u); }
        reinterpret_cast<uint16_t *>(outp)[(long long)m * N + n] = uint16_t(y);
      }
    }
}

void matmul_simt(const void *A, const void *B, const void *bias, void *out, int64_t M, int64_t N, int64_t K,
                 int trans_a, int trans_b, int in_kind, int relu, cudaStream_t stream) {
  device_state();
  dim3 grid(unsigned((N + 63) / 64), unsigned((M + 63) / 64));
  if (in_kind == 0)
    matmul_simt_kernel<0><<<grid, 256, 0, stream>>>(A, B, bias, out, int(M), int(N), int(K), trans_a, trans_b, relu);
  else
    matmul_simt_kernel<1><<<grid, 256, 0, stream>>>(A, B, bias, out, int(M), int(N), int(K), trans_a, trans_b, relu);
  GCB_CUDA(cudaGetLastError());
  count_launch();
}

} // namespace gcb
