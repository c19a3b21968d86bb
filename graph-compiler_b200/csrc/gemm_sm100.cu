// Persistent, warp-specialised GEMM for sm_100a.
//
// This single kernel replaces the reference's whole deep-tiled loop nest
// (lib/gc/Transforms/DeepTileContractionOp.cpp:545-949: 3 thread loops x 3 L2
// loops x 3 L1 loops) together with the brgemm microkernel it calls per
// innermost tile (lib/gc/ExecutionEngine/CPURuntime/Microkernel/
// BrgemmOnednn.cpp:145-168) and the elementwise post-ops that
// IterativeTilingAndFusion.cpp:743-828 fuses behind the last K block.
//
//   warps 0, 6  TMA producers (A and B): cp.async.bulk.tensor tiles into a
//               ring of 128-byte-swizzled shared-memory stages
//   warp 1      MMA issuer: tcgen05.mma (kind::f16 or kind::i8), accumulators
//               in tensor memory, two accumulator buffers so that the epilogue
//               of tile t overlaps the main loop of tile t+1
//   warps 2..5  epilogue: tcgen05.ld -> registers -> post-ops -> swizzled
//               shared-memory staging -> 128-byte coalesced global stores
//
// Numerics of the bf16 epilogue follow the reference exactly: one RNE cast of
// the f32 accumulator at the last K block (DeepTileContractionOp.cpp:872-889),
// bias add evaluated in f32 and rounded again (Pipeline.cpp:81-90), ReLU as
// max(x, 0) on the rounded value (OneDNNGraphToLinalg.cpp:355-358).
#include "gemm_epilogue.cuh"
#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace gcb {

constexpr int kThreads = 224;
constexpr int kBM = 128;             // MMA M (cta_group::1)
constexpr int kStageStaging = 8192;  // per epilogue warp: two slabs of 32 rows x 128 B
constexpr int kMaxStages = 8;

struct SmemBarriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

size_t gemm_smem_bytes(const GemmParams &p) {
  return 1024 /*alignment slack*/ + size_t(p.stages) * (p.a.bytes + p.b.bytes) + 4 * kStageStaging +
         sizeof(SmemBarriers);
}

__device__ __forceinline__ void tile_coords(const GemmParams &p, int tile, int &tm, int &tn) {
  // Grouped rasterisation: walk `group_m` tile rows per column sweep so that
  // CTAs running at the same time share A row panels and B column panels in L2.
  const int per_group = p.group_m * p.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.tiles_m - first_m, p.group_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

// Bounded wait until this step's rows of the activations (stored by other GPUs' kernels) have landed here.
__device__ __forceinline__ bool peer_rows_landed(const GemmParams &p) {
  const uint32_t target = (*reinterpret_cast<const volatile uint32_t *>(p.epoch) + 1u) * p.wait_per_step;
  return wait_counter_reached(p.wait_counter, target, 4 * WAIT_LIMIT_CYCLES);
}

template <int KIND, bool SWAPPED>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);
  const uint32_t stage_bytes = p.a.bytes + p.b.bytes;
  uint8_t *staging = smem + size_t(p.stages) * stage_bytes;
  SmemBarriers *bars = reinterpret_cast<SmemBarriers *>(staging + 4 * kStageStaging);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int units = p.tiles_m * p.tiles_n * p.splits;
  const int kb_per_split = (p.k_blocks + p.splits - 1) / p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 2);   // one expect-tx arrive per producer warp
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars->tmem_full[b]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[b]), 4);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(&bars->tmem_base);
  // Everything above touched only shared and tensor memory and may overlap the tail of the kernel
  // ahead in the stream; from here on operands are read and results written.
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_store(p.trace, 0);
  pdl_launch_dependents();
  pdl_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_store(p.trace, 1);

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------------ TMA producers
    // warp 0 streams the A operand, warp 6 the B operand.  Each is one thread whose instruction
    // stream is serial, so the per-stage work is kept to: wait, expect-tx, ONE tensor copy.
    if (lane == 0) {
      const bool is_a = (warp == 0);
      const CUtensorMap *tm = is_a ? &tmA : &tmB;
      const OperandGeom &g = is_a ? p.a : p.b;
      tma_prefetch_desc(tm);
      uint32_t it = 0;            // stages issued over the whole kernel (tear-down only)
      int s = 0;                  // ring position and phase, carried instead of derived
      uint32_t ph = 0;
      const int stages = p.stages;
      const uint32_t my_bytes = g.bytes, my_off = is_a ? 0u : p.a.bytes;
      const uint32_t boxes = g.boxes, box_bytes = g.box_bytes, box_mn = g.box_mn;
      const bool mn = g.mn_major != 0, one = g.one_load != 0, k3d = g.k3d != 0;
      const int bk = p.bk_elems, kpb = max(p.kpb, 1);
      int err = 0;
      // Activations that other GPUs' kernels store into this GPU's memory: their producer waits for this step's rows
      // before its first load; the weight producer fills the ring first (weights are local) and waits before it would
      // block on a stage the MMA thread cannot have released yet, so that no mbarrier wait of this CTA starts its
      // clock while the rows are still on their way.
      const bool gated = p.wait_counter != nullptr;
      const bool is_act = (is_a != SWAPPED);
      bool gate_open = !gated;
      auto peer_gate = [&]() {
        if (!peer_rows_landed(p)) err = ERR_WAIT_PEER;
        fence_proxy_async_global();
        gate_open = true;
        trace_max(p.trace, 2);
      };
      if (gated && is_act) peer_gate();
      for (int u = blockIdx.x; u < units && !err; u += gridDim.x) {
        const int tile = u / p.splits, split = u - tile * p.splits;
        int tm_, tn_;
        tile_coords(p, tile, tm_, tn_);
        const int mn_off = is_a ? tm_ * kBM : tn_ * p.BN;
        const int kb0 = split * kb_per_split, kb1 = min(p.k_blocks, kb0 + kb_per_split);
        int k_off = kb0 * bk;
        const int grp = mn_off / int(box_mn ? box_mn : 1u);   // 3-D form: index of the first 64-wide MN group
        for (int kb = kb0; kb < kb1; kb += kpb, ++it, k_off += bk * kpb) {
          if (!gate_open && it >= uint32_t(stages)) { peer_gate(); if (err) break; }
          if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u)) { err = ERR_WAIT_EMPTY; break; }
          const uint32_t full = smem_u32(&bars->full[s]);
          mbar_expect_tx(full, my_bytes);
          const uint32_t dst = base + uint32_t(s) * stage_bytes + my_off;
          if (!mn) {
            if (k3d) tma_load_3d(dst, tm, full, 0, mn_off, kb);
            else
              for (uint32_t i = 0; i < boxes; ++i) tma_load_2d(dst + i * box_bytes, tm, full, k_off + int(i) * bk, mn_off);
          } else if (one) {
            tma_load_3d(dst, tm, full, 0, k_off, grp);
          } else {
            for (uint32_t i = 0; i < boxes; ++i) tma_load_2d(dst + i * box_bytes, tm, full, mn_off + int(i * box_mn), k_off);
          }
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      if (err) { atomicExch(p.error, err); bars->abort_flag = 1; }
      // Tear-down: every copy this thread issued must have landed before the CTA
      // may exit.  In the normal path the MMA warp has consumed them all; after an
      // abort wait (bounded) for the stages still in flight.
      if (bars->abort_flag) {
        const uint32_t n = it < uint32_t(p.stages) ? it : uint32_t(p.stages);
        for (uint32_t j = 0; j < n; ++j) {
          const uint32_t i2 = it - 1 - j;
          if (!mbar_wait(smem_u32(&bars->full[i2 % p.stages]), (i2 / p.stages) & 1u)) atomicExch(p.error, ERR_WAIT_DRAIN);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // The issuing thread is alone in its warp, so every instruction it executes is on the tensor
      // pipe's critical path: descriptors are built once and advanced with one 32-bit add per MMA
      // (the start-address field is the low 14 bits, in 16-byte units), and the ring position is
      // carried in counters instead of being derived with divisions.
      const uint64_t adesc0 = umma_smem_desc(base, p.a.lbo, p.a.sbo);
      const uint64_t bdesc0 = umma_smem_desc(base + p.a.bytes, p.b.lbo, p.b.sbo);
      const uint32_t a_hi = uint32_t(adesc0 >> 32), b_hi = uint32_t(bdesc0 >> 32);
      const uint32_t a_lo0 = uint32_t(adesc0), b_lo0 = uint32_t(bdesc0);
      const uint32_t stage_step = stage_bytes >> 4, a_k = p.a.kstep >> 4, b_k = p.b.kstep >> 4;
      const uint32_t a_sub = p.a.sub_step >> 4, b_sub = p.b.sub_step >> 4;   // next K block inside a stage
      const int kpb = max(p.kpb, 1);
      const uint32_t idesc = p.idesc;
      const int stages = p.stages;
      auto desc = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | uint64_t(lo); };
      uint32_t tcount = 0;
      int s = 0;
      uint32_t ph = 0;
      int err = 0;
      if (p.wait_counter != nullptr && !peer_rows_landed(p)) err = ERR_WAIT_PEER;
      for (int u = blockIdx.x; u < units && !err; u += gridDim.x, ++tcount) {
        const int tile = u / p.splits, split = u - tile * p.splits;
        const int kb0 = split * kb_per_split, kb1 = min(p.k_blocks, kb0 + kb_per_split);
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_ph ^ 1u)) { err = ERR_WAIT_TMEM_EMPTY; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * uint32_t(p.BN);
        uint32_t accum = 0;   // the first MMA of a tile overwrites the accumulator (zero-init at the first K block)
        for (int kb = kb0; kb < kb1; kb += kpb) {
          if (!mbar_wait(smem_u32(&bars->full[s]), ph)) { err = ERR_WAIT_FULL; break; }
          tc_fence_after();
          uint32_t al = a_lo0 + uint32_t(s) * stage_step, bl = b_lo0 + uint32_t(s) * stage_step;
#pragma unroll 1
          for (int sub = 0; sub < kpb; ++sub, al += a_sub, bl += b_sub) {
            if (KIND == 0) {
              umma_f16(d_tmem, desc(al, a_hi), desc(bl, b_hi), idesc, accum);
              umma_f16(d_tmem, desc(al + a_k, a_hi), desc(bl + b_k, b_hi), idesc, 1u);
              umma_f16(d_tmem, desc(al + 2 * a_k, a_hi), desc(bl + 2 * b_k, b_hi), idesc, 1u);
              umma_f16(d_tmem, desc(al + 3 * a_k, a_hi), desc(bl + 3 * b_k, b_hi), idesc, 1u);
            } else {
              umma_i8(d_tmem, desc(al, a_hi), desc(bl, b_hi), idesc, accum);
              umma_i8(d_tmem, desc(al + a_k, a_hi), desc(bl + b_k, b_hi), idesc, 1u);
              umma_i8(d_tmem, desc(al + 2 * a_k, a_hi), desc(bl + 2 * b_k, b_hi), idesc, 1u);
              umma_i8(d_tmem, desc(al + 3 * a_k, a_hi), desc(bl + 3 * b_k, b_hi), idesc, 1u);
            }
            accum = 1u;
          }
          accum = 1u;
          umma_commit(smem_u32(&bars->empty[s]));   // stage reusable once these MMAs retire
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (err) break;
        umma_commit(smem_u32(&bars->tmem_full[acc])); // accumulator complete
      }
      if (err) { atomicExch(p.error, err); bars->abort_flag = 1; }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint8_t *stg = staging + (warp - 2) * kStageStaging;
    uint32_t tcount = 0;
    uint32_t slab = 0;   // TMA-store form: staging slab to fill next
    bool dead = false;
    if (p.wait_counter != nullptr) {
      bool ok = true;
      if (lane == 0) ok = peer_rows_landed(p);
      ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) atomicExch(p.error, ERR_WAIT_PEER);
        dead = true;
      }
    }
    for (int u = blockIdx.x; u < units && !dead; u += gridDim.x, ++tcount) {
      const int tile = u / p.splits, split = u - tile * p.splits;
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bars->tmem_full[acc]), acc_ph)) {
        if (lane == 0) atomicExch(p.error, ERR_WAIT_TMEM_FULL);
        dead = true;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * uint32_t(p.BN) + (uint32_t(q * 32) << 16);
      const int nn0 = tn * p.BN;                 // first MMA column of the tile

      if (!SWAPPED && p.tma_store) gemm_epilogue_tile_tma<KIND>(p, t_addr, tm * kBM, nn0, split, q, lane, stg, slab);
      else gemm_epilogue_tile<KIND, SWAPPED>(p, t_addr, tm * kBM, nn0, split, q, lane, stg);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
    }
    // the staging slabs must outlive the copy engine's reads, the stores must land before the grid ends
    if (!SWAPPED && p.tma_store && lane == 0) tma_store_wait<0>();
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace_max(p.trace, 3);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

template <int KIND, bool SWAPPED>
cudaError_t launch_gemm_kernel(const CUtensorMap &tmA, const CUtensorMap &tmB, const GemmParams &p, int grid,
                               size_t smem, cudaStream_t stream) {
  static bool configured[64] = {};
  auto kfn = gemm_kernel<KIND, SWAPPED>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return e;
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kfn, tmA, tmB, p);
}

template cudaError_t launch_gemm_kernel<0, false>(const CUtensorMap &, const CUtensorMap &, const GemmParams &, int,
                                                  size_t, cudaStream_t);
template cudaError_t launch_gemm_kernel<0, true>(const CUtensorMap &, const CUtensorMap &, const GemmParams &, int,
                                                 size_t, cudaStream_t);
template cudaError_t launch_gemm_kernel<1, false>(const CUtensorMap &, const CUtensorMap &, const GemmParams &, int,
                                                  size_t, cudaStream_t);
template cudaError_t launch_gemm_kernel<1, true>(const CUtensorMap &, const CUtensorMap &, const GemmParams &, int,
                                                 size_t, cudaStream_t);

} // namespace gcb
