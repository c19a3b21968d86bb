// CTA-pair form of the persistent GEMM (tcgen05.mma.cta_group::2): two CTAs on neighbouring SMs
// compute one 256 x BN output tile.  Each CTA stages its own 128 rows of A and its own half of the
// B tile's columns, the even CTA issues MMAs that read both CTAs' shared memory and write both
// CTAs' tensor memory.  Per SM and K block this halves the B bytes pulled from L2 relative to the
// one-CTA kernel (gemm_sm100.cu), which is what bounds that kernel.
//
// Same roles and numerics as the one-CTA kernel (it replaces the same reference code:
// DeepTileContractionOp.cpp:545-949 + BrgemmOnednn.cpp:145-168 + fused post-ops):
//   warps 0, 6  TMA producers of A and B (both CTAs; byte counts are credited to the even CTA's barrier)
//   warp 1      MMA issuer (even CTA only); allocates / frees TMEM in both CTAs
//   warps 2..5  epilogue of this CTA's 128 rows (both CTAs)
// Barrier traffic across the pair: the MMA completion arrives on the stage-empty and
// accumulator-full barriers of BOTH CTAs (tcgen05.commit with a CTA mask); the epilogue warps of
// both CTAs arrive on the even CTA's accumulator-empty barrier (remote mbarrier arrive).
#include "gemm_epilogue.cuh"
#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace gcb {

constexpr int kThreads2 = 224;
constexpr int kStaging2 = 8192;   // per epilogue warp: two slabs of 32 rows x 128 B
constexpr int kMaxStages2 = 8;

struct PairBarriers {
  uint64_t full[kMaxStages2];
  uint64_t empty[kMaxStages2];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t pad;
};

size_t gemm_pair_smem_bytes(const GemmParams &p) {
  return 1024 + size_t(p.stages) * (p.a.bytes + p.b.bytes) + 4 * kStaging2 + sizeof(PairBarriers);
}

__device__ __forceinline__ void pair_tile_coords(const GemmParams &p, int tile, int &tm, int &tn) {
  const int per_group = p.group_m * p.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.tiles_m - first_m, p.group_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

// Bounded wait until this step's rows of the activations (stored by other GPUs' kernels) have landed here.
__device__ __forceinline__ bool pair_rows_landed(const GemmParams &p) {
  const uint32_t target = (*reinterpret_cast<const volatile uint32_t *>(p.epoch) + 1u) * p.wait_per_step;
  return wait_counter_reached(p.wait_counter, target, 4 * WAIT_LIMIT_CYCLES);
}

// p.tiles_m counts 256-row tiles; p.b describes this CTA's half (BN/2 columns) of the B tile.
template <int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);
  const uint32_t stage_bytes = p.a.bytes + p.b.bytes;
  uint8_t *staging = smem + size_t(p.stages) * stage_bytes;
  PairBarriers *bars = reinterpret_cast<PairBarriers *>(staging + 4 * kStaging2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int units = p.tiles_m * p.tiles_n * p.splits;
  const int kb_per_split = (p.k_blocks + p.splits - 1) / p.splits;
  const int half_n = p.BN / 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 2);    // the even CTA's two expect-tx arrives (A and B producers)
      mbar_init(smem_u32(&bars->empty[s]), 1);   // one MMA commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars->tmem_full[b]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[b]), 8);  // four epilogue warps of each CTA
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&bars->tmem_base), p.tmem_cols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before any cross-CTA signal
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(&bars->tmem_base);
  // the set-up above touched only shared and tensor memory and may overlap the tail of the kernel ahead
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_store(p.trace, 0);
  pdl_launch_dependents();
  pdl_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) trace_store(p.trace, 1);

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------------ TMA producers (both CTAs)
    // warp 0 streams this CTA's A rows, warp 6 this CTA's half of the B tile; per stage each does
    // one wait, (even CTA) one expect-tx covering both CTAs' bytes of its operand, one tensor copy.
    if (lane == 0) {
      const bool is_a = (warp == 0);
      const CUtensorMap *tm = is_a ? &tmA : &tmB;
      const OperandGeom &g = is_a ? p.a : p.b;
      tma_prefetch_desc(tm);
      int s = 0;
      uint32_t ph = 0;
      const int stages = p.stages;
      const uint32_t my_bytes = g.bytes, my_off = is_a ? 0u : p.a.bytes;
      const uint32_t boxes = g.boxes, box_bytes = g.box_bytes, box_mn = g.box_mn;
      const bool mn = g.mn_major != 0, one = g.one_load != 0;
      const int bk = p.bk_elems;
      int err = 0;
      // see gemm_sm100.cu: the activation producer waits for this step's rows before its first load, the weight
      // producer after it has filled the ring
      const bool gated = p.wait_counter != nullptr;
      bool gate_open = !gated;
      uint32_t issued = 0;
      auto peer_gate = [&]() {
        if (!pair_rows_landed(p)) err = ERR_WAIT_PEER;
        fence_proxy_async_global();
        gate_open = true;
        trace_max(p.trace, 2);
      };
      if (gated && is_a) peer_gate();
      for (int u = pair; u < units && !err; u += pairs) {
        const int tile = u / p.splits, split = u - tile * p.splits;
        int tm_, tn_;
        pair_tile_coords(p, tile, tm_, tn_);
        const int mn_off = is_a ? tm_ * 256 + int(rank) * 128 : tn_ * p.BN + int(rank) * half_n;
        const int kb0 = split * kb_per_split, kb1 = min(p.k_blocks, kb0 + kb_per_split);
        int k_off = kb0 * bk;
        const int grp = mn_off / int(box_mn ? box_mn : 1u);
        for (int kb = kb0; kb < kb1; ++kb, k_off += bk, ++issued) {
          if (!gate_open && issued >= uint32_t(stages)) { peer_gate(); if (err) break; }
          if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u)) { err = ERR_WAIT_EMPTY; break; }
          const uint32_t full = smem_u32(&bars->full[s]);
          if (rank == 0) mbar_expect_tx(full, 2 * my_bytes);   // both CTAs' bytes of this operand land here
          const uint32_t dst = base + uint32_t(s) * stage_bytes + my_off;
          if (!mn) tma_load_2d_pair(dst, tm, full, k_off, mn_off);
          else if (one) tma_load_3d_pair(dst, tm, full, 0, k_off, grp);
          else
            for (uint32_t i = 0; i < boxes; ++i) tma_load_2d_pair(dst + i * box_bytes, tm, full, mn_off + int(i * box_mn), k_off);
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      if (err) atomicExch(p.error, err);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA)
    if (lane == 0 && rank == 0) {
      // The issuing thread is alone in its warp, so every instruction it executes is on the tensor
      // pipe's critical path: descriptors are built once and advanced with one 32-bit add per MMA
      // (the start-address field is the low 14 bits, in 16-byte units), and the ring position is
      // carried in counters instead of being derived with divisions.
      const uint64_t adesc0 = umma_smem_desc(base, p.a.lbo, p.a.sbo);
      const uint64_t bdesc0 = umma_smem_desc(base + p.a.bytes, p.b.lbo, p.b.sbo);
      const uint32_t a_hi = uint32_t(adesc0 >> 32), b_hi = uint32_t(bdesc0 >> 32);
      const uint32_t a_lo0 = uint32_t(adesc0), b_lo0 = uint32_t(bdesc0);
      const uint32_t stage_step = stage_bytes >> 4, a_k = p.a.kstep >> 4, b_k = p.b.kstep >> 4;
      const uint32_t idesc = p.idesc;
      const int stages = p.stages;
      auto desc = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | uint64_t(lo); };
      uint32_t tcount = 0;
      int s = 0;
      uint32_t ph = 0;
      int err = 0;
      if (p.wait_counter != nullptr && !pair_rows_landed(p)) err = ERR_WAIT_PEER;
      for (int u = pair; u < units && !err; u += pairs, ++tcount) {
        const int tile = u / p.splits, split = u - tile * p.splits;
        const int kb0 = split * kb_per_split, kb1 = min(p.k_blocks, kb0 + kb_per_split);
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_ph ^ 1u)) { err = ERR_WAIT_TMEM_EMPTY; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * uint32_t(p.BN);
        uint32_t accum = 0;   // the first MMA of a tile overwrites the accumulator (zero-init at the first K block)
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&bars->full[s]), ph)) { err = ERR_WAIT_FULL; break; }
          tc_fence_after();
          const uint32_t al = a_lo0 + uint32_t(s) * stage_step, bl = b_lo0 + uint32_t(s) * stage_step;
          if (KIND == 0) {
            umma_f16_pair(d_tmem, desc(al, a_hi), desc(bl, b_hi), idesc, accum);
            umma_f16_pair(d_tmem, desc(al + a_k, a_hi), desc(bl + b_k, b_hi), idesc, 1u);
            umma_f16_pair(d_tmem, desc(al + 2 * a_k, a_hi), desc(bl + 2 * b_k, b_hi), idesc, 1u);
            umma_f16_pair(d_tmem, desc(al + 3 * a_k, a_hi), desc(bl + 3 * b_k, b_hi), idesc, 1u);
          } else {
            umma_i8_pair(d_tmem, desc(al, a_hi), desc(bl, b_hi), idesc, accum);
            umma_i8_pair(d_tmem, desc(al + a_k, a_hi), desc(bl + b_k, b_hi), idesc, 1u);
            umma_i8_pair(d_tmem, desc(al + 2 * a_k, a_hi), desc(bl + 2 * b_k, b_hi), idesc, 1u);
            umma_i8_pair(d_tmem, desc(al + 3 * a_k, a_hi), desc(bl + 3 * b_k, b_hi), idesc, 1u);
          }
          accum = 1u;
          umma_commit_pair(smem_u32(&bars->empty[s]));   // stage reusable once these MMAs retire
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (err) break;
        umma_commit_pair(smem_u32(&bars->tmem_full[acc])); // accumulator complete
      }
      if (err) atomicExch(p.error, err);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    uint8_t *stg = staging + (warp - 2) * kStaging2;
    uint32_t tcount = 0;
    uint32_t slab = 0;   // TMA-store form: staging slab to fill next
    bool dead = false;
    if (p.wait_counter != nullptr) {
      bool ok = true;
      if (lane == 0) ok = pair_rows_landed(p);
      ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) atomicExch(p.error, ERR_WAIT_PEER);
        dead = true;
      }
    }
    for (int u = pair; u < units && !dead; u += pairs, ++tcount) {
      const int tile = u / p.splits, split = u - tile * p.splits;
      int tm, tn;
      pair_tile_coords(p, tile, tm, tn);
      const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bars->tmem_full[acc]), acc_ph)) {
        if (lane == 0) atomicExch(p.error, ERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * uint32_t(p.BN) + (uint32_t(q * 32) << 16);
      if (p.tma_store) gemm_epilogue_tile_tma<KIND>(p, t_addr, tm * 256 + int(rank) * 128, tn * p.BN, split, q, lane, stg, slab);
      else gemm_epilogue_tile<KIND, false>(p, t_addr, tm * 256 + int(rank) * 128, tn * p.BN, split, q, lane, stg);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&bars->tmem_empty[acc]), 0));
    }
    // the staging slabs must outlive the copy engine's reads, the stores must land before the grid ends
    if (p.tma_store && lane == 0) tma_store_wait<0>();
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace_max(p.trace, 3);
  cluster_sync_all();   // no CTA leaves while its peer may still signal it or read its shared memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, p.tmem_cols);
  }
}

template <int KIND>
cudaError_t launch_gemm_pair_kernel(const CUtensorMap &tmA, const CUtensorMap &tmB, const GemmParams &p, int grid,
                                    size_t smem, cudaStream_t stream) {
  static bool configured[64] = {};
  auto kfn = gemm_pair_kernel<KIND>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return e;
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(grid & ~1));
  cfg.blockDim = dim3(kThreads2);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kfn, tmA, tmB, p);
}

template cudaError_t launch_gemm_pair_kernel<0>(const CUtensorMap &, const CUtensorMap &, const GemmParams &, int, size_t,
                                                cudaStream_t);
template cudaError_t launch_gemm_pair_kernel<1>(const CUtensorMap &, const CUtensorMap &, const GemmParams &, int, size_t,
                                                cudaStream_t);

} // namespace gcb
