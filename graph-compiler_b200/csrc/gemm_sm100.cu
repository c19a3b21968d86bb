// Persistent, warp-specialised GEMM for sm_100a.
//
// This single kernel replaces the reference's whole deep-tiled loop nest
// (lib/gc/Transforms/DeepTileContractionOp.cpp:545-949: 3 thread loops x 3 L2
// loops x 3 L1 loops) together with the brgemm microkernel it calls per
// innermost tile (lib/gc/ExecutionEngine/CPURuntime/Microkernel/
// BrgemmOnednn.cpp:145-168) and the elementwise post-ops that
// IterativeTilingAndFusion.cpp:743-828 fuses behind the last K block.
//
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A and B into a
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
#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace gcb {

constexpr int kThreads = 192;
constexpr int kBM = 128;             // MMA M (cta_group::1)
constexpr int kStageStaging = 4096;  // per epilogue warp: 32 rows x 128 B
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
      mbar_init(smem_u32(&bars->full[s]), 1);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;            // running stage counter over the whole kernel
      int err = 0;
      for (int u = blockIdx.x; u < units && !err; u += gridDim.x) {
        const int tile = u / p.splits, split = u - tile * p.splits;
        int tm, tn;
        tile_coords(p, tile, tm, tn);
        const int m_off = tm * kBM, n_off = tn * p.BN;
        const int kb0 = split * kb_per_split, kb1 = min(p.k_blocks, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1u;
          if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u)) { err = ERR_WAIT_EMPTY; break; }
          const uint32_t full = smem_u32(&bars->full[s]);
          mbar_expect_tx(full, stage_bytes);
          const uint32_t sa = base + s * stage_bytes, sb = sa + p.a.bytes;
          const int k_off = kb * p.bk_elems;
          for (uint32_t bx = 0; bx < p.a.boxes; ++bx) {
            if (p.a.mn_major) tma_load_2d(sa + bx * p.a.box_bytes, &tmA, full, m_off + int(bx * p.a.box_mn), k_off);
            else              tma_load_2d(sa + bx * p.a.box_bytes, &tmA, full, k_off, m_off);
          }
          for (uint32_t bx = 0; bx < p.b.boxes; ++bx) {
            if (p.b.mn_major) tma_load_2d(sb + bx * p.b.box_bytes, &tmB, full, n_off + int(bx * p.b.box_mn), k_off);
            else              tma_load_2d(sb + bx * p.b.box_bytes, &tmB, full, k_off, n_off);
          }
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
      uint32_t it = 0, tcount = 0;
      int err = 0;
      for (int u = blockIdx.x; u < units && !err; u += gridDim.x, ++tcount) {
        const int tile = u / p.splits, split = u - tile * p.splits;
        const int kb0 = split * kb_per_split, kb1 = min(p.k_blocks, kb0 + kb_per_split);
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_ph ^ 1u)) { err = ERR_WAIT_TMEM_EMPTY; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * uint32_t(p.BN);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1u;
          if (!mbar_wait(smem_u32(&bars->full[s]), ph)) { err = ERR_WAIT_FULL; break; }
          tc_fence_after();
          const uint32_t sa = base + s * stage_bytes, sb = sa + p.a.bytes;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t ad = umma_smem_desc(sa + j * p.a.kstep, p.a.lbo, p.a.sbo);
            const uint64_t bd = umma_smem_desc(sb + j * p.b.kstep, p.b.lbo, p.b.sbo);
            const uint32_t accum = (kb > kb0 || j > 0) ? 1u : 0u;
            if (KIND == 0) umma_f16(d_tmem, ad, bd, p.idesc, accum);
            else           umma_i8(d_tmem, ad, bd, p.idesc, accum);
          }
          umma_commit(smem_u32(&bars->empty[s]));   // stage reusable once these MMAs retire
        }
        if (err) break;
        umma_commit(smem_u32(&bars->tmem_full[acc])); // accumulator complete
      }
      if (err) { atomicExch(p.error, err); bars->abort_flag = 1; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint8_t *stg = staging + (warp - 2) * kStageStaging;
    uint32_t tcount = 0;
    bool dead = false;
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
      const int mm = tm * kBM + q * 32 + lane;   // MMA row of this thread
      const int nn0 = tn * p.BN;                 // first MMA column of the tile

      if (!SWAPPED) {
        // ---- MMA row = output row.  Work in slabs of 128 output bytes per row.
        const int row = mm;
        const bool two_byte = (p.out_kind == OUT_BF16);
        const int slab_cols = two_byte ? 64 : 32;
        uint8_t *outp = reinterpret_cast<uint8_t *>(p.out);
        const size_t esz = two_byte ? 2 : 4;
        const size_t plane = (p.splits > 1) ? size_t(split) * size_t(p.split_stride) : 0;
        for (int c0 = 0; c0 < p.BN; c0 += slab_cols) {
          uint32_t v[64];
          {
            uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&v[0]);
            tmem_ld_x32(t_addr + c0, lo);
            if (two_byte) {
              uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&v[32]);
              tmem_ld_x32(t_addr + c0 + 32, hi);
            }
            tmem_wait_ld();
          }
          uint4 packed[8];
          const int col0 = nn0 + c0;
          if (p.out_kind == OUT_BF16) {
            uint32_t h[64];
#pragma unroll
            for (int j = 0; j < 64; ++j) {
              uint32_t y = f32_to_bf16_bits(__uint_as_float(v[j]));
              const int col = col0 + j;
              if (p.bias_kind == BIAS_BF16 && col < p.out_cols) {
                const uint32_t b = reinterpret_cast<const uint16_t *>(p.bias)[col];
                y = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(y), bf16_bits_to_f32(b)));
              }
              if (p.relu) {
                const float f = bf16_bits_to_f32(y);
                y = (f != f) ? y : (f > 0.f ? y : 0u);
              }
              h[j] = y;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c)
              packed[c] = make_uint4(h[8 * c] | (h[8 * c + 1] << 16), h[8 * c + 2] | (h[8 * c + 3] << 16),
                                     h[8 * c + 4] | (h[8 * c + 5] << 16), h[8 * c + 6] | (h[8 * c + 7] << 16));
          } else {
            uint32_t o[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + j;
              if (p.out_kind == OUT_DEQUANT_F32) {
                float f = 0.f;
                if (col < p.out_cols) {
                  const int32_t a = int32_t(v[j]) - (p.comp ? p.comp[col] : 0);
                  f = __fmul_rn(float(a), p.scale[col]);
                  if (p.bias_kind == BIAS_F32) f = __fadd_rn(f, reinterpret_cast<const float *>(p.bias)[col]);
                  if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
                }
                o[j] = __float_as_uint(f);
              } else if (p.out_kind == OUT_F32) {
                float f = __uint_as_float(v[j]);
                if (p.bias_kind == BIAS_F32 && col < p.out_cols)
                  f = __fadd_rn(f, reinterpret_cast<const float *>(p.bias)[col]);
                if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
                o[j] = __float_as_uint(f);
              } else {
                o[j] = v[j];
              }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) packed[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
          }
          // two passes when the raw accumulators are dumped as well
          const int passes = (p.acc_dump != nullptr && KIND == 1) ? 2 : 1;
          for (int pass = 0; pass < passes; ++pass) {
            if (pass == 1) {
#pragma unroll
              for (int c = 0; c < 8; ++c) packed[c] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
            }
            uint8_t *dstp = pass == 0 ? outp + plane * esz : reinterpret_cast<uint8_t *>(p.acc_dump);
            const size_t ld_b = pass == 0 ? size_t(p.ld_out) * esz : size_t(p.ld_dump) * 4;
            const size_t es = pass == 0 ? esz : 4;
            const int cols_per_chunk = int(16 / es);
            // stage: row = lane, 16-byte chunk c at position c ^ (lane & 7)
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4 *>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) = packed[c];
            __syncwarp();
            const bool vec_ok = ((ld_b & 15) == 0) && ((reinterpret_cast<uintptr_t>(dstp) & 15) == 0);
#pragma unroll
            for (int itr = 0; itr < 8; ++itr) {
              const int r = itr * 4 + (lane >> 3), c = lane & 7;
              const uint4 val = *reinterpret_cast<const uint4 *>(stg + r * 128 + ((c ^ (r & 7)) << 4));
              const int grow = tm * kBM + q * 32 + r;
              const int gcol = col0 + c * cols_per_chunk;
              if (grow < p.out_rows && gcol < p.out_cols) {
                uint8_t *g = dstp + size_t(grow) * ld_b + size_t(gcol) * es;
                if (vec_ok && gcol + cols_per_chunk <= p.out_cols) {
                  *reinterpret_cast<uint4 *>(g) = val;
                } else {
                  const uint32_t w[4] = {val.x, val.y, val.z, val.w};
                  const int nvalid = min(cols_per_chunk, p.out_cols - gcol);
                  for (int e = 0; e < nvalid; ++e) {
                    if (es == 2) reinterpret_cast<uint16_t *>(g)[e] = uint16_t(w[e >> 1] >> ((e & 1) * 16));
                    else         reinterpret_cast<uint32_t *>(g)[e] = w[e];
                  }
                }
              }
            }
            __syncwarp();
          }
          (void)row;
        }
      } else {
        // ---- swapped orientation: MMA row = output column (this thread),
        //      MMA column = output row.  A warp stores 32 consecutive output
        //      columns of one output row per instruction.
        const int ocol = mm;
        uint32_t bias_bits = 0;
        float bias_f = 0.f, scale_f = 1.f;
        int32_t comp_i = 0;
        if (ocol < p.out_cols) {
          if (p.bias_kind == BIAS_BF16) bias_bits = reinterpret_cast<const uint16_t *>(p.bias)[ocol];
          if (p.bias_kind == BIAS_F32) bias_f = reinterpret_cast<const float *>(p.bias)[ocol];
          if (p.out_kind == OUT_DEQUANT_F32) { scale_f = p.scale[ocol]; comp_i = p.comp ? p.comp[ocol] : 0; }
        }
        const size_t plane = (p.splits > 1) ? size_t(split) * size_t(p.split_stride) : 0;
        for (int c0 = 0; c0 < p.BN; c0 += 16) {
          uint32_t v[16];
          tmem_ld_x16(t_addr + c0, v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int orow = nn0 + c0 + j;
            if (orow < p.out_rows && ocol < p.out_cols) {
              const size_t idx = plane + size_t(orow) * size_t(p.ld_out) + size_t(ocol);
              if (p.out_kind == OUT_BF16) {
                uint32_t y = f32_to_bf16_bits(__uint_as_float(v[j]));
                if (p.bias_kind == BIAS_BF16)
                  y = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(y), bf16_bits_to_f32(bias_bits)));
                if (p.relu) { const float f = bf16_bits_to_f32(y); y = (f != f) ? y : (f > 0.f ? y : 0u); }
                reinterpret_cast<uint16_t *>(p.out)[idx] = uint16_t(y);
              } else if (p.out_kind == OUT_DEQUANT_F32) {
                float f = __fmul_rn(float(int32_t(v[j]) - comp_i), scale_f);
                if (p.bias_kind == BIAS_F32) f = __fadd_rn(f, bias_f);
                if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
                reinterpret_cast<float *>(p.out)[idx] = f;
                if (p.acc_dump) p.acc_dump[size_t(orow) * size_t(p.ld_dump) + size_t(ocol)] = int32_t(v[j]);
              } else if (p.out_kind == OUT_F32) {
                float f = __uint_as_float(v[j]);
                if (p.bias_kind == BIAS_F32) f = __fadd_rn(f, bias_f);
                if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
                reinterpret_cast<float *>(p.out)[idx] = f;
              } else {
                reinterpret_cast<uint32_t *>(p.out)[idx] = v[j];
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
    }
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  tc_fence_before();
  __syncthreads();
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
  kfn<<<grid, kThreads, smem, stream>>>(tmA, tmB, p);
  return cudaGetLastError();
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
