// Epilogue of one accumulator tile, shared by the one-CTA and the CTA-pair GEMM kernels:
// tcgen05.ld -> post-ops -> (row-major form) swizzled shared-memory staging -> 128-byte coalesced
// global stores.  Called by the four epilogue warps of a CTA, each on its own TMEM lane quadrant.
#pragma once
#include "gemm_sm100.cuh"
#include "sm100_ptx.cuh"

namespace gcb {

// t_addr : TMEM address of the accumulator (lane quadrant already applied)
// row0   : first output row (non-swapped) / first output column (swapped) of this CTA's 128 MMA rows
// nn0    : first MMA column of the tile;  q: lane quadrant;  stg: this warp's 4 KiB staging buffer
template <int KIND, bool SWAPPED>
__device__ __forceinline__ void gemm_epilogue_tile(const GemmParams &p, uint32_t t_addr, int row0, int nn0, int split,
                                                   int q, int lane, uint8_t *stg) {
  const int mm = row0 + q * 32 + lane;   // MMA row of this thread
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
        const int grow = row0 + q * 32 + r;
        const int gcol = col0 + c * cols_per_chunk;
        if (grow < p.out_rows && gcol < p.out_cols) {
          uint8_t *g = dstp + size_t(grow) * ld_b + size_t(gcol) * es;
          if (pass == 0 && p.n_peers > 0) {
            // Row-parallel layer across GPUs: this rank's partial sums go straight from the epilogue
            // into plane `peer_plane` of every rank's receive buffer (plain stores to peer memory over
            // NVLink), so the exchange overlaps the tiles still being computed.  Requires full
            // 16-byte chunks (checked by the launcher).
            const size_t off = (size_t(p.peer_plane) * size_t(p.out_rows) + size_t(grow)) * ld_b + size_t(gcol) * es;
            for (int d = 0; d < p.n_peers; ++d) *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.peer_out[d]) + off) = val;
          } else if (vec_ok && gcol + cols_per_chunk <= p.out_cols) {
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
}

} // namespace gcb
