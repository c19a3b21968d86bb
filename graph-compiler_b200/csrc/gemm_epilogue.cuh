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
    // ---- MMA row = output row.  Work in slabs of 128 output bytes per row, in two phases per slab:
    //  row phase    each thread owns one row: accumulators from TMEM, the first rounding (bf16 outputs),
    //               16-byte chunks into the warp's swizzled staging buffer;
    //  store phase  each thread owns one 16-byte chunk position (lane & 7) of rows (lane >> 3) + 4 i: its
    //               4 or 8 output columns are the same for all eight rows, so bias / scale / compensation
    //               are loaded once per slab, applied here, and the warp stores full 128-byte row segments.
    const bool two_byte = (p.out_kind == OUT_BF16);
    const int slab_cols = two_byte ? 64 : 32;
    const size_t esz = two_byte ? 2 : 4;
    const size_t plane = (p.splits > 1) ? size_t(split) * size_t(p.split_stride) : 0;
    uint8_t *dstp = reinterpret_cast<uint8_t *>(p.out) + plane * esz;
    const size_t ld_b = size_t(p.ld_out) * esz;
    const bool vec_ok = ((ld_b & 15) == 0) && ((reinterpret_cast<uintptr_t>(dstp) & 15) == 0);
    const bool dump = (KIND == 1) && p.acc_dump != nullptr;
    const bool dump_vec = dump && ((size_t(p.ld_dump) & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.acc_dump) & 15) == 0);
    const int chunk = lane & 7, rsub = lane >> 3;
    const int cpc = two_byte ? 8 : 4;   // columns per 16-byte chunk
    const int warp_owner = (p.peer_rows > 0 && (p.peer_rows & 31) == 0) ? (row0 + q * 32) / p.peer_rows : -1;
    const bool late_bf16 = two_byte && p.bias_kind == BIAS_BF16;   // bias (and ReLU) applied in the store phase
    for (int c0 = 0; c0 < p.BN; c0 += slab_cols) {
      const int col0 = nn0 + c0;
      if (col0 >= p.out_cols) break;   // the rest of the tile lies beyond the last output column
      // ------------------------------------------------------------ row phase
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
      if (two_byte) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t y0 = f32_to_bf16_bits(__uint_as_float(v[8 * c + 2 * e]));
            uint32_t y1 = f32_to_bf16_bits(__uint_as_float(v[8 * c + 2 * e + 1]));
            if (p.relu && !late_bf16) {
              const float f0 = bf16_bits_to_f32(y0), f1 = bf16_bits_to_f32(y1);
              y0 = (f0 != f0) ? y0 : (f0 > 0.f ? y0 : 0u);
              y1 = (f1 != f1) ? y1 : (f1 > 0.f ? y1 : 0u);
            }
            w[e] = y0 | (y1 << 16);
          }
          *reinterpret_cast<uint4 *>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4 *>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) =
              make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      }
      __syncwarp();
      // ------------------------------------------------------------ store phase
      const int gcol = col0 + chunk * cpc;
      // <= 0: this chunk is beyond the last column of the output or of the tile (a tile whose width is not a
      // whole number of slabs ends inside its last slab; the columns behind it belong to the next tile)
      const int nvalid = min(cpc, min(p.out_cols, nn0 + p.BN) - gcol);
      uint32_t bias_b[8];
      float bias_f[4], scale_f[4];
      int32_t comp_i[4];
      if (late_bf16) {
#pragma unroll
        for (int e = 0; e < 8; ++e) bias_b[e] = (e < nvalid) ? reinterpret_cast<const uint16_t *>(p.bias)[gcol + e] : 0u;
      }
      if (!two_byte) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const bool in = e < nvalid;
          bias_f[e] = (in && p.bias_kind == BIAS_F32) ? reinterpret_cast<const float *>(p.bias)[gcol + e] : 0.f;
          scale_f[e] = (in && p.out_kind == OUT_DEQUANT_F32) ? p.scale[gcol + e] : 1.f;
          comp_i[e] = (in && p.out_kind == OUT_DEQUANT_F32 && p.comp) ? p.comp[gcol + e] : 0;
        }
      }
#pragma unroll
      for (int itr = 0; itr < 8; ++itr) {
        const int r = itr * 4 + rsub;
        const uint4 raw = *reinterpret_cast<const uint4 *>(stg + r * 128 + ((chunk ^ (r & 7)) << 4));
        const int grow = row0 + q * 32 + r;
        if (grow >= p.out_rows || nvalid <= 0) continue;
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        if (late_bf16) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t y[2] = {w[e] & 0xFFFFu, w[e] >> 16};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t t = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(y[h]), bf16_bits_to_f32(bias_b[2 * e + h])));
              if (p.relu) {
                const float f = bf16_bits_to_f32(t);
                t = (f != f) ? t : (f > 0.f ? t : 0u);
              }
              y[h] = t;
            }
            w[e] = y[0] | (y[1] << 16);
          }
        } else if (p.out_kind == OUT_DEQUANT_F32) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float f = __fmul_rn(float(int32_t(w[e]) - comp_i[e]), scale_f[e]);
            if (p.bias_kind == BIAS_F32) f = __fadd_rn(f, bias_f[e]);
            if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
            w[e] = __float_as_uint(f);
          }
        } else if (p.out_kind == OUT_F32) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float f = __uint_as_float(w[e]);
            if (p.bias_kind == BIAS_F32) f = __fadd_rn(f, bias_f[e]);
            if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
            w[e] = __float_as_uint(f);
          }
        }
        const uint4 val = make_uint4(w[0], w[1], w[2], w[3]);
        uint8_t *g = dstp + size_t(grow) * ld_b + size_t(gcol) * esz;
        if (p.n_peers > 0) {
          // Row-parallel layer across GPUs: this rank's partial sums go straight from the epilogue
          // into plane `peer_plane` of every rank's receive buffer (plain stores to peer memory over
          // NVLink), so the exchange overlaps the tiles still being computed.  Requires full
          // 16-byte chunks (checked by the launcher).
          if (p.peer_rows > 0) {
            // reduce-scatter by rows: only the rank that will reduce this row receives it (a warp's 32 rows share
            // one owner whenever the rows per peer are a multiple of 32: one division per warp and tile then)
            int owner = warp_owner, lrow = grow - warp_owner * p.peer_rows;
            if (warp_owner < 0) { owner = grow / p.peer_rows; lrow = grow - owner * p.peer_rows; }
            // one plane per (rank, K split): the owner sums them in plane order
            const size_t pl = size_t(p.peer_plane) * size_t(p.splits) + size_t(split);
            const size_t off = (pl * size_t(p.peer_rows) + size_t(lrow)) * ld_b + size_t(gcol) * esz;
            *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.peer_out[owner]) + off) = val;
          } else {
            const size_t off = (size_t(p.peer_plane) * size_t(p.out_rows) + size_t(grow)) * ld_b + size_t(gcol) * esz;
            if (p.peer_multicast) multimem_st_16(reinterpret_cast<uint8_t *>(p.peer_out[0]) + off, val);
            else
              for (int d = 0; d < p.n_peers; ++d) *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.peer_out[d]) + off) = val;
          }
        } else if (vec_ok && nvalid == cpc) {
          *reinterpret_cast<uint4 *>(g) = val;
        } else {
          for (int e = 0; e < nvalid; ++e) {
            if (two_byte) reinterpret_cast<uint16_t *>(g)[e] = uint16_t(w[e >> 1] >> ((e & 1) * 16));
            else          reinterpret_cast<uint32_t *>(g)[e] = w[e];
          }
        }
        if (dump) {   // raw s32 accumulators beside the dequantised result
          int32_t *dg = p.acc_dump + size_t(grow) * size_t(p.ld_dump) + size_t(gcol);
          if (dump_vec && nvalid == 4) *reinterpret_cast<uint4 *>(dg) = raw;
          else {
            const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
            for (int e = 0; e < nvalid; ++e) dg[e] = int32_t(rw[e]);
          }
        }
      }
      __syncwarp();
    }
    if (p.n_peers > 0 && p.peer_rows > 0 && p.signal_peer[0] != nullptr) {
      // this warp's 32 rows of the tile are on their way to their owner: make them visible system-wide, then count
      // the warp in at the owner (the owner's reduction waits for every warp of every tile of every rank)
      __syncwarp();
      const int grow = row0 + q * 32;
      if (lane == 0 && grow < p.out_rows) publish_and_count(p.signal_peer[grow / p.peer_rows]);
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
          if (p.n_peers > 0) {   // column-sharded across GPUs: the finished element goes to every rank's result
            for (int d = 0; d < p.n_peers; ++d) reinterpret_cast<uint16_t *>(p.peer_out[d])[idx] = uint16_t(y);
          } else {
            reinterpret_cast<uint16_t *>(p.out)[idx] = uint16_t(y);
          }
        } else if (p.out_kind == OUT_DEQUANT_F32) {
          float f = __fmul_rn(float(int32_t(v[j]) - comp_i), scale_f);
          if (p.bias_kind == BIAS_F32) f = __fadd_rn(f, bias_f);
          if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
          if (p.n_peers > 0) {
            for (int d = 0; d < p.n_peers; ++d) reinterpret_cast<float *>(p.peer_out[d])[idx] = f;
          } else {
            reinterpret_cast<float *>(p.out)[idx] = f;
          }
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

// The columns of a tile behind its last whole slab (tiles whose width is a multiple of 16 but not of the
// slab width), 16 at a time: each thread owns one accumulator row, applies the same post-ops as the slab
// form and stores its 16 columns itself (two or four 16-byte stores to consecutive addresses).
// c0: first such column inside the tile; col0 = nn0 + c0; grow: this thread's output row.
template <int KIND>
__device__ __forceinline__ void gemm_epilogue_tail(const GemmParams &p, uint32_t t_addr, int c0, int col0, int grow, int split,
                                                   int lane) {
  const bool two_byte = (p.out_kind == OUT_BF16);
  const size_t esz = two_byte ? 2 : 4;
  const size_t plane = (p.splits > 1) ? size_t(split) * size_t(p.split_stride) : 0;
  uint8_t *rowp = reinterpret_cast<uint8_t *>(p.out) + (plane + size_t(grow) * size_t(p.ld_out)) * esz;
  const bool row_in = grow < p.out_rows;
  for (int g0 = c0; g0 < p.BN; g0 += 16) {
    const int gc = col0 + (g0 - c0);            // first output column of this group
    if (gc >= p.out_cols) break;
    uint32_t t[16];
    tmem_ld_x16(t_addr + g0, t);
    // post-op operands of column gc + lane (lanes 0..15), handed round by shuffles
    uint32_t b16 = 0;
    float q_scale = 1.f, q_bias = 0.f;
    int32_t q_comp = 0;
    {
      const int c = gc + lane;
      if (lane < 16 && c < p.out_cols) {
        if (two_byte && p.bias_kind == BIAS_BF16) b16 = reinterpret_cast<const uint16_t *>(p.bias)[c];
        if (p.out_kind == OUT_DEQUANT_F32) {
          q_scale = p.scale[c];
          if (p.bias_kind == BIAS_F32) q_bias = reinterpret_cast<const float *>(p.bias)[c];
          if (p.comp) q_comp = p.comp[c];
        }
      }
    }
    tmem_wait_ld();
    uint32_t w[16];
    if (two_byte) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        uint32_t y = pack_bf16x2_rn(__uint_as_float(t[2 * e]), __uint_as_float(t[2 * e + 1]));   // first rounding
        if (p.bias_kind == BIAS_BF16) {
          const uint32_t b0 = __shfl_sync(0xFFFFFFFFu, b16, 2 * e), b1 = __shfl_sync(0xFFFFFFFFu, b16, 2 * e + 1);
          const float f0 = __fadd_rn(__uint_as_float(y << 16), __uint_as_float(b0 << 16));
          const float f1 = __fadd_rn(__uint_as_float(y & 0xFFFF0000u), __uint_as_float(b1 << 16));
          y = pack_bf16x2_rn(f0, f1);                                                               // second rounding
        }
        if (p.relu) y = bf16x2_relu(y);
        w[e] = bf16x2_fix_nan(y);
      }
    } else if (p.out_kind == OUT_DEQUANT_F32) {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const float sc = __shfl_sync(0xFFFFFFFFu, q_scale, e), bi = __shfl_sync(0xFFFFFFFFu, q_bias, e);
        const int32_t cp = __shfl_sync(0xFFFFFFFFu, q_comp, e);
        float f = __fmul_rn(float(int32_t(t[e]) - cp), sc);
        if (p.bias_kind == BIAS_F32) f = __fadd_rn(f, bi);
        if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
        w[e] = __float_as_uint(f);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e) w[e] = t[e];
    }
    if (!row_in) continue;
    uint8_t *g = rowp + size_t(gc) * esz;
    if (gc + 16 <= p.out_cols) {
      const int nvec = two_byte ? 2 : 4;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < nvec) reinterpret_cast<uint4 *>(g)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    } else {
      const int nv = p.out_cols - gc;
      for (int e = 0; e < nv; ++e) {
        if (two_byte) reinterpret_cast<uint16_t *>(g)[e] = uint16_t(w[e >> 1] >> ((e & 1) * 16));
        else          reinterpret_cast<uint32_t *>(g)[e] = w[e];
      }
    }
  }
}

// TMA-store form of the row-major epilogue (bf16 with optional bias / ReLU, int8 dequantisation to f32, or
// raw f32 / s32 planes).
// Each thread owns one accumulator row: TMEM -> registers -> rounding and post-ops on packed pairs ->
// 16-byte chunks into a swizzled 32 x 128-byte staging slab -> one cp.async.bulk.tensor store per slab
// issued by lane 0.  Two staging slabs per warp alternate, so the copy engine drains one while the
// warp fills the other; rows and columns beyond the output are clipped by the copy engine.
// stg: this warp's two 4 KiB slabs (1 KiB aligned); buf: slab to fill next (kept by the caller across tiles).
template <int KIND>
__device__ __forceinline__ void gemm_epilogue_tile_tma(const GemmParams &p, uint32_t t_addr, int row0, int nn0, int split,
                                                       int q, int lane, uint8_t *stg, uint32_t &buf) {
  const bool two_byte = (p.out_kind == OUT_BF16);
  const int slab_cols = two_byte ? 64 : 32;
  const int grow0 = row0 + q * 32;
  const bool rows_in = grow0 < p.out_rows;
  // row scatter: this warp's 32 rows belong to one owner, whose buffer has its own tensor map
  // (tma_peer 1: row scatter to the owner; 2: the finished slab goes to EVERY rank's result - all-gather of C)
  const int owner = p.tma_peer == 1 ? grow0 / p.peer_rows : 0;
  const CUtensorMap *tmap = p.tma_peer == 1 ? &p.tmPeer[owner] : &p.tmC;
  const int store_row = p.tma_peer == 1 ? grow0 - owner * p.peer_rows : grow0;
  const int store_plane = p.tma_peer == 1 ? p.peer_plane * p.splits + split : split;
  for (int c0 = 0; c0 < p.BN; c0 += slab_cols) {
    const int col0 = nn0 + c0;
    if (col0 >= p.out_cols) break;
    if (p.tma_peer != 1 && p.BN - c0 < slab_cols) {
      // the tile is not a whole number of slabs wide (BN a multiple of 16 only): the last 16, 32 or 48 columns
      // go from registers straight to global memory, 16 columns (32 or 64 contiguous bytes per row) at a time
      gemm_epilogue_tail<KIND>(p, t_addr, c0, col0, grow0 + lane, split, lane);
      break;
    }
    uint32_t v[64];
    {
      uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&v[0]);
      tmem_ld_x32(t_addr + c0, lo);
      if (two_byte) {
        uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&v[32]);
        tmem_ld_x32(t_addr + c0 + 32, hi);
      }
    }
    // the slab filled two stores ago must have been read by the copy engine before it is overwritten
    if (lane == 0) tma_store_wait_read<1>();
    uint32_t bias2 = 0;   // bias of columns col0 + 2 lane, + 1 (bf16 pair), handed round by shuffles
    if (two_byte && p.bias_kind == BIAS_BF16) {
      const int c = col0 + 2 * lane;
      const uint16_t *b = reinterpret_cast<const uint16_t *>(p.bias);
      const uint32_t b0 = c < p.out_cols ? b[c] : 0u, b1 = c + 1 < p.out_cols ? b[c + 1] : 0u;
      bias2 = b0 | (b1 << 16);
    }
    // int8 dequantisation: this lane holds scale / bias / compensation of column col0 + lane
    float q_scale = 1.f, q_bias = 0.f;
    int32_t q_comp = 0;
    if (p.out_kind == OUT_DEQUANT_F32) {
      const int c = col0 + lane;
      if (c < p.out_cols) {
        q_scale = p.scale[c];
        if (p.bias_kind == BIAS_F32) q_bias = reinterpret_cast<const float *>(p.bias)[c];
        if (p.comp) q_comp = p.comp[c];
      }
    }
    tmem_wait_ld();
    __syncwarp();
    uint8_t *slab = stg + buf * 4096u;
    if (p.out_kind == OUT_DEQUANT_F32) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = 4 * c + e;
          const float sc = __shfl_sync(0xFFFFFFFFu, q_scale, j), bi = __shfl_sync(0xFFFFFFFFu, q_bias, j);
          const int32_t cp = __shfl_sync(0xFFFFFFFFu, q_comp, j);
          float f = __fmul_rn(float(int32_t(v[j]) - cp), sc);
          if (p.bias_kind == BIAS_F32) f = __fadd_rn(f, bi);
          if (p.relu) f = (f != f) ? f : (f > 0.f ? f : 0.f);
          w[e] = __float_as_uint(f);
        }
        *reinterpret_cast<uint4 *>(slab + lane * 128 + ((c ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else if (two_byte) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = 4 * c + e;   // pair index: columns 2j, 2j + 1 of the slab
          uint32_t y = pack_bf16x2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));   // first rounding
          if (p.bias_kind == BIAS_BF16) {
            const uint32_t bb = __shfl_sync(0xFFFFFFFFu, bias2, j);
            const float f0 = __fadd_rn(__uint_as_float(y << 16), __uint_as_float(bb << 16));
            const float f1 = __fadd_rn(__uint_as_float(y & 0xFFFF0000u), __uint_as_float(bb & 0xFFFF0000u));
            y = pack_bf16x2_rn(f0, f1);                                                             // second rounding
          }
          if (p.relu) y = bf16x2_relu(y);
          w[e] = bf16x2_fix_nan(y);
        }
        *reinterpret_cast<uint4 *>(slab + lane * 128 + ((c ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4 *>(slab + lane * 128 + ((c ^ (lane & 7)) << 4)) =
            make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    }
    fence_proxy_async();   // generic-proxy writes of the slab -> visible to the copy engine
    __syncwarp();
    if (lane == 0 && rows_in) {
      if (p.tma_peer == 2) {
        for (int d = 0; d < p.n_peers; ++d) tma_store_3d(&p.tmPeer[d], smem_u32(slab), col0, grow0, 0);
      } else {
        tma_store_3d(tmap, smem_u32(slab), col0, store_row, store_plane);
      }
      tma_store_commit();
    }
    buf ^= 1u;
  }
  if (p.tma_peer == 1 && p.signal_peer[0] != nullptr) {
    // the warp's rows of this tile are on their way to their owner: once the copy engine has completed the stores
    // (not merely read the slabs), publish them and count the warp in at the owner
    __syncwarp();
    if (lane == 0 && rows_in) {
      tma_store_wait<0>();
      publish_and_count(p.signal_peer[owner]);
    }
  }
}

} // namespace gcb
