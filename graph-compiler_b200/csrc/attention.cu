// Fused attention forward for sm_100a: O = softmax(Q K^T * scale [+ causal]) V.
//
// The reference has no fused attention pattern; what it has is the softmax
// decomposition (max, sub, exp, sum, div — lib/gc/Transforms/DecomposeAggregatedOps.cpp:24-38)
// and batch matmuls with f32 accumulation.  This kernel computes exactly that
// function blockwise (online softmax in f32) without ever writing the S x S
// score matrix to memory.
//
// One CTA owns two 128-row query tiles of one (batch, head) unit and walks the
// key/value tiles once for both ("two streams"), so that the tensor pipe works
// on one stream while the other stream's warps are in softmax.
//
//   warp 0       TMA producer: Q (once), then K_0, K_1, V_0, K_2, V_1, ... (the order the MMA warp
//                consumes them) into a ring of three 32 KiB slots
//   warp 1       MMA issuer: S_t = Q_t K_j^T and O_t += P_t V_j (tcgen05.mma, S and O in TMEM)
//   warps 2..5   softmax of stream 0 (one query row per thread)
//   warps 6..9   the same for stream 1
//
// Per key tile and stream the softmax warps copy the 128 scores of their row from TMEM to registers
// (which frees S for the next Q K^T at once), take the row maximum, write P = 2^(s*c - m) as bf16 into
// shared memory in the K-major 128-byte-swizzled layout the MMA reads, and the MMA warp accumulates
// P V into O, which stays in TMEM for the whole walk.  The reference maximum m is updated lazily:
// only when the running maximum has grown by more than 8 (a factor 256, harmless in f32 and bf16)
// is O rescaled in TMEM, so after the first few tiles no thread touches O until the epilogue
// divides it by the row sum l, which is accumulated with the same m and therefore exact.
//
// Shared memory: Q 2 x 32 KiB, K/V ring 3 x 32 KiB, P 2 x 32 KiB = 224 KiB.  TMEM: S0 S1 O0 O1,
// 128 columns each = 512 columns.
#include "attention.h"

#include <cmath>
#include <stdexcept>

#include "runtime.h"
#include "sm100_ptx.cuh"

namespace gcb {

namespace {

constexpr int kAttThreads = 320;
constexpr int kTile = 128;          // query rows per stream, key rows per tile
constexpr int kSlot = 32768;        // one 128 x 128 bf16 tile
constexpr int kRing = 3;
constexpr float kLazy = 8.0f;       // rescale O only when the row maximum grew by more than 2^kLazy

struct AttParams {
  int seq, bh, dim;
  int causal;
  float scale_log2e;   // scale * log2(e)
  void *O;
  int *error;
  int q_pairs;         // ceil(seq / 256)
};

struct AttBars {
  uint64_t q_full;
  uint64_t kv_full[kRing];
  uint64_t kv_empty[kRing];
  uint64_t s_full[2];    // MMA -> softmax: S_t holds the scores of the next tile
  uint64_t s_free[2];    // softmax -> MMA: S_t has been copied to registers
  uint64_t p_ready[2];   // softmax -> MMA: P_t written, O_t rescaled if needed
  uint64_t pv_full[2];   // MMA -> softmax: O_t += P_t V_j has retired
  uint32_t tmem_base;
  uint32_t pad;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// two f32 lanes per instruction (sm_100 packed f32x2 arithmetic)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Operand tiles in shared memory.  Q, K and P are K-major 128 x 128 bf16 tiles stored as two 128-row x
// 128-byte swizzled blocks (contraction index 0..63 in block 0, 64..127 in block 1): K step j starts at
// block (j >> 2), 32 bytes per step inside it.  V [128 keys x 128 d] is an MN-major B operand: two
// 64-wide d blocks 16 KiB apart (leading offset), 8-row groups 1 KiB apart (stride offset), 2 KiB
// per 16-key K step.

__global__ void __launch_bounds__(kAttThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ AttParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);
  // layout: Q0 Q1 | ring[3] | P0 P1 | barriers
  const uint32_t q_s = base, ring_s = base + 2 * kSlot, p_s = ring_s + kRing * kSlot;
  AttBars *bars = reinterpret_cast<AttBars *>(smem + (2 + kRing + 2) * kSlot);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavier (later) query pairs first when causal
  const int pair = p.causal ? (p.q_pairs - 1 - int(blockIdx.x)) : int(blockIdx.x);
  const int bh = blockIdx.y;
  const int q_base0 = pair * 256, q_base1 = q_base0 + 128;
  const bool act1 = q_base1 < p.seq;
  const int kv_tiles_all = (p.seq + kTile - 1) / kTile;
  // number of key tiles each stream visits
  const int n0 = p.causal ? min(kv_tiles_all, q_base0 / kTile + 1) : kv_tiles_all;
  const int n1 = act1 ? (p.causal ? min(kv_tiles_all, q_base1 / kTile + 1) : kv_tiles_all) : 0;
  const int n_kv = max(n0, n1);

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars->q_full), 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(smem_u32(&bars->kv_full[i]), 1);
      mbar_init(smem_u32(&bars->kv_empty[i]), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&bars->s_full[t]), 1);
      mbar_init(smem_u32(&bars->s_free[t]), 4);
      mbar_init(smem_u32(&bars->p_ready[t]), 4);
      mbar_init(smem_u32(&bars->pv_full[t]), 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&bars->tmem_base);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const uint32_t qf = smem_u32(&bars->q_full);
      mbar_expect_tx(qf, act1 ? 2 * kSlot : kSlot);
      for (int t = 0; t < (act1 ? 2 : 1); ++t)
        for (int h = 0; h < 2; ++h) tma_load_3d(q_s + t * kSlot + h * 16384, &tmQ, qf, h * 64, q_base0 + t * 128, bh);
      int err = 0, slot = 0;
      uint32_t ph = 0, issued = 0;
      // one ring entry: wait for the slot, then both 64-wide halves of a 128 x 128 tile
      auto load = [&](const CUtensorMap *tm, int row0) {
        if (!mbar_wait(smem_u32(&bars->kv_empty[slot]), ph ^ 1u)) { err = ERR_WAIT_EMPTY; return; }
        const uint32_t full = smem_u32(&bars->kv_full[slot]);
        mbar_expect_tx(full, kSlot);
        for (int h = 0; h < 2; ++h) tma_load_3d(ring_s + slot * kSlot + h * 16384, tm, full, h * 64, row0, bh);
        ++issued;
        if (++slot == kRing) { slot = 0; ph ^= 1u; }
      };
      load(&tmK, 0);
      for (int j = 0; j < n_kv && !err; ++j) {   // consumption order: K_{j+1} before V_j
        if (j + 1 < n_kv) load(&tmK, (j + 1) * kTile);
        if (!err) load(&tmV, j * kTile);
      }
      if (err) {
        atomicExch(p.error, err);
        // drain what was issued before leaving (bounded)
        mbar_wait(smem_u32(&bars->q_full), 0);
        for (uint32_t j = 0; j < min(issued, uint32_t(kRing)); ++j) {
          const uint32_t i2 = issued - 1 - j;
          if (!mbar_wait(smem_u32(&bars->kv_full[i2 % kRing]), (i2 / kRing) & 1u)) atomicExch(p.error, ERR_WAIT_DRAIN);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_qk = umma_instr_desc(1, 1, 1, 0, 0, 128, 128);   // A, B K-major
      // A (P) and B (V) must have the same 16-bit format: kind::f16 with an f16 A and a bf16 B operand
      // raises an illegal-instruction fault on sm_100a, so P is rounded to bf16 like V
      const uint32_t idesc_pv = umma_instr_desc(1, 1, 1, 0, 1, 128, 128);   // B (V) MN-major
      const int nt[2] = {n0, n1};
      int err = 0;
      // This thread's instruction stream is the tensor pipe's critical path: descriptors are split into
      // a constant high word and a low word (start address in 16-byte units | leading offset << 16)
      // that advances by a compile-time constant per K step.
      const uint32_t hi_k = uint32_t(umma_smem_desc(0, 16, 1024) >> 32);
      const uint32_t hi_v = uint32_t(umma_smem_desc(0, 16384, 1024) >> 32);
      auto lo_k = [](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1u << 16); };
      auto lo_v = [](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1024u << 16); };
      auto dsc = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | uint64_t(lo); };
      const uint32_t q_lo[2] = {lo_k(q_s), lo_k(q_s + kSlot)};
      const uint32_t p_lo[2] = {lo_k(p_s), lo_k(p_s + kSlot)};
      const uint32_t s_full_b[2] = {smem_u32(&bars->s_full[0]), smem_u32(&bars->s_full[1])};
      const uint32_t s_free_b[2] = {smem_u32(&bars->s_free[0]), smem_u32(&bars->s_free[1])};
      const uint32_t p_ready_b[2] = {smem_u32(&bars->p_ready[0]), smem_u32(&bars->p_ready[1])};
      const uint32_t pv_full_b[2] = {smem_u32(&bars->pv_full[0]), smem_u32(&bars->pv_full[1])};
      auto issue_qk = [&](int t, uint32_t kslot) {
        const uint32_t d = tmem + uint32_t(t) * 128u;
        const uint32_t a = q_lo[t], b = lo_k(kslot);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          const uint32_t off = uint32_t(s >> 2) * 1024u + uint32_t(s & 3) * 2u;
          umma_f16(d, dsc(a + off, hi_k), dsc(b + off, hi_k), idesc_qk, s > 0 ? 1u : 0u);
        }
        umma_commit(s_full_b[t]);
      };
      // ring position of the next entry to consume (same order as the producer fills it)
      int slot = 0;
      uint32_t ph = 0;
      auto ring_wait = [&]() { return mbar_wait(smem_u32(&bars->kv_full[slot]), ph); };
      auto ring_release = [&]() {
        umma_commit(smem_u32(&bars->kv_empty[slot]));   // free once the MMAs issued so far retire
        if (++slot == kRing) { slot = 0; ph ^= 1u; }
      };
      if (!mbar_wait(smem_u32(&bars->q_full), 0)) err = ERR_WAIT_FULL;
      if (!err && !ring_wait()) err = ERR_WAIT_FULL;
      if (!err) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (nt[t] > 0) issue_qk(t, ring_s + uint32_t(slot) * kSlot);
        ring_release();
      }
      for (int j = 0; j < n_kv && !err; ++j) {
        // ---- scores of the next key tile, as soon as each stream has copied its S to registers
        if (j + 1 < n_kv) {
          if (!ring_wait()) { err = ERR_WAIT_FULL; break; }
          const uint32_t kslot = ring_s + uint32_t(slot) * kSlot;
          for (int t = 0; t < 2 && !err; ++t) {
            if (j + 1 >= nt[t]) continue;
            if (!mbar_wait(s_free_b[t], uint32_t(j) & 1u)) { err = ERR_WAIT_TMEM_EMPTY; break; }
            tc_fence_after();
            issue_qk(t, kslot);
          }
          if (err) break;
          ring_release();
        }
        // ---- O_t += P_t V_j
        if (!ring_wait()) { err = ERR_WAIT_FULL; break; }
        const uint32_t v_lo = lo_v(ring_s + uint32_t(slot) * kSlot);
        for (int t = 0; t < 2 && !err; ++t) {
          if (j >= nt[t]) continue;
          if (!mbar_wait(p_ready_b[t], uint32_t(j) & 1u)) { err = ERR_WAIT_TMEM_EMPTY; break; }
          tc_fence_after();
          const uint32_t d = tmem + 256u + uint32_t(t) * 128u;
          const uint32_t a = p_lo[t];
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            const uint32_t off = uint32_t(s >> 2) * 1024u + uint32_t(s & 3) * 2u;
            umma_f16(d, dsc(a + off, hi_k), dsc(v_lo + uint32_t(s) * 128u, hi_v), idesc_pv, (j > 0 || s > 0) ? 1u : 0u);
          }
          umma_commit(pv_full_b[t]);
        }
        if (err) break;
        ring_release();
      }
      if (err) atomicExch(p.error, err);
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue
    const int t = (warp - 2) >> 2;                  // stream
    const int q = warp & 3;                         // TMEM lane quadrant
    const int row = q * 32 + lane;                  // row within the stream's query tile
    const int q_row = (t == 0 ? q_base0 : q_base1) + row;
    const int nk = (t == 0) ? n0 : n1;
    const uint32_t s_addr = tmem + uint32_t(t) * 128u + (uint32_t(q * 32) << 16);
    const uint32_t o_addr = tmem + 256u + uint32_t(t) * 128u + (uint32_t(q * 32) << 16);
    uint8_t *pbuf = smem + (2 + kRing + t) * kSlot + row * 128;
    const uint32_t s_full_b = smem_u32(&bars->s_full[t]), s_free_b = smem_u32(&bars->s_free[t]);
    const uint32_t p_ready_b = smem_u32(&bars->p_ready[t]), pv_full_b = smem_u32(&bars->pv_full[t]);
    const float c = p.scale_log2e;

    float m_used = -INFINITY;   // reference maximum the exponentials and O currently use (scaled, log2 domain)
    float l = 0.f;              // running row sum in that reference
    bool dead = false;

    for (int j = 0; j < nk && !dead; ++j) {
      if (!mbar_wait(s_full_b, uint32_t(j) & 1u)) {
        if (lane == 0) atomicExch(p.error, ERR_WAIT_TMEM_FULL);
        dead = true;
        break;
      }
      tc_fence_after();
      // ---- the whole score row to registers, then hand S back to the MMA warp
      uint32_t sv[128];
      {
        uint32_t(&c0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[0]);
        uint32_t(&c1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[32]);
        uint32_t(&c2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[64]);
        uint32_t(&c3)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[96]);
        tmem_ld_x32(s_addr, c0);
        tmem_ld_x32(s_addr + 32, c1);
        tmem_ld_x32(s_addr + 64, c2);
        tmem_ld_x32(s_addr + 96, c3);
        tmem_wait_ld();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free_b);

      // columns of this tile that take part: inside the sequence and, when causal, not above the diagonal
      const int kv0 = j * kTile;
      int lim = p.seq - kv0;
      if (p.causal) lim = min(lim, q_row - kv0 + 1);
      if (lim < kTile) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i >= lim) sv[i] = 0xFF800000u;   // -inf
      }
      float mx = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx = max3(mx, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
        mx_b = max3(mx_b, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
      }
      mx = fmaxf(mx, mx_b);
      const float m_tile = mx * c;
      // lazy reference update: keep the old reference unless the maximum grew by more than 2^kLazy
      const bool grow = m_tile > m_used + kLazy;
      const float alpha = grow ? ex2(m_used - m_tile) : 1.f;   // 0 on the first tile (m_used = -inf)
      if (grow) m_used = m_tile;
      l *= alpha;

      if (j > 0) {
        // P_t and O_t are free once the previous P V has retired
        if (!mbar_wait(pv_full_b, uint32_t(j - 1) & 1u)) {
          if (lane == 0) atomicExch(p.error, ERR_WAIT_TMEM_FULL);
          dead = true;
          break;
        }
        tc_fence_after();
        if (__any_sync(0xFFFFFFFFu, grow)) {
          // rescale this warp's 32 rows of O in place (rows that did not grow use alpha = 1)
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 16) {
            uint32_t v[16];
            tmem_ld_x16(o_addr + c0, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_x16(o_addr + c0, v);
          }
          tmem_wait_st();
        }
      }
      // ---- p = 2^(s*c - m_used), row sum, P -> shared memory (bf16, swizzled K-major)
      const uint64_t c2 = pack2(c, c), neg_m2 = pack2(-m_used, -m_used);
      uint64_t sum2 = pack2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 16; ++k) {   // sixteen 16-byte chunks of 8 columns
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x0, x1;
          unpack2(fma2(pack2(__uint_as_float(sv[k * 8 + e * 2]), __uint_as_float(sv[k * 8 + e * 2 + 1])), c2, neg_m2), x0, x1);
          const float p0 = ex2(x0), p1 = ex2(x1);
          sum2 = add2(sum2, pack2(p0, p1));
          w[e] = pack_bf16x2_rn(p0, p1);
        }
        // chunk k of the row: block (k >> 3), 16-byte slot (k & 7) ^ (row & 7)
        *reinterpret_cast<uint4 *>(pbuf + (k >> 3) * 16384 + (((k & 7) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      float sum, sum_hi;
      unpack2(sum2, sum, sum_hi);
      sum += sum_hi;
      l += sum;
      fence_proxy_async();     // P visible to the tensor core's shared-memory reads
      tc_fence_before();       // TMEM accesses above are ordered before the arrive
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready_b);
    }
    // ---- last P V, normalise, store
    if (!dead && nk > 0) {
      if (!mbar_wait(pv_full_b, uint32_t(nk - 1) & 1u)) {
        if (lane == 0) atomicExch(p.error, ERR_WAIT_TMEM_FULL);
      } else {
        tc_fence_after();
        const float inv = 1.f / l;
        uint16_t *orow = reinterpret_cast<uint16_t *>(p.O) + (size_t(bh) * p.seq + size_t(q_row)) * size_t(p.dim);
#pragma unroll
        for (int c0 = 0; c0 < 4; ++c0) {
          uint32_t v[32];
          tmem_ld_x32(o_addr + c0 * 32, v);
          tmem_wait_ld();
          if (q_row < p.seq) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = k * 8 + e * 2;
                w[e] = f32_to_bf16_bits(__uint_as_float(v[i]) * inv) | (f32_to_bf16_bits(__uint_as_float(v[i + 1]) * inv) << 16);
              }
              *reinterpret_cast<uint4 *>(orow + c0 * 32 + k * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

CUtensorMap make_qkv_map(const void *ptr, int64_t bh, int64_t seq, int64_t dim) {
  // [bh][seq][dim] bf16; box = 64 (dim) x 128 (rows) x 1; rows past `seq` read as zero
  typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      throw CudaError("cuTensorMapEncodeTiled is not available from the driver");
    fn = reinterpret_cast<EncodeTiledFn>(f);
  }
  CUtensorMap m;
  cuuint64_t dims[3] = {cuuint64_t(dim), cuuint64_t(seq), cuuint64_t(bh)};
  cuuint64_t strides[2] = {cuuint64_t(dim) * 2, cuuint64_t(dim) * cuuint64_t(seq) * 2};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw CudaError("cuTensorMapEncodeTiled (attention) failed with CUresult " + std::to_string(int(r)));
  return m;
}

} // namespace

void attention_bf16(const void *Q, const void *K, const void *V, void *O, int64_t bh, int64_t seq, int64_t dim,
                    float scale, int causal, cudaStream_t stream) {
  DeviceState &dev = device_state();
  if (dim != 128) throw std::logic_error("fused attention is built for head_dim 128");
  if (bh > 65535) throw std::logic_error("fused attention supports at most 65535 (batch x head) units per launch");
  for (const void *ptr : {Q, K, V, (const void *)O})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) throw std::invalid_argument("attention tensors must be 16-byte aligned");
  const CUtensorMap tq = make_qkv_map(Q, bh, seq, dim), tk = make_qkv_map(K, bh, seq, dim), tv = make_qkv_map(V, bh, seq, dim);
  AttParams p{};
  p.seq = int(seq);
  p.bh = int(bh);
  p.dim = int(dim);
  p.causal = causal;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.O = O;
  p.error = dev.d_error;
  p.q_pairs = int((seq + 255) / 256);
  const size_t smem = 1024 + size_t(2 + kRing + 2) * kSlot + sizeof(AttBars);
  static bool configured[64] = {};
  if (!configured[dev.device & 63]) {
    GCB_CUDA(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    configured[dev.device & 63] = true;
  }
  dim3 grid(unsigned(p.q_pairs), unsigned(bh));
  attention_kernel<<<grid, kAttThreads, smem, stream>>>(tq, tk, tv, p);
  GCB_CUDA(cudaGetLastError());
  count_launch();
}

} // namespace gcb
