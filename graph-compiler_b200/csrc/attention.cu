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
//   warp 0       TMA producer: Q (once), then K_0, V_0, K_1, V_1, ... into a ring of 32 KiB slots
//   warp 1       MMA issuer: S_t = Q_t K_j^T and PV_t = P_t V_j (tcgen05.mma, accumulators in TMEM)
//   warps 2..5   softmax / accumulate / epilogue of stream 0 (one query row per thread)
//   warps 6..9   the same for stream 1
//
// Per key tile and stream: the softmax warps read S from TMEM (row max; then exp2, row sum), write
// P as bf16 into shared memory in the K-major 128-byte-swizzled layout the MMA reads, the MMA warp
// issues P V into a fresh TMEM buffer, and the softmax warps fold it into their register
// accumulators with the usual rescale  O <- (O + PV_{j-1}) * 2^(m_{j-1} - m_j).
//
// Shared memory: Q 2 x 32 KiB, K/V ring 3 x 32 KiB, P 2 x 32 KiB = 224 KiB.  TMEM: S0 S1 PV0 PV1,
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
  uint64_t s_full[2];
  uint64_t p_ready[2];
  uint64_t pv_full[2];
  uint32_t tmem_base;
  uint32_t pad;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// descriptor of K-step `j` (16 elements of the contraction) of a K-major 128 x 128 bf16 tile stored as
// two 128-row x 128-byte swizzled blocks (contraction index 0..63 in block 0, 64..127 in block 1)
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile, int j) {
  return umma_smem_desc(tile + uint32_t(j >> 2) * 16384u + uint32_t(j & 3) * 32u, 16, 1024);
}
// descriptor of K-step `j` (16 key rows) of V [128 keys x 128 d] used as an MN-major B operand:
// two 64-wide d blocks 16 KiB apart (leading offset), 8-row groups 1 KiB apart (stride offset)
__device__ __forceinline__ uint64_t v_desc(uint32_t tile, int j) {
  return umma_smem_desc(tile + uint32_t(j) * 2048u, 16384, 1024);
}

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
      int err = 0;
      uint32_t issued = 0;
      for (int i = 0; i < 2 * n_kv && !err; ++i) {   // i even: K_{i/2}, odd: V_{i/2}
        const int slot = i % kRing;
        const uint32_t ph = (i / kRing) & 1u;
        if (!mbar_wait(smem_u32(&bars->kv_empty[slot]), ph ^ 1u)) { err = ERR_WAIT_EMPTY; break; }
        const uint32_t full = smem_u32(&bars->kv_full[slot]);
        mbar_expect_tx(full, kSlot);
        const CUtensorMap *tm = (i & 1) ? &tmV : &tmK;
        for (int h = 0; h < 2; ++h) tma_load_3d(ring_s + slot * kSlot + h * 16384, tm, full, h * 64, (i >> 1) * kTile, bh);
        issued = uint32_t(i) + 1;
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
      auto issue_qk = [&](int t, int j, uint32_t kslot) {
        const uint32_t d = tmem + uint32_t(t) * 128u;
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_f16(d, kmajor_desc(q_s + t * kSlot, s), kmajor_desc(kslot, s), idesc_qk, s > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bars->s_full[t]));
        (void)j;
      };
      if (!mbar_wait(smem_u32(&bars->q_full), 0)) err = ERR_WAIT_FULL;
      // ring index of K_j is 2j, of V_j is 2j+1
      if (!err) {
        if (!mbar_wait(smem_u32(&bars->kv_full[0]), 0)) err = ERR_WAIT_FULL;
        tc_fence_after();
        if (!err) {
          for (int t = 0; t < 2; ++t)
            if (nt[t] > 0) issue_qk(t, 0, ring_s);
          // K_0 is released when these MMAs retire — unless a later QK of tile 0 is pending (none)
          umma_commit(smem_u32(&bars->kv_empty[0]));
        }
      }
      for (int j = 0; j < n_kv && !err; ++j) {
        const int iv = 2 * j + 1, ik = 2 * j + 2;          // ring indices of V_j and K_{j+1}
        const uint32_t vslot = ring_s + (iv % kRing) * kSlot, kslot = ring_s + (ik % kRing) * kSlot;
        if (!mbar_wait(smem_u32(&bars->kv_full[iv % kRing]), (iv / kRing) & 1u)) { err = ERR_WAIT_FULL; break; }
        const bool more = (j + 1 < n_kv);
        if (more && !mbar_wait(smem_u32(&bars->kv_full[ik % kRing]), (ik / kRing) & 1u)) { err = ERR_WAIT_FULL; break; }
        tc_fence_after();
        for (int t = 0; t < 2 && !err; ++t) {
          if (j >= nt[t]) continue;
          // P_t(j) written and PV_t buffer drained (the softmax warps arrive after both)
          if (!mbar_wait(smem_u32(&bars->p_ready[t]), uint32_t(j) & 1u)) { err = ERR_WAIT_TMEM_EMPTY; break; }
          tc_fence_after();
          const uint32_t d = tmem + 256u + uint32_t(t) * 128u;
#pragma unroll
          for (int s = 0; s < 8; ++s)
            umma_f16(d, kmajor_desc(p_s + t * kSlot, s), v_desc(vslot, s), idesc_pv, s > 0 ? 1u : 0u);
          umma_commit(smem_u32(&bars->pv_full[t]));
          if (j + 1 < nt[t]) issue_qk(t, j + 1, kslot);   // S_t is free: its softmax finished before p_ready
        }
        if (err) break;
        umma_commit(smem_u32(&bars->kv_empty[iv % kRing]));
        if (more) umma_commit(smem_u32(&bars->kv_empty[ik % kRing]));
      }
      if (err) atomicExch(p.error, err);
    }
  } else {
    // ---------------------------------------------------------------- softmax / accumulate / epilogue
    const int t = (warp - 2) >> 2;                  // stream
    const int q = warp & 3;                         // TMEM lane quadrant
    const int row = q * 32 + lane;                  // row within the stream's query tile
    const int q_row = (t == 0 ? q_base0 : q_base1) + row;
    const int nk = (t == 0) ? n0 : n1;
    const uint32_t s_addr = tmem + uint32_t(t) * 128u + (uint32_t(q * 32) << 16);
    const uint32_t pv_addr = tmem + 256u + uint32_t(t) * 128u + (uint32_t(q * 32) << 16);
    uint8_t *pbuf = smem + (2 + kRing + t) * kSlot;

    float o[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;   // running max (scaled, log2 domain) and running sum
    bool dead = false;

    for (int j = 0; j < nk && !dead; ++j) {
      if (!mbar_wait(smem_u32(&bars->s_full[t]), uint32_t(j) & 1u)) {
        if (lane == 0) atomicExch(p.error, ERR_WAIT_TMEM_FULL);
        dead = true;
        break;
      }
      tc_fence_after();
      const int kv0 = j * kTile;
      // columns of this tile that take part: inside the sequence and, when causal, not above the diagonal
      int lim = p.seq - kv0;
      if (p.causal) lim = min(lim, q_row - kv0 + 1);
      const bool full_tile = lim >= kTile;
      // ---- pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_x32(s_addr + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(v[i]);
          mx = (full_tile || c * 32 + i < lim) ? fmaxf(mx, s) : mx;
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2e);
      const float alpha = ex2(m - m_new);           // 0 on the first tile (m = -inf)
      // ---- fold the previous tile's P V into the accumulator, then rescale
      if (j > 0) {
        if (!mbar_wait(smem_u32(&bars->pv_full[t]), uint32_t(j - 1) & 1u)) {
          if (lane == 0) atomicExch(p.error, ERR_WAIT_TMEM_FULL);
          dead = true;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_x32(pv_addr + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(v[i])) * alpha;
        }
      }
      l *= alpha;
      m = m_new;
      // ---- pass 2: p = 2^(s*scale*log2e - m), row sum, P -> shared memory (bf16, swizzled K-major)
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_x32(s_addr + c * 32, v);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2(fmaf(__uint_as_float(v[i]), p.scale_log2e, -m));
          float p1 = ex2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2e, -m));
          if (!full_tile) {
            p0 = (c * 32 + i < lim) ? p0 : 0.f;
            p1 = (c * 32 + i + 1 < lim) ? p1 : 0.f;
          }
          sum += p0 + p1;
pk[i >> 1] = f32_to_bf16_bits(p0) | (f32_to_bf16_bits(p1) << 16);
        }
        // 32 columns = 64 bytes = four 16-byte chunks of block (c >> 1), chunk index (c & 1) * 4 + k
        uint8_t *blk = pbuf + (c >> 1) * 16384 + row * 128;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int chunk = ((c & 1) * 4 + k) ^ (row & 7);
          *reinterpret_cast<uint4 *>(blk + chunk * 16) = make_uint4(pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3]);
        }
      }
      l += sum;
      fence_proxy_async();     // P visible to the tensor core's shared-memory reads
      tc_fence_before();       // our TMEM reads of S and PV are ordered before the arrive
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->p_ready[t]));
    }
    // ---- last P V, normalise, store
    if (!dead && nk > 0) {
      if (!mbar_wait(smem_u32(&bars->pv_full[t]), uint32_t(nk - 1) & 1u)) {
        if (lane == 0) atomicExch(p.error, ERR_WAIT_TMEM_FULL);
      } else {
        tc_fence_after();
        const float inv = 1.f / l;
        uint16_t *orow = reinterpret_cast<uint16_t *>(p.O) + (size_t(bh) * p.seq + size_t(q_row)) * size_t(p.dim);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_x32(pv_addr + c * 32, v);
          tmem_wait_ld();
          if (q_row < p.seq) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = k * 8 + e * 2;
                const float a = (o[c * 32 + i] + __uint_as_float(v[i])) * inv;
                const float b = (o[c * 32 + i + 1] + __uint_as_float(v[i + 1])) * inv;
                w[e] = f32_to_bf16_bits(a) | (f32_to_bf16_bits(b) << 16);
              }
              *reinterpret_cast<uint4 *>(orow + c * 32 + k * 8) = make_uint4(w[0], w[1], w[2], w[3]);
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
