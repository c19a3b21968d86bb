// Host-visible description of one launch of the tcgen05 GEMM kernel.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace gcb {

enum OutKind : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_S32 = 2, OUT_DEQUANT_F32 = 3 };
enum BiasKind : int { BIAS_NONE = 0, BIAS_BF16 = 1, BIAS_F32 = 2 };
enum ErrCode : int {
  ERR_NONE = 0,
  ERR_WAIT_EMPTY = 1,      // producer: a pipeline stage was never released
  ERR_WAIT_FULL = 2,       // MMA: a stage's TMA bytes never arrived
  ERR_WAIT_TMEM_EMPTY = 3, // MMA: an accumulator was never drained
  ERR_WAIT_TMEM_FULL = 4,  // epilogue: an accumulator was never committed
  ERR_WAIT_DRAIN = 5,      // tear-down: an issued copy did not land
  ERR_WAIT_PEER = 6,       // a cross-GPU counter (rows landed / partial sums landed) never reached its target
  ERR_SELFTEST = 7,        // the wait self-test: a wait nobody satisfies ran out, as intended
};

// Geometry of one operand's pipeline stage in shared memory and of the
// descriptors that walk it.
struct OperandGeom {
  uint32_t mn_major;   // 0: K contiguous in memory, 1: MN contiguous
  uint32_t boxes;      // TMA boxes per stage
  uint32_t box_bytes;  // bytes per box
  uint32_t box_mn;     // MN elements covered by one box (MN-major only)
  uint32_t lbo, sbo;   // descriptor leading / stride byte offsets
  uint32_t kstep;      // bytes to advance the start address per MMA K step
  uint32_t bytes;      // bytes per stage
  uint32_t one_load;   // 1: the whole stage arrives with ONE TMA instruction (K-major: a 2-D box, or a
                       //    3-D box over [128-byte K block][MN][K block index] when a stage holds several K
                       //    blocks; MN-major: a 3-D box over [128-byte MN group][K][group index])
  uint32_t k3d;        // K-major only: the tensor map is the 3-D form (coordinates 0, mn, K block)
  uint32_t sub_step;   // descriptor bytes from one K block of a stage to the next
};

struct GemmParams {
  // D[Mm x Nm] = A[Mm x K] . B[Nm x K]^T in MMA orientation (for the swapped
  // orientation Mm indexes output columns and Nm output rows).
  int Mm, Nm, K;
  int BN;               // MMA N of one tile (multiple of 16, <= 256)
  int tiles_m, tiles_n; // tile grid in MMA orientation
  int k_blocks;         // K blocks of BK elements over the whole K
  int splits;           // split-K factor (1 = none)
  int bk_elems;         // elements per K block (128 bytes worth)
  int stages;
  int kpb;              // K blocks (of 128 bytes) per pipeline stage
  int group_m;          // rasterisation: tiles_m rows walked per column sweep
  OperandGeom a, b;
  uint32_t idesc;
  uint32_t tmem_cols;   // allocated TMEM columns (power of two >= 2*BN, >= 32)
  // epilogue
  int out_kind;
  void *out;            // [rows x ld_out]
  long long ld_out;     // elements
  long long split_stride; // elements between split-K partial planes (out_kind F32/S32 only)
  int bias_kind;
  const void *bias;     // indexed by output column
  const float *scale;   // OUT_DEQUANT_F32: per output column
  const int32_t *comp;  // OUT_DEQUANT_F32: per output column, subtracted from the accumulator
  int32_t *acc_dump;    // optional raw s32 accumulators [rows x ld_dump]
  long long ld_dump;
  int relu;
  int out_rows, out_cols; // logical output extent (for edge predication)
  // peer push (row-parallel layers): when n_peers > 0 the f32 tile is stored into plane `peer_plane`
  // of each of peer_out[0..n_peers) (buffers of [planes][out_rows][ld_out] f32) instead of `out`
  int n_peers, peer_plane;
  int peer_rows;        // 0: every peer receives the whole tile; > 0: rows [d * peer_rows, (d + 1) * peer_rows) go to
                        // peer d only, whose buffer is [planes][peer_rows][ld_out] (reduce-scatter by rows)
  int peer_multicast;   // 1: peer_out[0] is a multicast address covering every rank's buffer; one multimem store per chunk
  void *peer_out[8];
  // Hand-off between GPUs without a host round trip (tensor-parallel layers; see sm100_ptx.cuh).
  //  signal_peer[d] != null (row scatter only): after an epilogue warp has stored its 32 rows of a tile into owner d's
  //    buffer it fences at system scope and adds 1 to this counter in d's memory;
  //  wait_counter != null: both operand producers wait, before their first load, until this LOCAL counter has
  //    reached (*epoch + 1) * wait_per_step - the rows of the activations that other GPUs store into this GPU's memory.
  uint32_t *signal_peer[8];
  const uint32_t *wait_counter;
  const uint32_t *epoch;
  uint32_t wait_per_step;
  int *error;           // device int, set to an ErrCode on a bounded-wait time-out
  unsigned long long *trace;   // optional time stamps of this launch (sm100_ptx.cuh: trace_store / trace_max)
  // TMA-store epilogue (one-CTA kernel, row-major orientation): tmC covers the output as
  // [planes][rows][cols] with a box of {128 bytes of columns, 32 rows, 1}; each epilogue warp hands its
  // 32 x 128-byte slabs to the copy engine instead of storing them itself.
  int tma_store;
  CUtensorMap tmC;
  // Row scatter through the copy engine (tma_peer = 1, with tma_store): tmPeer[d] covers owner d's receive buffer as
  // [planes][rows per peer][cols] f32 with the same box; a warp's 32-row slab goes to its owner's buffer with one
  // cp.async.bulk.tensor store (plain bulk stores over NVLink, no loads from a peer).
  int tma_peer;
  CUtensorMap tmPeer[8];
};

// KIND: 0 = bf16 x bf16 -> f32, 1 = u8 x s8 -> s32.  SWAPPED: MMA rows are output columns.
template <int KIND, bool SWAPPED>
cudaError_t launch_gemm_kernel(const CUtensorMap &tmA, const CUtensorMap &tmB, const GemmParams &p, int grid,
                               size_t smem, cudaStream_t stream);

size_t gemm_smem_bytes(const GemmParams &p);

// CTA-pair form (tcgen05 cta_group::2): 256 x BN tiles, p.tiles_m counts 256-row tiles, p.b is one
// CTA's half of the B tile.  KIND as above; row-major output orientation only.
template <int KIND>
cudaError_t launch_gemm_pair_kernel(const CUtensorMap &tmA, const CUtensorMap &tmB, const GemmParams &p, int grid,
                                    size_t smem, cudaStream_t stream);
size_t gemm_pair_smem_bytes(const GemmParams &p);

} // namespace gcb
