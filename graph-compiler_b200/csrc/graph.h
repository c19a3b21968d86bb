// Partition model: what a oneDNN-graph JSON partition contains (reader that
// mirrors src/dnnl/JsonParser.cpp of the reference key for key and error class
// for error class) and the launch plan built from it (fusion of bias/ReLU
// post-ops into matmul epilogues, lifetimes and arena offsets of temporaries).
// Pure host code: no CUDA types here, so it is usable and testable without a GPU.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace gcb {

enum class DType : int { F16, BF16, F32, S32, S8, U8, F64, BOOLEAN, F8_E5M2, F8_E4M3, S4, U4 };
size_t dtype_bytes(DType t); // 0 for sub-byte types
const char *dtype_name(DType t);

struct LogicalTensor {
  size_t id = 0;
  DType dtype = DType::F32;
  std::vector<int64_t> shape;
  bool unranked = false;
  bool strided = false;
  std::vector<int64_t> stride; // meaningful when strided
  bool constant = false;       // property_type == "constant"
  int64_t numel() const;
};

struct AttrValue {
  enum Kind { BOOL, S64, F32, S64_ARRAY, F32_ARRAY, STRING } kind = BOOL;
  bool b = false;
  int64_t i = 0;
  float f = 0.f;
  std::vector<int64_t> is;
  std::vector<float> fs;
  std::string s;
};

struct GraphOp {
  std::string kind;
  std::vector<std::pair<std::string, AttrValue>> attrs;
  std::vector<LogicalTensor> inputs, outputs;
  const AttrValue *attr(const std::string &name) const;
  bool attr_bool(const std::string &name, bool dflt) const;
};

struct Partition {
  std::vector<GraphOp> ops;
  std::vector<size_t> input_ids;  // first-use order (JsonParser.cpp:184-192)
  std::vector<size_t> output_ids; // output_ports, or the last op's outputs (JsonParser.cpp:91-94)
  std::unordered_map<size_t, LogicalTensor> tensors;
};

// Throws std::invalid_argument for a malformed graph (-> dnnl_invalid_graph) and
// std::logic_error for an unsupported kind/dtype/engine/fpmath/layout
// (-> dnnl_unimplemented), the classes the reference's reader throws
// (JsonParser.cpp:42-72,144-209,236-258,274-303).
Partition read_partition(const std::string &json);

// ----------------------------------------------------------------------------- plan
struct TensorSlot {
  enum Where { INPUT, OUTPUT, ARENA } where = ARENA;
  int index = 0;        // position in Partition::input_ids / output_ids
  size_t offset = 0;    // byte offset in the arena
  size_t bytes = 0;
};

enum class StepKind { MATMUL, QMATMUL, SDPA, BINARY, UNARY, REDUCE, COPY };

struct Step {
  StepKind kind = StepKind::MATMUL;
  std::string op;                 // source op kind, for dumps ("MatMul", "Add", ...)
  std::vector<size_t> in;         // logical tensor ids
  std::vector<size_t> out;
  // MATMUL / QMATMUL
  int64_t M = 0, N = 0, K = 0;
  bool trans_a = false, trans_b = false, relu = false;
  bool has_bias = false;          // bias is in[2]
  int64_t zp_a = 0;               // QMATMUL
  int scratch_slot = -1;          // QMATMUL: arena temp for column sums
  bool raw_acc = false;           // QMATMUL: no scales; the single output holds acc - src_zp * colsum(w) as s32
  // SDPA
  int64_t batch = 0, heads = 0, seq = 0, dim = 0;
  float scale = 1.f;
  bool causal = false;
  // BINARY: 0 add 1 sub 2 mul 3 div ; UNARY: 0 relu 1 sigmoid 2 pow 3 typecast 4 exp 5 negate
  int fn = 0;
  float beta = 1.f;
  // REDUCE
  std::vector<int64_t> axes;
  bool mean = false;
};

struct Plan {
  Partition part;
  std::vector<Step> steps;
  std::unordered_map<size_t, TensorSlot> slots; // every tensor the steps touch
  std::vector<TensorSlot> scratch;              // per-step extra temporaries (arena)
  size_t arena_bytes = 0;
  // Debug mode (GC_B200_GUARD=<bytes>, read when the partition is compiled): every arena slice is planned with this
  // many bytes of canary before and after it; `guards` lists the bands as (arena offset, tensor id or ~0 for a
  // scratch slot).  The counterpart of the canary the reference's debug memory pool keeps at the head of every
  // allocation (lib/gc/ExecutionEngine/CPURuntime/MemoryPool.cpp:55-60, checked at :213-217).
  size_t guard_bytes = 0;
  std::vector<std::pair<size_t, size_t>> guards;
  std::string dump() const;                     // human-readable, stable (tests read it)
};

// Fuses MatMul [+ Add(bias [N])] [+ ReLU] chains into single steps when the
// intermediate value has no other consumer and is not a partition output (what
// IterativeTilingAndFusion.cpp:743-828 does for the tiled matmul), assigns
// arena offsets to temporaries by lifetime.
Plan build_plan(Partition part);

// ----------------------------------------------------------------------------- arena planner
// One buffer request: live over steps [first, last] (inclusive).
struct BufferLife {
  size_t bytes;
  int first, last;
};
// Offsets (aligned to `align`) such that buffers with overlapping lifetimes do
// not overlap in memory; returns the arena size.  Greedy by decreasing size,
// lowest fitting offset — the role StaticMemoryPlanning.cpp:628-652 plays for
// the reference's merge-alloc pass.
size_t plan_arena(const std::vector<BufferLife> &bufs, size_t align, std::vector<size_t> &offsets);

} // namespace gcb
