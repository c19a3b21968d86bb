#include "graph.h"
#include "memplan.h"

#include <algorithm>
#include <cstdlib>
#include <limits>
#include <map>
#include <set>
#include <sstream>
#include <stdexcept>

#include "json.h"

namespace gcb {

// ----------------------------------------------------------------------------- small helpers
size_t dtype_bytes(DType t) {
  switch (t) {
  case DType::F16:
  case DType::BF16: return 2;
  case DType::F32:
  case DType::S32: return 4;
  case DType::S8:
  case DType::U8:
  case DType::BOOLEAN:
  case DType::F8_E5M2:
  case DType::F8_E4M3: return 1;
  case DType::F64: return 8;
  default: return 0;
  }
}

const char *dtype_name(DType t) {
  static const char *names[] = {"f16", "bf16", "f32", "s32", "s8", "u8", "f64", "boolean", "f8_e5m2", "f8_e4m3", "s4", "u4"};
  return names[int(t)];
}

int64_t LogicalTensor::numel() const {
  int64_t n = 1;
  for (int64_t d : shape) n *= d;
  return n;
}

const AttrValue *GraphOp::attr(const std::string &name) const {
  for (auto &kv : attrs)
    if (kv.first == name) return &kv.second;
  return nullptr;
}
bool GraphOp::attr_bool(const std::string &name, bool dflt) const {
  const AttrValue *a = attr(name);
  return a ? a->b : dflt;
}

namespace {

[[noreturn]] void invalid(const std::string &m) { throw std::invalid_argument(m); }
[[noreturn]] void unsupported(const std::string &m) { throw std::logic_error(m); }

// The literal meaning of the names: "u8" is unsigned, "s8" signed.  (The
// reference's table builds them with swapped signedness flags,
// src/dnnl/JsonParser.h:178-179, which is harmless there because every op of its
// dialect demands float tensors.)
const std::map<std::string, DType> kDTypes = {
    {"f16", DType::F16},         {"bf16", DType::BF16},       {"f32", DType::F32},   {"s32", DType::S32},
    {"s8", DType::S8},           {"u8", DType::U8},           {"f64", DType::F64},   {"boolean", DType::BOOLEAN},
    {"f8_e5m2", DType::F8_E5M2}, {"f8_e4m3", DType::F8_E4M3}, {"s4", DType::S4},     {"u4", DType::U4}};

// The eleven kinds of the reference (src/dnnl/JsonParser.h:152-164) plus the extension kinds this backend
// adds: the two partitions the reference front end cannot express (int8 matmul with dequantisation, fused
// attention) and three small ops that the linalg form of the reference's own llama2 case needs when it is
// lowered to a partition (test/benchgc/cases/llama2.mlir: tensor.collapse/expand_shape, linalg.exp, linalg.negf).
const std::set<std::string> kKinds = {"Add",     "Divide",  "MatMul",   "Multiply", "Pow",           "ReduceMean", "ReduceSum",
                                      "ReLU",    "Sigmoid", "Subtract", "Typecast", "QuantizedMatMul", "SDPA",
                                      "StaticReshape", "Exp", "Negate"};

const std::string &as_string(const JsonValue &v, const char *what) {
  if (v.kind != JsonValue::String) invalid(std::string("string expected for ") + what);
  return v.str;
}
int64_t as_int(const JsonValue &v, const char *what) {
  if (v.kind == JsonValue::Bool) return v.b ? 1 : 0;
  if (v.kind != JsonValue::Number) invalid(std::string("number expected for ") + what);
  return v.is_int ? v.inum : int64_t(v.num);
}
std::vector<int64_t> as_int_array(const JsonValue &v, const char *what) {
  if (v.kind != JsonValue::Array) invalid(std::string("array expected for ") + what);
  std::vector<int64_t> out;
  for (auto &e : v.arr) out.push_back(as_int(e, what));
  return out;
}

LogicalTensor read_tensor(const JsonValue &v) {
  if (v.kind != JsonValue::Object) invalid("tensor object expected");
  LogicalTensor t;
  bool has_dtype = false;
  for (auto &kv : v.obj) {
    const std::string &k = kv.first;
    if (k == "id") t.id = size_t(as_int(kv.second, "id"));
    else if (k == "dtype") {
      auto it = kDTypes.find(as_string(kv.second, "dtype"));
      if (it == kDTypes.end()) unsupported("Unsupported dtype: " + kv.second.str);
      t.dtype = it->second;
      has_dtype = true;
    } else if (k == "shape") t.shape = as_int_array(kv.second, "shape");
    else if (k == "stride") t.stride = as_int_array(kv.second, "stride");
    else if (k == "layout_type") {
      const std::string &s = as_string(kv.second, "layout_type");
      if (s == "strided") t.strided = true;
      else if (s != "undef" && s != "any") unsupported("Unsupported layout_type: " + s);
    } else if (k == "property_type") {
      const std::string &s = as_string(kv.second, "property_type");
      if (s == "constant") t.constant = true;
      else if (s != "undef" && s != "variable") unsupported("Unsupported property_type: " + s);
    } else invalid("Unrecognized key: " + k);
  }
  if (!has_dtype) invalid("dtype is not specified");
  if (!t.strided) t.stride.clear();
  if (t.shape.size() == 1 && t.shape[0] == std::numeric_limits<int64_t>::min()) {
    t.unranked = true;
    t.shape.clear();
  }
  return t;
}

AttrValue read_attr(const JsonValue &v) {
  // {"type": T, "value": V} in exactly this order, nothing else (JsonParser.cpp:228-265)
  if (v.kind != JsonValue::Object) invalid("attribute object expected");
  if (v.obj.size() < 1 || v.obj[0].first != "type") invalid("Key expected: type");
  if (v.obj.size() < 2 || v.obj[1].first != "value") invalid("Key expected: value");
  if (v.obj.size() > 2) invalid("Unrecognized key: " + v.obj[2].first);
  const std::string &ty = as_string(v.obj[0].second, "type");
  const JsonValue &val = v.obj[1].second;
  AttrValue a;
  if (ty == "bool") { a.kind = AttrValue::BOOL; a.b = as_int(val, "bool") != 0; }
  else if (ty == "s64") { a.kind = AttrValue::S64; a.i = as_int(val, "s64"); }
  else if (ty == "f32") {
    if (val.kind != JsonValue::Number) invalid("number expected for f32");
    a.kind = AttrValue::F32; a.f = float(val.num);
  } else if (ty == "s64[]") { a.kind = AttrValue::S64_ARRAY; a.is = as_int_array(val, "s64[]"); }
  else if (ty == "f32[]") {
    if (val.kind != JsonValue::Array) invalid("array expected for f32[]");
    a.kind = AttrValue::F32_ARRAY;
    for (auto &e : val.arr) {
      if (e.kind != JsonValue::Number) invalid("number expected in f32[]");
      a.fs.push_back(float(e.num));
    }
  } else if (ty == "string") { a.kind = AttrValue::STRING; a.s = as_string(val, "string"); }
  else unsupported("Unsupported attribute type: " + ty);
  return a;
}

bool same_type(const LogicalTensor &a, const LogicalTensor &b) {
  return a.dtype == b.dtype && a.shape == b.shape && a.unranked == b.unranked;
}

} // namespace

Partition read_partition(const std::string &json) {
  JsonValue root;
  try {
    root = parse_json(json);
  } catch (const JsonError &e) {
    invalid(e.what());
  }
  if (root.kind != JsonValue::Object) invalid("top-level JSON object expected");
  Partition p;
  std::vector<size_t> input_ports;
  bool has_in = false, has_out = false;
  std::set<size_t> produced;
  std::vector<size_t> last_outputs;

  for (auto &kv : root.obj) {
    const std::string &k = kv.first;
    if (k == "version") {
      as_string(kv.second, "version");
    } else if (k == "engine_kind") {
      const std::string &s = as_string(kv.second, "engine_kind");
      if (s != "cpu" && s != "gpu") unsupported("Unsupported engine: " + s);
    } else if (k == "fpmath_mode") {
      const std::string &s = as_string(kv.second, "fpmath_mode");
      if (s != "strict" && s != "any")
        unsupported("Unsupported fpmath_mode: " + s + ". Only 'strict' and 'any' are currently supported.");
    } else if (k == "input_ports") {
      has_in = true;
      for (int64_t v : as_int_array(kv.second, "input_ports")) input_ports.push_back(size_t(v));
    } else if (k == "output_ports") {
      has_out = true;
      for (int64_t v : as_int_array(kv.second, "output_ports")) p.output_ids.push_back(size_t(v));
    } else if (k == "graph") {
      if (kv.second.kind != JsonValue::Array) invalid("graph must be an array");
      for (auto &opv : kv.second.arr) {
        if (opv.kind != JsonValue::Object) invalid("operation object expected");
        GraphOp op;
        bool has_kind = false;
        for (auto &okv : opv.obj) {
          const std::string &ok = okv.first;
          if (ok == "id") as_int(okv.second, "id");
          else if (ok == "name") as_string(okv.second, "name");
          else if (ok == "kind") {
            op.kind = as_string(okv.second, "kind");
            if (!kKinds.count(op.kind)) unsupported("Unsupported operation: " + op.kind);
            has_kind = true;
          } else if (ok == "attrs") {
            if (okv.second.kind != JsonValue::Object) invalid("attrs must be an object");
            for (auto &akv : okv.second.obj) {
              AttrValue a = read_attr(akv.second);
              if (akv.first == "auto_broadcast") { // converted to a boolean (JsonParser.cpp:164-177)
                if (a.kind != AttrValue::STRING) invalid("Invalid attribute type: auto_broadcast");
                if (a.s == "numpy") { a.kind = AttrValue::BOOL; a.b = true; }
                else if (a.s == "none") { a.kind = AttrValue::BOOL; a.b = false; }
                else invalid("Invalid auto_broadcast attribute value: " + a.s);
              }
              op.attrs.emplace_back(akv.first, std::move(a));
            }
          } else if (ok == "inputs") {
            if (okv.second.kind != JsonValue::Array) invalid("inputs must be an array");
            for (auto &tv : okv.second.arr) {
              LogicalTensor t = read_tensor(tv);
              auto it = p.tensors.find(t.id);
              if (it == p.tensors.end()) {
                p.tensors[t.id] = t;          // not produced by an earlier op: a partition argument
                p.input_ids.push_back(t.id);
              } else if (!same_type(it->second, t)) {
                invalid("Type mismatch for input: " + std::to_string(t.id));
              }
              op.inputs.push_back(std::move(t));
            }
          } else if (ok == "outputs") {
            if (okv.second.kind != JsonValue::Array) invalid("outputs must be an array");
            for (auto &tv : okv.second.arr) op.outputs.push_back(read_tensor(tv));
          } else {
            invalid("Unrecognized key: " + ok);
          }
        }
        if (!has_kind) invalid("Operation kind is not specified");
        last_outputs.clear();
        for (auto &t : op.outputs) {
          if (p.tensors.count(t.id)) invalid("Duplicate output id: " + std::to_string(t.id));
          p.tensors[t.id] = t;
          produced.insert(t.id);
          last_outputs.push_back(t.id);
        }
        p.ops.push_back(std::move(op));
      }
    } else {
      invalid("Unrecognized key: " + k);
    }
  }
  if (has_in) {
    if (input_ports.size() != p.input_ids.size())
      invalid("Length mismatch between input_ports and inputs: " + std::to_string(p.input_ids.size()));
    for (size_t id : p.input_ids)
      if (std::find(input_ports.begin(), input_ports.end(), id) == input_ports.end())
        invalid("Input not found in input_ports: " + std::to_string(id));
  }
  if (!has_out) p.output_ids = last_outputs;
  for (size_t id : p.output_ids)
    if (!p.tensors.count(id)) invalid("Output value not found: " + std::to_string(id));
  return p;
}

// ----------------------------------------------------------------------------- arena planner
size_t plan_arena(const std::vector<BufferLife> &bufs, size_t align, std::vector<size_t> &offsets) {
  // Lifetimes -> the allocation / release trace the planner takes (the reference collects the same
  // trace from alloc and last-use ticks, MergeAllocTickBased.cpp:435-464): at step t first the
  // buffers born at t are allocated, then those last used at t are released, so a step's inputs
  // and outputs never share memory.
  offsets.assign(bufs.size(), 0);
  int last_step = -1;
  for (const BufferLife &b : bufs) last_step = std::max(last_step, std::max(b.first, b.last));
  std::vector<memplan::Trace> traces;
  for (int t = 0; t <= last_step; ++t) {
    for (size_t i = 0; i < bufs.size(); ++i)
      if (bufs[i].first == t && bufs[i].bytes > 0) traces.push_back(memplan::Trace{uint64_t(i) + 1, bufs[i].bytes});
    for (size_t i = 0; i < bufs.size(); ++i)
      if (std::max(bufs[i].last, bufs[i].first) == t && bufs[i].bytes > 0) traces.push_back(memplan::Trace{uint64_t(i) + 1, 0});
  }
  std::unordered_map<uint64_t, size_t> out;
  std::unordered_map<uint64_t, std::vector<uint64_t>> reused;
  const size_t total = memplan::schedule(traces, align, /*hot_first=*/false, memplan::InplaceHints(), out, reused);
  for (auto &kv : out) offsets[size_t(kv.first - 1)] = kv.second;
  return total;
}

// ----------------------------------------------------------------------------- plan builder
namespace {

bool is_float(DType t) { return t == DType::F32 || t == DType::BF16 || t == DType::F16; }

struct UseInfo {
  int consumers = 0;
  bool is_output = false;
};

} // namespace

Plan build_plan(Partition part) {
  Plan plan;
  plan.part = std::move(part);
  const Partition &p = plan.part;

  std::unordered_map<size_t, UseInfo> uses;
  for (auto &op : p.ops)
    for (auto &t : op.inputs) uses[t.id].consumers++;
  for (size_t id : p.output_ids) uses[id].is_output = true;
  auto single_use_temp = [&](size_t id) { return uses[id].consumers == 1 && !uses[id].is_output; };

  std::vector<bool> consumed(p.ops.size(), false);
  for (size_t oi = 0; oi < p.ops.size(); ++oi) {
    if (consumed[oi]) continue;
    const GraphOp &op = p.ops[oi];
    for (auto &t : op.inputs)
      if (t.unranked) unsupported("unranked tensors are not supported");
    for (auto &t : op.outputs)
      if (t.unranked) unsupported("unranked tensors are not supported");
    Step st;
    st.op = op.kind;
    for (auto &t : op.inputs) st.in.push_back(t.id);
    for (auto &t : op.outputs) st.out.push_back(t.id);

    if (op.kind == "MatMul") {
      if (op.inputs.size() < 2 || op.inputs.size() > 3 || op.outputs.size() != 1) invalid("MatMul expects 2 or 3 inputs and 1 output");
      const LogicalTensor &A = op.inputs[0], &B = op.inputs[1], &Y = op.outputs[0];
      if (!is_float(A.dtype) || A.dtype != B.dtype || A.dtype != Y.dtype) unsupported("MatMul supports matching f32/bf16 operands");
      if (A.dtype == DType::F16) unsupported("f16 MatMul is not implemented");
      st.kind = StepKind::MATMUL;
      st.trans_a = op.attr_bool("transpose_a", false);
      st.trans_b = op.attr_bool("transpose_b", false);
      if (B.shape.size() != 2) unsupported("MatMul needs a 2-D weight operand");
      if (A.shape.size() < 2) invalid("MatMul operand rank must be at least 2");
      if (A.shape.size() > 2 && st.trans_a) unsupported("batched MatMul with transpose_a is not supported");
      // rank > 2 A with a 2-D B is flattened (OneDNNGraphToLinalg.cpp:383-419)
      int64_t rows = 1;
      for (size_t d = 0; d + 1 < A.shape.size(); ++d) rows *= A.shape[d];
      const int64_t a0 = A.shape.size() == 2 ? A.shape[0] : rows, a1 = A.shape.back();
      st.M = st.trans_a ? a1 : a0;
      st.K = st.trans_a ? a0 : a1;
      const int64_t kb = st.trans_b ? B.shape[1] : B.shape[0];
      st.N = st.trans_b ? B.shape[0] : B.shape[1];
      if (kb != st.K) invalid("MatMul inner dimensions do not match");
      if (Y.numel() != st.M * st.N) invalid("MatMul output shape does not match");
      if (op.inputs.size() == 3) {
        if (op.inputs[2].numel() != st.N || op.inputs[2].dtype != A.dtype) unsupported("MatMul bias must be [N] of the operand dtype");
        st.has_bias = true;
      }
      // ---- fuse a following Add(bias [N]) and ReLU: the post-ops the reference pulls into the tile loop
      size_t cur_out = Y.id, next = oi + 1;
      if (!st.has_bias && next < p.ops.size() && !consumed[next] && p.ops[next].kind == "Add" &&
          p.ops[next].inputs.size() == 2 && p.ops[next].outputs.size() == 1 && single_use_temp(cur_out)) {
        const GraphOp &add = p.ops[next];
        int mi = add.inputs[0].id == cur_out ? 0 : (add.inputs[1].id == cur_out ? 1 : -1);
        if (mi >= 0) {
          const LogicalTensor &other = add.inputs[1 - mi];
          const bool is_arg = std::find(p.input_ids.begin(), p.input_ids.end(), other.id) != p.input_ids.end();
          if (is_arg && other.numel() == st.N && other.shape.size() >= 1 && other.shape.back() == st.N &&
              other.dtype == A.dtype && add.attr_bool("auto_broadcast", true) && add.outputs[0].numel() == st.M * st.N) {
            st.has_bias = true;
            st.in.push_back(other.id);
            cur_out = add.outputs[0].id;
            consumed[next] = true;
            st.op += "+Add";
            ++next;
          }
        }
      }
      if (next < p.ops.size() && !consumed[next] && p.ops[next].kind == "ReLU" && p.ops[next].inputs.size() == 1 &&
          p.ops[next].outputs.size() == 1 && p.ops[next].inputs[0].id == cur_out && single_use_temp(cur_out)) {
        st.relu = true;
        cur_out = p.ops[next].outputs[0].id;
        consumed[next] = true;
        st.op += "+ReLU";
      }
      st.out = {cur_out};
    } else if (op.kind == "QuantizedMatMul") {
      // extension: inputs src u8 [M,K], weights s8 [K,N], scales f32 [N], optional bias f32 [N];
      // outputs dst f32 [M,N] and optionally the raw s32 accumulators [M,N]; attr src_zp (s64)
      // a third form: src and weights only, one s32 output - the zero-point-corrected accumulators
      // sum_k (src[m,k] - src_zp) * w[k,n] without dequantisation (what linalg.quantized_matmul computes)
      const bool raw = op.inputs.size() == 2 && op.outputs.size() == 1 && op.outputs[0].dtype == DType::S32;
      if (!raw && (op.inputs.size() < 3 || op.inputs.size() > 4 || op.outputs.empty() || op.outputs.size() > 2))
        invalid("QuantizedMatMul expects 3 or 4 inputs and 1 or 2 outputs (or 2 inputs and one s32 output)");
      if (op.inputs[0].dtype != DType::U8 || op.inputs[1].dtype != DType::S8 ||
          (!raw && (op.inputs[2].dtype != DType::F32 || op.outputs[0].dtype != DType::F32)))
        unsupported("QuantizedMatMul supports u8 x s8 -> f32 with f32 scales, or -> s32");
      if (op.inputs[0].shape.size() != 2 || op.inputs[1].shape.size() != 2) invalid("QuantizedMatMul operands must be 2-D");
      st.kind = StepKind::QMATMUL;
      st.M = op.inputs[0].shape[0];
      st.K = op.inputs[0].shape[1];
      st.N = op.inputs[1].shape[1];
      st.raw_acc = raw;
      if (op.inputs[1].shape[0] != st.K) invalid("QuantizedMatMul inner dimensions do not match");
      if (op.outputs[0].numel() != st.M * st.N) invalid("QuantizedMatMul output shape does not match");
      if (!raw && op.inputs[2].numel() != st.N) invalid("QuantizedMatMul needs one scale per output channel");
      st.has_bias = op.inputs.size() == 4;
      if (st.has_bias && (op.inputs[3].dtype != DType::F32 || op.inputs[3].numel() != st.N)) invalid("QuantizedMatMul bias must be f32 [N]");
      if (op.outputs.size() == 2 && op.outputs[1].dtype != DType::S32) invalid("second output must be s32");
      if (const AttrValue *z = op.attr("src_zp")) st.zp_a = z->i;
      st.relu = op.attr_bool("relu", false);
    } else if (op.kind == "SDPA") {
      // extension: Q, K, V bf16 [B,H,S,D] -> O bf16 [B,H,S,D]; attrs scale (f32), causal (bool)
      if (op.inputs.size() != 3 || op.outputs.size() != 1) invalid("SDPA expects Q, K, V and one output");
      for (auto &t : op.inputs)
        if (t.dtype != DType::BF16 || t.shape != op.inputs[0].shape) unsupported("SDPA supports bf16 Q, K, V of one shape");
      const auto &s = op.inputs[0].shape;
      if (s.size() != 4 && s.size() != 3) invalid("SDPA tensors must be [B,H,S,D] or [BH,S,D]");
      st.kind = StepKind::SDPA;
      st.dim = s.back();
      st.seq = s[s.size() - 2];
      st.heads = s.size() == 4 ? s[1] : 1;
      st.batch = s[0];
      if (const AttrValue *a = op.attr("scale")) st.scale = a->f;
      st.causal = op.attr_bool("causal", false);
    } else if (op.kind == "Add" || op.kind == "Subtract" || op.kind == "Multiply" || op.kind == "Divide") {
      if (op.inputs.size() != 2 || op.outputs.size() != 1) invalid(op.kind + " expects 2 inputs and 1 output");
      st.kind = StepKind::BINARY;
      st.fn = op.kind == "Add" ? 0 : op.kind == "Subtract" ? 1 : op.kind == "Multiply" ? 2 : 3;
      for (auto &t : op.inputs)
        if (!is_float(t.dtype)) unsupported(op.kind + " supports float tensors");
    } else if (op.kind == "StaticReshape") {
      // same elements, another shape (tensor.collapse_shape / expand_shape of the linalg form): a device copy
      if (op.inputs.size() != 1 || op.outputs.size() != 1) invalid("StaticReshape expects 1 input and 1 output");
      if (op.inputs[0].numel() != op.outputs[0].numel() || op.inputs[0].dtype != op.outputs[0].dtype)
        invalid("StaticReshape must keep the element count and the dtype");
      st.kind = StepKind::COPY;
    } else if (op.kind == "ReLU" || op.kind == "Sigmoid" || op.kind == "Pow" || op.kind == "Typecast" || op.kind == "Exp" ||
               op.kind == "Negate") {
      if (op.inputs.size() != 1 || op.outputs.size() != 1) invalid(op.kind + " expects 1 input and 1 output");
      st.kind = StepKind::UNARY;
      st.fn = op.kind == "ReLU" ? 0 : op.kind == "Sigmoid" ? 1 : op.kind == "Pow" ? 2 : op.kind == "Typecast" ? 3 : op.kind == "Exp" ? 4 : 5;
      if (op.kind == "Pow") {
        const AttrValue *b = op.attr("beta");
        if (!b) invalid("Pow needs attribute beta");
        st.beta = b->f;
      }
      if (!is_float(op.inputs[0].dtype) || !is_float(op.outputs[0].dtype)) unsupported(op.kind + " supports float tensors");
    } else if (op.kind == "ReduceSum" || op.kind == "ReduceMean") {
      if (op.inputs.size() != 1 || op.outputs.size() != 1) invalid(op.kind + " expects 1 input and 1 output");
      st.kind = StepKind::REDUCE;
      st.mean = op.kind == "ReduceMean";
      const AttrValue *ax = op.attr("axes");
      if (!ax) invalid(op.kind + " needs attribute axes");
      const int64_t r = int64_t(op.inputs[0].shape.size());
      for (int64_t a : ax->is) {
        if (a < -r || a >= r) invalid("reduce axis out of range");
        st.axes.push_back(a < 0 ? a + r : a);
      }
      if (!is_float(op.inputs[0].dtype)) unsupported(op.kind + " supports float tensors");
    } else {
      unsupported("Unsupported operation: " + op.kind);
    }
    plan.steps.push_back(std::move(st));
  }

  // ---- storage: arguments and results are the caller's; everything else lives in the arena
  size_t guard = 0;
  if (const char *g = std::getenv("GC_B200_GUARD")) {
    const long v = std::atol(g);
    if (v > 0) guard = (size_t(std::min<long>(v, 1 << 20)) + 255) / 256 * 256;   // whole 256-byte units keep slices TMA-aligned
  }
  plan.guard_bytes = guard;
  std::vector<BufferLife> lives;
  std::vector<size_t> live_ids;
  std::unordered_map<size_t, size_t> live_index;
  auto slot_for = [&](size_t id, int step) {
    auto in_it = std::find(p.input_ids.begin(), p.input_ids.end(), id);
    auto out_it = std::find(p.output_ids.begin(), p.output_ids.end(), id);
    const LogicalTensor &t = p.tensors.at(id);
    const size_t bytes = size_t(t.numel()) * dtype_bytes(t.dtype);
    if (dtype_bytes(t.dtype) == 0) unsupported(std::string("sub-byte dtype ") + dtype_name(t.dtype));
    if (in_it != p.input_ids.end()) {
      plan.slots[id] = TensorSlot{TensorSlot::INPUT, int(in_it - p.input_ids.begin()), 0, bytes};
    } else if (out_it != p.output_ids.end()) {
      plan.slots[id] = TensorSlot{TensorSlot::OUTPUT, int(out_it - p.output_ids.begin()), 0, bytes};
    } else {
      auto li = live_index.find(id);
      if (li == live_index.end()) {
        live_index[id] = lives.size();
        live_ids.push_back(id);
        lives.push_back(BufferLife{bytes + 2 * guard, step, step});
        plan.slots[id] = TensorSlot{TensorSlot::ARENA, 0, 0, bytes};
      } else {
        lives[li->second].last = std::max(lives[li->second].last, step);
      }
    }
  };
  std::vector<std::pair<size_t, int>> scratch_reqs; // (index in lives, step)
  for (size_t si = 0; si < plan.steps.size(); ++si) {
    Step &st = plan.steps[si];
    for (size_t id : st.out) slot_for(id, int(si));
    for (size_t id : st.in) slot_for(id, int(si));
    if (st.kind == StepKind::QMATMUL) {
      st.scratch_slot = int(plan.scratch.size());
      plan.scratch.push_back(TensorSlot{TensorSlot::ARENA, 0, 0, size_t(st.N) * 4});
      scratch_reqs.emplace_back(lives.size(), int(si));
      // The column sums of a constant weight are computed by the first call and kept for the following ones,
      // so their region must not be handed to any other temporary: it is live over every step (and, as the
      // arena belongs to the executable, from one call to the next).
      lives.push_back(BufferLife{size_t(st.N) * 4 + 2 * guard, 0, int(plan.steps.size()) - 1});
    }
  }
  // an output may also be consumed by a later op.  Results are written densely: an output declared with
  // other strides, or an output that is one of the partition's own arguments (nothing here produces it),
  // is refused at compile time instead of returning memory nobody wrote.
  for (size_t id : p.output_ids) {
    const LogicalTensor &t = p.tensors.at(id);
    if (std::find(p.input_ids.begin(), p.input_ids.end(), id) != p.input_ids.end())
      unsupported("output " + std::to_string(id) + " is a partition input: pass-through outputs are not supported");
    if (t.strided && t.stride.size() == t.shape.size()) {
      int64_t expect = 1;
      for (int d = int(t.shape.size()) - 1; d >= 0; --d) {
        if (t.shape[size_t(d)] != 1 && t.stride[size_t(d)] != expect)
          unsupported("output " + std::to_string(id) + " has non-dense strides: results are written row-major dense");
        expect *= t.shape[size_t(d)];
      }
    }
  }
  std::vector<size_t> offsets;
  plan.arena_bytes = plan_arena(lives, 1024, offsets);
  for (size_t i = 0; i < live_ids.size(); ++i) plan.slots[live_ids[i]].offset = offsets[live_index[live_ids[i]]] + guard;
  for (size_t i = 0; i < scratch_reqs.size(); ++i) plan.scratch[i].offset = offsets[scratch_reqs[i].first] + guard;
  if (guard) {
    for (size_t id : live_ids) {
      const TensorSlot &sl = plan.slots[id];
      plan.guards.emplace_back(sl.offset - guard, id);
      plan.guards.emplace_back(sl.offset + sl.bytes, id);
    }
    for (const TensorSlot &sl : plan.scratch) {
      plan.guards.emplace_back(sl.offset - guard, ~size_t(0));
      plan.guards.emplace_back(sl.offset + sl.bytes, ~size_t(0));
    }
  }
  return plan;
}

std::string Plan::dump() const {
  std::ostringstream os;
  os << "inputs:";
  for (size_t id : part.input_ids) os << ' ' << id;
  os << "\noutputs:";
  for (size_t id : part.output_ids) os << ' ' << id;
  os << "\narena_bytes: " << arena_bytes << "\n";
  if (guard_bytes) os << "guard_bytes: " << guard_bytes << " (" << guards.size() << " bands)\n";
  auto where = [&](size_t id) {
    const TensorSlot &s = slots.at(id);
    std::ostringstream w;
    w << id << (s.where == TensorSlot::INPUT ? "@in" : s.where == TensorSlot::OUTPUT ? "@out" : "@arena+");
    if (s.where == TensorSlot::ARENA) w << s.offset;
    else w << s.index;
    return w.str();
  };
  for (size_t i = 0; i < steps.size(); ++i) {
    const Step &s = steps[i];
    os << "step " << i << ": " << s.op;
    if (s.kind == StepKind::MATMUL || s.kind == StepKind::QMATMUL)
      os << " M=" << s.M << " N=" << s.N << " K=" << s.K << " ta=" << s.trans_a << " tb=" << s.trans_b
         << " bias=" << s.has_bias << " relu=" << s.relu;
    if (s.kind == StepKind::SDPA)
      os << " B=" << s.batch << " H=" << s.heads << " S=" << s.seq << " D=" << s.dim << " causal=" << s.causal;
    os << " in[";
    for (size_t j = 0; j < s.in.size(); ++j) os << (j ? " " : "") << where(s.in[j]);
    os << "] out[";
    for (size_t j = 0; j < s.out.size(); ++j) os << (j ? " " : "") << where(s.out[j]);
    os << "]\n";
  }
  return os.str();
}

} // namespace gcb
