// Minimal JSON document model and parser (RFC 8259 subset: no surrogate-pair
// decoding beyond pass-through) for oneDNN-graph partition files.  Object
// members keep their order because the partition reader validates key order in
// attribute objects the same way the reference's streaming reader does.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace gcb {

struct JsonError : std::invalid_argument {
  using std::invalid_argument::invalid_argument;
};

struct JsonValue {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0.0;
  int64_t inum = 0;       // exact value when the literal is an integer that fits
  bool is_int = false;
  std::string str;
  std::vector<JsonValue> arr;
  std::vector<std::pair<std::string, JsonValue>> obj;

  const JsonValue *find(const std::string &key) const {
    for (auto &kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

JsonValue parse_json(const std::string &text);

} // namespace gcb
