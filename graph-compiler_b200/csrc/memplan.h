// Static memory planning: offsets inside one large buffer for temporaries whose lifetimes are known
// as a trace of allocations and releases.  Same contract, policies and results as the reference's
// planner (lib/gc/Transforms/StaticMemoryPlanning.cpp:628-652 `scheduleMemoryAllocations`, chunk scoring
// :256-286, in-place reuse :313-497, best-fit / hot-first choice :499-551, release with neighbour merge
// :553-600); the representation is different: memory is a flat ordered list of segments with integer
// positions, and a buffer remembers an anchor position that is shifted whenever a segment to its
// left is extended, instead of a tree of split / merged chunk objects that derive offsets lazily.
#pragma once
#include <cstddef>
#include <cstdint>
#include <unordered_map>
#include <utility>
#include <vector>

namespace gcb {
namespace memplan {

struct Trace {
  uint64_t buffer;   // unique buffer id
  size_t size;       // > 0: allocation of `size` elements; 0: release
};

enum class InplaceKind : int {
  ZeroOffset = 0,   // the new buffer must start where the reused buffer starts
  Free = 1,         // any offset inside the reused buffer
};

// buffer -> candidates (in order) it may take over while they are still live but about to be released
using InplaceHints = std::unordered_map<uint64_t, std::vector<std::pair<uint64_t, InplaceKind>>>;

// Returns the size of the large buffer (elements).  `offsets` receives the final offset of every
// buffer that was ever allocated; `reused` the candidates each buffer took over, in memory order.
size_t schedule(const std::vector<Trace> &traces, size_t alignment, bool hot_first, const InplaceHints &hints,
                std::unordered_map<uint64_t, size_t> &offsets,
                std::unordered_map<uint64_t, std::vector<uint64_t>> &reused);

} // namespace memplan
} // namespace gcb
