#include "memplan.h"

#include <algorithm>
#include <cmath>
#include <limits>
#include <stdexcept>

namespace gcb {
namespace memplan {

namespace {

// One contiguous piece of the large buffer.  `segs_` always tiles [0, total_) in address order.
struct Seg {
  uint64_t id;        // stable identity (buffers refer to segments by id)
  size_t start, size;
  bool free;
  size_t tick;        // when it was last released
  uint64_t stamp;     // order of insertion into the free set (ties between equal sizes / ticks)
  bool remainder;     // right part of an in-place take-over that still belongs to the reused buffer
};

class Planner {
public:
  Planner(size_t alignment, bool hot_first, const InplaceHints &hints,
          std::unordered_map<uint64_t, std::vector<uint64_t>> &reused)
      : align_(alignment ? alignment : 1), hot_first_(hot_first), hints_(hints), reused_(reused) {}

  void allocate(uint64_t buffer, size_t size) {
    ++tick_;
    const size_t need = (size + align_ - 1) / align_ * align_;
    long at = take_over(buffer, need);
    if (at < 0) at = place(need);
    anchor_of_[buffer] = anchors_.size();
    anchors_.push_back(segs_[size_t(at)].start);
    current_[buffer] = segs_[size_t(at)].id;
  }

  void release(uint64_t buffer) {
    if (!anchor_of_.count(buffer)) throw std::invalid_argument("release of a buffer that was never allocated");
    auto it = current_.find(buffer);
    if (it == current_.end()) return;   // taken over by another buffer earlier
    size_t i = index_of(it->second);
    current_.erase(it);
    segs_[i].remainder = false;
    ++tick_;
    segs_[i].tick = tick_;
    set_free(i);
    // merge with free neighbours on both sides
    size_t l = i, r = i;
    while (l > 0 && segs_[l - 1].free) --l;
    while (r + 1 < segs_.size() && segs_[r + 1].free) ++r;
    if (r > l) {
      merge(l, r);
      segs_[l].tick = tick_;
      set_free(l);
    }
  }

  size_t total() const { return total_; }

  void offsets(std::unordered_map<uint64_t, size_t> &out) const {
    for (auto &kv : anchor_of_) out[kv.first] = anchors_[kv.second];
  }

private:
  size_t index_of(uint64_t id) const {
    for (size_t i = 0; i < segs_.size(); ++i)
      if (segs_[i].id == id) return i;
    throw std::logic_error("memory planner: segment not found");
  }
  void set_free(size_t i) {
    segs_[i].free = true;
    segs_[i].stamp = ++stamp_;
  }
  bool any_free() const {
    return std::any_of(segs_.begin(), segs_.end(), [](const Seg &s) { return s.free; });
  }

  // Closeness of a piece of `have` elements to a request of `want`, +1 when no growth is needed
  // (StaticMemoryPlanning.cpp:256-269).
  static float size_score(size_t have, size_t want) {
    const float diff = std::fabs(float(int64_t(have) - int64_t(want)));
    float s = -diff / float(std::max(have, want));
    if (want <= have) s += 1.f;
    return s;
  }
  // ... plus how recently it was released: 1 - min(1, age / 10) (:277-286)
  float heat_score(const Seg &s, size_t want) const {
    const float age = float(int64_t(tick_) - int64_t(s.tick)) / 10.f;
    return size_score(s.size, want) + (1.f - std::min(age, 1.f));
  }

  // Grow segment i to `new_size`; everything to its right, and every recorded anchor there, moves.
  void grow(size_t i, size_t new_size) {
    const size_t d = new_size - segs_[i].size, old_end = segs_[i].start + segs_[i].size;
    segs_[i].size = new_size;
    segs_[i].free = false;
    total_ += d;
    for (size_t j = i + 1; j < segs_.size(); ++j) segs_[j].start += d;
    for (size_t &a : anchors_)
      if (a >= old_end) a += d;
  }

  // Use the first `need` elements of free segment i; the rest stays free with the same release tick.
  void carve(size_t i, size_t need) {
    if (segs_[i].size == need) {
      segs_[i].free = false;
      return;
    }
    Seg rest = segs_[i];
    rest.id = ++ids_;
    rest.start += need;
    rest.size -= need;
    rest.free = true;
    rest.stamp = ++stamp_;
    rest.remainder = false;
    segs_[i].size = need;
    segs_[i].free = false;
    segs_.insert(segs_.begin() + long(i) + 1, rest);
  }

  void merge(size_t l, size_t r) {
    Seg m = segs_[l];
    m.id = ++ids_;
    m.size = 0;
    for (size_t j = l; j <= r; ++j) m.size += segs_[j].size;
    m.remainder = false;
    segs_.erase(segs_.begin() + long(l) + 1, segs_.begin() + long(r) + 1);
    segs_[l] = m;
  }

  // Ordinary placement: a new piece at the end when nothing is free; otherwise the hottest / best
  // scoring free piece (hot first) or the smallest free piece that fits, else the largest one, grown.
  long place(size_t need) {
    if (!any_free()) {
      segs_.push_back(Seg{++ids_, total_, need, false, 0, 0, false});
      total_ += need;
      return long(segs_.size()) - 1;
    }
    long pick = -1;
    if (hot_first_) {
      // start from the most recently released piece, then walk from the coldest: a strictly better score wins
      std::vector<size_t> order;
      for (size_t i = 0; i < segs_.size(); ++i)
        if (segs_[i].free) order.push_back(i);
      std::sort(order.begin(), order.end(), [&](size_t a, size_t b) {
        return segs_[a].tick != segs_[b].tick ? segs_[a].tick < segs_[b].tick : segs_[a].stamp < segs_[b].stamp;
      });
      pick = long(order.back());
      float best = heat_score(segs_[size_t(pick)], need);
      for (size_t i : order) {
        const float sc = heat_score(segs_[i], need);
        if (sc > best) { best = sc; pick = long(i); }
      }
    } else {
      long largest = -1;
      for (size_t i = 0; i < segs_.size(); ++i) {
        const Seg &s = segs_[i];
        if (!s.free) continue;
        if (s.size >= need && (pick < 0 || s.size < segs_[size_t(pick)].size ||
                               (s.size == segs_[size_t(pick)].size && s.stamp < segs_[size_t(pick)].stamp)))
          pick = long(i);
        if (largest < 0 || s.size > segs_[size_t(largest)].size ||
            (s.size == segs_[size_t(largest)].size && s.stamp > segs_[size_t(largest)].stamp))
          largest = long(i);
      }
      if (pick < 0) pick = largest;
    }
    if (segs_[size_t(pick)].size < need) grow(size_t(pick), need);
    else carve(size_t(pick), need);
    return pick;
  }

  // In-place take-over of buffers that are still live but about to be released (:313-497).
  long take_over(uint64_t buffer, size_t need) {
    auto h = hints_.find(buffer);
    if (h == hints_.end() || h->second.empty()) return -1;
    const auto &cands = h->second;
    // segment id -> the candidate living there
    std::unordered_map<uint64_t, const std::pair<uint64_t, InplaceKind> *> owner;
    for (auto &c : cands) {
      auto it = current_.find(c.first);
      if (it != current_.end()) owner[it->second] = &c;
    }
    auto mergeable = [&](const Seg &s) {
      if (s.free) return true;
      auto o = owner.find(s.id);
      return o != owner.end() && o->second->second == InplaceKind::Free;
    };
    // the candidate whose neighbourhood comes closest to the request
    float best = -std::numeric_limits<float>::infinity();
    long first = -1, last = -1;
    size_t have = 0;
    for (auto &c : cands) {
      auto it = current_.find(c.first);
      if (it == current_.end()) continue;   // already taken over by someone else
      const size_t v = index_of(it->second);
      if (segs_[v].remainder && owner[segs_[v].id]->second == InplaceKind::ZeroOffset) continue;
      size_t got = segs_[v].size, e = v;
      while (e + 1 < segs_.size() && got < need && mergeable(segs_[e + 1])) got += segs_[++e].size;
      const float sc = size_score(got, need);
      if (sc > best) { best = sc; first = long(v); last = long(e); have = got; }
    }
    if (have * 10 < need || first < 0) return -1;   // too little to gain
    const size_t l = size_t(first), r = size_t(last);
    segs_[l].tick = tick_;
    for (size_t j = l; j <= r; ++j) {
      auto o = owner.find(segs_[j].id);
      if (o != owner.end() && o->second->first) reused_[buffer].push_back(o->second->first);
    }
    if (have < need) {
      grow(r, need - have + segs_[r].size);
      have = need;
    }
    const bool tail_owned = owner.count(segs_[r].id) != 0;
    const uint64_t tail_owner = tail_owned ? owner[segs_[r].id]->first : 0;
    for (size_t j = l; j <= r; ++j) {
      segs_[j].free = false;
      auto o = owner.find(segs_[j].id);
      if (o != owner.end()) current_.erase(o->second->first);
    }
    if (r > l) merge(l, r);
    segs_[l].tick = tick_;
    segs_[l].free = false;
    if (have > need) {
      segs_[l].free = true;
      carve(l, need);
      if (tail_owned) {
        // the right part still belongs to the buffer that was reused: it is released with that buffer
        segs_[l + 1].free = false;
        segs_[l + 1].remainder = true;
        current_[tail_owner] = segs_[l + 1].id;
      }
    }
    return long(l);
  }

  size_t align_;
  bool hot_first_;
  const InplaceHints &hints_;
  std::unordered_map<uint64_t, std::vector<uint64_t>> &reused_;
  std::vector<Seg> segs_;
  std::vector<size_t> anchors_;
  std::unordered_map<uint64_t, size_t> anchor_of_;    // buffer -> index into anchors_ (its final offset)
  std::unordered_map<uint64_t, uint64_t> current_;    // live buffer -> id of the segment it occupies now
  size_t total_ = 0, tick_ = 0;
  uint64_t ids_ = 0, stamp_ = 0;
};

} // namespace

size_t schedule(const std::vector<Trace> &traces, size_t alignment, bool hot_first, const InplaceHints &hints,
                std::unordered_map<uint64_t, size_t> &offsets,
                std::unordered_map<uint64_t, std::vector<uint64_t>> &reused) {
  Planner p(alignment, hot_first, hints, reused);
  for (const Trace &t : traces) {
    if (t.size > 0) p.allocate(t.buffer, t.size);
    else p.release(t.buffer);
  }
  p.offsets(offsets);
  return p.total();
}

} // namespace memplan
} // namespace gcb
