// Measured matmul configurations, kept per shape and persisted as text.
//
// The tile selector is a fitted time model; for shapes where the model is off, a configuration
// found by timing candidates on the device can be recorded here and takes precedence.  The
// reference has the per-op override attributes of MatmulConfigAnalysis.cpp:368-401 for the same
// purpose (a hand-written config per matmul op); a cache keyed by shape plays that role for a
// backend that never sees the op's attributes.
//
// File format, one entry per line ('#' starts a comment):
//   M N K dtype_bytes out_bytes : swapped bn splits stages group_m grid pair kpb
// A file is loaded once from the path in GC_B200_TUNE_CACHE (if set) and can be loaded / saved explicitly.
#pragma once
#include <cstdint>
#include <string>

#include "runtime.h"

namespace gcb {
namespace tune {

struct Key {
  int64_t M, N, K;
  int dtype_bytes, out_bytes;
  bool operator<(const Key &o) const;
};

// True (and *out filled) when the shape has a recorded configuration.  Loads GC_B200_TUNE_CACHE on first use.
bool lookup(const Key &k, MatmulConfig *out);
// Records (or replaces) the configuration of a shape.  Throws std::invalid_argument for a configuration
// that no kernel can run (tile width, split factor, stage count out of range).
void put(const Key &k, const MatmulConfig &c);
// Merges the entries of a file into the cache; returns how many were read.  Throws on a malformed line.
int load(const std::string &path);
// Writes every entry; returns how many were written.
int save(const std::string &path);
// Forgets one shape (no effect when it has no entry).
void erase(const Key &k);
void clear();
int size();

} // namespace tune
} // namespace gcb
