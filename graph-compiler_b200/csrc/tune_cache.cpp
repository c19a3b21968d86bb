#include "tune_cache.h"

#include <cstdlib>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <tuple>

namespace gcb {
namespace tune {

bool Key::operator<(const Key &o) const {
  return std::tie(M, N, K, dtype_bytes, out_bytes) < std::tie(o.M, o.N, o.K, o.dtype_bytes, o.out_bytes);
}

namespace {

struct Store {
  std::mutex mu;
  std::map<Key, MatmulConfig> entries;
  bool env_loaded = false;
};

Store &store() {
  static Store s;
  return s;
}

void validate(const Key &k, const MatmulConfig &c) {
  if (k.M <= 0 || k.N <= 0 || k.K <= 0 || (k.dtype_bytes != 1 && k.dtype_bytes != 2) || (k.out_bytes != 2 && k.out_bytes != 4))
    throw std::invalid_argument("tune cache: bad shape key");
  const bool bn_ok = c.swapped ? (c.bn >= 16 && c.bn <= 64 && c.bn % 16 == 0) : (c.bn >= 32 && c.bn <= 256 && c.bn % 32 == 0);
  if (!bn_ok || c.splits < 1 || c.splits > 64 || c.stages < 2 || c.stages > 8 || c.group_m < 1 || c.grid < 0 || c.kpb < 0 ||
      c.kpb > 4 || (c.pair != 0 && c.pair != 1) || (c.swapped != 0 && c.swapped != 1))
    throw std::invalid_argument("tune cache: configuration out of range");
}

int load_locked(Store &s, const std::string &path) {
  std::ifstream in(path);
  if (!in) throw std::invalid_argument("tune cache: cannot open " + path);
  std::string line;
  int n = 0, lineno = 0;
  while (std::getline(in, line)) {
    ++lineno;
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line.erase(hash);
    if (line.find_first_not_of(" \t\r") == std::string::npos) continue;
    std::istringstream ls(line);
    Key k{};
    MatmulConfig c{};
    char colon = 0;
    if (!(ls >> k.M >> k.N >> k.K >> k.dtype_bytes >> k.out_bytes >> colon >> c.swapped >> c.bn >> c.splits >> c.stages >>
          c.group_m >> c.grid >> c.pair >> c.kpb) ||
        colon != ':')
      throw std::invalid_argument("tune cache: malformed line " + std::to_string(lineno) + " in " + path);
    validate(k, c);
    s.entries[k] = c;
    ++n;
  }
  return n;
}

void ensure_env_loaded(Store &s) {
  if (s.env_loaded) return;
  s.env_loaded = true;
  if (const char *p = std::getenv("GC_B200_TUNE_CACHE")) {
    if (*p) {
      std::ifstream probe(p);
      if (probe) load_locked(s, p);   // a missing file is an empty cache (it is created by the first save)
    }
  }
}

} // namespace

bool lookup(const Key &k, MatmulConfig *out) {
  Store &s = store();
  std::lock_guard<std::mutex> g(s.mu);
  ensure_env_loaded(s);
  auto it = s.entries.find(k);
  if (it == s.entries.end()) return false;
  if (out) *out = it->second;
  return true;
}

void put(const Key &k, const MatmulConfig &c) {
  validate(k, c);
  Store &s = store();
  std::lock_guard<std::mutex> g(s.mu);
  ensure_env_loaded(s);
  s.entries[k] = c;
}

int load(const std::string &path) {
  Store &s = store();
  std::lock_guard<std::mutex> g(s.mu);
  ensure_env_loaded(s);
  return load_locked(s, path);
}

int save(const std::string &path) {
  Store &s = store();
  std::lock_guard<std::mutex> g(s.mu);
  std::ofstream out(path, std::ios::trunc);
  if (!out) throw std::invalid_argument("tune cache: cannot write " + path);
  out << "# gc_b200 matmul configurations found by timing candidates on the device\n"
      << "# M N K dtype_bytes out_bytes : swapped bn splits stages group_m grid pair kpb\n";
  for (const auto &kv : s.entries) {
    const Key &k = kv.first;
    const MatmulConfig &c = kv.second;
    out << k.M << ' ' << k.N << ' ' << k.K << ' ' << k.dtype_bytes << ' ' << k.out_bytes << " : " << c.swapped << ' ' << c.bn << ' '
        << c.splits << ' ' << c.stages << ' ' << c.group_m << ' ' << c.grid << ' ' << c.pair << ' ' << c.kpb << '\n';
  }
  if (!out) throw std::invalid_argument("tune cache: write failed for " + path);
  return int(s.entries.size());
}

void erase(const Key &k) {
  Store &s = store();
  std::lock_guard<std::mutex> g(s.mu);
  ensure_env_loaded(s);
  s.entries.erase(k);
}

void clear() {
  Store &s = store();
  std::lock_guard<std::mutex> g(s.mu);
  s.env_loaded = true;   // an explicit clear is not undone by the environment
  s.entries.clear();
}

int size() {
  Store &s = store();
  std::lock_guard<std::mutex> g(s.mu);
  ensure_env_loaded(s);
  return int(s.entries.size());
}

} // namespace tune
} // namespace gcb
