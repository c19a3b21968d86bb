// Logging with the reference's switches (include/gc/Utils/Log.h:43-66): gcLogD(...) prints
// "[DEBUG] [file:line] ..." to stdout when the environment variable GC_DEBUG holds an (extended) regular
// expression that matches the path of the source file the call sits in (GC_DEBUG=.* enables all of them,
// GC_DEBUG=executable only this backend's executor, ...); gcLogE(...) always prints "[ERROR] [file:line] ..."
// to stderr.  GC_B200_VERBOSE=1 additionally prints, once per compiled partition, the launch plan with the
// kernel and tile chosen for every step - what the reference prints under LLVM_DEBUG when it has picked a
// matmul configuration (lib/gc/Analysis/MatmulConfigAnalysis.cpp:544-546).
#pragma once
#include <cstdlib>
#include <iostream>
#include <regex>
#include <sstream>
#include <string>

namespace gcb::logging {

inline bool debug_enabled(const char *file_name) {
  static const std::regex *pattern = [] {
    const char *env = std::getenv("GC_DEBUG");
    if (!env || !*env) return static_cast<const std::regex *>(nullptr);
    try {
      return static_cast<const std::regex *>(new std::regex(env, std::regex::extended));
    } catch (const std::regex_error &) {
      std::cerr << "[ERROR] GC_DEBUG is not a valid extended regular expression: " << env << std::endl;
      return static_cast<const std::regex *>(nullptr);
    }
  }();
  return pattern && std::regex_search(file_name, *pattern);
}

inline bool verbose() {
  static const bool on = [] { const char *e = std::getenv("GC_B200_VERBOSE"); return e && *e && *e != '0'; }();
  return on;
}

template <typename... Args> void emit(std::ostream &stream, const char *pref, const char *file, int line, const Args &...args) {
  std::ostringstream os;   // one write per line, so that lines of different threads do not interleave
  os << "[" << pref << "] [" << file << ":" << line << "] ";
  (os << ... << args);
  os << "\n";
  stream << os.str() << std::flush;
}

} // namespace gcb::logging

#define gcLogD(...)                                                                              \
  do {                                                                                           \
    if (::gcb::logging::debug_enabled(__FILE__)) ::gcb::logging::emit(std::cout, "DEBUG", __FILE__, __LINE__, __VA_ARGS__); \
  } while (0)
#define gcLogE(...) ::gcb::logging::emit(std::cerr, "ERROR", __FILE__, __LINE__, __VA_ARGS__)
