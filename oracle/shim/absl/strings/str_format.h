// Test-infrastructure stand-in for abseil's StrFormat (absent on this image): printf-style formatting
// through snprintf, with std::string arguments passed as C strings.
#pragma once
#include <cstdio>
#include <string>
namespace absl {
namespace oracle_shim {
template <typename T>
inline T arg(const T& v) { return v; }
inline const char* arg(const std::string& s) { return s.c_str(); }
}  // namespace oracle_shim
template <typename... Args>
inline std::string StrFormat(const char* fmt, const Args&... args) {
  char buf[4096];
  std::snprintf(buf, sizeof(buf), fmt, oracle_shim::arg(args)...);
  return std::string(buf);
}
inline std::string StrFormat(const char* fmt) { return std::string(fmt); }
}  // namespace absl
