// Test-infrastructure stand-in for abseil's symbolizer (absent on this image): never resolves a symbol.
#pragma once
namespace absl {
inline bool Symbolize(const void*, char*, int) { return false; }
}  // namespace absl
