// Test-infrastructure stand-in for abseil's make_unique (absent on this image).
#pragma once
#include <memory>
namespace absl {
using std::make_unique;
}  // namespace absl
