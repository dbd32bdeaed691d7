// Test-infrastructure stand-in for abseil's variant (absent on this image): the C++17 std equivalents.
#pragma once
#include <variant>
namespace absl {
using std::get;
using std::holds_alternative;
using std::monostate;
using std::variant;
using std::visit;
}  // namespace absl
