// 64-bit FNV-1a (the reference's hash, csrc/common/hash.cc:3-15) — used here for schedule-cache
// keys and topology fingerprints.
#pragma once
#include <cstdint>
#include <string_view>

namespace pccl {
constexpr uint64_t kFnvOffset = 14695981039346656037ull;
constexpr uint64_t kFnvPrime = 1099511628211ull;
constexpr uint64_t fnv1a(std::string_view s, uint64_t h = kFnvOffset) {
  for (char c : s) {
    h ^= static_cast<unsigned char>(c);
    h *= kFnvPrime;
  }
  return h;
}
}  // namespace pccl
