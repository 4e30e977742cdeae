// Binary <-> lower-case hex text.  Same job as the reference's serialize/deserialize
// (include/common/serialize.h:6-7): opaque handles (memory handles, socket addresses) travel
// inside JSON endpoint documents as hex.  decodeHex() reports malformed input instead of
// writing garbage.
#pragma once
#include <cstddef>
#include <string>

namespace pccl {
std::string encodeHex(const void* data, size_t n);
// Returns false if `text` has odd length, a non-hex digit, or does not hold exactly n bytes.
bool decodeHex(void* out, size_t n, const std::string& text);
std::string decodeHexToString(const std::string& text, bool* ok = nullptr);
}  // namespace pccl
