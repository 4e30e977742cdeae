#include "hex.h"

namespace pccl {

std::string encodeHex(const void* data, size_t n) {
  static const char digits[] = "0123456789abcdef";
  const unsigned char* p = static_cast<const unsigned char*>(data);
  std::string s(n * 2, '0');
  for (size_t i = 0; i < n; ++i) {
    s[2 * i] = digits[p[i] >> 4];
    s[2 * i + 1] = digits[p[i] & 15];
  }
  return s;
}

static inline int nibble(char c) {
  if (c >= '0' && c <= '9') return c - '0';
  if (c >= 'a' && c <= 'f') return c - 'a' + 10;
  if (c >= 'A' && c <= 'F') return c - 'A' + 10;
  return -1;
}

bool decodeHex(void* out, size_t n, const std::string& text) {
  if (text.size() != 2 * n) return false;
  unsigned char* p = static_cast<unsigned char*>(out);
  for (size_t i = 0; i < n; ++i) {
    int hi = nibble(text[2 * i]), lo = nibble(text[2 * i + 1]);
    if (hi < 0 || lo < 0) return false;
    p[i] = static_cast<unsigned char>((hi << 4) | lo);
  }
  return true;
}

std::string decodeHexToString(const std::string& text, bool* ok) {
  std::string out(text.size() / 2, '\0');
  bool good = decodeHex(out.data(), out.size(), text);
  if (ok) *ok = good;
  return good ? out : std::string();
}

}  // namespace pccl
