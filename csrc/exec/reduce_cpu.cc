#include "reduce_cpu.h"

#include <algorithm>
#include <cmath>
#include <cstring>

#include "../base/instr.h"

namespace pccl {

float bf16ToFloat(uint16_t v) {
  uint32_t u = static_cast<uint32_t>(v) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

uint16_t floatToBf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);   // NaN
  u += 0x7fffu + ((u >> 16) & 1u);   // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}

float f16ToFloat(uint16_t h) {
  uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      u = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
  else u = sign | ((exp + 112) << 23) | (man << 13);
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

uint16_t floatToF16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    uint32_t shift = static_cast<uint32_t>(14 - exp);
    uint32_t half = man >> shift, rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(exp) << 10) | (man >> 13), rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

float e4m3ToFloat(uint8_t v) {
  uint32_t sign = v >> 7, exp = (v >> 3) & 0xf, man = v & 7;
  float out;
  if (exp == 0xf && man == 7) out = NAN;
  else if (exp == 0) out = std::ldexp(static_cast<float>(man), -9);
  else out = std::ldexp(1.0f + man / 8.0f, static_cast<int>(exp) - 7);
  return sign ? -out : out;
}

uint8_t floatToE4m3(float f) {
  if (std::isnan(f)) return 0x7f;
  uint8_t sign = std::signbit(f) ? 0x80 : 0;
  float a = std::fabs(f);
  if (a >= 448.0f) return sign | 0x7e;
  if (a < std::ldexp(1.0f, -10)) return sign;   // below half the smallest subnormal
  int e;
  float m = std::frexp(a, &e);   // a = m * 2^e, m in [0.5,1)
  int exp = e - 1 + 7;
  float q;
  if (exp <= 0) {   // subnormal: units of 2^-9
    q = std::nearbyint(std::ldexp(a, 9));
    if (q >= 8) return sign | 0x08;
    return sign | static_cast<uint8_t>(q);
  }
  q = std::nearbyint((m * 2.0f - 1.0f) * 8.0f);
  if (q >= 8) { q = 0; ++exp; }
  if (exp > 15 || (exp == 15 && q > 6)) return sign | 0x7e;
  return sign | static_cast<uint8_t>((exp << 3) | static_cast<int>(q));
}

namespace {
template <typename T>
inline T apply(T a, T b, uint32_t op) {
  switch (op) {
    case RED_SUM: return a + b;
    case RED_MAX: return std::max(a, b);
    case RED_MIN: return std::min(a, b);
    default: return a * b;
  }
}
template <typename T>
void reduceTyped(T* d, const T* s, size_t n, uint32_t op) {
  switch (op) {
    case RED_SUM: for (size_t i = 0; i < n; ++i) d[i] = d[i] + s[i]; break;
    case RED_MAX: for (size_t i = 0; i < n; ++i) d[i] = std::max(d[i], s[i]); break;
    case RED_MIN: for (size_t i = 0; i < n; ++i) d[i] = std::min(d[i], s[i]); break;
    default: for (size_t i = 0; i < n; ++i) d[i] = d[i] * s[i];
  }
}
}  // namespace

bool reduceInto(void* dst, const void* src, size_t bytes, uint32_t dtype, uint32_t op) {
  if (op > RED_PROD) return false;
  switch (dtype) {
    case DT_F32: reduceTyped(static_cast<float*>(dst), static_cast<const float*>(src), bytes / 4, op); return true;
    case DT_F64: reduceTyped(static_cast<double*>(dst), static_cast<const double*>(src), bytes / 8, op); return true;
    case DT_I32: reduceTyped(static_cast<int32_t*>(dst), static_cast<const int32_t*>(src), bytes / 4, op); return true;
    case DT_I64: reduceTyped(static_cast<int64_t*>(dst), static_cast<const int64_t*>(src), bytes / 8, op); return true;
    case DT_U8: reduceTyped(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), bytes, op); return true;
    case DT_BF16: {
      uint16_t* d = static_cast<uint16_t*>(dst);
      const uint16_t* s = static_cast<const uint16_t*>(src);
      for (size_t i = 0; i < bytes / 2; ++i) d[i] = floatToBf16(apply(bf16ToFloat(d[i]), bf16ToFloat(s[i]), op));
      return true;
    }
    case DT_F16: {
      uint16_t* d = static_cast<uint16_t*>(dst);
      const uint16_t* s = static_cast<const uint16_t*>(src);
      for (size_t i = 0; i < bytes / 2; ++i) d[i] = floatToF16(apply(f16ToFloat(d[i]), f16ToFloat(s[i]), op));
      return true;
    }
    case DT_FP8_E4M3: {
      uint8_t* d = static_cast<uint8_t*>(dst);
      const uint8_t* s = static_cast<const uint8_t*>(src);
      for (size_t i = 0; i < bytes; ++i) d[i] = floatToE4m3(apply(e4m3ToFloat(d[i]), e4m3ToFloat(s[i]), op));
      return true;
    }
    default: return false;
  }
}

}  // namespace pccl
