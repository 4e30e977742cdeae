// Typed element-wise reductions on host memory (dst = dst (op) src), used by the CPU executor.
// (No counterpart in the reference: its CPU executor header is empty, include/plugins/cpu_executor/executor.h.)
#pragma once
#include <cstddef>
#include <cstdint>

namespace pccl {
// Returns false for an unsupported (dtype, op) pair.  `bytes` must be a multiple of the element size.
bool reduceInto(void* dst, const void* src, size_t bytes, uint32_t dtype, uint32_t redop);
float bf16ToFloat(uint16_t v);
uint16_t floatToBf16(float f);
float f16ToFloat(uint16_t v);
uint16_t floatToF16(float f);
float e4m3ToFloat(uint8_t v);
uint8_t floatToE4m3(float f);   // round-to-nearest-even, saturating to +-448
}  // namespace pccl
