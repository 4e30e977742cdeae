// Host helper that builds TMA descriptors (cuTensorMapEncodeTiled, resolved through the runtime so
// that nothing links against libcuda).  Tile mode, 128-byte swizzle, zero fill out of bounds.
#pragma once
#include <cuda.h>

#include <cstdint>
#include <string>

namespace pccl {

enum TmDType { TM_BF16 = 0, TM_U8 = 1, TM_F32 = 2 };

// 2-D tensor: `inner` elements contiguous, `outer` rows `row_stride` elements apart; the box is
// box_inner x box_outer elements (box_inner * element size must be 128 bytes for the swizzle).
bool makeTensorMap2D(CUtensorMap* out, const void* base, TmDType dt, uint64_t inner, uint64_t outer, uint64_t row_stride,
                     uint32_t box_inner, uint32_t box_outer, std::string* err);

}  // namespace pccl
