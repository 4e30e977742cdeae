// Host entry points of the tcgen05 GEMM family (declared here, defined in gemm_*.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace pccl {
}  // namespace pccl
