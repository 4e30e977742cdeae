// Instruction format shared by the host loader, the CPU executor and the GPU interpreter kernel.
//
// This is the flattened, device-readable twin of the reference's operator-graph layout
// (include/base/operator.h:19-38: OperationLayoutHeader with dependency counters, next-op lists and
// ready queues).  Dependencies were already turned into program order plus counting signals by the
// lowering pass, so an executor worker just walks its stream front to back.
#pragma once
#include <cstdint>

namespace pccl {

enum Opcode : uint32_t {
  OP_NOP = 0, OP_COPY = 1, OP_REDUCE = 2, OP_NOTIFY = 3, OP_WAIT = 4,
  OP_MM_LD_REDUCE = 5, OP_MM_ST = 6, OP_BARRIER = 7, OP_END = 8
};

enum BufId : uint32_t { BUF_INPUT = 0, BUF_OUTPUT = 1, BUF_SCRATCH = 2, BUF_COUNT = 3 };

enum DType : uint32_t {
  DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2, DT_F64 = 3, DT_I32 = 4, DT_I64 = 5, DT_U8 = 6, DT_FP8_E4M3 = 7
};

enum RedOp : uint32_t { RED_SUM = 0, RED_MAX = 1, RED_MIN = 2, RED_PROD = 3 };

inline uint32_t dtypeSize(uint32_t dt) {
  switch (dt) {
    case DT_F32: case DT_I32: return 4;
    case DT_BF16: case DT_F16: return 2;
    case DT_F64: case DT_I64: return 8;
    default: return 1;
  }
}

// 64 bytes, 16-byte aligned so that a warp can fetch an instruction with four 16-byte loads.
struct alignas(16) Instr {
  uint32_t op;
  int32_t src_rank;
  int32_t dst_rank;
  uint32_t src_buf;
  uint32_t dst_buf;
  uint32_t slot;       // signal slot (index into the executing/target rank's signal array)
  uint32_t value;      // ordinal of this notify/wait/barrier within one launch (1-based)
  uint32_t count;      // notifies (or barriers) on `slot` per launch
  uint64_t src_off;    // bytes
  uint64_t dst_off;    // bytes
  uint64_t bytes;
  uint64_t reserved;
};
static_assert(sizeof(Instr) == 64, "Instr must be 64 bytes");

// Status codes written by executors (0 = success).
enum ExecStatus : uint32_t {
  ST_OK = 0,
  ST_TIMEOUT = 1,        // a bounded wait ran out
  ST_BOUNDS = 2,         // an instruction named memory outside its buffer
  ST_BAD_OP = 3,
  ST_UNSUPPORTED = 4,    // e.g. multimem op without a multicast mapping
  ST_PEER_GONE = 5,
};

}  // namespace pccl
