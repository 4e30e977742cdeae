// Schedule loader: JSON schedule document -> concrete per-worker instruction streams.
//
// Engine::regOp(name, file) in the reference takes a file path and does nothing with it
// (csrc/engine.cc:102-104); the OperatorManager that was to parse it is an empty class
// (include/base/operator.h:40-45).  This is that parser.  A schedule is size-independent (offsets
// in units); materialize() binds it to a message size and to a worker budget:
//   * units -> bytes: a buffer is a sequence of blocks of `block_units` units, a block is exactly
//     `block_bytes` bytes, and unit j of a block is the j-th 16-byte-aligned slice of it;
//   * width w ("runtime resource control"): every channel stream is replicated w times and replica
//     j works on the j-th slice of each instruction's byte range with its own signal slots, so the
//     same schedule runs on w x channels workers (CTAs on the GPU, threads on the CPU).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../base/instr.h"
#include "../common/json.h"

namespace pccl {

struct RawInstr {
  uint32_t op;
  int32_t src_rank, dst_rank;
  uint32_t src_buf, dst_buf;
  int64_t src_off, dst_off, size;   // units
  uint32_t slot, value;
};

struct Materialized {
  std::vector<std::vector<Instr>> streams;   // one per worker
  uint64_t buf_bytes[BUF_COUNT] = {0, 0, 0};
  uint32_t num_slots = 0;                    // signal slots used (after widening)
  int width = 1;
  uint64_t bytes_moved = 0;                  // payload bytes this rank's COPY/REDUCE/MM ops touch
};

class Program {
 public:
  static Program fromJson(const Json& doc);
  static Program fromFile(const std::string& path) { return fromJson(Json::parseFile(path)); }

  // Streams of `rank` for blocks of `block_bytes` bytes, replicated `width` times.
  Materialized materialize(int rank, uint64_t block_bytes, int width) const;
  // block_bytes such that the input buffer is `input_bytes` long.
  uint64_t blockBytesForInput(uint64_t input_bytes) const;
  bool widenable() const { return widenable_; }

  std::string name, collective, redop;
  int world = 0, units = 0, block_units = 1, channels = 0;
  uint32_t num_slots = 0;
  bool in_place = false, needs_multicast = false, remote_io = false;
  int64_t buf_units[BUF_COUNT] = {0, 0, 0};
  std::vector<uint32_t> slot_counts;
  std::vector<std::vector<std::vector<RawInstr>>> streams;   // [rank][channel]

 private:
  bool widenable_ = true;
};

uint32_t parseRedOp(const std::string& s);
uint32_t parseDType(const std::string& s);
const char* dtypeName(uint32_t dt);

}  // namespace pccl
