#include "program.h"

#include <algorithm>
#include <stdexcept>

namespace pccl {

static inline uint64_t alignUp(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

uint32_t parseRedOp(const std::string& s) {
  if (s == "sum" || s == "add") return RED_SUM;
  if (s == "max") return RED_MAX;
  if (s == "min") return RED_MIN;
  if (s == "prod") return RED_PROD;
  throw std::runtime_error("unknown reduce op '" + s + "'");
}

uint32_t parseDType(const std::string& s) {
  if (s == "f32" || s == "float32" || s == "float") return DT_F32;
  if (s == "bf16" || s == "bfloat16") return DT_BF16;
  if (s == "f16" || s == "float16" || s == "half") return DT_F16;
  if (s == "f64" || s == "float64" || s == "double") return DT_F64;
  if (s == "i32" || s == "int32") return DT_I32;
  if (s == "i64" || s == "int64") return DT_I64;
  if (s == "u8" || s == "uint8" || s == "int8") return DT_U8;
  if (s == "fp8_e4m3" || s == "float8_e4m3fn" || s == "e4m3") return DT_FP8_E4M3;
  throw std::runtime_error("unknown dtype '" + s + "'");
}

const char* dtypeName(uint32_t dt) {
  static const char* n[] = {"f32", "bf16", "f16", "f64", "i32", "i64", "u8", "fp8_e4m3"};
  return dt < 8 ? n[dt] : "?";
}

Program Program::fromJson(const Json& doc) {
  if (!doc.isObject()) throw std::runtime_error("schedule: top level must be an object");
  Program p;
  p.name = doc["name"].asString();
  p.collective = doc["collective"].asString();
  p.redop = doc["redop"].isString() ? doc["redop"].asString() : "sum";
  p.world = static_cast<int>(doc["world_size"].asInt());
  p.units = static_cast<int>(doc["units"].asInt(1));
  p.in_place = doc["in_place"].asBool(false);
  const Json& attrs = doc["attrs"];
  p.block_units = static_cast<int>(attrs["block_units"].asInt(p.units));
  if (p.block_units <= 0) throw std::runtime_error("schedule: block_units must be positive");
  p.needs_multicast = attrs["requires"].asString() == "multicast";
  const Json& bufs = doc["buffers"];
  p.buf_units[BUF_INPUT] = bufs["input"].asInt(p.units);
  p.buf_units[BUF_OUTPUT] = bufs["output"].asInt(p.units);
  p.buf_units[BUF_SCRATCH] = bufs["scratch"].asInt(0);
  for (int b = 0; b < static_cast<int>(BUF_COUNT); ++b)
    if (p.buf_units[b] % p.block_units)
      throw std::runtime_error("schedule: buffer sizes must be multiples of block_units");
  const Json& low = doc["lowered"];
  if (!low.isObject()) throw std::runtime_error("schedule: missing 'lowered' section (run pccl.lang.to_schedule)");
  if (low["num_ranks"].asInt() != p.world) throw std::runtime_error("schedule: lowered rank count differs from world_size");
  p.channels = static_cast<int>(low["num_channels"].asInt());
  p.num_slots = static_cast<uint32_t>(low["num_slots"].asInt());
  for (auto& c : low["slot_counts"].items()) p.slot_counts.push_back(static_cast<uint32_t>(c.asInt()));
  if (p.slot_counts.size() != p.num_slots) throw std::runtime_error("schedule: slot_counts length mismatch");
  const Json& progs = low["programs"];
  if (static_cast<int>(progs.size()) != p.world) throw std::runtime_error("schedule: programs length mismatch");
  p.streams.resize(p.world);
  for (int r = 0; r < p.world; ++r) {
    const Json& chans = progs.at(r);
    if (static_cast<int>(chans.size()) != p.channels) throw std::runtime_error("schedule: channel count mismatch");
    p.streams[r].resize(p.channels);
    for (int c = 0; c < p.channels; ++c) {
      for (auto& ins : chans.at(c).items()) {
        if (ins.size() != 10) throw std::runtime_error("schedule: instruction must have 10 fields");
        RawInstr ri;
        ri.op = static_cast<uint32_t>(ins.at(0).asInt());
        ri.src_rank = static_cast<int32_t>(ins.at(1).asInt());
        ri.src_buf = static_cast<uint32_t>(ins.at(2).asInt());
        ri.src_off = ins.at(3).asInt();
        ri.dst_rank = static_cast<int32_t>(ins.at(4).asInt());
        ri.dst_buf = static_cast<uint32_t>(ins.at(5).asInt());
        ri.dst_off = ins.at(6).asInt();
        ri.size = ins.at(7).asInt();
        ri.slot = static_cast<uint32_t>(ins.at(8).asInt());
        ri.value = static_cast<uint32_t>(ins.at(9).asInt());
        if (ri.op >= OP_END) throw std::runtime_error("schedule: bad opcode");
        if (ri.src_rank < 0 || ri.src_rank >= p.world || ri.dst_rank < 0 || ri.dst_rank >= p.world)
          throw std::runtime_error("schedule: rank out of range");
        if (ri.src_buf >= BUF_COUNT || ri.dst_buf >= BUF_COUNT) throw std::runtime_error("schedule: bad buffer id");
        bool data = ri.op == OP_COPY || ri.op == OP_REDUCE || ri.op == OP_MM_LD_REDUCE || ri.op == OP_MM_ST;
        if (data) {
          if (ri.size <= 0 || ri.src_off < 0 || ri.dst_off < 0 ||
              ri.src_off + ri.size > p.buf_units[ri.src_buf] || ri.dst_off + ri.size > p.buf_units[ri.dst_buf])
            throw std::runtime_error("schedule: chunk outside its buffer");
          if (ri.size != 1) p.widenable_ = false;
          if ((ri.src_rank != r && ri.src_buf != BUF_SCRATCH) || (ri.dst_rank != r && ri.dst_buf != BUF_SCRATCH))
            p.remote_io = true;   // peers touch user tensors: they must live in the symmetric heap
        } else if (ri.op != OP_NOP) {
          if (ri.slot >= p.num_slots) throw std::runtime_error("schedule: signal slot out of range");
        }
        p.streams[r][c].push_back(ri);
      }
    }
  }
  return p;
}

uint64_t Program::blockBytesForInput(uint64_t input_bytes) const {
  uint64_t blocks = static_cast<uint64_t>(buf_units[BUF_INPUT] / block_units);
  if (blocks == 0 || input_bytes % blocks) throw std::runtime_error("exeOp: input size is not a whole number of blocks");
  return input_bytes / blocks;
}

Materialized Program::materialize(int rank, uint64_t bb, int width) const {
  if (rank < 0 || rank >= world) throw std::runtime_error("materialize: rank out of range");
  if (width < 1) width = 1;
  if (!widenable_) width = 1;
  Materialized m;
  m.width = width;
  m.num_slots = num_slots * width;
  const uint64_t bu = static_cast<uint64_t>(block_units);
  const uint64_t ub = alignUp((bb + bu - 1) / bu, 16);
  for (int b = 0; b < static_cast<int>(BUF_COUNT); ++b) m.buf_bytes[b] = static_cast<uint64_t>(buf_units[b]) / bu * bb;
  auto start = [&](int64_t u) { return (u / bu) * bb + std::min<uint64_t>((u % bu) * ub, bb); };
  auto stop = [&](int64_t last) { return (last / bu) * bb + std::min<uint64_t>((last % bu + 1) * ub, bb); };
  m.streams.resize(static_cast<size_t>(channels) * width);
  for (int c = 0; c < channels; ++c) {
    for (int j = 0; j < width; ++j) {
      auto& out = m.streams[static_cast<size_t>(c) * width + j];
      for (const RawInstr& ri : streams[rank][c]) {
        Instr in{};
        in.op = ri.op;
        in.src_rank = ri.src_rank;
        in.dst_rank = ri.dst_rank;
        in.src_buf = ri.src_buf;
        in.dst_buf = ri.dst_buf;
        bool data = ri.op == OP_COPY || ri.op == OP_REDUCE || ri.op == OP_MM_LD_REDUCE || ri.op == OP_MM_ST;
        if (data) {
          uint64_t s0 = start(ri.src_off), s1 = stop(ri.src_off + ri.size - 1);
          uint64_t d0 = start(ri.dst_off), d1 = stop(ri.dst_off + ri.size - 1);
          if (s1 - s0 != d1 - d0) throw std::runtime_error("materialize: source and target byte lengths differ");
          uint64_t len = s1 - s0;
          uint64_t sub = alignUp((len + width - 1) / width, 16);
          uint64_t lo = std::min<uint64_t>(static_cast<uint64_t>(j) * sub, len);
          uint64_t hi = std::min<uint64_t>(static_cast<uint64_t>(j + 1) * sub, len);
          in.src_off = s0 + lo;
          in.dst_off = d0 + lo;
          in.bytes = hi - lo;
          m.bytes_moved += in.bytes;
        } else if (ri.op != OP_NOP) {
          in.slot = ri.slot * width + j;
          in.value = ri.value;
          in.count = slot_counts[ri.slot];
        }
        out.push_back(in);
      }
      Instr end{};
      end.op = OP_END;
      out.push_back(end);
    }
  }
  return m;
}

}  // namespace pccl
