// Host-callable entry points of the sm_100a kernels.  Plain C++ types only (no torch headers):
// (The reference ships no kernel: its only device code is three inline-PTX multimem helpers,
// include/plugins/cuda_executor/utils/multimem.h:12-127, and register-packing types, vector_datatype.h:21-80.)
// the Python layer passes raw device pointers and the CUDA stream handle.
//
// Multi-rank convention.  Every communication kernel takes a `World`: the table of all ranks'
// symmetric-heap base addresses as mapped into THIS process, the multicast address of the heap
// (or null), and the offset of the signal area.  In production one process drives one GPU and
// launches the kernel for its own rank (`nvirt == 1`).  For single-GPU tests the same kernel is
// launched once, cooperatively, with `nvirt == world` and blockIdx.y selecting the rank whose
// part a block plays, all "heaps" being buffers of that one GPU (ranks that wait on one another
// must never be separate launches on one GPU).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../base/instr.h"

namespace pccl {

constexpr int kMaxRanks = 16;
constexpr int kMaxBlocksPerColl = 160;        // flag rows reserved per collective "lane"
constexpr uint64_t kDefaultSpinLimit = 2000ull * 1000 * 1000;   // nanoseconds a device-side wait may last

struct World {
  int world;
  int pad;
  char* heap[kMaxRanks];     // heap[r] = rank r's symmetric heap, addressable from the launching GPU
  char* mc_heap;             // multicast (NVLS) address of the heap, or nullptr
  uint64_t signal_off;       // byte offset of the uint64 signal words inside every heap
  uint64_t flag_off;         // byte offset of the per-block barrier flags inside every heap
};

// ---------------------------------------------------------------------------------------------
// K6: persistent interpreter of lowered collective programs
// ---------------------------------------------------------------------------------------------
struct InterpRank {
  int rank;
  int n_streams;
  const Instr* instrs;            // all streams of this rank, back to back
  const uint32_t* stream_start;   // n_streams entries: index of each stream's first instruction
  char* input;
  char* output;
  long long input_heap_off;       // >= 0 when the tensor lives in the symmetric heap (peers may touch it)
  long long output_heap_off;
  uint64_t scratch_off;           // offset of this launch's scratch lane inside the heap
  uint64_t buf_bytes[BUF_COUNT];
  uint32_t* status;               // [0]=status code, [1]=stream, [2]=pc, [3]=detail
  uint64_t* trace;                // nullptr, or two words per instruction of this rank (indexed like `instrs`):
                                  // %globaltimer when the CTA began it and when all its threads had finished it
};

constexpr uint32_t kNoTurnSlot = 0xffffffffu;
// The interpreter reads instructions a chunk of this many at a time; the array that InterpRank::instrs points to must
// be followed by that many readable (no-op) instructions.
constexpr uint32_t kInstrPad = 32;

struct InterpLaunch {
  World w;
  int nvirt;                      // 1, or world for single-GPU emulation
  uint32_t slot_base;
  uint64_t epoch;
  // Workspace turn-taking.  Launches on one workspace lane alternate between the lane's two scratch halves, so
  // launch n reuses the half of launch n - 2.  Programs differ in which ranks they tie together, so a rank may
  // run ahead of a peer across a program that does not involve both.  Every rank therefore publishes "I have
  // finished n launches on this lane" to all peers when its last stream ends, and before a launch touches any
  // scratch it waits until every peer has finished launch n - 2.  Words turn_slot + r (absolute signal indices)
  // count rank r's finished launches; finish_slot counts this rank's streams that have ended (wraps to zero).
  // kNoTurnSlot switches the protocol off (single-launch emulation).
  uint32_t turn_slot = kNoTurnSlot;
  uint32_t finish_slot = 0;
  uint64_t launch_no = 0;         // 0-based launch number on the lane
  uint32_t dtype, redop;
  uint64_t spin_limit;
  int bounds_check;
  InterpRank r[kMaxRanks];
};

// grid = (max n_streams, nvirt); cooperative launch.  Returns a cudaError_t as int.
int launchInterpreter(const InterpLaunch& L, int threads, cudaStream_t stream);
// Foldings of COPY instructions in the interpreter kernel (bit 0: copy + reduces, bit 1: one source, many destinations); default 3.
int setInterpreterFusion(int mask);
// ---- resident interpreter: launches queued by the host, taken by a kernel that stays on the GPU ----------------------
struct alignas(16) ResidentDesc { // what InterpLaunch carries, for this rank only; copied with 16-byte vector loads
  World w;
  InterpRank r;
  uint64_t epoch;
  uint64_t spin_limit;
  uint64_t launch_no;
  uint32_t slot_base;
  uint32_t dtype, redop;
  int bounds_check;
  uint32_t turn_slot, finish_slot;
  uint64_t pad;
};
static_assert(sizeof(ResidentDesc) % 16 == 0, "ResidentDesc is copied in 16-byte vectors");
constexpr uint32_t kResidentSlots = 64;
constexpr int kResidentChannels = 4;        // the resident grid holds width x this many CTAs (streams = channels x width)
struct ResidentQueue {           // pinned, mapped host memory: written by the host, polled by the kernel
  volatile uint64_t tail;        // host: descriptors published so far
  volatile uint64_t completed;   // device: descriptors finished so far
  volatile uint32_t stop;        // host: leave now
  volatile uint32_t running;     // host sets 1 before a launch, the kernel clears it when it leaves
  uint64_t idle_ns;              // leave after this long without work
  uint64_t pad[4];               // the descriptors start on a 16-byte boundary (offset 64)
  ResidentDesc slots[kResidentSlots];
};
static_assert(offsetof(ResidentQueue, slots) % 16 == 0, "queued descriptors are read with 16-byte vector loads");
struct ResidentCtl {             // device memory: CTA 0's decision and the descriptor for the other CTAs
  uint32_t run;
  uint32_t pad[3];
  ResidentDesc desc;
};
static_assert(offsetof(ResidentCtl, desc) % 16 == 0, "the descriptor copy is written with 16-byte vector stores");
// Cooperative launch of `ctas` CTAs that serve the queue from descriptor `head` on.
int launchResident(ResidentQueue* queue_device_view, ResidentCtl* ctl, uint64_t head, int ctas, int threads, cudaStream_t stream);

// dst = dst (redop) src over `bytes` of device memory: the REDUCE instruction as a kernel of its own, for the
// host-driven executor of engines whose peers are partly reached over the network.
int launchDeviceReduce(void* dst, const void* src, uint64_t bytes, uint32_t dtype, uint32_t redop, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// K1-K4, K10: hand-written collectives over the symmetric heap (offsets are heap-relative)
// ---------------------------------------------------------------------------------------------
enum CollAlgo : int { ALGO_P2P = 0, ALGO_NVLS = 1 };

struct CollArgs {
  World w;
  int nvirt;                 // 1 or world (emulation)
  int rank;                  // ignored when nvirt > 1
  int algo;                  // CollAlgo
  uint32_t dtype, redop;
  uint64_t in_off;           // heap offset of the input (symmetric)
  uint64_t out_off;          // heap offset of the output (symmetric)
  uint64_t count;            // elements: AR total, RS/AG per-shard, A2A per-block
  uint64_t epoch;            // strictly increasing per launch on a given flag lane
  int flag_lane;             // which flag rows this launch uses (concurrent launches use distinct lanes)
  float scale;               // RS epilogue: out = reduce(in) * scale
  uint32_t out_dtype;        // RS epilogue cast (DT_F32 or same as dtype)
  uint64_t spin_limit;
  uint32_t* status[kMaxRanks];   // per virtual rank status words (4 x u32)
  // Optional plain (non-symmetric) local tensors, per virtual rank: the all-gather / all-to-all
  // input and the reduce-scatter output are only touched by their own rank.
  const void* local_in[kMaxRanks];
  void* local_out[kMaxRanks];
  // block-scaled fp8 collectives only: heap offsets of the fp32 scales (one per 128 values) of input and output
  uint64_t s_in_off, s_out_off;
  // Heap offset of the low-latency receive area of this flag lane (kLlLaneBytes: two epochs x kMaxRanks sources x
  // kLlSlotBytes), or 0 when the heap has none.  All-reduces of at most kLlMaxBytes then take the flag-in-data path.
  uint64_t ll_off;
};

// Low-latency all-reduce: every rank stores each 4-byte word of its input into every peer's receive slot as an 8-byte
// packet {word, launch number} -- the flag travels with the data in one store, so there is no barrier before or after --
// and reduces its own slots as the packets arrive.  Two receive areas alternate by launch parity.
constexpr uint64_t kLlMaxBytes = 64ull << 10;
constexpr uint64_t kLlSlotBytes = 2 * kLlMaxBytes;
constexpr uint64_t kLlLaneBytes = 2ull * kMaxRanks * kLlSlotBytes;
constexpr int kLlLanes = 4;

int launchAllReduce(const CollArgs& a, int blocks, int threads, cudaStream_t stream);
int launchReduceScatter(const CollArgs& a, int blocks, int threads, cudaStream_t stream);
// Reduce-scatter of a bf16 gradient bucket fused with the sharded AdamW step: this rank's slice is
// summed over the ranks (fp32), scaled, and consumed at once by the optimizer update of the fp32
// master weights / moments; the new parameters are written as bf16.  No gradient shard is ever stored.
struct AdamArgs {
  float* p; float* m; float* v;   // fp32 shard state, `count` elements
  void* p_bf16;                   // bf16 parameters of the shard (output)
  float lr, b1, b2, eps, wd, inv_bc1, inv_sqrt_bc2;
};
int launchReduceScatterAdamW(const CollArgs& a, const AdamArgs& o, int blocks, int threads, cudaStream_t stream);
// Block-scaled fp8 (e4m3 payload + one fp32 scale per 128 values) all-reduce and reduce-scatter: every 128-value block is
// dequantised, accumulated in fp32 over the ranks and re-quantised with a fresh scale (block maximum / 448), all inside
// the transfer.  `count` = elements (AR: whole vector; RS: per shard), a multiple of 128.  Sum or max.  P2P only.
int launchAllReduceFp8(const CollArgs& a, int blocks, int threads, cudaStream_t stream);
int launchReduceScatterFp8(const CollArgs& a, int blocks, int threads, cudaStream_t stream);
int launchAllGather(const CollArgs& a, int blocks, int threads, cudaStream_t stream);
int launchAllToAll(const CollArgs& a, int blocks, int threads, cudaStream_t stream);
// Bounded-wait self test: waits on a flag nobody sets; must come back with ST_TIMEOUT.
int launchWaitTimeoutProbe(uint64_t* flag, uint64_t spin_limit, uint32_t* status, cudaStream_t stream);

int deviceSmCount();
const char* cudaErrorName(int err);

}  // namespace pccl
