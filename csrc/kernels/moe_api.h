// Host entry points of the expert-parallel MoE kernels (moe.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "api.h"

namespace pccl {

struct MoeArgs {
  World w;
  int nvirt;              // 1, or the emulated world size (single-GPU tests)
  int rank;               // ignored when nvirt > 1
  int tokens;             // tokens of this rank
  int hidden;             // multiple of 128
  int topk;               // <= 8
  int experts_per_rank;
  uint64_t recv_q_off;    // heap offset: fp8 rows received [cap, hidden]
  uint64_t recv_s_off;    // heap offset: fp32 scales received [cap, hidden/128]
  uint64_t y_off;         // heap offset: expert outputs [cap, hidden] bf16 (read by the combine of every rank)
  uint64_t epoch;
  int flag_lane;
  int dedupe;             // 1: an assignment whose rank already receives this token through an earlier k is not sent again
  uint64_t spin_ns;
  // De-duplicated exchange (dedupe = 1; needs the three areas below in the symmetric heap, 0 = feature off).  The FIRST of a
  // token's assignments that goes to a rank is its primary on that rank; the others are told where the payload is.
  uint64_t alias_off;     // int32 [cap]: row that holds the fp8 payload of row r (r itself for a primary)
  uint64_t group_off;     // [cap] x {int32 rows[8], float weight[8]}: for a primary row, the rows of the same token on this
                          // rank (-1 padded) with their gate weights; written by the dispatch, read by the group reduction
  uint64_t z_off;         // bf16 [cap, hidden]: sum over a group of weight x expert output, for groups of two or more
  // per (virtual) rank local tensors
  const void* x[kMaxRanks];          // [tokens, hidden] bf16
  const int* expert_ids[kMaxRanks];  // [tokens, topk] global expert ids
  const int* dst_rows[kMaxRanks];    // [tokens, topk] row inside the destination rank's receive buffer
  const float* probs[kMaxRanks];     // [tokens, topk] gate probabilities (combine); dispatch: scale per destination
  const float* gate[kMaxRanks];      // [tokens, topk] gate probabilities for the group records of a de-duplicating dispatch
  void* out[kMaxRanks];              // [tokens, hidden] bf16 (combine)
  uint32_t* status[kMaxRanks];
};

// fp8 (e4m3, one fp32 scale per 128 values) quantisation fused with the push to the experts' ranks.  With `probs` set,
// destination k of token t receives probs[t,k] * x[t] (the backward pass sends gate-weighted output gradients this way).
int launchMoeDispatch(const MoeArgs& a, int blocks, cudaStream_t stream);
// out (fp32 [tokens, topk]) = <x[t], y[rank of expert (t,k)][dst_rows[t,k]]>: gradients of the gate weights.
int launchMoeCombineDot(const MoeArgs& a, int blocks, cudaStream_t stream);
// out[t] = sum_k probs[t,k] * y[rank of expert (t,k)][dst_rows[t,k]]: pulls the rows over NVLink.
int launchMoeCombine(const MoeArgs& a, int blocks, cudaStream_t stream);
// bf16 rows from fp8 rows + scales, for rows [0, *n_rows) (device count).  `alias` (or null): row r is read from alias[r].
int launchMoeDequant(const void* q, const float* scales, void* out, const int* n_rows, int max_rows, int hidden, const int* alias,
                     cudaStream_t stream);
// z[r] = sum over the group of primary row r of weight x y[row], for groups of two or more rows (local; after the experts).
int launchMoeReduceGroups(const void* y, void* z, const int* alias, const void* groups, const int* n_rows, int max_rows, int hidden,
                          cudaStream_t stream);
// Stand-alone block quantiser (1 x 128 blocks, e4m3 + fp32 scales).
int launchQuantFp8Rows(const void* x, void* q, float* scales, long long rows, int hidden, cudaStream_t stream);
// 128 x 128 block quantiser for weights [rows, cols] (both multiples of 128): e4m3 + fp32 scale per block.
int launchQuantFp8Blocks(const void* w, void* q, float* scales, int rows, int cols, cudaStream_t stream);

// Routing: softmax over `experts` gate logits (fp32 [tokens, experts], experts <= 1024), top-k by
// probability; writes ids / probs [tokens, k] and pos[tokens, k] = the assignment's arrival number among this
// rank's assignments to the same expert (counts[experts] must be zero on entry and holds the totals afterwards).
int launchMoeRoute(const float* logits, int* ids, float* probs, int* pos, int* counts, int tokens, int experts, int topk,
                   cudaStream_t stream);
// Placement: from the counts of all ranks ([world, experts]) compute, for every assignment, its row in the receive
// buffer of the expert's rank (-1 when the buffer of `cap` rows is full), and for this rank row_off[experts_per_rank+1].
int launchMoePlan(const int* counts_all, const int* ids, const int* pos, int* rows, int* row_off, int world, int rank, int experts,
                  int tokens, int topk, int cap, cudaStream_t stream);

}  // namespace pccl
