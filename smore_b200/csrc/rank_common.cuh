// Pieces of the filtered-rank computation shared by rank_kernels.cu (ranks from a logits matrix) and
// dist_kernels.cu (ranks straight from the scoring tiles, without a logits matrix).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace smore {

// Logits are compared through an order-preserving integer key: the order of torch.sort, in which
// NaN is the largest value, -0 equals +0, and everything else is the usual float order.
__device__ __forceinline__ uint32_t rank_key(float x) {
  if (x != x) return 0xFFFFFFFFu;
  const uint32_t b = __float_as_uint(x + 0.f);   // -0 + 0 = +0
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// candidate (key x, entity e) is ahead of answer (key t, entity id): the order of a stable descending sort
__device__ __forceinline__ bool rank_ahead(uint32_t x, long long e, uint32_t t, long long id) {
  return x > t || (x == t && e < id);
}

struct RankWorkspace {
  int64_t* sorted_id;       // [n_answers] entity ids, per query best first
  uint32_t* sorted_logit;   // [n_answers] their keys
  int32_t* perm;            // [n_answers] position in the caller's answer list
  int32_t* hist;            // [n_answers] candidates whose first answer behind them is this one
  size_t bytes;
};

RankWorkspace carve_rank_workspace(void* workspace, size_t n_answers);

// Per query: sort the answers best first (keys from logits[q, col], col = the answer's entity id, or
// its position in answer_ids when cols_are_positions) and clear the histogram.
int rank_sort_answers(const float* logits, size_t n_cols, const int64_t* answer_ptr, const int64_t* answer_ids,
                      bool cols_are_positions, size_t n_queries, size_t n_answers, size_t max_answers,
                      const RankWorkspace& w, cudaStream_t st);

// ranks[p] = candidates ahead of answer p - answers ahead of it + 1, in the caller's answer order
int rank_finalize(const int64_t* answer_ptr, const RankWorkspace& w, int64_t* ranks, size_t n_queries, cudaStream_t st);

}  // namespace smore
