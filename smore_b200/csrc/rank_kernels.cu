// Filtered ranks of a query's answers among all candidates, without sorting the candidates.
//
// The reference evaluation (smore/training/train_process.py:113-146) scores one query against
// every entity, argsorts the N logits in descending order, turns the permutation into a rank per
// entity with a scatter, picks the ranks of the easy and hard answers, sorts those and subtracts
// the position in that small sorted list: rank(a) = 1 + #{entities ahead of a} - #{answers ahead
// of a}.  Only the answers' ranks are used, so the argsort over N is replaced by counting:
//   1. rank_sort_answers_kernel   per query: gather the answers' logits, sort the (few) answers
//                                 best first by (logit descending, entity id ascending);
//   2. rank_count_kernel          one pass over the N logits: binary search of each candidate in
//                                 the sorted answers gives the first answer it is ahead of; one
//                                 histogram increment (most candidates are ahead of none: one
//                                 comparison, no increment);
//   3. rank_finalize_kernel       prefix sum of the histogram = candidates ahead of each answer;
//                                 rank = ahead - position in the sorted answers + 1, written
//                                 back in the caller's answer order.
// "Ahead" is the order of a stable descending sort: higher logit first, lower entity id first
// among equal logits (torch.argsort leaves ties unspecified; this picks one of its outcomes).
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdint>

#include "common.cuh"
#include "rank_common.cuh"

namespace smore {

constexpr int kRankThreads = 256;
constexpr size_t kRankMaxAnswers = 8192;   // per query: sorted in shared memory

// one CTA per query; P = power of two >= the longest answer list
__global__ void __launch_bounds__(kRankThreads)
    rank_sort_answers_kernel(const float* __restrict__ logits, size_t n_candidates, int cols_are_positions,
                             const int64_t* __restrict__ answer_ptr, const int64_t* __restrict__ answer_ids,
                             int P, uint32_t* __restrict__ sorted_logit, int64_t* __restrict__ sorted_id,
                             int32_t* __restrict__ perm) {
  extern __shared__ unsigned char rank_smem[];
  uint32_t* key = reinterpret_cast<uint32_t*>(rank_smem);    // [P]
  int32_t* pos = reinterpret_cast<int32_t*>(key + P);        // [P] index into the query's answer list
  const size_t q = blockIdx.x;
  const int64_t begin = answer_ptr[q];
  const int A = (int)(answer_ptr[q + 1] - begin);
  const float* row = logits + q * n_candidates;
  for (int i = threadIdx.x; i < P; i += kRankThreads) {
    uint32_t k = 0;
    int32_t p = INT_MAX;
    if (i < A) {
      // the answer's logit sits in the column of its entity id, or (scores computed for the answers
      // alone, one column per listed answer) in the column of its position in the list
      const int64_t id = cols_are_positions ? begin + i : answer_ids[begin + i];
      k = (id >= 0 && (size_t)id < n_candidates) ? rank_key(row[id]) : 0u;
      p = i;
    }
    key[i] = k;
    pos[i] = p;
  }
  __syncthreads();
  // a sorts before b: higher logit, then lower entity id; padding (pos == INT_MAX) last
  auto before = [&](uint32_t ka, int32_t pa, uint32_t kb, int32_t pb) -> bool {
    if (pa == INT_MAX || pb == INT_MAX) return pb == INT_MAX && pa != INT_MAX;
    if (ka != kb) return ka > kb;
    const int64_t ia = answer_ids[begin + pa], ib = answer_ids[begin + pb];
    return ia != ib ? ia < ib : pa < pb;
  };
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < P; i += kRankThreads) {
        const int j = i ^ stride;
        if (j > i) {
          const bool up = (i & size) == 0;     // this pair sorts into "best first" order
          const uint32_t ki = key[i], kj = key[j];
          const int32_t pi = pos[i], pj = pos[j];
          const bool swap = up ? before(kj, pj, ki, pi) : before(ki, pi, kj, pj);
          if (swap) {
            key[i] = kj; key[j] = ki;
            pos[i] = pj; pos[j] = pi;
          }
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < A; i += kRankThreads) {
    sorted_logit[begin + i] = key[i];
    sorted_id[begin + i] = answer_ids[begin + pos[i]];
    perm[begin + i] = pos[i];
  }
}

// grid (chunks over the candidates, queries)
__global__ void __launch_bounds__(kRankThreads)
    rank_count_kernel(const float* __restrict__ logits, size_t n_candidates, const int64_t* __restrict__ answer_ptr,
                      const uint32_t* __restrict__ sorted_logit, const int64_t* __restrict__ sorted_id,
                      size_t per_cta, int32_t* __restrict__ hist) {
  extern __shared__ unsigned char rank_smem[];
  const size_t q = blockIdx.y;
  const int64_t begin = answer_ptr[q];
  const int A = (int)(answer_ptr[q + 1] - begin);
  if (A == 0) return;
  int64_t* ids = reinterpret_cast<int64_t*>(rank_smem);      // [A]
  uint32_t* thr = reinterpret_cast<uint32_t*>(ids + A);      // [A]
  int32_t* local = reinterpret_cast<int32_t*>(thr + A);      // [A]
  for (int i = threadIdx.x; i < A; i += kRankThreads) {
    ids[i] = sorted_id[begin + i];
    thr[i] = sorted_logit[begin + i];
    local[i] = 0;
  }
  __syncthreads();
  const uint32_t worst = thr[A - 1];
  const long long worst_id = ids[A - 1];
  const float* row = logits + q * n_candidates;
  const size_t c0 = (size_t)blockIdx.x * per_cta;
  const size_t c1 = c0 + per_cta < n_candidates ? c0 + per_cta : n_candidates;
  auto place = [&](float logit, size_t e) {
    const uint32_t x = rank_key(logit);
    if (!rank_ahead(x, (long long)e, worst, worst_id)) return;   // ahead of no answer (the usual case)
    int lo = 0, hi = A - 1;   // first answer this candidate is ahead of
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (rank_ahead(x, (long long)e, thr[mid], ids[mid])) hi = mid;
      else lo = mid + 1;
    }
    atomicAdd(&local[lo], 1);
  };
  // four independent, coalesced loads per thread and iteration
  size_t e = c0 + threadIdx.x;
  for (; e + 3 * kRankThreads < c1; e += 4 * kRankThreads) {
    const float x0 = row[e], x1 = row[e + kRankThreads], x2 = row[e + 2 * kRankThreads], x3 = row[e + 3 * kRankThreads];
    place(x0, e);
    place(x1, e + kRankThreads);
    place(x2, e + 2 * kRankThreads);
    place(x3, e + 3 * kRankThreads);
  }
  for (; e < c1; e += kRankThreads) place(row[e], e);
  __syncthreads();
  for (int i = threadIdx.x; i < A; i += kRankThreads)
    if (local[i]) atomicAdd(&hist[begin + i], local[i]);
}

// one CTA per query
__global__ void __launch_bounds__(kRankThreads)
    rank_finalize_kernel(const int64_t* __restrict__ answer_ptr, const int32_t* __restrict__ hist,
                         const int32_t* __restrict__ perm, int64_t* __restrict__ ranks) {
  __shared__ long long seg[kRankThreads];
  const size_t q = blockIdx.x;
  const int64_t begin = answer_ptr[q];
  const int A = (int)(answer_ptr[q + 1] - begin);
  const int per = (A + kRankThreads - 1) / kRankThreads;
  const int i0 = threadIdx.x * per, i1 = min(A, i0 + per);
  long long s = 0;
  for (int i = i0; i < i1; ++i) s += hist[begin + i];
  seg[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    long long run = 0;
    for (int t = 0; t < kRankThreads; ++t) {
      const long long v = seg[t];
      seg[t] = run;
      run += v;
    }
  }
  __syncthreads();
  long long ahead = seg[threadIdx.x];
  for (int i = i0; i < i1; ++i) {
    ahead += hist[begin + i];                        // candidates (answers included) ahead of sorted answer i
    ranks[begin + perm[begin + i]] = ahead - i + 1;  // i answers are ahead of it
  }
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

RankWorkspace carve_rank_workspace(void* workspace, size_t n_answers) {
  RankWorkspace w;
  unsigned char* p = static_cast<unsigned char*>(workspace);
  w.sorted_id = reinterpret_cast<int64_t*>(p);
  p += align_up(n_answers * sizeof(int64_t), 256);
  w.sorted_logit = reinterpret_cast<uint32_t*>(p);
  p += align_up(n_answers * sizeof(int32_t), 256);
  w.perm = reinterpret_cast<int32_t*>(p);
  p += align_up(n_answers * sizeof(int32_t), 256);
  w.hist = reinterpret_cast<int32_t*>(p);
  p += align_up(n_answers * sizeof(int32_t), 256);
  w.bytes = (size_t)(p - static_cast<unsigned char*>(workspace)) + 256;
  return w;
}

int rank_sort_answers(const float* logits, size_t n_cols, const int64_t* answer_ptr, const int64_t* answer_ids,
                      bool cols_are_positions, size_t n_queries, size_t n_answers, size_t max_answers,
                      const RankWorkspace& w, cudaStream_t st) {
  if (max_answers > kRankMaxAnswers)
    return fail(SMORE_ERR_TOO_LARGE, "filtered_ranks: at most %zu answers per query", kRankMaxAnswers);
  if (n_queries > 65535) return fail(SMORE_ERR_TOO_LARGE, "filtered_ranks: at most 65535 queries per call");
  if (cudaMemsetAsync(w.hist, 0, n_answers * sizeof(int32_t), st) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "filtered_ranks: cudaMemsetAsync failed");
  int P = 1;
  while ((size_t)P < max_answers) P <<= 1;
  if (int rc = allow_large_smem(rank_sort_answers_kernel, (int)(kRankMaxAnswers * 8), false)) return rc;
  rank_sort_answers_kernel<<<(unsigned)n_queries, kRankThreads, (size_t)P * 8, st>>>(
      logits, n_cols, cols_are_positions ? 1 : 0, answer_ptr, answer_ids, P, w.sorted_logit, w.sorted_id, w.perm);
  return check_launch("rank_sort_answers_kernel");
}

int rank_finalize(const int64_t* answer_ptr, const RankWorkspace& w, int64_t* ranks, size_t n_queries, cudaStream_t st) {
  rank_finalize_kernel<<<(unsigned)n_queries, kRankThreads, 0, st>>>(answer_ptr, w.hist, w.perm, ranks);
  return check_launch("rank_finalize_kernel");
}

}  // namespace smore

using namespace smore;

extern "C" {

size_t smore_filtered_ranks_workspace_bytes(size_t n_answers) { return carve_rank_workspace(nullptr, n_answers).bytes; }

int smore_filtered_ranks(const float* logits, size_t n_queries, size_t n_candidates, const int64_t* answer_ptr,
                         const int64_t* answer_ids, size_t n_answers, size_t max_answers, int64_t* ranks,
                         void* workspace, size_t workspace_bytes, void* stream) {
  if (n_queries == 0 || n_answers == 0) return SMORE_OK;
  if (!logits || !answer_ptr || !answer_ids || !ranks || !workspace)
    return fail(SMORE_ERR_NULL, "filtered_ranks: NULL pointer");
  if (n_candidates == 0 || max_answers == 0) return fail(SMORE_ERR_BAD_SHAPE, "filtered_ranks: empty candidate set");
  if (n_candidates > ((size_t)1 << 40)) return fail(SMORE_ERR_TOO_LARGE, "filtered_ranks: too many candidates");
  if (workspace_bytes < smore_filtered_ranks_workspace_bytes(n_answers) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(SMORE_ERR_WORKSPACE, "filtered_ranks: workspace too small or not 256-byte aligned");
  const RankWorkspace w = carve_rank_workspace(workspace, n_answers);
  cudaStream_t st = (cudaStream_t)stream;
  if (int rc = rank_sort_answers(logits, n_candidates, answer_ptr, answer_ids, false, n_queries, n_answers, max_answers,
                                 w, st))
    return rc;
  const size_t count_smem = max_answers * 16;
  if (int rc = allow_large_smem(rank_count_kernel, (int)(kRankMaxAnswers * 16), false)) return rc;
  // enough CTAs per query to fill the GPU a few times over, at least 4096 candidates each
  size_t chunks = std::max<size_t>(1, (size_t)sm_count() * 8 / n_queries);
  size_t per_cta = std::max<size_t>(4096, (n_candidates + chunks - 1) / chunks);
  chunks = (n_candidates + per_cta - 1) / per_cta;
  dim3 grid((unsigned)chunks, (unsigned)n_queries);
  rank_count_kernel<<<grid, kRankThreads, count_smem, st>>>(logits, n_candidates, answer_ptr, w.sorted_logit,
                                                            w.sorted_id, per_cta, w.hist);
  if (int rc = check_launch("rank_count_kernel")) return rc;
  return rank_finalize(answer_ptr, w, ranks, n_queries, st);
}

}  // extern "C"
