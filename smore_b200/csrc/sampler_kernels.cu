// Negative sampling on the GPU: the step before the row gathers.
//
// The reference's online sampler draws, for every query, `negative_sample_size` entity ids that are
// not answers of the query - uniformly, or with degree-proportional weights through an alias table
// (smore/cpp_sampler/src/lib/naive_sampler.cpp:28-50, alias_method.cpp:33-99, sampler.cpp:90-99 for
// one shared list per batch) - on host threads, with a std::mt19937 per thread seeded from the clock
// (utils.cpp:33-39), so its draws are not reproducible.  Here one thread draws one id with a
// counter-based generator (Philox 4x32-10 keyed by a seed, counted by step and position): the same
// (seed, offset) gives the same ids on every run and any number of GPUs can draw disjoint streams.
// The alias table is built on the host by the reference's procedure (two first-in-first-out work
// lists), so the tables - and with them the distribution - are identical to the reference's.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <deque>
#include <vector>

#include "common.cuh"

namespace smore {

struct Philox {
  uint32_t c[4];
};

__device__ __forceinline__ Philox philox4x32_10(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, uint32_t c2,
                                                uint32_t c3) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0;
    k1 += W1;
  }
  return Philox{{c0, c1, c2, c3}};
}

// 53 random bits -> [0, 1)
__device__ __forceinline__ double unit_double(uint32_t hi, uint32_t lo) {
  const unsigned long long x = (((unsigned long long)hi << 32) | lo) >> 11;
  return (double)x * (1.0 / 9007199254740992.0);
}

struct SampleArgs {
  unsigned long long seed, offset;
  unsigned long long n_entities;
  const double* prob_small;      // nullable trio: uniform draws
  const int64_t* choice_small;
  const int64_t* choice_large;
  const int64_t* answer_ptr;     // nullable pair: nothing is rejected
  const int64_t* answer_ids;     // per query ascending
  size_t n_queries, k;
};

constexpr int kMaxDraws = 64;     // redraws of one position before the last draw is kept

__global__ void __launch_bounds__(256) sample_negatives_kernel(SampleArgs a, int64_t* __restrict__ out) {
  const size_t total = a.n_queries * a.k;
  for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += (size_t)gridDim.x * blockDim.x) {
    const size_t b = p / a.k;
    const int64_t* ans = nullptr;
    long long n_ans = 0;
    if (a.answer_ptr != nullptr) {
      ans = a.answer_ids + a.answer_ptr[b];
      n_ans = a.answer_ptr[b + 1] - a.answer_ptr[b];
    }
    const unsigned long long ctr = a.offset + p;
    long long id = 0;
    for (int attempt = 0; attempt < kMaxDraws; ++attempt) {
      const Philox r = philox4x32_10((uint32_t)a.seed, (uint32_t)(a.seed >> 32), (uint32_t)ctr, (uint32_t)(ctr >> 32),
                                     (uint32_t)attempt, 0x534d4f52u);
      // alias_method.cpp:41-52: slot = floor(n * u1), then the small or the large choice of the slot
      unsigned long long slot = (unsigned long long)((double)a.n_entities * unit_double(r.c[0], r.c[1]));
      if (slot >= a.n_entities) slot = a.n_entities - 1;
      if (a.prob_small != nullptr)
        id = unit_double(r.c[2], r.c[3]) < a.prob_small[slot] ? a.choice_small[slot] : a.choice_large[slot];
      else
        id = (long long)slot;
      // naive_sampler.cpp:40-46: draw again while the id is one of the query's answers
      long long lo = 0, hi = n_ans;
      while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if (ans[mid] < id) lo = mid + 1; else hi = mid;
      }
      if (!(lo < n_ans && ans[lo] == id)) break;
    }
    out[p] = id;
  }
}

// shared negatives: is_negative[b, j] = 0 where negatives[j] is an answer of query b (naive_sampler.cpp:33-38)
__global__ void __launch_bounds__(256)
    negative_mask_kernel(const int64_t* __restrict__ negatives, size_t k, const int64_t* __restrict__ answer_ptr,
                         const int64_t* __restrict__ answer_ids, size_t n_queries, float* __restrict__ is_negative) {
  const size_t total = n_queries * k;
  for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += (size_t)gridDim.x * blockDim.x) {
    const size_t b = p / k, j = p - b * k;
    const int64_t* ans = answer_ids + answer_ptr[b];
    const long long n_ans = answer_ptr[b + 1] - answer_ptr[b];
    const long long id = negatives[j];
    long long lo = 0, hi = n_ans;
    while (lo < hi) {
      const long long mid = (lo + hi) >> 1;
      if (ans[mid] < id) lo = mid + 1; else hi = mid;
    }
    is_negative[p] = (lo < n_ans && ans[lo] == id) ? 0.f : 1.f;
  }
}

static int sampler_grid(size_t items) {
  return (int)std::max<size_t>(1, std::min<size_t>((items + 255) / 256, (size_t)sm_count() * 16));
}

}  // namespace smore

using namespace smore;

extern "C" {

int smore_alias_build(const double* weights, size_t n, double* prob_small, int64_t* choice_small,
                      int64_t* choice_large) {
  if (!weights || !prob_small || !choice_small || !choice_large) return fail(SMORE_ERR_NULL, "alias_build: NULL pointer");
  if (n == 0) return fail(SMORE_ERR_BAD_SHAPE, "alias_build: no choices");
  double total = 0.0;
  for (size_t i = 0; i < n; ++i) total += weights[i];
  if (!(total > 0.0)) return fail(SMORE_ERR_BAD_SHAPE, "alias_build: weights must sum to a positive value");
  // alias_method.cpp:55-99: scaled probabilities; two first-in-first-out lists of the entries above
  // and below one; slot i pairs the oldest large entry with the oldest small one
  const double factor = (double)n / total;
  std::vector<double> probs(n);
  std::deque<size_t> large, small;
  for (size_t i = 0; i < n; ++i) {
    probs[i] = weights[i] * factor;
    (probs[i] >= 1.0 ? large : small).push_back(i);
  }
  for (size_t i = 0; i < n; ++i) {
    if (large.empty()) {
      const size_t s = small.front();     // (the reference does not pop here either)
      prob_small[i] = 1.0;
      choice_small[i] = choice_large[i] = (int64_t)s;
      continue;
    }
    const size_t l = large.front();
    large.pop_front();
    size_t s = 0;
    double ps = 0.0;
    if (!small.empty()) {
      s = small.front();
      small.pop_front();
      ps = probs[s];
    }
    probs[l] -= 1.0 - ps;
    prob_small[i] = ps;
    choice_small[i] = (int64_t)s;
    choice_large[i] = (int64_t)l;
    (probs[l] < 1.0 ? small : large).push_back(l);
  }
  return SMORE_OK;
}

int smore_sample_negatives(uint64_t seed, uint64_t offset, size_t n_entities, const double* prob_small,
                           const int64_t* choice_small, const int64_t* choice_large, const int64_t* answer_ptr,
                           const int64_t* answer_ids, size_t n_queries, size_t k, int64_t* negatives, void* stream) {
  if (n_queries == 0 || k == 0) return SMORE_OK;
  if (!negatives) return fail(SMORE_ERR_NULL, "sample_negatives: NULL pointer");
  if (n_entities == 0) return fail(SMORE_ERR_BAD_SHAPE, "sample_negatives: no entities");
  const int tables = (prob_small != nullptr) + (choice_small != nullptr) + (choice_large != nullptr);
  if (tables != 0 && tables != 3) return fail(SMORE_ERR_NULL, "sample_negatives: give all three alias tables or none");
  if ((answer_ptr != nullptr) != (answer_ids != nullptr))
    return fail(SMORE_ERR_NULL, "sample_negatives: give answer_ptr and answer_ids together");
  SampleArgs a{seed, offset, n_entities, prob_small, choice_small, choice_large, answer_ptr, answer_ids, n_queries, k};
  sample_negatives_kernel<<<sampler_grid(n_queries * k), 256, 0, (cudaStream_t)stream>>>(a, negatives);
  return check_launch("sample_negatives_kernel");
}

int smore_negative_mask(const int64_t* negatives, size_t k, const int64_t* answer_ptr, const int64_t* answer_ids,
                        size_t n_queries, float* is_negative, void* stream) {
  if (n_queries == 0 || k == 0) return SMORE_OK;
  if (!negatives || !answer_ptr || !answer_ids || !is_negative) return fail(SMORE_ERR_NULL, "negative_mask: NULL pointer");
  negative_mask_kernel<<<sampler_grid(n_queries * k), 256, 0, (cudaStream_t)stream>>>(negatives, k, answer_ptr, answer_ids,
                                                                                     n_queries, is_negative);
  return check_launch("negative_mask_kernel");
}

}  // extern "C"
