// Row gather, per-step gradient merge (sorted unique + inverse map, scatter-sum) and the
// row-wise optimizers for sm_100a, with their C entry points.
//
// Replaces, for a table that lives in GPU memory:
//   smore/common/embedding/embed_rw.py:74-77,102-111       (embed[indices], index_add_)
//   smore/common/embedding/embed_optimizer.py:39-48        (torch.unique + torch_scatter sum)
//   smore/common/embedding/embed_optimizer.py:166-185      (SGD rows)
//   smore/common/embedding/embed_optimizer.py:208-252      (Adam rows, ~15 torch kernels)
//   smore/common/embedding/embed_optimizer.py:328-349      (Adagrad rows)
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <mutex>

#include "common.cuh"
#include "update_math.cuh"

namespace smore {

// ----------------------------------------------------------------------------------------
// gather
// ----------------------------------------------------------------------------------------

__device__ int g_rows_status = 0;   // kStatusBadRowId: a gathered id lay outside the table

template <bool VEC>
__global__ void __launch_bounds__(256)
    gather_rows_kernel(const float* __restrict__ table, const int64_t* __restrict__ idx, long long n_rows,
                       float* __restrict__ out, size_t n, size_t width) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  for (size_t p = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < n; p += warps) {
    long long rid = 0;
    if (lane == 0) rid = checked_row_id(idx, p, n_rows, &g_rows_status);
    rid = __shfl_sync(0xffffffffu, rid, 0);
    if (rid < 0) {   // an id outside the table: the gathered row is NaN, nothing is read
      for (size_t d = lane; d < width; d += kWarp) out[p * width + d] = NAN;
      continue;
    }
    const size_t row = (size_t)rid;
    if (VEC) {
      const float4* src = reinterpret_cast<const float4*>(table + row * width);
      float4* dst = reinterpret_cast<float4*>(out + p * width);
      for (size_t d = lane; d < width / 4; d += kWarp) dst[d] = __ldg(src + d);
    } else {
      const float* src = table + row * width;
      float* dst = out + p * width;
      for (size_t d = lane; d < width; d += kWarp) dst[d] = __ldg(src + d);
    }
  }
}

// ----------------------------------------------------------------------------------------
// sorted unique over a bounded id space: presence bitmap + popcount scan
// ----------------------------------------------------------------------------------------

constexpr int kScanThreads = 256;
constexpr int kWordsPerThread = 4;
constexpr int kWordsPerBlock = kScanThreads * kWordsPerThread;  // 1024 words = 32768 ids

struct UniqueWorkspace {
  uint32_t* bitmap;      // [nwords]   bit v set <=> id v occurs
  uint32_t* wordprefix;  // [nwords]   distinct ids below word w
  uint32_t* blocksum;    // [nblocks]  distinct ids per 1024-word block, then their exclusive scan
  size_t nwords, nblocks, bytes;
};

static size_t round256(size_t x) { return (x + 255) & ~(size_t)255; }

static UniqueWorkspace carve_unique_workspace(void* base, size_t n_table_rows) {
  UniqueWorkspace w;
  w.nwords = (n_table_rows + 31) / 32;
  w.nblocks = (w.nwords + kWordsPerBlock - 1) / kWordsPerBlock;
  const size_t b0 = round256(w.nwords * sizeof(uint32_t));
  const size_t b2 = round256(w.nblocks * sizeof(uint32_t));
  char* p = static_cast<char*>(base);
  w.bitmap = reinterpret_cast<uint32_t*>(p);
  w.wordprefix = reinterpret_cast<uint32_t*>(p + b0);
  w.blocksum = reinterpret_cast<uint32_t*>(p + 2 * b0);
  w.bytes = 2 * b0 + b2;
  return w;
}

__global__ void __launch_bounds__(256)
    unique_mark_kernel(const int64_t* __restrict__ idx, size_t n, const int32_t* __restrict__ n_dev,
                       size_t n_table_rows, uint32_t* __restrict__ bitmap, int32_t* __restrict__ n_unique) {
  if (n_dev != nullptr) n = min(n, (size_t)max(n_dev[0], 0));   // the caller's count lives on the device
  for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; p < n;
       p += (size_t)gridDim.x * blockDim.x) {
    const int64_t v = idx[p];
    if (v >= 0 && (size_t)v < n_table_rows) {
      const uint32_t bit = 1u << (v & 31);
      uint32_t* w = bitmap + (v >> 5);
      if (!(*w & bit)) atomicOr(w, bit);
    } else {
      atomicAdd(n_unique + 1, 1);
    }
  }
}

__device__ __forceinline__ uint32_t block_sum_256(uint32_t v, uint32_t* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  uint32_t t = 0;
#pragma unroll
  for (int w = 0; w < kScanThreads / 32; ++w) t += sh[w];
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(kScanThreads)
    unique_blocksum_kernel(const uint32_t* __restrict__ bitmap, size_t nwords,
                           uint32_t* __restrict__ blocksum) {
  __shared__ uint32_t sh[kScanThreads / 32];
  const size_t w0 = (size_t)blockIdx.x * kWordsPerBlock + (size_t)threadIdx.x * kWordsPerThread;
  uint32_t c = 0;
#pragma unroll
  for (int k = 0; k < kWordsPerThread; ++k)
    if (w0 + k < nwords) c += __popc(bitmap[w0 + k]);
  const uint32_t t = block_sum_256(c, sh);
  if (threadIdx.x == 0) blocksum[blockIdx.x] = t;
}

// exclusive scan of blocksum in place by one CTA; total -> n_unique[0]
__global__ void __launch_bounds__(1024)
    unique_scan_blocks_kernel(uint32_t* __restrict__ blocksum, size_t nblocks,
                              int32_t* __restrict__ n_unique) {
  __shared__ uint32_t warp_tot[32];
  __shared__ uint32_t carry_sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_sh = 0;
  __syncthreads();
  for (size_t base = 0; base < nblocks; base += 1024) {
    const size_t i = base + threadIdx.x;
    const uint32_t v = i < nblocks ? blocksum[i] : 0;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      uint32_t w = warp_tot[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
      }
      warp_tot[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const uint32_t carry = carry_sh;
    const uint32_t before_warp = warp ? warp_tot[warp - 1] : 0;
    if (i < nblocks) blocksum[i] = carry + before_warp + inc - v;
    __syncthreads();
    if (threadIdx.x == 0) carry_sh = carry + warp_tot[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) n_unique[0] = (int32_t)carry_sh;
}

__global__ void __launch_bounds__(kScanThreads)
    unique_wordprefix_kernel(const uint32_t* __restrict__ bitmap, size_t nwords,
                             const uint32_t* __restrict__ blockoff, uint32_t* __restrict__ wordprefix) {
  __shared__ uint32_t warp_tot[kScanThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t w0 = (size_t)blockIdx.x * kWordsPerBlock + (size_t)threadIdx.x * kWordsPerThread;
  uint32_t c[kWordsPerThread];
  uint32_t mine = 0;
#pragma unroll
  for (int k = 0; k < kWordsPerThread; ++k) {
    c[k] = (w0 + k < nwords) ? __popc(bitmap[w0 + k]) : 0;
    mine += c[k];
  }
  uint32_t inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  uint32_t before = blockoff[blockIdx.x];
  for (int w = 0; w < warp; ++w) before += warp_tot[w];
  uint32_t run = before + inc - mine;
#pragma unroll
  for (int k = 0; k < kWordsPerThread; ++k) {
    if (w0 + k < nwords) wordprefix[w0 + k] = run;
    run += c[k];
  }
}

__global__ void __launch_bounds__(256)
    unique_assign_kernel(const int64_t* __restrict__ idx, size_t n, const int32_t* __restrict__ n_dev,
                         size_t n_table_rows, const uint32_t* __restrict__ bitmap,
                         const uint32_t* __restrict__ wordprefix, int64_t* __restrict__ uniq,
                         int32_t* __restrict__ inverse, int32_t* __restrict__ counts) {
  if (n_dev != nullptr) n = min(n, (size_t)max(n_dev[0], 0));
  for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; p < n;
       p += (size_t)gridDim.x * blockDim.x) {
    const int64_t v = idx[p];
    if (v < 0 || (size_t)v >= n_table_rows) {
      inverse[p] = -1;
      continue;
    }
    const uint32_t word = bitmap[v >> 5];
    const uint32_t below = word & ((1u << (v & 31)) - 1u);
    const int32_t s = (int32_t)(wordprefix[v >> 5] + __popc(below));
    inverse[p] = s;
    if (atomicAdd(counts + s, 1) == 0) uniq[s] = v;
  }
}


// ----------------------------------------------------------------------------------------
// sorted unique of a SHORT id list (a step's anchor lookups: about a thousand ids) over a LARGE id
// space: the bitmap route costs O(n_table_rows / 32) whatever n is (0.3 ms for 86M rows), a sort of
// n keys in one CTA's shared memory does not.  Same results: ascending distinct ids, inverse map,
// multiplicities, counters.
// ----------------------------------------------------------------------------------------

constexpr int kSmallUniqueMax = 4096;      // ids per call on this route
constexpr int kSmallUniqueThreads = 1024;
constexpr int kSmallPosBits = 12;          // position within the call, packed below the id
constexpr unsigned long long kSmallInvalid = ~0ull;

__global__ void __launch_bounds__(kSmallUniqueThreads)
    unique_small_kernel(const int64_t* __restrict__ idx, int n, size_t n_table_rows, int P,
                        int64_t* __restrict__ uniq, int32_t* __restrict__ inverse, int32_t* __restrict__ counts,
                        int32_t* __restrict__ n_unique) {
  extern __shared__ unsigned long long keys[];   // [P], P = power of two >= n
  __shared__ int warp_tot[kSmallUniqueThreads / 32];
  __shared__ int n_bad_sh;
  const int tid = threadIdx.x;
  if (tid == 0) n_bad_sh = 0;
  __syncthreads();
  int bad = 0;
  for (int i = tid; i < P; i += kSmallUniqueThreads) {
    unsigned long long k = kSmallInvalid;
    if (i < n) {
      const int64_t v = idx[i];
      if (v >= 0 && (size_t)v < n_table_rows) k = ((unsigned long long)v << kSmallPosBits) | (unsigned)i;
      else ++bad;
      counts[i] = 0;
    }
    keys[i] = k;
  }
  if (bad) atomicAdd(&n_bad_sh, bad);
  // bitonic sort, ascending
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int t = tid; t < (P >> 1); t += kSmallUniqueThreads) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool up = (lo & size) == 0;
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == up) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
    }
  }
  __syncthreads();
  // heads of runs of equal ids -> slots: every thread owns P / 1024 consecutive sorted positions
  const int per = (P + kSmallUniqueThreads - 1) / kSmallUniqueThreads;
  const int i0 = tid * per;
  int heads = 0;
  for (int i = i0; i < min(i0 + per, P); ++i) {
    const unsigned long long k = keys[i];
    if (k != kSmallInvalid && (i == 0 || (keys[i - 1] >> kSmallPosBits) != (k >> kSmallPosBits))) ++heads;
  }
  int inc = heads;
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    warp_tot[lane] = w;
  }
  __syncthreads();
  int slot = (warp ? warp_tot[warp - 1] : 0) + inc - heads - 1;   // slot of the last head before i0
  for (int i = i0; i < min(i0 + per, P); ++i) {
    const unsigned long long k = keys[i];
    if (k == kSmallInvalid) break;                                  // invalid keys sort last
    const int64_t id = (int64_t)(k >> kSmallPosBits);
    if (i == 0 || (keys[i - 1] >> kSmallPosBits) != (k >> kSmallPosBits)) {
      ++slot;
      uniq[slot] = id;
    }
    inverse[(int)(k & ((1u << kSmallPosBits) - 1u))] = slot;
    atomicAdd(counts + slot, 1);
  }
  // positions whose id was out of range
  for (int i = tid; i < n; i += kSmallUniqueThreads) {
    const int64_t v = idx[i];
    if (v < 0 || (size_t)v >= n_table_rows) inverse[i] = -1;
  }
  if (tid == 0) {
    n_unique[0] = warp_tot[31];
    n_unique[1] = n_bad_sh;
  }
}

// ----------------------------------------------------------------------------------------
// compact gradient buffer helpers
// ----------------------------------------------------------------------------------------

// Each lane tests one slot of a 32-slot batch; the warp then clears the marked rows together
// (16-byte stores when the row allows it).  Only ~5 % of the slots are shared at the benchmark.
template <bool VEC>
__global__ void __launch_bounds__(256)
    zero_shared_rows_kernel(float* __restrict__ g_rows, const int32_t* __restrict__ slot_count,
                            const int32_t* __restrict__ n_unique, size_t width) {
  const int lane = threadIdx.x & 31;
  const size_t nu = (size_t)max(n_unique[0], 0);
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  for (size_t u0 = ((size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 32; u0 < nu; u0 += warps * 32) {
    const bool shared = u0 + lane < nu && slot_count[u0 + lane] > 1;
    unsigned todo = __ballot_sync(0xffffffffu, shared);
    while (todo) {
      const int l = __ffs(todo) - 1;
      todo &= todo - 1;
      float* r = g_rows + (u0 + l) * width;
      if (VEC) {
        float4* r4 = reinterpret_cast<float4*>(r);
        for (size_t d = lane; d < (width >> 2); d += kWarp) r4[d] = make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
        for (size_t d = lane; d < width; d += kWarp) r[d] = 0.f;
      }
    }
  }
}

template <bool VEC>
__global__ void __launch_bounds__(256)
    scatter_add_rows_kernel(const float* __restrict__ grad, const int32_t* __restrict__ slot,
                            const int32_t* __restrict__ slot_count, float* __restrict__ g_rows, size_t n,
                            size_t width) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  for (size_t p = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < n; p += warps) {
    const int32_t s = slot[p];
    if (s < 0) continue;
    const bool single = slot_count != nullptr && slot_count[s] == 1;
    if (VEC) {
      const float4* src = reinterpret_cast<const float4*>(grad + p * width);
      float4* dst = reinterpret_cast<float4*>(g_rows + (size_t)s * width);
      for (size_t d = lane; d < width / 4; d += kWarp) {
        const float4 v = __ldg(src + d);
        if (single) dst[d] = v; else atomicAdd(dst + d, v);
      }
    } else {
      const float* src = grad + p * width;
      float* dst = g_rows + (size_t)s * width;
      for (size_t d = lane; d < width; d += kWarp) {
        if (single) dst[d] = src[d]; else atomicAdd(dst + d, src[d]);
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// row-wise optimizers: one warp per touched row, one pass over (g, p, m, v)
// ----------------------------------------------------------------------------------------

// UpdateArgs, adam_elem, adam_elem_rowwise: update_math.cuh

// Adam for rows of at most 32 * NCH 16-byte chunks: every load of a row (gradient, parameters,
// first moment and, with a full second moment, that too) is issued before anything is computed,
// so each warp keeps 3-4 x NCH 512-byte requests in flight; the gradient is read once even when
// the row-wise mean of its square is needed first.
template <int NCH, bool ROWWISE>
__global__ void __launch_bounds__(256) adam_rows_reg_kernel(UpdateArgs a) {
  load_dyn(a);
  const int lane = threadIdx.x & 31;
  const size_t nu = (size_t)max(a.n_unique[0], 0);
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  const int w4 = (int)(a.width >> 2);
  // a warp takes kBatch consecutive entries of the list at a time: one read of their row ids, then the
  // rows one after the other (small batches keep the warps' loads even).  Entries with a negative id
  // were updated inside the backward pass (smore_rows_backward_fused_adam) and cost nothing here
  // beyond that read.
  constexpr int kBatch = 8;
  for (size_t u0 = ((size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kBatch; u0 < nu;
       u0 += warps * kBatch) {
    const long long my_row = (lane < kBatch && u0 + lane < nu) ? a.uniq[u0 + lane] : -1;
    unsigned live = __ballot_sync(0xffffffffu, my_row >= 0);
    while (live) {
      const int l = __ffs(live) - 1;
      live &= live - 1;
      const long long row = __shfl_sync(0xffffffffu, my_row, l);
      const size_t u = u0 + l;
      const float4* g4 = reinterpret_cast<const float4*>(a.g_rows + u * a.width);
      float4* p4 = reinterpret_cast<float4*>(a.table + (size_t)row * a.width);
      float4* m4 = reinterpret_cast<float4*>(a.m + (size_t)row * a.width);
      float4* v4 = ROWWISE ? nullptr : reinterpret_cast<float4*>(a.v + (size_t)row * a.width);
      float4 g[NCH], p[NCH], m[NCH], v[NCH];
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int d = lane + 32 * j;
        if (d < w4) {
          g[j] = __ldcs(g4 + d);
          p[j] = p4[d];
          m[j] = m4[d];
          if (!ROWWISE) v[j] = v4[d];
        }
      }
      float denom = 0.f, v_old = 0.f, v_new = 0.f;
      if (ROWWISE) {
        v_old = a.v[row];
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NCH; ++j)
          if (lane + 32 * j < w4) s += g[j].x * g[j].x + g[j].y * g[j].y + g[j].z * g[j].z + g[j].w * g[j].w;
        const float g2mean = warp_sum(s) / (float)a.width;
        v_new = v_old * a.beta2 + g2mean * a.omb2;
        denom = sqrtf(v_new) / a.sqrt_bc2 + a.eps;
      }
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int d = lane + 32 * j;
        if (d < w4) {
          if (ROWWISE) {
            adam_elem_rowwise(g[j].x, p[j].x, m[j].x, denom, a);
            adam_elem_rowwise(g[j].y, p[j].y, m[j].y, denom, a);
            adam_elem_rowwise(g[j].z, p[j].z, m[j].z, denom, a);
            adam_elem_rowwise(g[j].w, p[j].w, m[j].w, denom, a);
          } else {
            adam_elem(g[j].x, p[j].x, m[j].x, v[j].x, a);
            adam_elem(g[j].y, p[j].y, m[j].y, v[j].y, a);
            adam_elem(g[j].z, p[j].z, m[j].z, v[j].z, a);
            adam_elem(g[j].w, p[j].w, m[j].w, v[j].w, a);
            v4[d] = v[j];
          }
          p4[d] = p[j];
          m4[d] = m[j];
        }
      }
      if (ROWWISE && lane == 0) a.v[row] = v_old + (v_new - v_old);
    }
  }
}

template <int OPT, bool VEC>
__global__ void __launch_bounds__(256) sparse_update_rows_kernel(UpdateArgs a) {
  load_dyn(a);
  const int lane = threadIdx.x & 31;
  const size_t nu = (size_t)max(a.n_unique[0], 0);
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  const size_t W = a.width;
  for (size_t u = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); u < nu; u += warps) {
    if (a.uniq[u] < 0) continue;   // updated already, inside the backward pass
    const size_t row = (size_t)a.uniq[u];
    const float* g = a.g_rows + u * W;
    float* p = a.table + row * W;

    float g2mean = 0.f;
    if (OPT != SMORE_OPT_SGD && a.squeeze) {
      float s = 0.f;
      if (VEC) {
        const float4* g4 = reinterpret_cast<const float4*>(g);
        for (size_t d = lane; d < W / 4; d += kWarp) {
          const float4 x = g4[d];
          s += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        }
      } else {
        for (size_t d = lane; d < W; d += kWarp) s += g[d] * g[d];
      }
      g2mean = warp_sum(s) / (float)W;
    }

    if (OPT == SMORE_OPT_SGD) {
      if (VEC) {
        const float4* g4 = reinterpret_cast<const float4*>(g);
        float4* p4 = reinterpret_cast<float4*>(p);
        for (size_t d = lane; d < W / 4; d += kWarp) {
          const float4 x = g4[d];
          float4 y = p4[d];
          y.x += -a.lr * x.x; y.y += -a.lr * x.y; y.z += -a.lr * x.z; y.w += -a.lr * x.w;
          p4[d] = y;
        }
      } else {
        for (size_t d = lane; d < W; d += kWarp) p[d] += -a.lr * g[d];
      }
    } else if (OPT == SMORE_OPT_ADAGRAD) {
      if (a.squeeze) {
        const float s_old = a.v[row];
        const float avg = sqrtf(s_old + g2mean) + a.eps;
        if (VEC) {
          const float4* g4 = reinterpret_cast<const float4*>(g);
          float4* p4 = reinterpret_cast<float4*>(p);
          for (size_t d = lane; d < W / 4; d += kWarp) {
            const float4 x = g4[d];
            float4 y = p4[d];
            y.x += -a.lr * x.x / avg; y.y += -a.lr * x.y / avg;
            y.z += -a.lr * x.z / avg; y.w += -a.lr * x.w / avg;
            p4[d] = y;
          }
        } else {
          for (size_t d = lane; d < W; d += kWarp) p[d] += -a.lr * g[d] / avg;
        }
        __syncwarp();
        if (lane == 0) a.v[row] = s_old + g2mean;
      } else {
        float* sv = a.v + row * W;
        for (size_t d = lane; d < W; d += kWarp) {
          const float gs = g[d] * g[d];
          const float s_old = sv[d];
          p[d] += -a.lr * g[d] / (sqrtf(s_old + gs) + a.eps);
          sv[d] = s_old + gs;
        }
      }
    } else {  // Adam
      float* m = a.m + row * W;
      if (a.squeeze) {
        const float v_old = a.v[row];
        const float v_new = v_old * a.beta2 + g2mean * a.omb2;
        const float denom = sqrtf(v_new) / a.sqrt_bc2 + a.eps;
        if (VEC) {
          const float4* g4 = reinterpret_cast<const float4*>(g);
          float4* p4 = reinterpret_cast<float4*>(p);
          float4* m4 = reinterpret_cast<float4*>(m);
          for (size_t d = lane; d < W / 4; d += kWarp) {
            const float4 x = g4[d];
            float4 y = p4[d], mm = m4[d];
            adam_elem_rowwise(x.x, y.x, mm.x, denom, a);
            adam_elem_rowwise(x.y, y.y, mm.y, denom, a);
            adam_elem_rowwise(x.z, y.z, mm.z, denom, a);
            adam_elem_rowwise(x.w, y.w, mm.w, denom, a);
            p4[d] = y;
            m4[d] = mm;
          }
        } else {
          for (size_t d = lane; d < W; d += kWarp) {
            float y = p[d], mm = m[d];
            adam_elem_rowwise(g[d], y, mm, denom, a);
            p[d] = y;
            m[d] = mm;
          }
        }
        __syncwarp();
        if (lane == 0) a.v[row] = v_old + (v_new - v_old);
      } else {
        float* v = a.v + row * W;
        if (VEC) {
          const float4* g4 = reinterpret_cast<const float4*>(g);
          float4* p4 = reinterpret_cast<float4*>(p);
          float4* m4 = reinterpret_cast<float4*>(m);
          float4* v4 = reinterpret_cast<float4*>(v);
          for (size_t d = lane; d < W / 4; d += kWarp) {
            const float4 x = g4[d];
            float4 y = p4[d], mm = m4[d], vv = v4[d];
            adam_elem(x.x, y.x, mm.x, vv.x, a);
            adam_elem(x.y, y.y, mm.y, vv.y, a);
            adam_elem(x.z, y.z, mm.z, vv.z, a);
            adam_elem(x.w, y.w, mm.w, vv.w, a);
            p4[d] = y;
            m4[d] = mm;
            v4[d] = vv;
          }
        } else {
          for (size_t d = lane; d < W; d += kWarp) {
            float y = p[d], mm = m[d], vv = v[d];
            adam_elem(g[d], y, mm, vv, a);
            p[d] = y;
            m[d] = mm;
            v[d] = vv;
          }
        }
      }
    }
  }
}

static int warp_grid(size_t items) {
  const size_t blocks = (items + 7) / 8;
  return (int)std::max<size_t>(1, std::min<size_t>(blocks, (size_t)sm_count() * 16));
}

static int thread_grid(size_t items) {
  const size_t blocks = (items + 255) / 256;
  return (int)std::max<size_t>(1, std::min<size_t>(blocks, (size_t)sm_count() * 16));
}

}  // namespace smore

using namespace smore;

extern "C" {

int smore_rows_status(int* status) {   // not part of the public header; smore_async_status adds it in
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_rows_status, sizeof(int));
  if (e != cudaSuccess) return fail(SMORE_ERR_CUDA, "async_status: %s", cudaGetErrorString(e));
  *status = v;
  return SMORE_OK;
}

int smore_rows_status_clear(void) {
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_rows_status, &zero, sizeof(int)) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "async_status_clear: cannot write the status word");
  return SMORE_OK;
}

int smore_gather_rows(const float* table, const int64_t* idx, size_t n_table_rows, float* out, size_t n,
                      size_t width, void* stream) {
  if (!table || !idx || !out) return fail(SMORE_ERR_NULL, "gather_rows: NULL pointer");
  if (!width) return fail(SMORE_ERR_BAD_SHAPE, "gather_rows: width is 0");
  if (n == 0) return SMORE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (width % 4 == 0) && aligned16(table) && aligned16(out);
  if (vec)
    gather_rows_kernel<true><<<warp_grid(n), 256, 0, st>>>(table, idx, (long long)n_table_rows, out, n, width);
  else
    gather_rows_kernel<false><<<warp_grid(n), 256, 0, st>>>(table, idx, (long long)n_table_rows, out, n, width);
  return check_launch("gather_rows_kernel");
}

size_t smore_unique_rows_workspace_bytes(size_t n_table_rows) {
  return carve_unique_workspace(nullptr, n_table_rows).bytes;
}

}  // extern "C"

namespace smore {
// Shared by smore_unique_rows and the owner side of the sharded update (peer_kernels.cu), whose number
// of ids is only known on the device: with n_dev != nullptr the first min(n, *n_dev) ids count.
int unique_rows_impl(const int64_t* idx, size_t n, const int32_t* n_dev, size_t n_table_rows, int64_t* uniq,
                     int32_t* inverse, int32_t* counts, int32_t* n_unique, void* workspace, size_t workspace_bytes,
                     cudaStream_t st) {
  if (!n_unique) return fail(SMORE_ERR_NULL, "unique_rows: n_unique is NULL");
  if (n && (!idx || !uniq || !inverse || !counts)) return fail(SMORE_ERR_NULL, "unique_rows: NULL pointer");
  if (n_table_rows == 0 || n_table_rows > ((size_t)1 << 36))
    return fail(SMORE_ERR_BAD_SHAPE, "unique_rows: n_table_rows out of range");
  if (n > ((size_t)1 << 31) - 1) return fail(SMORE_ERR_TOO_LARGE, "unique_rows: more than 2^31-1 ids");
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(SMORE_ERR_WORKSPACE, "unique_rows: workspace missing or not 256-byte aligned");
  const UniqueWorkspace w = carve_unique_workspace(workspace, n_table_rows);
  if (workspace_bytes < w.bytes)
    return fail(SMORE_ERR_WORKSPACE, "unique_rows: workspace has %zu bytes, %zu needed", workspace_bytes,
                w.bytes);
  if (n_dev == nullptr && n > 0 && n <= (size_t)kSmallUniqueMax && n_table_rows >= ((size_t)1 << 18)) {
    // few ids over a large id space: sort them in one CTA instead of scanning a bitmap of the space
    int P = 32;
    while ((size_t)P < n) P <<= 1;
    unique_small_kernel<<<1, kSmallUniqueThreads, (size_t)P * sizeof(unsigned long long), st>>>(
        idx, (int)n, n_table_rows, P, uniq, inverse, counts, n_unique);
    return check_launch("unique_small_kernel");
  }
  if (cudaMemsetAsync(n_unique, 0, 2 * sizeof(int32_t), st) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "unique_rows: cudaMemsetAsync failed");
  if (n == 0) return check_launch("unique_rows memset", 0);
  if (cudaMemsetAsync(w.bitmap, 0, w.nwords * sizeof(uint32_t), st) != cudaSuccess ||
      cudaMemsetAsync(counts, 0, n * sizeof(int32_t), st) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "unique_rows: cudaMemsetAsync failed");
  unique_mark_kernel<<<thread_grid(n), 256, 0, st>>>(idx, n, n_dev, n_table_rows, w.bitmap, n_unique);
  unique_blocksum_kernel<<<(unsigned)w.nblocks, kScanThreads, 0, st>>>(w.bitmap, w.nwords, w.blocksum);
  unique_scan_blocks_kernel<<<1, 1024, 0, st>>>(w.blocksum, w.nblocks, n_unique);
  unique_wordprefix_kernel<<<(unsigned)w.nblocks, kScanThreads, 0, st>>>(w.bitmap, w.nwords, w.blocksum,
                                                                         w.wordprefix);
  unique_assign_kernel<<<thread_grid(n), 256, 0, st>>>(idx, n, n_dev, n_table_rows, w.bitmap, w.wordprefix, uniq,
                                                        inverse, counts);
  return check_launch("unique_rows kernels", 5);
}
}  // namespace smore

extern "C" {

int smore_unique_rows(const int64_t* idx, size_t n, size_t n_table_rows, int64_t* uniq, int32_t* inverse,
                      int32_t* counts, int32_t* n_unique, void* workspace, size_t workspace_bytes,
                      void* stream) {
  return unique_rows_impl(idx, n, nullptr, n_table_rows, uniq, inverse, counts, n_unique, workspace, workspace_bytes,
                          (cudaStream_t)stream);
}

int smore_zero_shared_rows(float* g_rows, const int32_t* slot_count, const int32_t* n_unique, size_t capacity,
                           size_t width, void* stream) {
  if (!g_rows || !slot_count || !n_unique) return fail(SMORE_ERR_NULL, "zero_shared_rows: NULL pointer");
  if (capacity == 0) return SMORE_OK;
  if ((width & 3) == 0 && aligned16(g_rows))
    zero_shared_rows_kernel<true><<<warp_grid((capacity + 31) / 32), 256, 0, (cudaStream_t)stream>>>(
        g_rows, slot_count, n_unique, width);
  else
    zero_shared_rows_kernel<false><<<warp_grid((capacity + 31) / 32), 256, 0, (cudaStream_t)stream>>>(
        g_rows, slot_count, n_unique, width);
  return check_launch("zero_shared_rows_kernel");
}

int smore_scatter_add_rows(const float* grad, const int32_t* slot, const int32_t* slot_count, float* g_rows,
                           size_t n, size_t width, void* stream) {
  if (n == 0) return SMORE_OK;
  if (!grad || !slot || !g_rows) return fail(SMORE_ERR_NULL, "scatter_add_rows: NULL pointer");
  if (!width) return fail(SMORE_ERR_BAD_SHAPE, "scatter_add_rows: width is 0");
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (width % 4 == 0) && aligned16(grad) && aligned16(g_rows);
  if (vec)
    scatter_add_rows_kernel<true><<<warp_grid(n), 256, 0, st>>>(grad, slot, slot_count, g_rows, n, width);
  else
    scatter_add_rows_kernel<false><<<warp_grid(n), 256, 0, st>>>(grad, slot, slot_count, g_rows, n, width);
  return check_launch("scatter_add_rows_kernel");
}

}  // extern "C"

namespace smore {
// *step += 1; out = {-lr / (1 - beta1^step), sqrt(1 - beta2^step)} in double, narrowed once
__global__ void adam_step_scalars_kernel(long long* step, double lr, double beta1, double beta2, float* out) {
  const long long t = *step + 1;
  *step = t;
  out[0] = (float)(-lr / (1.0 - pow(beta1, (double)t)));
  out[1] = (float)sqrt(1.0 - pow(beta2, (double)t));
}
}  // namespace smore

static int update_rows_impl(int opt_id, float* table, float* m, float* v, const int64_t* uniq,
                            const float* g_rows, const int32_t* n_unique, size_t capacity, size_t width,
                            double lr, double beta1, double beta2, double eps, int64_t step,
                            const float* step_scalars, int squeeze, void* stream);

extern "C" {

int smore_adam_step_scalars(int64_t* step, double lr, double beta1, double beta2, float* step_scalars,
                            void* stream) {
  if (!step || !step_scalars) return fail(SMORE_ERR_NULL, "adam_step_scalars: NULL pointer");
  adam_step_scalars_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(reinterpret_cast<long long*>(step), lr, beta1, beta2,
                                                               step_scalars);
  return check_launch("adam_step_scalars_kernel");
}

int smore_sparse_update_rows(int opt_id, float* table, float* m, float* v, const int64_t* uniq,
                             const float* g_rows, const int32_t* n_unique, size_t capacity, size_t width,
                             double lr, double beta1, double beta2, double eps, int64_t step, int squeeze,
                             void* stream) {
  if (opt_id == SMORE_OPT_ADAM && step < 1) return fail(SMORE_ERR_BAD_SHAPE, "adam step must be >= 1");
  return update_rows_impl(opt_id, table, m, v, uniq, g_rows, n_unique, capacity, width, lr, beta1, beta2, eps,
                          step < 1 ? 1 : step, nullptr, squeeze, stream);
}

int smore_sparse_update_rows_dev(int opt_id, float* table, float* m, float* v, const int64_t* uniq,
                                 const float* g_rows, const int32_t* n_unique, size_t capacity, size_t width,
                                 double lr, double beta1, double beta2, double eps, const float* step_scalars,
                                 int squeeze, void* stream) {
  if (!step_scalars) return fail(SMORE_ERR_NULL, "sparse_update_rows_dev: step_scalars is NULL");
  return update_rows_impl(opt_id, table, m, v, uniq, g_rows, n_unique, capacity, width, lr, beta1, beta2, eps, 1,
                          step_scalars, squeeze, stream);
}

}  // extern "C"

static int update_rows_impl(int opt_id, float* table, float* m, float* v, const int64_t* uniq,
                            const float* g_rows, const int32_t* n_unique, size_t capacity, size_t width,
                            double lr, double beta1, double beta2, double eps, int64_t step,
                            const float* step_scalars, int squeeze, void* stream) {
  if (opt_id < SMORE_OPT_SGD || opt_id > SMORE_OPT_ADAGRAD)
    return fail(SMORE_ERR_BAD_DIST, "unknown optimizer id %d", opt_id);
  if (capacity == 0) return SMORE_OK;
  if (!table || !uniq || !g_rows || !n_unique) return fail(SMORE_ERR_NULL, "sparse_update_rows: NULL pointer");
  if (opt_id == SMORE_OPT_ADAM && (!m || !v)) return fail(SMORE_ERR_NULL, "adam needs m and v");
  if (opt_id == SMORE_OPT_ADAGRAD && !v) return fail(SMORE_ERR_NULL, "adagrad needs v");
  if (!width) return fail(SMORE_ERR_BAD_SHAPE, "sparse_update_rows: width is 0");
  UpdateArgs a;
  a.table = table; a.m = m; a.v = v; a.uniq = uniq; a.g_rows = g_rows; a.n_unique = n_unique;
  a.width = width;
  set_hyper(a, lr, beta1, beta2, eps, step, squeeze);
  a.dyn = step_scalars;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (width % 4 == 0) && aligned16(table) && aligned16(g_rows) && (!m || aligned16(m)) &&
                   (!v || squeeze || aligned16(v));
  const int grid = warp_grid(capacity);
  const size_t w4 = width >> 2;
  if (opt_id == SMORE_OPT_ADAM && vec && w4 <= 256) {
    // rows of up to 1024 floats: the register-resident kernel
#define ADAM_REG(NCH)                                                         \
  if (a.squeeze) adam_rows_reg_kernel<NCH, true><<<grid, 256, 0, st>>>(a);    \
  else adam_rows_reg_kernel<NCH, false><<<grid, 256, 0, st>>>(a)
    if (w4 <= 32) { ADAM_REG(1); }
    else if (w4 <= 64) { ADAM_REG(2); }
    else if (w4 <= 128) { ADAM_REG(4); }
    else { ADAM_REG(8); }
#undef ADAM_REG
    return check_launch("adam_rows_reg_kernel");
  }
#define LAUNCH(OPT)                                                                  \
  if (vec) sparse_update_rows_kernel<OPT, true><<<grid, 256, 0, st>>>(a);            \
  else sparse_update_rows_kernel<OPT, false><<<grid, 256, 0, st>>>(a)
  if (opt_id == SMORE_OPT_SGD) { LAUNCH(SMORE_OPT_SGD); }
  else if (opt_id == SMORE_OPT_ADAM) { LAUNCH(SMORE_OPT_ADAM); }
  else { LAUNCH(SMORE_OPT_ADAGRAD); }
#undef LAUNCH
  return check_launch("sparse_update_rows_kernel");
}

// ----------------------------------------------------------------------------------------
// smore_unique_rows_static: the same de-duplication with its scratch inside the library
// ----------------------------------------------------------------------------------------
//
// Some hosts cannot hand this library a scratch buffer because they cannot allocate one at the
// moment of the call: an embedding server whose memory manager claimed the whole GPU at start-up
// (a later cudaMalloc simply fails), or a training loop that must not call cudaMalloc in steady
// state because the call synchronises the device and stalls every stream.  For them the scratch
// lives in this file as a fixed device array.  Every GPU that loads the library carries the
// array (about 4 MiB) until the process exits, which is why its size is capped.

namespace smore {

// presence bitmap + per-word prefix for 2^24 ids, plus the per-block sums
constexpr size_t kStaticUniqueMaxRows = SMORE_UNIQUE_STATIC_MAX_ROWS;
constexpr size_t kStaticUniqueWords = kStaticUniqueMaxRows / 32;
constexpr size_t kStaticUniqueBytes =
    2 * kStaticUniqueWords * sizeof(uint32_t) + ((kStaticUniqueWords / kWordsPerBlock) * sizeof(uint32_t) + 255) / 256 * 256;

static __device__ __align__(256) unsigned char g_unique_scratch[kStaticUniqueBytes];

constexpr int kMaxDevices = 64;
static void* g_unique_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_unique_scratch_mutex;

// Device address of g_unique_scratch on the current device.  In host code the array's name is
// only a handle for the runtime, not a pointer a kernel could use: the address has to be asked
// for, once per device, while that device is current.
static int static_unique_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(SMORE_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(SMORE_ERR_TOO_LARGE, "device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_unique_scratch_mutex);
  if (g_unique_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_unique_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(SMORE_ERR_CUDA, "cudaGetSymbolAddress(unique scratch): %s", cudaGetErrorString(e));
    g_unique_scratch_addr[dev] = p;
  }
  *out = g_unique_scratch_addr[dev];
  return SMORE_OK;
}

}  // namespace smore

extern "C" int smore_unique_rows_static(const int64_t* idx, size_t n, size_t n_table_rows, int64_t* uniq,
                                        int32_t* inverse, int32_t* counts, int32_t* n_unique, void* stream) {
  if (!n_unique) return fail(SMORE_ERR_NULL, "unique_rows_static: n_unique is NULL");
  if (n && (!idx || !uniq || !inverse || !counts)) return fail(SMORE_ERR_NULL, "unique_rows_static: NULL pointer");
  if (n_table_rows == 0) return fail(SMORE_ERR_BAD_SHAPE, "unique_rows_static: n_table_rows is 0");
  if (n_table_rows > kStaticUniqueMaxRows)
    return fail(SMORE_ERR_TOO_LARGE,
                "unique_rows_static: table has %zu rows, the built-in scratch covers at most %zu; use "
                "smore_unique_rows with a caller-provided workspace",
                n_table_rows, (size_t)kStaticUniqueMaxRows);
  if (n > ((size_t)1 << 31) - 1) return fail(SMORE_ERR_TOO_LARGE, "unique_rows_static: more than 2^31-1 ids");
  void* scratch = nullptr;
  if (int rc = static_unique_scratch(&scratch)) return rc;
  const UniqueWorkspace w = carve_unique_workspace(scratch, n_table_rows);
  if (w.bytes > kStaticUniqueBytes) return fail(SMORE_ERR_WORKSPACE, "unique_rows_static: scratch layout overflow");
  cudaStream_t st = (cudaStream_t)stream;
  // the array still holds the previous call's bitmap: everything that must start at zero is cleared here
  if (cudaMemsetAsync(n_unique, 0, 2 * sizeof(int32_t), st) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "unique_rows_static: cudaMemsetAsync failed");
  if (n == 0) return check_launch("unique_rows_static memset", 0);
  if (cudaMemsetAsync(w.bitmap, 0, w.nwords * sizeof(uint32_t), st) != cudaSuccess ||
      cudaMemsetAsync(counts, 0, n * sizeof(int32_t), st) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "unique_rows_static: cudaMemsetAsync failed");
  unique_mark_kernel<<<thread_grid(n), 256, 0, st>>>(idx, n, nullptr, n_table_rows, w.bitmap, n_unique);
  unique_blocksum_kernel<<<(unsigned)w.nblocks, kScanThreads, 0, st>>>(w.bitmap, w.nwords, w.blocksum);
  unique_scan_blocks_kernel<<<1, 1024, 0, st>>>(w.blocksum, w.nblocks, n_unique);
  unique_wordprefix_kernel<<<(unsigned)w.nblocks, kScanThreads, 0, st>>>(w.bitmap, w.nwords, w.blocksum,
                                                                         w.wordprefix);
  unique_assign_kernel<<<thread_grid(n), 256, 0, st>>>(idx, n, nullptr, n_table_rows, w.bitmap, w.wordprefix, uniq,
                                                        inverse, counts);
  return check_launch("unique_rows_static kernels", 5);
}
