// Row-sharded entity table over the GPUs of one NVLink / NVSwitch box: peer-memory plumbing and
// the kernels that move rows and row gradients between owners and requesters.
//
// The reference shares its table between GPU processes through CPU shared memory and PCIe staging
// (smore/common/embedding/embed_rw.py:53-134, smore/common/torchext/extlib_cuda.cpp:82-144,
// smore/models/kg_reasoning.py:144-147).  Here rows [g*S, (g+1)*S) of the table and of its Adam
// state live in the HBM of GPU g, and every exchange is a kernel of this file doing plain 128-bit
// loads from peer-mapped memory:
//   fetch_rows_kernel          requester pulls each distinct row of its step once into a local
//                              staging block (forward and backward then run on local memory)
//   shard_collect_ids_kernel   owner reads every rank's list of distinct row ids and keeps those in
//                              its range (as local ids; everything else becomes -1)
//   shard_reduce_update_kernel owner pulls the gradient rows of each of its touched rows from the
//                              ranks that produced them, sums them in a fixed order and applies
//                              Adam to its shard — transfer, reduction and update in one pass
// No kernel here waits on another rank: ordering between the phases of a step is the caller's
// (stream-ordered collectives).  Peer data is read with ordinary loads or, in the background row
// pull, with untiled bulk asynchronous copies (no tensor maps, no multicast).
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cstring>

#include "bulk_copy.cuh"
#include "common.cuh"
#include "update_math.cuh"

namespace smore {

constexpr int kMaxPlans = 4;    // id lists a rank may publish per step
constexpr int kMaxLists = 32;   // ranks x plans; one lane per list in the search below

struct PlanCaps {
  int n_plans;
  int cap[kMaxPlans];
  int prefix[kMaxPlans + 1];  // prefix[p] = first position of plan p inside one rank's span
};

static int make_caps(const int32_t* plan_caps, size_t n_plans, PlanCaps* out) {
  if (n_plans == 0 || n_plans > (size_t)kMaxPlans || !plan_caps)
    return fail(SMORE_ERR_BAD_SHAPE, "n_plans must be 1..%d", kMaxPlans);
  out->n_plans = (int)n_plans;
  out->prefix[0] = 0;
  for (int p = 0; p < kMaxPlans; ++p) {
    out->cap[p] = p < (int)n_plans ? plan_caps[p] : 0;
    if (out->cap[p] < 0) return fail(SMORE_ERR_BAD_SHAPE, "negative plan capacity");
    if ((long long)out->prefix[p] + out->cap[p] > INT_MAX) return fail(SMORE_ERR_TOO_LARGE, "plan capacities");
    out->prefix[p + 1] = out->prefix[p] + out->cap[p];
  }
  return SMORE_OK;
}

__device__ __forceinline__ void decode_position(const PlanCaps& c, int64_t i, int& list, int& j) {
  const int span = c.prefix[kMaxPlans];
  const int g = (int)(i / span);
  const int rem = (int)(i - (int64_t)g * span);
  int p = 0;
#pragma unroll
  for (int q = 1; q < kMaxPlans; ++q)
    if (q < c.n_plans && rem >= c.prefix[q]) p = q;
  list = g * c.n_plans + p;
  j = rem - c.prefix[p];
}

// staging[u, :] = shard[owner(uniq[u])][local(uniq[u]), :]
// A warp copies ROWS rows per iteration and issues every 16-byte load of all of them before the
// first store, so that ROWS x NCH 512-byte requests per warp are in flight over NVLink.
// uniq is sorted, i.e. grouped by owner.  Walking it front to back would make every rank pull
// from the same owner at the same time (one NVLink port serving all); instead consecutive
// iterations take rows from kFetchSegments evenly spaced segments of the list, so the requests in
// flight are spread over all owners at all times.
constexpr int kFetchSegments = 16;

template <int NCH, int ROWS>
__global__ void __launch_bounds__(256)
    fetch_rows_kernel(const float* const* __restrict__ shard_ptrs, size_t rows_per_shard,
                      const int64_t* __restrict__ uniq, const int32_t* __restrict__ n_unique, int w4,
                      float4* __restrict__ staging) {
  const int lane = threadIdx.x & 31;
  const size_t nu = (size_t)max(n_unique[0], 0);
  const size_t seglen = (nu + kFetchSegments - 1) / kFetchSegments;
  const size_t total = seglen * kFetchSegments;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  for (size_t t0 = ((size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * ROWS; t0 < total;
       t0 += warps * ROWS) {
    float4 x[ROWS][NCH];
    size_t urow[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const size_t t = t0 + r;
      urow[r] = (t % kFetchSegments) * seglen + t / kFetchSegments;
      if (t >= total || urow[r] >= nu) urow[r] = nu;  // nothing to copy for this slot
      const size_t id = (size_t)uniq[urow[r] < nu ? urow[r] : 0];
      const size_t owner = id / rows_per_shard, local = id - owner * rows_per_shard;
      const float4* src = reinterpret_cast<const float4*>(shard_ptrs[owner]) + local * (size_t)w4;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int d = lane + 32 * j;
        if (d < w4 && urow[r] < nu) x[r][j] = src[d];
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (urow[r] < nu) {
        float4* dst = staging + urow[r] * (size_t)w4;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          const int d = lane + 32 * j;
          if (d < w4) dst[d] = x[r][j];
        }
      }
    }
  }
}

// The background form of the row pull: no registers or load/store slots to speak of.  A CTA is two
// warps; every active lane owns one row slot in shared memory and moves one row at a time with
// two bulk asynchronous copies, peer (or local) global memory -> slot -> local staging block,
// tracked by the lane's mbarrier and bulk group.  The copy engine does the work; the SM's
// registers, issue slots and load/store units stay with the kernels of the step in progress.
// No multicast, no tensor maps: plain untiled bulk copies, which may read a peer's memory.
__device__ int g_peer_async_status = 0;   // bit 0: a bounded wait for a bulk copy gave up

constexpr int kBulkFetchWarps = 2;

__global__ void __launch_bounds__(kBulkFetchWarps * 32)
    fetch_rows_bulk_kernel(const float* const* __restrict__ shard_ptrs, size_t rows_per_shard,
                           const int64_t* __restrict__ uniq, const int32_t* __restrict__ n_unique,
                           unsigned row_bytes, int slots_per_warp, unsigned char* __restrict__ staging) {
  extern __shared__ __align__(128) unsigned char fetch_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fetch_smem);                       // [warps][32]
  unsigned char* slots = fetch_smem + kBulkFetchWarps * 32 * sizeof(uint64_t);    // [warps][slots_per_warp][row_bytes]
  uint64_t* bar = bars + warp * 32 + lane;
  unsigned char* slot = slots + ((size_t)warp * slots_per_warp + lane) * row_bytes;
  const bool owns_slot = lane < slots_per_warp;
  if (owns_slot) bulk::barrier_init(bar, 1);
  bulk::fence_barrier_init();
  __syncthreads();
  const size_t nu = (size_t)max(n_unique[0], 0);
  const size_t seglen = (nu + kFetchSegments - 1) / kFetchSegments;
  const size_t total = seglen * kFetchSegments;
  const size_t per_sweep = (size_t)gridDim.x * kBulkFetchWarps * slots_per_warp;
  unsigned parity = 0;
  for (size_t t0 = ((size_t)blockIdx.x * kBulkFetchWarps + warp) * slots_per_warp; t0 < total; t0 += per_sweep) {
    const size_t t = t0 + lane;
    // the same interleaving of the sorted id list as fetch_rows_kernel: neighbours hit different owners
    size_t u = (t % kFetchSegments) * seglen + t / kFetchSegments;
    const bool work = owns_slot && t < total && u < nu;
    if (work) {
      const size_t id = (size_t)uniq[u];
      const size_t owner = id / rows_per_shard, local = id - owner * rows_per_shard;
      const unsigned char* src = reinterpret_cast<const unsigned char*>(shard_ptrs[owner]) + local * (size_t)row_bytes;
      bulk::barrier_expect(bar, row_bytes);
      bulk::load(slot, src, row_bytes, bar);
    }
    bool ok = !work || bulk::barrier_wait(bar, parity);
    if (!__all_sync(0xffffffffu, ok)) {
      // give up: flag it, let the copies that are still on their way land (one more bounded wait by
      // the lanes that own them, so that nothing writes into this CTA's shared memory after it has
      // left), and stop.  The rows not copied keep whatever the staging block held.
      if (lane == 0) atomicOr(&g_peer_async_status, 1);
      if (!ok) bulk::barrier_wait(bar, parity);
      break;
    }
    if (work) {
      bulk::store(staging + u * (size_t)row_bytes, slot, row_bytes);
      bulk::commit_group();
      bulk::wait_group_read<0>();   // the slot may be overwritten by the next sweep's load
    }
    parity ^= 1u;
  }
  bulk::wait_group<0>();
}

// Rows that were pulled into `staging` BEFORE their owners finished the previous step's update may
// be stale (or torn).  Owners publish the set of rows they updated as a bitmap over their shard.
// pull_bitmaps_kernel copies every rank's bitmap into local memory (a few MB in all, one bulk
// transfer instead of one 4-byte peer read per row); refresh_rows_kernel then tests each distinct
// row of the step against the local copy and re-pulls exactly the marked rows.
__global__ void __launch_bounds__(256)
    pull_bitmaps_kernel(const uint32_t* const* __restrict__ dirty_ptrs, int n_ranks, size_t words,
                        uint32_t* __restrict__ local) {
  const size_t total = (size_t)n_ranks * words;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t g = i / words;
    local[i] = dirty_ptrs[g][i - g * words];
  }
}

__global__ void __launch_bounds__(256)
    refresh_rows_kernel(const float* const* __restrict__ shard_ptrs, const uint32_t* __restrict__ dirty_local,
                        size_t words, size_t rows_per_shard, const int64_t* __restrict__ uniq,
                        const int32_t* __restrict__ n_unique, int w4, float4* __restrict__ staging) {
  const int lane = threadIdx.x & 31;
  const size_t nu = (size_t)max(n_unique[0], 0);
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  for (size_t u0 = ((size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 32; u0 < nu; u0 += warps * 32) {
    // each lane tests one row of a 32-row batch, then the warp copies the marked ones together
    bool marked = false;
    size_t owner = 0, local = 0;
    if (u0 + lane < nu) {
      const size_t id = (size_t)uniq[u0 + lane];
      owner = id / rows_per_shard;
      local = id - owner * rows_per_shard;
      marked = (dirty_local[owner * words + (local >> 5)] >> (local & 31)) & 1u;
    }
    unsigned todo = __ballot_sync(0xffffffffu, marked);
    while (todo) {
      const int l = __ffs(todo) - 1;
      todo &= todo - 1;
      const size_t o = __shfl_sync(0xffffffffu, owner, l), r = __shfl_sync(0xffffffffu, local, l);
      const float4* src = reinterpret_cast<const float4*>(shard_ptrs[o]) + r * (size_t)w4;
      float4* dst = staging + (u0 + l) * (size_t)w4;
      for (int d = lane; d < w4; d += kWarp) dst[d] = src[d];
    }
  }
}

__global__ void __launch_bounds__(256)
    shard_mark_dirty_kernel(const int64_t* __restrict__ uniq, const int32_t* __restrict__ n_unique,
                            uint32_t* __restrict__ dirty) {
  const size_t nu = (size_t)max(n_unique[0], 0);
  for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < nu; u += (size_t)gridDim.x * blockDim.x) {
    const int64_t row = uniq[u];
    atomicOr(dirty + (row >> 5), 1u << (row & 31));
  }
}

__global__ void __launch_bounds__(256)
    shard_collect_ids_kernel(const int64_t* const* __restrict__ uniq_ptrs,
                             const int32_t* const* __restrict__ nuniq_ptrs, PlanCaps c, int n_ranks,
                             int64_t base, int64_t shard_rows, int64_t* __restrict__ out_ids,
                             int32_t* __restrict__ bounds) {
  __shared__ int counts_sh[kMaxLists];  // each list's length is read from its owner once per CTA
  if (threadIdx.x < n_ranks * c.n_plans) counts_sh[threadIdx.x] = nuniq_ptrs[threadIdx.x][0];
  __syncthreads();
  const int64_t total = (int64_t)n_ranks * c.prefix[kMaxPlans];
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int list, j;
    decode_position(c, i, list, j);
    int64_t local = -1;
    const int count = counts_sh[list];
    if (j < count) {
      const int64_t* ids = uniq_ptrs[list];
      const int64_t id = ids[j] - base;
      if (id >= 0 && id < shard_rows) {
        local = id;
        // ids ascend, so the kept entries of a list are one run: only its two ends write the bounds
        if (j == 0 || ids[j - 1] < base) bounds[2 * list] = j;
        if (j + 1 == count || ids[j + 1] - base >= shard_rows) bounds[2 * list + 1] = j + 1;
      }
    }
    out_ids[i] = local;
  }
}

__global__ void __launch_bounds__(256) shard_init_bounds_kernel(int32_t* bounds, int n_lists) {
  const int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l < n_lists) {
    bounds[2 * l] = INT_MAX;
    bounds[2 * l + 1] = 0;
  }
}

__global__ void __launch_bounds__(256)
    shard_record_sources_kernel(const int32_t* __restrict__ slot, size_t n, int32_t* __restrict__ src) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int32_t s = slot[i];
    if (s >= 0) src[s] = (int32_t)i;  // any contributor will do; rows with several are searched for
  }
}

struct ReduceArgs {
  const int32_t* counts;            // contributors per distinct row
  const int32_t* src;               // one contributing position per distinct row
  const float* const* grad_ptrs;    // [lists] gradient blocks (peer memory)
  const int64_t* ids;               // collected local ids, [ranks][span]
  const int32_t* bounds;            // [lists][2] valid range of each list inside its span
  PlanCaps caps;
  int n_lists;
};

template <int NCH>
__device__ __forceinline__ void add_row(float4 (&g)[NCH], const float4* row, int lane, int w4) {
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int d = lane + 32 * j;
    if (d < w4) {
      const float4 x = row[d];
      g[j].x += x.x;
      g[j].y += x.y;
      g[j].z += x.z;
      g[j].w += x.w;
    }
  }
}

template <int NCH, bool ROWWISE>
__global__ void __launch_bounds__(256) shard_reduce_update_kernel(UpdateArgs a, ReduceArgs r) {
  load_dyn(a);
  const int lane = threadIdx.x & 31;
  const size_t nu = (size_t)max(a.n_unique[0], 0);
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  const int w4 = (int)(a.width >> 2);
  const int span = r.caps.prefix[kMaxPlans];
  for (size_t u = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); u < nu; u += warps) {
    const int64_t row = a.uniq[u];
    float4* p4 = reinterpret_cast<float4*>(a.table + (size_t)row * a.width);
    float4* m4 = reinterpret_cast<float4*>(a.m + (size_t)row * a.width);
    float4* v4 = ROWWISE ? nullptr : reinterpret_cast<float4*>(a.v + (size_t)row * a.width);
    float4 g[NCH], p[NCH], m[NCH], v[NCH];
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int d = lane + 32 * j;
      g[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d < w4) {
        p[j] = p4[d];
        m[j] = m4[d];
        if (!ROWWISE) v[j] = v4[d];
      }
    }
    // ---- pull and sum this row's gradient contributions ----------------------------------------
    if (r.counts[u] == 1) {
      int list, j;
      decode_position(r.caps, (int64_t)r.src[u], list, j);
      add_row<NCH>(g, reinterpret_cast<const float4*>(r.grad_ptrs[list]) + (size_t)j * w4, lane, w4);
    } else {
      // lane l searches list l (ids ascending inside [lo, hi)); contributions are then added in
      // list order, so the sum does not depend on timing
      int found = -1;
      if (lane < r.n_lists) {
        const int g_rank = lane / r.caps.n_plans, pl = lane - g_rank * r.caps.n_plans;
        const int64_t* ids = r.ids + (size_t)g_rank * span + r.caps.prefix[pl];
        int lo = r.bounds[2 * lane], hi = r.bounds[2 * lane + 1];
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          const int64_t x = ids[mid];
          if (x < row) lo = mid + 1; else hi = mid;
        }
        if (lo < r.bounds[2 * lane + 1] && ids[lo] == row) found = lo;
      }
      unsigned hits = __ballot_sync(0xffffffffu, found >= 0);
      while (hits) {
        const int l = __ffs(hits) - 1;
        hits &= hits - 1;
        const int j = __shfl_sync(0xffffffffu, found, l);
        add_row<NCH>(g, reinterpret_cast<const float4*>(r.grad_ptrs[l]) + (size_t)j * w4, lane, w4);
      }
    }
    // ---- Adam on the local row -----------------------------------------------------------------
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

static int grid_warps(size_t items) {
  return (int)std::max<size_t>(1, std::min<size_t>((items + 7) / 8, (size_t)sm_count() * 16));
}
static int grid_threads(size_t items) {
  return (int)std::max<size_t>(1, std::min<size_t>((items + 255) / 256, (size_t)sm_count() * 16));
}

}  // namespace smore

using namespace smore;

extern "C" {

static int fetch_rows_impl(const float* const* shard_ptrs, size_t rows_per_shard, const int64_t* uniq,
                           const int32_t* n_unique, size_t capacity, size_t width, float* staging, size_t max_ctas,
                           void* stream) {
  if (capacity == 0) return SMORE_OK;
  if (!shard_ptrs || !uniq || !n_unique || !staging) return fail(SMORE_ERR_NULL, "fetch_rows: NULL pointer");
  if (rows_per_shard == 0 || width == 0 || (width & 3) || width > 1024 || !aligned16(staging))
    return fail(SMORE_ERR_BAD_SHAPE,
                "fetch_rows: width must be a multiple of 4 floats, at most 1024; staging 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int w4 = (int)(width >> 2);
  float4* out = reinterpret_cast<float4*>(staging);
  const auto grid = [&](size_t warp_items) {
    const int g = grid_warps(warp_items);
    return max_ctas ? (int)std::min<size_t>((size_t)g, max_ctas) : g;
  };
  if (w4 <= 32)
    fetch_rows_kernel<1, 8><<<grid((capacity + 7) / 8), 256, 0, st>>>(shard_ptrs, rows_per_shard, uniq, n_unique, w4, out);
  else if (w4 <= 64)
    fetch_rows_kernel<2, 4><<<grid((capacity + 3) / 4), 256, 0, st>>>(shard_ptrs, rows_per_shard, uniq, n_unique, w4, out);
  else if (w4 <= 128)
    fetch_rows_kernel<4, 4><<<grid((capacity + 3) / 4), 256, 0, st>>>(shard_ptrs, rows_per_shard, uniq, n_unique, w4, out);
  else
    fetch_rows_kernel<8, 2><<<grid((capacity + 1) / 2), 256, 0, st>>>(shard_ptrs, rows_per_shard, uniq, n_unique, w4, out);
  return check_launch("fetch_rows_kernel");
}

int smore_fetch_rows(const float* const* shard_ptrs, size_t rows_per_shard, const int64_t* uniq,
                     const int32_t* n_unique, size_t capacity, size_t width, float* staging, void* stream) {
  return fetch_rows_impl(shard_ptrs, rows_per_shard, uniq, n_unique, capacity, width, staging, 0, stream);
}

int smore_peer_async_status(int* status) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_peer_async_status, sizeof(int));
  if (e != cudaSuccess) return fail(SMORE_ERR_CUDA, "async_status: %s", cudaGetErrorString(e));
  *status = v;
  return SMORE_OK;
}

int smore_peer_status_clear(void) {
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_peer_async_status, &zero, sizeof(int)) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "async_status_clear: cannot write the status word");
  return SMORE_OK;
}

int smore_fetch_rows_background(const float* const* shard_ptrs, size_t rows_per_shard, const int64_t* uniq,
                                const int32_t* n_unique, size_t capacity, size_t width, float* staging,
                                size_t max_ctas, void* stream) {
  if (max_ctas == 0) return fail(SMORE_ERR_BAD_SHAPE, "fetch_rows_background: max_ctas must be positive");
  const size_t row_bytes = width * sizeof(float);
  if (capacity && shard_ptrs && uniq && n_unique && staging && rows_per_shard && width && (width & 3) == 0 &&
      aligned16(staging) && row_bytes <= 20 * 1024) {
    // rows of up to 20 KB: the copy-engine kernel (about 20 KB of slots per warp, two warps per CTA)
    const int slots = (int)std::min<size_t>(32, std::max<size_t>(1, 20 * 1024 / row_bytes));
    const size_t smem = kBulkFetchWarps * 32 * sizeof(uint64_t) + (size_t)kBulkFetchWarps * slots * row_bytes;
    if (int rc = allow_large_smem(fetch_rows_bulk_kernel, 48 * 1024, false)) return rc;
    const size_t want = (capacity + (size_t)kBulkFetchWarps * slots - 1) / ((size_t)kBulkFetchWarps * slots);
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min(want, max_ctas));
    fetch_rows_bulk_kernel<<<grid, kBulkFetchWarps * 32, smem, (cudaStream_t)stream>>>(
        shard_ptrs, rows_per_shard, uniq, n_unique, (unsigned)row_bytes, slots,
        reinterpret_cast<unsigned char*>(staging));
    return check_launch("fetch_rows_bulk_kernel");
  }
  return fetch_rows_impl(shard_ptrs, rows_per_shard, uniq, n_unique, capacity, width, staging, max_ctas, stream);
}

int smore_refresh_rows(const float* const* shard_ptrs, const uint32_t* const* dirty_ptrs, size_t n_ranks,
                       size_t rows_per_shard, const int64_t* uniq, const int32_t* n_unique, size_t capacity,
                       size_t width, float* staging, uint32_t* bitmap_scratch, void* stream) {
  if (capacity == 0) return SMORE_OK;
  if (!shard_ptrs || !dirty_ptrs || !uniq || !n_unique || !staging || !bitmap_scratch)
    return fail(SMORE_ERR_NULL, "refresh_rows: NULL pointer");
  if (n_ranks == 0 || rows_per_shard == 0 || width == 0 || (width & 3) || !aligned16(staging))
    return fail(SMORE_ERR_BAD_SHAPE, "refresh_rows: width must be a multiple of 4 floats; staging 16-byte aligned");
  const size_t words = (rows_per_shard + 31) / 32;
  cudaStream_t st = (cudaStream_t)stream;
  pull_bitmaps_kernel<<<grid_threads(n_ranks * words), 256, 0, st>>>(dirty_ptrs, (int)n_ranks, words, bitmap_scratch);
  refresh_rows_kernel<<<grid_warps(capacity), 256, 0, st>>>(shard_ptrs, bitmap_scratch, words, rows_per_shard, uniq,
                                                            n_unique, (int)(width >> 2),
                                                            reinterpret_cast<float4*>(staging));
  return check_launch("refresh_rows kernels", 2);
}

int smore_shard_mark_dirty(const int64_t* uniq, const int32_t* n_unique, size_t capacity, size_t shard_rows,
                           uint32_t* dirty, void* stream) {
  if (!uniq || !n_unique || !dirty) return fail(SMORE_ERR_NULL, "shard_mark_dirty: NULL pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(dirty, 0, ((shard_rows + 31) / 32) * sizeof(uint32_t), st) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "shard_mark_dirty: cudaMemsetAsync failed");
  if (capacity)
    shard_mark_dirty_kernel<<<grid_threads(capacity), 256, 0, st>>>(uniq, n_unique, dirty);
  return check_launch("shard_mark_dirty_kernel", capacity ? 1 : 0);
}

int smore_shard_collect_ids(const int64_t* const* uniq_ptrs, const int32_t* const* nuniq_ptrs, size_t n_ranks,
                            size_t n_plans, const int32_t* plan_caps, int64_t base, size_t shard_rows,
                            int64_t* out_ids, int32_t* list_bounds, void* stream) {
  if (!uniq_ptrs || !nuniq_ptrs || !out_ids || !list_bounds) return fail(SMORE_ERR_NULL, "shard_collect_ids: NULL pointer");
  PlanCaps c;
  if (int rc = make_caps(plan_caps, n_plans, &c)) return rc;
  if (n_ranks == 0 || n_ranks * n_plans > (size_t)kMaxLists)
    return fail(SMORE_ERR_BAD_SHAPE, "ranks x plans must be 1..%d", kMaxLists);
  const size_t total = n_ranks * (size_t)c.prefix[kMaxPlans];
  if (total > (size_t)INT_MAX) return fail(SMORE_ERR_TOO_LARGE, "shard_collect_ids: more than 2^31-1 positions");
  cudaStream_t st = (cudaStream_t)stream;
  shard_init_bounds_kernel<<<1, 256, 0, st>>>(list_bounds, (int)(n_ranks * n_plans));
  if (total)
    shard_collect_ids_kernel<<<grid_threads(total), 256, 0, st>>>(uniq_ptrs, nuniq_ptrs, c, (int)n_ranks, base,
                                                                  (int64_t)shard_rows, out_ids, list_bounds);
  return check_launch("shard_collect_ids kernels", 2);
}

int smore_shard_record_sources(const int32_t* slot, size_t n, int32_t* src, void* stream) {
  if (n == 0) return SMORE_OK;
  if (!slot || !src) return fail(SMORE_ERR_NULL, "shard_record_sources: NULL pointer");
  shard_record_sources_kernel<<<grid_threads(n), 256, 0, (cudaStream_t)stream>>>(slot, n, src);
  return check_launch("shard_record_sources_kernel");
}

static int shard_reduce_update_impl(float* table, float* m, float* v, const int64_t* uniq, const int32_t* counts,
                                   const int32_t* src, const int32_t* n_unique, size_t capacity,
                                   const float* const* grad_ptrs, const int64_t* ids, const int32_t* list_bounds,
                                   size_t n_ranks, size_t n_plans, const int32_t* plan_caps, size_t width,
                                   double lr, double beta1, double beta2, double eps, int64_t step,
                                   const float* step_scalars, int squeeze, void* stream) {
  if (capacity == 0) return SMORE_OK;
  if (!table || !m || !v || !uniq || !counts || !src || !n_unique || !grad_ptrs || !ids || !list_bounds)
    return fail(SMORE_ERR_NULL, "shard_reduce_update_rows: NULL pointer");
  if (!step_scalars && step < 1) return fail(SMORE_ERR_BAD_SHAPE, "adam step must be >= 1");
  if (width == 0 || (width & 3) || width > 1024 || !aligned16(table) || !aligned16(m) || (!squeeze && !aligned16(v)))
    return fail(SMORE_ERR_BAD_SHAPE, "shard_reduce_update_rows: width must be a multiple of 4 floats, at most 1024");
  ReduceArgs r;
  if (int rc = make_caps(plan_caps, n_plans, &r.caps)) return rc;
  if (n_ranks == 0 || n_ranks * n_plans > (size_t)kMaxLists)
    return fail(SMORE_ERR_BAD_SHAPE, "ranks x plans must be 1..%d", kMaxLists);
  r.counts = counts; r.src = src; r.grad_ptrs = grad_ptrs; r.ids = ids; r.bounds = list_bounds;
  r.n_lists = (int)(n_ranks * n_plans);
  UpdateArgs a;
  a.table = table; a.m = m; a.v = v; a.uniq = uniq; a.g_rows = nullptr; a.n_unique = n_unique; a.width = width;
  set_hyper(a, lr, beta1, beta2, eps, step_scalars ? 1 : step, squeeze);
  a.dyn = step_scalars;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_warps(capacity);
  const size_t w4 = width >> 2;
#define REDUCE(NCH)                                                                \
  if (a.squeeze) shard_reduce_update_kernel<NCH, true><<<grid, 256, 0, st>>>(a, r); \
  else shard_reduce_update_kernel<NCH, false><<<grid, 256, 0, st>>>(a, r)
  if (w4 <= 32) { REDUCE(1); }
  else if (w4 <= 64) { REDUCE(2); }
  else if (w4 <= 128) { REDUCE(4); }
  else { REDUCE(8); }
#undef REDUCE
  return check_launch("shard_reduce_update_kernel");
}

int smore_shard_reduce_update_rows(float* table, float* m, float* v, const int64_t* uniq, const int32_t* counts,
                                   const int32_t* src, const int32_t* n_unique, size_t capacity,
                                   const float* const* grad_ptrs, const int64_t* ids, const int32_t* list_bounds,
                                   size_t n_ranks, size_t n_plans, const int32_t* plan_caps, size_t width,
                                   double lr, double beta1, double beta2, double eps, int64_t step, int squeeze,
                                   void* stream) {
  return shard_reduce_update_impl(table, m, v, uniq, counts, src, n_unique, capacity, grad_ptrs, ids, list_bounds,
                                  n_ranks, n_plans, plan_caps, width, lr, beta1, beta2, eps, step, nullptr, squeeze,
                                  stream);
}

int smore_shard_reduce_update_rows_dev(float* table, float* m, float* v, const int64_t* uniq, const int32_t* counts,
                                       const int32_t* src, const int32_t* n_unique, size_t capacity,
                                       const float* const* grad_ptrs, const int64_t* ids,
                                       const int32_t* list_bounds, size_t n_ranks, size_t n_plans,
                                       const int32_t* plan_caps, size_t width, double lr, double beta1, double beta2,
                                       double eps, const float* step_scalars, int squeeze, void* stream) {
  if (!step_scalars) return fail(SMORE_ERR_NULL, "shard_reduce_update_rows_dev: step_scalars is NULL");
  return shard_reduce_update_impl(table, m, v, uniq, counts, src, n_unique, capacity, grad_ptrs, ids, list_bounds,
                                  n_ranks, n_plans, plan_caps, width, lr, beta1, beta2, eps, 1, step_scalars, squeeze,
                                  stream);
}

}  // extern "C"
