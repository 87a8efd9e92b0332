// Row-sharded entity table over the GPUs of one NVLink / NVSwitch box: peer-memory plumbing and
// the kernels that move rows and row gradients between owners and requesters.
//
// The reference shares its table between GPU processes through CPU shared memory and PCIe staging
// (smore/common/embedding/embed_rw.py:53-134, smore/common/torchext/extlib_cuda.cpp:82-144,
// smore/models/kg_reasoning.py:144-147).  Here rows [g*S, (g+1)*S) of the table and of its Adam
// state live in the HBM of GPU g, and every exchange is a kernel of this file doing plain 128-bit
// loads from peer-mapped memory:
//   fetch_rows_kernel            requester pulls each distinct row of its step once into a local
//                                staging block (forward and backward then run on local memory)
//   shard_find_runs / gather_runs owner finds, in every rank's sorted list of distinct row ids, the
//                                run that lies in its range
//   shard_reduce_update_ring     owner pulls the gradient rows of each of its touched rows from the
//                                ranks that produced them, sums them in a fixed order and applies
//                                Adam to its shard: transfer, reduction and update in one pass
//   owner_* kernels              owner-side scoring: instead of moving candidate rows to the queries
//                                (1.6 KB per pair and direction), the queries go to the rows: every
//                                owner picks the (query, candidate) pairs of all ranks that fall in
//                                its range, scores and differentiates them against its own rows with
//                                the row-stream kernels, and only scores, upstream gradients and
//                                query gradients cross NVLink (a few bytes per pair)
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

// rows_kernels.cu: sorted unique + inverse map; with n_dev != nullptr only the first *n_dev ids count
int unique_rows_impl(const int64_t* idx, size_t n, const int32_t* n_dev, size_t n_table_rows, int64_t* uniq,
                     int32_t* inverse, int32_t* counts, int32_t* n_unique, void* workspace, size_t workspace_bytes,
                     cudaStream_t st);

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

// The refresh with bulk copies: a warp tests 32 consecutive rows of the step's list against the local
// bitmap copy, then its lanes move the marked ones concurrently - lane i owns row slot i in shared
// memory (as in fetch_rows_bulk_kernel) and takes the i-th marked row of the batch.
__global__ void __launch_bounds__(kBulkFetchWarps * 32)
    refresh_rows_bulk_kernel(const float* const* __restrict__ shard_ptrs, const uint32_t* __restrict__ dirty_local,
                             size_t words, size_t rows_per_shard, const int64_t* __restrict__ uniq,
                             const int32_t* __restrict__ n_unique, unsigned row_bytes, int slots_per_warp,
                             unsigned char* __restrict__ staging) {
  extern __shared__ __align__(128) unsigned char fetch_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fetch_smem);
  unsigned char* slots = fetch_smem + kBulkFetchWarps * 32 * sizeof(uint64_t);
  uint64_t* bar = bars + warp * 32 + lane;
  unsigned char* slot = slots + ((size_t)warp * slots_per_warp + lane) * row_bytes;
  const bool owns_slot = lane < slots_per_warp;
  if (owns_slot) bulk::barrier_init(bar, 1);
  bulk::fence_barrier_init();
  __syncthreads();
  const size_t nu = (size_t)max(n_unique[0], 0);
  const size_t warps = (size_t)gridDim.x * kBulkFetchWarps;
  unsigned parity = 0;
  bool gave_up = false;
  for (size_t u0 = ((size_t)blockIdx.x * kBulkFetchWarps + warp) * 32; u0 < nu && !gave_up; u0 += warps * 32) {
    bool marked = false;
    unsigned long long owner = 0, local = 0;
    if (u0 + lane < nu) {
      const size_t id = (size_t)uniq[u0 + lane];
      owner = id / rows_per_shard;
      local = id - owner * rows_per_shard;
      marked = (dirty_local[owner * words + (local >> 5)] >> (local & 31)) & 1u;
    }
    unsigned todo = __ballot_sync(0xffffffffu, marked);
    while (todo) {
      // lane i takes the i-th marked row still to do (if there is one)
      const int take = owns_slot ? (int)__fns(todo, 0, lane + 1) : -1;     // 0xffffffff -> -1: none
      const bool work = owns_slot && take >= 0 && take < 32;
      const int from = work ? take : 0;
      const unsigned long long o = __shfl_sync(0xffffffffu, owner, from), r = __shfl_sync(0xffffffffu, local, from);
      if (work) {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(shard_ptrs[o]) + r * (size_t)row_bytes;
        bulk::barrier_expect(bar, row_bytes);
        bulk::load(slot, src, row_bytes, bar);
      }
      const bool ok = !work || bulk::barrier_wait(bar, parity);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) atomicOr(&g_peer_async_status, 1);
        if (!ok) bulk::barrier_wait(bar, parity);   // let a copy that is still on its way land
        gave_up = true;
        break;
      }
      if (work) {
        bulk::store(staging + (u0 + take) * (size_t)row_bytes, slot, row_bytes);
        bulk::commit_group();
        bulk::wait_group_read<0>();
        parity ^= 1u;
      }
      // drop the rows just taken: the lowest min(slots_per_warp, popc) set bits
      const int taken = min(slots_per_warp, __popc(todo));
      for (int i = 0; i < taken; ++i) todo &= todo - 1;
    }
  }
  bulk::wait_group<0>();
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

// ----------------------------------------------------------------------------------------
// Owner side of the gradient return.
//
// Every rank publishes up to n_plans sorted lists of distinct global row ids with one gradient row
// per id.  Because the lists are sorted and an owner's rows are one contiguous id range, what an
// owner needs from a list is one contiguous RUN of it, found with two binary searches.  The runs of
// all lists are copied, as local row ids, into one compact array (run after run, list order), which
// is then de-duplicated; the compact position of a contribution encodes its list and its index.
// ----------------------------------------------------------------------------------------

struct OwnerRuns {          // device-resident, written by shard_find_runs_kernel
  int lo[kMaxLists];        // first index of the run inside its list
  int start[kMaxLists + 1]; // first compact position of the run; start[n_lists] = total
};

__device__ __forceinline__ int lower_bound_ids(const int64_t* ids, int n, int64_t key) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (ids[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(32)
    shard_find_runs_kernel(const int64_t* const* __restrict__ uniq_ptrs, const int32_t* const* __restrict__ nuniq_ptrs,
                           PlanCaps c, int n_lists, int64_t base, int64_t shard_rows, OwnerRuns* __restrict__ runs,
                           int32_t* __restrict__ total_out, const int32_t* __restrict__ n_prefix, int prefix_cap) {
  // ids already sitting at the front of the compact array (owner-side scoring's pairs): the runs follow them
  const int pre = n_prefix != nullptr ? min(max(n_prefix[0], 0), prefix_cap) : 0;
  const int l = threadIdx.x;
  int lo = 0, len = 0;
  if (l < n_lists) {
    const int cap = c.cap[l % c.n_plans];
    const int count = min(max(nuniq_ptrs[l][0], 0), cap);
    const int64_t* ids = uniq_ptrs[l];
    lo = lower_bound_ids(ids, count, base);
    len = lower_bound_ids(ids, count, base + shard_rows) - lo;
  }
  int inc = len;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (l >= o) inc += t;
  }
  if (l < n_lists) {
    runs->lo[l] = lo;
    runs->start[l] = pre + inc - len;
  }
  const int total = pre + __shfl_sync(0xffffffffu, inc, 31);
  if (l == 0) {
    runs->start[n_lists] = total;
    total_out[0] = total;
  }
}

// list that holds compact position p (runs are in list order; start[] ascends)
__device__ __forceinline__ int list_of_position(const int* start, int n_lists, int p) {
  int l = 0;
  for (int q = 1; q < n_lists; ++q)
    if (start[q] <= p) l = q;
  return l;
}

__global__ void __launch_bounds__(256)
    shard_gather_runs_kernel(const int64_t* const* __restrict__ uniq_ptrs, const OwnerRuns* __restrict__ runs,
                             int n_lists, int64_t base, int64_t* __restrict__ out_ids) {
  __shared__ int s_lo[kMaxLists], s_start[kMaxLists + 1];
  if (threadIdx.x < n_lists) s_lo[threadIdx.x] = runs->lo[threadIdx.x];
  if (threadIdx.x <= n_lists) s_start[threadIdx.x] = runs->start[threadIdx.x];
  __syncthreads();
  const int total = s_start[n_lists];
  for (int p = s_start[0] + blockIdx.x * blockDim.x + threadIdx.x; p < total; p += gridDim.x * blockDim.x) {
    const int l = list_of_position(s_start, n_lists, p);
    out_ids[p] = uniq_ptrs[l][s_lo[l] + (p - s_start[l])] - base;
  }
}

__global__ void __launch_bounds__(256)
    shard_record_sources_kernel(const int32_t* __restrict__ slot, const int32_t* __restrict__ total,
                                int32_t* __restrict__ src) {
  const int n = total[0];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int32_t s = slot[i];
    if (s >= 0) src[s] = i;  // any contributor will do; rows with several are searched for
  }
}

struct ReduceArgs {
  const int32_t* counts;            // contributors per distinct row
  const int32_t* src;               // one contributing compact position per distinct row
  const float* const* grad_ptrs;    // [lists] gradient blocks (peer memory)
  const int64_t* ids;               // compact array of local row ids (runs in list order)
  const OwnerRuns* runs;
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

// A row with several contributors: lane l searches run l of the compact id array (ascending inside
// a run); the contributions are then added in list order, so the sum does not depend on timing.
template <int NCH>
__device__ __forceinline__ void add_contributions(float4 (&g)[NCH], const ReduceArgs& r, const int* s_lo,
                                                  const int* s_start, int64_t row, int lane, int w4) {
  int found = -1;
  if (lane < r.n_lists) {
    int lo = s_start[lane], hi = s_start[lane + 1];
    const int end = hi;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (r.ids[mid] < row) lo = mid + 1; else hi = mid;
    }
    if (lo < end && r.ids[lo] == row) found = s_lo[lane] + (lo - s_start[lane]);
  }
  unsigned hits = __ballot_sync(0xffffffffu, found >= 0);
  while (hits) {
    const int l = __ffs(hits) - 1;
    hits &= hits - 1;
    const int j = __shfl_sync(0xffffffffu, found, l);
    add_row<NCH>(g, reinterpret_cast<const float4*>(r.grad_ptrs[l]) + (size_t)j * w4, lane, w4);
  }
}

template <int NCH, bool ROWWISE>
__device__ __forceinline__ void adam_row(float4 (&g)[NCH], float4 (&p)[NCH], float4 (&m)[NCH], float4 (&v)[NCH],
                                         float4* p4, float4* m4, float4* v4, int64_t row, int lane, int w4,
                                         const UpdateArgs& a) {
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

// Plain form: one warp per row, the gradient row read with ordinary loads.  Kept for rows the ring
// kernel below does not take (row sizes that are no multiple of 16 bytes or too large for its ring).
template <int NCH, bool ROWWISE>
__global__ void __launch_bounds__(256) shard_reduce_update_kernel(UpdateArgs a, ReduceArgs r) {
  __shared__ int s_lo[kMaxLists], s_start[kMaxLists + 1];
  if (threadIdx.x < r.n_lists) s_lo[threadIdx.x] = r.runs->lo[threadIdx.x];
  if (threadIdx.x <= r.n_lists) s_start[threadIdx.x] = r.runs->start[threadIdx.x];
  __syncthreads();
  load_dyn(a);
  const int lane = threadIdx.x & 31;
  const size_t nu = (size_t)max(a.n_unique[0], 0);
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  const int w4 = (int)(a.width >> 2);
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
    if (r.counts[u] == 1) {
      const int pos = r.src[u];
      const int l = list_of_position(s_start, r.n_lists, pos);
      const int j = s_lo[l] + (pos - s_start[l]);
      add_row<NCH>(g, reinterpret_cast<const float4*>(r.grad_ptrs[l]) + (size_t)j * w4, lane, w4);
    } else {
      add_contributions<NCH>(g, r, s_lo, s_start, row, lane, w4);
    }
    adam_row<NCH, ROWWISE>(g, p, m, v, p4, m4, v4, row, lane, w4, a);
  }
}

// Ring form.  The gradient rows cross NVLink; a warp that asks for one row at a time spends most of
// its time waiting for it.  Here every warp owns a ring of `stages` row slots in shared memory and
// one mbarrier per slot; lane 0 keeps `stages` bulk asynchronous copies (peer memory -> slot, one
// instruction per row, untiled, no multicast) in flight ahead of the row the warp is updating, so
// the bytes in flight per SM depend neither on registers nor on how many warps are resident, while
// the local rows (parameters, moments) are read with ordinary loads behind them.  A warp takes rows
// u = w, w + W, w + 2W, ... (W = warps in the grid): consecutive rows of the sorted list come from
// unrelated requesters, so the copies in flight are spread over all peers.  Rows with several
// contributors (a few per cent) are not copied into the ring: they are searched for and read with
// ordinary loads, in list order.  Every wait is bounded; a wait that runs out sets the status word
// (kStatusPeerWait) and the warp stops.
constexpr int kRingWarps = 8;

template <int NCH, bool ROWWISE>
__global__ void __launch_bounds__(kRingWarps * 32, 2)
    shard_reduce_update_ring_kernel(UpdateArgs a, ReduceArgs r, int stages) {
  extern __shared__ __align__(128) unsigned char ring_smem[];
  __shared__ int s_lo[kMaxLists], s_start[kMaxLists + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < r.n_lists) s_lo[threadIdx.x] = r.runs->lo[threadIdx.x];
  if (threadIdx.x <= r.n_lists) s_start[threadIdx.x] = r.runs->start[threadIdx.x];
  const int w4 = (int)(a.width >> 2);
  const unsigned row_bytes = (unsigned)w4 * 16u;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring_smem) + warp * stages;
  const size_t ring_off = ((size_t)kRingWarps * stages * sizeof(uint64_t) + 127) & ~(size_t)127;
  unsigned char* ring = ring_smem + ring_off + (size_t)warp * stages * row_bytes;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) bulk::barrier_init(bars + s, 1);
    bulk::fence_barrier_init();
  }
  __syncthreads();
  load_dyn(a);
  const long long nu = max(a.n_unique[0], 0);
  const long long W = (long long)gridDim.x * kRingWarps;
  const long long w = (long long)blockIdx.x * kRingWarps + warp;
  const int n_k = nu > w ? (int)((nu - w + W - 1) / W) : 0;   // rows of this warp

  // per-lane scalars of a batch of 32 of the warp's rows: local row, where its (single) gradient row
  // lives, or nullptr when the row has several contributors
  struct Meta {
    long long row;
    const unsigned char* src;
  };
  auto load_meta = [&](int first_k) {
    Meta mt{0, nullptr};
    const int k = first_k + lane;
    if (k < n_k) {
      const long long u = w + (long long)k * W;
      mt.row = a.uniq[u];
      if (r.counts[u] == 1) {
        const int pos = r.src[u];
        const int l = list_of_position(s_start, r.n_lists, pos);
        const int j = s_lo[l] + (pos - s_start[l]);
        mt.src = reinterpret_cast<const unsigned char*>(r.grad_ptrs[l]) + (size_t)j * row_bytes;
      }
    }
    return mt;
  };
  Meta cur = load_meta(0), nxt = cur;
  unsigned phase_bits = 0;   // parity each slot's barrier will complete next
  unsigned armed_bits = 0;   // slots with a copy in flight
  const int ahead = min(stages, n_k);
  for (int k = 0; k < ahead; ++k) {
    const unsigned char* src = reinterpret_cast<const unsigned char*>(
        __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(cur.src), k));
    if (src != nullptr) {
      if (lane == 0) {
        bulk::barrier_expect(bars + k, row_bytes);
        bulk::load(ring + (size_t)k * row_bytes, src, row_bytes, bars + k);
      }
      armed_bits |= 1u << k;
    }
  }
  int slot = 0;
  for (int k = 0; k < n_k; ++k) {
    const int tl = k & 31;
    if (tl == 0) nxt = load_meta(k + 32);
    const long long row = __shfl_sync(0xffffffffu, cur.row, tl);
    const bool single = (armed_bits >> slot) & 1u;
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
    if (single) {
      bool ok = bulk::barrier_wait(bars + slot, (phase_bits >> slot) & 1u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        // give up: flag it, let the other copies in flight land (bounded waits), stop
        if (lane == 0) atomicOr(&g_peer_async_status, 1);
        armed_bits &= ~(1u << slot);
        for (int s2 = 0; s2 < stages; ++s2)
          if ((armed_bits >> s2) & 1u) bulk::barrier_wait(bars + s2, (phase_bits >> s2) & 1u);
        break;
      }
      phase_bits ^= 1u << slot;
      armed_bits &= ~(1u << slot);
      const float4* row4 = reinterpret_cast<const float4*>(ring + (size_t)slot * row_bytes);
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int d = lane + 32 * j;
        if (d < w4) g[j] = row4[d];
      }
    } else {
      add_contributions<NCH>(g, r, s_lo, s_start, row, lane, w4);
    }
    // every lane has taken its pieces of the slot: it may be refilled with the row `stages` ahead
    __syncwarp();
    const int kn = k + stages;
    if (kn < n_k) {
      const unsigned long long nsrc_bits = __shfl_sync(
          0xffffffffu, reinterpret_cast<unsigned long long>((kn >> 5) == (k >> 5) ? cur.src : nxt.src), kn & 31);
      const unsigned char* nsrc = reinterpret_cast<const unsigned char*>(nsrc_bits);
      if (nsrc != nullptr) {
        if (lane == 0) {
          bulk::barrier_expect(bars + slot, row_bytes);
          bulk::load(ring + (size_t)slot * row_bytes, nsrc, row_bytes, bars + slot);
        }
        armed_bits |= 1u << slot;
      }
    }
    adam_row<NCH, ROWWISE>(g, p, m, v, p4, m4, v4, row, lane, w4, a);
    if (tl == 31) cur = nxt;
    if (++slot == stages) slot = 0;
  }
}

// ----------------------------------------------------------------------------------------
// Owner-side scoring.  Every rank publishes, in peer-visible memory, the candidate row ids of its
// queries ([n_queries, K] global ids), the queries, and a descriptor {n_queries, K}.  The owner
//   1. selects the pairs whose row lies in its range: per (rank, query) one contiguous segment of
//      the compact arrays rows[] (local row ids) and positions[] (query * K + k on the requester),
//      in increasing k (owner_select_pairs_kernel);
//   2. copies all queries into one local array indexed by rank * max_queries + query;
//   3. runs the ragged row-stream kernels over the segments (dist_kernels.cu), which write each
//      result to / read each upstream gradient from its position in the requester's arrays;
//   4. leaves its partial query gradients for the requesters to sum (owner_sum_query_grads_kernel).
// ----------------------------------------------------------------------------------------

// 128 threads: a CTA spends its time waiting for one NVLink round trip, so the SM should hold many
// of them (16 at this size)
constexpr int kSelectThreads = 128;

// A rank's descriptor {n_queries, K, branches} is checked against the (n_queries, K, branches) this
// owner's kernels were launched for - every rank of a step runs the same scoring op - and a rank that
// says otherwise is left out (its scores read NaN, the capacity bit is set).  The host has checked that
// the expected sizes fit the buffers.
__device__ __forceinline__ bool owner_desc(const int32_t* desc, int want_nq, int want_k, int want_branches) {
  const int q = desc[0], k = desc[1], br = desc[2];
  if (q == want_nq && k == want_k && br == want_branches) return true;
  if (q != 0 || k != 0) atomicOr(&g_peer_async_status, kStatusCapacity);   // (all zero: the rank published nothing)
  return false;
}

__global__ void __launch_bounds__(kSelectThreads)
    owner_select_pairs_kernel(const int64_t* const* __restrict__ pair_id_ptrs, const int32_t* const* __restrict__ desc_ptrs,
                              int max_queries, int want_nq, int want_k, int branches, int64_t base,
                              int64_t shard_rows, int capacity, int64_t* __restrict__ rows,
                              int32_t* __restrict__ positions, int2* __restrict__ segments,
                              int32_t* __restrict__ n_selected) {
  __shared__ int s_warp[kSelectThreads / 32];
  __shared__ int s_pos0;
  // Every owner runs this grid at the same time: owner o starts with rank o's ids, then o + 1, ... so
  // that at any moment the owners read from different peers instead of all from the same one.
  const int r = (int)((blockIdx.y + (unsigned)(base / shard_rows)) % gridDim.y);
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seg = r * max_queries + b;
  const int K = want_k;
  if (b >= want_nq || K == 0) {            // a segment slot no rank uses in this step: no peer is asked
    if (tid == 0) segments[seg] = make_int2(0, 0);
    return;
  }
  // The ids of query b under the expected layout are requested together with the descriptor that
  // confirms the layout (both come over NVLink: one round trip instead of two).
  const int64_t* ids = pair_id_ptrs[r] + (size_t)b * K;
  // pass 1: how many of the query's candidates live here.  The ids come over NVLink: the first
  // kSelectCache per thread stay in registers for the second pass.
  constexpr int kSelectCache = 8;
  int64_t cache[kSelectCache];
  int cnt = 0;
#pragma unroll
  for (int i = 0; i < kSelectCache; ++i) {
    const int k = tid + i * kSelectThreads;
    cache[i] = k < K ? ids[k] - base : -1;
  }
  if (!owner_desc(desc_ptrs[r], want_nq, want_k, branches)) {      // (the same answer in every thread)
    if (tid == 0) segments[seg] = make_int2(0, 0);
    return;
  }
#pragma unroll
  for (int i = 0; i < kSelectCache; ++i) cnt += (cache[i] >= 0 && cache[i] < shard_rows) ? 1 : 0;
  for (int k = tid + kSelectCache * kSelectThreads; k < K; k += kSelectThreads) {
    const int64_t id = ids[k] - base;
    cnt += (id >= 0 && id < shard_rows) ? 1 : 0;
  }
  cnt = __reduce_add_sync(0xffffffffu, cnt);
  if (lane == 0) s_warp[warp] = cnt;
  __syncthreads();
  if (tid == 0) {
    int total = 0;
    for (int w = 0; w < kSelectThreads / 32; ++w) total += s_warp[w];
    int pos0 = total ? atomicAdd(n_selected, total) : 0;
    if (pos0 + total > capacity) {   // the compact arrays are full: drop the segment and say so
      atomicOr(&g_peer_async_status, kStatusCapacity);
      pos0 = -1;
      total = 0;
    }
    segments[seg] = make_int2(max(pos0, 0), total);
    s_pos0 = pos0;
  }
  __syncthreads();
  int running = s_pos0;
  if (running < 0) return;
  // pass 2: the same scan, writing in increasing k
#pragma unroll
  for (int i = 0; i < kSelectCache; ++i) {
    const int k0 = i * kSelectThreads;
    if (k0 >= K) break;
    const int64_t id = cache[i];
    const bool mine = id >= 0 && id < shard_rows;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    __syncthreads();   // s_warp of the previous chunk has been read
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, chunk = 0;
    for (int w = 0; w < kSelectThreads / 32; ++w) {
      before += w < warp ? s_warp[w] : 0;
      chunk += s_warp[w];
    }
    if (mine) {
      const int p = running + before + __popc(ballot & ((1u << lane) - 1u));
      rows[p] = id;
      positions[p] = b * branches * K + k0 + tid;
    }
    running += chunk;
  }
  for (int k0 = kSelectCache * kSelectThreads; k0 < K; k0 += kSelectThreads) {
    const int k = k0 + tid;
    int64_t id = -1;
    if (k < K) id = ids[k] - base;
    const bool mine = id >= 0 && id < shard_rows;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    __syncthreads();
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, chunk = 0;
    for (int w = 0; w < kSelectThreads / 32; ++w) {
      before += w < warp ? s_warp[w] : 0;
      chunk += s_warp[w];
    }
    if (mine) {
      const int p = running + before + __popc(ballot & ((1u << lane) - 1u));
      rows[p] = id;
      positions[p] = b * branches * K + k;
    }
    running += chunk;
  }
}

__global__ void __launch_bounds__(256)
    owner_gather_queries_kernel(const float* const* __restrict__ first_ptrs, const float* const* __restrict__ second_ptrs,
                                const int32_t* const* __restrict__ desc_ptrs, int max_queries, int want_nq, int want_k,
                                int branches, int dim4, int first_rank, float4* __restrict__ first_all,
                                float4* __restrict__ second_all) {
  const int r = (int)((blockIdx.y + (unsigned)first_rank) % gridDim.y);   // (owners start at different peers)
  if (!owner_desc(desc_ptrs[r], want_nq, want_k, branches)) return;
  const size_t total = (size_t)want_nq * branches * dim4, base = (size_t)r * max_queries * dim4;
  const float4* f = reinterpret_cast<const float4*>(first_ptrs[r]);
  const float4* s = second_all != nullptr ? reinterpret_cast<const float4*>(second_ptrs[r]) : nullptr;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    first_all[base + i] = f[i];
    if (s != nullptr) second_all[base + i] = s[i];
  }
}

// g_rows[slot[p]] (+)= the gradient row that list position p names, for the compact positions of the
// lists' runs (the positions after the selected pairs)
__global__ void __launch_bounds__(256)
    owner_add_list_rows_kernel(const float* const* __restrict__ grad_ptrs, const OwnerRuns* __restrict__ runs, int n_lists,
                               const int32_t* __restrict__ slot, const int32_t* __restrict__ counts,
                               float4* __restrict__ g_rows, int w4) {
  __shared__ int s_lo[kMaxLists], s_start[kMaxLists + 1];
  if (threadIdx.x < n_lists) s_lo[threadIdx.x] = runs->lo[threadIdx.x];
  if (threadIdx.x <= n_lists) s_start[threadIdx.x] = runs->start[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int first = s_start[0], total = s_start[n_lists];
  const int warps = gridDim.x * (blockDim.x >> 5);
  for (int p = first + blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < total; p += warps) {
    const int32_t s = slot[p];
    if (s < 0) continue;
    const int l = list_of_position(s_start, n_lists, p);
    const float4* src = reinterpret_cast<const float4*>(grad_ptrs[l]) + (size_t)(s_lo[l] + (p - s_start[l])) * w4;
    float4* dst = g_rows + (size_t)s * w4;
    const bool single = counts[s] == 1;
    for (int d = lane; d < w4; d += 32) {
      const float4 g = src[d];
      if (single) dst[d] = g;
      else atomicAdd(dst + d, g);
    }
  }
}

__global__ void __launch_bounds__(256)
    owner_sum_query_grads_kernel(const float* const* __restrict__ part_ptrs, int n_ranks, size_t offset4, size_t total4,
                                 float4* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int o = 0; o < n_ranks; ++o) {     // owner order: the same sum on every run
      const float4 v = reinterpret_cast<const float4*>(part_ptrs[o])[offset4 + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    out[i] = acc;
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
  const size_t row_bytes = width * sizeof(float);
  if (row_bytes <= 20 * 1024) {
    // marked rows move with bulk copies, several per warp at a time (about 20 KB of slots per warp)
    const int slots = (int)std::min<size_t>(32, std::max<size_t>(1, 20 * 1024 / row_bytes));
    const size_t smem = kBulkFetchWarps * 32 * sizeof(uint64_t) + (size_t)kBulkFetchWarps * slots * row_bytes;
    if (int rc = allow_large_smem(refresh_rows_bulk_kernel, 48 * 1024, false)) return rc;
    const size_t want = (capacity + (size_t)kBulkFetchWarps * 32 - 1) / ((size_t)kBulkFetchWarps * 32);
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>(want, (size_t)sm_count() * 8));
    refresh_rows_bulk_kernel<<<grid, kBulkFetchWarps * 32, smem, st>>>(
        shard_ptrs, bitmap_scratch, words, rows_per_shard, uniq, n_unique, (unsigned)row_bytes, slots,
        reinterpret_cast<unsigned char*>(staging));
    return check_launch("refresh_rows kernels", 2);
  }
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

size_t smore_shard_owner_plan_workspace_bytes(size_t shard_rows) {
  return 256 + smore_unique_rows_workspace_bytes(shard_rows ? shard_rows : 1);
}

static int owner_plan_impl(const int64_t* const* uniq_ptrs, const int32_t* const* nuniq_ptrs, size_t n_ranks,
                           size_t n_plans, const int32_t* plan_caps, int64_t base, size_t shard_rows,
                           size_t capacity, int64_t* ids, int32_t* runs, int64_t* uniq, int32_t* slot,
                           int32_t* counts, int32_t* src, int32_t* n_unique, uint32_t* dirty, void* workspace,
                           size_t workspace_bytes, const int32_t* n_prefix, size_t prefix_capacity, void* stream) {
  if (!uniq_ptrs || !nuniq_ptrs || !ids || !runs || !uniq || !slot || !counts || !n_unique || !workspace)
    return fail(SMORE_ERR_NULL, "shard_owner_plan: NULL pointer");
  PlanCaps c;
  if (int rc = make_caps(plan_caps, n_plans, &c)) return rc;
  if (n_ranks == 0 || n_ranks * n_plans > (size_t)kMaxLists)
    return fail(SMORE_ERR_BAD_SHAPE, "ranks x plans must be 1..%d", kMaxLists);
  if (shard_rows == 0) return fail(SMORE_ERR_BAD_SHAPE, "shard_owner_plan: shard_rows is 0");
  const size_t worst = prefix_capacity + n_ranks * (size_t)c.prefix[kMaxPlans];
  if (worst > (size_t)INT_MAX) return fail(SMORE_ERR_TOO_LARGE, "shard_owner_plan: more than 2^31-1 positions");
  if (capacity < worst)
    return fail(SMORE_ERR_BAD_SHAPE, "shard_owner_plan: capacity %zu, but the lists can hold %zu ids", capacity, worst);
  if (workspace_bytes < smore_shard_owner_plan_workspace_bytes(shard_rows) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(SMORE_ERR_WORKSPACE, "shard_owner_plan: workspace too small or not 256-byte aligned");
  static_assert(sizeof(OwnerRuns) <= SMORE_SHARD_RUNS_INTS * sizeof(int32_t), "runs buffer size");
  cudaStream_t st = (cudaStream_t)stream;
  const int n_lists = (int)(n_ranks * n_plans);
  OwnerRuns* r = reinterpret_cast<OwnerRuns*>(runs);
  int32_t* total = reinterpret_cast<int32_t*>(workspace);            // device count of collected ids
  void* uws = static_cast<unsigned char*>(workspace) + 256;
  shard_find_runs_kernel<<<1, 32, 0, st>>>(uniq_ptrs, nuniq_ptrs, c, n_lists, base, (int64_t)shard_rows, r, total,
                                           n_prefix, (int)prefix_capacity);
  // the collected ids are expected to be about 1 / n_ranks of the worst case; the kernels below loop
  // over the device-side total, so the grids only have to be large enough to fill the GPU
  const size_t expect = std::max<size_t>(worst / n_ranks, 1);
  shard_gather_runs_kernel<<<grid_threads(expect), 256, 0, st>>>(uniq_ptrs, r, n_lists, base, ids);
  count_launches(2);
  if (int rc = unique_rows_impl(ids, worst, total, shard_rows, uniq, slot, counts, n_unique, uws,
                                workspace_bytes - 256, st))
    return rc;
  if (src != nullptr) {
    shard_record_sources_kernel<<<grid_threads(expect), 256, 0, st>>>(slot, total, src);
    count_launches(1);
  }
  if (dirty != nullptr) {
    // publish which rows this step updates (readers: the next step's refresh on every rank)
    if (cudaMemsetAsync(dirty, 0, ((shard_rows + 31) / 32) * sizeof(uint32_t), st) != cudaSuccess)
      return fail(SMORE_ERR_CUDA, "shard_owner_plan: cudaMemsetAsync failed");
    shard_mark_dirty_kernel<<<grid_threads(expect), 256, 0, st>>>(uniq, n_unique, dirty);
    count_launches(1);
  }
  return check_launch("shard_owner_plan kernels", 0);
}

int smore_shard_owner_plan(const int64_t* const* uniq_ptrs, const int32_t* const* nuniq_ptrs, size_t n_ranks,
                           size_t n_plans, const int32_t* plan_caps, int64_t base, size_t shard_rows,
                           size_t capacity, int64_t* ids, int32_t* runs, int64_t* uniq, int32_t* slot,
                           int32_t* counts, int32_t* src, int32_t* n_unique, uint32_t* dirty, void* workspace,
                           size_t workspace_bytes, void* stream) {
  if (!src) return fail(SMORE_ERR_NULL, "shard_owner_plan: NULL pointer");
  return owner_plan_impl(uniq_ptrs, nuniq_ptrs, n_ranks, n_plans, plan_caps, base, shard_rows, capacity, ids, runs, uniq,
                         slot, counts, src, n_unique, dirty, workspace, workspace_bytes, nullptr, 0, stream);
}

int smore_owner_plan(const int64_t* const* uniq_ptrs, const int32_t* const* nuniq_ptrs, size_t n_ranks, size_t n_plans,
                     const int32_t* plan_caps, int64_t base, size_t shard_rows, size_t capacity, int64_t* ids,
                     int32_t* runs, int64_t* uniq, int32_t* slot, int32_t* counts, int32_t* n_unique, uint32_t* dirty,
                     void* workspace, size_t workspace_bytes, const int32_t* n_selected, size_t pair_capacity,
                     void* stream) {
  if (!n_selected) return fail(SMORE_ERR_NULL, "owner_plan: NULL pointer");
  return owner_plan_impl(uniq_ptrs, nuniq_ptrs, n_ranks, n_plans, plan_caps, base, shard_rows, capacity, ids, runs, uniq,
                         slot, counts, nullptr, n_unique, dirty, workspace, workspace_bytes, n_selected, pair_capacity,
                         stream);
}

static int check_owner_sizes(const char* what, size_t n_ranks, size_t max_queries) {
  if (n_ranks == 0 || n_ranks > (size_t)kMaxLists || max_queries == 0 || max_queries > 65535u * 64u ||
      n_ranks * max_queries > (size_t)INT_MAX)
    return fail(SMORE_ERR_BAD_SHAPE, "%s: 1..%d ranks, 1..%u queries per rank", what, kMaxLists, 65535u * 64u);
  return SMORE_OK;
}

static int check_owner_op(const char* what, size_t max_queries, size_t pairs_capacity, size_t n_queries,
                          size_t rows_per_query, size_t branches) {
  if (branches == 0 || branches > 2 || n_queries * branches > max_queries || rows_per_query > (size_t)INT_MAX ||
      n_queries * branches * rows_per_query > pairs_capacity || pairs_capacity > (size_t)INT_MAX)
    return fail(SMORE_ERR_BAD_SHAPE, "%s: %zu queries x %zu branches x %zu rows do not fit %zu query rows / %zu pairs",
                what, n_queries, branches, rows_per_query, max_queries, pairs_capacity);
  return SMORE_OK;
}

int smore_owner_select_pairs(const int64_t* const* pair_id_ptrs, const int32_t* const* desc_ptrs, size_t n_ranks,
                             size_t max_queries, size_t pairs_capacity, size_t n_queries, size_t rows_per_query,
                             size_t branches, int64_t base, size_t shard_rows, size_t capacity, int64_t* rows,
                             int32_t* positions, int32_t* segments, int32_t* n_selected, void* stream) {
  if (!pair_id_ptrs || !desc_ptrs || !rows || !positions || !segments || !n_selected)
    return fail(SMORE_ERR_NULL, "owner_select_pairs: NULL pointer");
  if (int rc = check_owner_sizes("owner_select_pairs", n_ranks, max_queries)) return rc;
  if (int rc = check_owner_op("owner_select_pairs", max_queries, pairs_capacity, n_queries, rows_per_query, branches))
    return rc;
  if (capacity > (size_t)INT_MAX || shard_rows == 0)
    return fail(SMORE_ERR_BAD_SHAPE, "owner_select_pairs: capacity must fit 31 bits, shard_rows > 0");
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(n_selected, 0, 2 * sizeof(int32_t), st) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "owner_select_pairs: cudaMemsetAsync failed");
  dim3 grid((unsigned)max_queries, (unsigned)n_ranks);
  owner_select_pairs_kernel<<<grid, kSelectThreads, 0, st>>>(pair_id_ptrs, desc_ptrs, (int)max_queries, (int)n_queries,
                                                             (int)rows_per_query, (int)branches, base,
                                                             (int64_t)shard_rows, (int)capacity, rows, positions,
                                                             reinterpret_cast<int2*>(segments), n_selected);
  return check_launch("owner_select_pairs_kernel");
}

int smore_owner_gather_queries(const float* const* first_ptrs, const float* const* second_ptrs,
                               const int32_t* const* desc_ptrs, size_t n_ranks, size_t max_queries,
                               size_t pairs_capacity, size_t n_queries, size_t rows_per_query, size_t branches,
                               size_t dim, size_t first_rank, float* first_all, float* second_all, void* stream) {
  if (!first_ptrs || !desc_ptrs || !first_all || (second_all && !second_ptrs))
    return fail(SMORE_ERR_NULL, "owner_gather_queries: NULL pointer");
  if (int rc = check_owner_sizes("owner_gather_queries", n_ranks, max_queries)) return rc;
  if (int rc = check_owner_op("owner_gather_queries", max_queries, pairs_capacity, n_queries, rows_per_query, branches))
    return rc;
  if (dim == 0 || (dim & 3) || !aligned16(first_all) || (second_all && !aligned16(second_all)))
    return fail(SMORE_ERR_BAD_SHAPE, "owner_gather_queries: dim must be a multiple of 4, buffers 16-byte aligned");
  dim3 grid((unsigned)std::min<size_t>((max_queries * (dim >> 2) + 255) / 256, (size_t)sm_count() * 4), (unsigned)n_ranks);
  owner_gather_queries_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      first_ptrs, second_ptrs, desc_ptrs, (int)max_queries, (int)n_queries, (int)rows_per_query, (int)branches,
      (int)(dim >> 2), (int)(first_rank % n_ranks), reinterpret_cast<float4*>(first_all),
      reinterpret_cast<float4*>(second_all));
  return check_launch("owner_gather_queries_kernel");
}

int smore_owner_add_list_rows(const float* const* grad_ptrs, const int32_t* runs, size_t n_lists, const int32_t* slot,
                              const int32_t* counts, float* g_rows, size_t width, size_t expect, void* stream) {
  if (!grad_ptrs || !runs || !slot || !counts || !g_rows) return fail(SMORE_ERR_NULL, "owner_add_list_rows: NULL pointer");
  if (n_lists == 0 || n_lists > (size_t)kMaxLists) return fail(SMORE_ERR_BAD_SHAPE, "ranks x plans must be 1..%d", kMaxLists);
  if (width == 0 || (width & 3) || !aligned16(g_rows))
    return fail(SMORE_ERR_BAD_SHAPE, "owner_add_list_rows: width must be a multiple of 4 floats");
  owner_add_list_rows_kernel<<<grid_warps(std::max<size_t>(expect, 1)), 256, 0, (cudaStream_t)stream>>>(
      grad_ptrs, reinterpret_cast<const OwnerRuns*>(runs), (int)n_lists, slot, counts, reinterpret_cast<float4*>(g_rows),
      (int)(width >> 2));
  return check_launch("owner_add_list_rows_kernel");
}

int smore_owner_sum_query_grads(const float* const* part_ptrs, size_t n_ranks, size_t my_rank, size_t max_queries,
                                size_t n_queries, size_t dim, float* out, void* stream) {
  if (!part_ptrs || !out) return fail(SMORE_ERR_NULL, "owner_sum_query_grads: NULL pointer");
  if (int rc = check_owner_sizes("owner_sum_query_grads", n_ranks, max_queries)) return rc;
  if (my_rank >= n_ranks || n_queries > max_queries || dim == 0 || (dim & 3) || !aligned16(out))
    return fail(SMORE_ERR_BAD_SHAPE, "owner_sum_query_grads: bad sizes");
  if (n_queries == 0) return SMORE_OK;
  const size_t dim4 = dim >> 2, total4 = n_queries * dim4;
  owner_sum_query_grads_kernel<<<grid_threads(total4), 256, 0, (cudaStream_t)stream>>>(
      part_ptrs, (int)n_ranks, my_rank * max_queries * dim4, total4, reinterpret_cast<float4*>(out));
  return check_launch("owner_sum_query_grads_kernel");
}

static int shard_reduce_update_impl(float* table, float* m, float* v, const int64_t* uniq, const int32_t* counts,
                                   const int32_t* src, const int32_t* n_unique, size_t capacity,
                                   const float* const* grad_ptrs, const int64_t* ids, const int32_t* runs,
                                   size_t n_lists, size_t width, double lr, double beta1, double beta2, double eps,
                                   int64_t step, const float* step_scalars, int squeeze, void* stream) {
  if (capacity == 0) return SMORE_OK;
  if (!table || !m || !v || !uniq || !counts || !src || !n_unique || !grad_ptrs || !ids || !runs)
    return fail(SMORE_ERR_NULL, "shard_reduce_update_rows: NULL pointer");
  if (!step_scalars && step < 1) return fail(SMORE_ERR_BAD_SHAPE, "adam step must be >= 1");
  if (width == 0 || (width & 3) || width > 1024 || !aligned16(table) || !aligned16(m) || (!squeeze && !aligned16(v)))
    return fail(SMORE_ERR_BAD_SHAPE, "shard_reduce_update_rows: width must be a multiple of 4 floats, at most 1024");
  if (n_lists == 0 || n_lists > (size_t)kMaxLists)
    return fail(SMORE_ERR_BAD_SHAPE, "ranks x plans must be 1..%d", kMaxLists);
  ReduceArgs r;
  r.counts = counts; r.src = src; r.grad_ptrs = grad_ptrs; r.ids = ids;
  r.runs = reinterpret_cast<const OwnerRuns*>(runs);
  r.n_lists = (int)n_lists;
  UpdateArgs a;
  a.table = table; a.m = m; a.v = v; a.uniq = uniq; a.g_rows = nullptr; a.n_unique = n_unique; a.width = width;
  set_hyper(a, lr, beta1, beta2, eps, step_scalars ? 1 : step, squeeze);
  a.dyn = step_scalars;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t w4 = width >> 2;
  // the ring form: 2..8 row slots per warp, about 6 KB of remote rows in flight per warp
  const size_t row_bytes = width * sizeof(float);
  const int stages = (int)std::min<size_t>(8, std::max<size_t>(2, 6400 / row_bytes));
  const size_t ring_smem = (((size_t)kRingWarps * stages * sizeof(uint64_t) + 127) & ~(size_t)127) +
                           (size_t)kRingWarps * stages * row_bytes;
  if (w4 > 32 && ring_smem <= 100 * 1024) {
    const int grid = (int)std::max<size_t>(1, std::min<size_t>((capacity + kRingWarps - 1) / kRingWarps,
                                                               (size_t)sm_count() * 2));
#define RING(NCH)                                                                                            \
  {                                                                                                          \
    auto kern = a.squeeze ? shard_reduce_update_ring_kernel<NCH, true> : shard_reduce_update_ring_kernel<NCH, false>; \
    if (int rc = allow_large_smem(kern, 100 * 1024)) return rc;                                              \
    kern<<<grid, kRingWarps * 32, ring_smem, st>>>(a, r, stages);                                            \
  }
    if (w4 <= 64) RING(2)
    else if (w4 <= 128) RING(4)
    else RING(8)
#undef RING
    return check_launch("shard_reduce_update_ring_kernel");
  }
  const int grid = grid_warps(capacity);
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
                                   const float* const* grad_ptrs, const int64_t* ids, const int32_t* runs,
                                   size_t n_lists, size_t width, double lr, double beta1, double beta2, double eps,
                                   int64_t step, int squeeze, void* stream) {
  return shard_reduce_update_impl(table, m, v, uniq, counts, src, n_unique, capacity, grad_ptrs, ids, runs, n_lists,
                                  width, lr, beta1, beta2, eps, step, nullptr, squeeze, stream);
}

int smore_shard_reduce_update_rows_dev(float* table, float* m, float* v, const int64_t* uniq, const int32_t* counts,
                                       const int32_t* src, const int32_t* n_unique, size_t capacity,
                                       const float* const* grad_ptrs, const int64_t* ids, const int32_t* runs,
                                       size_t n_lists, size_t width, double lr, double beta1, double beta2,
                                       double eps, const float* step_scalars, int squeeze, void* stream) {
  if (!step_scalars) return fail(SMORE_ERR_NULL, "shard_reduce_update_rows_dev: step_scalars is NULL");
  return shard_reduce_update_impl(table, m, v, uniq, counts, src, n_unique, capacity, grad_ptrs, ids, runs, n_lists,
                                  width, lr, beta1, beta2, eps, 1, step_scalars, squeeze, stream);
}

}  // extern "C"
