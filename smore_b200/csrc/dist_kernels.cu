// Distance-op kernels for sm_100a and their C entry points.
//
// Two kernel families:
//   * "cell" kernels — any broadcast combination the op contract allows, any dim, fp32 or fp64.
//     Forward: one warp per output cell.  Backward: one thread per gradient element that walks
//     the cells using it in a fixed order (deterministic, coalesced over the embedding dim).
//   * "row-stream" kernels — the training shape in which every query owns its own candidate
//     rows (entity [B, K, W] or table + idx[B, K]; query [B, 1, dim]).  A CTA keeps one query
//     in registers and streams a block of that query's candidate rows with 128-bit loads,
//     several rows in flight per warp; backward produces the row gradients and the query
//     gradient in the same pass.  This is the HBM-bound hot path.
//
// Replaces smore/common/torchext/common_kernel.h:33-145 (the three reference kernels and their
// launchers) and the dispatch of smore/common/torchext/ext_cuda_kernel.cu:25-77.
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "bulk_copy.cuh"
#include "dist_terms.cuh"
#include "rank_common.cuh"
#include "shared_kernels.cuh"
#include "update_math.cuh"

namespace smore {

// ----------------------------------------------------------------------------------------
// cell kernels
// ----------------------------------------------------------------------------------------

template <typename T>
struct CellArgs {
  const T* ent;        // [be*ne, mul*dim] or table when idx != nullptr
  const int64_t* idx;  // nullable: row ids into `ent`
  const T* first;      // [bc*nc, dim]
  const T* second;     // [bc*nc, dim] (== first for single-operand distances)
  size_t bsize, num, be, ne, bc, nc, dim;
  long long n_rows;    // rows of `ent` when idx != nullptr (0: ids are not checked)
};

template <typename T, class Term>
__global__ void __launch_bounds__(256) cell_forward_kernel(CellArgs<T> a, T* __restrict__ dst0,
                                                           T* __restrict__ dst1) {
  const int lane = threadIdx.x & 31;
  const size_t warps_per_grid = (size_t)gridDim.x * (blockDim.x >> 5);
  const size_t cells = a.bsize * a.num;
  for (size_t cell = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); cell < cells;
       cell += warps_per_grid) {
    const size_t i = cell / a.num, j = cell - i * a.num;
    size_t row = (i % a.be) * a.ne + (j % a.ne);
    bool bad = false;
    if (a.idx) {
      const long long r = checked_row_id(a.idx, row, a.n_rows, &g_async_status);
      bad = r < 0;
      row = bad ? 0 : (size_t)r;
    }
    const T* pe = a.ent + row * a.dim * Term::kMul;
    const size_t qrow = (i % a.bc) * a.nc + (j % a.nc);
    const T* p0 = a.first + qrow * a.dim;
    const T* p1 = a.second + qrow * a.dim;
    T acc[Term::kNOut];
#pragma unroll
    for (int o = 0; o < Term::kNOut; ++o) acc[o] = T(0);
    for (size_t d = lane; d < a.dim; d += kWarp) {
      const T e0 = pe[d];
      const T e1 = Term::kMul == 2 ? pe[d + a.dim] : T(0);
      Term::fwd(e0, e1, p0[d], p1[d], acc);
    }
#pragma unroll
    for (int o = 0; o < Term::kNOut; ++o) {
#pragma unroll
      for (int m = kWarp / 2; m > 0; m >>= 1) acc[o] += __shfl_xor_sync(0xffffffffu, acc[o], m);
    }
    if (lane == 0) {
      dst0[cell] = bad ? T(NAN) : acc[0];
      if (Term::kNOut == 2) dst1[cell] = bad ? T(NAN) : acc[Term::kNOut - 1];
    }
  }
}

// One thread per (entity position, d).  With slot == nullptr the result is stored to
// g_ent[position]; otherwise it goes to g_rows[slot[position]] (store when that slot has a
// single contributor in the whole step, atomic otherwise).
template <typename T, class Term>
__global__ void __launch_bounds__(256)
    cell_backward_ent_kernel(CellArgs<T> a, const T* __restrict__ gout0, const T* __restrict__ gout1,
                             T* __restrict__ g_ent, const int32_t* __restrict__ slot,
                             const int32_t* __restrict__ slot_count, T* __restrict__ g_rows) {
  const size_t total = a.be * a.ne * a.dim;
  const size_t nji = a.bsize / a.be, njj = a.num / a.ne;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (size_t)gridDim.x * blockDim.x) {
    const size_t pos = t / a.dim, d = t - pos * a.dim;
    const size_t r0 = pos / a.ne, r1 = pos - r0 * a.ne;
    size_t row = pos;
    if (a.idx) {
      const long long r = checked_row_id(a.idx, pos, a.n_rows, &g_async_status);
      if (r < 0) continue;   // no gradient from (or for) a row that does not exist
      row = (size_t)r;
    }
    const T* pe = a.ent + row * a.dim * Term::kMul;
    const T e0 = pe[d];
    const T e1 = Term::kMul == 2 ? pe[d + a.dim] : T(0);
    T ge0 = T(0), ge1 = T(0), t0 = T(0), t1 = T(0);
    for (size_t ji = 0; ji < nji; ++ji) {
      const size_t i = ji * a.be + r0;
      for (size_t jj = 0; jj < njj; ++jj) {
        const size_t j = jj * a.ne + r1;
        const size_t qrow = (i % a.bc) * a.nc + (j % a.nc);
        T g[Term::kNOut];
        g[0] = gout0[i * a.num + j];
        if (Term::kNOut == 2) g[Term::kNOut - 1] = gout1[i * a.num + j];
        Term::bwd(g, e0, e1, a.first[qrow * a.dim + d], a.second[qrow * a.dim + d], ge0, ge1, t0, t1);
      }
    }
    if (slot == nullptr) {
      T* out = g_ent + pos * a.dim * Term::kMul;
      out[d] = ge0;
      if (Term::kMul == 2) out[d + a.dim] = ge1;
    } else {
      const int32_t s = slot[pos];
      if (s < 0) continue;
      T* out = g_rows + (size_t)s * a.dim * Term::kMul;
      if (slot_count != nullptr && slot_count[s] == 1) {
        out[d] = ge0;
        if (Term::kMul == 2) out[d + a.dim] = ge1;
      } else {
        atomicAdd(out + d, ge0);
        if (Term::kMul == 2) atomicAdd(out + d + a.dim, ge1);
      }
    }
  }
}

template <typename T, class Term>
__global__ void __launch_bounds__(256)
    cell_backward_query_kernel(CellArgs<T> a, const T* __restrict__ gout0, const T* __restrict__ gout1,
                               T* __restrict__ g_first, T* __restrict__ g_second) {
  const size_t total = a.bc * a.nc * a.dim;
  const size_t nji = a.bsize / a.bc, njj = a.num / a.nc;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (size_t)gridDim.x * blockDim.x) {
    const size_t qrow = t / a.dim, d = t - qrow * a.dim;
    const size_t r0 = qrow / a.nc, r1 = qrow - r0 * a.nc;
    const T q0 = a.first[qrow * a.dim + d], q1 = a.second[qrow * a.dim + d];
    T gq0 = T(0), gq1 = T(0), t0 = T(0), t1 = T(0);
    for (size_t ji = 0; ji < nji; ++ji) {
      const size_t i = ji * a.bc + r0;
      for (size_t jj = 0; jj < njj; ++jj) {
        const size_t j = jj * a.nc + r1;
        size_t row = (i % a.be) * a.ne + (j % a.ne);
        if (a.idx) {
          const long long r = checked_row_id(a.idx, row, a.n_rows, &g_async_status);
          if (r < 0) continue;
          row = (size_t)r;
        }
        const T* pe = a.ent + row * a.dim * Term::kMul;
        T g[Term::kNOut];
        g[0] = gout0[i * a.num + j];
        if (Term::kNOut == 2) g[Term::kNOut - 1] = gout1[i * a.num + j];
        Term::bwd(g, pe[d], Term::kMul == 2 ? pe[d + a.dim] : T(0), q0, q1, t0, t1, gq0, gq1);
      }
    }
    g_first[qrow * a.dim + d] = gq0;
    if (Term::kNQ == 2) g_second[qrow * a.dim + d] = gq1;
  }
}

// ----------------------------------------------------------------------------------------
// row-stream kernels (per-query candidate rows)
// ----------------------------------------------------------------------------------------

constexpr int kUnionBranches = 2;   // query branches the fused union kernels take
constexpr int kRowCtaThreads = 256;
constexpr int kRowCtaWarps = kRowCtaThreads / kWarp;

struct RowArgs {
  const float* ent;        // dense [B*K, W] or table [N, W] when idx != nullptr
  const int64_t* idx;      // nullable [B*K]
  const float* first;      // [B, dim]
  const float* second;     // [B, dim]
  int K;                   // candidate rows per query
  int dim;                 // multiple of 4
  int rows_per_cta;        // multiple of kRowCtaWarps * wrows
  int chunks;              // CTAs per query
  int wrows;               // rows a warp takes per sweep (<= 32)
  long long n_rows;        // rows of `ent` when idx != nullptr (0: ids are not checked)
  // Ragged form (bulk-copy kernels): query q has the seg[q].y candidate rows whose ids are
  // idx[seg[q].x ...]; results and upstream gradients are indexed by the same compact positions.
  // One CTA per query; K, rows_per_cta and chunks are not used.
  const int2* seg;
  // Ragged form on the owner of a row shard: query q belongs to rank q / seg_per_rank, and the
  // result / upstream gradient of compact position p lives at positions[p] in THAT rank's arrays
  // (peer memory): out_ptrs / up_ptrs hold one base pointer per rank and output.  positions ==
  // nullptr: results and upstream gradients are local arrays indexed by compact position.
  // With NB branches per query the rank's arrays are [query][branch][K]: positions[p] names branch 0,
  // branch u sits u * branch_stride (= that rank's K) further.
  const int32_t* positions;
  int seg_per_rank;
  int branch_stride;
  float* const* out_ptrs[2];
  const float* const* up_ptrs[2];
};

// The block of candidate rows a CTA of the row-stream kernels works on.
struct RowBlock {
  int b;            // query
  int r_begin, r_end;
  size_t pos_base;  // position of the query's row 0 in idx / results
};

__device__ __forceinline__ RowBlock row_block(const RowArgs& a) {
  RowBlock rb;
  if (a.seg != nullptr) {
    const int2 s = a.seg[blockIdx.x];
    rb.b = (int)blockIdx.x;
    rb.r_begin = 0;
    rb.r_end = s.y;
    rb.pos_base = (size_t)s.x;
  } else {
    rb.b = blockIdx.x / a.chunks;
    const int c = blockIdx.x - rb.b * a.chunks;
    rb.r_begin = c * a.rows_per_cta;
    rb.r_end = min(a.K, rb.r_begin + a.rows_per_cta);
    rb.pos_base = (size_t)rb.b * a.K;
  }
  return rb;
}

// First float of the block's NB query rows in `first` / `second` / the query-gradient arrays.  Dense
// form: query b's rows start at b * NB * dim.  Ragged form: rank r's queries occupy seg_per_rank * dim
// floats starting at r * seg_per_rank * dim, query q of that rank at q * NB * dim inside them.
template <int NB>
__device__ __forceinline__ size_t query_offset(const RowArgs& a, int b) {
  if (a.seg == nullptr) return (size_t)b * NB * a.dim;
  const int rank = b / a.seg_per_rank, q = b - rank * a.seg_per_rank;
  return ((size_t)rank * a.seg_per_rank + (size_t)q * NB) * a.dim;
}

__device__ __forceinline__ float4 ld_row4(const float4* p) { return __ldg(p); }

// acc over the 4 components of one 16-byte chunk
template <class Term>
__device__ __forceinline__ void fwd4(const float4& e0, const float4& e1, const float4& q0,
                                     const float4& q1, float* acc) {
  Term::fwd(e0.x, e1.x, q0.x, q1.x, acc);
  Term::fwd(e0.y, e1.y, q0.y, q1.y, acc);
  Term::fwd(e0.z, e1.z, q0.z, q1.z, acc);
  Term::fwd(e0.w, e1.w, q0.w, q1.w, acc);
}

template <class Term>
__device__ __forceinline__ void bwd4(const float* g, const float4& e0, const float4& e1,
                                     const float4& q0, const float4& q1, float4& ge0, float4& ge1,
                                     float4& gq0, float4& gq1) {
  Term::bwd(g, e0.x, e1.x, q0.x, q1.x, ge0.x, ge1.x, gq0.x, gq1.x);
  Term::bwd(g, e0.y, e1.y, q0.y, q1.y, ge0.y, ge1.y, gq0.y, gq1.y);
  Term::bwd(g, e0.z, e1.z, q0.z, q1.z, ge0.z, ge1.z, gq0.z, gq1.z);
  Term::bwd(g, e0.w, e1.w, q0.w, q1.w, ge0.w, ge1.w, gq0.w, gq1.w);
}

template <class Term, int NCH, int R>
__global__ void __launch_bounds__(kRowCtaThreads)
    row_forward_kernel(RowArgs a, float* __restrict__ dst0, float* __restrict__ dst1) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.x / a.chunks, c = blockIdx.x - b * a.chunks;
  const int dim4 = a.dim >> 2;
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);

  float4 q0[NCH], q1[NCH];
  {
    const float4* p0 = reinterpret_cast<const float4*>(a.first + (size_t)b * a.dim);
    const float4* p1 = reinterpret_cast<const float4*>(a.second + (size_t)b * a.dim);
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int d4 = lane + 32 * j;
      q0[j] = d4 < dim4 ? __ldg(p0 + d4) : z4;
      q1[j] = (Term::kNQ == 2 && d4 < dim4) ? __ldg(p1 + d4) : z4;
    }
  }

  const int r_begin = c * a.rows_per_cta;
  const int r_end = min(a.K, r_begin + a.rows_per_cta);
  const size_t w4 = (size_t)dim4 * Term::kMul;
  const float4* ent4 = reinterpret_cast<const float4*>(a.ent);

  for (int base = r_begin + warp * a.wrows; base < r_end; base += kRowCtaWarps * a.wrows) {
    const int n = min(a.wrows, r_end - base);
    const size_t pos = (size_t)b * a.K + base + lane;
    long long myrow = 0;   // -1: an id outside the table (row 0 is read instead, the result is NaN)
    if (lane < n) myrow = a.idx ? checked_row_id(a.idx, pos, a.n_rows, &g_async_status) : (long long)pos;
    float out0 = 0.f, out1 = 0.f;
    for (int t = 0; t < n; t += R) {
      float4 e[R][Term::kMul][NCH];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const long long row = max(__shfl_sync(0xffffffffu, myrow, min(t + r, n - 1)), 0LL);
        const float4* pe = ent4 + (size_t)row * w4;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          const int d4 = lane + 32 * j;
          if (d4 < dim4) {
            e[r][0][j] = ld_row4(pe + d4);
            if (Term::kMul == 2) e[r][Term::kMul - 1][j] = ld_row4(pe + dim4 + d4);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float acc[Term::kNOut];
#pragma unroll
        for (int o = 0; o < Term::kNOut; ++o) acc[o] = 0.f;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          if (lane + 32 * j < dim4) fwd4<Term>(e[r][0][j], e[r][Term::kMul - 1][j], q0[j], q1[j], acc);
        }
#pragma unroll
        for (int o = 0; o < Term::kNOut; ++o) acc[o] = warp_sum(acc[o]);
        if (lane == t + r) {
          out0 = acc[0];
          out1 = acc[Term::kNOut - 1];
        }
      }
    }
    if (lane < n) {
      dst0[pos] = myrow < 0 ? NAN : out0;
      if (Term::kNOut == 2) dst1[pos] = myrow < 0 ? NAN : out1;
    }
  }
}

struct RowGradArgs {
  const float* gout0;         // [B, K]
  const float* gout1;         // [B, K] (two-output term only)
  float* g_ent;               // dense [B*K, W], or nullptr when slot != nullptr
  const int32_t* slot;        // [B*K] -> row of g_rows, < 0 to skip
  const int32_t* slot_count;  // contributors per slot over the whole step
  float* g_rows;              // [capacity, W]
  float* g_first;             // [B, dim]
  float* g_second;            // [B, dim]
  int query_atomic;           // several CTAs share one query: accumulate into zeroed g_first/second
};

__device__ __forceinline__ void add4(float4& a, const float4& b) {
  a.x += b.x;
  a.y += b.y;
  a.z += b.z;
  a.w += b.w;
}

// Backward of the row-stream shape.  The gradient of a row element needs no reduction over the
// embedding dim, so the CTA is laid out by columns: `tpr` consecutive threads (a multiple of 32)
// own the 16-byte columns of a row and `groups` such thread groups take alternate rows of the
// CTA's block.  A thread keeps only its column of the query and of the query gradient in
// registers (a handful of registers: high occupancy), has U row loads in flight, and writes its
// column of each row gradient.  Per-row scalars (row offset, output gradients, destination) are
// fetched 32 rows at a time by the lanes of each warp into a warp-private shared-memory table, so
// the inner loop is one broadcast read, one add and one 16-byte access per operand: the kernel
// has to stay well under the SM's issue rate to be bound by HBM instead.
template <class Term, int U>
__global__ void __launch_bounds__(kRowCtaThreads)
    col_backward_kernel(RowArgs a, RowGradArgs ga, int tpr, int groups) {
  extern __shared__ float4 red[];  // [groups][kNQ][dim4]
  __shared__ size_t meta_src[kRowCtaWarps][32];
  __shared__ long long meta_dst[kRowCtaWarps][32];
  __shared__ float2 meta_g[kRowCtaWarps][32];
  __shared__ int meta_single[kRowCtaWarps][32];
  const int lane = threadIdx.x & 31;
  const int grp = threadIdx.x / tpr, col = threadIdx.x - grp * tpr;
  const int b = blockIdx.x / a.chunks, c = blockIdx.x - b * a.chunks;
  const int dim4 = a.dim >> 2;
  const bool active = grp < groups && col < dim4;
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const size_t w4 = (size_t)dim4 * Term::kMul;
  const float4* ent4 = reinterpret_cast<const float4*>(a.ent);
  float4* gbase = reinterpret_cast<float4*>(ga.slot ? ga.g_rows : ga.g_ent);

  float4 q0 = z4, q1 = z4, gq0 = z4, gq1 = z4;
  if (active) {
    q0 = __ldg(reinterpret_cast<const float4*>(a.first + (size_t)b * a.dim) + col);
    if (Term::kNQ == 2) q1 = __ldg(reinterpret_cast<const float4*>(a.second + (size_t)b * a.dim) + col);
  }

  const int r_begin = c * a.rows_per_cta;
  const int r_end = min(a.K, r_begin + a.rows_per_cta);
  if (grp < groups) {
    // this group's rows: r_begin + grp + groups * t, t = 0, 1, ...
    const int n_mine = (r_end - r_begin - grp + groups - 1) / groups;
    const int warp = threadIdx.x >> 5;
    for (int t0 = 0; t0 < n_mine; t0 += 32) {
      const int n = min(32, n_mine - t0);
      // Each warp keeps its own copy of the next 32 rows' scalars in shared memory: where the row
      // starts, where its gradient goes (in 16-byte units, so the inner loop only adds its column),
      // the output gradients, and whether the destination is stored or accumulated.
      __syncwarp();
      {
        const int l = lane < n ? lane : 0;   // surplus lanes repeat the tile's first row: harmless loads
        const size_t pos = (size_t)b * a.K + r_begin + grp + (size_t)groups * (t0 + l);
        const long long row = a.idx ? checked_row_id(a.idx, pos, a.n_rows, &g_async_status) : (long long)pos;
        long long dst = (long long)pos;
        int single = 1;
        if (ga.slot) {
          const int32_t s = ga.slot[pos];
          dst = s;
          single = (s >= 0 && ga.slot_count != nullptr) ? (ga.slot_count[s] == 1) : 0;
        }
        // an id outside the table: row 0 is read, no gradient is written and, with the output
        // gradients zeroed, nothing reaches the query gradient either
        const bool bad = row < 0;
        meta_src[warp][lane] = bad ? 0 : (size_t)row * w4;
        meta_dst[warp][lane] = (dst < 0 || bad) ? -1 : dst * (long long)w4;
        meta_g[warp][lane] = bad ? make_float2(0.f, 0.f)
                                 : make_float2(ga.gout0[pos], Term::kNOut == 2 ? ga.gout1[pos] : 0.f);
        meta_single[warp][lane] = single;
      }
      __syncwarp();
      for (int t = 0; t < n; t += U) {
        float4 e0[U], e1[U];
        if (active) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const float4* pe = ent4 + meta_src[warp][t + u] + col;
            e0[u] = ld_row4(pe);
            if (Term::kMul == 2) e1[u] = ld_row4(pe + dim4);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (t + u < n) {
              const float2 g2 = meta_g[warp][t + u];
              const long long dst = meta_dst[warp][t + u];
              float g[Term::kNOut];
              g[0] = g2.x;
              if (Term::kNOut == 2) g[Term::kNOut - 1] = g2.y;
              float4 ge0 = z4, ge1 = z4;
              bwd4<Term>(g, e0[u], Term::kMul == 2 ? e1[u] : e0[u], q0, q1, ge0, ge1, gq0, gq1);
              if (dst >= 0) {
                float4* out = gbase + dst + col;
                if (meta_single[warp][t + u]) {
                  out[0] = ge0;
                  if (Term::kMul == 2) out[dim4] = ge1;
                } else {
                  atomicAdd(out, ge0);
                  if (Term::kMul == 2) atomicAdd(out + dim4, ge1);
                }
              }
            }
          }
        }
      }
    }
  }

  // fold the groups' query gradients in group order (fixed order: deterministic per CTA)
  if (active) {
    red[(size_t)grp * Term::kNQ * dim4 + col] = gq0;
    if (Term::kNQ == 2) red[(size_t)grp * Term::kNQ * dim4 + dim4 + col] = gq1;
  }
  __syncthreads();
  if (grp == 0 && active) {
    for (int gi = 1; gi < groups; ++gi) {
      add4(gq0, red[(size_t)gi * Term::kNQ * dim4 + col]);
      if (Term::kNQ == 2) add4(gq1, red[(size_t)gi * Term::kNQ * dim4 + dim4 + col]);
    }
    float4* gf = reinterpret_cast<float4*>(ga.g_first + (size_t)b * a.dim) + col;
    float4* gs = reinterpret_cast<float4*>(ga.g_second + (size_t)b * a.dim) + col;
    if (ga.query_atomic) {
      atomicAdd(gf, gq0);
      if (Term::kNQ == 2) atomicAdd(gs, gq1);
    } else {
      *gf = gq0;
      if (Term::kNQ == 2) *gs = gq1;
    }
  }
}

// ----------------------------------------------------------------------------------------
// Row-stream forward with the rows staged through shared memory by bulk asynchronous copies.
// Each warp owns a ring of `stages` row slots and one mbarrier per slot; lane 0 keeps `stages`
// row copies (one instruction per row) in flight ahead of the row the warp is reducing, so the
// bytes in flight per SM no longer depend on registers or on how many warps are resident.
// Work split: the CTA's block of rows is cut into one contiguous run per warp.
// ----------------------------------------------------------------------------------------

__host__ __device__ inline size_t bulk_ring_offset(int stages) {
  return ((size_t)kRowCtaWarps * stages * sizeof(uint64_t) + 127) & ~(size_t)127;
}

// NB: query branches scored against every row (union queries; results [query][branch][row]).
template <class Term, int NB, int NCH>
__global__ void __launch_bounds__(kRowCtaThreads)
    row_forward_bulk_kernel(RowArgs a, float* __restrict__ dst0, float* __restrict__ dst1, int stages) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const RowBlock rb = row_block(a);
  if (rb.r_end <= rb.r_begin) return;    // (ragged form: a query without rows here)
  const int b = rb.b;
  const int dim4 = a.dim >> 2;
  const unsigned row_bytes = (unsigned)dim4 * Term::kMul * 16u;
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  uint64_t* bars = reinterpret_cast<uint64_t*>(bulk_smem) + warp * stages;
  unsigned char* ring = bulk_smem + bulk_ring_offset(stages) + (size_t)warp * stages * row_bytes;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) bulk::barrier_init(bars + s, 1);
    bulk::fence_barrier_init();
  }
  __syncthreads();

  float4 q0[NB][NCH], q1[NB][NCH];
  {
    const size_t q_off = query_offset<NB>(a, b);
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      const float4* p0 = reinterpret_cast<const float4*>(a.first + q_off + (size_t)u * a.dim);
      const float4* p1 = reinterpret_cast<const float4*>(a.second + q_off + (size_t)u * a.dim);
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int d4 = lane + 32 * j;
        q0[u][j] = d4 < dim4 ? __ldg(p0 + d4) : z4;
        q1[u][j] = (Term::kNQ == 2 && d4 < dim4) ? __ldg(p1 + d4) : z4;
      }
    }
  }

  const int r_begin = rb.r_begin, r_end = rb.r_end;
  const int per_warp = (r_end - r_begin + kRowCtaWarps - 1) / kRowCtaWarps;
  const int w_begin = r_begin + warp * per_warp;
  const int n = max(0, min(r_end, w_begin + per_warp) - w_begin);
  const size_t pos0 = rb.pos_base + w_begin;
  const unsigned char* ent = reinterpret_cast<const unsigned char*>(a.ent);

  // row ids of a batch of 32 rows, one per lane; -1 marks an id outside the table (row 0 is copied
  // in its place and the result written for it is NaN)
  auto batch_ids = [&](int first_t) -> long long {
    const int t = first_t + lane;
    if (t >= n) return 0;
    return a.idx ? checked_row_id(a.idx, pos0 + t, a.n_rows, &g_async_status) : (long long)(pos0 + t);
  };
  long long cur = batch_ids(0), nxt = 0;
  // prologue: fill the ring
  const int ahead = min(stages, n);
  for (int t = 0; t < ahead; ++t) {
    const long long row = max(__shfl_sync(0xffffffffu, cur, t), 0LL);
    if (lane == 0) {
      bulk::barrier_expect(bars + t, row_bytes);
      bulk::load(ring + (size_t)t * row_bytes, ent + (size_t)row * row_bytes, row_bytes, bars + t);
    }
  }
  int slot = 0;
  unsigned parity = 0;
  float out0[NB], out1[NB];
#pragma unroll
  for (int u = 0; u < NB; ++u) out0[u] = out1[u] = 0.f;
  for (int t = 0; t < n; ++t) {
    const int tl = t & 31;
    if (tl == 0) nxt = batch_ids(t + 32);
    bool ok = bulk::barrier_wait(bars + slot, parity);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      // give up: let the copies still in flight land (bounded), flag the failure, stop
      if (lane == 0) atomicOr(&g_async_status, kStatusCopyWait);
      for (int k = 1; k < stages && t + k < n; ++k) {
        const int s2 = (slot + k) % stages;
        bulk::barrier_wait(bars + s2, s2 > slot ? parity : parity ^ 1u);
      }
      break;
    }
    const float4* row4 = reinterpret_cast<const float4*>(ring + (size_t)slot * row_bytes);
    float acc[NB][Term::kNOut];
#pragma unroll
    for (int u = 0; u < NB; ++u)
#pragma unroll
      for (int o = 0; o < Term::kNOut; ++o) acc[u][o] = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int d4 = lane + 32 * j;
      if (d4 < dim4) {
        const float4 e0 = row4[d4];
        const float4 e1 = Term::kMul == 2 ? row4[dim4 + d4] : e0;
#pragma unroll
        for (int u = 0; u < NB; ++u) fwd4<Term>(e0, e1, q0[u][j], q1[u][j], acc[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < NB; ++u)
#pragma unroll
      for (int o = 0; o < Term::kNOut; ++o) acc[u][o] = warp_sum(acc[u][o]);
    // the sums above consumed every lane's reads of the slot: it may be refilled
    __syncwarp();
    const int tn = t + stages;
    if (tn < n) {
      const long long row = max(__shfl_sync(0xffffffffu, (tn >> 5) == (t >> 5) ? cur : nxt, tn & 31), 0LL);
      if (lane == 0) {
        bulk::barrier_expect(bars + slot, row_bytes);
        bulk::load(ring + (size_t)slot * row_bytes, ent + (size_t)row * row_bytes, row_bytes, bars + slot);
      }
    }
    if (lane == tl) {
#pragma unroll
      for (int u = 0; u < NB; ++u) {
        out0[u] = acc[u][0];
        out1[u] = acc[u][Term::kNOut - 1];
      }
    }
    if (tl == 31 || t == n - 1) {
      if (lane <= tl) {
        const size_t o = pos0 + (t - tl) + lane;
        if (a.positions != nullptr) {          // straight into the requesting rank's result arrays
          const int rank = b / a.seg_per_rank;
          const size_t at = (size_t)a.positions[o];
#pragma unroll
          for (int u = 0; u < NB; ++u) {
            a.out_ptrs[0][rank][at + (size_t)u * a.branch_stride] = cur < 0 ? NAN : out0[u];
            if (Term::kNOut == 2) a.out_ptrs[1][rank][at + (size_t)u * a.branch_stride] = cur < 0 ? NAN : out1[u];
          }
        } else {                                // (local result arrays: one branch)
          dst0[o] = cur < 0 ? NAN : out0[0];
          if (Term::kNOut == 2) dst1[o] = cur < 0 ? NAN : out1[0];
        }
      }
      cur = nxt;
    }
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
}

// ----------------------------------------------------------------------------------------
// Row-stream backward on the same bulk-copy ring.  A warp takes a contiguous run of rows; each
// row is copied into a ring slot, its gradient is computed IN PLACE over the row (every lane
// overwrites exactly the 16-byte pieces it read), and lane 0 sends the slot to the gradient
// buffer with one bulk store - or one bulk floating-point add where several positions of the
// step share the destination row.  The slot is refilled once that transfer has read it.
// NB query branches (union queries) are applied to every row; their row gradients are summed in
// registers before the slot is written.  The query gradients stay in registers over the warp's
// run and are folded over the CTA's warps through the ring at the end, in warp order.
// ----------------------------------------------------------------------------------------

template <class Term, int NB, int NCH>
__global__ void __launch_bounds__(kRowCtaThreads, 2)
    row_backward_bulk_kernel(RowArgs a, RowGradArgs ga, int stages) {
  constexpr int NG = NB * Term::kNOut;
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.x / a.chunks, c = blockIdx.x - b * a.chunks;
  const int dim4 = a.dim >> 2;
  const unsigned row_bytes = (unsigned)dim4 * Term::kMul * 16u;
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  uint64_t* bars = reinterpret_cast<uint64_t*>(bulk_smem) + warp * stages;
  float4* sq = reinterpret_cast<float4*>(bulk_smem + bulk_ring_offset(stages));   // [kNQ][NB][dim4]
  unsigned char* ring_all = reinterpret_cast<unsigned char*>(sq + (size_t)Term::kNQ * NB * dim4);
  unsigned char* ring = ring_all + (size_t)warp * stages * row_bytes;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) bulk::barrier_init(bars + s, 1);
    bulk::fence_barrier_init();
  }
  {
    const float4* p0 = reinterpret_cast<const float4*>(a.first + (size_t)b * NB * a.dim);
    const float4* p1 = reinterpret_cast<const float4*>(a.second + (size_t)b * NB * a.dim);
    for (int i = threadIdx.x; i < NB * dim4; i += kRowCtaThreads) {
      sq[i] = __ldg(p0 + i);
      if (Term::kNQ == 2) sq[NB * dim4 + i] = __ldg(p1 + i);
    }
  }
  __syncthreads();
  const float4* sq0 = sq;
  const float4* sq1 = Term::kNQ == 2 ? sq + NB * dim4 : sq;

  float4 gq0[NB][NCH], gq1[NB][NCH];
#pragma unroll
  for (int u = 0; u < NB; ++u)
#pragma unroll
    for (int j = 0; j < NCH; ++j) gq0[u][j] = gq1[u][j] = z4;

  const int r_begin = c * a.rows_per_cta;
  const int r_end = min(a.K, r_begin + a.rows_per_cta);
  const int per_warp = (r_end - r_begin + kRowCtaWarps - 1) / kRowCtaWarps;
  const int w_begin = r_begin + warp * per_warp;
  const int n = max(0, min(r_end, w_begin + per_warp) - w_begin);
  const size_t pos0 = (size_t)b * a.K + w_begin;
  const unsigned char* ent = reinterpret_cast<const unsigned char*>(a.ent);
  unsigned char* gbase = reinterpret_cast<unsigned char*>(ga.slot ? ga.g_rows : ga.g_ent);

  // per-lane scalars of one batch of 32 rows: source row, destination row (-1: none), whether the
  // destination is written by this position alone, output gradients of every branch
  struct Meta {
    long long src, dst;
    int single;
    float g[NG];
  };
  auto load_meta = [&](int first_t) {
    Meta m;
    m.src = 0;
    m.dst = -1;
    m.single = 1;
#pragma unroll
    for (int i = 0; i < NG; ++i) m.g[i] = 0.f;
    const int t = first_t + lane;
    if (t < n) {
      const size_t pos = pos0 + t;
      m.src = a.idx ? checked_row_id(a.idx, pos, a.n_rows, &g_async_status) : (long long)pos;
      m.dst = (long long)pos;
      if (ga.slot) {
        const int32_t sl = ga.slot[pos];
        m.dst = sl;
        m.single = (sl >= 0 && ga.slot_count != nullptr) ? (ga.slot_count[sl] == 1) : 0;
      }
      if (m.src < 0) {
        // an id outside the table: row 0 is copied, nothing is written for it and its output
        // gradients stay zero, so the query gradients see nothing of it either
        m.src = 0;
        m.dst = -1;
      } else {
#pragma unroll
        for (int u = 0; u < NB; ++u) {
          const size_t o = ((size_t)b * NB + u) * a.K + (w_begin + t);
          m.g[u * Term::kNOut] = ga.gout0[o];
          if (Term::kNOut == 2) m.g[u * Term::kNOut + Term::kNOut - 1] = ga.gout1[o];
        }
      }
    }
    return m;
  };
  Meta cur = load_meta(0), nxt = cur;

  const int ahead = min(stages - 1, n);   // one slot always belongs to the store in flight
  for (int t = 0; t < ahead; ++t) {
    const long long row = __shfl_sync(0xffffffffu, cur.src, t);
    if (lane == 0) {
      bulk::barrier_expect(bars + t, row_bytes);
      bulk::load(ring + (size_t)t * row_bytes, ent + (size_t)row * row_bytes, row_bytes, bars + t);
    }
  }
  int slot = 0;
  unsigned parity = 0;
  for (int t = 0; t < n; ++t) {
    const int tl = t & 31;
    if (tl == 0) nxt = load_meta(t + 32);
    bool ok = bulk::barrier_wait(bars + slot, parity);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0) atomicOr(&g_async_status, kStatusCopyWait);
      for (int k = 1; k < stages - 1 && t + k < n; ++k) {
        const int s2 = (slot + k) % stages;
        bulk::barrier_wait(bars + s2, s2 > slot ? parity : parity ^ 1u);
      }
      break;
    }
    float g[NG];
#pragma unroll
    for (int i = 0; i < NG; ++i) g[i] = __shfl_sync(0xffffffffu, cur.g[i], tl);
    const long long dst = __shfl_sync(0xffffffffu, cur.dst, tl);
    const int single = __shfl_sync(0xffffffffu, cur.single, tl);
    float4* row4 = reinterpret_cast<float4*>(ring + (size_t)slot * row_bytes);
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int d4 = lane + 32 * j;
      if (d4 < dim4) {
        const float4 e0 = row4[d4];
        const float4 e1 = Term::kMul == 2 ? row4[dim4 + d4] : e0;
        float4 ge0 = z4, ge1 = z4;
#pragma unroll
        for (int u = 0; u < NB; ++u)
          bwd4<Term>(g + u * Term::kNOut, e0, e1, sq0[u * dim4 + d4], sq1[u * dim4 + d4], ge0, ge1, gq0[u][j],
                     gq1[u][j]);
        row4[d4] = ge0;
        if (Term::kMul == 2) row4[dim4 + d4] = ge1;
      }
    }
    bulk::fence_async_shared();   // the gradient row is visible to the copy engine
    __syncwarp();
    // refill target: the slot of the previous row, whose transfer was committed one row ago
    const int tn = t + stages - 1;
    const long long next_row = __shfl_sync(0xffffffffu, (tn >> 5) == (t >> 5) ? cur.src : nxt.src, tn & 31);
    if (lane == 0) {
      if (dst >= 0) {
        unsigned char* out = gbase + (size_t)dst * row_bytes;
        if (single) bulk::store(out, row4, row_bytes);
        else bulk::reduce_add_f32(out, row4, row_bytes);
      }
      bulk::commit_group();
      if (tn < n) {
        bulk::wait_group_read<1>();   // all transfers but the one just committed have read their slots
        const int s2 = slot == 0 ? stages - 1 : slot - 1;
        bulk::barrier_expect(bars + s2, row_bytes);
        bulk::load(ring + (size_t)s2 * row_bytes, ent + (size_t)next_row * row_bytes, row_bytes, bars + s2);
      }
    }
    if (tl == 31) cur = nxt;
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
  if (lane == 0) bulk::wait_group<0>();   // every gradient row has left shared memory and landed
  __syncthreads();

  // fold the warps' query gradients through the (now idle) ring, in warp order
  float4* red = reinterpret_cast<float4*>(ring_all);
  const size_t per_warp4 = (size_t)NB * Term::kNQ * dim4;
#pragma unroll
  for (int u = 0; u < NB; ++u)
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int d4 = lane + 32 * j;
      if (d4 < dim4) {
        red[warp * per_warp4 + (size_t)u * Term::kNQ * dim4 + d4] = gq0[u][j];
        if (Term::kNQ == 2) red[warp * per_warp4 + (size_t)u * Term::kNQ * dim4 + dim4 + d4] = gq1[u][j];
      }
    }
  __syncthreads();
  for (size_t i = threadIdx.x; i < per_warp4; i += kRowCtaThreads) {
    float4 acc = red[i];
    for (int w = 1; w < kRowCtaWarps; ++w) add4(acc, red[w * per_warp4 + i]);
    const size_t u = i / ((size_t)Term::kNQ * dim4), rem = i - u * Term::kNQ * dim4;
    const bool second = rem >= (size_t)dim4;
    float* base = second ? ga.g_second : ga.g_first;
    float4* out = reinterpret_cast<float4*>(base + ((size_t)b * NB + u) * a.dim) + (rem - (second ? dim4 : 0));
    if (ga.query_atomic) atomicAdd(out, acc);
    else *out = acc;
  }
}

// ----------------------------------------------------------------------------------------
// Row-stream backward with the optimizer step folded in (Adam, row-wise second moment).
//
// Most rows a step touches are touched by exactly one (query, candidate) position (about 95 % at
// the Freebase-scale benchmark).  For such a row the gradient this kernel computes IS the step's
// merged gradient, so writing it to the gradient buffer only to have the update kernel read it
// back - together with the parameter row this kernel has just read - is wasted traffic: per row
// 1.6 KB written and 3.2 KB read again.  Here the warp that owns the row also copies the row of
// the first moment into the ring (same bulk copy group as the parameter row), applies the update
// in shared memory and sends both rows back with bulk stores; the row's entry in the step's list
// of distinct rows is complemented (~row, negative), which the update kernel skips.  Rows with
// several contributors take the ordinary route (bulk floating-point add into the gradient buffer,
// updated afterwards by smore_sparse_update_rows).
// Safe because a row with a single contributor is read by no other position of the backward pass
// and the forward pass has finished.  The arithmetic is that of adam_rows_reg_kernel.
// ----------------------------------------------------------------------------------------

template <class Term, int NB, int NCH>
__global__ void __launch_bounds__(kRowCtaThreads, 2)
    row_backward_adam_bulk_kernel(RowArgs a, RowGradArgs ga, UpdateArgs ua, int64_t* __restrict__ uniq_rw, int stages) {
  constexpr int NG = NB * Term::kNOut;
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const RowBlock rb = row_block(a);
  const int b = rb.b;
  const int dim4 = a.dim >> 2;
  const unsigned row_bytes = (unsigned)dim4 * Term::kMul * 16u;
  const unsigned stage_bytes = 2u * row_bytes;          // [parameter row | first-moment row]
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const size_t q_off = query_offset<NB>(a, b);
  if (rb.r_end <= rb.r_begin) {
    // (ragged form: a query without rows here) its query gradient is zero.  A rank has room for
    // seg_per_rank / NB queries of NB rows: the segment slots beyond that are never used and own no
    // part of the query-gradient array (their offset would fall into the next rank's part).
    const bool has_slot = a.seg == nullptr || ((b % a.seg_per_rank) + 1) * NB <= a.seg_per_rank;
    if (has_slot) {
      for (int i = threadIdx.x; i < NB * dim4; i += kRowCtaThreads) {
        reinterpret_cast<float4*>(ga.g_first + q_off)[i] = z4;
        if (Term::kNQ == 2) reinterpret_cast<float4*>(ga.g_second + q_off)[i] = z4;
      }
    }
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(bulk_smem) + warp * stages;
  float4* sq = reinterpret_cast<float4*>(bulk_smem + bulk_ring_offset(stages));   // [kNQ][NB][dim4]
  unsigned char* ring_all = reinterpret_cast<unsigned char*>(sq + (size_t)Term::kNQ * NB * dim4);
  unsigned char* ring = ring_all + (size_t)warp * stages * stage_bytes;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) bulk::barrier_init(bars + s, 1);
    bulk::fence_barrier_init();
  }
  {
    const float4* p0 = reinterpret_cast<const float4*>(a.first + q_off);
    const float4* p1 = reinterpret_cast<const float4*>(a.second + q_off);
    for (int i = threadIdx.x; i < NB * dim4; i += kRowCtaThreads) {
      sq[i] = __ldg(p0 + i);
      if (Term::kNQ == 2) sq[NB * dim4 + i] = __ldg(p1 + i);
    }
  }
  __syncthreads();
  load_dyn(ua);
  const float4* sq0 = sq;
  const float4* sq1 = Term::kNQ == 2 ? sq + NB * dim4 : sq;

  float4 gq0[NB][NCH], gq1[NB][NCH];
#pragma unroll
  for (int u = 0; u < NB; ++u)
#pragma unroll
    for (int j = 0; j < NCH; ++j) gq0[u][j] = gq1[u][j] = z4;

  const int r_begin = rb.r_begin, r_end = rb.r_end;
  const int per_warp = (r_end - r_begin + kRowCtaWarps - 1) / kRowCtaWarps;
  const int w_begin = r_begin + warp * per_warp;
  const int n = max(0, min(r_end, w_begin + per_warp) - w_begin);
  const size_t pos0 = rb.pos_base + w_begin;
  const unsigned char* ent = reinterpret_cast<const unsigned char*>(a.ent);
  const unsigned char* mom = reinterpret_cast<const unsigned char*>(ua.m);
  unsigned char* gbase = reinterpret_cast<unsigned char*>(ga.g_rows);

  struct Meta {
    long long src, dst;
    int single;
    float v;          // second moment of a row that is updated here
    float g[NG];
  };
  auto load_meta = [&](int first_t) {
    Meta m;
    m.src = 0;
    m.dst = -1;
    m.single = 0;
    m.v = 0.f;
#pragma unroll
    for (int i = 0; i < NG; ++i) m.g[i] = 0.f;
    const int t = first_t + lane;
    if (t < n) {
      const size_t pos = pos0 + t;
      m.src = checked_row_id(a.idx, pos, a.n_rows, &g_async_status);
      const int32_t sl = ga.slot[pos];
      m.dst = sl;
      m.single = (sl >= 0 && ga.slot_count != nullptr) ? (ga.slot_count[sl] == 1) : 0;
      if (m.src < 0) {
        m.src = 0;
        m.dst = -1;
        m.single = 0;
      } else {
        if (m.single) m.v = ua.v[m.src];
#pragma unroll
        for (int u = 0; u < NB; ++u) {
          if (a.positions != nullptr) {        // from the requesting rank's arrays ([query][branch][row])
            const int rank = b / a.seg_per_rank;
            const size_t at = (size_t)a.positions[pos] + (size_t)u * a.branch_stride;
            m.g[u * Term::kNOut] = a.up_ptrs[0][rank][at];
            if (Term::kNOut == 2) m.g[u * Term::kNOut + Term::kNOut - 1] = a.up_ptrs[1][rank][at];
            continue;
          }
          // (ragged form with local arrays: upstream gradients sit at the rows' compact positions)
          const size_t o = a.seg != nullptr ? pos : ((size_t)b * NB + u) * a.K + (w_begin + t);
          m.g[u * Term::kNOut] = ga.gout0[o];
          if (Term::kNOut == 2) m.g[u * Term::kNOut + Term::kNOut - 1] = ga.gout1[o];
        }
      }
    }
    return m;
  };
  // lane 0: start the copies of one row (and, for a row updated here, of its first-moment row)
  auto issue = [&](int s, long long row, int single) {
    unsigned char* dst = ring + (size_t)s * stage_bytes;
    bulk::barrier_expect(bars + s, single ? stage_bytes : row_bytes);
    bulk::load(dst, ent + (size_t)row * row_bytes, row_bytes, bars + s);
    if (single) bulk::load(dst + row_bytes, mom + (size_t)row * row_bytes, row_bytes, bars + s);
  };
  Meta cur = load_meta(0), nxt = cur;

  const int ahead = min(stages - 1, n);   // one slot always belongs to the stores in flight
  for (int t = 0; t < ahead; ++t) {
    const long long row = __shfl_sync(0xffffffffu, cur.src, t);
    const int single = __shfl_sync(0xffffffffu, (cur.dst >= 0) ? cur.single : 0, t);
    if (lane == 0) issue(t, row, single);
  }
  int slot = 0;
  unsigned parity = 0;
  for (int t = 0; t < n; ++t) {
    const int tl = t & 31;
    if (tl == 0) nxt = load_meta(t + 32);
    bool ok = bulk::barrier_wait(bars + slot, parity);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0) atomicOr(&g_async_status, kStatusCopyWait);
      for (int k = 1; k < stages - 1 && t + k < n; ++k) {
        const int s2 = (slot + k) % stages;
        bulk::barrier_wait(bars + s2, s2 > slot ? parity : parity ^ 1u);
      }
      break;
    }
    float g[NG];
#pragma unroll
    for (int i = 0; i < NG; ++i) g[i] = __shfl_sync(0xffffffffu, cur.g[i], tl);
    const long long dst = __shfl_sync(0xffffffffu, cur.dst, tl);
    const long long row = __shfl_sync(0xffffffffu, cur.src, tl);
    const int single = dst >= 0 ? __shfl_sync(0xffffffffu, cur.single, tl) : 0;
    float4* row4 = reinterpret_cast<float4*>(ring + (size_t)slot * stage_bytes);
    float4* mom4 = reinterpret_cast<float4*>(ring + (size_t)slot * stage_bytes + row_bytes);
    float4 ge[Term::kMul][NCH];
    float sumsq = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int d4 = lane + 32 * j;
      ge[0][j] = z4;
      if (Term::kMul == 2) ge[Term::kMul - 1][j] = z4;
      if (d4 < dim4) {
        const float4 e0 = row4[d4];
        const float4 e1 = Term::kMul == 2 ? row4[dim4 + d4] : e0;
        float4 ge0 = z4, ge1 = z4;
#pragma unroll
        for (int u = 0; u < NB; ++u)
          bwd4<Term>(g + u * Term::kNOut, e0, e1, sq0[u * dim4 + d4], sq1[u * dim4 + d4], ge0, ge1, gq0[u][j],
                     gq1[u][j]);
        ge[0][j] = ge0;
        sumsq += ge0.x * ge0.x + ge0.y * ge0.y + ge0.z * ge0.z + ge0.w * ge0.w;
        if (Term::kMul == 2) {
          ge[Term::kMul - 1][j] = ge1;
          sumsq += ge1.x * ge1.x + ge1.y * ge1.y + ge1.z * ge1.z + ge1.w * ge1.w;
        }
      }
    }
    float v_new = 0.f;
    const float v_old = __shfl_sync(0xffffffffu, cur.v, tl);
    if (single) {
      // the row's Adam step, in place: the slot holds the parameter row and the first-moment row
      const float g2mean = warp_sum(sumsq) / (float)ua.width;
      v_new = v_old * ua.beta2 + g2mean * ua.omb2;
      const float denom = sqrtf(v_new) / ua.sqrt_bc2 + ua.eps;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int d4 = lane + 32 * j;
        if (d4 < dim4) {
#pragma unroll
          for (int part = 0; part < Term::kMul; ++part) {
            float4 p = row4[part * dim4 + d4], m = mom4[part * dim4 + d4];
            const float4 gg = ge[part][j];
            adam_elem_rowwise(gg.x, p.x, m.x, denom, ua);
            adam_elem_rowwise(gg.y, p.y, m.y, denom, ua);
            adam_elem_rowwise(gg.z, p.z, m.z, denom, ua);
            adam_elem_rowwise(gg.w, p.w, m.w, denom, ua);
            row4[part * dim4 + d4] = p;
            mom4[part * dim4 + d4] = m;
          }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int d4 = lane + 32 * j;
        if (d4 < dim4) {
          row4[d4] = ge[0][j];
          if (Term::kMul == 2) row4[dim4 + d4] = ge[Term::kMul - 1][j];
        }
      }
    }
    bulk::fence_async_shared();   // what the lanes wrote is visible to the copy engine
    __syncwarp();
    const int tn = t + stages - 1;
    const bool same = (tn >> 5) == (t >> 5);
    const long long next_row = __shfl_sync(0xffffffffu, same ? cur.src : nxt.src, tn & 31);
    const int next_single = __shfl_sync(0xffffffffu, same ? ((cur.dst >= 0) ? cur.single : 0)
                                                          : ((nxt.dst >= 0) ? nxt.single : 0), tn & 31);
    if (lane == 0) {
      if (single) {
        bulk::store(const_cast<unsigned char*>(ent) + (size_t)row * row_bytes, row4, row_bytes);
        bulk::store(const_cast<unsigned char*>(mom) + (size_t)row * row_bytes, mom4, row_bytes);
        ua.v[row] = v_old + (v_new - v_old);
        uniq_rw[dst] = ~(int64_t)row;       // this row's update is done: the update kernel skips it
      } else if (dst >= 0) {
        bulk::reduce_add_f32(gbase + (size_t)dst * row_bytes, row4, row_bytes);
      }
      bulk::commit_group();
      if (tn < n) {
        bulk::wait_group_read<1>();   // all transfers but the ones just committed have read their slots
        const int s2 = slot == 0 ? stages - 1 : slot - 1;
        issue(s2, next_row, next_single);
      }
    }
    if (tl == 31) cur = nxt;
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
  if (lane == 0) bulk::wait_group<0>();
  __syncthreads();

  // fold the warps' query gradients through the (now idle) ring, in warp order
  float4* red = reinterpret_cast<float4*>(ring_all);
  const size_t per_warp4 = (size_t)NB * Term::kNQ * dim4;
#pragma unroll
  for (int u = 0; u < NB; ++u)
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int d4 = lane + 32 * j;
      if (d4 < dim4) {
        red[warp * per_warp4 + (size_t)u * Term::kNQ * dim4 + d4] = gq0[u][j];
        if (Term::kNQ == 2) red[warp * per_warp4 + (size_t)u * Term::kNQ * dim4 + dim4 + d4] = gq1[u][j];
      }
    }
  __syncthreads();
  for (size_t i = threadIdx.x; i < per_warp4; i += kRowCtaThreads) {
    float4 acc = red[i];
    for (int w = 1; w < kRowCtaWarps; ++w) add4(acc, red[w * per_warp4 + i]);
    const size_t u = i / ((size_t)Term::kNQ * dim4), rem = i - u * Term::kNQ * dim4;
    const bool second = rem >= (size_t)dim4;
    float* base = second ? ga.g_second : ga.g_first;
    float4* out = reinterpret_cast<float4*>(base + q_off + u * a.dim) + (rem - (second ? dim4 : 0));
    if (ga.query_atomic) atomicAdd(out, acc);
    else *out = acc;
  }
}

// ----------------------------------------------------------------------------------------
// Union queries: NB branches of every query scored against the same candidate rows.
// The reference runs the op once per branch and stacks the results (a Python loop over the
// branch axis of a 4-D query operand); here one pass over the rows serves all branches, and the
// backward pass writes the sum of the branches' row gradients once.
// Operands: first / second [B, NB, dim]; outputs and output gradients [B, NB, K].
// ----------------------------------------------------------------------------------------

template <class Term, int NB, int NCH, int R>
__global__ void __launch_bounds__(kRowCtaThreads)
    row_forward_union_kernel(RowArgs a, float* __restrict__ dst0, float* __restrict__ dst1) {
  extern __shared__ float4 sq[];  // [2][NB][dim4]: the query's branches, first then second operand
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.x / a.chunks, c = blockIdx.x - b * a.chunks;
  const int dim4 = a.dim >> 2;
  {
    const float4* p0 = reinterpret_cast<const float4*>(a.first + (size_t)b * NB * a.dim);
    const float4* p1 = reinterpret_cast<const float4*>(a.second + (size_t)b * NB * a.dim);
    for (int i = threadIdx.x; i < NB * dim4; i += kRowCtaThreads) {
      sq[i] = __ldg(p0 + i);
      if (Term::kNQ == 2) sq[NB * dim4 + i] = __ldg(p1 + i);
    }
  }
  __syncthreads();
  const float4* sq0 = sq;
  const float4* sq1 = Term::kNQ == 2 ? sq + NB * dim4 : sq;

  const int r_begin = c * a.rows_per_cta;
  const int r_end = min(a.K, r_begin + a.rows_per_cta);
  const size_t w4 = (size_t)dim4 * Term::kMul;
  const float4* ent4 = reinterpret_cast<const float4*>(a.ent);

  for (int base = r_begin + warp * a.wrows; base < r_end; base += kRowCtaWarps * a.wrows) {
    const int n = min(a.wrows, r_end - base);
    const size_t pos = (size_t)b * a.K + base + lane;
    long long myrow = 0;   // -1: an id outside the table (row 0 is read instead, the result is NaN)
    if (lane < n) myrow = a.idx ? checked_row_id(a.idx, pos, a.n_rows, &g_async_status) : (long long)pos;
    float out0[NB], out1[NB];
#pragma unroll
    for (int u = 0; u < NB; ++u) out0[u] = out1[u] = 0.f;
    for (int t = 0; t < n; t += R) {
      float4 e[R][Term::kMul][NCH];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const long long row = max(__shfl_sync(0xffffffffu, myrow, min(t + r, n - 1)), 0LL);
        const float4* pe = ent4 + (size_t)row * w4;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          const int d4 = lane + 32 * j;
          if (d4 < dim4) {
            e[r][0][j] = ld_row4(pe + d4);
            if (Term::kMul == 2) e[r][Term::kMul - 1][j] = ld_row4(pe + dim4 + d4);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int u = 0; u < NB; ++u) {
          float acc[Term::kNOut];
#pragma unroll
          for (int o = 0; o < Term::kNOut; ++o) acc[o] = 0.f;
#pragma unroll
          for (int j = 0; j < NCH; ++j) {
            const int d4 = lane + 32 * j;
            if (d4 < dim4)
              fwd4<Term>(e[r][0][j], e[r][Term::kMul - 1][j], sq0[u * dim4 + d4], sq1[u * dim4 + d4], acc);
          }
#pragma unroll
          for (int o = 0; o < Term::kNOut; ++o) acc[o] = warp_sum(acc[o]);
          if (lane == t + r) {
            out0[u] = acc[0];
            out1[u] = acc[Term::kNOut - 1];
          }
        }
      }
    }
    if (lane < n) {
#pragma unroll
      for (int u = 0; u < NB; ++u) {
        const size_t o = ((size_t)b * NB + u) * a.K + base + lane;
        dst0[o] = myrow < 0 ? NAN : out0[u];
        if (Term::kNOut == 2) dst1[o] = myrow < 0 ? NAN : out1[u];
      }
    }
  }
}

template <int N>
struct alignas(4 * N) GoutVec {
  float v[N];
};

template <class Term, int NB, int U>
__global__ void __launch_bounds__(kRowCtaThreads)
    col_backward_union_kernel(RowArgs a, RowGradArgs ga, int tpr, int groups) {
  constexpr int NG = NB * Term::kNOut;   // output gradients per row: 2 or 4
  extern __shared__ float4 red[];        // [groups][NB][kNQ][dim4]
  __shared__ size_t meta_src[kRowCtaWarps][32];
  __shared__ long long meta_dst[kRowCtaWarps][32];
  __shared__ GoutVec<NG> meta_g[kRowCtaWarps][32];
  __shared__ int meta_single[kRowCtaWarps][32];
  const int lane = threadIdx.x & 31;
  const int grp = threadIdx.x / tpr, col = threadIdx.x - grp * tpr;
  const int b = blockIdx.x / a.chunks, c = blockIdx.x - b * a.chunks;
  const int dim4 = a.dim >> 2;
  const bool active = grp < groups && col < dim4;
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const size_t w4 = (size_t)dim4 * Term::kMul;
  const float4* ent4 = reinterpret_cast<const float4*>(a.ent);
  float4* gbase = reinterpret_cast<float4*>(ga.g_rows);

  float4 q0[NB], q1[NB], gq0[NB], gq1[NB];
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    q0[u] = q1[u] = gq0[u] = gq1[u] = z4;
    if (active) {
      q0[u] = __ldg(reinterpret_cast<const float4*>(a.first + ((size_t)b * NB + u) * a.dim) + col);
      if (Term::kNQ == 2)
        q1[u] = __ldg(reinterpret_cast<const float4*>(a.second + ((size_t)b * NB + u) * a.dim) + col);
    }
  }

  const int r_begin = c * a.rows_per_cta;
  const int r_end = min(a.K, r_begin + a.rows_per_cta);
  if (grp < groups) {
    const int n_mine = (r_end - r_begin - grp + groups - 1) / groups;
    const int warp = threadIdx.x >> 5;
    for (int t0 = 0; t0 < n_mine; t0 += 32) {
      const int n = min(32, n_mine - t0);
      __syncwarp();
      {
        const int l = lane < n ? lane : 0;
        const int k = r_begin + grp + groups * (t0 + l);
        const size_t pos = (size_t)b * a.K + k;
        const long long row = checked_row_id(a.idx, pos, a.n_rows, &g_async_status);
        const bool bad = row < 0;   // as in col_backward_kernel: read row 0, write and contribute nothing
        const int32_t s = ga.slot[pos];
        meta_src[warp][lane] = bad ? 0 : (size_t)row * w4;
        meta_dst[warp][lane] = (s < 0 || bad) ? -1 : s * (long long)w4;
        GoutVec<NG> g;
#pragma unroll
        for (int u = 0; u < NB; ++u) {
          const size_t o = ((size_t)b * NB + u) * a.K + k;
          g.v[u * Term::kNOut] = bad ? 0.f : ga.gout0[o];
          if (Term::kNOut == 2) g.v[u * Term::kNOut + Term::kNOut - 1] = bad ? 0.f : ga.gout1[o];
        }
        meta_g[warp][lane] = g;
        meta_single[warp][lane] = (s >= 0 && ga.slot_count != nullptr) ? (ga.slot_count[s] == 1) : 0;
      }
      __syncwarp();
      for (int t = 0; t < n; t += U) {
        float4 e0[U], e1[U];
        if (active) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const float4* pe = ent4 + meta_src[warp][t + u] + col;
            e0[u] = ld_row4(pe);
            if (Term::kMul == 2) e1[u] = ld_row4(pe + dim4);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (t + u < n) {
              const GoutVec<NG> gv = meta_g[warp][t + u];
              const long long dst = meta_dst[warp][t + u];
              float4 ge0 = z4, ge1 = z4;
#pragma unroll
              for (int br = 0; br < NB; ++br) {
                float g[Term::kNOut];
                g[0] = gv.v[br * Term::kNOut];
                if (Term::kNOut == 2) g[Term::kNOut - 1] = gv.v[br * Term::kNOut + Term::kNOut - 1];
                bwd4<Term>(g, e0[u], Term::kMul == 2 ? e1[u] : e0[u], q0[br], q1[br], ge0, ge1, gq0[br], gq1[br]);
              }
              if (dst >= 0) {
                float4* out = gbase + dst + col;
                if (meta_single[warp][t + u]) {
                  out[0] = ge0;
                  if (Term::kMul == 2) out[dim4] = ge1;
                } else {
                  atomicAdd(out, ge0);
                  if (Term::kMul == 2) atomicAdd(out + dim4, ge1);
                }
              }
            }
          }
        }
      }
    }
  }

  // fold the groups' query gradients in group order
  const size_t per_group = (size_t)NB * Term::kNQ * dim4;
  if (active) {
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      red[grp * per_group + (size_t)u * Term::kNQ * dim4 + col] = gq0[u];
      if (Term::kNQ == 2) red[grp * per_group + (size_t)u * Term::kNQ * dim4 + dim4 + col] = gq1[u];
    }
  }
  __syncthreads();
  if (grp == 0 && active) {
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      for (int gi = 1; gi < groups; ++gi) {
        add4(gq0[u], red[gi * per_group + (size_t)u * Term::kNQ * dim4 + col]);
        if (Term::kNQ == 2) add4(gq1[u], red[gi * per_group + (size_t)u * Term::kNQ * dim4 + dim4 + col]);
      }
      float4* gf = reinterpret_cast<float4*>(ga.g_first + ((size_t)b * NB + u) * a.dim) + col;
      float4* gs = reinterpret_cast<float4*>(ga.g_second + ((size_t)b * NB + u) * a.dim) + col;
      if (ga.query_atomic) {
        atomicAdd(gf, gq0[u]);
        if (Term::kNQ == 2) atomicAdd(gs, gq1[u]);
      } else {
        *gf = gq0[u];
        if (Term::kNQ == 2) *gs = gq1[u];
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// Evaluation: scores of a batch of queries against EVERY entity, ranked on the fly.
// The reference's test step (smore/training/train_process.py:104-146) materialises the [Q, N] logits,
// argsorts them and scatters ranks; smore_filtered_ranks already replaces the sort by counting but
// still reads a logits matrix.  Here the scoring tile never leaves the registers: every cell is
// turned into the model's logit with the arithmetic torch would use on the distances
// (custom_cal_logit: gamma - d_out - cen * d_in for Query2box, box.py:157-164; gamma - d for GQE and
// RotatE; the similarity itself for ComplEx / DistMult), compared with the query's worst answer and,
// if it is ahead of it, placed among the query's sorted answers (binary search, one histogram
// increment).  The answers' own logits come from the same tile code run on the answers' rows, so a
// candidate that is an answer meets exactly its own value.
// ----------------------------------------------------------------------------------------

enum LogitKind { kLogitGammaMinus = 0, kLogitGammaMinusSqrt = 1, kLogitIdentity = 2 };

template <int NOUT>
__device__ __forceinline__ float logit_of(const float* acc, int kind, float gamma, float cen) {
  if (NOUT == 2) return __fsub_rn(__fsub_rn(gamma, acc[0]), __fmul_rn(cen, acc[NOUT - 1]));
  if (kind == kLogitGammaMinus) return __fsub_rn(gamma, acc[0]);
  if (kind == kLogitGammaMinusSqrt) return __fsub_rn(gamma, sqrtf(acc[0]));
  return acc[0];
}

// answer scores [Q, n_answers] (one or two distances) -> logits, in place of dst0
template <int NOUT>
__global__ void __launch_bounds__(256)
    answer_logits_kernel(float* __restrict__ d0, const float* __restrict__ d1, size_t n, int kind, float gamma, float cen) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float acc[2] = {d0[i], NOUT == 2 ? d1[i] : 0.f};
    d0[i] = logit_of<NOUT>(acc, kind, gamma, cen);
  }
}

template <class Term>
__global__ void __launch_bounds__(256)
    score_rank_kernel(SharedArgs a, int kind, float gamma, float cen, const int64_t* __restrict__ answer_ptr,
                      const uint32_t* __restrict__ sorted_logit, const int64_t* __restrict__ sorted_id,
                      int32_t* __restrict__ hist) {
  __shared__ __align__(16) TileSmem<Term> sm;
  __shared__ long long q_begin[kTileB], q_worst_id[kTileB];
  __shared__ int q_count[kTileB];
  __shared__ uint32_t q_worst[kTileB];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int b0 = blockIdx.y * kTileB, k0 = blockIdx.x * kTileK;
  if (threadIdx.x < kTileB) {
    const int b = b0 + threadIdx.x;
    long long begin = 0, wid = 0;
    int A = 0;
    uint32_t wk = 0;
    if (b < a.B) {
      begin = answer_ptr[b];
      A = (int)(answer_ptr[b + 1] - begin);
      if (A > 0) {
        wk = sorted_logit[begin + A - 1];
        wid = sorted_id[begin + A - 1];
      }
    }
    q_begin[threadIdx.x] = begin;
    q_count[threadIdx.x] = A;
    q_worst[threadIdx.x] = wk;
    q_worst_id[threadIdx.x] = wid;
  }
  float acc[4][4][Term::kNOut];
  tile_scores<Term>(a, sm, b0, k0, acc);      // (its barriers also order the writes above)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int bl = ty * 4 + i;
    const int A = q_count[bl];
    if (b0 + bl >= a.B || A == 0) continue;
    const long long begin = q_begin[bl];
    const uint32_t worst = q_worst[bl];
    const long long worst_id = q_worst_id[bl];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long e = k0 + tx * 4 + j;
      if (e >= a.K) continue;
      const uint32_t x = rank_key(logit_of<Term::kNOut>(acc[i][j], kind, gamma, cen));
      if (!rank_ahead(x, e, worst, worst_id)) continue;      // ahead of no answer (the usual case)
      int lo = 0, hi = A - 1;   // first answer this candidate is ahead of
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (rank_ahead(x, e, sorted_logit[begin + mid], sorted_id[begin + mid])) hi = mid;
        else lo = mid + 1;
      }
      atomicAdd(hist + begin + lo, 1);
    }
  }
}

// ----------------------------------------------------------------------------------------
// host side: validation, shape classification, launches
// ----------------------------------------------------------------------------------------

struct Shape {
  size_t bsize, num, be, ne, bc, nc, dim;
  size_t n_rows = 0;   // rows of the table when the entity operand is (table, idx); 0: ids unchecked
};

static int validate_shape(const Shape& s) {
  if (!s.bsize || !s.num || !s.be || !s.ne || !s.bc || !s.nc || !s.dim)
    return fail(SMORE_ERR_BAD_SHAPE, "all sizes must be positive");
  if (s.bsize != std::max(s.be, s.bc) || s.num != std::max(s.ne, s.nc))
    return fail(SMORE_ERR_BAD_SHAPE, "output must be [max(be,bc), max(ne,nc)]");
  if (s.bsize % s.be || s.bsize % s.bc || s.num % s.ne || s.num % s.nc)
    return fail(SMORE_ERR_BAD_SHAPE, "operand sizes must divide the output sizes");
  if (s.dim > (size_t)1 << 30 || s.bsize * s.num > (size_t)1 << 40)
    return fail(SMORE_ERR_TOO_LARGE, "operand too large");
  return SMORE_OK;
}

static int grid_for(size_t work_items, int per_block) {
  size_t blocks = (work_items + per_block - 1) / per_block;
  const size_t cap = (size_t)sm_count() * 32;
  return (int)std::max<size_t>(1, std::min(blocks, cap));
}

// row-stream launch plan; chunks == 0 means "not eligible"
struct RowPlan {
  int nch, wrows, rows_per_cta, chunks;
};

static RowPlan plan_rows(const Shape& s, bool aligned) {
  RowPlan p{0, 0, 0, 0};
  const bool shape_ok = s.be == s.bsize && s.bc == s.bsize && s.ne == s.num && s.nc == 1;
  if (!shape_ok || !aligned || (s.dim & 3) || s.dim > 1024 || s.num < 4 || s.num > (size_t)1 << 30 ||
      s.bsize > (size_t)1 << 24)
    return p;
  const int dim4 = (int)(s.dim >> 2);
  p.nch = dim4 <= 32 ? 1 : dim4 <= 64 ? 2 : dim4 <= 128 ? 4 : 8;
  const size_t K = s.num;
  int wrows = 32;
  while (wrows > 4 && (size_t)wrows * kRowCtaWarps / 2 >= K) wrows >>= 1;
  p.wrows = wrows;
  const size_t sweep = (size_t)wrows * kRowCtaWarps;
  size_t sweeps_per_cta = 1;
  const size_t sweeps_total = (K + sweep - 1) / sweep;
  // keep the grid within a few dozen waves; larger blocks of rows amortise the query load
  const size_t max_ctas = (size_t)sm_count() * 32;
  while (s.bsize * ((sweeps_total + sweeps_per_cta - 1) / sweeps_per_cta) > max_ctas &&
         sweeps_per_cta < sweeps_total)
    sweeps_per_cta *= 2;
  p.rows_per_cta = (int)std::min<size_t>(sweep * sweeps_per_cta, (size_t)1 << 30);
  p.chunks = (int)((K + p.rows_per_cta - 1) / p.rows_per_cta);
  return p;
}

// one candidate set scored against every query (shared negatives, full-table evaluation)
static bool shared_shape(const Shape& s, bool aligned) {
  return aligned && s.be == 1 && s.bc == s.bsize && s.ne == s.num && s.nc == 1 && (s.dim & 3) == 0 &&
         s.bsize >= 8 && s.num >= 8 && s.bsize < ((size_t)1 << 24) && s.num < ((size_t)1 << 30) &&
         s.dim < ((size_t)1 << 20) && (s.bsize + kTileB - 1) / kTileB <= 65535;   // grid.y / grid.z limits
}

// Launches row_backward_bulk_kernel when the row width suits it.  Returns 1 when launched, 0 when
// the caller should use another kernel, a negative status on failure.
template <class Term, int NB>
static int launch_backward_bulk(const Shape& s, RowArgs a, RowGradArgs ga, int nch, cudaStream_t st) {
  // Measured on B200: ahead of the column-thread kernel for rows of 2 KB and more (RotatE rows of
  // 4000 B: 1.59 ms against 1.67 ms per 1M rows); for 1600-byte rows it executes more instructions
  // per row (waits, per-row scalars) than that kernel and ends level with it, so those stay there.
  const size_t row_bytes = s.dim * Term::kMul * sizeof(float);
  if ((nch != 4 && nch != 8) || row_bytes < 2048) return 0;
  const int need = (NB * Term::kNQ + Term::kMul - 1) / Term::kMul;   // ring must hold the final fold
  const int stages = std::max(3, need);
  const size_t q_bytes = (size_t)NB * Term::kNQ * s.dim * sizeof(float);
  const size_t smem = bulk_ring_offset(stages) + q_bytes + (size_t)kRowCtaWarps * stages * row_bytes;
  if (smem > 110 * 1024) return 0;
  a.rows_per_cta = (int)std::min<size_t>(s.num, 512);
  a.chunks = (int)((s.num + a.rows_per_cta - 1) / a.rows_per_cta);
  ga.query_atomic = a.chunks > 1;
  if (a.chunks > 1) {
    const size_t bytes = s.bsize * NB * s.dim * sizeof(float);
    if (cudaMemsetAsync(ga.g_first, 0, bytes, st) != cudaSuccess ||
        (Term::kNQ == 2 && cudaMemsetAsync(ga.g_second, 0, bytes, st) != cudaSuccess))
      return fail(SMORE_ERR_CUDA, "row_backward_bulk_kernel: cudaMemsetAsync failed");
  }
  auto kern = nch == 4 ? row_backward_bulk_kernel<Term, NB, 4> : row_backward_bulk_kernel<Term, NB, 8>;
  if (int rc = allow_large_smem(kern, 110 * 1024)) return rc;
  kern<<<(unsigned)(s.bsize * a.chunks), kRowCtaThreads, smem, st>>>(a, ga, stages);
  if (int rc = check_launch("row_backward_bulk_kernel")) return rc;
  return 1;
}

// Launches row_backward_adam_bulk_kernel when the shape suits it.  Returns 1 when launched, 0 when the
// caller should use the ordinary backward + update, a negative status on failure.
template <class Term, int NB>
static int launch_backward_adam(const Shape& s, RowArgs a, RowGradArgs ga, const UpdateArgs& ua, int64_t* uniq,
                                int nch, cudaStream_t st) {
  const size_t row_bytes = s.dim * Term::kMul * sizeof(float);
  if ((nch != 4 && nch != 8) || row_bytes < 1024) return 0;
  const int need = (NB * Term::kNQ + 2 * Term::kMul - 1) / (2 * Term::kMul);   // ring must hold the final fold
  const size_t q_bytes = (size_t)NB * Term::kNQ * s.dim * sizeof(float);
  // as many stages (3..5) as fit two CTAs per SM: every stage holds a parameter row and a moment row
  int stages = 5;
  while (stages > 3 && bulk_ring_offset(stages) + q_bytes + (size_t)kRowCtaWarps * stages * 2 * row_bytes > 110 * 1024)
    --stages;
  stages = std::max(stages, need);
  const size_t smem = bulk_ring_offset(stages) + q_bytes + (size_t)kRowCtaWarps * stages * 2 * row_bytes;
  if (smem > 200 * 1024) return 0;      // wide rows (RotatE, 4000 bytes): one CTA per SM
  if (a.seg != nullptr) {
    a.chunks = 1;         // ragged form: one CTA per query, s.bsize queries
  } else {
    a.rows_per_cta = (int)std::min<size_t>(s.num, 512);
    a.chunks = (int)((s.num + a.rows_per_cta - 1) / a.rows_per_cta);
  }
  ga.query_atomic = a.chunks > 1;
  if (a.chunks > 1) {
    const size_t bytes = s.bsize * NB * s.dim * sizeof(float);
    if (cudaMemsetAsync(ga.g_first, 0, bytes, st) != cudaSuccess ||
        (Term::kNQ == 2 && cudaMemsetAsync(ga.g_second, 0, bytes, st) != cudaSuccess))
      return fail(SMORE_ERR_CUDA, "row_backward_adam_bulk_kernel: cudaMemsetAsync failed");
  }
  auto kern = nch == 4 ? row_backward_adam_bulk_kernel<Term, NB, 4> : row_backward_adam_bulk_kernel<Term, NB, 8>;
  if (int rc = allow_large_smem(kern, 200 * 1024)) return rc;
  kern<<<(unsigned)(s.bsize * a.chunks), kRowCtaThreads, smem, st>>>(a, ga, ua, uniq, stages);
  if (int rc = check_launch("row_backward_adam_bulk_kernel")) return rc;
  return 1;
}

template <class Term>
static int backward_adam_common(size_t branches, const Shape& s, const float* gout0, const float* gout1, float* table,
                                const int64_t* idx, const float* first, const float* second, const int32_t* slot,
                                const int32_t* slot_count, float* g_rows, float* g_first, float* g_second,
                                const UpdateArgs& ua, int64_t* uniq, cudaStream_t st) {
  if (Term::kNQ == 1) {
    second = first;
    g_second = g_first;
  }
  const bool aligned = aligned16(table) && aligned16(first) && aligned16(second) && aligned16(g_rows) &&
                       aligned16(g_first) && aligned16(g_second) && aligned16(ua.m);
  const RowPlan p = plan_rows(s, aligned);
  if (p.chunks == 0) return 0;
  RowArgs a{table, idx, first, second, (int)s.num, (int)s.dim, p.rows_per_cta, p.chunks, p.wrows, (long long)s.n_rows};
  RowGradArgs ga{gout0, gout1, nullptr, slot, slot_count, g_rows, g_first, g_second, 0};
  if (branches == 1) return launch_backward_adam<Term, 1>(s, a, ga, ua, uniq, p.nch, st);
  return launch_backward_adam<Term, kUnionBranches>(s, a, ga, ua, uniq, p.nch, st);
}

// ---- ragged form: query q scores / differentiates the candidate rows idx[seg[q].x .. + seg[q].y) ----
// (the owner side of a row-sharded table: the queries of every rank against this shard's rows).
// Returns 1 when launched, 0 when the row width is outside the bulk-copy kernels' range.
static int ragged_nch(size_t dim, size_t mul) {
  const size_t dim4 = dim >> 2, row_bytes = dim * mul * sizeof(float);
  if ((dim & 3) || dim > 1024 || dim4 <= 64 || row_bytes < 1024) return 0;
  return dim4 <= 128 ? 4 : 8;
}

struct RaggedPeers {        // where results go / upstream gradients come from (see RowArgs)
  const int32_t* positions;
  size_t seg_per_rank;
  size_t branch_stride;
  float* const* out0;
  float* const* out1;
  const float* const* up0;
  const float* const* up1;
};

static void set_peers(RowArgs& a, const RaggedPeers& pr) {
  a.positions = pr.positions;
  a.seg_per_rank = (int)std::max<size_t>(pr.seg_per_rank, 1);
  a.branch_stride = (int)pr.branch_stride;
  a.out_ptrs[0] = pr.out0; a.out_ptrs[1] = pr.out1;
  a.up_ptrs[0] = pr.up0; a.up_ptrs[1] = pr.up1;
}

template <class Term>
static int launch_forward_ragged(size_t branches, size_t n_seg, size_t dim, size_t n_rows, const float* table,
                                 const int64_t* rows, const float* first, const float* second, const int2* seg,
                                 float* out0, float* out1, const RaggedPeers& pr, cudaStream_t st) {
  if (Term::kNQ == 1) second = first;
  const int nch = ragged_nch(dim, Term::kMul);
  if (!nch || !aligned16(table) || !aligned16(first) || !aligned16(second)) return 0;
  const size_t row_bytes = dim * Term::kMul * sizeof(float);
  const int stages = (int)std::min<size_t>(8, std::max<size_t>(2, (96 * 1024 / 32 + row_bytes - 1) / row_bytes));
  const size_t smem = std::max<size_t>(bulk_ring_offset(stages) + (size_t)kRowCtaWarps * stages * row_bytes, 46 * 1024);
  if (smem > 110 * 1024) return 0;
  RowArgs a{table, rows, first, second, 0, (int)dim, 0, 1, 0, (long long)n_rows, seg};
  set_peers(a, pr);
  auto kern = branches == 1 ? (nch == 4 ? row_forward_bulk_kernel<Term, 1, 4> : row_forward_bulk_kernel<Term, 1, 8>)
                            : (nch == 4 ? row_forward_bulk_kernel<Term, kUnionBranches, 4>
                                        : row_forward_bulk_kernel<Term, kUnionBranches, 8>);
  if (int rc = allow_large_smem(kern, 110 * 1024)) return rc;
  kern<<<(unsigned)n_seg, kRowCtaThreads, smem, st>>>(a, out0, out1, stages);
  if (int rc = check_launch("row_forward_bulk_kernel")) return rc;
  return 1;
}

template <class Term>
static int launch_backward_adam_ragged(size_t branches, size_t n_seg, size_t dim, size_t n_rows, const float* gout0, const float* gout1,
                                       float* table, const int64_t* rows, const float* first, const float* second,
                                       const int2* seg, const int32_t* slot, const int32_t* slot_count, float* g_rows,
                                       float* g_first, float* g_second, const UpdateArgs& ua, int64_t* uniq,
                                       const RaggedPeers& pr, cudaStream_t st) {
  if (Term::kNQ == 1) {
    second = first;
    g_second = g_first;
  }
  const int nch = ragged_nch(dim, Term::kMul);
  if (!nch || !aligned16(table) || !aligned16(first) || !aligned16(second) || !aligned16(g_rows) || !aligned16(g_first) ||
      !aligned16(g_second) || !aligned16(ua.m))
    return 0;
  const Shape s{n_seg, 4, n_seg, 4, n_seg, 1, dim, n_rows};
  RowArgs a{table, rows, first, second, 0, (int)dim, 0, 1, 0, (long long)n_rows, seg};
  set_peers(a, pr);
  RowGradArgs ga{gout0, gout1, nullptr, slot, slot_count, g_rows, g_first, g_second, 0};
  if (branches == 1) return launch_backward_adam<Term, 1>(s, a, ga, ua, uniq, nch, st);
  return launch_backward_adam<Term, kUnionBranches>(s, a, ga, ua, uniq, nch, st);
}

template <class Term>
static int launch_forward(const Shape& s, const float* ent, const int64_t* idx, const float* first,
                          const float* second, float* dst0, float* dst1, cudaStream_t st) {
  if (Term::kNQ == 1) second = first;
  const bool aligned = aligned16(ent) && aligned16(first) && aligned16(second);
  const RowPlan p = plan_rows(s, aligned);
  if (p.chunks > 0) {
    RowArgs a{ent, idx, first, second, (int)s.num, (int)s.dim, p.rows_per_cta, p.chunks, p.wrows, (long long)s.n_rows};
    const unsigned grid = (unsigned)(s.bsize * p.chunks);
    constexpr int R = 2;  // rows in flight per warp at 4 chunks per lane
    // Rows of 1 KB and more go through the bulk-copy kernel: 2..8 slots per warp (about 96 KB of
    // row copies in flight per SM at 32 resident warps; more in flight measured slower), CTAs of
    // 512 rows.  It needs at least two CTAs per SM to cover the reduction latency.
    const size_t row_bytes = s.dim * Term::kMul * sizeof(float);
    const int stages = (int)std::min<size_t>(8, std::max<size_t>(2, (96 * 1024 / 32 + row_bytes - 1) / row_bytes));
    // at least 46 KB per CTA keeps the residency at four CTAs per SM whatever the register count:
    // five and more (terms with few registers) put more row copies in flight than the memory
    // system likes and measured up to 1.8x slower
    const size_t bulk_smem = std::max<size_t>(bulk_ring_offset(stages) + (size_t)kRowCtaWarps * stages * row_bytes,
                                              46 * 1024);
    if ((p.nch == 4 || p.nch == 8) && bulk_smem <= 110 * 1024) {
      RowArgs ab = a;
      ab.rows_per_cta = (int)std::min<size_t>(s.num, 512);
      ab.chunks = (int)((s.num + ab.rows_per_cta - 1) / ab.rows_per_cta);
      auto kern = p.nch == 4 ? row_forward_bulk_kernel<Term, 1, 4> : row_forward_bulk_kernel<Term, 1, 8>;
      if (int rc = allow_large_smem(kern, 110 * 1024)) return rc;
      kern<<<(unsigned)(s.bsize * ab.chunks), kRowCtaThreads, bulk_smem, st>>>(ab, dst0, dst1, stages);
      return check_launch("row_forward_bulk_kernel");
    }
    switch (p.nch) {
      case 1: row_forward_kernel<Term, 1, 4><<<grid, kRowCtaThreads, 0, st>>>(a, dst0, dst1); break;
      case 2: row_forward_kernel<Term, 2, 4><<<grid, kRowCtaThreads, 0, st>>>(a, dst0, dst1); break;
      case 4: row_forward_kernel<Term, 4, R><<<grid, kRowCtaThreads, 0, st>>>(a, dst0, dst1); break;
      default: row_forward_kernel<Term, 8, 1><<<grid, kRowCtaThreads, 0, st>>>(a, dst0, dst1); break;
    }
    return check_launch("row_forward_kernel");
  }
  if (shared_shape(s, aligned)) {
    SharedArgs a{ent, idx, first, second, (int)s.bsize, (int)s.num, (int)s.dim, (long long)s.n_rows};
    dim3 grid((unsigned)((s.num + kTileK - 1) / kTileK), (unsigned)((s.bsize + kTileB - 1) / kTileB));
    shared_forward_kernel<Term><<<grid, 256, 0, st>>>(a, dst0, dst1);
    return check_launch("shared_forward_kernel");
  }
  CellArgs<float> a{ent, idx, first, second, s.bsize, s.num, s.be, s.ne, s.bc, s.nc, s.dim, (long long)s.n_rows};
  cell_forward_kernel<float, Term><<<grid_for(s.bsize * s.num, 8), 256, 0, st>>>(a, dst0, dst1);
  return check_launch("cell_forward_kernel");
}

// Both gradients of the shared-candidate shape from one evaluation of every term
// (shared_backward_tile_kernel): a cluster of up to 8 CTAs per (KT candidate rows, 128 dims) splits
// the queries; the query gradients are reduced into zeroed buffers.  The device runs about one
// 8-CTA cluster per SM at a time whatever the CTA's size, so CTAs are 4 warps wide.
template <class Term, int KT>
static int launch_shared_backward_kt(const Shape& s, const SharedArgs& a, const SharedGradArgs& ga, cudaStream_t st) {
  const size_t qbytes = s.bsize * s.dim * sizeof(float);
  if (cudaMemsetAsync(ga.g_first, 0, qbytes, st) != cudaSuccess ||
      (Term::kNQ == 2 && cudaMemsetAsync(ga.g_second, 0, qbytes, st) != cudaSuccess))
    return fail(SMORE_ERR_CUDA, "dist_backward: cudaMemsetAsync failed");
  // dims per CTA: whole warps, at most 128 (a warp past the last dim idles at the barriers only)
  const int threads = (int)std::min<size_t>(128, ((s.dim + 31) / 32) * 32);
  const unsigned dchunks = (unsigned)((s.dim + threads - 1) / threads);
  unsigned split = 1;   // query segments = CTAs per cluster: enough CTAs to fill the device, >= 32 queries each
  const size_t base_ctas = ((s.num + KT - 1) / KT) * dchunks;
  while (split < 8 && s.bsize / (split * 2) >= 32 && base_ctas * split * threads < (size_t)sm_count() * 2048 * 4) split *= 2;
  const int seg_b = (int)((s.bsize + split - 1) / split);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((s.num + KT - 1) / KT), split, dchunks);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = (size_t)KT * Term::kMul * threads * sizeof(float);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = split;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, shared_backward_tile_kernel<Term, KT>, a, ga, seg_b) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "shared_backward_tile_kernel: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
  return check_launch("shared_backward_tile_kernel");
}

template <class Term>
static int launch_shared_backward(const Shape& s, const SharedArgs& a, const SharedGradArgs& ga, cudaStream_t st) {
  // terms of one operand each and one output are cheap next to the per-query loads and reductions:
  // twice the rows per thread halves those
  if (Term::kMul == 1 && Term::kNQ == 1 && Term::kNOut == 1 && s.num >= 16)
    return launch_shared_backward_kt<Term, 16>(s, a, ga, st);
  return launch_shared_backward_kt<Term, 8>(s, a, ga, st);
}

template <class Term>
static int launch_backward(const Shape& s, const float* gout0, const float* gout1, const float* ent,
                           const int64_t* idx, const float* first, const float* second, float* g_ent,
                           const int32_t* slot, const int32_t* slot_count, float* g_rows,
                           float* g_first, float* g_second, cudaStream_t st) {
  if (Term::kNQ == 1) {
    second = first;
    g_second = g_first;
  }
  float* gdst = slot ? g_rows : g_ent;
  const bool aligned = aligned16(ent) && aligned16(first) && aligned16(second) && aligned16(gdst) &&
                       aligned16(g_first) && aligned16(g_second);
  const RowPlan p = plan_rows(s, aligned);
  if (p.chunks > 0) {
    RowArgs a{ent, idx, first, second, (int)s.num, (int)s.dim, p.rows_per_cta, p.chunks, p.wrows, (long long)s.n_rows};
    RowGradArgs ga{gout0, gout1, g_ent, slot, slot_count, g_rows, g_first, g_second, p.chunks > 1};
    if (int rc = launch_backward_bulk<Term, 1>(s, a, ga, p.nch, st)) return rc < 0 ? rc : SMORE_OK;
    if (p.chunks > 1) {
      const size_t bytes = s.bsize * s.dim * sizeof(float);
      if (cudaMemsetAsync(g_first, 0, bytes, st) != cudaSuccess ||
          (Term::kNQ == 2 && cudaMemsetAsync(g_second, 0, bytes, st) != cudaSuccess))
        return fail(SMORE_ERR_CUDA, "dist_backward: cudaMemsetAsync failed");
    }
    const unsigned grid = (unsigned)(s.bsize * p.chunks);
    const int dim4 = (int)(s.dim >> 2);
    const int tpr = ((dim4 + 31) / 32) * 32;          // threads that own the columns of one row
    const int groups = kRowCtaThreads / tpr;          // row groups per CTA (dim <= 1024 -> >= 1)
    const size_t smem = (size_t)groups * Term::kNQ * s.dim * sizeof(float);
    if (Term::kMul == 2)
      col_backward_kernel<Term, 4><<<grid, kRowCtaThreads, smem, st>>>(a, ga, tpr, groups);
    else
      col_backward_kernel<Term, 8><<<grid, kRowCtaThreads, smem, st>>>(a, ga, tpr, groups);
    return check_launch("col_backward_kernel");
  }
  if (shared_shape(s, aligned)) {
    SharedArgs a{ent, idx, first, second, (int)s.bsize, (int)s.num, (int)s.dim, (long long)s.n_rows};
    SharedGradArgs ga{gout0, gout1, g_ent, slot, slot_count, g_rows, g_first, g_second};
    return launch_shared_backward<Term>(s, a, ga, st);
  }
  CellArgs<float> a{ent, idx, first, second, s.bsize, s.num, s.be, s.ne, s.bc, s.nc, s.dim, (long long)s.n_rows};
  cell_backward_ent_kernel<float, Term><<<grid_for(s.be * s.ne * s.dim, 256), 256, 0, st>>>(
      a, gout0, gout1, g_ent, slot, slot_count, g_rows);
  cell_backward_query_kernel<float, Term><<<grid_for(s.bc * s.nc * s.dim, 256), 256, 0, st>>>(
      a, gout0, gout1, g_first, g_second);
  return check_launch("cell_backward kernels", 2);
}

static int check_union(const char* what, size_t branches, const Shape& s, bool aligned, RowPlan* p) {
  if (branches != kUnionBranches)
    return fail(SMORE_ERR_BAD_SHAPE, "%s: %d branches per query are supported (run other counts branch by branch)",
                what, kUnionBranches);
  if (int rc = validate_shape(s)) return rc;
  *p = plan_rows(s, aligned);
  if (p->chunks == 0)
    return fail(SMORE_ERR_BAD_SHAPE,
                "%s: needs 16-byte aligned operands, dim a multiple of 4 and <= 1024, at least 4 rows per query", what);
  return SMORE_OK;
}

template <class Term>
static int launch_forward_union(size_t branches, const Shape& s, const float* table, const int64_t* idx,
                                const float* first, const float* second, float* dst0, float* dst1,
                                cudaStream_t st) {
  if (Term::kNQ == 1) second = first;
  RowPlan p;
  if (int rc = check_union("union_forward_rows", branches, s, aligned16(table) && aligned16(first) && aligned16(second),
                           &p))
    return rc;
  RowArgs a{table, idx, first, second, (int)s.num, (int)s.dim, p.rows_per_cta, p.chunks, p.wrows, (long long)s.n_rows};
  constexpr int NB = kUnionBranches;
  // (staging the rows with bulk copies, as row_forward_bulk_kernel does, measured no faster here:
  // with two branches per row the kernel is bound by instruction issue, not by memory latency)
  const unsigned grid = (unsigned)(s.bsize * p.chunks);
  const size_t smem = (size_t)kUnionBranches * Term::kNQ * s.dim * sizeof(float);
  switch (p.nch) {
    case 1: row_forward_union_kernel<Term, NB, 1, 4><<<grid, kRowCtaThreads, smem, st>>>(a, dst0, dst1); break;
    case 2: row_forward_union_kernel<Term, NB, 2, 4><<<grid, kRowCtaThreads, smem, st>>>(a, dst0, dst1); break;
    case 4: row_forward_union_kernel<Term, NB, 4, 2><<<grid, kRowCtaThreads, smem, st>>>(a, dst0, dst1); break;
    default: row_forward_union_kernel<Term, NB, 8, 1><<<grid, kRowCtaThreads, smem, st>>>(a, dst0, dst1); break;
  }
  return check_launch("row_forward_union_kernel");
}

template <class Term>
static int launch_backward_union(size_t branches, const Shape& s, const float* gout0, const float* gout1,
                                 const float* table, const int64_t* idx, const float* first, const float* second,
                                 const int32_t* slot, const int32_t* slot_count, float* g_rows, float* g_first,
                                 float* g_second, cudaStream_t st) {
  if (Term::kNQ == 1) {
    second = first;
    g_second = g_first;
  }
  RowPlan p;
  const bool aligned = aligned16(table) && aligned16(first) && aligned16(second) && aligned16(g_rows) &&
                       aligned16(g_first) && aligned16(g_second);
  if (int rc = check_union("union_backward_rows", branches, s, aligned, &p)) return rc;
  constexpr int NB = kUnionBranches;
  RowArgs a{table, idx, first, second, (int)s.num, (int)s.dim, p.rows_per_cta, p.chunks, p.wrows, (long long)s.n_rows};
  RowGradArgs ga{gout0, gout1, nullptr, slot, slot_count, g_rows, g_first, g_second, p.chunks > 1};
  if (p.chunks > 1) {
    const size_t bytes = s.bsize * NB * s.dim * sizeof(float);
    if (cudaMemsetAsync(g_first, 0, bytes, st) != cudaSuccess ||
        (Term::kNQ == 2 && cudaMemsetAsync(g_second, 0, bytes, st) != cudaSuccess))
      return fail(SMORE_ERR_CUDA, "union_backward_rows: cudaMemsetAsync failed");
  }
  const unsigned grid = (unsigned)(s.bsize * p.chunks);
  const int dim4 = (int)(s.dim >> 2);
  const int tpr = ((dim4 + 31) / 32) * 32;
  const int groups = kRowCtaThreads / tpr;
  const size_t smem = (size_t)groups * NB * Term::kNQ * s.dim * sizeof(float);
  if (Term::kMul == 2)
    col_backward_union_kernel<Term, NB, 4><<<grid, kRowCtaThreads, smem, st>>>(a, ga, tpr, groups);
  else
    col_backward_union_kernel<Term, NB, 8><<<grid, kRowCtaThreads, smem, st>>>(a, ga, tpr, groups);
  return check_launch("col_backward_union_kernel");
}

template <class Term>
static int launch_forward_f64(const Shape& s, const double* ent, const double* first,
                              const double* second, double* dst, cudaStream_t st) {
  if (Term::kNQ == 1) second = first;
  CellArgs<double> a{ent, nullptr, first, second, s.bsize, s.num, s.be, s.ne, s.bc, s.nc, s.dim, (long long)s.n_rows};
  cell_forward_kernel<double, Term><<<grid_for(s.bsize * s.num, 8), 256, 0, st>>>(a, dst, dst);
  return check_launch("cell_forward_kernel<double>");
}

template <class Term>
static int launch_backward_f64(const Shape& s, const double* gout, const double* ent,
                               const double* first, const double* second, double* g_ent,
                               double* g_first, double* g_second, cudaStream_t st) {
  if (Term::kNQ == 1) {
    second = first;
    g_second = g_first;
  }
  CellArgs<double> a{ent, nullptr, first, second, s.bsize, s.num, s.be, s.ne, s.bc, s.nc, s.dim, (long long)s.n_rows};
  cell_backward_ent_kernel<double, Term><<<grid_for(s.be * s.ne * s.dim, 256), 256, 0, st>>>(
      a, gout, gout, g_ent, nullptr, nullptr, nullptr);
  cell_backward_query_kernel<double, Term><<<grid_for(s.bc * s.nc * s.dim, 256), 256, 0, st>>>(
      a, gout, gout, g_first, g_second);
  return check_launch("cell_backward kernels<double>", 2);
}

static bool needs_second(int id) {
  return id == SMORE_DIST_BOX_OUT || id == SMORE_DIST_BOX_IN || id == SMORE_DIST_ROTATE ||
         id == SMORE_DIST_COMPLEX;
}

#define SMORE_DISPATCH(id, CALL)                                        \
  switch (id) {                                                         \
    case SMORE_DIST_BOX_OUT: { using Term = TermBoxOut; return CALL; }  \
    case SMORE_DIST_BOX_IN: { using Term = TermBoxIn; return CALL; }    \
    case SMORE_DIST_ROTATE: { using Term = TermRotate; return CALL; }   \
    case SMORE_DIST_L1: { using Term = TermL1; return CALL; }           \
    case SMORE_DIST_L2: { using Term = TermL2; return CALL; }           \
    case SMORE_DIST_COMPLEX: { using Term = TermComplex; return CALL; } \
    case SMORE_DIST_DISTMULT: { using Term = TermDistmult; return CALL; } \
    default: return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", id); \
  }

static int forward_common(int id, const float* ent, const int64_t* idx, const float* first,
                          const float* second, float* dst, const Shape& s, void* stream) {
  if (id < 0 || id >= SMORE_DIST_COUNT) return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", id);
  if (!ent || !first || !dst || (needs_second(id) && !second))
    return fail(SMORE_ERR_NULL, "forward: required pointer is NULL");
  if (int rc = validate_shape(s)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  SMORE_DISPATCH(id, launch_forward<Term>(s, ent, idx, first, second, dst, dst, st));
}

static int backward_common(int id, const float* gout, const float* ent, const int64_t* idx,
                           const float* first, const float* second, float* g_ent, const int32_t* slot,
                           const int32_t* slot_count, float* g_rows, float* g_first, float* g_second,
                           const Shape& s, void* stream) {
  if (id < 0 || id >= SMORE_DIST_COUNT) return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", id);
  if (!gout || !ent || !first || !g_first || (needs_second(id) && (!second || !g_second)))
    return fail(SMORE_ERR_NULL, "backward: required pointer is NULL");
  if (slot ? !g_rows : !g_ent)
    return fail(SMORE_ERR_NULL, "backward: entity gradient destination is NULL");
  if (int rc = validate_shape(s)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  SMORE_DISPATCH(id, launch_backward<Term>(s, gout, gout, ent, idx, first, second, g_ent, slot, slot_count,
                                           g_rows, g_first, g_second, st));
}

}  // namespace smore

using namespace smore;

extern "C" {

int smore_dist_forward(int dist_id, const float* ent, const float* first, const float* second, float* dst,
                       size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc, size_t dim,
                       void* stream) {
  return forward_common(dist_id, ent, nullptr, first, second, dst, Shape{bsize, num, be, ne, bc, nc, dim},
                        stream);
}

int smore_dist_backward(int dist_id, const float* gout, const float* ent, const float* first,
                        const float* second, float* g_ent, float* g_first, float* g_second, size_t bsize,
                        size_t num, size_t be, size_t ne, size_t bc, size_t nc, size_t dim, void* stream) {
  return backward_common(dist_id, gout, ent, nullptr, first, second, g_ent, nullptr, nullptr, nullptr,
                         g_first, g_second, Shape{bsize, num, be, ne, bc, nc, dim}, stream);
}

int smore_dist_forward_rows(int dist_id, const float* table, const int64_t* idx, size_t n_table_rows,
                            const float* first, const float* second, float* dst, size_t bsize, size_t num,
                            size_t be, size_t ne, size_t bc, size_t nc, size_t dim, void* stream) {
  if (!idx) return fail(SMORE_ERR_NULL, "forward_rows: idx is NULL");
  return forward_common(dist_id, table, idx, first, second, dst,
                        Shape{bsize, num, be, ne, bc, nc, dim, n_table_rows}, stream);
}

int smore_dist_backward_rows(int dist_id, const float* gout, const float* table, const int64_t* idx,
                             size_t n_table_rows, const float* first, const float* second, const int32_t* slot,
                             const int32_t* slot_count, float* g_rows, float* g_first, float* g_second,
                             size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc,
                             size_t dim, void* stream) {
  if (!idx || !slot) return fail(SMORE_ERR_NULL, "backward_rows: idx or slot is NULL");
  return backward_common(dist_id, gout, table, idx, first, second, nullptr, slot, slot_count, g_rows,
                         g_first, g_second, Shape{bsize, num, be, ne, bc, nc, dim, n_table_rows}, stream);
}

int smore_box_forward(const float* ent, const int64_t* idx, size_t n_table_rows, const float* center,
                      const float* offset, float* dst_out, float* dst_in, size_t bsize, size_t num, size_t be,
                      size_t ne, size_t bc, size_t nc, size_t dim, void* stream) {
  if (!ent || !center || !offset || !dst_out || !dst_in)
    return fail(SMORE_ERR_NULL, "box_forward: required pointer is NULL");
  const Shape s{bsize, num, be, ne, bc, nc, dim, idx ? n_table_rows : 0};
  if (int rc = validate_shape(s)) return rc;
  return launch_forward<TermBoxBoth>(s, ent, idx, center, offset, dst_out, dst_in, (cudaStream_t)stream);
}

int smore_box_backward(const float* gout_out, const float* gout_in, const float* ent, const int64_t* idx,
                       size_t n_table_rows, const float* center, const float* offset, float* g_ent,
                       const int32_t* slot,
                       const int32_t* slot_count, float* g_rows, float* g_center, float* g_offset,
                       size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc, size_t dim,
                       void* stream) {
  if (!gout_out || !gout_in || !ent || !center || !offset || !g_center || !g_offset)
    return fail(SMORE_ERR_NULL, "box_backward: required pointer is NULL");
  if (idx ? (!slot || !g_rows || g_ent) : (!g_ent || slot || g_rows))
    return fail(SMORE_ERR_NULL, "box_backward: pass g_ent (materialised) or slot/g_rows (indexed)");
  const Shape s{bsize, num, be, ne, bc, nc, dim, idx ? n_table_rows : 0};
  if (int rc = validate_shape(s)) return rc;
  return launch_backward<TermBoxBoth>(s, gout_out, gout_in, ent, idx, center, offset, g_ent, slot, slot_count,
                                      g_rows, g_center, g_offset, (cudaStream_t)stream);
}

int smore_union_forward_rows(int dist_id, const float* table, const int64_t* idx, size_t n_table_rows,
                             const float* first, const float* second, float* dst0, float* dst1, size_t branches,
                             size_t bsize, size_t num, size_t dim, void* stream) {
  const bool both = dist_id == SMORE_DIST_BOX_BOTH;
  if (!both && (dist_id < 0 || dist_id >= SMORE_DIST_COUNT))
    return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", dist_id);
  if (!table || !idx || !first || !dst0 || (both && !dst1) || ((both || needs_second(dist_id)) && !second))
    return fail(SMORE_ERR_NULL, "union_forward_rows: required pointer is NULL");
  const Shape s{bsize, num, bsize, num, bsize, 1, dim, n_table_rows};
  cudaStream_t st = (cudaStream_t)stream;
  if (both) return launch_forward_union<TermBoxBoth>(branches, s, table, idx, first, second, dst0, dst1, st);
  SMORE_DISPATCH(dist_id, launch_forward_union<Term>(branches, s, table, idx, first, second, dst0, dst0, st));
}

int smore_union_backward_rows(int dist_id, const float* gout0, const float* gout1, const float* table,
                              const int64_t* idx, size_t n_table_rows, const float* first, const float* second,
                              const int32_t* slot,
                              const int32_t* slot_count, float* g_rows, float* g_first, float* g_second,
                              size_t branches, size_t bsize, size_t num, size_t dim, void* stream) {
  const bool both = dist_id == SMORE_DIST_BOX_BOTH;
  if (!both && (dist_id < 0 || dist_id >= SMORE_DIST_COUNT))
    return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", dist_id);
  const bool two = both || needs_second(dist_id);
  if (!gout0 || (both && !gout1) || !table || !idx || !first || !slot || !g_rows || !g_first ||
      (two && (!second || !g_second)))
    return fail(SMORE_ERR_NULL, "union_backward_rows: required pointer is NULL");
  const Shape s{bsize, num, bsize, num, bsize, 1, dim, n_table_rows};
  cudaStream_t st = (cudaStream_t)stream;
  if (both)
    return launch_backward_union<TermBoxBoth>(branches, s, gout0, gout1, table, idx, first, second, slot, slot_count,
                                              g_rows, g_first, g_second, st);
  SMORE_DISPATCH(dist_id, launch_backward_union<Term>(branches, s, gout0, gout0, table, idx, first, second, slot,
                                                      slot_count, g_rows, g_first, g_second, st));
}

int smore_rows_backward_fused_adam(int dist_id, const float* gout0, const float* gout1, float* table,
                                   const int64_t* idx, size_t n_table_rows, const float* first, const float* second,
                                   const int32_t* slot, const int32_t* slot_count, float* g_rows, float* g_first,
                                   float* g_second, size_t branches, size_t bsize, size_t num, size_t dim, float* m,
                                   float* v, int64_t* uniq, double lr, double beta1, double beta2, double eps,
                                   int64_t step, const float* step_scalars, void* stream) {
  const bool both = dist_id == SMORE_DIST_BOX_BOTH;
  if (!both && (dist_id < 0 || dist_id >= SMORE_DIST_COUNT))
    return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", dist_id);
  const bool two = both || needs_second(dist_id);
  if (!gout0 || (both && !gout1) || !table || !idx || !first || !slot || !slot_count || !g_rows || !g_first || !m ||
      !v || !uniq || (two && (!second || !g_second)))
    return fail(SMORE_ERR_NULL, "rows_backward_fused_adam: required pointer is NULL");
  if (branches != 1 && branches != (size_t)kUnionBranches)
    return fail(SMORE_ERR_BAD_SHAPE, "rows_backward_fused_adam: 1 or %d query branches", kUnionBranches);
  if (!step_scalars && step < 1) return fail(SMORE_ERR_BAD_SHAPE, "adam step must be >= 1");
  const Shape s{bsize, num, bsize, num, bsize, 1, dim, n_table_rows};
  if (int rc = validate_shape(s)) return rc;
  const size_t mul = (dist_id == SMORE_DIST_ROTATE || dist_id == SMORE_DIST_COMPLEX) ? 2 : 1;
  UpdateArgs ua;
  ua.table = table; ua.m = m; ua.v = v; ua.uniq = nullptr; ua.g_rows = nullptr; ua.n_unique = nullptr;
  ua.width = dim * mul;
  set_hyper(ua, lr, beta1, beta2, eps, step_scalars ? 1 : step, 1);
  ua.dyn = step_scalars;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = 0;
  if (both) {
    rc = backward_adam_common<TermBoxBoth>(branches, s, gout0, gout1, table, idx, first, second, slot, slot_count, g_rows,
                                           g_first, g_second, ua, uniq, st);
  } else {
    switch (dist_id) {
#define FUSED_CASE(ID, TERM)                                                                                        \
  case ID:                                                                                                          \
    rc = backward_adam_common<TERM>(branches, s, gout0, gout0, table, idx, first, second, slot, slot_count, g_rows, \
                                    g_first, g_second, ua, uniq, st);                                               \
    break;
      FUSED_CASE(SMORE_DIST_BOX_OUT, TermBoxOut)
      FUSED_CASE(SMORE_DIST_BOX_IN, TermBoxIn)
      FUSED_CASE(SMORE_DIST_ROTATE, TermRotate)
      FUSED_CASE(SMORE_DIST_L1, TermL1)
      FUSED_CASE(SMORE_DIST_L2, TermL2)
      FUSED_CASE(SMORE_DIST_COMPLEX, TermComplex)
      FUSED_CASE(SMORE_DIST_DISTMULT, TermDistmult)
#undef FUSED_CASE
    }
  }
  if (rc < 0) return rc;
  if (rc == 0)
    return fail(SMORE_ERR_BAD_SHAPE,
                "rows_backward_fused_adam: shape not covered (rows of 1 KB to about 4 KB, dim a multiple of 4, at "
                "least 4 rows per query, 16-byte aligned operands); use the separate backward and update calls");
  return SMORE_OK;
}

int smore_rows_forward_ragged(int dist_id, const float* table, const int64_t* rows, size_t n_table_rows,
                              const float* first, const float* second, const int32_t* segments, size_t n_segments,
                              size_t dim, float* out0, float* out1, const int32_t* positions,
                              size_t segments_per_rank, float* const* out0_ptrs, float* const* out1_ptrs,
                              size_t branches, size_t branch_stride, void* stream) {
  const bool both = dist_id == SMORE_DIST_BOX_BOTH;
  if (!both && (dist_id < 0 || dist_id >= SMORE_DIST_COUNT))
    return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", dist_id);
  if (!table || !rows || !first || !segments || ((both || needs_second(dist_id)) && !second))
    return fail(SMORE_ERR_NULL, "rows_forward_ragged: required pointer is NULL");
  if (positions ? (!out0_ptrs || (both && !out1_ptrs) || segments_per_rank == 0) : (!out0 || (both && !out1)))
    return fail(SMORE_ERR_NULL, "rows_forward_ragged: pass local result arrays, or positions with per-rank pointers");
  if (branches != 1 && (branches != (size_t)kUnionBranches || !positions))
    return fail(SMORE_ERR_BAD_SHAPE, "rows_forward_ragged: 1 branch, or %d with per-rank result arrays", kUnionBranches);
  const RaggedPeers pr{positions, segments_per_rank, branch_stride, out0_ptrs, both ? out1_ptrs : out0_ptrs, nullptr,
                       nullptr};
  if (n_segments == 0) return SMORE_OK;
  if (n_segments > (size_t)INT_MAX || dim == 0) return fail(SMORE_ERR_BAD_SHAPE, "rows_forward_ragged: bad sizes");
  cudaStream_t st = (cudaStream_t)stream;
  const int2* seg = reinterpret_cast<const int2*>(segments);
  int rc = 0;
  if (both) {
    rc = launch_forward_ragged<TermBoxBoth>(branches, n_segments, dim, n_table_rows, table, rows, first, second, seg, out0, out1, pr, st);
  } else {
    switch (dist_id) {
#define RAGGED_CASE(ID, TERM)                                                                                          \
  case ID:                                                                                                             \
    rc = launch_forward_ragged<TERM>(branches, n_segments, dim, n_table_rows, table, rows, first, second, seg, out0, out0, pr, st); \
    break;
      RAGGED_CASE(SMORE_DIST_BOX_OUT, TermBoxOut)
      RAGGED_CASE(SMORE_DIST_BOX_IN, TermBoxIn)
      RAGGED_CASE(SMORE_DIST_ROTATE, TermRotate)
      RAGGED_CASE(SMORE_DIST_L1, TermL1)
      RAGGED_CASE(SMORE_DIST_L2, TermL2)
      RAGGED_CASE(SMORE_DIST_COMPLEX, TermComplex)
      RAGGED_CASE(SMORE_DIST_DISTMULT, TermDistmult)
#undef RAGGED_CASE
    }
  }
  if (rc < 0) return rc;
  if (rc == 0)
    return fail(SMORE_ERR_BAD_SHAPE, "rows_forward_ragged: rows of 1 KB to about 6 KB, dim a multiple of 4 above 256, "
                                     "16-byte aligned operands");
  return SMORE_OK;
}

int smore_rows_backward_fused_adam_ragged(int dist_id, const float* gout0, const float* gout1, float* table,
                                          const int64_t* rows, size_t n_table_rows, const float* first,
                                          const float* second, const int32_t* segments, size_t n_segments,
                                          const int32_t* slot, const int32_t* slot_count, float* g_rows, float* g_first,
                                          float* g_second, size_t dim, float* m, float* v, int64_t* uniq, double lr,
                                          double beta1, double beta2, double eps, int64_t step,
                                          const float* step_scalars, const int32_t* positions,
                                          size_t segments_per_rank, const float* const* gout0_ptrs,
                                          const float* const* gout1_ptrs, size_t branches, size_t branch_stride,
                                          void* stream) {
  const bool both = dist_id == SMORE_DIST_BOX_BOTH;
  if (!both && (dist_id < 0 || dist_id >= SMORE_DIST_COUNT))
    return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", dist_id);
  const bool two = both || needs_second(dist_id);
  if (!table || !rows || !first || !segments || !slot || !slot_count || !g_rows || !g_first || !m || !v || !uniq ||
      (two && (!second || !g_second)))
    return fail(SMORE_ERR_NULL, "rows_backward_fused_adam_ragged: required pointer is NULL");
  if (positions ? (!gout0_ptrs || (both && !gout1_ptrs) || segments_per_rank == 0) : (!gout0 || (both && !gout1)))
    return fail(SMORE_ERR_NULL, "rows_backward_fused_adam_ragged: pass local upstream gradients, or positions with "
                                "per-rank pointers");
  if (branches != 1 && (branches != (size_t)kUnionBranches || !positions))
    return fail(SMORE_ERR_BAD_SHAPE, "rows_backward_fused_adam_ragged: 1 branch, or %d with per-rank upstream arrays",
                kUnionBranches);
  const RaggedPeers pr{positions, segments_per_rank, branch_stride, nullptr, nullptr, gout0_ptrs,
                       both ? gout1_ptrs : gout0_ptrs};
  if (!step_scalars && step < 1) return fail(SMORE_ERR_BAD_SHAPE, "adam step must be >= 1");
  if (n_segments == 0) return SMORE_OK;
  if (n_segments > (size_t)INT_MAX || dim == 0) return fail(SMORE_ERR_BAD_SHAPE, "rows_backward_fused_adam_ragged: bad sizes");
  const size_t mul = (dist_id == SMORE_DIST_ROTATE || dist_id == SMORE_DIST_COMPLEX) ? 2 : 1;
  UpdateArgs ua;
  ua.table = table; ua.m = m; ua.v = v; ua.uniq = nullptr; ua.g_rows = nullptr; ua.n_unique = nullptr;
  ua.width = dim * mul;
  set_hyper(ua, lr, beta1, beta2, eps, step_scalars ? 1 : step, 1);
  ua.dyn = step_scalars;
  cudaStream_t st = (cudaStream_t)stream;
  const int2* seg = reinterpret_cast<const int2*>(segments);
  int rc = 0;
  if (both) {
    rc = launch_backward_adam_ragged<TermBoxBoth>(branches, n_segments, dim, n_table_rows, gout0, gout1, table, rows, first, second,
                                                  seg, slot, slot_count, g_rows, g_first, g_second, ua, uniq, pr, st);
  } else {
    switch (dist_id) {
#define RAGGED_CASE(ID, TERM)                                                                                      \
  case ID:                                                                                                         \
    rc = launch_backward_adam_ragged<TERM>(branches, n_segments, dim, n_table_rows, gout0, gout0, table, rows, first, second, \
                                           seg, slot, slot_count, g_rows, g_first, g_second, ua, uniq, pr, st);    \
    break;
      RAGGED_CASE(SMORE_DIST_BOX_OUT, TermBoxOut)
      RAGGED_CASE(SMORE_DIST_BOX_IN, TermBoxIn)
      RAGGED_CASE(SMORE_DIST_ROTATE, TermRotate)
      RAGGED_CASE(SMORE_DIST_L1, TermL1)
      RAGGED_CASE(SMORE_DIST_L2, TermL2)
      RAGGED_CASE(SMORE_DIST_COMPLEX, TermComplex)
      RAGGED_CASE(SMORE_DIST_DISTMULT, TermDistmult)
#undef RAGGED_CASE
    }
  }
  if (rc < 0) return rc;
  if (rc == 0)
    return fail(SMORE_ERR_BAD_SHAPE, "rows_backward_fused_adam_ragged: rows of 1 KB to about 4 KB, dim a multiple of 4 "
                                     "above 256, 16-byte aligned operands");
  return SMORE_OK;
}

size_t smore_score_filtered_ranks_workspace_bytes(size_t n_queries, size_t n_answers) {
  const size_t scores = ((n_queries * n_answers * sizeof(float) + 255) / 256) * 256;
  return carve_rank_workspace(nullptr, n_answers).bytes + 2 * scores + 256;
}

int smore_score_filtered_ranks(int dist_id, const float* table, size_t n_candidates, const float* first,
                               const float* second, size_t n_queries, size_t dim, double gamma, double cen,
                               const int64_t* answer_ptr, const int64_t* answer_ids, size_t n_answers,
                               size_t max_answers, int64_t* ranks, void* workspace, size_t workspace_bytes,
                               void* stream) {
  if (n_queries == 0 || n_answers == 0) return SMORE_OK;
  const bool both = dist_id == SMORE_DIST_BOX_BOTH;
  if (!both && (dist_id < 0 || dist_id >= SMORE_DIST_COUNT))
    return fail(SMORE_ERR_BAD_DIST, "unknown distance id %d", dist_id);
  if (dist_id == SMORE_DIST_BOX_OUT || dist_id == SMORE_DIST_BOX_IN)
    return fail(SMORE_ERR_BAD_DIST, "score_filtered_ranks: Query2box logits need both distances (SMORE_DIST_BOX_BOTH)");
  const bool two = both || needs_second(dist_id);
  if (!table || !first || (two && !second) || !answer_ptr || !answer_ids || !ranks || !workspace)
    return fail(SMORE_ERR_NULL, "score_filtered_ranks: NULL pointer");
  if (workspace_bytes < smore_score_filtered_ranks_workspace_bytes(n_queries, n_answers) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(SMORE_ERR_WORKSPACE, "score_filtered_ranks: workspace too small or not 256-byte aligned");
  if (!second) second = first;
  const Shape s_all{n_queries, n_candidates, 1, n_candidates, n_queries, 1, dim, 0};
  const Shape s_ans{n_queries, n_answers, 1, n_answers, n_queries, 1, dim, n_candidates};
  if (int rc = validate_shape(s_all)) return rc;
  const bool aligned = aligned16(table) && aligned16(first) && aligned16(second);
  if (!shared_shape(s_all, aligned) || !shared_shape(s_ans, aligned) || max_answers == 0)
    return fail(SMORE_ERR_BAD_SHAPE,
                "score_filtered_ranks: needs 16-byte aligned operands, dim a multiple of 4, at least 8 queries, "
                "8 candidates and 8 answers in all");
  const RankWorkspace w = carve_rank_workspace(workspace, n_answers);
  const size_t scores = ((n_queries * n_answers * sizeof(float) + 255) / 256) * 256;
  float* d0 = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + w.bytes);
  float* d1 = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + w.bytes + scores);
  const int kind = (dist_id == SMORE_DIST_COMPLEX || dist_id == SMORE_DIST_DISTMULT) ? kLogitIdentity
                   : dist_id == SMORE_DIST_L2 ? kLogitGammaMinusSqrt : kLogitGammaMinus;
  cudaStream_t st = (cudaStream_t)stream;
  SharedArgs a_ans{table, answer_ids, first, second, (int)n_queries, (int)n_answers, (int)dim, (long long)n_candidates};
  SharedArgs a_all{table, nullptr, first, second, (int)n_queries, (int)n_candidates, (int)dim, 0};
  dim3 grid_ans((unsigned)((n_answers + kTileK - 1) / kTileK), (unsigned)((n_queries + kTileB - 1) / kTileB));
  dim3 grid_all((unsigned)((n_candidates + kTileK - 1) / kTileK), (unsigned)((n_queries + kTileB - 1) / kTileB));
  const int egrid = grid_for(n_queries * n_answers, 256);
#define SCORE_RANK(TERM)                                                                                          \
  {                                                                                                               \
    shared_forward_kernel<TERM><<<grid_ans, 256, 0, st>>>(a_ans, d0, d1);                                         \
    answer_logits_kernel<TERM::kNOut><<<egrid, 256, 0, st>>>(d0, d1, n_queries * n_answers, kind, (float)gamma,  \
                                                             (float)cen);                                         \
    count_launches(2);                                                                                            \
    if (int rc = rank_sort_answers(d0, n_answers, answer_ptr, answer_ids, true, n_queries, n_answers, max_answers, \
                                   w, st))                                                                        \
      return rc;                                                                                                  \
    score_rank_kernel<TERM><<<grid_all, 256, 0, st>>>(a_all, kind, (float)gamma, (float)cen, answer_ptr,          \
                                                      w.sorted_logit, w.sorted_id, w.hist);                       \
  }
  if (both) SCORE_RANK(TermBoxBoth)
  else if (dist_id == SMORE_DIST_ROTATE) SCORE_RANK(TermRotate)
  else if (dist_id == SMORE_DIST_L1) SCORE_RANK(TermL1)
  else if (dist_id == SMORE_DIST_L2) SCORE_RANK(TermL2)
  else if (dist_id == SMORE_DIST_COMPLEX) SCORE_RANK(TermComplex)
  else SCORE_RANK(TermDistmult)
#undef SCORE_RANK
  if (int rc = check_launch("score_rank_kernel")) return rc;
  return rank_finalize(answer_ptr, w, ranks, n_queries, st);
}

extern "C" int smore_peer_async_status(int* status);   // peer_kernels.cu (not part of the public header)
extern "C" int smore_rows_status(int* status);         // rows_kernels.cu (likewise)
extern "C" int smore_query_status(int* status);        // query_kernels.cu (likewise)
extern "C" int smore_peer_status_clear(void);
extern "C" int smore_rows_status_clear(void);
extern "C" int smore_query_status_clear(void);

int smore_async_status(int* status) {
  if (!status) return fail(SMORE_ERR_NULL, "async_status: NULL pointer");
  int v = 0, peer = 0, rows = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_async_status, sizeof(int));
  if (e != cudaSuccess) return fail(SMORE_ERR_CUDA, "async_status: %s", cudaGetErrorString(e));
  if (int rc = smore_peer_async_status(&peer)) return rc;   // the other files' kernels keep their own words
  if (int rc = smore_rows_status(&rows)) return rc;
  int query = 0;
  if (int rc = smore_query_status(&query)) return rc;
  *status = v | ((peer & 1) ? kStatusPeerWait : 0) | (peer & ~1) | rows | query;
  return SMORE_OK;
}

int smore_async_status_clear(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(SMORE_ERR_CUDA, "async_status_clear: device error");
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_async_status, &zero, sizeof(int)) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "async_status_clear: cannot write the status word");
  if (int rc = smore_peer_status_clear()) return rc;
  if (int rc = smore_query_status_clear()) return rc;
  return smore_rows_status_clear();
}

int smore_dist_forward_f64(int dist_id, const double* ent, const double* first, const double* second,
                           double* dst, size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc,
                           size_t dim, void* stream) {
  if (!ent || !first || !dst || (needs_second(dist_id) && !second))
    return fail(SMORE_ERR_NULL, "forward_f64: required pointer is NULL");
  const Shape s{bsize, num, be, ne, bc, nc, dim};
  if (int rc = validate_shape(s)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  SMORE_DISPATCH(dist_id, launch_forward_f64<Term>(s, ent, first, second, dst, st));
}

int smore_dist_backward_f64(int dist_id, const double* gout, const double* ent, const double* first,
                            const double* second, double* g_ent, double* g_first, double* g_second,
                            size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc, size_t dim,
                            void* stream) {
  if (!gout || !ent || !first || !g_ent || !g_first || (needs_second(dist_id) && (!second || !g_second)))
    return fail(SMORE_ERR_NULL, "backward_f64: required pointer is NULL");
  const Shape s{bsize, num, be, ne, bc, nc, dim};
  if (int rc = validate_shape(s)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  SMORE_DISPATCH(dist_id, launch_backward_f64<Term>(s, gout, ent, first, second, g_ent, g_first, g_second, st));
}

}  // extern "C"
