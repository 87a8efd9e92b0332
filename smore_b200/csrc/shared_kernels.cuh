// Kernels for the shared-candidate shape: one set of K candidate rows scored against every one of
// B queries (entity [1, K, W] or table + idx[K]; query [B, 1, dim]) — the reference's
// `--share_negative` training shape and its full-table evaluation shape.
//
// Every (query, candidate) pair re-uses rows that other pairs also use, so this shape is bound by
// fp32 ALU throughput and on-chip bandwidth, not by HBM: B*K*dim term evaluations against only
// (B + K)*dim*4 bytes.  The forward kernel is tiled like a SIMT matrix product (a 64 x 64 tile of
// cells per CTA, operands staged through shared memory, 4 x 4 cells per thread); the backward
// kernel evaluates every term once for both gradients: candidate-row gradients are summed in a fixed
// order (registers, then across a thread-block cluster), query gradients by floating-point
// reductions in L2.
//
// The reference runs this shape through the same three kernels as every other shape
// (smore/common/torchext/common_kernel.h:33-123): one warp per cell re-reading both rows from L2
// in the forward pass, and column-strided walks (one 32-byte sector per 4 useful bytes) in the
// backward pass.
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "dist_terms.cuh"

namespace smore {

constexpr int kTileB = 64;     // queries per CTA tile
constexpr int kTileK = 64;     // candidate rows per CTA tile
constexpr int kTileD = 16;     // embedding dims staged per step
constexpr int kTilePad = 4;    // keeps rows of the transposed tiles 16-byte aligned, off the same bank

struct SharedArgs {
  const float* ent;        // [K, W] or table when idx != nullptr
  const int64_t* idx;      // nullable [K]
  const float* first;      // [B, dim]
  const float* second;     // [B, dim]
  int B, K, dim;           // dim % 4 == 0
  long long n_rows;        // rows of `ent` when idx != nullptr (0: ids are not checked)
};

// Device status word of the distance kernels (kStatus* bits): a bulk-copy wait that gave up, a row
// id outside the table.  Either makes the results of the launch invalid; smore_async_status reads
// it.  (Defined here because this header is part of exactly one translation unit, dist_kernels.cu.)
__device__ int g_async_status = 0;

// Shared memory of one 64 x 64 tile of scores.
template <class Term>
struct TileSmem {
  float q0s[kTileD][kTileB + kTilePad];
  float q1s[kTileD][kTileB + kTilePad];
  float e0s[kTileD][kTileK + kTilePad];
  float e1s[Term::kMul == 2 ? kTileD : 1][kTileK + kTilePad];
  unsigned char ebad[kTileK];   // candidate rows of the tile whose id lay outside the table
};

// Scores of the tile (queries b0.., candidates k0..) into acc: thread (ty, tx) owns queries
// b0 + 4 ty + i and candidates k0 + 4 tx + j.  Every cell accumulates its terms in the order of the
// embedding dim, one after the other, so a (query, candidate) pair gets the same value wherever it
// falls in a tile and whatever the tile's neighbours are.
template <class Term>
__device__ __forceinline__ void tile_scores(const SharedArgs& a, TileSmem<Term>& sm, int b0, int k0,
                                            float (&acc)[4][4][Term::kNOut]) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int dim4 = a.dim >> 2;
  const size_t w4 = (size_t)dim4 * Term::kMul;
  // staging role: one 16-byte piece of one row per operand per step
  const int lrow = threadIdx.x >> 2, lq = threadIdx.x & 3;
  const bool qrow_ok = b0 + lrow < a.B, erow_ok = k0 + lrow < a.K;
  const float4* q0p = reinterpret_cast<const float4*>(a.first) + (size_t)(qrow_ok ? b0 + lrow : 0) * dim4;
  const float4* q1p = reinterpret_cast<const float4*>(a.second) + (size_t)(qrow_ok ? b0 + lrow : 0) * dim4;
  size_t erow = 0;
  if (erow_ok) {
    const long long r = a.idx ? checked_row_id(a.idx, k0 + lrow, a.n_rows, &g_async_status) : (long long)(k0 + lrow);
    erow = r < 0 ? 0 : (size_t)r;
    if (lq == 0) sm.ebad[lrow] = r < 0;
  } else if (lq == 0) {
    sm.ebad[lrow] = 0;
  }
  const float4* e0p = reinterpret_cast<const float4*>(a.ent) + erow * w4;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int o = 0; o < Term::kNOut; ++o) acc[i][j][o] = 0.f;

  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int d0 = 0; d0 < a.dim; d0 += kTileD) {
    const int d4 = (d0 >> 2) + lq;
    const bool d_ok = d4 < dim4;
    const float4 vq0 = (qrow_ok && d_ok) ? __ldg(q0p + d4) : z4;
    const float4 vq1 = (Term::kNQ == 2 && qrow_ok && d_ok) ? __ldg(q1p + d4) : z4;
    const float4 ve0 = (erow_ok && d_ok) ? __ldg(e0p + d4) : z4;
    const float4 ve1 = (Term::kMul == 2 && erow_ok && d_ok) ? __ldg(e0p + dim4 + d4) : z4;
    __syncthreads();  // the previous step's tiles are no longer being read
    sm.q0s[lq * 4 + 0][lrow] = vq0.x; sm.q0s[lq * 4 + 1][lrow] = vq0.y; sm.q0s[lq * 4 + 2][lrow] = vq0.z; sm.q0s[lq * 4 + 3][lrow] = vq0.w;
    if (Term::kNQ == 2) {
      sm.q1s[lq * 4 + 0][lrow] = vq1.x; sm.q1s[lq * 4 + 1][lrow] = vq1.y; sm.q1s[lq * 4 + 2][lrow] = vq1.z; sm.q1s[lq * 4 + 3][lrow] = vq1.w;
    }
    sm.e0s[lq * 4 + 0][lrow] = ve0.x; sm.e0s[lq * 4 + 1][lrow] = ve0.y; sm.e0s[lq * 4 + 2][lrow] = ve0.z; sm.e0s[lq * 4 + 3][lrow] = ve0.w;
    if (Term::kMul == 2) {
      sm.e1s[lq * 4 + 0][lrow] = ve1.x; sm.e1s[lq * 4 + 1][lrow] = ve1.y; sm.e1s[lq * 4 + 2][lrow] = ve1.z; sm.e1s[lq * 4 + 3][lrow] = ve1.w;
    }
    __syncthreads();
    const int dcount = min(kTileD, a.dim - d0);
#pragma unroll 4
    for (int dd = 0; dd < dcount; ++dd) {
      const float4 q0 = *reinterpret_cast<const float4*>(&sm.q0s[dd][ty * 4]);
      const float4 q1 = Term::kNQ == 2 ? *reinterpret_cast<const float4*>(&sm.q1s[dd][ty * 4]) : q0;
      const float4 e0 = *reinterpret_cast<const float4*>(&sm.e0s[dd][tx * 4]);
      const float4 e1 = Term::kMul == 2 ? *reinterpret_cast<const float4*>(&sm.e1s[dd][tx * 4]) : e0;
      const float qa[4] = {q0.x, q0.y, q0.z, q0.w}, qb[4] = {q1.x, q1.y, q1.z, q1.w};
      const float ea[4] = {e0.x, e0.y, e0.z, e0.w}, eb[4] = {e1.x, e1.y, e1.z, e1.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) Term::fwd(ea[j], eb[j], qa[i], qb[i], acc[i][j]);
    }
  }
}

template <class Term>
__global__ void __launch_bounds__(256)
    shared_forward_kernel(SharedArgs a, float* __restrict__ dst0, float* __restrict__ dst1) {
  __shared__ __align__(16) TileSmem<Term> sm;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int b0 = blockIdx.y * kTileB, k0 = blockIdx.x * kTileK;
  float acc[4][4][Term::kNOut];
  tile_scores<Term>(a, sm, b0, k0, acc);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int b = b0 + ty * 4 + i;
    if (b >= a.B) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + tx * 4 + j;
      if (k < a.K) {
        const bool bad = sm.ebad[tx * 4 + j];   // written before the first barrier of the tile loop
        dst0[(size_t)b * a.K + k] = bad ? NAN : acc[i][j][0];
        if (Term::kNOut == 2) dst1[(size_t)b * a.K + k] = bad ? NAN : acc[i][j][Term::kNOut - 1];
      }
    }
  }
}

struct SharedGradArgs {
  const float* gout0;         // [B, K]
  const float* gout1;         // [B, K] (two-output term only)
  float* g_ent;               // dense [K, W], or nullptr when slot != nullptr
  const int32_t* slot;        // [K] -> row of g_rows (< 0: skip)
  const int32_t* slot_count;  // nullable: nullptr = accumulate everywhere
  float* g_rows;
  float* g_first;             // [B, dim]
  float* g_second;            // [B, dim]
};

// ---- both gradients of the shared-candidate shape from ONE evaluation of every term ----
//
// Thread = one embedding dim d; CTA = KT candidate rows x a segment of the queries x blockDim.x
// dims.  The thread keeps e[k, d] and its gradient for the KT rows in registers and walks the
// segment's queries: per query it loads q[b, d], evaluates the KT terms (upstream gradients
// broadcast from shared memory) and sends the query's partial gradient (the sum over the CTA's KT
// rows) to g_first / g_second with one coalesced reduction per warp, so those must be zero at
// launch.  The CTAs that share rows and dims but hold different query segments form one
// thread-block cluster: at the end they add their row gradients through distributed shared memory
// in rank order (deterministic) and each rank writes KT / cluster-size of the rows.
constexpr int kBwdChunkB = 64;    // queries whose upstream gradients are staged at a time
constexpr int kBwdAhead = 4;      // query rows loaded ahead of the one being used
constexpr int kBwdMaxThreads = 512;

template <class Term, int KT>
__global__ void __launch_bounds__(kBwdMaxThreads)
    shared_backward_tile_kernel(SharedArgs a, SharedGradArgs ga, int seg_b) {
  static_assert((KT * Term::kNOut) % 4 == 0, "a query's upstream gradients are read 16 bytes at a time");
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  constexpr int NO = Term::kNOut, M = Term::kMul;
  __shared__ __align__(16) float gs[kBwdChunkB][KT][NO];
  __shared__ long long rows_sh[KT];
  extern __shared__ float tile_red[];   // [KT * M][blockDim.x]
  float* red = tile_red;

  const int tid = threadIdx.x, T = blockDim.x;
  const int k0 = blockIdx.x * KT;
  const int d = blockIdx.z * T + tid;
  const bool d_ok = d < a.dim;
  const bool warp_live = blockIdx.z * T + (tid & ~31) < a.dim;   // warps past the last dim only take part in barriers
  const unsigned rank = cluster.block_rank(), n_ranks = cluster.num_blocks();
  const int b_begin = min(a.B, (int)rank * seg_b), b_end = min(a.B, b_begin + seg_b);

  if (tid < KT) {
    const int k = k0 + tid;
    rows_sh[tid] = k < a.K ? (a.idx ? checked_row_id(a.idx, k, a.n_rows, &g_async_status) : (long long)k) : -1;
  }
  __syncthreads();
  const size_t W = (size_t)a.dim * M;
  float e0[KT], e1[KT], ge0[KT], ge1[KT];
#pragma unroll
  for (int j = 0; j < KT; ++j) {
    const long long r = rows_sh[j];
    const bool ok = r >= 0 && d_ok;
    e0[j] = ok ? __ldg(a.ent + (size_t)r * W + d) : 0.f;
    e1[j] = (M == 2 && ok) ? __ldg(a.ent + (size_t)r * W + a.dim + d) : e0[j];
    ge0[j] = 0.f;
    ge1[j] = 0.f;
  }
  const float* __restrict__ q0p = a.first + d;
  const float* __restrict__ q1p = a.second + d;

  for (int bs = b_begin; bs < b_end; bs += kBwdChunkB) {
    const int nb = min(kBwdChunkB, b_end - bs);
    __syncthreads();   // the previous chunk's gradients are no longer being read
    // upstream gradients of the chunk; zero for rows that do not exist, so their terms add nothing
    for (int i = tid; i < nb * KT; i += T) {
      const int bb = i / KT, j = i % KT;
      const bool ok = rows_sh[j] >= 0;
      const size_t at = (size_t)(bs + bb) * a.K + k0 + j;
      gs[bb][j][0] = ok ? __ldg(ga.gout0 + at) : 0.f;
      if (NO == 2) gs[bb][j][NO - 1] = ok ? __ldg(ga.gout1 + at) : 0.f;
    }
    __syncthreads();
    if (!warp_live) continue;
    float q0n[kBwdAhead], q1n[kBwdAhead];
#pragma unroll
    for (int u = 0; u < kBwdAhead; ++u) {
      const bool ok = d_ok && u < nb;
      q0n[u] = ok ? __ldg(q0p + (size_t)(bs + u) * a.dim) : 0.f;
      q1n[u] = (Term::kNQ == 2 && ok) ? __ldg(q1p + (size_t)(bs + u) * a.dim) : q0n[u];
    }
    for (int bb0 = 0; bb0 < nb; bb0 += kBwdAhead) {
      float q0c[kBwdAhead], q1c[kBwdAhead];
#pragma unroll
      for (int u = 0; u < kBwdAhead; ++u) {
        q0c[u] = q0n[u];
        q1c[u] = q1n[u];
        const int bn = bb0 + kBwdAhead + u;
        const bool ok = d_ok && bn < nb;
        q0n[u] = ok ? __ldg(q0p + (size_t)(bs + bn) * a.dim) : 0.f;
        q1n[u] = (Term::kNQ == 2 && ok) ? __ldg(q1p + (size_t)(bs + bn) * a.dim) : q0n[u];
      }
#pragma unroll
      for (int u = 0; u < kBwdAhead; ++u) {
        const int bb = bb0 + u;
        if (bb >= nb) break;
        float gq0 = 0.f, gq1 = 0.f;
        // the query's KT x NO upstream gradients: a few 16-byte broadcast loads instead of one load per value
        float gl[KT * NO];
        const float4* g4 = reinterpret_cast<const float4*>(&gs[bb][0][0]);
#pragma unroll
        for (int i = 0; i < KT * NO / 4; ++i) {
          const float4 t = g4[i];
          gl[4 * i + 0] = t.x; gl[4 * i + 1] = t.y; gl[4 * i + 2] = t.z; gl[4 * i + 3] = t.w;
        }
#pragma unroll
        for (int j = 0; j < KT; ++j) Term::bwd(&gl[j * NO], e0[j], e1[j], q0c[u], q1c[u], ge0[j], ge1[j], gq0, gq1);
        if (d_ok) {
          const size_t at = (size_t)(bs + bb) * a.dim + d;
          atomicAdd(ga.g_first + at, gq0);
          if (Term::kNQ == 2) atomicAdd(ga.g_second + at, gq1);
        }
      }
    }
  }

  // row gradients: sum over the cluster's query segments in rank order
#pragma unroll
  for (int j = 0; j < KT; ++j) {
    red[(j * M) * T + tid] = ge0[j];
    if (M == 2) red[(j * M + M - 1) * T + tid] = ge1[j];
  }
  cluster.sync();
  for (int j = (int)rank; j < KT; j += (int)n_ranks) {
    const int k = k0 + j;
    if (k >= a.K || rows_sh[j] < 0 || !d_ok) continue;
    float s0 = 0.f, s1 = 0.f;
    for (unsigned r = 0; r < n_ranks; ++r) {
      const float* remote = cluster.map_shared_rank(red, r);
      s0 += remote[(j * M) * T + tid];
      if (M == 2) s1 += remote[(j * M + M - 1) * T + tid];
    }
    if (ga.slot == nullptr) {
      ga.g_ent[(size_t)k * W + d] = s0;
      if (M == 2) ga.g_ent[(size_t)k * W + a.dim + d] = s1;
    } else {
      const int32_t s = ga.slot[k];
      if (s < 0) continue;
      float* out = ga.g_rows + (size_t)s * W + d;
      if (ga.slot_count != nullptr && ga.slot_count[s] == 1) {
        out[0] = s0;
        if (M == 2) out[a.dim] = s1;
      } else {
        atomicAdd(out, s0);
        if (M == 2) atomicAdd(out + a.dim, s1);
      }
    }
  }
  cluster.sync();   // no CTA leaves while another still reads its shared memory
}

}  // namespace smore
