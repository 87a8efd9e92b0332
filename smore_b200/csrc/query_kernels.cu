// Relation projection of a batch of path queries in one pass, for the additive geometries.
//
// The reference embeds a path query hop by hop (smore/models/kg_reasoning.py:229-236): every hop
// looks up the relation rows of the batch and adds them to the running embedding
// (GQE: vec.py:58-60; Query2box: box.py:126-129, where the box offset grows by the relation's
// offset row, optionally passed through relu).  Per hop that is two lookups, two additions and, in
// backward, two sort-based index_put kernels.  Here all H hops of a batch are one kernel each way:
//   center[b] = start_center[b] + sum_h rel[ids[b, h]]            (added in hop order)
//   offset[b] = start_offset[b] + sum_h act(off[ids[b, h]])       (Query2box only)
// and the backward pass adds the output gradients to the H relation rows of every query.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "common.cuh"

namespace smore {

struct PathArgs {
  const float* start_center;   // [B, D]
  const float* start_offset;   // [B, D] or nullptr (zero)
  const float* rel;            // [R, D]
  const float* off;            // [R, D] or nullptr (no offset part)
  const int64_t* ids;          // ids[b * id_stride + h]
  size_t id_stride, B, H, D, R;
  int relu_offset;
};

template <bool VEC>
__global__ void __launch_bounds__(256)
    path_project_forward_kernel(PathArgs a, float* __restrict__ center, float* __restrict__ offset) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  constexpr int V = VEC ? 4 : 1;
  for (size_t b = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < a.B; b += warps) {
    for (size_t d = (size_t)lane * V; d < a.D; d += 32 * V) {
      float c[V], o[V];
#pragma unroll
      for (int k = 0; k < V; ++k) {
        c[k] = a.start_center[b * a.D + d + k];
        o[k] = a.start_offset ? a.start_offset[b * a.D + d + k] : 0.f;
      }
      for (size_t h = 0; h < a.H; ++h) {
        const size_t r = (size_t)a.ids[b * a.id_stride + h];
        if (r >= a.R) continue;   // out-of-range relation id: contributes nothing
#pragma unroll
        for (int k = 0; k < V; ++k) {
          c[k] += __ldg(a.rel + r * a.D + d + k);
          if (a.off) {
            const float x = __ldg(a.off + r * a.D + d + k);
            o[k] += a.relu_offset ? fmaxf(x, 0.f) : x;
          }
        }
      }
#pragma unroll
      for (int k = 0; k < V; ++k) {
        center[b * a.D + d + k] = c[k];
        if (a.off) offset[b * a.D + d + k] = o[k];
      }
    }
  }
}

// one warp per (query, hop): the relation row's gradient += the query's output gradient
__global__ void __launch_bounds__(256)
    path_project_backward_kernel(PathArgs a, const float* __restrict__ g_center, const float* __restrict__ g_offset,
                                 float* __restrict__ g_rel, float* __restrict__ g_off) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  const size_t total = a.B * a.H;
  for (size_t p = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < total; p += warps) {
    const size_t b = p / a.H, h = p - b * a.H;
    const size_t r = (size_t)a.ids[b * a.id_stride + h];
    if (r >= a.R) continue;
    for (size_t d = lane; d < a.D; d += 32) {
      atomicAdd(g_rel + r * a.D + d, g_center[b * a.D + d]);
      if (g_off) {
        float g = g_offset[b * a.D + d];
        if (a.relu_offset && !(__ldg(a.off + r * a.D + d) > 0.f)) g = 0.f;
        atomicAdd(g_off + r * a.D + d, g);
      }
    }
  }
}

static int path_grid(size_t warps_needed) {
  return (int)std::max<size_t>(1, std::min<size_t>((warps_needed + 7) / 8, (size_t)sm_count() * 16));
}

}  // namespace smore

using namespace smore;

extern "C" {

int smore_path_project_forward(const float* start_center, const float* start_offset, const float* rel_table,
                               const float* off_table, size_t n_relations, const int64_t* rel_ids, size_t id_stride,
                               size_t n_queries, size_t hops, size_t dim, int relu_offset, float* center,
                               float* offset, void* stream) {
  if (n_queries == 0) return SMORE_OK;
  if (!start_center || !rel_table || !rel_ids || !center || (off_table && !offset))
    return fail(SMORE_ERR_NULL, "path_project_forward: NULL pointer");
  if (dim == 0 || hops == 0 || id_stride < hops || n_relations == 0)
    return fail(SMORE_ERR_BAD_SHAPE, "path_project_forward: dim, hops, n_relations must be positive, id_stride >= hops");
  PathArgs a{start_center, off_table ? start_offset : nullptr, rel_table, off_table, rel_ids, id_stride, n_queries,
             hops, dim, n_relations, relu_offset != 0};
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (dim % 4 == 0) && aligned16(start_center) && aligned16(rel_table) && aligned16(center) &&
                   (!off_table || (aligned16(off_table) && aligned16(offset) &&
                                   (!start_offset || aligned16(start_offset))));
  if (vec) path_project_forward_kernel<true><<<path_grid(n_queries), 256, 0, st>>>(a, center, offset);
  else path_project_forward_kernel<false><<<path_grid(n_queries), 256, 0, st>>>(a, center, offset);
  return check_launch("path_project_forward_kernel");
}

int smore_path_project_backward(const float* g_center, const float* g_offset, const float* off_table,
                                size_t n_relations, const int64_t* rel_ids, size_t id_stride, size_t n_queries,
                                size_t hops, size_t dim, int relu_offset, float* g_rel_table, float* g_off_table,
                                void* stream) {
  if (!g_rel_table || (g_off_table && (!g_offset || (relu_offset && !off_table))))
    return fail(SMORE_ERR_NULL, "path_project_backward: NULL pointer");
  if (dim == 0 || hops == 0 || id_stride < hops || n_relations == 0)
    return fail(SMORE_ERR_BAD_SHAPE, "path_project_backward: dim, hops, n_relations must be positive, id_stride >= hops");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t bytes = n_relations * dim * sizeof(float);
  if (cudaMemsetAsync(g_rel_table, 0, bytes, st) != cudaSuccess ||
      (g_off_table && cudaMemsetAsync(g_off_table, 0, bytes, st) != cudaSuccess))
    return fail(SMORE_ERR_CUDA, "path_project_backward: cudaMemsetAsync failed");
  if (n_queries == 0) return SMORE_OK;
  if (!g_center || !rel_ids) return fail(SMORE_ERR_NULL, "path_project_backward: NULL pointer");
  PathArgs a{nullptr, nullptr, nullptr, off_table, rel_ids, id_stride, n_queries, hops, dim, n_relations,
             relu_offset != 0};
  path_project_backward_kernel<<<path_grid(n_queries * hops), 256, 0, st>>>(a, g_center, g_off_table ? g_offset : nullptr,
                                                                            g_rel_table, g_off_table);
  return check_launch("path_project_backward_kernel");
}

}  // extern "C"
