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

// ----------------------------------------------------------------------------------------
// The general form: any geometry, and the path may start from table rows named by index, so that
// the anchor rows are never gathered into a tensor of their own and their gradient goes straight
// into the step's compact gradient buffer (kg_reasoning.py:217-250 with the models' hooks).
//   geometry 0  additive          GQE (vec.py:58-60), Query2box (box.py:126-129)
//   geometry 1  rotation          RotatE: relation rows are phases, each hop multiplies the complex
//                                 state by cos(phase) + i sin(phase), phase = row * phase_scale
//                                 (rotate.py:101-109)
//   geometry 2  complex product   ComplEx: relation rows [re | im] (complex.py:108-117, identity normaliser)
//   geometry 3  product           DistMult (distmult.py:106-111, identity normaliser)
// State rows of the multiplicative geometries are [re | im] (2 * dim floats), dim floats for DistMult.
// ----------------------------------------------------------------------------------------

constexpr int kMaxHops = 8;
__device__ int g_query_status = 0;   // kStatusBadRowId: a start-row id lay outside the table

struct EmbedArgs {
  int geometry;
  const float* start;          // [B, W] rows, or the table when start_idx != nullptr
  const int64_t* start_idx;    // nullable [B]
  long long n_start_rows;
  const float* start_offset;   // additive: [B, D] or nullptr
  const float* rel;            // [R, D] ([R, 2D] for geometry 2)
  const float* off;            // additive: [R, D] or nullptr
  const int64_t* ids;
  size_t id_stride, B, H, D, R;
  int relu_offset;
  float phase_scale;
};

__device__ __forceinline__ void hop_multiplier(const EmbedArgs& a, size_t r, size_t d, float& c, float& s) {
  if (a.geometry == 1) {
    const float ph = __ldg(a.rel + r * a.D + d) * a.phase_scale;
    c = cosf(ph);
    s = sinf(ph);
  } else if (a.geometry == 2) {
    c = __ldg(a.rel + r * 2 * a.D + d);
    s = __ldg(a.rel + r * 2 * a.D + a.D + d);
  } else {
    c = __ldg(a.rel + r * a.D + d);
    s = 0.f;
  }
}

// one warp per query, lanes over the embedding dim
__global__ void __launch_bounds__(256)
    path_embed_forward_kernel(EmbedArgs a, float* __restrict__ out0, float* __restrict__ out1) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  const bool two = a.geometry == 1 || a.geometry == 2;
  const size_t W = two ? 2 * a.D : a.D;
  for (size_t b = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < a.B; b += warps) {
    long long row = (long long)b;
    if (a.start_idx) row = checked_row_id(a.start_idx, b, a.n_start_rows, &g_query_status);
    const bool bad = row < 0;
    const float* x = a.start + (size_t)(bad ? 0 : row) * W;
    for (size_t d = lane; d < a.D; d += 32) {
      float re = x[d], im = two ? x[a.D + d] : 0.f;
      if (a.geometry == 0) {
        float o = a.start_offset ? a.start_offset[b * a.D + d] : 0.f;
        for (size_t h = 0; h < a.H; ++h) {
          const size_t r = (size_t)a.ids[b * a.id_stride + h];
          if (r >= a.R) continue;
          re += __ldg(a.rel + r * a.D + d);
          if (a.off) {
            const float v = __ldg(a.off + r * a.D + d);
            o += a.relu_offset ? fmaxf(v, 0.f) : v;
          }
        }
        out0[b * a.D + d] = bad ? NAN : re;
        if (a.off) out1[b * a.D + d] = bad ? NAN : o;
        continue;
      }
      for (size_t h = 0; h < a.H; ++h) {
        const size_t r = (size_t)a.ids[b * a.id_stride + h];
        if (r >= a.R) continue;
        float c, s;
        hop_multiplier(a, r, d, c, s);
        if (two) {
          const float nre = re * c - im * s, nim = re * s + im * c;
          re = nre;
          im = nim;
        } else {
          re *= c;
        }
      }
      out0[b * a.D + d] = bad ? NAN : re;
      if (two) out1[b * a.D + d] = bad ? NAN : im;
    }
  }
}

struct EmbedGradArgs {
  const float* g0;             // gradient of out0 [B, D]
  const float* g1;             // gradient of out1 [B, D] (nullable)
  float* g_rel;                // dense [R, D] ([R, 2D] for geometry 2), zeroed before the launch
  float* g_off;                // additive, nullable
  float* g_start;              // dense [B, W], or nullptr when slot != nullptr
  const int32_t* slot;         // [B] -> row of g_rows (< 0: skip)
  const int32_t* slot_count;   // nullable: nullptr = accumulate everywhere
  float* g_rows;
};

__global__ void __launch_bounds__(256) path_embed_backward_kernel(EmbedArgs a, EmbedGradArgs ga) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
  const bool two = a.geometry == 1 || a.geometry == 2;
  const size_t W = two ? 2 * a.D : a.D;
  for (size_t b = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < a.B; b += warps) {
    long long row = (long long)b;
    if (a.start_idx) row = checked_row_id(a.start_idx, b, a.n_start_rows, &g_query_status);
    if (row < 0) continue;      // a start row that does not exist: no gradient from it or for it
    const float* x = a.geometry == 0 ? nullptr : a.start + (size_t)row * W;
    float* gs = nullptr;
    bool store = true;
    if (ga.slot) {
      const int32_t sl = ga.slot[b];
      if (sl >= 0) {
        gs = ga.g_rows + (size_t)sl * W;
        store = ga.slot_count != nullptr && ga.slot_count[sl] == 1;
      }
    } else if (ga.g_start) {
      gs = ga.g_start + b * W;
    }
    for (size_t d = lane; d < a.D; d += 32) {
      float gre = ga.g0[b * a.D + d], gim = (two && ga.g1) ? ga.g1[b * a.D + d] : 0.f;
      if (a.geometry == 0) {
        const float go = (ga.g_off && ga.g1) ? ga.g1[b * a.D + d] : 0.f;
        for (size_t h = 0; h < a.H; ++h) {
          const size_t r = (size_t)a.ids[b * a.id_stride + h];
          if (r >= a.R) continue;
          atomicAdd(ga.g_rel + r * a.D + d, gre);
          if (ga.g_off) {
            float g = go;
            if (a.relu_offset && !(__ldg(a.off + r * a.D + d) > 0.f)) g = 0.f;
            atomicAdd(ga.g_off + r * a.D + d, g);
          }
        }
      } else {
        // recompute the states before every hop, then walk the hops backwards
        float xre[kMaxHops], xim[kMaxHops], cs[kMaxHops], sn[kMaxHops];
        float re = x[d], im = two ? x[a.D + d] : 0.f;
        for (size_t h = 0; h < a.H; ++h) {
          xre[h] = re;
          xim[h] = im;
          const size_t r = (size_t)a.ids[b * a.id_stride + h];
          if (r >= a.R) {
            cs[h] = 1.f;
            sn[h] = 0.f;
            continue;
          }
          hop_multiplier(a, r, d, cs[h], sn[h]);
          if (two) {
            const float nre = re * cs[h] - im * sn[h], nim = re * sn[h] + im * cs[h];
            re = nre;
            im = nim;
          } else {
            re *= cs[h];
          }
        }
        for (int h = (int)a.H - 1; h >= 0; --h) {
          const size_t r = (size_t)a.ids[b * a.id_stride + h];
          if (r >= a.R) continue;
          const float g_c = gre * xre[h] + gim * xim[h];
          const float g_s = gim * xre[h] - gre * xim[h];
          if (a.geometry == 1)
            atomicAdd(ga.g_rel + r * a.D + d, (g_s * cs[h] - g_c * sn[h]) * a.phase_scale);
          else if (a.geometry == 2) {
            atomicAdd(ga.g_rel + r * 2 * a.D + d, g_c);
            atomicAdd(ga.g_rel + r * 2 * a.D + a.D + d, g_s);
          } else {
            atomicAdd(ga.g_rel + r * a.D + d, g_c);
          }
          const float nre = gre * cs[h] + gim * sn[h], nim = gim * cs[h] - gre * sn[h];
          gre = nre;
          gim = nim;
        }
      }
      if (gs != nullptr) {
        if (store) {
          gs[d] = gre;
          if (two) gs[a.D + d] = gim;
        } else {
          atomicAdd(gs + d, gre);
          if (two) atomicAdd(gs + a.D + d, gim);
        }
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

static int embed_check(const char* what, int geometry, size_t n_relations, size_t id_stride, size_t hops, size_t dim) {
  if (geometry < 0 || geometry > 3) return fail(SMORE_ERR_BAD_DIST, "%s: unknown geometry %d", what, geometry);
  if (dim == 0 || hops == 0 || id_stride < hops || n_relations == 0)
    return fail(SMORE_ERR_BAD_SHAPE, "%s: dim, hops, n_relations must be positive, id_stride >= hops", what);
  if (geometry != 0 && hops > (size_t)kMaxHops)
    return fail(SMORE_ERR_TOO_LARGE, "%s: at most %d hops per call for the multiplicative geometries", what, kMaxHops);
  return SMORE_OK;
}

int smore_path_embed_forward(int geometry, const float* start, const int64_t* start_idx, size_t n_start_rows,
                             const float* start_offset, const float* rel_table, const float* off_table,
                             size_t n_relations, const int64_t* rel_ids, size_t id_stride, size_t n_queries,
                             size_t hops, size_t dim, int relu_offset, double phase_scale, float* out0, float* out1,
                             void* stream) {
  if (n_queries == 0) return SMORE_OK;
  if (int rc = embed_check("path_embed_forward", geometry, n_relations, id_stride, hops, dim)) return rc;
  const bool two = geometry == 1 || geometry == 2;
  if (!start || !rel_table || !rel_ids || !out0 || ((two || (geometry == 0 && off_table)) && !out1))
    return fail(SMORE_ERR_NULL, "path_embed_forward: NULL pointer");
  EmbedArgs a{geometry, start, start_idx, start_idx ? (long long)n_start_rows : 0,
              geometry == 0 && off_table ? start_offset : nullptr, rel_table, geometry == 0 ? off_table : nullptr,
              rel_ids, id_stride, n_queries, hops, dim, n_relations, relu_offset != 0, (float)phase_scale};
  path_embed_forward_kernel<<<path_grid(n_queries), 256, 0, (cudaStream_t)stream>>>(a, out0, out1);
  return check_launch("path_embed_forward_kernel");
}

int smore_path_embed_backward(int geometry, const float* g_out0, const float* g_out1, const float* start,
                              const int64_t* start_idx, size_t n_start_rows, const float* rel_table,
                              const float* off_table, size_t n_relations, const int64_t* rel_ids, size_t id_stride,
                              size_t n_queries, size_t hops, size_t dim, int relu_offset, double phase_scale,
                              float* g_rel_table, float* g_off_table, float* g_start, const int32_t* slot,
                              const int32_t* slot_count, float* g_rows, void* stream) {
  if (int rc = embed_check("path_embed_backward", geometry, n_relations, id_stride, hops, dim)) return rc;
  if (!g_rel_table) return fail(SMORE_ERR_NULL, "path_embed_backward: g_rel_table is NULL");
  if (slot ? (!g_rows || g_start) : (g_rows != nullptr))
    return fail(SMORE_ERR_NULL, "path_embed_backward: pass g_start (rows given as a tensor) or slot / g_rows (table rows)");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t rel_width = geometry == 2 ? 2 * dim : dim;
  if (cudaMemsetAsync(g_rel_table, 0, n_relations * rel_width * sizeof(float), st) != cudaSuccess ||
      (geometry == 0 && g_off_table &&
       cudaMemsetAsync(g_off_table, 0, n_relations * dim * sizeof(float), st) != cudaSuccess))
    return fail(SMORE_ERR_CUDA, "path_embed_backward: cudaMemsetAsync failed");
  if (n_queries == 0) return SMORE_OK;
  if (!g_out0 || !rel_ids || (geometry != 0 && (!start || !rel_table)) ||
      (geometry == 0 && g_off_table && relu_offset && !off_table))
    return fail(SMORE_ERR_NULL, "path_embed_backward: NULL pointer");
  EmbedArgs a{geometry, start, start_idx, start_idx ? (long long)n_start_rows : 0, nullptr, rel_table,
              geometry == 0 ? off_table : nullptr, rel_ids, id_stride, n_queries, hops, dim, n_relations,
              relu_offset != 0, (float)phase_scale};
  EmbedGradArgs ga{g_out0, g_out1, g_rel_table, geometry == 0 ? g_off_table : nullptr, g_start, slot, slot_count, g_rows};
  path_embed_backward_kernel<<<path_grid(n_queries), 256, 0, st>>>(a, ga);
  return check_launch("path_embed_backward_kernel");
}

int smore_query_status(int* status) {    // not part of the public header; smore_async_status adds it in
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_query_status, sizeof(int)) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "async_status: cannot read the status word");
  *status = v;
  return SMORE_OK;
}

int smore_query_status_clear(void) {
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_query_status, &zero, sizeof(int)) != cudaSuccess)
    return fail(SMORE_ERR_CUDA, "async_status_clear: cannot write the status word");
  return SMORE_OK;
}

}  // extern "C"
