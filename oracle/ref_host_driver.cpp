// Host driver around the reference's OWN functor source.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit contains no distance math:
// it includes smore/common/torchext/dist_kernel.h from the mounted reference
// tree (via -I, never copied) and calls the functor classes defined there
// (DistOut, DistIn, DistRotate, DistL1, DistL2, DistComplex, Distmult) from
// plain host loops that walk the same cells, rows and jobs as
// smore/common/torchext/common_kernel.h:39-55, :62-88 and :95-122.
// g++ treats __device__ as an ignorable attribute, so the functors run on the
// CPU unchanged.  The library it produces (oracle/_ref/libsmore_ref_host.so)
// is used to validate the C restatement in smore_oracle.c and as the timed
// CPU baseline.
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>

// CUDA device intrinsics the functor header expects, supplied for the host.
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline double rsqrt(double x) { return 1.0 / sqrt(x); }

#include "dist_kernel.h"

namespace {

constexpr int kLanes = 32;

template <typename T>
T fold(T* v) {
  for (int mask = kLanes / 2; mask > 0; mask /= 2) {
    T t[kLanes];
    for (int l = 0; l < kLanes; ++l) t[l] = v[l] + v[l ^ mask];
    std::memcpy(v, t, sizeof(t));
  }
  return v[0];
}

template <typename T, class Dist>
void run_forward(size_t mul, Dist f, const T* ent, const T* first, const T* second, T* dst,
                 size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc, size_t dim) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t cell = 0; cell < (ptrdiff_t)(bsize * num); ++cell) {
    Dist g = f;
    size_t i = (size_t)cell / num, j = (size_t)cell % num;
    const T* pe = ent + ((i % be) * ne + (j % ne)) * dim * mul;
    const T* pc = first + ((i % bc) * nc + (j % nc)) * dim;
    const T* po = second + ((i % bc) * nc + (j % nc)) * dim;
    T lanes[kLanes];
    for (int l = 0; l < kLanes; ++l) {
      T s = 0;
      for (int d = l; d < (int)dim; d += kLanes) s += g.forward(pe, pc, po, d);
      lanes[l] = s;
    }
    dst[cell] = fold(lanes);
  }
}

template <typename T, class Dist>
void run_backward(size_t mul, Dist f, const T* gout, const T* ent, const T* first, const T* second,
                  T* g_ent, T* g_first, T* g_second, size_t bsize, size_t num, size_t be, size_t ne,
                  size_t bc, size_t nc, size_t dim) {
  {
    const size_t nji = bsize / be, njj = num / ne, njobs = nji * njj;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t row = 0; row < (ptrdiff_t)(be * ne); ++row) {
      Dist g = f;
      size_t r0 = (size_t)row / ne, r1 = (size_t)row % ne;
      const T* pe = ent + (size_t)row * dim * mul;
      T* gpe = g_ent + (size_t)row * dim * mul;
      for (int d = 0; d < (int)dim; ++d) {
        T l0[kLanes], l1[kLanes];
        for (int l = 0; l < kLanes; ++l) {
          T a0 = 0, a1 = 0, t0 = 0, t1 = 0;
          for (size_t job = (size_t)l; job < njobs; job += kLanes) {
            size_t i = (job / njj) * be + r0, j = (job % njj) * ne + r1;
            const T* pc = first + ((i % bc) * nc + (j % nc)) * dim;
            const T* po = second + ((i % bc) * nc + (j % nc)) * dim;
            g.backward(gout[i * num + j], pe, pc, po, d, a0, a1, t0, t1);
          }
          l0[l] = a0;
          l1[l] = a1;
        }
        g.update_ent(gpe, d, fold(l0), fold(l1));
      }
    }
  }
  {
    const size_t nji = bsize / bc, njj = num / nc, njobs = nji * njj;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t row = 0; row < (ptrdiff_t)(bc * nc); ++row) {
      Dist g = f;
      size_t r0 = (size_t)row / nc, r1 = (size_t)row % nc;
      const T* pc = first + (size_t)row * dim;
      const T* po = second + (size_t)row * dim;
      T* gpc = g_first + (size_t)row * dim;
      T* gpo = g_second + (size_t)row * dim;
      for (int d = 0; d < (int)dim; ++d) {
        T l0[kLanes], l1[kLanes];
        for (int l = 0; l < kLanes; ++l) {
          T t = 0, a0 = 0, a1 = 0;
          for (size_t job = (size_t)l; job < njobs; job += kLanes) {
            size_t i = (job / njj) * bc + r0, j = (job % njj) * nc + r1;
            const T* pe = ent + ((i % be) * ne + (j % ne)) * dim * mul;
            g.backward(gout[i * num + j], pe, pc, po, d, t, t, a0, a1);
          }
          l0[l] = a0;
          l1[l] = a1;
        }
        g.update_query(gpc, gpo, d, fold(l0), fold(l1));
      }
    }
  }
}

}  // namespace

// dist ids: 0 box_out, 1 box_in, 2 rotate, 3 l1, 4 l2, 5 complex, 6 distmult
// (the order of the name tests in smore/common/torchext/ext_cuda_kernel.cu:27-46,
// without the beta family).
extern "C" int ref_host_dist_forward(int id, const float* ent, const float* first,
                                     const float* second, float* dst, size_t bsize, size_t num,
                                     size_t be, size_t ne, size_t bc, size_t nc, size_t dim) {
  if (!second) second = first;
#define FWD(mul, functor) \
  run_forward<float>(mul, functor, ent, first, second, dst, bsize, num, be, ne, bc, nc, dim)
  switch (id) {
    case 0: FWD(1, DistOut<float>()); break;
    case 1: FWD(1, DistIn<float>()); break;
    case 2: FWD(2, DistRotate<float>((int)dim)); break;
    case 3: FWD(1, DistL1<float>()); break;
    case 4: FWD(1, DistL2<float>()); break;
    case 5: FWD(2, DistComplex<float>((int)dim)); break;
    case 6: FWD(1, Distmult<float>()); break;
    default: return -1;
  }
#undef FWD
  return 0;
}

extern "C" int ref_host_dist_backward(int id, const float* gout, const float* ent,
                                      const float* first, const float* second, float* g_ent,
                                      float* g_first, float* g_second, size_t bsize, size_t num,
                                      size_t be, size_t ne, size_t bc, size_t nc, size_t dim) {
  if (!second) second = first;
  if (!g_second) g_second = g_first;
#define BWD(mul, functor)                                                                      \
  run_backward<float>(mul, functor, gout, ent, first, second, g_ent, g_first, g_second, bsize, \
                      num, be, ne, bc, nc, dim)
  switch (id) {
    case 0: BWD(1, DistOut<float>()); break;
    case 1: BWD(1, DistIn<float>()); break;
    case 2: BWD(2, DistRotate<float>((int)dim)); break;
    case 3: BWD(1, DistL1<float>()); break;
    case 4: BWD(1, DistL2<float>()); break;
    case 5: BWD(2, DistComplex<float>((int)dim)); break;
    case 6: BWD(1, Distmult<float>()); break;
    default: return -1;
  }
#undef BWD
  return 0;
}
