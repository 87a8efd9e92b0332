// C entry points around the reference's OWN CUDA kernels.
//
// TEST / MEASUREMENT INFRASTRUCTURE ONLY.  Compiled together with
// smore/common/torchext/ext_cuda_kernel.cu straight from the mounted
// reference tree (nothing is copied) into oracle/_ref/libsmore_ref_cuda.so.
// It forwards to DistImpl<float> (smore/common/torchext/ext_cuda_kernel.h:24-32)
// so the reference kernels, recompiled for sm_100a, can serve as a GPU-side
// cross-check and as the "kernel to beat" in measurements.
#include <cuda_runtime.h>

#include <string>

#include "ext_cuda_kernel.h"

static const char* kNames[] = {"box_out", "box_in", "rotate", "l1", "l2", "complex", "distmult"};

extern "C" int ref_cuda_dist_forward(int id, const float* ent, const float* first,
                                     const float* second, float* dst, size_t bsize, size_t num,
                                     size_t be, size_t ne, size_t bc, size_t nc, size_t dim,
                                     void* stream) {
  if (id < 0 || id > 6) return -1;
  DistImpl<float> impl{std::string(kNames[id])};
  impl.forward((cudaStream_t)stream, ent, first, second ? second : first, dst, bsize, num, be, ne,
               bc, nc, dim);
  return (int)cudaGetLastError();
}

extern "C" int ref_cuda_dist_backward(int id, const float* gout, const float* ent,
                                      const float* first, const float* second, float* g_ent,
                                      float* g_first, float* g_second, size_t bsize, size_t num,
                                      size_t be, size_t ne, size_t bc, size_t nc, size_t dim,
                                      void* stream) {
  if (id < 0 || id > 6) return -1;
  DistImpl<float> impl{std::string(kNames[id])};
  impl.backward((cudaStream_t)stream, gout, ent, first, second ? second : first, g_ent, g_first,
                g_second ? g_second : g_first, bsize, num, be, ne, bc, nc, dim);
  return (int)cudaGetLastError();
}
