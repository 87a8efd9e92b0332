// Per-element arithmetic of the row-wise Adam update, shared by the single-GPU kernels
// (rows_kernels.cu) and the sharded pull-reduce-update kernel (peer_kernels.cu).
// Restates smore/common/embedding/embed_optimizer.py:208-252.
#pragma once
#include <cuda_runtime.h>

#include <cmath>
#include <cstddef>
#include <cstdint>

namespace smore {

struct UpdateArgs {
  float* table;
  float* m;
  float* v;
  const int64_t* uniq;
  const float* g_rows;
  const int32_t* n_unique;
  size_t width;
  float lr, beta1, beta2, omb1, omb2, eps, step_size, sqrt_bc2;
  int squeeze;
  const float* dyn;  // nullable: device [2] = {step_size, sqrt_bc2}, overrides the two fields above
};

// Hyper-parameters arrive as doubles (Python floats in the reference) and are narrowed once,
// where they would meet a float tensor there.
inline void set_hyper(UpdateArgs& a, double lr, double beta1, double beta2, double eps, int64_t step,
                      int squeeze) {
  const double bc1 = 1.0 - std::pow(beta1, (double)step);
  const double bc2 = 1.0 - std::pow(beta2, (double)step);
  a.lr = (float)lr;
  a.beta1 = (float)beta1;
  a.beta2 = (float)beta2;
  a.omb1 = (float)(1.0 - beta1);
  a.omb2 = (float)(1.0 - beta2);
  a.eps = (float)eps;
  a.step_size = (float)(-lr / bc1);
  a.sqrt_bc2 = (float)std::sqrt(bc2);
  a.squeeze = squeeze != 0;
  a.dyn = nullptr;
}

// The two scalars that depend on the optimizer's step count may come from device memory (written
// by adam_step_scalars_kernel from a step counter that lives on the device), so that a captured
// CUDA graph can be replayed step after step.
__device__ __forceinline__ void load_dyn(UpdateArgs& a) {
  if (a.dyn != nullptr) {
    a.step_size = a.dyn[0];
    a.sqrt_bc2 = a.dyn[1];
  }
}

__device__ __forceinline__ void adam_elem(float g, float& p, float& m, float& v, const UpdateArgs& a) {
  const float v_new = v * a.beta2 + g * g * a.omb2;
  const float m_new = m * a.beta1 + g * a.omb1;
  const float denom = sqrtf(v_new) / a.sqrt_bc2 + a.eps;
  p += a.step_size * m_new / denom;
  m = m + (m_new - m);  // the reference stores state as old + (new - old), embed_optimizer.py:251-252
  v = v + (v_new - v);
}

__device__ __forceinline__ void adam_elem_rowwise(float g, float& p, float& m, float denom,
                                                  const UpdateArgs& a) {
  const float m_new = m * a.beta1 + g * a.omb1;
  p += a.step_size * m_new / denom;
  m = m + (m_new - m);
}

}  // namespace smore
