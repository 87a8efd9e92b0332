// Per-element distance terms and their derivative rules.
//
// One struct per distance; all of them expose
//   kMul   entity row parts (1, or 2 for rows laid out [part0 | part1])
//   kNQ    query operands read (1 or 2)
//   kNOut  outputs produced per (entity row, query row) pair
//   fwd(e0, e1, q0, q1, acc[kNOut])                       adds one element's term(s)
//   bwd(g[kNOut], e0, e1, q0, q1, ge0, ge1, gq0, gq1)     adds one element's gradients
// Semantics, tie rules included, follow the reference functors
// (smore/common/torchext/dist_kernel.h): sign(0) counts as -1 (:74,:97,:141), the box
// "out" gradient flows when |e-c|-o is exactly 0 (:71), the box "in" test is strict (:94),
// and the rotation distance adds 1e-20 under the root (cuda_math_ext.h:21,100-118).
#pragma once
#include <cuda_runtime.h>

namespace smore {

template <typename T>
__device__ __forceinline__ T t_abs(T x) { return x < T(0) ? -x : x; }
template <>
__device__ __forceinline__ float t_abs<float>(float x) { return fabsf(x); }
template <>
__device__ __forceinline__ double t_abs<double>(double x) { return fabs(x); }
__device__ __forceinline__ float t_min(float a, float b) { return fminf(a, b); }
__device__ __forceinline__ double t_min(double a, double b) { return fmin(a, b); }
__device__ __forceinline__ float t_sqrt_eps(float s) { return sqrtf(s + 1e-20f); }
__device__ __forceinline__ double t_sqrt_eps(double s) { return sqrt(s + 1e-20); }
__device__ __forceinline__ float t_rsqrt_eps(float s) { return rsqrtf(s + 1e-20f); }
__device__ __forceinline__ double t_rsqrt_eps(double s) { return rsqrt(s + 1e-20); }
template <typename T>
__device__ __forceinline__ T t_sign(T x) { return x > T(0) ? T(1) : T(-1); }

struct TermBoxOut {
  static constexpr int kMul = 1, kNQ = 2, kNOut = 1;
  template <typename T>
  __device__ __forceinline__ static void fwd(T e0, T, T c, T o, T* acc) {
    T t = t_abs(e0 - c) - o;
    acc[0] += t > T(0) ? t : T(0);
  }
  template <typename T>
  __device__ __forceinline__ static void bwd(const T* g, T e0, T, T c, T o, T& ge0, T&, T& gc, T& go) {
    if (t_abs(e0 - c) - o >= T(0)) {
      T s = t_sign(e0 - c) * g[0];
      go -= g[0];
      ge0 += s;
      gc -= s;
    }
  }
};

struct TermBoxIn {
  static constexpr int kMul = 1, kNQ = 2, kNOut = 1;
  template <typename T>
  __device__ __forceinline__ static void fwd(T e0, T, T c, T o, T* acc) {
    acc[0] += t_abs(t_min(t_abs(e0 - c), o));
  }
  template <typename T>
  __device__ __forceinline__ static void bwd(const T* g, T e0, T, T c, T o, T& ge0, T&, T& gc, T& go) {
    T a = t_abs(e0 - c);
    T outer = t_sign(t_min(a, o)) * g[0];
    if (a < o) {
      T s = t_sign(e0 - c) * outer;
      ge0 += s;
      gc -= s;
    } else {
      go += outer;
    }
  }
};

// Both box distances of one operand pair in a single pass: acc[0] = out, acc[1] = in.
struct TermBoxBoth {
  static constexpr int kMul = 1, kNQ = 2, kNOut = 2;
  template <typename T>
  __device__ __forceinline__ static void fwd(T e0, T, T c, T o, T* acc) {
    T a = t_abs(e0 - c);
    T t = a - o;
    acc[0] += t > T(0) ? t : T(0);
    acc[1] += t_abs(t_min(a, o));
  }
  template <typename T>
  __device__ __forceinline__ static void bwd(const T* g, T e0, T, T c, T o, T& ge0, T&, T& gc, T& go) {
    // The two rules folded together.  For finite operands exactly one of "a < o" (the entity
    // gradient comes from the in-box term) and "a - o >= 0" (it comes from the out-of-box term,
    // and the in-box term feeds the offset) holds, so selects replace the branches.
    const T diff = e0 - c;
    const T a = t_abs(diff);
    const T outer = t_min(a, o) > T(0) ? g[1] : -g[1];
    const bool in_side = a < o;
    const T w = in_side ? outer : g[0];
    const T de = diff > T(0) ? w : -w;
    const T dofs = in_side ? T(0) : outer - g[0];
    ge0 += de;
    gc -= de;
    go += dofs;
  }
};

struct TermRotate {
  static constexpr int kMul = 2, kNQ = 2, kNOut = 1;
  template <typename T>
  __device__ __forceinline__ static void fwd(T e0, T e1, T re, T im, T* acc) {
    T a = e0 - re, b = e1 - im;
    acc[0] += t_sqrt_eps(a * a + b * b);
  }
  template <typename T>
  __device__ __forceinline__ static void bwd(const T* g, T e0, T e1, T re, T im, T& ge0, T& ge1, T& gre, T& gim) {
    T a = e0 - re, b = e1 - im;
    T den = t_rsqrt_eps(a * a + b * b);
    T x = a * den * g[0], y = b * den * g[0];
    ge0 += x;
    ge1 += y;
    gre -= x;
    gim -= y;
  }
};

struct TermL1 {
  static constexpr int kMul = 1, kNQ = 1, kNOut = 1;
  template <typename T>
  __device__ __forceinline__ static void fwd(T e0, T, T c, T, T* acc) { acc[0] += t_abs(e0 - c); }
  template <typename T>
  __device__ __forceinline__ static void bwd(const T* g, T e0, T, T c, T, T& ge0, T&, T& gc, T&) {
    T s = t_sign(e0 - c) * g[0];
    ge0 += s;
    gc -= s;
  }
};

struct TermL2 {
  static constexpr int kMul = 1, kNQ = 1, kNOut = 1;
  template <typename T>
  __device__ __forceinline__ static void fwd(T e0, T, T c, T, T* acc) {
    T a = e0 - c;
    acc[0] += a * a;
  }
  template <typename T>
  __device__ __forceinline__ static void bwd(const T* g, T e0, T, T c, T, T& ge0, T&, T& gc, T&) {
    T d = g[0] * (e0 - c) * T(2);
    ge0 += d;
    gc -= d;
  }
};

struct TermComplex {
  static constexpr int kMul = 2, kNQ = 2, kNOut = 1;
  template <typename T>
  __device__ __forceinline__ static void fwd(T e0, T e1, T re, T im, T* acc) { acc[0] += e0 * re + e1 * im; }
  template <typename T>
  __device__ __forceinline__ static void bwd(const T* g, T e0, T e1, T re, T im, T& ge0, T& ge1, T& gre, T& gim) {
    ge0 += re * g[0];
    ge1 += im * g[0];
    gre += e0 * g[0];
    gim += e1 * g[0];
  }
};

struct TermDistmult {
  static constexpr int kMul = 1, kNQ = 1, kNOut = 1;
  template <typename T>
  __device__ __forceinline__ static void fwd(T e0, T, T c, T, T* acc) { acc[0] += e0 * c; }
  template <typename T>
  __device__ __forceinline__ static void bwd(const T* g, T e0, T, T c, T, T& ge0, T&, T& gc, T&) {
    ge0 += c * g[0];
    gc += e0 * g[0];
  }
};

}  // namespace smore
