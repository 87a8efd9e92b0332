/*
 * CPU oracle for the distance-op / sparse-row-update hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product package may call this
 * file; it exists so the CUDA kernels can be checked against an independent,
 * plain-C restatement of the reference algorithm, and so a CPU baseline can
 * be timed beside the GPU numbers.
 *
 * What it restates (paths are relative to the reference project root):
 *   - the per-element distance terms and their derivative rules:
 *       smore/common/torchext/dist_kernel.h:58-79   (box "out")
 *       smore/common/torchext/dist_kernel.h:82-105  (box "in")
 *       smore/common/torchext/dist_kernel.h:108-126 (rotate)
 *       smore/common/torchext/dist_kernel.h:129-155 (l1)
 *       smore/common/torchext/dist_kernel.h:158-184 (l2)
 *       smore/common/torchext/dist_kernel.h:187-204 (complex)
 *       smore/common/torchext/dist_kernel.h:324-349 (distmult)
 *     with the epsilon handling of smore/common/torchext/cuda_math_ext.h:21,100-118
 *   - the broadcast index arithmetic and the reduction order of the three
 *     kernels in smore/common/torchext/common_kernel.h:33-56 (forward),
 *     :59-89 (entity gradient) and :92-123 (query gradient): 32 lane-strided
 *     partial sums that are then folded by an xor butterfly (:25-31)
 *   - the per-step gradient merge and row-wise optimizers of
 *     smore/common/embedding/embed_optimizer.py:39-48,155-163 (sorted unique +
 *     scatter-sum), :166-185 (SGD), :188-252 (Adam), :312-349 (Adagrad)
 *
 * Parity pin: checked in tests against (a) golden vectors produced by the
 * reference's own pure-torch twins (the naive_* functions beside each op),
 * stored under tests/golden/, and (b) the reference's functor source compiled
 * as host C++ (oracle/_ref) when the reference tree is mounted.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum {
  DIST_BOX_OUT = 0,
  DIST_BOX_IN = 1,
  DIST_ROTATE = 2,
  DIST_L1 = 3,
  DIST_L2 = 4,
  DIST_COMPLEX = 5,
  DIST_DISTMULT = 6,
  DIST_COUNT = 7
};

#define LANES 32

static int dist_mul(int id) { return (id == DIST_ROTATE || id == DIST_COMPLEX) ? 2 : 1; }
static int dist_has_second(int id) {
  return id == DIST_BOX_OUT || id == DIST_BOX_IN || id == DIST_ROTATE || id == DIST_COMPLEX;
}

/* sqrt / rsqrt with the reference's epsilon: the float argument is widened,
 * 1e-20 is added in double, and the sum is narrowed back before the float
 * root (cuda_math_ext.h:21,100-118). */
static float eps_sqrtf(float s) { return sqrtf((float)((double)s + 1e-20)); }
static float eps_rsqrtf(float s) { return 1.0f / sqrtf((float)((double)s + 1e-20)); }

/* one forward term; e1 / q1 are ignored by the single-part distances */
static float fwd_term(int id, float e0, float e1, float q0, float q1) {
  switch (id) {
    case DIST_BOX_OUT: {
      float t = fabsf(e0 - q0) - q1;
      return t > 0 ? t : 0.0f;
    }
    case DIST_BOX_IN:
      return fabsf(fminf(fabsf(e0 - q0), q1));
    case DIST_ROTATE: {
      float a = e0 - q0, b = e1 - q1;
      return eps_sqrtf(a * a + b * b);
    }
    case DIST_L1:
      return fabsf(e0 - q0);
    case DIST_L2: {
      float a = e0 - q0;
      return a * a;
    }
    case DIST_COMPLEX:
      return e0 * q0 + e1 * q1;
    case DIST_DISTMULT:
      return e0 * q0;
  }
  return 0.0f;
}

/* derivative rule for one element: adds g-weighted contributions into the four
 * accumulators (entity part 0/1, query part 0/1). Tie conventions follow the
 * reference: sign(0) is -1; box "out" passes gradient at exactly 0. */
static void bwd_term(int id, float g, float e0, float e1, float q0, float q1, float *ge0, float *ge1,
                     float *gq0, float *gq1) {
  switch (id) {
    case DIST_BOX_OUT: {
      float before = fabsf(e0 - q0) - q1;
      if (before >= 0) {
        *gq1 -= g;
        float s = (e0 - q0 > 0) ? 1.0f : -1.0f;
        *ge0 += s * g;
        *gq0 += -s * g;
      }
      break;
    }
    case DIST_BOX_IN: {
      float a = fabsf(e0 - q0);
      float outer = (fminf(a, q1) > 0) ? 1.0f : -1.0f;
      if (a < q1) {
        float s = (e0 - q0 > 0) ? 1.0f : -1.0f;
        *ge0 += outer * s * g;
        *gq0 += -outer * s * g;
      } else {
        *gq1 += outer * g;
      }
      break;
    }
    case DIST_ROTATE: {
      float a = e0 - q0, b = e1 - q1;
      float den = eps_rsqrtf(a * a + b * b);
      *ge0 += a * den * g;
      *ge1 += b * den * g;
      *gq0 += -a * den * g;
      *gq1 += -b * den * g;
      break;
    }
    case DIST_L1: {
      float s = (e0 - q0 > 0) ? 1.0f : -1.0f;
      *ge0 += s * g;
      *gq0 += -s * g;
      break;
    }
    case DIST_L2: {
      float d = g * (e0 - q0) * 2.0f;
      *ge0 += d;
      *gq0 += -d;
      break;
    }
    case DIST_COMPLEX:
      *ge0 += q0 * g;
      *ge1 += q1 * g;
      *gq0 += e0 * g;
      *gq1 += e1 * g;
      break;
    case DIST_DISTMULT:
      *ge0 += q0 * g;
      *gq0 += e0 * g;
      break;
  }
}

/* fold 32 lane partials the way an xor butterfly does (mask 16,8,4,2,1):
 * every lane ends with the same value, so lane 0 is enough. */
static float butterfly(float *v) {
  for (int mask = LANES / 2; mask > 0; mask /= 2) {
    float t[LANES];
    for (int l = 0; l < LANES; ++l) t[l] = v[l] + v[l ^ mask];
    memcpy(v, t, sizeof(t));
  }
  return v[0];
}

int oracle_dist_mul(int dist_id) { return dist_mul(dist_id); }
int oracle_dist_has_second(int dist_id) { return dist_has_second(dist_id); }

/* dst[i,j] = sum_d term(ent[i%be, j%ne], query[i%bc, j%nc])   (common_kernel.h:39-55) */
int oracle_dist_forward(int id, const float *ent, const float *first, const float *second,
                        float *dst, size_t bsize, size_t num, size_t be, size_t ne, size_t bc,
                        size_t nc, size_t dim) {
  if (id < 0 || id >= DIST_COUNT) return -1;
  const size_t mul = (size_t)dist_mul(id);
  const int two = dist_has_second(id);
  if (!two) second = first;
#pragma omp parallel for schedule(static)
  for (ptrdiff_t cell = 0; cell < (ptrdiff_t)(bsize * num); ++cell) {
    size_t i = (size_t)cell / num, j = (size_t)cell % num;
    const float *pe = ent + ((i % be) * ne + (j % ne)) * dim * mul;
    const float *p0 = first + ((i % bc) * nc + (j % nc)) * dim;
    const float *p1 = second + ((i % bc) * nc + (j % nc)) * dim;
    float lanes[LANES];
    for (int l = 0; l < LANES; ++l) {
      float s = 0.0f;
      for (size_t d = (size_t)l; d < dim; d += LANES)
        s += fwd_term(id, pe[d], mul == 2 ? pe[d + dim] : 0.0f, p0[d], p1[d]);
      lanes[l] = s;
    }
    dst[cell] = butterfly(lanes);
  }
  return 0;
}

/* Same sums accumulated in double, for judging how far either fp32 order may
 * drift: not a restatement of the reference, an error yardstick. */
int oracle_dist_forward_f64acc(int id, const float *ent, const float *first, const float *second,
                               double *dst, size_t bsize, size_t num, size_t be, size_t ne,
                               size_t bc, size_t nc, size_t dim) {
  if (id < 0 || id >= DIST_COUNT) return -1;
  const size_t mul = (size_t)dist_mul(id);
  if (!dist_has_second(id)) second = first;
#pragma omp parallel for schedule(static)
  for (ptrdiff_t cell = 0; cell < (ptrdiff_t)(bsize * num); ++cell) {
    size_t i = (size_t)cell / num, j = (size_t)cell % num;
    const float *pe = ent + ((i % be) * ne + (j % ne)) * dim * mul;
    const float *p0 = first + ((i % bc) * nc + (j % nc)) * dim;
    const float *p1 = second + ((i % bc) * nc + (j % nc)) * dim;
    double s = 0.0;
    for (size_t d = 0; d < dim; ++d)
      s += (double)fwd_term(id, pe[d], mul == 2 ? pe[d + dim] : 0.0f, p0[d], p1[d]);
    dst[cell] = s;
  }
  return 0;
}

/* Entity and query gradients (common_kernel.h:62-88 and :95-122).  Every
 * element of g_ent, g_first (and g_second for two-part queries) is written. */
int oracle_dist_backward(int id, const float *gout, const float *ent, const float *first,
                         const float *second, float *g_ent, float *g_first, float *g_second,
                         size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc,
                         size_t dim) {
  if (id < 0 || id >= DIST_COUNT) return -1;
  const size_t mul = (size_t)dist_mul(id);
  const int two = dist_has_second(id);
  if (!two) second = first;

  /* entity rows */
  {
    const size_t nji = bsize / be, njj = num / ne, njobs = nji * njj;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t row = 0; row < (ptrdiff_t)(be * ne); ++row) {
      size_t r0 = (size_t)row / ne, r1 = (size_t)row % ne;
      const float *pe = ent + (size_t)row * dim * mul;
      float *gpe = g_ent + (size_t)row * dim * mul;
      for (size_t d = 0; d < dim; ++d) {
        float l0[LANES], l1[LANES];
        for (int l = 0; l < LANES; ++l) {
          float a0 = 0, a1 = 0, t0 = 0, t1 = 0;
          for (size_t job = (size_t)l; job < njobs; job += LANES) {
            size_t i = (job / njj) * be + r0, j = (job % njj) * ne + r1;
            const float *p0 = first + ((i % bc) * nc + (j % nc)) * dim;
            const float *p1 = second + ((i % bc) * nc + (j % nc)) * dim;
            bwd_term(id, gout[i * num + j], pe[d], mul == 2 ? pe[d + dim] : 0.0f, p0[d], p1[d],
                     &a0, &a1, &t0, &t1);
          }
          l0[l] = a0;
          l1[l] = a1;
        }
        gpe[d] = butterfly(l0);
        if (mul == 2) gpe[d + dim] = butterfly(l1);
      }
    }
  }
  /* query rows */
  {
    const size_t nji = bsize / bc, njj = num / nc, njobs = nji * njj;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t row = 0; row < (ptrdiff_t)(bc * nc); ++row) {
      size_t r0 = (size_t)row / nc, r1 = (size_t)row % nc;
      const float *p0 = first + (size_t)row * dim;
      const float *p1 = second + (size_t)row * dim;
      for (size_t d = 0; d < dim; ++d) {
        float l0[LANES], l1[LANES];
        for (int l = 0; l < LANES; ++l) {
          float t0 = 0, t1 = 0, a0 = 0, a1 = 0;
          for (size_t job = (size_t)l; job < njobs; job += LANES) {
            size_t i = (job / njj) * bc + r0, j = (job % njj) * nc + r1;
            const float *pe = ent + ((i % be) * ne + (j % ne)) * dim * mul;
            bwd_term(id, gout[i * num + j], pe[d], mul == 2 ? pe[d + dim] : 0.0f, p0[d], p1[d],
                     &t0, &t1, &a0, &a1);
          }
          l0[l] = a0;
          l1[l] = a1;
        }
        g_first[(size_t)row * dim + d] = butterfly(l0);
        if (two) g_second[(size_t)row * dim + d] = butterfly(l1);
      }
    }
  }
  return 0;
}

/* ---- gradient merge: sorted unique + inverse map (embed_optimizer.py:39-42) ---- */

typedef struct {
  int64_t key;
  int64_t pos;
} keypos_t;

static int keypos_cmp(const void *a, const void *b) {
  const keypos_t *x = (const keypos_t *)a, *y = (const keypos_t *)b;
  if (x->key != y->key) return x->key < y->key ? -1 : 1;
  return x->pos < y->pos ? -1 : (x->pos > y->pos);
}

/* uniq: ascending distinct ids (capacity n); inverse[p] = rank of idx[p];
 * counts[u] = multiplicity.  Returns the number of distinct ids, or -1. */
int64_t oracle_unique_rows(const int64_t *idx, size_t n, int64_t *uniq, int32_t *inverse,
                           int32_t *counts) {
  if (n == 0) return 0;
  keypos_t *kp = (keypos_t *)malloc(n * sizeof(keypos_t));
  if (!kp) return -1;
  for (size_t p = 0; p < n; ++p) {
    kp[p].key = idx[p];
    kp[p].pos = (int64_t)p;
  }
  qsort(kp, n, sizeof(keypos_t), keypos_cmp);
  int64_t nu = 0;
  for (size_t p = 0; p < n; ++p) {
    if (p == 0 || kp[p].key != kp[p - 1].key) {
      uniq[nu] = kp[p].key;
      if (counts) counts[nu] = 0;
      ++nu;
    }
    inverse[kp[p].pos] = (int32_t)(nu - 1);
    if (counts) counts[nu - 1] += 1;
  }
  free(kp);
  return nu;
}

/* merged[inverse[p], :] += grad[p, :] in position order (embed_optimizer.py:45-48) */
int oracle_scatter_sum_rows(const float *grad, const int32_t *inverse, size_t n, size_t width,
                            float *merged, size_t n_unique) {
  memset(merged, 0, n_unique * width * sizeof(float));
  for (size_t p = 0; p < n; ++p) {
    float *dst = merged + (size_t)inverse[p] * width;
    const float *src = grad + p * width;
    for (size_t d = 0; d < width; ++d) dst[d] += src[d];
  }
  return 0;
}

/* ---- row-wise optimizers on the touched rows (embed_optimizer.py:166-185,208-252,312-349) ---- */

enum { OPT_SGD = 0, OPT_ADAM = 1, OPT_ADAGRAD = 2 };

/* table[N,width], m[N,width], v[N,width] or v[N] when squeeze.  step >= 1 is
 * the optimizer-wide counter (one per optimizer, not per row).  Adam state is
 * stored the way the reference stores it: old + (new - old). */
int oracle_sparse_update_rows(int opt, float *table, float *m, float *v, const int64_t *uniq,
                              const float *grad, size_t n_unique, size_t width, double lr_d,
                              double beta1_d, double beta2_d, double eps_d, int64_t step,
                              int squeeze) {
  /* hyper-parameters are Python doubles in the reference; each scalar that
   * meets a float tensor is narrowed once, at that point */
  const double bc1 = 1.0 - pow(beta1_d, (double)step);
  const double bc2 = 1.0 - pow(beta2_d, (double)step);
  const float sqrt_bc2 = (float)sqrt(bc2);
  const float step_size = (float)(-lr_d / bc1);
  const float lr = (float)lr_d, eps = (float)eps_d;
  const float beta1 = (float)beta1_d, beta2 = (float)beta2_d;
  const float omb1 = (float)(1.0 - beta1_d), omb2 = (float)(1.0 - beta2_d);
#pragma omp parallel for schedule(static)
  for (ptrdiff_t u = 0; u < (ptrdiff_t)n_unique; ++u) {
    const size_t row = (size_t)uniq[u];
    const float *g = grad + (size_t)u * width;
    float *p = table + row * width;
    if (opt == OPT_SGD) {
      for (size_t d = 0; d < width; ++d) p[d] += -lr * g[d];
      continue;
    }
    float g2mean = 0.0f;
    if (squeeze) {
      float s = 0.0f;
      for (size_t d = 0; d < width; ++d) s += g[d] * g[d];
      g2mean = s / (float)width;
    }
    if (opt == OPT_ADAGRAD) {
      float *sv = squeeze ? v + row : v + row * width;
      if (squeeze) {
        float sq = sv[0] + g2mean;
        float avg = sqrtf(sq) + eps;
        for (size_t d = 0; d < width; ++d) p[d] += -lr * g[d] / avg;
        sv[0] += g2mean;
      } else {
        for (size_t d = 0; d < width; ++d) {
          float gs = g[d] * g[d];
          float avg = sqrtf(sv[d] + gs) + eps;
          p[d] += -lr * g[d] / avg;
          sv[d] += gs;
        }
      }
      continue;
    }
    /* Adam */
    float *pm = m + row * width;
    if (squeeze) {
      float v_old = v[row];
      float v_new = v_old * beta2 + g2mean * omb2;
      float denom = sqrtf(v_new) / sqrt_bc2 + eps;
      for (size_t d = 0; d < width; ++d) {
        float m_old = pm[d];
        float m_new = m_old * beta1 + g[d] * omb1;
        p[d] += step_size * m_new / denom;
        pm[d] = m_old + (m_new - m_old);
      }
      v[row] = v_old + (v_new - v_old);
    } else {
      float *pv = v + row * width;
      for (size_t d = 0; d < width; ++d) {
        float m_old = pm[d], v_old = pv[d];
        float v_new = v_old * beta2 + g[d] * g[d] * omb2;
        float m_new = m_old * beta1 + g[d] * omb1;
        float denom = sqrtf(v_new) / sqrt_bc2 + eps;
        p[d] += step_size * m_new / denom;
        pm[d] = m_old + (m_new - m_old);
        pv[d] = v_old + (v_new - v_old);
      }
    }
  }
  return 0;
}

/* out[p,:] = table[idx[p],:]  (embed_rw.py:74-77) */
int oracle_gather_rows(const float *table, const int64_t *idx, size_t n, size_t width, float *out) {
#pragma omp parallel for schedule(static)
  for (ptrdiff_t p = 0; p < (ptrdiff_t)n; ++p)
    memcpy(out + (size_t)p * width, table + (size_t)idx[p] * width, width * sizeof(float));
  return 0;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
