// Dot-product scoring against a shared candidate set on the 5th-generation tensor cores.
//
// DistMult / ComplEx score a query against a candidate with an inner product
// (smore/common/torchext/dist_kernel.h:187-204 and :324-349); with one candidate set shared by all
// B queries (`--share_negative`, smore/models/complex.py:186 uses torch.mm for exactly this) the
// op is a dense GEMM and so are both of its gradients:
//     score[B, K]   = query[B, W] . cand[K, W]^T
//     g_query[B, W] = g[B, K]     . cand[K, W]
//     g_cand[K, W]  = g[B, K]^T   . query[B, W]
// W is the row length (dim for DistMult; 2*dim for ComplEx, with the query laid out [re | im] like
// the entity rows).  The kernels are CUTLASS 3.x sm100 templates instantiated here: TMA loads
// (never multicast), tcgen05.mma with TMEM accumulators, two SMs per 256 x 128 tile, fp32 in / fp32
// out, in two
// precisions: TF32 (10-bit mantissa products) and "fast fp32" (each fp32 operand split into three
// bf16 terms, nine bf16 MMAs per product, fp32-level accuracy).
//
// Built only when a CUTLASS header tree is found (see build.py); without it the entry points
// report SMORE_ERR_BAD_SHAPE and callers use the SIMT tile kernels.
#include <cuda_runtime.h>

#include <algorithm>

#include "common.cuh"

#ifdef SMORE_HAVE_CUTLASS
#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

namespace smore {
using namespace cute;

// Tile variants.  TwoSm pairs two SMs on one 256 x 128 tile (tcgen05 cta_group::2, cluster 2 x 1): each
// CTA of the pair loads its own halves of the operand tiles, so with this static cluster shape the
// builder picks the plain two-SM TMA loads - no operand is multicast.
struct OneSm {
  using Tile = Shape<_128, _128, _32>;
  using Cluster = Shape<_1, _1, _1>;
  using Tf32 = cutlass::gemm::KernelTmaWarpSpecialized1SmSm100;
  using Fp32x9 = cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100;
  using Epilogue = cutlass::epilogue::TmaWarpSpecialized1Sm;
};
struct TwoSm {
  using Tile = Shape<_256, _128, _32>;
  using Cluster = Shape<_2, _1, _1>;
  using Tf32 = cutlass::gemm::KernelTmaWarpSpecialized2SmSm100;
  using Fp32x9 = cutlass::gemm::KernelTmaWarpSpecialized2SmFastFP32Sm100;
  using Epilogue = cutlass::epilogue::TmaWarpSpecialized2Sm;
};

struct TwoSmWide : TwoSm {      // 256 x 256 tiles: half the operand traffic per flop, for outputs with many columns
  using Tile = Shape<_256, _256, _32>;
};

template <class LayoutA, class LayoutB, class Variant, bool kFast, class Scheduler>
struct DotGemm {
  using Acc = float;
  using LayoutC = cutlass::layout::RowMajor;
  using Tile = typename Variant::Tile;
  using Cluster = typename Variant::Cluster;
  using Schedule = cute::conditional_t<kFast, typename Variant::Fp32x9, typename Variant::Tf32>;
  using Epi = typename cutlass::epilogue::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, Tile, Cluster,
      cutlass::epilogue::collective::EpilogueTileAuto, Acc, Acc, float, LayoutC, 4, float, LayoutC, 4,
      typename Variant::Epilogue>::CollectiveOp;
  using Main = typename cutlass::gemm::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, float, LayoutA, 4, float, LayoutB, 4, Acc, Tile, Cluster,
      cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epi::SharedStorage))>,
      Schedule>::CollectiveOp;
  using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Main, Epi, Scheduler>;
  using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
};

// D[M, N] = A . B with A(m, k), B(k, n) in the given layouts ("column-major B" = an [N, K] row-major array)
template <class LayoutA, class LayoutB, class Variant, bool kFast, class Scheduler>
static int run_gemm(const float* A, const float* B, float* D, int M, int N, int K, void* ws, size_t ws_bytes,
                    cudaStream_t st, size_t* need) {
  using Gemm = typename DotGemm<LayoutA, LayoutB, Variant, kFast, Scheduler>::Gemm;
  using StrideA = typename Gemm::GemmKernel::StrideA;
  using StrideB = typename Gemm::GemmKernel::StrideB;
  using StrideC = typename Gemm::GemmKernel::StrideC;
  using StrideD = typename Gemm::GemmKernel::StrideD;
  auto sa = cutlass::make_cute_packed_stride(StrideA{}, make_shape(M, K, 1));
  auto sb = cutlass::make_cute_packed_stride(StrideB{}, make_shape(N, K, 1));
  auto sc = cutlass::make_cute_packed_stride(StrideC{}, make_shape(M, N, 1));
  auto sd = cutlass::make_cute_packed_stride(StrideD{}, make_shape(M, N, 1));
  typename Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm, {M, N, K, 1}, {A, sa, B, sb},
                                {{1.0f, 0.0f}, D, sc, D, sd}};
  if (need) {
    *need = Gemm::get_workspace_size(args);
    return SMORE_OK;
  }
  Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess)
    return fail(SMORE_ERR_BAD_SHAPE, "tensor-core GEMM cannot take M=%d N=%d K=%d (sizes must be multiples of 4)", M, N, K);
  if (Gemm::get_workspace_size(args) > ws_bytes)
    return fail(SMORE_ERR_WORKSPACE, "tensor-core GEMM needs %zu bytes of workspace", Gemm::get_workspace_size(args));
  if (gemm.initialize(args, ws, st) != cutlass::Status::kSuccess) return fail(SMORE_ERR_CUDA, "GEMM initialize failed");
  if (gemm.run(st) != cutlass::Status::kSuccess) return fail(SMORE_ERR_CUDA, "GEMM launch failed");
  count_launches(1);
  return SMORE_OK;
}

using RowM = cutlass::layout::RowMajor;
using ColM = cutlass::layout::ColumnMajor;

// Output tiles are handed to the SMs by the persistent scheduler; products whose tile count is a
// small non-multiple of the SM count (the query gradient: 128 two-SM tiles on 74 SM pairs) use the
// stream-K scheduler, which splits the contraction of the last partial wave over the idle SMs.
template <class LayoutA, class LayoutB>
static int run_precision(int precision, const float* A, const float* B, float* D, int M, int N, int K, void* ws,
                         size_t ws_bytes, cudaStream_t st, size_t* need) {
  if (precision != SMORE_DOT_TF32 && precision != SMORE_DOT_FP32)
    return fail(SMORE_ERR_BAD_DIST, "unknown dot precision %d", precision);
  const bool fast = precision == SMORE_DOT_FP32;
  const size_t tiles = ((size_t)(M + 255) / 256) * ((size_t)(N + 127) / 128);
  const size_t pairs = std::max(1, sm_count() / 2);
  const double waves = (double)tiles / (double)pairs;
  const bool stream_k = M >= 256 && waves < 4.0 && (waves - (double)(size_t)waves) > 0.05 && K >= 1024;
  using StreamK = cutlass::gemm::StreamKScheduler;
  if (M < 256) {
    return fast ? run_gemm<LayoutA, LayoutB, OneSm, true, void>(A, B, D, M, N, K, ws, ws_bytes, st, need)
                : run_gemm<LayoutA, LayoutB, OneSm, false, void>(A, B, D, M, N, K, ws, ws_bytes, st, need);
  }
  if (N >= 2048 && !fast) {
    return run_gemm<LayoutA, LayoutB, TwoSmWide, false, void>(A, B, D, M, N, K, ws, ws_bytes, st, need);
  }
  if (stream_k) {
    return fast ? run_gemm<LayoutA, LayoutB, TwoSm, true, StreamK>(A, B, D, M, N, K, ws, ws_bytes, st, need)
                : run_gemm<LayoutA, LayoutB, TwoSm, false, StreamK>(A, B, D, M, N, K, ws, ws_bytes, st, need);
  }
  return fast ? run_gemm<LayoutA, LayoutB, TwoSm, true, void>(A, B, D, M, N, K, ws, ws_bytes, st, need)
              : run_gemm<LayoutA, LayoutB, TwoSm, false, void>(A, B, D, M, N, K, ws, ws_bytes, st, need);
}

}  // namespace smore
#endif  // SMORE_HAVE_CUTLASS

using namespace smore;

static int check_sizes(size_t B, size_t K, size_t W) {
  if (!B || !K || !W) return fail(SMORE_ERR_BAD_SHAPE, "dot: sizes must be positive");
  if (B > (1u << 30) || K > (1u << 30) || W > (1u << 30)) return fail(SMORE_ERR_TOO_LARGE, "dot: size too large");
  return SMORE_OK;
}

extern "C" {

int smore_dot_available(void) {
#ifdef SMORE_HAVE_CUTLASS
  return 1;
#else
  return 0;
#endif
}

size_t smore_dot_workspace_bytes(size_t B, size_t K, size_t W, int precision) {
#ifdef SMORE_HAVE_CUTLASS
  size_t n0 = 0, n1 = 0, n2 = 0;
  if (check_sizes(B, K, W)) return 0;
  run_precision<RowM, ColM>(precision, nullptr, nullptr, nullptr, (int)B, (int)K, (int)W, nullptr, 0, nullptr, &n0);
  run_precision<RowM, RowM>(precision, nullptr, nullptr, nullptr, (int)B, (int)W, (int)K, nullptr, 0, nullptr, &n1);
  run_precision<ColM, RowM>(precision, nullptr, nullptr, nullptr, (int)K, (int)W, (int)B, nullptr, 0, nullptr, &n2);
  size_t n = n0 > n1 ? n0 : n1;
  n = n > n2 ? n : n2;
  return n < 256 ? 256 : n;
#else
  (void)B; (void)K; (void)W; (void)precision;
  return 0;
#endif
}

int smore_dot_forward_shared(const float* cand, const float* query, float* dst, size_t B, size_t K, size_t W,
                             int precision, void* workspace, size_t workspace_bytes, void* stream) {
  if (!cand || !query || !dst) return fail(SMORE_ERR_NULL, "dot_forward_shared: NULL pointer");
  if (int rc = check_sizes(B, K, W)) return rc;
#ifdef SMORE_HAVE_CUTLASS
  return run_precision<RowM, ColM>(precision, query, cand, dst, (int)B, (int)K, (int)W, workspace, workspace_bytes,
                                   (cudaStream_t)stream, nullptr);
#else
  (void)precision; (void)workspace; (void)workspace_bytes; (void)stream;
  return fail(SMORE_ERR_BAD_SHAPE, "library built without the tensor-core GEMM path");
#endif
}

int smore_dot_backward_shared(const float* gout, const float* cand, const float* query, float* g_cand,
                              float* g_query, size_t B, size_t K, size_t W, int precision, void* workspace,
                              size_t workspace_bytes, void* stream) {
  if (!gout || !cand || !query || !g_cand || !g_query) return fail(SMORE_ERR_NULL, "dot_backward_shared: NULL pointer");
  if (int rc = check_sizes(B, K, W)) return rc;
#ifdef SMORE_HAVE_CUTLASS
  cudaStream_t st = (cudaStream_t)stream;
  // g_query[B, W] = gout[B, K] . cand[K, W]
  if (int rc = run_precision<RowM, RowM>(precision, gout, cand, g_query, (int)B, (int)W, (int)K, workspace,
                                         workspace_bytes, st, nullptr))
    return rc;
  // g_cand[K, W] = gout^T[K, B] . query[B, W]
  return run_precision<ColM, RowM>(precision, gout, query, g_cand, (int)K, (int)W, (int)B, workspace, workspace_bytes,
                                   st, nullptr);
#else
  (void)precision; (void)workspace; (void)workspace_bytes; (void)stream;
  return fail(SMORE_ERR_BAD_SHAPE, "library built without the tensor-core GEMM path");
#endif
}

}  // extern "C"
