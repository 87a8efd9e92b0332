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
// the entity rows).  The kernels are CUTLASS 3.x sm100 templates instantiated here: TMA loads,
// tcgen05.mma with TMEM accumulators, one SM per 128 x 128 tile (cluster 1x1x1), fp32 in / fp32 out,
// in two
// precisions: TF32 (10-bit mantissa products) and "fast fp32" (each fp32 operand split into three
// bf16 terms, nine bf16 MMAs per product, fp32-level accuracy).
//
// Built only when a CUTLASS header tree is found (see build.py); without it the entry points
// report SMORE_ERR_BAD_SHAPE and callers use the SIMT tile kernels.
#include <cuda_runtime.h>

#include "common.cuh"

extern "C" int smore_dot_available(void);

#ifdef SMORE_HAVE_CUTLASS
#include <dlfcn.h>

#include <mutex>
#include <string>

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"


namespace smore_gemm {
using namespace cute;

enum { kOk = 0, kBadShape = 1, kWorkspace = 2, kCuda = 3 };

// One SM per 128 x 128 tile, cluster 1 x 1 x 1.
template <class LayoutA, class LayoutB, bool kFast>
struct DotGemm {
  using Acc = float;
  using LayoutC = cutlass::layout::RowMajor;
  using Tile = Shape<_128, _128, _32>;
  using Cluster = Shape<_1, _1, _1>;
  using Schedule = cute::conditional_t<kFast, cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100,
                                       cutlass::gemm::KernelTmaWarpSpecialized1SmSm100>;
  using Epi = typename cutlass::epilogue::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, Tile, Cluster,
      cutlass::epilogue::collective::EpilogueTileAuto, Acc, Acc, float, LayoutC, 4, float, LayoutC, 4,
      cutlass::epilogue::TmaWarpSpecialized1Sm>::CollectiveOp;
  using Main = typename cutlass::gemm::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, float, LayoutA, 4, float, LayoutB, 4, Acc, Tile, Cluster,
      cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epi::SharedStorage))>,
      Schedule>::CollectiveOp;
  using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Main, Epi, void>;
  using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
};

// D[M, N] = A . B with A(m, k), B(k, n) in the given layouts ("column-major B" = an [N, K] row-major
// array).  need != nullptr: only report the workspace size.  Returns one of the codes above;
// *ws_needed receives the workspace size when that is what is missing.
template <class LayoutA, class LayoutB, bool kFast>
static int run_gemm(const float* A, const float* B, float* D, int M, int N, int K, void* ws, size_t ws_bytes,
                    cudaStream_t st, size_t* need) {
  using Gemm = typename DotGemm<LayoutA, LayoutB, kFast>::Gemm;
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
    return kOk;
  }
  Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess) return kBadShape;
  if (Gemm::get_workspace_size(args) > ws_bytes) return kWorkspace;
  if (gemm.initialize(args, ws, st) != cutlass::Status::kSuccess) return kCuda;
  if (gemm.run(st) != cutlass::Status::kSuccess) return kCuda;
  return kOk;
}

using RowM = cutlass::layout::RowMajor;
using ColM = cutlass::layout::ColumnMajor;

}  // namespace smore_gemm

namespace smore {
using namespace smore_gemm;

// The companion library (libsmore_b200_2sm.so, built from gemm_sm100_2sm.cu) holds the same products
// on tiles shared by two SMs.  It is optional: when the file sits next to this library it is loaded
// on first use and takes the products with at least 256 output rows; without it everything runs on
// the one-SM tiles.
typedef int (*TwoSmRun)(int layout, int fast, const float* A, const float* B, float* D, int M, int N, int K, void* ws,
                        size_t ws_bytes, void* stream, size_t* need);
static TwoSmRun g_two_sm = nullptr;
static std::once_flag g_two_sm_once;

static TwoSmRun two_sm() {
  std::call_once(g_two_sm_once, [] {
    Dl_info info;
    if (!dladdr(reinterpret_cast<void*>(&smore_dot_available), &info) || !info.dli_fname) return;
    std::string path(info.dli_fname);
    const size_t slash = path.rfind('/');
    path = (slash == std::string::npos ? std::string(".") : path.substr(0, slash)) + "/libsmore_b200_2sm.so";
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h) g_two_sm = reinterpret_cast<TwoSmRun>(dlsym(h, "smore_dot2sm_run"));
  });
  return g_two_sm;
}

static int gemm_status(int code, int M, int N, int K) {
  switch (code) {
    case kOk: return SMORE_OK;
    case kBadShape:
      return fail(SMORE_ERR_BAD_SHAPE, "tensor-core GEMM cannot take M=%d N=%d K=%d (sizes must be multiples of 4)", M, N, K);
    case kWorkspace: return fail(SMORE_ERR_WORKSPACE, "tensor-core GEMM: workspace too small (smore_dot_workspace_bytes)");
    default: return fail(SMORE_ERR_CUDA, "tensor-core GEMM: initialize or launch failed");
  }
}

enum { kLayoutRowCol = 0, kLayoutRowRow = 1, kLayoutColRow = 2 };

template <class LayoutA, class LayoutB, int kLayout>
static int run_precision(int precision, const float* A, const float* B, float* D, int M, int N, int K, void* ws,
                         size_t ws_bytes, cudaStream_t st, size_t* need) {
  if (precision != SMORE_DOT_TF32 && precision != SMORE_DOT_FP32)
    return fail(SMORE_ERR_BAD_DIST, "unknown dot precision %d", precision);
  const bool fast = precision == SMORE_DOT_FP32;
  int code;
  TwoSmRun wide = M >= 256 ? two_sm() : nullptr;
  if (wide != nullptr) {
    code = wide(kLayout, fast ? 1 : 0, A, B, D, M, N, K, ws, ws_bytes, st, need);
  } else {
    code = fast ? run_gemm<LayoutA, LayoutB, true>(A, B, D, M, N, K, ws, ws_bytes, st, need)
                : run_gemm<LayoutA, LayoutB, false>(A, B, D, M, N, K, ws, ws_bytes, st, need);
  }
  if (code == kOk && !need) count_launches(1);
  return gemm_status(code, M, N, K);
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

int smore_dot_two_sm(void) {
#ifdef SMORE_HAVE_CUTLASS
  return two_sm() != nullptr ? 1 : 0;
#else
  return 0;
#endif
}

size_t smore_dot_workspace_bytes(size_t B, size_t K, size_t W, int precision) {
#ifdef SMORE_HAVE_CUTLASS
  size_t n0 = 0, n1 = 0, n2 = 0;
  if (check_sizes(B, K, W)) return 0;
  run_precision<RowM, ColM, kLayoutRowCol>(precision, nullptr, nullptr, nullptr, (int)B, (int)K, (int)W, nullptr, 0, nullptr, &n0);
  run_precision<RowM, RowM, kLayoutRowRow>(precision, nullptr, nullptr, nullptr, (int)B, (int)W, (int)K, nullptr, 0, nullptr, &n1);
  run_precision<ColM, RowM, kLayoutColRow>(precision, nullptr, nullptr, nullptr, (int)K, (int)W, (int)B, nullptr, 0, nullptr, &n2);
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
  return run_precision<RowM, ColM, kLayoutRowCol>(precision, query, cand, dst, (int)B, (int)K, (int)W, workspace, workspace_bytes,
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
  if (int rc = run_precision<RowM, RowM, kLayoutRowRow>(precision, gout, cand, g_query, (int)B, (int)W, (int)K, workspace,
                                         workspace_bytes, st, nullptr))
    return rc;
  // g_cand[K, W] = gout^T[K, B] . query[B, W]
  return run_precision<ColM, RowM, kLayoutColRow>(precision, gout, query, g_cand, (int)K, (int)W, (int)B, workspace, workspace_bytes,
                                   st, nullptr);
#else
  (void)precision; (void)workspace; (void)workspace_bytes; (void)stream;
  return fail(SMORE_ERR_BAD_SHAPE, "library built without the tensor-core GEMM path");
#endif
}

}  // extern "C"
