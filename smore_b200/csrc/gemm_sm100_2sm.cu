// The dot-product GEMMs of gemm_sm100.cu on tiles shared by two SMs (tcgen05 cta_group::2): 256 x 128,
// or 256 x 256 for the score matrix in TF32, with the stream-K scheduler where the tile count is a
// small non-multiple of the SM-pair count (the query gradient: 128 tiles on 74 pairs).  Built as a
// library of its own, libsmore_b200_2sm.so, which libsmore_b200.so loads when the file sits next to
// it; single-GPU deployments ship it, and without it the one-SM tiles of the main library run.
// All operands are this GPU's own memory.
#include <cuda_runtime.h>

#include <algorithm>

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

// D[M, N] = A . B with A(m, k), B(k, n) in the given layouts ("column-major B" = an [N, K] row-major
// array).  need != nullptr: only report the workspace size.  Returns one of the codes above;
// *ws_needed receives the workspace size when that is what is missing.
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

namespace {
using namespace smore_gemm;

struct TwoSm {
  using Tile = Shape<_256, _128, _32>;
  using Cluster = Shape<_2, _1, _1>;
  using Tf32 = cutlass::gemm::KernelTmaWarpSpecialized2SmSm100;
  using Fp32x9 = cutlass::gemm::KernelTmaWarpSpecialized2SmFastFP32Sm100;
  using Epilogue = cutlass::epilogue::TmaWarpSpecialized2Sm;
};
struct TwoSmWide : TwoSm {      // half the operand traffic per flop, for outputs with many columns
  using Tile = Shape<_256, _256, _32>;
};

int sm_pairs() {
  static int pairs = 0;
  if (pairs == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2)
      sms = 148;
    pairs = sms / 2;
  }
  return pairs;
}

template <class LayoutA, class LayoutB>
int run(int fast, const float* A, const float* B, float* D, int M, int N, int K, void* ws, size_t ws_bytes,
        cudaStream_t st, size_t* need) {
  const size_t tiles = ((size_t)(M + 255) / 256) * ((size_t)(N + 127) / 128);
  const double waves = (double)tiles / (double)sm_pairs();
  const bool stream_k = waves < 4.0 && (waves - (double)(size_t)waves) > 0.05 && K >= 1024;
  using StreamK = cutlass::gemm::StreamKScheduler;
  if (N >= 2048 && !fast) return run_gemm<LayoutA, LayoutB, TwoSmWide, false, void>(A, B, D, M, N, K, ws, ws_bytes, st, need);
  if (stream_k) {
    return fast ? run_gemm<LayoutA, LayoutB, TwoSm, true, StreamK>(A, B, D, M, N, K, ws, ws_bytes, st, need)
                : run_gemm<LayoutA, LayoutB, TwoSm, false, StreamK>(A, B, D, M, N, K, ws, ws_bytes, st, need);
  }
  return fast ? run_gemm<LayoutA, LayoutB, TwoSm, true, void>(A, B, D, M, N, K, ws, ws_bytes, st, need)
              : run_gemm<LayoutA, LayoutB, TwoSm, false, void>(A, B, D, M, N, K, ws, ws_bytes, st, need);
}

}  // namespace

// layout: 0 = A row-major, B column-major ([N, K] array); 1 = both row-major; 2 = A column-major, B row-major.
// Returns the smore_gemm status codes (0 = done / size reported).
extern "C" __attribute__((visibility("default"))) int smore_dot2sm_run(int layout, int fast, const float* A,
                                                                        const float* B, float* D, int M, int N, int K,
                                                                        void* ws, size_t ws_bytes, void* stream,
                                                                        size_t* need) {
  cudaStream_t st = (cudaStream_t)stream;
  switch (layout) {
    case 0: return run<RowM, ColM>(fast, A, B, D, M, N, K, ws, ws_bytes, st, need);
    case 1: return run<RowM, RowM>(fast, A, B, D, M, N, K, ws, ws_bytes, st, need);
    case 2: return run<ColM, RowM>(fast, A, B, D, M, N, K, ws, ws_bytes, st, need);
    default: return kBadShape;
  }
}
