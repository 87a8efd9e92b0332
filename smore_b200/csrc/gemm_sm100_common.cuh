// CUTLASS 3.x sm100 GEMM instantiation shared by the dot-product kernels: D[M, N] = A . B in fp32
// with TF32 or bf16 x 9 ("fast fp32") tensor-core products, parameterised by a tile variant.
#pragma once
#include <cuda_runtime.h>

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
