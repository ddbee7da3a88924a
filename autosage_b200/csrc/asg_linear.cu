// The layer's Linear on the tensor cores at float32 accuracy: out = x @ weight^T + bias.
//
// AutoSAGEConv ends with nn.Linear (autosage/conv.py:55), a float32 GEMM that cuBLAS runs on the CUDA
// cores when TF32 is off (the reference's setting): 157 GFLOP at the layer's largest shape
// (2,449,029 x 128 -> 256), compute-bound at a third of the whole forward.  This file instantiates
// CUTLASS's sm_100 "emulated float32" collective instead: every float32 operand is split on the fly into
// three bfloat16 pieces, the piece products that matter at float32 precision (six of the nine) run as
// tcgen05 bf16 MMAs (operands staged by TMA, accumulators in tensor memory) and are summed in float32,
// which reproduces the float32 product to within a few ulp (measured: closer to the float64 result than
// cuBLAS SGEMM).  The bias is added in
// the epilogue, so the output is written once.  Cluster shape 1x1x1: every TMA load is a plain,
// single-CTA load of this GPU's own memory.
//
// This is library code in the sense that a cuBLAS call is: the kernel is CUTLASS's, only the
// instantiation (tile 128x128x16, one SM per tile, per-column bias fusion) and the C entry are ours.
#include "asg_common.cuh"

#ifdef ASG_NO_CUTLASS
// Built without a CUTLASS header tree: the entry point exists (the ABI stays complete) and says so.
extern "C" int asg_linear_available(void) { return 0; }
extern "C" int asg_linear_bias(const float*, const float*, const float*, float*, int64_t, int64_t, int64_t, void*) {
  return asg::fail(ASG_EINVAL, "%s", "asg_linear_bias was built without CUTLASS; use asg_linear_bias_umma or a cuBLAS product");
}
#else
extern "C" int asg_linear_available(void) { return 1; }

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/fusion/operations.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/kernel_hardware_info.h"

namespace asg {
namespace linear {

using namespace cute;

using Element = float;
using LayoutX = cutlass::layout::RowMajor;       // x: rows x in_features
using LayoutW = cutlass::layout::ColumnMajor;    // weight (out x in, row-major) read as in x out, column-major
using LayoutOut = cutlass::layout::RowMajor;
constexpr int kAlign = 4;                        // 16 bytes, the TMA granule
using Arch = cutlass::arch::Sm100;
using OpClass = cutlass::arch::OpClassTensorOp;
using Tile = Shape<_128, _128, _16>;
using Cluster = Shape<_1, _1, _1>;
using Fusion = cutlass::epilogue::fusion::LinCombPerColBias<Element, Element, Element>;

using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    Arch, OpClass, Tile, Cluster, cutlass::epilogue::collective::EpilogueTileAuto, Element, Element, void, LayoutOut,
    kAlign, Element, LayoutOut, kAlign, cutlass::epilogue::TmaWarpSpecialized1Sm, Fusion>::CollectiveOp;

using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    Arch, OpClass, Element, LayoutX, kAlign, Element, LayoutW, kAlign, Element, Tile, Cluster,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
    cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100>::CollectiveOp;

// The builder always asks for all five "bands" of the nine piece products.  Bands 4 and 5 (a1*b2, a2*b1,
// a2*b2 with a0/b0 the leading pieces) are below 2^-24 of the product, i.e. below float32 rounding: the
// measured error against float64 is the same with three bands (six MMAs), so the collective is
// re-instantiated with the builder's own types and NumBandsToCompute = 3.
using Built = typename Mainloop::DispatchPolicy;
using ThreeBands = cutlass::gemm::MainloopSm100TmaUmmaWarpSpecializedFastF32<
    Built::Load2TransformPipelineStageCount, Built::Transform2MmaPipelineStageCount,
    Built::Schedule::SchedulerPipelineStageCount, Built::Schedule::AccumulatorPipelineStageCount, 3,
    Built::ScalingFactor, Built::AccPromotionInterval, typename Built::ClusterShape,
    typename Built::AccumulatorCopyAtom, typename Built::ArchTag>;
using MainloopThreeBands = cutlass::gemm::collective::CollectiveMma<
    ThreeBands, typename Mainloop::TileShape, float, typename Mainloop::StrideA, float, typename Mainloop::StrideB,
    typename Mainloop::TiledMma, typename Mainloop::GmemTiledCopyA, typename Mainloop::SmemLayoutAtomsA,
    typename Mainloop::CopyAtomsA, typename Mainloop::TransformA, typename Mainloop::GmemTiledCopyB,
    typename Mainloop::SmemLayoutAtomsB, typename Mainloop::CopyAtomsB, typename Mainloop::TransformB>;

using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, MainloopThreeBands, Epilogue, void>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;

}  // namespace linear
}  // namespace asg

extern "C" int asg_linear_bias(const float* x, const float* weight, const float* bias, float* out, int64_t rows,
                               int64_t in_features, int64_t out_features, void* stream_ptr) {
  using namespace asg;
  using namespace asg::linear;
  ASG_REQUIRE(rows >= 0 && in_features > 0 && out_features > 0, ASG_EINVAL,
              "rows must be non-negative, in_features and out_features positive");
  ASG_REQUIRE(rows <= 2147483647ll && in_features <= 2147483647ll && out_features <= 2147483647ll, ASG_ERANGE,
              "a dimension exceeds the kernel index range");
  if (rows == 0) return ASG_OK;
  ASG_REQUIRE(x != nullptr && weight != nullptr && out != nullptr, ASG_EINVAL, "x, weight and out must not be null");
  ASG_REQUIRE(in_features % 4 == 0 && out_features % 4 == 0, ASG_EINVAL,
              "in_features and out_features must be multiples of 4 (16-byte rows for the bulk tensor copies)");
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
                         reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias);
  ASG_REQUIRE((bits & 15) == 0, ASG_EINVAL, "x, weight, bias and out must be 16-byte aligned");
  DeviceGuard guard(out);
  ASG_CUDA(guard.status);

  using StrideX = typename Gemm::GemmKernel::StrideA;
  using StrideW = typename Gemm::GemmKernel::StrideB;
  using StrideOut = typename Gemm::GemmKernel::StrideD;
  const int m = static_cast<int>(rows), n = static_cast<int>(out_features), k = static_cast<int>(in_features);
  StrideX stride_x{};
  StrideW stride_w{};
  StrideOut stride_out{};
  get<0>(stride_x) = in_features;    // x[r, c] at r * in_features + c
  get<0>(stride_w) = in_features;    // weight[o, c] at o * in_features + c
  get<0>(stride_out) = out_features;
  typename Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                                {m, n, k, 1},
                                {x, stride_x, weight, stride_w},
                                {{}, nullptr, stride_out, out, stride_out}};
  args.epilogue.thread.alpha = 1.0f;
  args.epilogue.thread.beta = 0.0f;
  args.epilogue.thread.bias_ptr = bias;  // null: no bias
  args.hw_info.device_id = guard.target;
  args.hw_info.sm_count = sm_count(guard.target);

  Gemm gemm;
  ASG_REQUIRE(gemm.can_implement(args) == cutlass::Status::kSuccess, ASG_EINVAL,
              "the tensor-core Linear cannot take these sizes");
  ASG_REQUIRE(Gemm::get_workspace_size(args) == 0, ASG_EWORKSPACE, "unexpected scratch requirement of the Linear kernel");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  cutlass::Status status = gemm.initialize(args, nullptr, stream);
  if (status == cutlass::Status::kSuccess) status = gemm.run(stream);
  if (status != cutlass::Status::kSuccess) {
    const cudaError_t last = cudaGetLastError();
    return fail(ASG_ECUDA, "the tensor-core Linear failed to launch: %s (%s)", cutlass::cutlassGetStatusString(status),
                cudaGetErrorString(last));
  }
  return ASG_OK;
}
#endif  // ASG_NO_CUTLASS
