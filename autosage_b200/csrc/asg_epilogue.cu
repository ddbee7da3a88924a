// Row-bias epilogue of the layer's Linear: out[r, :] += bias[:], in place.
//
// AutoSAGEConv ends with nn.Linear (autosage/conv.py:55).  On B200 cuBLAS's SGEMM with the bias folded
// in (addmm) runs at half the speed of the plain product at the layer's shapes, and torch's broadcast
// add after a plain product moves the 2.5 GB output at well under half of HBM speed; this kernel does
// the add at copy speed (128-bit loads and stores, grid-stride, streaming stores).
#include "asg_common.cuh"

namespace asg {

__global__ void __launch_bounds__(256) add_row_bias_kernel(float* __restrict__ out, const float* __restrict__ bias,
                                                           long long rows, int cols4) {
  const long long total = rows * cols4;  // float4 elements
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float4* out4 = reinterpret_cast<float4*>(out);
  const float4* bias4 = reinterpret_cast<const float4*>(bias);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const float4 b = __ldg(bias4 + (i % cols4));
    float4 v = out4[i];
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    st_stream4(reinterpret_cast<float*>(out4 + i), v);
  }
}

__global__ void __launch_bounds__(256) add_row_bias_scalar_kernel(float* __restrict__ out,
                                                                  const float* __restrict__ bias, long long rows,
                                                                  int cols) {
  const long long total = rows * cols;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    out[i] += __ldg(bias + (i % cols));
}

}  // namespace asg

extern "C" int asg_add_row_bias(float* out, const float* bias, int64_t rows, int64_t cols, void* stream_ptr) {
  using namespace asg;
  ASG_REQUIRE(rows >= 0 && cols >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(cols <= 2147483647ll, ASG_ERANGE, "cols exceeds the kernel index range");
  if (rows == 0 || cols == 0) return ASG_OK;
  ASG_REQUIRE(out != nullptr && bias != nullptr, ASG_EINVAL, "out and bias must not be null");
  DeviceGuard guard(out);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const int grid = sm_count(guard.target) * 8;
  const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(bias) & 15) == 0;
  if (vec) {
    add_row_bias_kernel<<<grid, 256, 0, stream>>>(out, bias, rows, static_cast<int>(cols / 4));
  } else {
    add_row_bias_scalar_kernel<<<grid, 256, 0, stream>>>(out, bias, rows, static_cast<int>(cols));
  }
  ASG_CUDA(cudaGetLastError());
  return ASG_OK;
}

// Pitched device-to-device copy (cudaMemcpy2DAsync: copy engines, no kernel).  The sharded path uses it
// to pull a band of feature columns of another GPU's rows out of its peer-mapped X.
extern "C" int asg_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                           size_t height, void* stream_ptr) {
  using namespace asg;
  if (width_bytes == 0 || height == 0) return ASG_OK;
  ASG_REQUIRE(dst != nullptr && src != nullptr, ASG_EINVAL, "dst and src must not be null");
  ASG_REQUIRE(dst_pitch >= width_bytes && src_pitch >= width_bytes, ASG_EINVAL, "pitch smaller than the row width");
  DeviceGuard guard(dst);
  ASG_CUDA(guard.status);
  ASG_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, height, cudaMemcpyDefault,
                             static_cast<cudaStream_t>(stream_ptr)));
  return ASG_OK;
}
