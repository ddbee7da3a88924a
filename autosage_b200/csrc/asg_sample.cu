// Row sample of a CSR matrix for the scheduler's probe: the rows listed in `rows` (ascending, no
// duplicates needed) are cut out with every one of their edges, column ids unchanged.
//
// Replaces the torch formulation of the sample (autosage/_auto.py:95-154 in the reference builds an
// induced sub-graph with about fifteen ATen kernels and a host synchronisation; the work-sized row
// sample of this package needed eight ATen kernels and one).  Here: one kernel reads the degrees, one
// device-wide scan (CUB) turns them into the sample's row pointers, one kernel copies the column and
// weight segments (a warp per sampled row, coalesced), and the two numbers the host needs to size its
// views - rows kept and edges kept - land in a two-word result the caller reads whenever it next
// synchronises.  Nothing here synchronises the host.
#include "asg_common.cuh"

#include <cub/device/device_scan.cuh>

namespace asg {
namespace sample {

constexpr int kThreads = 256;

inline cudaError_t scan_temp_bytes(int64_t k, size_t* bytes) {
  *bytes = 0;
  return cub::DeviceScan::InclusiveSum(nullptr, *bytes, static_cast<const int64_t*>(nullptr),
                                       static_cast<int64_t*>(nullptr), k);
}

// degree[i] = crow[rows[i] + 1] - crow[rows[i]]  (written to out_crow[i + 1]); out_crow[0] = 0
__global__ void __launch_bounds__(kThreads) degree_kernel(const int64_t* __restrict__ crow, const int64_t* __restrict__ rows,
                                                          long long k, int64_t* __restrict__ out_crow) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < k; i += stride) {
    const long long r = rows[i];
    out_crow[i + 1] = crow[r + 1] - crow[r];
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) out_crow[0] = 0;
}

// kept[0] = number of leading sampled rows whose edges fit `capacity`, kept[1] = their edge count
// (one thread: a binary search over the scanned row pointers).
__global__ void boundary_kernel(const int64_t* __restrict__ out_crow, long long k, long long capacity,
                                int64_t* __restrict__ kept) {
  long long lo = 0, hi = k;  // largest i with out_crow[i] <= capacity
  while (lo < hi) {
    const long long mid = (lo + hi + 1) >> 1;
    if (out_crow[mid] <= capacity) lo = mid; else hi = mid - 1;
  }
  kept[0] = lo;
  kept[1] = out_crow[lo];
}

// Row pointers past the last kept row are clamped to kept[1], so that the arrays stay a valid CSR
// whatever the caller does with the tail.
__global__ void __launch_bounds__(kThreads) clamp_tail(int64_t* __restrict__ out_crow, long long k,
                                                       const int64_t* __restrict__ kept) {
  const long long rows_kept = kept[0], edges_kept = kept[1];
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = rows_kept + 1 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i <= k; i += stride)
    out_crow[i] = edges_kept;
}

// one warp per kept row: out_col[out_crow[i] + j] = col[crow[rows[i]] + j]
__global__ void __launch_bounds__(kThreads) gather_kernel(const int64_t* __restrict__ crow, const int64_t* __restrict__ col,
                                                          const float* __restrict__ val, const int64_t* __restrict__ rows,
                                                          const int64_t* __restrict__ out_crow, const int64_t* __restrict__ kept,
                                                          int64_t* __restrict__ out_col, float* __restrict__ out_val) {
  const long long rows_kept = kept[0];
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; i < rows_kept; i += warps) {
    const long long src = crow[rows[i]];
    const long long dst = out_crow[i];
    const long long count = out_crow[i + 1] - dst;
    for (long long j = lane; j < count; j += 32) {
      out_col[dst + j] = col[src + j];
      if (out_val != nullptr) out_val[dst + j] = val[src + j];
    }
  }
}

}  // namespace sample
}  // namespace asg

extern "C" size_t asg_row_sample_workspace_bytes(int64_t n_sampled_rows) {
  using namespace asg::sample;
  if (n_sampled_rows <= 0) return 256;
  size_t temp = 0;
  if (scan_temp_bytes(n_sampled_rows, &temp) != cudaSuccess) return 0;
  return asg::align256(temp) + 256;
}

extern "C" int asg_csr_row_sample(const int64_t* crow, const int64_t* col, const float* val, const int64_t* rows,
                                  int64_t n_sampled_rows, int64_t capacity, int64_t* out_crow, int64_t* out_col,
                                  float* out_val, int64_t* kept, void* workspace, size_t workspace_bytes,
                                  void* stream_ptr) {
  using namespace asg;
  using namespace asg::sample;
  ASG_REQUIRE(n_sampled_rows >= 0 && capacity >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(out_crow != nullptr && kept != nullptr, ASG_EINVAL, "out_crow and kept must not be null");
  ASG_REQUIRE((val == nullptr) == (out_val == nullptr), ASG_EINVAL, "val and out_val must both be given or both be null");
  DeviceGuard guard(out_crow);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (n_sampled_rows == 0) {
    ASG_CUDA(cudaMemsetAsync(out_crow, 0, sizeof(int64_t), stream));
    ASG_CUDA(cudaMemsetAsync(kept, 0, 2 * sizeof(int64_t), stream));
    return ASG_OK;
  }
  ASG_REQUIRE(crow != nullptr && rows != nullptr, ASG_EINVAL, "crow and rows must not be null");
  ASG_REQUIRE(capacity == 0 || (col != nullptr && out_col != nullptr), ASG_EINVAL, "col and out_col must not be null");
  size_t temp = 0;
  ASG_CUDA(scan_temp_bytes(n_sampled_rows, &temp));
  ASG_REQUIRE(workspace != nullptr && workspace_bytes >= align256(temp) + 256, ASG_EWORKSPACE,
              "workspace smaller than asg_row_sample_workspace_bytes(n_sampled_rows)");
  const int grid = sm_count(guard.target) * 8;
  degree_kernel<<<grid, kThreads, 0, stream>>>(crow, rows, n_sampled_rows, out_crow);
  ASG_CUDA(cudaGetLastError());
  ASG_CUDA(cub::DeviceScan::InclusiveSum(workspace, temp, out_crow + 1, out_crow + 1, n_sampled_rows, stream));
  boundary_kernel<<<1, 1, 0, stream>>>(out_crow, n_sampled_rows, capacity, kept);
  ASG_CUDA(cudaGetLastError());
  clamp_tail<<<grid, kThreads, 0, stream>>>(out_crow, n_sampled_rows, kept);
  ASG_CUDA(cudaGetLastError());
  gather_kernel<<<grid, kThreads, 0, stream>>>(crow, col, val, rows, out_crow, kept, out_col, out_val);
  ASG_CUDA(cudaGetLastError());
  return ASG_OK;
}
