// Degree binning ("plan"): a deterministic counting sort of row ids by (hub?, floor(log2 degree)).
//
// The reference splits rows on every call with degree subtraction, two nonzero() calls (each a
// host synchronisation) and int32 casts (csrc/launcher_spmm.cu:49-59).  Here three kernels write
// the processing order into the caller's workspace without touching the host:
//   plan_rank<false>  per-block bucket histogram          -> block_hist[bucket][block]
//   plan_scan         exclusive scan of block_hist (bucket-major), header fields, zeroed counters
//   plan_rank<true>   stable scatter: order[base(bucket, block) + rank in block] = row
// Hubs (degree >= threshold) occupy order[0, n_hub) and, restricted to one bucket, appear in
// ascending row id; over all buckets they are the same set as nonzero(degree >= threshold).
#include "asg_common.cuh"

namespace asg {

__device__ __forceinline__ int bucket_of(long long degree, long long threshold) {
  int lg = degree <= 0 ? 0 : 64 - __clzll(degree);  // 1 + floor(log2 degree)
  if (lg > 23) lg = 23;
  const int descending = 23 - lg;
  const bool hub = threshold > 0 && degree >= threshold;
  return hub ? descending : 24 + descending;
}

template <bool SCATTER>
__global__ void __launch_bounds__(kPlanBlock) plan_rank(const int64_t* __restrict__ crow, int n_rows,
                                                        long long threshold, int n_blocks,
                                                        int* __restrict__ block_hist,
                                                        int* __restrict__ order) {
  __shared__ int warp_hist[kPlanBlock / 32][kBuckets + 1];
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  for (int i = tid; i < (kPlanBlock / 32) * (kBuckets + 1); i += kPlanBlock) (&warp_hist[0][0])[i] = 0;
  __syncthreads();

  const long long row = static_cast<long long>(blockIdx.x) * kPlanBlock + tid;
  int bucket = kBuckets;  // dummy bucket for threads past the last row
  if (row < n_rows) bucket = bucket_of(crow[row + 1] - crow[row], threshold);

  const unsigned peers = __match_any_sync(kFull, bucket);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (rank_in_warp == 0) warp_hist[warp][bucket] = __popc(peers);
  __syncthreads();

  // Exclusive prefix over warps for each bucket; thread b owns bucket b.
  if (tid < kBuckets) {
    int running = 0;
    for (int w = 0; w < kPlanBlock / 32; ++w) {
      const int c = warp_hist[w][tid];
      warp_hist[w][tid] = running;
      running += c;
    }
    if (!SCATTER) block_hist[static_cast<size_t>(tid) * n_blocks + blockIdx.x] = running;
  }
  if (SCATTER) {
    __syncthreads();
    if (row < n_rows) {
      const int base = block_hist[static_cast<size_t>(bucket) * n_blocks + blockIdx.x];
      order[base + warp_hist[warp][bucket] + rank_in_warp] = static_cast<int>(row);
    }
  }
}

// One block scans block_hist (length = kBuckets * n_blocks) in place and fills the header.
__global__ void __launch_bounds__(1024) plan_scan(int* __restrict__ block_hist, long long length, int n_blocks,
                                                  int n_rows, long long threshold, Header* __restrict__ header) {
  __shared__ int warp_total[32];
  const int tid = threadIdx.x;
  const long long per = (length + 1023) / 1024;
  const long long begin = per * tid < length ? per * tid : length;
  const long long end = begin + per < length ? begin + per : length;
  int sum = 0;
  for (long long i = begin; i < end; ++i) sum += block_hist[i];

  // block-wide exclusive scan of `sum`
  int inclusive = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(kFull, inclusive, o);
    if ((tid & 31) >= o) inclusive += up;
  }
  if ((tid & 31) == 31) warp_total[tid >> 5] = inclusive;
  __syncthreads();
  if (tid < 32) {
    int v = warp_total[tid];
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(kFull, inc, o);
      if (tid >= o) inc += up;
    }
    warp_total[tid] = inc - v;
  }
  __syncthreads();
  int running = warp_total[tid >> 5] + inclusive - sum;
  for (long long i = begin; i < end; ++i) {
    const int c = block_hist[i];
    block_hist[i] = running;
    running += c;
  }
  __syncthreads();
  if (tid == 0) {
    // hubs are buckets [0, 24): their count is the exclusive prefix at the start of bucket 24
    const long long first_light = 24ll * n_blocks;
    int n_hub = 0;
    if (length > 0) n_hub = first_light < length ? block_hist[first_light] : n_rows;
    header->n_hub = n_hub;
    header->n_light = n_rows - n_hub;
    // light rows with degree < 32 have 1 + floor(log2 degree) <= 5, i.e. light buckets 24 + (23 - 5) = 42 .. 47
    const long long first_short = 42ll * n_blocks;
    header->n_short = length > 0 ? n_rows - block_hist[first_short] : 0;
    header->status = 0;
    header->n_rows = n_rows;
    header->hub_threshold = threshold;
    for (int i = 0; i < kCounters; ++i) header->counter[i] = 0ull;
  }
}

int plan_build(const int64_t* crow, int64_t n_rows, int64_t hub_threshold, void* workspace, cudaStream_t stream) {
  Header* header = static_cast<Header*>(workspace);
  char* base = static_cast<char*>(workspace);
  int* order = reinterpret_cast<int*>(base + order_offset());
  int* block_hist = reinterpret_cast<int*>(base + hist_offset(n_rows));
  const int n_blocks = static_cast<int>(plan_blocks(n_rows));
  const long long length = static_cast<long long>(kBuckets) * n_blocks;
  if (n_blocks > 0) {
    plan_rank<false><<<n_blocks, kPlanBlock, 0, stream>>>(crow, static_cast<int>(n_rows), hub_threshold, n_blocks,
                                                           block_hist, order);
    ASG_CUDA(cudaGetLastError());
  }
  plan_scan<<<1, 1024, 0, stream>>>(block_hist, length, n_blocks, static_cast<int>(n_rows), hub_threshold, header);
  ASG_CUDA(cudaGetLastError());
  if (n_blocks > 0) {
    plan_rank<true><<<n_blocks, kPlanBlock, 0, stream>>>(crow, static_cast<int>(n_rows), hub_threshold, n_blocks,
                                                          block_hist, order);
    ASG_CUDA(cudaGetLastError());
  }
  return ASG_OK;
}

}  // namespace asg

extern "C" {

int asg_plan_build(const int64_t* crow, int64_t n_rows, int64_t hub_threshold, void* workspace,
                   size_t workspace_bytes, void* stream) {
  ASG_REQUIRE(n_rows >= 0, ASG_EINVAL, "n_rows must be non-negative");
  ASG_REQUIRE(n_rows <= 2147483647ll - 2048, ASG_ERANGE, "n_rows exceeds the kernel index range");
  ASG_REQUIRE(crow != nullptr, ASG_EINVAL, "crow must not be null");
  if (int rc = asg::check_workspace(workspace, workspace_bytes, n_rows)) return rc;
  asg::DeviceGuard guard(workspace);
  ASG_CUDA(guard.status);
  return asg::plan_build(crow, n_rows, hub_threshold, workspace, static_cast<cudaStream_t>(stream));
}

int asg_plan_export(const void* workspace, int64_t n_rows, int32_t* order, int32_t* counts, void* stream) {
  ASG_REQUIRE(workspace != nullptr, ASG_EWORKSPACE, "workspace pointer is null");
  ASG_REQUIRE(n_rows >= 0, ASG_EINVAL, "n_rows must be non-negative");
  asg::DeviceGuard guard(workspace);
  ASG_CUDA(guard.status);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const char* base = static_cast<const char*>(workspace);
  if (order != nullptr && n_rows > 0)
    ASG_CUDA(cudaMemcpyAsync(order, base + asg::order_offset(), size_t(4) * size_t(n_rows), cudaMemcpyDeviceToDevice, s));
  if (counts != nullptr) ASG_CUDA(cudaMemcpyAsync(counts, base, 8, cudaMemcpyDeviceToDevice, s));
  return ASG_OK;
}

}  // extern "C"
