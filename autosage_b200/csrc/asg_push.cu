// SM-driven push of one contiguous buffer into the same-shaped buffers of up to 7 peer GPUs.
//
// Used by the sharded path as an alternative to copy-engine pulls: every rank stores its own shard of
// the dense operand straight into the other ranks' gathered buffers (peer-mapped symmetric memory).
// Each 16-byte element is read ONCE from local memory and stored to every destination with plain
// 128-bit global stores; the destinations are visited in a rotated order (starting after this rank), so
// that at any moment the ranks write to different peers.  No multicast, no bulk/TMA copy, nothing waits
// on another GPU inside the kernel: ordering against the readers is the caller's (stream order plus the
// symmetric-memory barrier that follows).  No counterpart in the reference, which is single-GPU.
#include "asg_common.cuh"

namespace asg {
namespace push {

constexpr int kMaxPeers = 7;
constexpr int kThreads = 256;
constexpr int kUnroll = 4;

struct Args {
  const uint4* src;
  uint4* dst[kMaxPeers];
  int n_dst;
  unsigned long long vectors;  // 16-byte elements
};

__global__ void __launch_bounds__(kThreads) push_kernel(const Args a) {
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kThreads;
  unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < a.vectors; i += kUnroll * stride) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) v[u] = __ldg(a.src + i + u * stride);
    for (int p = 0; p < a.n_dst; ++p) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) a.dst[p][i + u * stride] = v[u];
    }
  }
  for (; i < a.vectors; i += stride) {
    const uint4 v = __ldg(a.src + i);
    for (int p = 0; p < a.n_dst; ++p) a.dst[p][i] = v;
  }
}

}  // namespace push
}  // namespace asg

extern "C" int asg_push_to_peers(const void* src, void* const* destinations, int n_destinations, size_t bytes,
                                 int n_ctas, void* stream_ptr) {
  using namespace asg;
  using namespace asg::push;
  ASG_REQUIRE(n_destinations >= 0 && n_destinations <= kMaxPeers, ASG_EINVAL, "at most 7 destinations");
  if (bytes == 0 || n_destinations == 0) return ASG_OK;
  ASG_REQUIRE(src != nullptr && destinations != nullptr, ASG_EINVAL, "src and destinations must not be null");
  ASG_REQUIRE(bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0, ASG_EINVAL,
              "src must be 16-byte aligned and bytes a multiple of 16");
  Args args;
  args.src = static_cast<const uint4*>(src);
  args.n_dst = n_destinations;
  args.vectors = bytes / 16;
  for (int p = 0; p < kMaxPeers; ++p) args.dst[p] = nullptr;
  for (int p = 0; p < n_destinations; ++p) {
    ASG_REQUIRE(destinations[p] != nullptr && (reinterpret_cast<uintptr_t>(destinations[p]) & 15) == 0, ASG_EINVAL,
                "every destination must be a 16-byte aligned pointer");
    args.dst[p] = static_cast<uint4*>(destinations[p]);
  }
  DeviceGuard guard(src);
  ASG_CUDA(guard.status);
  if (n_ctas <= 0) n_ctas = 32;
  const unsigned long long needed = (args.vectors + kThreads - 1) / kThreads;
  if (static_cast<unsigned long long>(n_ctas) > needed) n_ctas = static_cast<int>(needed);
  push_kernel<<<n_ctas, kThreads, 0, static_cast<cudaStream_t>(stream_ptr)>>>(args);
  ASG_CUDA(cudaGetLastError());
  return ASG_OK;
}
