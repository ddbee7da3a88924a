// Shared host/device helpers of libautosage_b200: error reporting, workspace layout, warp
// primitives, cache-hinted loads and the mbarrier / 1-D bulk-copy (TMA) wrappers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "autosage_b200.h"

namespace asg {

// ---------------------------------------------------------------------------------------------
// Host side: per-thread error message, argument checks, device guard.
// ---------------------------------------------------------------------------------------------
char* error_buffer();  // thread-local, 512 bytes (defined in asg_api.cu)

inline int fail(int code, const char* fmt, const char* a = "", const char* b = "") {
  snprintf(error_buffer(), 512, fmt, a, b);
  return code;
}

inline int cuda_fail(cudaError_t e, const char* what) {
  snprintf(error_buffer(), 512, "%s: %s", what, cudaGetErrorString(e));
  return ASG_ECUDA;
}

#define ASG_REQUIRE(cond, code, msg) \
  do {                               \
    if (!(cond)) return ::asg::fail((code), "%s", (msg)); \
  } while (0)

#define ASG_CUDA(call)                                        \
  do {                                                        \
    cudaError_t e__ = (call);                                 \
    if (e__ != cudaSuccess) return ::asg::cuda_fail(e__, #call); \
  } while (0)

// Makes the device that owns `ptr` current for the lifetime of the object.
struct DeviceGuard {
  int previous = -1;
  int target = -1;
  cudaError_t status = cudaSuccess;
  explicit DeviceGuard(const void* ptr) {
    status = cudaGetDevice(&previous);
    if (status != cudaSuccess) return;
    target = previous;
    if (ptr != nullptr) {
      cudaPointerAttributes attr;
      cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
      if (e == cudaSuccess && (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged)) {
        target = attr.device;
      } else if (e != cudaSuccess) {
        cudaGetLastError();  // clear; keep the current device
      }
    }
    if (target != previous) status = cudaSetDevice(target);
  }
  ~DeviceGuard() {
    if (previous >= 0 && target != previous) cudaSetDevice(previous);
  }
};

int sm_count(int device);  // cached per device (asg_api.cu)
long long l2_bytes(int device);  // L2 cache size, cached per device (asg_api.cu)

// ---------------------------------------------------------------------------------------------
// Workspace layout (device memory owned by the caller).
//   [0, 256)                      Header
//   [256, 256 + 4*n_rows)         order[n_rows]: row ids, hubs first, then light rows
//   [align256(...), ...)          block_hist[kBuckets][n_blocks]: scratch of the counting sort
// ---------------------------------------------------------------------------------------------
constexpr int kBuckets = 48;        // 24 hub buckets + 24 light buckets (by floor(log2(degree)))
constexpr int kPlanBlock = 1024;    // rows per block of the counting sort
constexpr int kCounters = 8;
constexpr int kShortDegree = 32;     // rows below this degree form the "short" tail of the light class

struct Header {
  int n_hub;
  int n_light;
  int status;  // first non-zero error a kernel recorded (bounded wait expired, ...)
  int n_rows;
  unsigned long long counter[kCounters];  // work queues of the persistent kernels
  long long hub_threshold;
  int n_short;  // light rows with fewer than kShortDegree edges: the tail of `order`, taken 32 at a time
  int reserved[41];
};
static_assert(sizeof(Header) == 256, "header must stay 256 bytes");

inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }
inline int64_t plan_blocks(int64_t n_rows) { return (n_rows + kPlanBlock - 1) / kPlanBlock; }
inline size_t order_offset() { return sizeof(Header); }
inline size_t hist_offset(int64_t n_rows) { return align256(sizeof(Header) + size_t(4) * size_t(n_rows)); }
inline size_t workspace_bytes(int64_t n_rows) {
  return align256(hist_offset(n_rows) + size_t(4) * kBuckets * size_t(plan_blocks(n_rows) + 1));
}

int check_workspace(const void* workspace, size_t bytes, int64_t n_rows);

// Internal launchers shared between translation units.
int plan_build(const int64_t* crow, int64_t n_rows, int64_t hub_threshold, void* workspace,
               cudaStream_t stream);
int reset_counters(void* workspace, cudaStream_t stream);
// Hub rows (degree >= hub_threshold) only: the aggregated row of hub item i of the plan goes to
// hub_y + i * f and hub_slot[row] = i (asg_spmm.cu).  Takes the flags of asg_spmm_csr_ex.
int spmm_hub_rows_compact(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* hub_y,
                          int* hub_slot, int64_t n_rows, int64_t nnz, int64_t f, int feature_tile, int warps,
                          int64_t hub_threshold, unsigned flags, void* workspace, size_t workspace_bytes,
                          cudaStream_t stream);

// status codes kernels may record in Header::status
constexpr int kStatusBulkWaitExpired = 1;

// ---------------------------------------------------------------------------------------------
// Device side.
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
  return v;
}

__device__ __forceinline__ void st_stream4(float* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_stream1(float* p, float v) {
  asm volatile("st.global.cs.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

// Warp-wide grab of the next item of a work queue.
__device__ __forceinline__ unsigned long long warp_next(unsigned long long* counter) {
  unsigned long long v = 0;
  if (lane_id() == 0) v = atomicAdd(counter, 1ull);
  return __shfl_sync(kFull, v, 0);
}

// ---- mbarrier + 1-D bulk async copy (TMA without a tensor map) -------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while before it answers).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: polls until the phase completes or `limit_ns` of wall time has passed (global
// nanosecond timer; one second unless the caller says otherwise), then returns false so the caller can
// record an error and leave.
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // one second of wall time
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity,
                                                  unsigned long long limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (global_ns() - start > limit_ns) return false;
  }
}
// global -> shared bulk copy; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, unsigned bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// ---- programmatic dependent launch ------------------------------------------------------------
// A kernel launched with launch_overlapped() may start while the kernel before it on the stream is
// still running (as soon as every CTA of that kernel has executed pdl_release_dependents() or has
// exited).  It must call pdl_wait_for_primary() before it ends, so that whatever follows on the
// stream still sees both kernels complete.  Used for the short-row kernels, which touch rows the main
// kernel never touches: they fill the SMs the main kernel's last long rows leave idle.
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_for_primary() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

template <typename Args>
inline cudaError_t launch_overlapped(void (*kernel)(Args), int grid, int threads, size_t smem, cudaStream_t stream,
                                     const Args& args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(grid));
  config.blockDim = dim3(static_cast<unsigned>(threads));
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, args);
}

#endif  // __CUDACC__

}  // namespace asg
