// SpMM for callers that must not allocate device memory.
//
// Every other entry point takes a caller-owned workspace, which normally comes from cudaMalloc or
// a framework's caching allocator.  Some hosts cannot do that at the point where they call us:
// code running inside a region where the allocator is frozen (a memory-budgeted serving process
// that pins its pools at start-up, a plugin called from inside another runtime's callback where
// cudaMalloc would synchronise the device or is simply forbidden), or a thin foreign-language
// binding that has no device allocator at all.  For them the scratch of the SpMM kernel - the
// degree-binned row order and the work-queue counters - lives in a fixed array inside this library's
// device image, so the call needs nothing but its inputs and its output.
#include "asg_common.cuh"

#include <mutex>

namespace asg {

// Largest graph the built-in scratch can hold.
constexpr int64_t kStaticMaxRows = 1 << 20;  // 1,048,576 rows
// Same layout as a caller-provided workspace for kStaticMaxRows rows:
// 256 B header + 4 B per row + counting-sort histogram (48 buckets x 1025 blocks x 4 B).
constexpr size_t kStaticBytes = 256 + size_t(4) * kStaticMaxRows + 256 + size_t(4) * kBuckets * (kStaticMaxRows / kPlanBlock + 1) + 256;

// One copy per GPU that loads the library (about 4.4 MB each), alive until the process exits.  With
// the CUDA runtime's default lazy module loading the copy - and the kernels' code - is placed on a GPU
// the first time this file's code touches that GPU, i.e. during the first asg_spmm_csr_split_noalloc
// call there: that first call makes the driver allocate device memory and may synchronise the device,
// so it belongs in the host's start-up phase, before its allocator is frozen and before any capture.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address, so the
// real address is asked for once per device (with that device current) and remembered.
static std::mutex g_lock;
static void* g_scratch_address[64] = {nullptr};

static int static_scratch(int device, void** out) {
  if (device < 0 || device >= 64) return fail(ASG_EINVAL, "%s", "device index out of range for the built-in scratch");
  std::lock_guard<std::mutex> hold(g_lock);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    ASG_CUDA(cudaGetSymbolAddress(&address, g_static_scratch));
    if (address == nullptr) return fail(ASG_ECUDA, "%s", "cudaGetSymbolAddress returned a null address");
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return ASG_OK;
}

}  // namespace asg

extern "C" {

int64_t asg_static_max_rows(void) { return asg::kStaticMaxRows; }

int asg_spmm_csr_split_noalloc(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* y,
                               int64_t n_rows, int64_t nnz, int64_t f, int feature_tile, int warps_per_block,
                               int64_t hub_threshold, void* stream) {
  using namespace asg;
  if (n_rows > kStaticMaxRows) {
    return fail(ASG_ERANGE, "%s",
                "asg_spmm_csr_split_noalloc handles at most 1048576 rows (the size of its built-in scratch); "
                "use asg_spmm_csr_split with a caller-provided workspace for larger graphs");
  }
  ASG_REQUIRE(n_rows >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(workspace_bytes(n_rows) <= kStaticBytes, ASG_ERANGE, "built-in scratch is too small for n_rows");
  void* scratch = nullptr;
  {
    DeviceGuard guard(x);  // the scratch that matters is the one on the device that owns x
    ASG_CUDA(guard.status);
    if (int rc = static_scratch(guard.target, &scratch)) return rc;
  }
  // Same kernels as asg_spmm_csr_split; the plan is rebuilt on every call, which also resets the
  // status word and the work counters left behind by the previous call.
  return asg_spmm_csr_split(crow, col, val, x, y, n_rows, nnz, f, feature_tile, warps_per_block, hub_threshold,
                            scratch, kStaticBytes, stream);
}

int asg_static_status(const void* device_pointer, int32_t* host_status, void* stream) {
  using namespace asg;
  ASG_REQUIRE(host_status != nullptr, ASG_EINVAL, "host_status must not be null");
  void* scratch = nullptr;
  DeviceGuard guard(device_pointer);  // null: the current device
  ASG_CUDA(guard.status);
  if (int rc = static_scratch(guard.target, &scratch)) return rc;
  return asg_workspace_status(scratch, host_status, stream);
}

}  // extern "C"
