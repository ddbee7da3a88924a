// Library-level entry points: version, error string, workspace sizing and status read-back.
#include "asg_common.cuh"

#include <mutex>

namespace asg {

char* error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

int sm_count(int device) {
  static std::mutex lock;
  static int cached[64];
  static bool known[64] = {false};
  if (device < 0 || device >= 64) device = 0;
  std::lock_guard<std::mutex> hold(lock);
  if (!known[device]) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || value <= 0) {
      cudaGetLastError();
      value = 148;
    }
    cached[device] = value;
    known[device] = true;
  }
  return cached[device];
}

int check_workspace(const void* workspace, size_t bytes, int64_t n_rows) {
  if (workspace == nullptr) return fail(ASG_EWORKSPACE, "%s", "workspace pointer is null");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return fail(ASG_EWORKSPACE, "%s", "workspace must be 256-byte aligned");
  if (bytes < workspace_bytes(n_rows))
    return fail(ASG_EWORKSPACE, "%s", "workspace is smaller than asg_workspace_bytes(n_rows)");
  return ASG_OK;
}

int reset_counters(void* workspace, cudaStream_t stream) {
  Header* h = static_cast<Header*>(workspace);
  ASG_CUDA(cudaMemsetAsync(h->counter, 0, sizeof(h->counter), stream));
  return ASG_OK;
}

}  // namespace asg

extern "C" {

int asg_version(void) { return 100; /* 0.1.0, the reference package's version */ }

const char* asg_last_error_string(void) { return asg::error_buffer(); }

size_t asg_workspace_bytes(int64_t n_rows) {
  if (n_rows < 0) n_rows = 0;
  return asg::workspace_bytes(n_rows);
}

int asg_workspace_status(const void* workspace, int32_t* host_status, void* stream) {
  ASG_REQUIRE(workspace != nullptr && host_status != nullptr, ASG_EINVAL, "workspace and host_status must not be null");
  asg::DeviceGuard guard(workspace);
  ASG_CUDA(guard.status);
  const asg::Header* h = static_cast<const asg::Header*>(workspace);
  ASG_CUDA(cudaMemcpyAsync(host_status, &h->status, sizeof(int32_t), cudaMemcpyDeviceToHost,
                           static_cast<cudaStream_t>(stream)));
  return ASG_OK;
}

}  // extern "C"

namespace asg {
long long l2_bytes(int device) {
  static std::mutex lock;
  static long long cached[64];
  static bool known[64] = {false};
  if (device < 0 || device >= 64) device = 0;
  std::lock_guard<std::mutex> hold(lock);
  if (!known[device]) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrL2CacheSize, device) != cudaSuccess || value <= 0) {
      cudaGetLastError();
      value = 126 << 20;
    }
    cached[device] = value;
    known[device] = true;
  }
  return cached[device];
}
}  // namespace asg
