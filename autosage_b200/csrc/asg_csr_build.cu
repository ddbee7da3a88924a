// COO -> CSR on the device: rows keyed by one endpoint of every edge, edges of a row in input order.
//
// Replaces edge_index_to_csr (autosage/utils/csr.py:6-26: stable argsort of the row ids, bincount,
// cumsum, gather) and the second stable argsort that AutoSAGEConv.forward runs to permute edge weights
// (autosage/conv.py:44-45).  Those sort 64-bit keys over all 64 bits, twice.  Here the row ids are
// narrowed to 32 bits and paired with their edge number, the pairs go through ONE least-significant-
// digit radix sort over only the bits a row id can have (22 bits for 2.4 M rows: three 8-bit passes
// instead of eight; CUB's DeviceRadixSort, which is stable), and one gather pass writes the column
// array, the permutation and the permuted weights together.  Row pointers come from a binary search of
// the sorted keys (no atomics, no scan): crow[r] = number of edges whose row id is below r, which is
// what bincount + cumsum give.  Row ids must lie in [0, n_rows): only the low key_bits(n_rows) bits of
// an id take part in the sort, so an id outside that range would be placed by its low bits and the row
// pointers would no longer describe the column array.  The kernels do not check this (the Python
// caller does under AUTOSAGE_CHECK_INDICES=1).
#include "asg_common.cuh"

#include <cub/device/device_radix_sort.cuh>

namespace asg {
namespace csr_build {

constexpr int kThreads = 256;

struct Layout {
  size_t keys_in, keys_out, ids_in, ids_out, sort_temp, total;
};

inline size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

inline int key_bits(int64_t n_rows) {
  int bits = 1;
  while (bits < 31 && (int64_t{1} << bits) < n_rows) ++bits;
  return bits;
}

inline cudaError_t sort_temp_bytes(int64_t n_edges, int64_t n_rows, size_t* bytes) {
  *bytes = 0;
  return cub::DeviceRadixSort::SortPairs(nullptr, *bytes, static_cast<const int32_t*>(nullptr),
                                         static_cast<int32_t*>(nullptr), static_cast<const int32_t*>(nullptr),
                                         static_cast<int32_t*>(nullptr), n_edges, 0, key_bits(n_rows));
}

inline cudaError_t layout(int64_t n_edges, int64_t n_rows, Layout* out) {
  size_t temp = 0;
  cudaError_t e = sort_temp_bytes(n_edges, n_rows, &temp);
  const size_t column = align256(static_cast<size_t>(n_edges) * sizeof(int32_t));
  out->keys_in = 0;
  out->keys_out = column;
  out->ids_in = 2 * column;
  out->ids_out = 3 * column;
  out->sort_temp = 4 * column;
  out->total = 4 * column + align256(temp) + 256;
  return e;
}

// keys[e] = row id narrowed to 32 bits, ids[e] = e
__global__ void __launch_bounds__(kThreads) narrow_kernel(const int64_t* __restrict__ row_of_edge, int32_t* __restrict__ keys,
                                                          int32_t* __restrict__ ids, long long n_edges) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < n_edges; e += stride) {
    keys[e] = static_cast<int32_t>(row_of_edge[e]);
    ids[e] = static_cast<int32_t>(e);
  }
}

// crow[r] = first position whose sorted key is >= r (r = 0 .. n_rows)
__global__ void __launch_bounds__(kThreads) row_pointer_kernel(const int32_t* __restrict__ sorted_keys, long long n_edges,
                                                               int64_t* __restrict__ crow, long long n_rows) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long r = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; r <= n_rows; r += stride) {
    long long lo = 0, hi = n_edges;
    while (lo < hi) {
      const long long mid = (lo + hi) >> 1;
      if (static_cast<long long>(sorted_keys[mid]) < r) lo = mid + 1; else hi = mid;
    }
    crow[r] = lo;
  }
}

// col[i] = col_of_edge[order[i]], perm[i] = order[i], val_out[i] = val_in[order[i]]
__global__ void __launch_bounds__(kThreads) gather_kernel(const int32_t* __restrict__ order, const int64_t* __restrict__ col_of_edge,
                                                          const float* __restrict__ val_in, int64_t* __restrict__ col,
                                                          int64_t* __restrict__ perm, float* __restrict__ val_out,
                                                          long long n_edges) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_edges; i += stride) {
    const int32_t e = order[i];
    col[i] = col_of_edge[e];
    if (perm != nullptr) perm[i] = e;
    if (val_out != nullptr) val_out[i] = val_in[e];
  }
}

}  // namespace csr_build
}  // namespace asg

extern "C" size_t asg_csr_build_workspace_bytes(int64_t n_edges, int64_t n_rows) {
  using namespace asg::csr_build;
  if (n_edges <= 0 || n_rows < 0 || n_edges > 2147483647ll) return 256;
  Layout l;
  if (layout(n_edges, n_rows, &l) != cudaSuccess) return 0;
  return l.total;
}

extern "C" int asg_csr_from_edges(const int64_t* row_of_edge, const int64_t* col_of_edge, const float* val_in,
                                  int64_t n_edges, int64_t n_rows, int64_t* crow, int64_t* col, int64_t* perm,
                                  float* val_out, void* workspace, size_t workspace_bytes, void* stream_ptr) {
  using namespace asg;
  using namespace asg::csr_build;
  ASG_REQUIRE(n_edges >= 0 && n_rows >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(n_edges <= 2147483647ll && n_rows <= 2147483647ll, ASG_ERANGE,
              "edge and row counts must fit 31 bits (edge numbers and row ids are sorted as 32-bit values)");
  ASG_REQUIRE(crow != nullptr, ASG_EINVAL, "crow must not be null");
  ASG_REQUIRE((val_out == nullptr) || (val_in != nullptr), ASG_EINVAL, "val_out needs val_in");
  DeviceGuard guard(crow);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const int grid = sm_count(guard.target) * 8;
  if (n_edges == 0) {
    ASG_CUDA(cudaMemsetAsync(crow, 0, static_cast<size_t>(n_rows + 1) * sizeof(int64_t), stream));
    return ASG_OK;
  }
  ASG_REQUIRE(row_of_edge != nullptr && col_of_edge != nullptr && col != nullptr, ASG_EINVAL,
              "row_of_edge, col_of_edge and col must not be null");
  Layout l;
  ASG_CUDA(layout(n_edges, n_rows, &l));
  ASG_REQUIRE(workspace != nullptr && workspace_bytes >= l.total, ASG_EWORKSPACE,
              "workspace smaller than asg_csr_build_workspace_bytes(n_edges, n_rows)");
  ASG_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, ASG_EINVAL, "workspace must be 256-byte aligned");
  char* base = static_cast<char*>(workspace);
  int32_t* keys_in = reinterpret_cast<int32_t*>(base + l.keys_in);
  int32_t* keys_out = reinterpret_cast<int32_t*>(base + l.keys_out);
  int32_t* ids_in = reinterpret_cast<int32_t*>(base + l.ids_in);
  int32_t* ids_out = reinterpret_cast<int32_t*>(base + l.ids_out);
  size_t temp_bytes = l.total - l.sort_temp;

  narrow_kernel<<<grid, kThreads, 0, stream>>>(row_of_edge, keys_in, ids_in, n_edges);
  ASG_CUDA(cudaGetLastError());
  ASG_CUDA(cub::DeviceRadixSort::SortPairs(base + l.sort_temp, temp_bytes, keys_in, keys_out, ids_in, ids_out, n_edges, 0,
                                           key_bits(n_rows), stream));
  row_pointer_kernel<<<grid, kThreads, 0, stream>>>(keys_out, n_edges, crow, n_rows);
  ASG_CUDA(cudaGetLastError());
  gather_kernel<<<grid, kThreads, 0, stream>>>(ids_out, col_of_edge, val_in, col, perm, val_out, n_edges);
  ASG_CUDA(cudaGetLastError());
  return ASG_OK;
}
