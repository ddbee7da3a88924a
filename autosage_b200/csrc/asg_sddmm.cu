// CSR SDDMM for sm_100a: out[e] = <Q[row(e), :], K[col[e], :]>.
//
// Persistent kernels over the work queues of the plan (see asg_plan.cu):
//   queue 0  hub rows, one CTA each: the warps of the CTA take the row's 32-edge batches round-robin
//   queue 1  light rows of 32 edges or more, one warp each
//   queue 2  light rows of fewer than 32 edges, 32 rows per grab (sddmm_short_kernel)
// For a batch the warp loads 32 column indices with one coalesced load, keeps the Q row in
// registers, gathers the K rows with vector loads (U instructions in flight per lane), and
// turns the per-lane partial dot products into one finished value per lane with a
// reduce-scatter (about one shuffle per edge instead of five), so the 32 results leave as one
// coalesced 128-byte store.
//
// Replaces csrc/sddmm_csr_op.cu:19-83 of the reference (warp-per-row kernel with scalar loads, a
// five-step shuffle reduction and a 4-byte store per edge; CTA-per-hub kernel of the same shape).
#include "asg_tile.cuh"

namespace asg {

struct SddmmArgs {
  const int64_t* crow;
  const int64_t* col;
  const float* q;
  const float* k;
  float* out;
  Header* header;
  const int* order;
  int f;
  int n_tiles;
  int fixed_tile;  // >= 0: this launch covers only that feature tile and, for tile > 0, adds to out
};

constexpr int kTilePasses = -2;  // SddmmArgs::fixed_tile on the host side: "launch once per tile"

// FULL: the feature count is a multiple of the tile (chosen on the host), so no lane is ever outside the
// row and the gathers need no predicates.  Every batch then runs as a whole 32-edge batch: the last, partly
// filled batch of a row is moved back to end at the row's last edge - the edges it shares with the batch
// before it are computed twice and stored once - and in a row shorter than 32 edges the spare lanes gather
// the row's first column and store nothing.
template <int VW, int G, int NV, int U, bool FULL>
__device__ __forceinline__ void sddmm_row_batches(const SddmmArgs& a, int row, long long first, long long stride,
                                                  int lane, uint64_t pol_keep, uint64_t pol_stream) {
  constexpr int EPI = 32 / G;
  constexpr int FT = VW * G * NV;
  const int l = lane % G;
  const int sub = lane / G;
  const int f = a.f;
  const long long e = a.crow[row + 1];
  const float* qrow = a.q + static_cast<size_t>(row) * f;

  float q[NV][VW];
  bool fvalid[NV];
  int foff[NV];
  auto load_q = [&](int tile) {
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      foff[v] = tile * FT + VW * (l + G * v);
      fvalid[v] = foff[v] < f;
      if (fvalid[v]) {
        VecIO<VW>::load(q[v], qrow + foff[v], pol_stream);  // read once: must not push K out of L2
      } else {
#pragma unroll
        for (int i = 0; i < VW; ++i) q[v][i] = 0.f;
      }
    }
  };
  const bool one_tile = a.n_tiles == 1 || a.fixed_tile >= 0;
  if (one_tile) load_q(a.fixed_tile >= 0 ? a.fixed_tile : 0);

  if (FULL) {
    const long long s_row = a.crow[row];
    const int edge = l * EPI + sub;
    for (long long p = first; p < e; p += stride) {
      long long start = p;
      int skip = 0;  // leading edges of the batch that an earlier batch has already written
      if (e - p < 32 && e - s_row >= 32) {
        start = e - 32;
        skip = static_cast<int>(p - start);
      }
      long long at = start + lane;
      if (at >= e) at = s_row;
      const int c_l = static_cast<int>(ld_index(a.col + at, pol_stream));
      float part[G];
#pragma unroll
      for (int i = 0; i < G; ++i) part[i] = 0.f;
      if (one_tile) {
        batch_dots_impl<VW, G, NV, U, false>(a.k, f, c_l, 32, sub, q, fvalid, foff, pol_keep, part);
      } else {
        for (int tile = 0; tile < a.n_tiles; ++tile) {
          load_q(tile);
          batch_dots_impl<VW, G, NV, U, false>(a.k, f, c_l, 32, sub, q, fvalid, foff, pol_keep, part);
        }
      }
      float dot = group_reduce_scatter<G>(part, l);
      const long long pos = start + edge;
      if (edge >= skip && pos < e) {
        if (a.fixed_tile > 0) dot += a.out[pos];  // partial sum of the earlier tiles (earlier launches)
        st_stream1(a.out + pos, dot);
      }
    }
    return;
  }
  for (long long p = first; p < e; p += stride) {
    const int cnt = e - p < 32 ? static_cast<int>(e - p) : 32;
    int c_l = 0;
    if (lane < cnt) c_l = static_cast<int>(ld_index(a.col + p + lane, pol_stream));
    float part[G];
#pragma unroll
    for (int i = 0; i < G; ++i) part[i] = 0.f;
    if (one_tile) {
      batch_dots<VW, G, NV, U, false>(a.k, f, c_l, cnt, sub, q, fvalid, foff, pol_keep, part);
    } else {
      for (int tile = 0; tile < a.n_tiles; ++tile) {
        load_q(tile);
        batch_dots<VW, G, NV, U, false>(a.k, f, c_l, cnt, sub, q, fvalid, foff, pol_keep, part);
      }
    }
    float dot = group_reduce_scatter<G>(part, l);
    const int edge = l * EPI + sub;
    if (edge < cnt) {
      if (a.fixed_tile > 0) dot += a.out[p + edge];  // partial sum of the earlier tiles (earlier launches)
      st_stream1(a.out + p + edge, dot);
    }
  }
}

// 64-feature tiles (the L2-resident passes): at most 64 registers, so that four 8-warp CTAs fit an SM; the
// gather is latency-bound there and pays for warps, not for registers.
template <int VW, int G, int NV, int U, bool FULL>
__global__ void __launch_bounds__(512, (VW * G * NV <= 64 ? 2 : 1)) sddmm_kernel(const SddmmArgs a) {
  pdl_release_dependents();  // the short-row kernel may move in as CTAs of this one retire
  __shared__ int s_item;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  const uint64_t pol_keep = policy_evict_last();
  const uint64_t pol_stream = policy_evict_first();
  const int n_hub = a.header->n_hub;
  const int n_light = a.header->n_light;

  if (n_hub > 0) {
    for (;;) {
      __syncthreads();
      if (tid == 0) {
        const unsigned long long it = atomicAdd(&a.header->counter[0], 1ull);
        s_item = it < static_cast<unsigned long long>(n_hub) ? static_cast<int>(it) : -1;
      }
      __syncthreads();
      const int item = s_item;
      if (item < 0) break;
      const int row = a.order[item];
      const long long s = a.crow[row];
      sddmm_row_batches<VW, G, NV, U, FULL>(a, row, s + 32ll * warp, 32ll * n_warps, lane, pol_keep, pol_stream);
    }
  }
  const int n_short = a.header->n_short;
  const int n_medium = n_light - n_short;  // light rows of 32 edges or more: one row per grab
  if (n_medium > 0) {
    const int* light = a.order + n_hub;
    for (;;) {
      const unsigned long long it = warp_next(&a.header->counter[1]);
      if (it >= static_cast<unsigned long long>(n_medium)) break;
      const int row = light[it];
      sddmm_row_batches<VW, G, NV, U, FULL>(a, row, a.crow[row], 32ll, lane, pol_keep, pol_stream);
    }
  }
}

// Queue 2 as a kernel of its own (launched right after the main one; inlined it raised the main
// kernel from 78 to 120 registers).  Rows of fewer than 32 edges, 32 rows per grab: ids and row
// pointers arrive with one coalesced load each and the next row's columns are fetched while the current
// row's K rows are gathered.
template <int VW, int G, int NV, int U>
__global__ void __launch_bounds__(512) sddmm_short_kernel(const SddmmArgs a) {
  const int lane = threadIdx.x & 31;
  const uint64_t pol_keep = policy_evict_last();
  const uint64_t pol_stream = policy_evict_first();
  const int n_hub = a.header->n_hub;
  const int n_short = a.header->n_short;
  const int n_medium = a.header->n_light - n_short;
  if (n_short > 0) {
    constexpr int EPI = 32 / G;
    constexpr int FT = VW * G * NV;
    const int l = lane % G;
    const int sub = lane / G;
    const int f = a.f;
    const int* shorts = a.order + n_hub + n_medium;
    const int n_batches = (n_short + 31) / 32;
    for (;;) {
      const unsigned long long it = warp_next(&a.header->counter[2]);
      if (it >= static_cast<unsigned long long>(n_batches)) break;
      const int first = static_cast<int>(it) * 32;
      const int n_here = n_short - first < 32 ? n_short - first : 32;
      int row_l = 0;
      long long s_l = 0, e_l = 0;
      if (lane < n_here) {
        row_l = shorts[first + lane];
        s_l = a.crow[row_l];
        e_l = a.crow[row_l + 1];
      }
      long long s_cur = __shfl_sync(kFull, s_l, 0);
      int cnt_cur = static_cast<int>(__shfl_sync(kFull, e_l, 0) - s_cur);
      int c_next = 0;
      if (lane < cnt_cur) c_next = static_cast<int>(ld_index(a.col + s_cur + lane, pol_stream));
      for (int r = 0; r < n_here; ++r) {
        const int row = __shfl_sync(kFull, row_l, r);
        const long long s = s_cur;
        const int cnt = cnt_cur;
        const int c_l = c_next;
        if (r + 1 < n_here) {
          s_cur = __shfl_sync(kFull, s_l, r + 1);
          cnt_cur = static_cast<int>(__shfl_sync(kFull, e_l, r + 1) - s_cur);
          if (lane < cnt_cur) c_next = static_cast<int>(ld_index(a.col + s_cur + lane, pol_stream));
        }
        if (cnt == 0) continue;
        const float* qrow = a.q + static_cast<size_t>(row) * f;
        float part[G];
#pragma unroll
        for (int i = 0; i < G; ++i) part[i] = 0.f;
        for (int tile = 0; tile < a.n_tiles; ++tile) {
          float q[NV][VW];
          bool fvalid[NV];
          int foff[NV];
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            foff[v] = tile * FT + VW * (l + G * v);
            fvalid[v] = foff[v] < f;
            if (fvalid[v]) {
              VecIO<VW>::load(q[v], qrow + foff[v], pol_stream);
            } else {
#pragma unroll
              for (int i = 0; i < VW; ++i) q[v][i] = 0.f;
            }
          }
          batch_dots<VW, G, NV, U, false>(a.k, f, c_l, cnt, sub, q, fvalid, foff, pol_keep, part);
        }
        const float dot = group_reduce_scatter<G>(part, l);
        const int edge = l * EPI + sub;
        if (edge < cnt) st_stream1(a.out + s + edge, dot);
      }
    }
  }
  pdl_wait_for_primary();  // do not complete before the main kernel has
}

template <int VW, int G, int NV, int U>
static int launch_instance(const SddmmArgs& args, int warps, cudaStream_t stream, int device) {
  // whole feature tiles only: the kernel without predicates on the gathers
  auto kernel = args.f % (VW * G * NV) == 0 ? sddmm_kernel<VW, G, NV, U, true> : sddmm_kernel<VW, G, NV, U, false>;
  const int threads = warps * 32;
  int per_sm = 0;
  ASG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0));
  if (per_sm < 1) per_sm = 1;
  if (args.fixed_tile == kTilePasses) {
    // One launch per feature tile, tile 0 first: while a pass runs only an N x FT slice of K is hot
    // in L2.  Partial sums travel through `out`; stream order makes pass t see pass t-1.
    SddmmArgs pass = args;
    for (int t = 0; t < args.n_tiles; ++t) {
      if (t > 0) {
        if (int rc = reset_counters(args.header, stream)) return rc;
      }
      pass.fixed_tile = t;
      kernel<<<sm_count(device) * per_sm, threads, 0, stream>>>(pass);
      ASG_CUDA(cudaGetLastError());
    }
  } else {
    kernel<<<sm_count(device) * per_sm, threads, 0, stream>>>(args);
    ASG_CUDA(cudaGetLastError());
  }
  auto short_kernel = sddmm_short_kernel<VW, G, NV, U>;
  int short_per_sm = 0;
  ASG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&short_per_sm, short_kernel, threads, 0));
  if (short_per_sm < 1) short_per_sm = 1;
  ASG_CUDA(launch_overlapped(short_kernel, sm_count(device) * short_per_sm, threads, 0, stream, args));
  return ASG_OK;
}

constexpr int kSddmmLoadsInFlight = 8;  // gather instructions issued per lane before their results are used

// K larger than this (bytes) no longer sits comfortably in L2 next to the streamed CSR and output:
// the product is then computed in passes of 64 features.
constexpr long long kTilePassBytes = 64ll << 20;

// Picks the narrowest tile that covers f (so Q stays in registers); above 512 floats the tile is
// 512 wide and Q is re-read per batch.
static int launch_sddmm(SddmmArgs& args, int vw, cudaStream_t stream, int warps, int device) {
  constexpr int U = kSddmmLoadsInFlight;
  const int f = args.f;
  auto tiles = [&](int ft) { args.n_tiles = (f + ft - 1) / ft; };
  if (vw == 8 && args.fixed_tile == kTilePasses) {
    tiles(64);
    return launch_instance<8, 8, 1, U / 2>(args, warps, stream, device);
  }
  if (vw == 8) {
    if (f <= 32) { tiles(32); return launch_instance<8, 4, 1, U / 2>(args, warps, stream, device); }
    if (f <= 64) { tiles(64); return launch_instance<8, 8, 1, U / 2>(args, warps, stream, device); }
    if (f <= 128) { tiles(128); return launch_instance<8, 16, 1, U / 2>(args, warps, stream, device); }
    if (f <= 256) { tiles(256); return launch_instance<8, 32, 1, U / 2>(args, warps, stream, device); }
    tiles(512);
    return launch_instance<8, 32, 2, U / 4>(args, warps, stream, device);
  }
  if (vw == 4) {
    if (f <= 32) { tiles(32); return launch_instance<4, 8, 1, U>(args, warps, stream, device); }
    if (f <= 64) { tiles(64); return launch_instance<4, 16, 1, U>(args, warps, stream, device); }
    if (f <= 128) { tiles(128); return launch_instance<4, 32, 1, U>(args, warps, stream, device); }
    if (f <= 256) { tiles(256); return launch_instance<4, 32, 2, U / 2>(args, warps, stream, device); }
    tiles(512);
    return launch_instance<4, 32, 4, U / 4>(args, warps, stream, device);
  }
  if (f <= 32) { tiles(32); return launch_instance<1, 32, 1, U>(args, warps, stream, device); }
  if (f <= 64) { tiles(64); return launch_instance<1, 32, 2, U / 2>(args, warps, stream, device); }
  tiles(128);
  return launch_instance<1, 32, 4, U / 4>(args, warps, stream, device);
}

static bool aligned_to(const void* p, size_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; }

static int sddmm_entry(const int64_t* crow, const int64_t* col, const float* q, const float* k, float* out,
                       int64_t n_rows, int64_t nnz, int64_t f, int warps, int64_t hub_threshold, unsigned flags,
                       void* workspace, size_t workspace_bytes, void* stream_ptr) {
  ASG_REQUIRE(n_rows >= 0 && nnz >= 0 && f >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(n_rows <= 2147483647ll - 2048 && f <= 2147483647ll, ASG_ERANGE,
              "SDDMM dimensions exceed the kernel index range");
  ASG_REQUIRE(warps == 2 || warps == 4 || warps == 8 || warps == 16, ASG_EINVAL,
              "warps_per_block must be 2, 4, or 8");
  ASG_REQUIRE(!(flags & ASG_FLAG_ACCUMULATE), ASG_EINVAL, "SDDMM does not accumulate");
  if (n_rows == 0 || nnz == 0) return ASG_OK;
  ASG_REQUIRE(crow != nullptr && col != nullptr && out != nullptr, ASG_EINVAL, "crow, col and out must not be null");
  ASG_REQUIRE(f == 0 || (q != nullptr && k != nullptr), ASG_EINVAL, "query and key must not be null");
  if (int rc = check_workspace(workspace, workspace_bytes, n_rows)) return rc;
  DeviceGuard guard(out);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (f == 0) {
    ASG_CUDA(cudaMemsetAsync(out, 0, size_t(4) * size_t(nnz), stream));
    return ASG_OK;
  }
  if (flags & ASG_FLAG_PLAN_READY) {
    if (int rc = reset_counters(workspace, stream)) return rc;
  } else {
    if (int rc = plan_build(crow, n_rows, hub_threshold, workspace, stream)) return rc;
  }
  int vw = 1;
  if (!(flags & ASG_FLAG_NO_VEC4)) {
    if (f % 8 == 0 && aligned_to(q, 32) && aligned_to(k, 32)) vw = 8;
    else if (f % 4 == 0 && aligned_to(q, 16) && aligned_to(k, 16)) vw = 4;
  }
  SddmmArgs args;
  args.crow = crow;
  args.col = col;
  args.q = q;
  args.k = k;
  args.out = out;
  args.header = static_cast<Header*>(workspace);
  args.order = reinterpret_cast<const int*>(static_cast<const char*>(workspace) + order_offset());
  args.f = static_cast<int>(f);
  args.n_tiles = 1;
  const bool passes = vw == 8 && f >= 128 && f % 64 == 0 && !(flags & ASG_FLAG_NO_TILE_PASSES) &&
                      static_cast<long long>(n_rows) * f * 4 > kTilePassBytes;
  args.fixed_tile = passes ? kTilePasses : -1;
  return launch_sddmm(args, vw, stream, warps, guard.target);
}

}  // namespace asg

extern "C" {

int asg_sddmm_csr_ex(const int64_t* crow, const int64_t* col, const float* q, const float* k, float* out,
                     int64_t n_rows, int64_t nnz, int64_t f, int warps_per_block, int64_t hub_threshold,
                     unsigned flags, void* workspace, size_t workspace_bytes, void* stream) {
  return asg::sddmm_entry(crow, col, q, k, out, n_rows, nnz, f, warps_per_block, hub_threshold, flags, workspace,
                          workspace_bytes, stream);
}

int asg_sddmm_csr_split(const int64_t* crow, const int64_t* col, const float* q, const float* k, float* out,
                        int64_t n_rows, int64_t nnz, int64_t f, int warps_per_block, int64_t hub_threshold,
                        void* workspace, size_t workspace_bytes, void* stream) {
  if (hub_threshold <= 0 || hub_threshold > 2147483647ll)
    return asg::fail(ASG_EINVAL, "%s", "hub_threshold must be a positive 32-bit integer");
  return asg::sddmm_entry(crow, col, q, k, out, n_rows, nnz, f, warps_per_block, hub_threshold, 0u, workspace,
                          workspace_bytes, stream);
}

int asg_sddmm_csr(const int64_t* crow, const int64_t* col, const float* q, const float* k, float* out,
                  int64_t n_rows, int64_t nnz, int64_t f, void* workspace, size_t workspace_bytes, void* stream) {
  // SDDMM has no reduction across the edges of a row, so only very long rows gain from a whole CTA
  return asg::sddmm_entry(crow, col, q, k, out, n_rows, nnz, f, 8, 8192, 0u, workspace, workspace_bytes, stream);
}

}  // extern "C"
