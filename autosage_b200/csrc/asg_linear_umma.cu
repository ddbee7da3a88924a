// The layer's Linear (autosage/conv.py:55: out = aggregated @ weight^T + bias) on the 5th-generation
// tensor cores at float32 accuracy, hand-written for sm_100a.
//
// Every float32 operand is split into three bfloat16 pieces (hi + mid + lo reproduces the value to
// 2^-24); of the nine piece products the six that matter at float32 precision are issued as
// tcgen05.mma (bf16 x bf16 -> f32, M = 128, N = out_features, K = 16 per instruction) into ONE float32
// accumulator in tensor memory, smallest terms first.
//
// One persistent CTA per SM walks row tiles of 128 rows.  Warp roles:
//   warp 0        allocates tensor memory; its lane 0 issues every MMA and commit
//   warp 1        lane 0 streams the weight pieces into a 3-stage shared-memory ring with 1-D bulk
//                 async copies; the pieces were split once and stored in global memory in exactly the
//                 128-byte-swizzled K-major image the MMA reads (asg::linear_umma::pack_weight)
//   warps 4-11    epilogue, two warps per tensor-memory lane quarter: tensor memory -> registers
//                 (tcgen05.ld) -> + bias -> a per-warp staging tile in shared memory -> coalesced
//                 streaming stores, 512 bytes per instruction
//   warps 12-19   producers: read 128 rows x 64 features of x (float4 loads, 8 in flight per lane),
//                 split them, write the three pieces into a 2-stage ring in the swizzled layout
// The accumulator is double-buffered (2 x N tensor-memory columns), so the epilogue of tile t runs under
// the MMAs of tile t+1, and the producers refill one 64-feature stage while the MMAs read the other.
// Every wait is on an mbarrier, bounded in time, and a wait that gives up sets a status word, raises a
// CTA-wide abort flag and the CTA leaves through the common exit, which frees its tensor memory.
#include "asg_umma.cuh"
#include "asg_tile.cuh"

namespace asg {
namespace linear_umma {

using namespace umma;

constexpr int kBlockM = 128;
constexpr int kPieces = 3;
constexpr int kAStages = 2;   // ring of (tile, 64-feature block) stages of the split x tile
constexpr int kBStages = 3;   // ring of weight-piece stages
constexpr int kThreads = 640;
constexpr int kEpilogueWarp0 = 4;    // a multiple of 4: warp index mod 4 is the tensor-memory lane quarter
constexpr int kEpilogueWarps = 8;
constexpr int kProducerWarp0 = 12;
constexpr int kProducerWarps = 8;
constexpr int kMaxN = 256;
constexpr int kAPieceBytes = kBlockM * kSwizzleRowBytes;          // 16 KB: 128 rows x 64 bf16
constexpr int kAStageBytes = kPieces * kAPieceBytes;               // 48 KB
constexpr int kBStageStride = kMaxN * kSwizzleRowBytes;            // 32 KB
constexpr int kStagingRow = 32;                                    // floats; 16-byte chunks XOR-swizzled by row
constexpr int kStagingBytes = 8 * 32 * kStagingRow * 4;            // one 32 x 32 tile per epilogue warp
constexpr unsigned long long kWaitLimitNs = 500ull * 1000ull * 1000ull;

constexpr int kStatusWaitExpired = 2;
constexpr unsigned long long kSelftestLimitNs = 20ull * 1000ull * 1000ull;   // the self-test's wait gives up after 20 ms

struct Smem {
  static constexpr int a_ring = 0;
  static constexpr int b_ring = a_ring + kAStages * kAStageBytes;
  static constexpr int staging = b_ring + kBStages * kBStageStride;
  static constexpr int bias = staging + kStagingBytes;
  static constexpr int barriers = bias + kMaxN * 4;
  static constexpr int total = barriers + 256;
};
constexpr int kDynamicSmem = Smem::total + 1024;  // slack to align the carve-up to 1024 bytes

struct Barriers {
  uint64_t a_full[kAStages], a_empty[kAStages];
  uint64_t b_full[kBStages], b_empty[kBStages];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t mma_done;   // the MMA thread's last commit when it leaves early
  uint64_t idle;       // self-test: nothing ever arrives here
  uint32_t tmem_base;
  int abort;
};
static_assert(kDynamicSmem <= 232448, "exceeds the 227 KB a CTA may use");
static_assert(sizeof(Barriers) <= 256, "barrier block must fit its slot");

struct Args {
  const float* x;
  const float* bias;
  float* out;
  const unsigned char* packed;  // weight pieces in the shared-memory image, stage after stage
  int* status;
  int rows, k, n;
  int k_blocks, n_tiles;
  unsigned tmem_columns;
  int selftest_stall;  // ASG_FLAG_SELFTEST_STALL: the MMA thread waits, before its second tile, on a barrier nothing arrives on
};

// One thread per weight element: split it and store the pieces where the MMA will read them.
// Stage (kb, j) holds piece j (0 = lo, 1 = mid, 2 = hi) of weight[:, 64 kb .. 64 kb + 63] as N rows of
// 128 swizzled bytes; stages follow one another in the order the kernel consumes them.
__global__ void __launch_bounds__(256) pack_weight(const float* __restrict__ weight, unsigned char* __restrict__ packed,
                                                   int n, int k) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n * k) return;
  const int row = e / k, col = e - row * k;
  const int kb = col / kBlockK, kk = col - kb * kBlockK;
  const float w = weight[e];
  const __nv_bfloat16 hi = __float2bfloat16_rn(w);
  const float r1 = w - __bfloat162float(hi);
  const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
  const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
  const size_t stage_bytes = static_cast<size_t>(n) * kSwizzleRowBytes;
  unsigned char* base = packed + static_cast<size_t>(kb) * kPieces * stage_bytes + swizzled_offset(row, kk);
  *reinterpret_cast<__nv_bfloat16*>(base) = lo;
  *reinterpret_cast<__nv_bfloat16*>(base + stage_bytes) = mid;
  *reinterpret_cast<__nv_bfloat16*>(base + 2 * stage_bytes) = hi;
}

__global__ void __launch_bounds__(kThreads, 1) linear_kernel(const Args a) {
  extern __shared__ unsigned char raw_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + Smem::barriers);
  float* bias_s = reinterpret_cast<float*>(smem + Smem::bias);
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile int* abort_flag = &bars->abort;

  if (tid == 0) {
    for (int i = 0; i < kAStages; ++i) {
      mbar_init(&bars->a_full[i], kProducerWarps);
      mbar_init(&bars->a_empty[i], 1);
    }
    for (int i = 0; i < kBStages; ++i) {
      mbar_init(&bars->b_full[i], 1);
      mbar_init(&bars->b_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->acc_full[i], 1);
      mbar_init(&bars->acc_empty[i], kEpilogueWarps);
    }
    mbar_init(&bars->mma_done, 1);
    mbar_init(&bars->idle, 1);
    bars->abort = 0;
    mbar_fence_init();
  }
  for (int i = tid; i < a.n; i += kThreads) bias_s[i] = a.bias != nullptr ? a.bias[i] : 0.f;
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, a.tmem_columns);
    tmem_relinquish_alloc_permit();
  }
  fence_before_thread_sync();
  __syncthreads();
  fence_after_thread_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t a_ring = smem_u32(smem + Smem::a_ring);
  const uint32_t b_ring = smem_u32(smem + Smem::b_ring);
  const int first_tile = blockIdx.x;
  const int tile_step = gridDim.x;

  auto give_up = [&]() {
    atomicCAS(a.status, 0, kStatusWaitExpired);
    bars->abort = 1;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = instruction_descriptor(kBlockM, a.n);
      unsigned ia = 0, ib = 0, it = 0;
      bool alive = true;
      for (int tile = first_tile; tile < a.n_tiles && alive; tile += tile_step, ++it) {
        const unsigned buf = it & 1u;
        if (a.selftest_stall && it == 1 && !mbar_wait_or_abort(&bars->idle, 0u, abort_flag, kSelftestLimitNs)) {
          give_up();
          alive = false;
          break;
        }
        if (!mbar_wait_or_abort(&bars->acc_empty[buf], ((it >> 1) & 1u) ^ 1u, abort_flag, kWaitLimitNs)) {
          give_up();
          alive = false;
          break;
        }
        fence_after_thread_sync();
        const uint32_t acc = tmem_base + buf * static_cast<uint32_t>(a.n);
        uint32_t accumulate = 0;
        for (int kb = 0; kb < a.k_blocks && alive; ++kb, ++ia) {
          const unsigned sa = ia % kAStages;
          if (!mbar_wait_or_abort(&bars->a_full[sa], (ia / kAStages) & 1u, abort_flag, kWaitLimitNs)) {
            give_up();
            alive = false;
            break;
          }
          // weight piece j (0 = lo, 1 = mid, 2 = hi) meets the x pieces that keep the product above
          // 2^-24: lo x hi; mid x {mid, hi}; hi x {lo, mid, hi}.  x piece index: 0 = hi, 1 = mid, 2 = lo.
          for (int j = 0; j < kPieces; ++j, ++ib) {
            const unsigned sb = ib % kBStages;
            if (!mbar_wait_or_abort(&bars->b_full[sb], (ib / kBStages) & 1u, abort_flag, kWaitLimitNs)) {
              give_up();
              alive = false;
              break;
            }
            fence_after_thread_sync();
            const uint32_t b_stage = b_ring + sb * kBStageStride;
            for (int xp = j; xp >= 0; --xp) {  // smallest x piece first
              const uint32_t a_piece = a_ring + sa * kAStageBytes + xp * kAPieceBytes;
#pragma unroll
              for (int kk = 0; kk < kBlockK / kInstrK; ++kk) {
                mma_bf16(acc, smem_descriptor(a_piece + kk * kInstrK * 2), smem_descriptor(b_stage + kk * kInstrK * 2),
                         idesc, accumulate);
                accumulate = 1;
              }
            }
            mma_commit(&bars->b_empty[sb]);  // the weight stage may be refilled once these MMAs are done
          }
          if (alive) mma_commit(&bars->a_empty[sa]);
        }
        if (alive) mma_commit(&bars->acc_full[buf]);
      }
      if (!alive || *abort_flag != 0) {
        // leaving early: tensor memory is freed at the common exit, so the MMAs issued so far have to be
        // complete by then (bounded wait on a commit of their own)
        mma_commit(&bars->mma_done);
        mbar_wait_bounded(&bars->mma_done, 0u, kWaitLimitNs);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------ weight loader
    if (lane == 0) {
      const unsigned stage_bytes = static_cast<unsigned>(a.n) * kSwizzleRowBytes;
      unsigned ib = 0;
      bool alive = true;
      for (int tile = first_tile; tile < a.n_tiles && alive; tile += tile_step) {
        for (int s = 0; s < a.k_blocks * kPieces; ++s, ++ib) {
          const unsigned sb = ib % kBStages;
          if (!mbar_wait_or_abort(&bars->b_empty[sb], ((ib / kBStages) & 1u) ^ 1u, abort_flag, kWaitLimitNs)) {
            give_up();
            alive = false;
            break;
          }
          mbar_expect_tx(&bars->b_full[sb], stage_bytes);
          bulk_g2s(smem + Smem::b_ring + sb * kBStageStride, a.packed + static_cast<size_t>(s) * stage_bytes, stage_bytes,
                   &bars->b_full[sb]);
        }
      }
      if (!alive || *abort_flag != 0) {
        // leaving early: wait (bounded) for the copies still in flight into this CTA's shared memory
        for (unsigned back = 1; back <= kBStages && back <= ib; ++back) {
          const unsigned use = ib - back;
          mbar_wait_bounded(&bars->b_full[use % kBStages], (use / kBStages) & 1u, kWaitLimitNs);
        }
      }
    }
  } else if (warp >= kEpilogueWarp0 && warp < kEpilogueWarp0 + kEpilogueWarps) {
    // ------------------------------------------------------------------------------ epilogue
    // Two warps per tensor-memory lane quarter; the pair splits the 32-column chunks by parity.
    const int quarter = warp & 3;                              // the tensor-memory lanes this warp may read
    const int parity = (warp - kEpilogueWarp0) >> 2;           // 0: even chunks, 1: odd chunks
    float* stage = reinterpret_cast<float*>(smem + Smem::staging) + (warp - kEpilogueWarp0) * 32 * kStagingRow;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int n_chunks = a.n / 32;
    unsigned it = 0;
    for (int tile = first_tile; tile < a.n_tiles; tile += tile_step, ++it) {
      const unsigned buf = it & 1u;
      bool ok = mbar_wait_or_abort(&bars->acc_full[buf], (it >> 1) & 1u, abort_flag, kWaitLimitNs);
      ok = __all_sync(kFull, ok);
      if (!ok) {
        if (lane == 0) give_up();
        break;
      }
      fence_after_thread_sync();
      const long long row0 = static_cast<long long>(tile) * kBlockM + quarter * 32;
      const uint32_t acc = tmem_base + lane_base + buf * static_cast<uint32_t>(a.n);
      for (int chunk = parity; chunk < n_chunks; chunk += 2) {
        float v[32];
        tmem_load_32x32(acc + chunk * 32, v);
        // row `lane` of the 32 x 32 block -> staging; the 16-byte chunk index is XORed with the row so
        // that both this write (one row per lane) and the read below (one row per 8 lanes) are conflict-free
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 bj = *reinterpret_cast<const float4*>(bias_s + chunk * 32 + j);
          *reinterpret_cast<float4*>(stage + lane * kStagingRow + (((j >> 2) ^ (lane & 7)) << 2)) =
              make_float4(v[j] + bj.x, v[j + 1] + bj.y, v[j + 2] + bj.z, v[j + 3] + bj.w);
        }
        __syncwarp();
        // staging -> global: each instruction stores four rows x 128 contiguous bytes
        float4 w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          w[i] = *reinterpret_cast<const float4*>(stage + (i * 4 + (lane >> 3)) * kStagingRow +
                                                  (((lane & 7) ^ ((i * 4 + (lane >> 3)) & 7)) << 2));
        __syncwarp();  // staging may be overwritten by the next chunk from here on
        float* dst = a.out + (row0 + (lane >> 3)) * a.n + chunk * 32 + (lane & 7) * 4;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (row0 + i * 4 + (lane >> 3) < a.rows)
            st_stream4(dst + static_cast<long long>(i) * 4 * a.n, w[i]);
        }
      }
      fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
    }
  } else if (warp >= kProducerWarp0) {
    // ----------------------------------------------------------------------------- producers
    const int pw = warp - kProducerWarp0;
    const int half = lane >> 4;   // which of the two rows this instruction covers
    const int c = lane & 15;      // float4 column inside the 64-feature block
    const uint64_t pol_stream = policy_evict_first();
    unsigned ia = 0;
    bool alive = true;
    for (int tile = first_tile; tile < a.n_tiles && alive; tile += tile_step) {
      for (int kb = 0; kb < a.k_blocks; ++kb, ++ia) {
        float v[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = pw * 16 + i * 2 + half;
          const long long g = static_cast<long long>(tile) * kBlockM + r;
          if (g < a.rows) {
            VecIO<4>::load(v[i], a.x + g * a.k + kb * kBlockK + c * 4, pol_stream);
          } else {
            v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
          }
        }
        const unsigned sa = ia % kAStages;
        bool ok = mbar_wait_or_abort(&bars->a_empty[sa], ((ia / kAStages) & 1u) ^ 1u, abort_flag, kWaitLimitNs);
        ok = __all_sync(kFull, ok);
        if (!ok) {
          if (lane == 0) give_up();
          alive = false;
          break;
        }
        unsigned char* stage = smem + Smem::a_ring + sa * kAStageBytes;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = pw * 16 + i * 2 + half;
          const Pieces2 p0 = split_pair(v[i][0], v[i][1]);
          const Pieces2 p1 = split_pair(v[i][2], v[i][3]);
          const uint32_t off = swizzled_offset(r, c * 4);
          *reinterpret_cast<uint2*>(stage + off) = make_uint2(p0.hi, p1.hi);
          *reinterpret_cast<uint2*>(stage + kAPieceBytes + off) = make_uint2(p0.mid, p1.mid);
          *reinterpret_cast<uint2*>(stage + 2 * kAPieceBytes + off) = make_uint2(p0.lo, p1.lo);
        }
        fence_proxy_async();  // the MMA reads shared memory through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->a_full[sa]);
      }
    }
  }

  // common exit: every thread of the CTA, whatever happened above
  fence_before_thread_sync();
  __syncthreads();
  if (warp == 0) {
    fence_after_thread_sync();
    tmem_dealloc(tmem_base, a.tmem_columns);
  }
}

inline size_t packed_bytes(int64_t k, int64_t n) {
  return static_cast<size_t>(k / kBlockK) * kPieces * static_cast<size_t>(n) * kSwizzleRowBytes;
}

// Also called by the fused aggregation + Linear kernel (asg_conv_fused.cu), which reads the same image.
int pack_weight_pieces(const float* weight, unsigned char* packed, int n, int k, cudaStream_t stream) {
  pack_weight<<<(n * k + 255) / 256, 256, 0, stream>>>(weight, packed, n, k);
  ASG_CUDA(cudaGetLastError());
  return ASG_OK;
}

}  // namespace linear_umma
}  // namespace asg

extern "C" size_t asg_linear_workspace_bytes(int64_t in_features, int64_t out_features) {
  if (in_features <= 0 || out_features <= 0) return 256;
  const int64_t k = (in_features + 63) / 64 * 64;
  return 256 + asg::linear_umma::packed_bytes(k, out_features);
}

extern "C" int asg_linear_supported(int64_t in_features, int64_t out_features) {
  return in_features > 0 && in_features % 64 == 0 && in_features <= 4096 && out_features >= 32 &&
                 out_features % 32 == 0 && out_features <= asg::linear_umma::kMaxN
             ? 1
             : 0;
}

extern "C" int asg_linear_bias_umma_ex(const float* x, const float* weight, const float* bias, float* out, int64_t rows,
                                       int64_t in_features, int64_t out_features, unsigned flags, void* workspace,
                                       size_t workspace_bytes, void* stream_ptr) {
  using namespace asg;
  using namespace asg::linear_umma;
  ASG_REQUIRE(rows >= 0, ASG_EINVAL, "rows must be non-negative");
  ASG_REQUIRE(rows <= 2147483647ll - kBlockM, ASG_ERANGE, "rows exceed the kernel index range");
  ASG_REQUIRE(asg_linear_supported(in_features, out_features) == 1, ASG_EINVAL,
              "asg_linear_bias_umma takes in_features in multiples of 64 and out_features in multiples of 32 up to 256");
  if (rows == 0) return ASG_OK;
  ASG_REQUIRE(x != nullptr && weight != nullptr && out != nullptr, ASG_EINVAL, "x, weight and out must not be null");
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out);
  ASG_REQUIRE((bits & 15) == 0, ASG_EINVAL, "x and out must be 16-byte aligned");
  ASG_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0, ASG_EWORKSPACE,
              "workspace must be a 256-byte aligned device pointer");
  ASG_REQUIRE(workspace_bytes >= asg_linear_workspace_bytes(in_features, out_features), ASG_EWORKSPACE,
              "workspace smaller than asg_linear_workspace_bytes(in_features, out_features)");
  DeviceGuard guard(out);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);

  Header* header = static_cast<Header*>(workspace);
  unsigned char* packed = static_cast<unsigned char*>(workspace) + 256;
  ASG_CUDA(cudaMemsetAsync(&header->status, 0, sizeof(int), stream));
  const int n = static_cast<int>(out_features), k = static_cast<int>(in_features);
  if (int rc = pack_weight_pieces(weight, packed, n, k, stream)) return rc;

  Args args;
  args.x = x;
  args.bias = bias;
  args.out = out;
  args.packed = packed;
  args.status = &header->status;
  args.rows = static_cast<int>(rows);
  args.k = k;
  args.n = n;
  args.k_blocks = k / kBlockK;
  args.n_tiles = static_cast<int>((rows + kBlockM - 1) / kBlockM);
  unsigned columns = 32;
  while (columns < 2u * static_cast<unsigned>(n)) columns <<= 1;  // two accumulators, a power of two >= 32
  args.tmem_columns = columns;
  args.selftest_stall = (flags & ASG_FLAG_SELFTEST_STALL) ? 1 : 0;
  ASG_CUDA(cudaFuncSetAttribute(linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynamicSmem));
  const int sms = sm_count(guard.target);
  const int grid = args.n_tiles < sms ? args.n_tiles : sms;
  linear_kernel<<<grid, kThreads, kDynamicSmem, stream>>>(args);
  ASG_CUDA(cudaGetLastError());
  return ASG_OK;
}

extern "C" int asg_linear_bias_umma(const float* x, const float* weight, const float* bias, float* out, int64_t rows,
                                    int64_t in_features, int64_t out_features, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  return asg_linear_bias_umma_ex(x, weight, bias, out, rows, in_features, out_features, 0u, workspace, workspace_bytes,
                                 stream);
}
