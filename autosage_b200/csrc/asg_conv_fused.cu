// Aggregation and Linear of the layer in one kernel (autosage/conv.py:54-55: aggregated =
// spmm_csr(crow, col, val, x); out = linear(aggregated)): the aggregated rows never reach global
// memory.  Hand-written for sm_100a.
//
// Two launches.  The first is the CTA-per-hub path of the SpMM kernel restricted to hub rows
// (degree >= hub_threshold: too long for one warp), writing their sums to a compact side buffer.  The
// second is this file's kernel: one persistent CTA per SM walks tiles of 128 consecutive rows.  Warp roles:
//   warp 0        allocates tensor memory; its lane 0 issues every MMA and commit
//   warp 1        lane 0 streams the weight pieces (split once into three bfloat16 pieces and stored in
//                 the 128-byte-swizzled K-major image the MMA reads) through a 2-stage ring of 16 KB
//                 with 1-D bulk async copies, half of the output columns per stage
//   warps 2-5     epilogue, one warp per tensor-memory lane quarter: accumulator -> registers
//                 (tcgen05.ld) -> + bias -> 128 contiguous bytes of an output row per lane and chunk
//   warps 6-23    gather warps.  They take groups of four consecutive rows from a CTA-wide counter (one
//                 group ahead, so the row pointers of the next group are in flight).  The edges of
//                 consecutive rows below the threshold are one contiguous stream of the col array: the
//                 warp reads 32 columns per lane-coalesced load (the next 32, or the head of the next
//                 group, prefetched) and gathers X rows six at a time, one 128-bit load per lane and edge,
//                 so batches stay full across row boundaries; a row whose last edge has passed is split
//                 into three bfloat16 pieces, stored into the tile's operand buffer in shared memory, and
//                 announced by one arrival on the tile's barrier.  Hub rows are read from the side buffer.
// The operand buffer is double-buffered (2 x 96 KB at 128 input features), so warps run ahead into the
// next tile while the slowest row of this one finishes, and the accumulator is double-buffered in tensor
// memory (2 x out_features columns).  The float32 accuracy comes from the six piece products of
// asg_linear_umma.cu.  Every wait is on an mbarrier, bounded in time; a wait that gives up sets a status
// word and a CTA-wide abort flag, the loader waits for its copies in flight, and the CTA leaves through
// the common exit, which frees its tensor memory.
//
// Measured on the 2.45 M-row, 123 M-edge power-law graph (128 -> 256 features): 10.95 ms at
// hub_threshold 64 against 9.8-10.0 ms for the SpMM kernels followed by asg_linear_bias_umma, so the
// layer keeps the two-kernel path by default.  One CTA per SM (the operand buffers fill shared memory)
// caps the gather at 18 warps x 6 loads in flight, where the stand-alone SpMM kernels keep 16-32 warps
// x 8 edges in flight with nothing else resident; the gather here is latency-bound (45 % of DRAM
// bandwidth, 72 % of stall cycles on the scoreboard of global loads), and what fusion saves - 2.5 GB of
// the 69 GB the layer moves - is less than that loss.
#include "asg_umma.cuh"
#include "asg_tile.cuh"

namespace asg {
namespace conv_fused {

using namespace umma;

constexpr int kBlockM = 128;
constexpr int kPieces = 3;
constexpr int kEpilogueWarp0 = 2;   // four warps, one per tensor-memory lane quarter (warp index mod 4)
constexpr int kEpilogueWarps = 4;
constexpr int kGatherWarp0 = kEpilogueWarp0 + kEpilogueWarps;
// 18 gather warps with 6 loads in flight each measured best of (26, 4), (18, 6), (18, 8), (14, 12), (10, 16):
// the register file (64 K registers, one CTA per SM) bounds warps x loads in flight.
constexpr int kGatherWarps = 18;
constexpr int kThreads = (kGatherWarp0 + kGatherWarps) * 32;
constexpr int kLoadsInFlight = 6;
constexpr int kGroupRows = 4;                      // consecutive rows a warp takes per grab
constexpr int kGroupsPerTile = kBlockM / kGroupRows;
constexpr int kMaxN = 256;
constexpr int kMaxKBlocks = 2;                     // 128 input features
constexpr int kAPieceBytes = kBlockM * kSwizzleRowBytes;              // 16 KB: 128 rows x 64 bf16
constexpr int kABufferBytes = kMaxKBlocks * kPieces * kAPieceBytes;   // 96 KB
constexpr int kBStages = 2;
constexpr int kBStageBytes = (kMaxN / 2) * kSwizzleRowBytes;          // 16 KB: half of the output columns
constexpr unsigned long long kWaitLimitNs = 500ull * 1000ull * 1000ull;
constexpr int kStatusWaitExpired = 3;
constexpr unsigned long long kSelftestLimitNs = 20ull * 1000ull * 1000ull;   // the self-test's wait gives up after 20 ms

struct Smem {
  static constexpr int a_buffers = 0;
  static constexpr int b_ring = a_buffers + 2 * kABufferBytes;
  static constexpr int bias = b_ring + kBStages * kBStageBytes;
  static constexpr int barriers = bias + kMaxN * 4;
  static constexpr int total = barriers + 256;
};
constexpr int kDynamicSmem = Smem::total + 1024;  // slack to align the carve-up to 1024 bytes
static_assert(kDynamicSmem <= 232448, "exceeds the 227 KB a CTA may use");

struct Barriers {
  uint64_t a_full[2], a_empty[2];
  uint64_t b_full[kBStages], b_empty[kBStages];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t mma_done;   // the MMA thread's last commit when it leaves early
  uint64_t idle;       // self-test: nothing ever arrives here
  uint32_t tmem_base;
  int abort;
  int next_group;
};
static_assert(sizeof(Barriers) <= 256, "barrier block must fit its slot");

struct Args {
  const int64_t* crow;
  const int64_t* col;
  const float* val;
  const float* x;
  const float* hub_y;      // [hub item][k]: sums of the hub rows
  const int* hub_slot;     // row -> hub item (defined for hub rows only)
  const float* bias;
  float* out;
  const unsigned char* packed;  // weight pieces in the shared-memory image (asg_linear_umma.cu: pack_weight)
  int* status;
  long long hub_threshold;
  int rows, k, n;
  int n_tiles;
  unsigned tmem_columns;
  int selftest_stall;  // ASG_FLAG_SELFTEST_STALL: the MMA thread waits, before its second tile, on a barrier nothing arrives on
};

// VW floats of a dense row per lane: a 64-bit or a 128-bit load.
template <int VW>
struct VecRow;
template <>
struct VecRow<4> {
  static __device__ __forceinline__ void load(float (&d)[4], const float* p, uint64_t pol) { VecIO<4>::load(d, p, pol); }
  static __device__ __forceinline__ void load_plain(float (&d)[4], const float* p) { VecIO<4>::load_plain(d, p); }
};
template <>
struct VecRow<2> {
  static __device__ __forceinline__ void load(float (&d)[2], const float* p, uint64_t pol) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v2.f32 {%0,%1}, [%2], %3;"
                 : "=f"(d[0]), "=f"(d[1])
                 : "l"(p), "l"(pol));
  }
  static __device__ __forceinline__ void load_plain(float (&d)[2], const float* p) {
    const float2 t = *reinterpret_cast<const float2*>(p);
    d[0] = t.x;
    d[1] = t.y;
  }
};

template <int KB, bool HAS_VAL>
__global__ void __launch_bounds__(kThreads, 1) conv_fused_kernel(const Args a) {
  constexpr int U = kLoadsInFlight;    // gathered rows in flight per warp
  constexpr int VW = 2 * KB;           // floats per lane and load: a warp covers one row of 64 * KB features
  constexpr int F = 64 * KB;

  extern __shared__ unsigned char raw_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + Smem::barriers);
  float* bias_s = reinterpret_cast<float*>(smem + Smem::bias);
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile int* abort_flag = &bars->abort;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->a_full[i], kBlockM);   // one arrival per finished row
      mbar_init(&bars->a_empty[i], 1);
      mbar_init(&bars->acc_full[i], 1);
      mbar_init(&bars->acc_empty[i], kEpilogueWarps);
    }
    for (int i = 0; i < kBStages; ++i) {
      mbar_init(&bars->b_full[i], 1);
      mbar_init(&bars->b_empty[i], 1);
    }
    mbar_init(&bars->mma_done, 1);
    mbar_init(&bars->idle, 1);
    bars->abort = 0;
    bars->next_group = 0;
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
  const int first_tile = blockIdx.x;
  const int tile_step = gridDim.x;
  const int my_tiles = first_tile < a.n_tiles ? (a.n_tiles - first_tile + tile_step - 1) / tile_step : 0;
  const int half_n = a.n / 2;
  const unsigned half_bytes = static_cast<unsigned>(half_n) * kSwizzleRowBytes;

  auto give_up = [&]() {
    atomicCAS(a.status, 0, kStatusWaitExpired);
    bars->abort = 1;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = instruction_descriptor(kBlockM, half_n);
      const uint32_t a_base = smem_u32(smem + Smem::a_buffers);
      const uint32_t b_base = smem_u32(smem + Smem::b_ring);
      unsigned ib = 0;
      bool alive = true;
      for (int j = 0; j < my_tiles && alive; ++j) {
        const unsigned buf = j & 1u;
        if (a.selftest_stall && j == 1 && !mbar_wait_or_abort(&bars->idle, 0u, abort_flag, kSelftestLimitNs)) {
          give_up();
          alive = false;
          break;
        }
        if (!mbar_wait_or_abort(&bars->acc_empty[buf], ((j >> 1) & 1u) ^ 1u, abort_flag, kWaitLimitNs) ||
            !mbar_wait_or_abort(&bars->a_full[buf], (j >> 1) & 1u, abort_flag, kWaitLimitNs)) {
          give_up();
          alive = false;
          break;
        }
        fence_after_thread_sync();
        const uint32_t acc = tmem_base + buf * static_cast<uint32_t>(a.n);
        // weight piece p (0 = lo, 1 = mid, 2 = hi) meets the row pieces that keep the product above 2^-24:
        // lo x hi; mid x {mid, hi}; hi x {lo, mid, hi}.  Row piece index: 0 = hi, 1 = mid, 2 = lo.
        for (int kb = 0; kb < KB && alive; ++kb) {
          for (int p = 0; p < kPieces && alive; ++p) {
            for (int h = 0; h < 2; ++h, ++ib) {
              const unsigned sb = ib % kBStages;
              if (!mbar_wait_or_abort(&bars->b_full[sb], (ib / kBStages) & 1u, abort_flag, kWaitLimitNs)) {
                give_up();
                alive = false;
                break;
              }
              fence_after_thread_sync();
              const uint32_t b_stage = b_base + sb * kBStageBytes;
              uint32_t accumulate = (kb > 0 || p > 0) ? 1u : 0u;
              for (int xp = p; xp >= 0; --xp) {  // smallest row piece first
                const uint32_t a_piece = a_base + buf * kABufferBytes + (kb * kPieces + xp) * kAPieceBytes;
#pragma unroll
                for (int kk = 0; kk < kBlockK / kInstrK; ++kk) {
                  mma_bf16(acc + h * half_n, smem_descriptor(a_piece + kk * kInstrK * 2),
                           smem_descriptor(b_stage + kk * kInstrK * 2), idesc, accumulate);
                  accumulate = 1;
                }
              }
              mma_commit(&bars->b_empty[sb]);  // the weight stage may be refilled once these MMAs are done
            }
          }
        }
        if (alive) {
          mma_commit(&bars->a_empty[buf]);
          mma_commit(&bars->acc_full[buf]);
        }
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
      const size_t piece_bytes = static_cast<size_t>(a.n) * kSwizzleRowBytes;
      unsigned ib = 0;
      bool alive = true;
      for (int j = 0; j < my_tiles && alive; ++j) {
        for (int s = 0; s < KB * kPieces && alive; ++s) {
          for (int h = 0; h < 2; ++h, ++ib) {
            const unsigned sb = ib % kBStages;
            if (!mbar_wait_or_abort(&bars->b_empty[sb], ((ib / kBStages) & 1u) ^ 1u, abort_flag, kWaitLimitNs)) {
              give_up();
              alive = false;
              break;
            }
            mbar_expect_tx(&bars->b_full[sb], half_bytes);
            bulk_g2s(smem + Smem::b_ring + sb * kBStageBytes, a.packed + s * piece_bytes + static_cast<size_t>(h) * half_bytes,
                     half_bytes, &bars->b_full[sb]);
          }
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
  } else if (warp < kGatherWarp0) {
    // ------------------------------------------------------------------------------ epilogue
    // One warp per tensor-memory lane quarter: tensor memory -> + bias -> global, 128 contiguous bytes
    // of an output row per lane and 32-column chunk.
    const int quarter = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int n_chunks = a.n / 32;
    for (int j = 0; j < my_tiles; ++j) {
      const unsigned buf = j & 1u;
      bool ok = mbar_wait_or_abort(&bars->acc_full[buf], (j >> 1) & 1u, abort_flag, kWaitLimitNs);
      ok = __all_sync(kFull, ok);
      if (!ok) {
        if (lane == 0) give_up();
        break;
      }
      fence_after_thread_sync();
      const long long row = static_cast<long long>(first_tile + j * tile_step) * kBlockM + quarter * 32 + lane;
      const uint32_t acc_at = tmem_base + lane_base + buf * static_cast<uint32_t>(a.n);
      for (int chunk = 0; chunk < n_chunks; ++chunk) {
        float v[32];
        tmem_load_32x32(acc_at + chunk * 32, v);
        if (row < a.rows) {
          float* dst = a.out + row * a.n + chunk * 32;
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 bj = *reinterpret_cast<const float4*>(bias_s + chunk * 32 + c);
            st_stream4(dst + c, make_float4(v[c] + bj.x, v[c + 1] + bj.y, v[c + 2] + bj.z, v[c + 3] + bj.w));
          }
        }
      }
      fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
    }
  } else {
    // ------------------------------------------------------------------------------ gather warps
    const uint64_t pol_keep = policy_evict_last();
    const float* x_lane = a.x + VW * lane;    // the features of a row this lane owns
    bool alive = true;

    // Groups of kGroupRows consecutive rows are taken from the CTA-wide counter, one group ahead of the
    // one being processed.  `raw` holds crow[first row of the group + lane] for lanes 0 .. kGroupRows.
    auto grab_group = [&](int& group, long long& raw) {
      int g = 0;
      if (lane == 0) g = atomicAdd(&bars->next_group, 1);
      g = __shfl_sync(kFull, g, 0);
      group = g;
      raw = 0;
      const int j = g / kGroupsPerTile;
      if (j < my_tiles && lane <= kGroupRows) {
        long long r = static_cast<long long>(first_tile + j * tile_step) * kBlockM + (g % kGroupsPerTile) * kGroupRows + lane;
        if (r > a.rows) r = a.rows;   // rows past the end of the matrix are empty
        raw = a.crow[r];
      }
    };
    int group_now, group_next;
    long long raw_now, raw_next;
    grab_group(group_now, raw_now);
    grab_group(group_next, raw_next);

    int c_next = 0;
    float w_next = 0.f;
    int head_group = -1;       // the group whose first 32 columns c_next / w_next hold (prefetched)
    int held_j = -1;           // the tile whose operand buffer this warp may write
    const int threshold = a.hub_threshold > 0x7fffffffll ? 0x7fffffff : static_cast<int>(a.hub_threshold);

    while (alive) {
      const int j_now = group_now / kGroupsPerTile;
      if (j_now >= my_tiles) break;
      if (j_now != held_j) {
        // first group of a new tile: its buffer is free once the MMAs of the tile two before it are done
        bool ok = mbar_wait_or_abort(&bars->a_empty[j_now & 1], ((j_now >> 1) & 1u) ^ 1u, abort_flag, kWaitLimitNs);
        ok = __all_sync(kFull, ok);
        if (!ok) {
          if (lane == 0) give_up();
          alive = false;
          break;
        }
        held_j = j_now;
      }
      // positions inside the group's contiguous edge range, relative to its first edge
      const long long base = __shfl_sync(kFull, raw_now, 0);
      const int off = static_cast<int>(raw_now - base);   // lanes 0 .. kGroupRows: where row `lane` starts
      const int64_t* col_at = a.col + base;
      const float* val_at = HAS_VAL ? a.val + base : nullptr;
      const int row0 = (group_now % kGroupsPerTile) * kGroupRows;   // first row of the group inside the tile

      float acc[VW];
#pragma unroll
      for (int i = 0; i < VW; ++i) acc[i] = 0.f;
      // the finished row `r` of the group: split the sum, store the pieces, announce the row
      auto flush = [&](int r) {
        // features VW lane .. VW lane + VW - 1 of the row: VW bfloat16 of each piece
        unsigned char* block = smem + Smem::a_buffers + (j_now & 1) * kABufferBytes +
                               ((VW * lane) >> 6) * kPieces * kAPieceBytes +
                               swizzled_offset(static_cast<uint32_t>(row0 + r), static_cast<uint32_t>((VW * lane) & 63));
        const Pieces2 p0 = split_pair(acc[0], acc[1]);
        if (VW == 4) {
          const Pieces2 p1 = split_pair(acc[VW - 2], acc[VW - 1]);
          *reinterpret_cast<uint2*>(block) = make_uint2(p0.hi, p1.hi);
          *reinterpret_cast<uint2*>(block + kAPieceBytes) = make_uint2(p0.mid, p1.mid);
          *reinterpret_cast<uint2*>(block + 2 * kAPieceBytes) = make_uint2(p0.lo, p1.lo);
        } else {
          *reinterpret_cast<uint32_t*>(block) = p0.hi;
          *reinterpret_cast<uint32_t*>(block + kAPieceBytes) = p0.mid;
          *reinterpret_cast<uint32_t*>(block + 2 * kAPieceBytes) = p0.lo;
        }
        fence_proxy_async();  // the MMA reads shared memory through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->a_full[j_now & 1]);
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[i] = 0.f;
      };
      auto fetch_columns = [&](int at, int end) {
        if (at + lane < end) {
          c_next = static_cast<int>(__ldg(col_at + at + lane));
          if (HAS_VAL) w_next = __ldg(val_at + at + lane);
        }
      };

      int i = 0;
      while (i < kGroupRows) {
        const int s_i = __shfl_sync(kFull, off, i);
        int e_cur = __shfl_sync(kFull, off, i + 1);
        if (e_cur - s_i >= threshold) {
          // a hub row: its sum was computed by the first launch
          const long long g_row = static_cast<long long>(first_tile + j_now * tile_step) * kBlockM + row0 + i;
          VecRow<VW>::load_plain(acc, a.hub_y + static_cast<size_t>(a.hub_slot[g_row]) * F + VW * lane);
          flush(i);
          ++i;
          continue;
        }
        // a run of rows below the hub threshold: their edges are one contiguous stream [s_i, seg_e)
        int i_end = i + 1;
        int seg_e = e_cur;
        while (i_end < kGroupRows) {
          const int e_more = __shfl_sync(kFull, off, i_end + 1);
          if (e_more - seg_e >= threshold) break;
          seg_e = e_more;
          ++i_end;
        }
        int cur = i;  // the row the stream position belongs to; e_cur = where its edges end
        if (s_i < seg_e && !(head_group == group_now && s_i == 0)) fetch_columns(s_i, seg_e);
        head_group = -1;
        for (int p = s_i; p < seg_e; p += 32) {
          const int c_l = c_next;
          const float w_l = w_next;
          const int cnt = seg_e - p < 32 ? seg_e - p : 32;
          if (p + 32 < seg_e) {
            fetch_columns(p + 32, seg_e);
          } else if (i_end == kGroupRows && group_next / kGroupsPerTile < my_tiles) {
            // the last chunk of the group: the first columns of the next group
            const long long first = __shfl_sync(kFull, raw_next, 0);
            const long long last = __shfl_sync(kFull, raw_next, kGroupRows);
            if (first + lane < last) {
              c_next = static_cast<int>(__ldg(a.col + first + lane));
              if (HAS_VAL) w_next = __ldg(a.val + first + lane);
            }
            head_group = group_next;
          }
#pragma unroll 1
          for (int j = 0; j < cnt; j += U) {
            float xv[U][VW];
            float wu[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int c = __shfl_sync(kFull, c_l, (j + u) & 31);
              if (HAS_VAL) wu[u] = __shfl_sync(kFull, w_l, (j + u) & 31);
              if (j + u < cnt) {
                VecRow<VW>::load(xv[u], x_lane + static_cast<long long>(c) * F, pol_keep);
              } else {
                if (HAS_VAL) wu[u] = 0.f;
#pragma unroll
                for (int k = 0; k < VW; ++k) xv[u][k] = 0.f;
              }
            }
            // the batch holds edges [first, first + valid) of the stream; rows may end inside it
            const int first = p + j;
            const int valid = cnt - j < U ? cnt - j : U;
            int lo = 0;
            for (;;) {
              int hi = cur == i_end - 1 ? valid : e_cur - first;   // edges of the batch that belong to row `cur`
              hi = hi > valid ? valid : hi;
#pragma unroll
              for (int u = 0; u < U; ++u) {
                if (u >= lo && u < hi) {
#pragma unroll
                  for (int k = 0; k < VW; ++k) acc[k] = HAS_VAL ? fmaf(wu[u], xv[u][k], acc[k]) : acc[k] + xv[u][k];
                }
              }
              if (hi >= valid) break;
              flush(cur);   // the row's last edge has passed
              ++cur;
              e_cur = __shfl_sync(kFull, off, cur + 1);
              lo = hi > lo ? hi : lo;
            }
          }
        }
        // the rows of the run still open: the last one with edges, and empty rows after it
        while (cur < i_end) {
          flush(cur);
          ++cur;
        }
        i = i_end;
      }
      group_now = group_next;
      raw_now = raw_next;
      grab_group(group_next, raw_next);
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

constexpr int kPackedHeader = 256;  // the workspace starts with a Header (status word)

inline size_t packed_bytes(int64_t k, int64_t n) {
  return static_cast<size_t>(k / kBlockK) * kPieces * static_cast<size_t>(n) * kSwizzleRowBytes;
}
inline int64_t hub_capacity(int64_t n_rows, int64_t nnz, int64_t hub_threshold) {
  const int64_t by_edges = hub_threshold > 0 ? nnz / hub_threshold : n_rows;
  return by_edges < n_rows ? by_edges : n_rows;
}
struct Layout {
  size_t packed, slot, hub_y, total;
};
inline Layout layout(int64_t n_rows, int64_t nnz, int64_t k, int64_t n, int64_t hub_threshold) {
  Layout at;
  at.packed = kPackedHeader;
  at.slot = align256(at.packed + packed_bytes(k, n));
  at.hub_y = align256(at.slot + size_t(4) * static_cast<size_t>(n_rows));
  at.total = align256(at.hub_y + size_t(4) * static_cast<size_t>(k) * static_cast<size_t>(hub_capacity(n_rows, nnz, hub_threshold)));
  return at;
}

}  // namespace conv_fused

namespace linear_umma {
// defined in asg_linear_umma.cu: splits the weight and stores the pieces in the MMA's shared-memory image
int pack_weight_pieces(const float* weight, unsigned char* packed, int n, int k, cudaStream_t stream);
}  // namespace linear_umma

}  // namespace asg

extern "C" int asg_conv_fused_supported(int64_t in_features, int64_t out_features) {
  return (in_features == 64 || in_features == 128) && out_features >= 32 && out_features % 32 == 0 &&
                 out_features <= asg::conv_fused::kMaxN
             ? 1
             : 0;
}

extern "C" size_t asg_conv_fused_workspace_bytes(int64_t n_rows, int64_t nnz, int64_t in_features, int64_t out_features,
                                                 int64_t hub_threshold) {
  if (n_rows < 0 || nnz < 0 || in_features <= 0 || out_features <= 0 || hub_threshold <= 0) return 256;
  return asg::conv_fused::layout(n_rows, nnz, (in_features + 63) / 64 * 64, out_features, hub_threshold).total;
}

extern "C" int asg_conv_fused(const int64_t* crow, const int64_t* col, const float* val, const float* x,
                              const float* weight, const float* bias, float* out, int64_t n_rows, int64_t nnz,
                              int64_t in_features, int64_t out_features, int64_t hub_threshold, int hub_warps,
                              unsigned flags, void* plan_workspace, size_t plan_workspace_bytes, void* workspace,
                              size_t workspace_bytes, void* stream_ptr) {
  using namespace asg;
  using namespace asg::conv_fused;
  ASG_REQUIRE(n_rows >= 0 && nnz >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(n_rows <= 2147483647ll - 2048, ASG_ERANGE, "n_rows exceeds the kernel index range");
  ASG_REQUIRE(asg_conv_fused_supported(in_features, out_features) == 1, ASG_EINVAL,
              "asg_conv_fused takes 64 or 128 input features and output features in multiples of 32 up to 256");
  ASG_REQUIRE(hub_threshold >= 32, ASG_EINVAL, "hub_threshold must be at least 32");
  ASG_REQUIRE(hub_warps == 2 || hub_warps == 4 || hub_warps == 8 || hub_warps == 16, ASG_EINVAL,
              "hub_warps must be 2, 4, 8 or 16");
  if (n_rows == 0) return ASG_OK;
  ASG_REQUIRE(crow != nullptr && x != nullptr && weight != nullptr && out != nullptr, ASG_EINVAL,
              "crow, x, weight and out must not be null");
  ASG_REQUIRE(nnz == 0 || col != nullptr, ASG_EINVAL, "col must not be null");
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out);
  ASG_REQUIRE((bits & 31) == 0, ASG_EINVAL, "x and out must be 32-byte aligned");
  ASG_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0, ASG_EWORKSPACE,
              "workspace must be a 256-byte aligned device pointer");
  const Layout at = layout(n_rows, nnz, in_features, out_features, hub_threshold);
  ASG_REQUIRE(workspace_bytes >= at.total, ASG_EWORKSPACE,
              "workspace smaller than asg_conv_fused_workspace_bytes(n_rows, nnz, in_features, out_features, hub_threshold)");
  DeviceGuard guard(out);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);

  unsigned char* base = static_cast<unsigned char*>(workspace);
  Header* header = static_cast<Header*>(workspace);
  int* hub_slot = reinterpret_cast<int*>(base + at.slot);
  float* hub_y = reinterpret_cast<float*>(base + at.hub_y);
  ASG_CUDA(cudaMemsetAsync(&header->status, 0, sizeof(int), stream));
  const int n = static_cast<int>(out_features), k = static_cast<int>(in_features);
  if (int rc = linear_umma::pack_weight_pieces(weight, base + at.packed, n, k, stream)) return rc;

  // first launch: the hub rows, compactly
  if (int rc = spmm_hub_rows_compact(crow, col, val, x, hub_y, hub_slot, n_rows, nnz, in_features, k, hub_warps,
                                     hub_threshold, flags & (ASG_FLAG_PLAN_READY | ASG_FLAG_NO_BULK_STAGE),
                                     plan_workspace, plan_workspace_bytes, stream))
    return rc;

  Args args;
  args.crow = crow;
  args.col = col;
  args.val = val;
  args.x = x;
  args.hub_y = hub_y;
  args.hub_slot = hub_slot;
  args.bias = bias;
  args.out = out;
  args.packed = base + at.packed;
  args.status = &header->status;
  args.hub_threshold = hub_threshold;
  args.rows = static_cast<int>(n_rows);
  args.k = k;
  args.n = n;
  args.n_tiles = static_cast<int>((n_rows + kBlockM - 1) / kBlockM);
  unsigned columns = 32;
  while (columns < 2u * static_cast<unsigned>(n)) columns <<= 1;  // two accumulators, a power of two >= 32
  args.tmem_columns = columns;
  args.selftest_stall = (flags & ASG_FLAG_SELFTEST_STALL) ? 1 : 0;
  const int sms = sm_count(guard.target);
  const int grid = args.n_tiles < sms ? args.n_tiles : sms;
  auto launch = [&](auto kernel) -> int {
    ASG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynamicSmem));
    kernel<<<grid, kThreads, kDynamicSmem, stream>>>(args);
    ASG_CUDA(cudaGetLastError());
    return ASG_OK;
  };
  if (k == 128) return val != nullptr ? launch(conv_fused_kernel<2, true>) : launch(conv_fused_kernel<2, false>);
  return val != nullptr ? launch(conv_fused_kernel<1, true>) : launch(conv_fused_kernel<1, false>);
}
