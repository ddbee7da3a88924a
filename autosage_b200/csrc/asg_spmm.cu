// CSR SpMM for sm_100a: persistent kernels that drain three work queues built by the plan: the main
// kernel takes queues 0 and 1 below, a second small kernel takes queue 2 (light rows of fewer than
// 32 edges, 32 rows per grab; see spmm_short_rows).
//
//   queue 0  hub rows (degree >= threshold): one CTA per (hub row, feature tile).  The row's
//            col/val segment is staged into shared memory in chunks by 1-D bulk async copies (TMA
//            without a tensor map, mbarrier completion, two stages); every warp of the CTA then
//            gathers rows of X for its share of the chunk and the per-warp partial sums are
//            combined through shared memory.
//   queue 1  light rows: one warp per (row, feature tile).  col/val are fetched 32 edges at a time
//            with one coalesced load per lane and broadcast by shuffles; X rows are gathered with
//            scalar, 128-bit or 256-bit loads, U load instructions in flight per lane.
//
// Items are ordered tile-major (all rows for tile 0, then tile 1, ...) so that, when X is larger
// than L2, the part of X being gathered at any time is N x FT floats only.
//
// Replaces csrc/spmm_csr_vec4.cu:23-89 (scalar and vec4 warp-per-row kernels),
// csrc/spmm_rows.cu:11-81 (row-list kernel) and csrc/spmm_hub.cu:13-93 (CTA-per-hub kernel) of the
// reference.  Offsets into X and Y are 64-bit (the reference multiplies 32-bit ints).
#include "asg_tile.cuh"

namespace asg {

struct SpmmArgs {
  const int64_t* crow;
  const int64_t* col;
  const float* val;
  const float* x;
  float* y;
  Header* header;
  const int* order;
  int f;
  int n_tiles;      // feature tiles this launch covers
  int tile_begin;   // index of the first of them (0 unless a feature range was requested)
  int accumulate;
  int bulk_stage;
  int pack_short;  // queue 2 in the packed form (one row per lane group)
  int selftest_stall;  // ASG_FLAG_SELFTEST_STALL: hub staging announces 16 bytes that never arrive
  unsigned long long wait_limit_ns;
  // Hub rows only, written compactly (the first pass of the fused aggregation + Linear kernel): the sum
  // of hub item i goes to y + i * f instead of y + row * f, and hub_slot[row] = i tells the second pass
  // where to find it.  Queues 1 and 2 are not touched.
  int hubs_only;
  int* hub_slot;
  int streaming;  // host side: X is much larger than L2, the gathers stream from HBM
};

constexpr int kChunkPerWarp = 128;  // staged edges per warp and stage in the hub path

// Queue 2: light rows of fewer than 32 edges, taken 32 rows per grab.  Rows that short are
// latency-bound when taken one at a time (queue grab, row id, two row pointers, columns, X rows,
// output: five dependent memory round trips for a handful of edges).  Here a warp reads the ids
// and pointers of 32 rows with one coalesced load each and walks them with the next row's columns
// already in flight.  It runs as a kernel of its own so that its registers and schedule do not disturb
// the long-row loops (inlined into the main kernel it cost the long-row workloads about 10 %), launched
// right after the main kernel as a programmatic dependent: it starts filling SMs as the main kernel's
// CTAs retire instead of waiting for its last hub row.
template <int VW, int G, int NV, int U_REQUESTED, bool HAS_VAL, bool EXTRAS>
__device__ __forceinline__ void spmm_short_rows(const SpmmArgs& a, int n_hub, int n_medium, int n_short) {
  constexpr int U = U_REQUESTED < G ? U_REQUESTED : G;
  constexpr int EPI = 32 / G;
  constexpr int FT = VW * G * NV;
  constexpr int BU = EPI * U;
  const int lane = threadIdx.x & 31;
  const int l = lane % G;
  const int sub = lane / G;
  const int f = a.f;
  const uint64_t pol_keep = policy_evict_last();
  const uint64_t pol_stream = policy_evict_first();
  if (n_short > 0) {
    const int* shorts = a.order + n_hub + n_medium;
    const int n_batches = (n_short + 31) / 32;
    const long long total = static_cast<long long>(n_batches) * a.n_tiles;
    for (;;) {
      const unsigned long long it = warp_next(&a.header->counter[2]);
      if (it >= static_cast<unsigned long long>(total)) break;
      const int tile = static_cast<int>(it / n_batches);
      const int first = static_cast<int>(it - static_cast<unsigned long long>(tile) * n_batches) * 32;
      const int n_here = n_short - first < 32 ? n_short - first : 32;
      const int fbase = (a.tile_begin + tile) * FT;
      int row_l = 0;
      long long s_l = 0, e_l = 0;
      if (lane < n_here) {
        row_l = shorts[first + lane];
        s_l = a.crow[row_l];
        e_l = a.crow[row_l + 1];
      }
      bool fvalid[NV];
      int foff[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        foff[v] = fbase + VW * (l + G * v);
        fvalid[v] = foff[v] < f;
      }
      // columns / weights of row 0 of the batch
      long long s_cur = __shfl_sync(kFull, s_l, 0);
      int cnt_cur = static_cast<int>(__shfl_sync(kFull, e_l, 0) - s_cur);
      int c_next = 0;
      float w_next = 0.f;
      if (lane < cnt_cur) {
        c_next = static_cast<int>(ld_index(a.col + s_cur + lane, pol_stream));
        if (HAS_VAL) w_next = ld_weight(a.val + s_cur + lane, pol_stream);
      }
      for (int r = 0; r < n_here; ++r) {
        const int row = __shfl_sync(kFull, row_l, r);
        const int cnt = cnt_cur;
        const int c_l = c_next;
        const float w_l = w_next;
        if (r + 1 < n_here) {  // next row's columns while this row's X rows are gathered
          s_cur = __shfl_sync(kFull, s_l, r + 1);
          cnt_cur = static_cast<int>(__shfl_sync(kFull, e_l, r + 1) - s_cur);
          if (lane < cnt_cur) {
            c_next = static_cast<int>(ld_index(a.col + s_cur + lane, pol_stream));
            if (HAS_VAL) w_next = ld_weight(a.val + s_cur + lane, pol_stream);
          }
        }
        if (cnt == 0 && (EXTRAS && a.accumulate)) continue;  // y += 0
        // Accumulating (column blocks of the sharded path): the lanes that will store start from the
        // row's current output, fetched before the gathers so that its latency hides behind them.
        float acc[NV][VW];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          if ((EXTRAS && a.accumulate) && sub == 0 && fvalid[v]) {
            VecIO<VW>::load_plain(acc[v], a.y + static_cast<size_t>(row) * f + foff[v]);
          } else {
#pragma unroll
            for (int i = 0; i < VW; ++i) acc[v][i] = 0.f;
          }
        }
        // whole batches of edges inside a full feature tile need no predicates or zero fill; only the
        // row's last, partly filled batch goes through the checked form
        int j_checked = 0;
        if (fbase + FT <= f) {
          const int whole = cnt & ~(BU - 1);
#pragma unroll 1
          for (int j = 0; j < whole; j += BU) {
            float xv[U][NV][VW];
            float wu[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int src = j + u * EPI + sub;
              const int c = __shfl_sync(kFull, c_l, src);
              if (HAS_VAL) wu[u] = __shfl_sync(kFull, w_l, src);
              const float* xrow = a.x + static_cast<long long>(c) * f;
#pragma unroll
              for (int v = 0; v < NV; ++v) VecIO<VW>::load(xv[u][v], xrow + foff[v], pol_keep);
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
              for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int i = 0; i < VW; ++i)
                  acc[v][i] = HAS_VAL ? fmaf(wu[u], xv[u][v][i], acc[v][i]) : acc[v][i] + xv[u][v][i];
          }
          j_checked = whole;
        }
        for (int j = j_checked; j < cnt; j += BU) {
          float xv[U][NV][VW];
          float wu[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int src = j + u * EPI + sub;
            const int c = __shfl_sync(kFull, c_l, src);
            if (HAS_VAL) wu[u] = __shfl_sync(kFull, w_l, src);
            const bool ok = src < cnt;
            if (!HAS_VAL) wu[u] = ok ? 1.f : 0.f;
            if (HAS_VAL && !ok) wu[u] = 0.f;
            const float* xrow = a.x + static_cast<long long>(c) * f;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
              if (ok && fvalid[v]) {
                VecIO<VW>::load(xv[u][v], xrow + foff[v], pol_keep);
              } else {
#pragma unroll
                for (int i = 0; i < VW; ++i) xv[u][v][i] = 0.f;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
              for (int i = 0; i < VW; ++i) acc[v][i] = fmaf(wu[u], xv[u][v][i], acc[v][i]);
        }
#pragma unroll
        for (int o = G; o < 32; o <<= 1)
#pragma unroll
          for (int v = 0; v < NV; ++v)
#pragma unroll
            for (int i = 0; i < VW; ++i) acc[v][i] += __shfl_xor_sync(kFull, acc[v][i], o);
        if (sub == 0) {
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            if (fvalid[v]) VecIO<VW>::store(a.y + static_cast<size_t>(row) * f + foff[v], acc[v]);
          }
        }
      }
    }
  }
}

// Queue 2, packed form (ASG_FLAG_PACK_SHORT_ROWS; the column blocks of the sharded path, whose rows hold a
// quarter or an eighth of their edges): the warp still reads ids and pointers of 32 rows at once, but
// walks them 32/G rows at a time - every group of G lanes, the lanes that together hold one feature tile
// of a row, owns a row of its own, reads that row's columns (and weights) itself, gathers one X row per
// step with U steps in flight and stores its own output tile, so nothing is reduced across groups.  A
// 3-edge row costs the shared form two half-empty gather instructions, a cross-group reduction and a
// store by half the lanes; two such rows share three instructions here.  On whole rows (a dozen edges,
// degrees inside a 32-row grab differing by up to 2x) the shared form is faster: paired rows wait for
// the longer of the two (measured: +10 % on the short-row kernel of the 2.4 M-row graph), so it stays the
// default.
template <int VW, int G, int NV, int U_REQUESTED, bool HAS_VAL, bool EXTRAS>
__device__ __forceinline__ void spmm_short_rows_packed(const SpmmArgs& a, int n_hub, int n_medium, int n_short) {
  constexpr int U = U_REQUESTED < 4 ? U_REQUESTED : 4;  // X rows in flight per lane group
  constexpr int FT = VW * G * NV;
  constexpr int RPW = 32 / G;                      // rows a warp processes side by side
  constexpr int CREG = (kShortDegree + G - 1) / G;  // column registers per lane: G columns each
  const int lane = threadIdx.x & 31;
  const int l = lane % G;
  const int sub = lane / G;
  const int f = a.f;
  const uint64_t pol_keep = policy_evict_last();
  const uint64_t pol_stream = policy_evict_first();
  if (n_short > 0) {
    const int* shorts = a.order + n_hub + n_medium;
    const int n_batches = (n_short + 31) / 32;
    const long long total = static_cast<long long>(n_batches) * a.n_tiles;
    for (;;) {
      const unsigned long long it = warp_next(&a.header->counter[2]);
      if (it >= static_cast<unsigned long long>(total)) break;
      const int tile = static_cast<int>(it / n_batches);
      const int first = static_cast<int>(it - static_cast<unsigned long long>(tile) * n_batches) * 32;
      const int n_here = n_short - first < 32 ? n_short - first : 32;
      const int fbase = (a.tile_begin + tile) * FT;
      int row_l = 0;
      long long s_l = 0;
      int d_l = 0;
      if (lane < n_here) {
        row_l = shorts[first + lane];
        s_l = a.crow[row_l];
        d_l = static_cast<int>(a.crow[row_l + 1] - s_l);
      }
      bool fvalid[NV];
      int foff[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        foff[v] = fbase + VW * (l + G * v);
        fvalid[v] = foff[v] < f;
      }
      // columns / weights of the first rows: lane l of a group holds entries l, l + G, ... of its row
      int c_next[CREG];
      float w_next[CREG];
      {
        const long long s0 = __shfl_sync(kFull, s_l, sub);
        const int d0 = __shfl_sync(kFull, d_l, sub);
#pragma unroll
        for (int k = 0; k < CREG; ++k) {
          const bool has = l + k * G < d0;
          c_next[k] = has ? static_cast<int>(ld_index(a.col + s0 + l + k * G, pol_stream)) : 0;
          w_next[k] = (HAS_VAL && has) ? ld_weight(a.val + s0 + l + k * G, pol_stream) : 0.f;
        }
      }
      for (int r0 = 0; r0 < n_here; r0 += RPW) {
        const int mine = r0 + sub;  // this group's row of the batch (may lie past its end)
        const int src = mine < 32 ? mine : 31;
        const int row = __shfl_sync(kFull, row_l, src);
        const int cnt_any = __shfl_sync(kFull, d_l, src);  // every lane takes part in the shuffles
        const int cnt = mine < n_here ? cnt_any : 0;
        int c_cur[CREG];
        float w_cur[CREG];
#pragma unroll
        for (int k = 0; k < CREG; ++k) {
          c_cur[k] = c_next[k];
          w_cur[k] = w_next[k];
        }
        if (r0 + RPW < n_here) {  // warp-uniform: the next rows' columns while these rows gather
          const int ahead = r0 + RPW + sub < 32 ? r0 + RPW + sub : 31;
          const long long s1 = __shfl_sync(kFull, s_l, ahead);
          const int d1_any = __shfl_sync(kFull, d_l, ahead);
          const int d1 = r0 + RPW + sub < n_here ? d1_any : 0;
#pragma unroll
          for (int k = 0; k < CREG; ++k) {
            const bool has = l + k * G < d1;
            c_next[k] = has ? static_cast<int>(ld_index(a.col + s1 + l + k * G, pol_stream)) : 0;
            w_next[k] = (HAS_VAL && has) ? ld_weight(a.val + s1 + l + k * G, pol_stream) : 0.f;
          }
        }
        // Accumulating (column blocks of the sharded path): start from the row's current output,
        // fetched before the gathers so that its latency hides behind them.
        const bool writes = mine < n_here && (cnt > 0 || !(EXTRAS && a.accumulate));
        float acc[NV][VW];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          if ((EXTRAS && a.accumulate) && writes && fvalid[v]) {
            VecIO<VW>::load_plain(acc[v], a.y + static_cast<size_t>(row) * f + foff[v]);
          } else {
#pragma unroll
            for (int i = 0; i < VW; ++i) acc[v][i] = 0.f;
          }
        }
        const int longest = __reduce_max_sync(kFull, cnt);
        for (int j = 0; j < longest; j += U) {
          float xv[U][NV][VW];
          float wu[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int e = j + u;
            int c = 0;
            float w = 0.f;
#pragma unroll
            for (int k = 0; k < CREG; ++k) {
              const int lane_of = sub * G + ((e - k * G) & (G - 1));
              const int got_c = __shfl_sync(kFull, c_cur[k], lane_of);
              const float got_w = HAS_VAL ? __shfl_sync(kFull, w_cur[k], lane_of) : 1.f;
              if (e >= k * G && e < (k + 1) * G) {
                c = got_c;
                w = got_w;
              }
            }
            const bool ok = e < cnt;
            wu[u] = ok ? w : 0.f;
            const float* xrow = a.x + static_cast<long long>(c) * f;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
              if (ok && fvalid[v]) {
                VecIO<VW>::load(xv[u][v], xrow + foff[v], pol_keep);
              } else {
#pragma unroll
                for (int i = 0; i < VW; ++i) xv[u][v][i] = 0.f;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
              for (int i = 0; i < VW; ++i) acc[v][i] = fmaf(wu[u], xv[u][v][i], acc[v][i]);
        }
        if (writes) {
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            if (fvalid[v]) VecIO<VW>::store(a.y + static_cast<size_t>(row) * f + foff[v], acc[v]);
          }
        }
      }
    }
  }
}

// EXTRAS = false is the plain product y = A x: the instances without the accumulate, hub-only and self-test
// code, whose registers cost the L2-bound workloads a CTA per SM.  The host picks EXTRAS = true when any of
// those is asked for.
template <int VW, int G, int NV, int U_REQUESTED, bool HAS_VAL, bool EXTRAS>
__device__ __forceinline__ void spmm_body(const SpmmArgs& a) {
  constexpr int U = U_REQUESTED < G ? U_REQUESTED : G;  // an unrolled batch never exceeds 32 edges
  constexpr int EPI = 32 / G;          // edges per load instruction
  constexpr int FT = VW * G * NV;      // feature tile
  constexpr int BU = EPI * U;          // edges per unrolled batch
  static_assert(32 % BU == 0, "batch must divide a 32-edge chunk");

  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  const int l = lane % G;
  const int sub = lane / G;
  const int chunk = kChunkPerWarp * n_warps;

  // shared memory carve-up
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                       // 2 mbarriers
  uint64_t* idle_bar = reinterpret_cast<uint64_t*>(smem + 32);              // self-test: nothing ever arrives here
  int* s_item = reinterpret_cast<int*>(smem + 16);                          // CTA-wide item id
  long long* s_col = reinterpret_cast<long long*>(smem + 128);              // [2][chunk]
  float* s_val = reinterpret_cast<float*>(smem + 128 + size_t(16) * chunk); // [2][chunk]
  float* s_red = reinterpret_cast<float*>(smem + 128 + size_t(24) * chunk); // [n_warps][FT]

  const uint64_t pol_keep = policy_evict_last();
  const uint64_t pol_stream = policy_evict_first();
  const int f = a.f;
  const int n_hub = a.header->n_hub;
  const int n_light = a.header->n_light;

  // ------------------------------------------------------------------ queue 0: hub rows
  if (n_hub > 0) {
    if (tid == 0) {
      mbar_init(&bars[0], 1);
      mbar_init(&bars[1], 1);
      mbar_init(idle_bar, 1);
      mbar_fence_init();
    }
    unsigned seq = 0;  // chunks staged so far by this CTA: stage = seq & 1, parity = (seq >> 1) & 1
    const long long total = static_cast<long long>(n_hub) * a.n_tiles;
    bool alive = true;
    while (alive) {
      __syncthreads();
      if (tid == 0) {
        const unsigned long long it = atomicAdd(&a.header->counter[0], 1ull);
        *s_item = it < static_cast<unsigned long long>(total) ? static_cast<int>(it) : -1;
      }
      __syncthreads();
      const int item = *s_item;
      if (item < 0) break;
      const int tile = item / n_hub;
      const int hub_index = item - tile * n_hub;
      const int row = a.order[hub_index];
      const int fbase = (a.tile_begin + tile) * FT;
      if ((EXTRAS && a.hubs_only) && tile == 0 && tid == 0) a.hub_slot[row] = hub_index;
      const long long s = a.crow[row];
      const long long e = a.crow[row + 1];
      const long long a0 = s & ~3ll;  // staging starts on a 4-edge boundary (32 B of col, 16 B of val)
      const int n_chunks = static_cast<int>((e - a0 + chunk - 1) / chunk);

      float acc[NV][VW];
#pragma unroll
      for (int v = 0; v < NV; ++v)
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[v][i] = 0.f;
      bool fvalid[NV];
      int foff[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        foff[v] = fbase + VW * (l + G * v);
        fvalid[v] = foff[v] < f;
      }

      const bool hub_tile_full = fbase + FT <= f;

      // stage one chunk [g0, g1) of col/val into stage `st`
      auto stage_chunk = [&](int k, unsigned sq) {
        const int st = sq & 1;
        const long long g0 = a0 + static_cast<long long>(k) * chunk;
        const long long g1 = g0 + chunk < e ? g0 + chunk : e;
        const int count = static_cast<int>(g1 - g0);
        long long* dcol = s_col + st * chunk;
        float* dval = s_val + st * chunk;
        if (a.bulk_stage) {
          const int body = count & ~3;
          if (tid == 0) {
            const unsigned bytes = static_cast<unsigned>(body) * (HAS_VAL ? 12u : 8u);
            mbar_expect_tx(&bars[st], bytes);
            if (body > 0) {
              bulk_g2s(dcol, a.col + g0, static_cast<unsigned>(body) * 8u, &bars[st]);
              if (HAS_VAL) bulk_g2s(dval, a.val + g0, static_cast<unsigned>(body) * 4u, &bars[st]);
            }
          }
          if (tid < count - body) {
            dcol[body + tid] = a.col[g0 + body + tid];
            if (HAS_VAL) dval[body + tid] = a.val[g0 + body + tid];
          }
        } else {
          for (int i = tid; i < count; i += blockDim.x) {
            dcol[i] = ld_index(a.col + g0 + i, pol_stream);
            if (HAS_VAL) dval[i] = ld_weight(a.val + g0 + i, pol_stream);
          }
        }
      };

      if (n_chunks > 0) stage_chunk(0, seq);
      __syncthreads();
      // `alive` is the same in every thread at the head of an iteration: once any thread's bounded wait
      // has run out, nothing more is staged (a barrier whose phase never completed must not be armed a
      // second time) and the CTA leaves together after the loop.
      int staged_ahead = 0;  // a chunk beyond the one being waited for is in flight
      for (int k = 0; k < n_chunks && alive; ++k) {
        staged_ahead = k + 1 < n_chunks ? 1 : 0;
        if (staged_ahead) stage_chunk(k + 1, seq + 1);
        const int st = seq & 1;
        bool arrived = true;
        if (a.bulk_stage) {
          // self-test: wait on a barrier nobody arrives on (no copy targets it, so nothing is pending
          // on it when the CTA leaves); the staging itself runs and completes as usual
          uint64_t* awaited = (EXTRAS && a.selftest_stall) ? idle_bar : &bars[st];
          arrived = mbar_wait_bounded(awaited, (EXTRAS && a.selftest_stall) ? 0u : ((seq >> 1) & 1), a.wait_limit_ns);
          if (!arrived) atomicCAS(&a.header->status, 0, kStatusBulkWaitExpired);
        }
        if (arrived) {
          const long long g0 = a0 + static_cast<long long>(k) * chunk;
          const long long g1 = g0 + chunk < e ? g0 + chunk : e;
          const long long lo = g0 > s ? g0 : s;
          const int base = static_cast<int>(lo - g0);
          const int cnt = static_cast<int>(g1 - lo);
          const long long* ccol = s_col + st * chunk + base;
          const float* cval = s_val + st * chunk + base;
          const int n_batches = (cnt + BU - 1) / BU;
          for (int b = warp; b < n_batches; b += n_warps) {
            float xv[U][NV][VW];
            float wu[U];
            if ((b + 1) * BU <= cnt && hub_tile_full) {
              // whole batch inside the chunk and the feature tile: no predicates, no zero fill
#pragma unroll
              for (int u = 0; u < U; ++u) {
                const int j = b * BU + u * EPI + sub;
                const int c = static_cast<int>(ccol[j]);
                if (HAS_VAL) wu[u] = cval[j];
                const float* xrow = a.x + static_cast<long long>(c) * f;
#pragma unroll
                for (int v = 0; v < NV; ++v) VecIO<VW>::load(xv[u][v], xrow + foff[v], pol_keep);
              }
#pragma unroll
              for (int u = 0; u < U; ++u)
#pragma unroll
                for (int v = 0; v < NV; ++v)
#pragma unroll
                  for (int i = 0; i < VW; ++i)
                    acc[v][i] = HAS_VAL ? fmaf(wu[u], xv[u][v][i], acc[v][i]) : acc[v][i] + xv[u][v][i];
              continue;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int j = b * BU + u * EPI + sub;
              const bool ok = j < cnt;
              long long c = 0;
              wu[u] = 0.f;
              if (ok) {
                c = ccol[j];
                wu[u] = HAS_VAL ? cval[j] : 1.f;
              }
              const float* xrow = a.x + static_cast<size_t>(c) * f;
#pragma unroll
              for (int v = 0; v < NV; ++v) {
                if (ok && fvalid[v]) {
                  VecIO<VW>::load(xv[u][v], xrow + foff[v], pol_keep);
                } else {
#pragma unroll
                  for (int i = 0; i < VW; ++i) xv[u][v][i] = 0.f;
                }
              }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
              for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int i = 0; i < VW; ++i) acc[v][i] = fmaf(wu[u], xv[u][v][i], acc[v][i]);
          }
        }
        ++seq;
        // All warps have finished reading this stage (and the plain-store tail of the next stage
        // is visible) before the stage is refilled; the same barrier tells every thread whether
        // some thread's wait ran out.
        if (a.bulk_stage) fence_proxy_async();
        alive = __syncthreads_or(!arrived) == 0;
      }
      // a bounded wait gave up in some thread: every thread leaves together, after one more bounded
      // wait for each copy that may still be in flight into this CTA's shared memory (the chunk that
      // was being waited for and the one staged ahead of it)
      if (!alive) {
        if (tid == 0 && a.bulk_stage && seq > 0) {
          mbar_wait_bounded(&bars[(seq - 1) & 1], ((seq - 1) >> 1) & 1, a.wait_limit_ns);
          if (staged_ahead) mbar_wait_bounded(&bars[seq & 1], (seq >> 1) & 1, a.wait_limit_ns);
        }
        __syncthreads();
        break;
      }

      // combine lane groups, then warps
#pragma unroll
      for (int o = G; o < 32; o <<= 1)
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[v][i] += __shfl_xor_sync(kFull, acc[v][i], o);
      if (sub == 0) {
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) s_red[warp * FT + VW * (l + G * v) + i] = acc[v][i];
      }
      __syncthreads();
      for (int i = tid; i < FT; i += blockDim.x) {
        if (fbase + i < f) {
          float total_i = 0.f;
          for (int w = 0; w < n_warps; ++w) total_i += s_red[w * FT + i];
          float* dst = a.y + static_cast<size_t>((EXTRAS && a.hubs_only) ? hub_index : row) * f + fbase + i;
          if ((EXTRAS && a.accumulate)) total_i += *dst;
          st_stream1(dst, total_i);
        }
      }
    }
    if (!alive) return;
  }

  if ((EXTRAS && a.hubs_only)) return;

  // ------------------------------------------------------------------ queue 1: light rows
  const int n_short = a.header->n_short;
  const int n_medium = n_light - n_short;  // light rows of 32 edges or more: one (row, tile) per grab
  if (n_medium > 0) {
    const long long total = static_cast<long long>(n_medium) * a.n_tiles;
    const int* light = a.order + n_hub;
    for (;;) {
      const unsigned long long it = warp_next(&a.header->counter[1]);
      if (it >= static_cast<unsigned long long>(total)) break;
      const int tile = static_cast<int>(it / n_medium);
      const int row = light[it - static_cast<unsigned long long>(tile) * n_medium];
      const int fbase = (a.tile_begin + tile) * FT;
      const long long s = a.crow[row];
      const long long e = a.crow[row + 1];

      bool fvalid[NV];
      int foff[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        foff[v] = fbase + VW * (l + G * v);
        fvalid[v] = foff[v] < f;
      }
      // accumulating: the storing lanes start from the row's current output (fetched under the gathers)
      float acc[NV][VW];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        if ((EXTRAS && a.accumulate) && sub == 0 && fvalid[v]) {
          VecIO<VW>::load_plain(acc[v], a.y + static_cast<size_t>(row) * f + foff[v]);
        } else {
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[v][i] = 0.f;
        }
      }

      const bool tile_full = fbase + FT <= f;

      int c_next = 0;
      float w_next = 0.f;
      if (s + lane < e) {
        c_next = static_cast<int>(ld_index(a.col + s + lane, pol_stream));
        if (HAS_VAL) w_next = ld_weight(a.val + s + lane, pol_stream);
      }
      for (long long p = s; p < e; p += 32) {
        const int c_l = c_next;
        const float w_l = w_next;
        const int cnt = e - p < 32 ? static_cast<int>(e - p) : 32;
        if (p + 32 + lane < e) {
          c_next = static_cast<int>(ld_index(a.col + p + 32 + lane, pol_stream));
          if (HAS_VAL) w_next = ld_weight(a.val + p + 32 + lane, pol_stream);
        }
        int j_checked = 0;  // where the predicated batches start
        // Whole-row tiles (the HBM-streaming configuration): every whole batch of edges takes the form
        // without predicates and zero fill, only the last, partly filled batch of a row's last chunk the
        // checked one.  Narrower tiles (gathers served by L2, where warps per SM count most): only whole
        // 32-edge chunks do, which keeps the kernel at 64 registers.
        constexpr bool kWholeBatches = (VW == 8 && FT == 128);
        if (tile_full && (kWholeBatches || cnt == 32)) {
          const int whole = kWholeBatches ? (cnt & ~(BU - 1)) : 32;
#pragma unroll 1
          for (int j = 0; j < whole; j += BU) {
            float xv[U][NV][VW];
            float wu[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int src = j + u * EPI + sub;
              const int c = __shfl_sync(kFull, c_l, src);
              if (HAS_VAL) wu[u] = __shfl_sync(kFull, w_l, src);
              const float* xrow = a.x + static_cast<long long>(c) * f;
#pragma unroll
              for (int v = 0; v < NV; ++v) VecIO<VW>::load(xv[u][v], xrow + foff[v], pol_keep);
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
              for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int i = 0; i < VW; ++i)
                  acc[v][i] = HAS_VAL ? fmaf(wu[u], xv[u][v][i], acc[v][i]) : acc[v][i] + xv[u][v][i];
          }
          if (!kWholeBatches || whole == cnt) continue;  // nothing left for the checked form
          j_checked = whole;
        }
        for (int j = j_checked; j < cnt; j += BU) {
          float xv[U][NV][VW];
          float wu[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int src = j + u * EPI + sub;
            const int c = __shfl_sync(kFull, c_l, src);
            if (HAS_VAL) wu[u] = __shfl_sync(kFull, w_l, src);
            const bool ok = src < cnt;
            if (!HAS_VAL) wu[u] = ok ? 1.f : 0.f;
            if (HAS_VAL && !ok) wu[u] = 0.f;
            const float* xrow = a.x + static_cast<size_t>(c) * f;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
              if (ok && fvalid[v]) {
                VecIO<VW>::load(xv[u][v], xrow + foff[v], pol_keep);
              } else {
#pragma unroll
                for (int i = 0; i < VW; ++i) xv[u][v][i] = 0.f;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
              for (int i = 0; i < VW; ++i) acc[v][i] = fmaf(wu[u], xv[u][v][i], acc[v][i]);
        }
      }
#pragma unroll
      for (int o = G; o < 32; o <<= 1)
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[v][i] += __shfl_xor_sync(kFull, acc[v][i], o);
      if (sub == 0) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          if (fvalid[v]) VecIO<VW>::store(a.y + static_cast<size_t>(row) * f + foff[v], acc[v]);
        }
      }
    }
  }

}

// Two entry kernels over the same body.  They differ only in the register budget the compiler is
// given: with launch bounds (512, 2) it stays at 64 registers, eight 4-warp CTAs per SM (best when the
// gather is served by L2: left to itself the compiler took 79 and the 233 k-row graph ran 4 % slower);
// with (512, 1) it may use 128 registers and schedules loads further ahead, which measured 10 % faster
// when the gathered rows come from HBM (whole-row 128-float tiles).
template <int VW, int G, int NV, int U, bool HAS_VAL, bool EXTRAS>
__global__ void __launch_bounds__(512, 2) spmm_kernel(const SpmmArgs a) {
  pdl_release_dependents();  // the short-row kernel may move in as CTAs of this one retire
  spmm_body<VW, G, NV, U, HAS_VAL, EXTRAS>(a);
}
template <int VW, int G, int NV, int U, bool HAS_VAL, bool EXTRAS>
__global__ void __launch_bounds__(512, 1) spmm_kernel_deep(const SpmmArgs a) {
  pdl_release_dependents();
  spmm_body<VW, G, NV, U, HAS_VAL, EXTRAS>(a);
}

template <int VW, int G, int NV, int U, bool HAS_VAL, bool PACKED, bool EXTRAS>
__global__ void __launch_bounds__(512) spmm_short_kernel(const SpmmArgs a) {
  const int n_hub = a.header->n_hub;
  const int n_short = a.header->n_short;
  if (n_short > 0) {
    if (PACKED) spmm_short_rows_packed<VW, G, NV, U, HAS_VAL, EXTRAS>(a, n_hub, a.header->n_light - n_short, n_short);
    else spmm_short_rows<VW, G, NV, U, HAS_VAL, EXTRAS>(a, n_hub, a.header->n_light - n_short, n_short);
  }
  pdl_wait_for_primary();  // do not complete before the main kernel has
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
template <int VW, int G, int NV, int U, bool HAS_VAL>
static int launch_instance(const SpmmArgs& args, int warps, cudaStream_t stream, int device) {
  constexpr int FT = VW * G * NV;
  // The entry with the roomy register budget when the gathers stream from HBM: always for whole-row tiles
  // of 128 floats with 256-bit loads, and for narrower tiles when X is much larger than L2 (there the
  // 64-register entry lost 8 % on the 2.4 M-row graph; on the 233 k-row graph, whose X fits L2, it wins 4 %).
  constexpr bool kWholeRow = (VW == 8 && FT == 128);
  const bool deep = kWholeRow || args.streaming;
  const bool extras = args.accumulate || args.hubs_only || args.selftest_stall || args.pack_short;
  auto kernel = deep ? (extras ? spmm_kernel_deep<VW, G, NV, U, HAS_VAL, true> : spmm_kernel_deep<VW, G, NV, U, HAS_VAL, false>)
                     : (extras ? spmm_kernel<VW, G, NV, U, HAS_VAL, true> : spmm_kernel<VW, G, NV, U, HAS_VAL, false>);
  const int threads = warps * 32;
  const int chunk = kChunkPerWarp * warps;
  const size_t smem = 128 + size_t(24) * chunk + size_t(4) * warps * FT;
  if (smem > 48 * 1024) {
    ASG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  }
  int per_sm = 0;
  ASG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem));
  if (per_sm < 1) per_sm = 1;
  const int grid = sm_count(device) * per_sm;
  kernel<<<grid, threads, smem, stream>>>(args);
  ASG_CUDA(cudaGetLastError());
  if (args.hubs_only) return ASG_OK;
  // queue 2 (rows of fewer than 32 edges); leaves at once when the plan has none
  auto short_kernel = args.pack_short ? spmm_short_kernel<VW, G, NV, U, HAS_VAL, true, true>
                      : extras        ? spmm_short_kernel<VW, G, NV, U, HAS_VAL, false, true>
                                      : spmm_short_kernel<VW, G, NV, U, HAS_VAL, false, false>;
  int short_per_sm = 0;
  ASG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&short_per_sm, short_kernel, threads, 0));
  if (short_per_sm < 1) short_per_sm = 1;
  ASG_CUDA(launch_overlapped(short_kernel, sm_count(device) * short_per_sm, threads, 0, stream, args));
  return ASG_OK;
}

template <int VW, int G, int NV, int U>
static int launch_val(const SpmmArgs& args, int warps, cudaStream_t stream, int device) {
  if (args.val != nullptr) return launch_instance<VW, G, NV, U, true>(args, warps, stream, device);
  return launch_instance<VW, G, NV, U, false>(args, warps, stream, device);
}

// Gather instructions issued per lane before their results are used (measured best on B200):
// 8 with 128-bit loads, 4 with 256-bit loads, 4 with scalar loads (each times FT/32 loads).
constexpr int kLoadsInFlight128 = 8;
constexpr int kLoadsInFlight256 = 4;
constexpr int kLoadsInFlightScalar = 4;

static int launch_spmm(const SpmmArgs& args, int vw, int feature_tile, int warps, cudaStream_t stream, int device) {
  constexpr int U4 = kLoadsInFlight128, U8 = kLoadsInFlight256, U1 = kLoadsInFlightScalar;
  if (vw == 8) {
    switch (feature_tile) {
      case 32: return launch_val<8, 4, 1, U8>(args, warps, stream, device);
      case 64: return launch_val<8, 8, 1, U8>(args, warps, stream, device);
      case 128: return launch_val<8, 16, 1, (U8 > 2 ? U8 : 2)>(args, warps, stream, device);
      default: return launch_val<8, 32, 1, U8>(args, warps, stream, device);
    }
  }
  if (vw == 4) {
    switch (feature_tile) {
      case 32: return launch_val<4, 8, 1, U4>(args, warps, stream, device);
      case 64: return launch_val<4, 16, 1, U4>(args, warps, stream, device);
      case 128: return launch_val<4, 32, 1, U4>(args, warps, stream, device);
      default: return launch_val<4, 32, 2, (U4 > 4 ? U4 / 2 : U4)>(args, warps, stream, device);
    }
  }
  switch (feature_tile) {
    case 32: return launch_val<1, 32, 1, U1 * 2>(args, warps, stream, device);
    case 64: return launch_val<1, 32, 2, U1>(args, warps, stream, device);
    case 128: return launch_val<1, 32, 4, U1>(args, warps, stream, device);
    default: return launch_val<1, 32, 8, (U1 > 2 ? U1 / 2 : U1)>(args, warps, stream, device);
  }
}

static bool aligned_to(const void* p, size_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; }

static int spmm_entry(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* y,
                      int64_t n_rows, int64_t nnz, int64_t f, int feature_tile, int warps, int64_t hub_threshold,
                      unsigned flags, void* workspace, size_t workspace_bytes, void* stream_ptr,
                      int64_t feature_begin = 0, int64_t feature_count = 0, int* hub_slot = nullptr) {
  ASG_REQUIRE(n_rows >= 0 && nnz >= 0 && f >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(n_rows <= 2147483647ll - 2048 && f <= 2147483647ll, ASG_ERANGE,
              "SpMM dimensions exceed the kernel index range");
  ASG_REQUIRE(feature_tile == 32 || feature_tile == 64 || feature_tile == 128 || feature_tile == 256, ASG_EINVAL,
              "feature_tile must be 64 or 128");
  ASG_REQUIRE(warps == 2 || warps == 4 || warps == 8 || warps == 16, ASG_EINVAL,
              "warps_per_block must be 2, 4, or 8");
  if (n_rows == 0 || f == 0) return ASG_OK;
  ASG_REQUIRE(crow != nullptr && x != nullptr && y != nullptr, ASG_EINVAL, "crow, x and y must not be null");
  ASG_REQUIRE(nnz == 0 || col != nullptr, ASG_EINVAL, "col must not be null");
  if (int rc = check_workspace(workspace, workspace_bytes, n_rows)) return rc;
  DeviceGuard guard(x);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);

  if (flags & ASG_FLAG_PLAN_READY) {
    if (int rc = reset_counters(workspace, stream)) return rc;
  } else {
    if (int rc = plan_build(crow, n_rows, hub_threshold, workspace, stream)) return rc;
  }

  int vw = 1;
  if (!(flags & ASG_FLAG_NO_VEC4)) {
    if (f % 8 == 0 && aligned_to(x, 32) && aligned_to(y, 32)) vw = 8;
    else if (f % 4 == 0 && aligned_to(x, 16) && aligned_to(y, 16)) vw = 4;
  }
  // a tile wider than the (rounded-up) feature count only wastes lanes
  while (feature_tile > 32 && feature_tile / 2 >= f) feature_tile /= 2;

  SpmmArgs args;
  args.crow = crow;
  args.col = col;
  args.val = val;
  args.x = x;
  args.y = y;
  args.header = static_cast<Header*>(workspace);
  args.order = reinterpret_cast<const int*>(static_cast<const char*>(workspace) + order_offset());
  args.f = static_cast<int>(f);
  args.n_tiles = static_cast<int>((f + feature_tile - 1) / feature_tile);
  args.tile_begin = 0;
  if (feature_count > 0) {  // only the columns [feature_begin, feature_begin + feature_count) of y
    ASG_REQUIRE(feature_begin >= 0 && feature_begin + feature_count <= f, ASG_EINVAL, "feature range exceeds f");
    ASG_REQUIRE(feature_begin % feature_tile == 0 &&
                    (feature_count % feature_tile == 0 || feature_begin + feature_count == f),
                ASG_EINVAL, "feature range must start and end on a feature_tile boundary (or at f)");
    args.tile_begin = static_cast<int>(feature_begin / feature_tile);
    args.n_tiles = static_cast<int>((feature_count + feature_tile - 1) / feature_tile);
  }
  args.accumulate = (flags & ASG_FLAG_ACCUMULATE) ? 1 : 0;
  args.pack_short = (flags & ASG_FLAG_PACK_SHORT_ROWS) ? 1 : 0;
  // Self-test of the give-up path: the hub staging waits on a barrier on which nothing ever arrives, so
  // the wait can only run out (after 20 ms instead of a second); the copies themselves complete normally
  // on their own barriers, which the leaving CTA still waits for.
  args.selftest_stall = (flags & ASG_FLAG_SELFTEST_STALL) ? 1 : 0;
  args.wait_limit_ns = args.selftest_stall ? 20000000ull : kWaitLimitNs;
  args.bulk_stage = (!(flags & ASG_FLAG_NO_BULK_STAGE) && aligned_to(col, 16) && (val == nullptr || aligned_to(val, 16))) ? 1 : 0;
  args.hubs_only = hub_slot != nullptr ? 1 : 0;
  args.hub_slot = hub_slot;
  // Items run tile-major, so what has to stay in L2 during a pass is one feature tile of every X row
  // (square graphs: X has about n_rows rows).
  const long long slice = static_cast<long long>(n_rows) * (f < feature_tile ? f : feature_tile) * 4;
  args.streaming = slice > l2_bytes(guard.target) * 3 / 2 ? 1 : 0;
  return launch_spmm(args, vw, feature_tile, warps, stream, guard.target);
}

int spmm_hub_rows_compact(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* hub_y,
                          int* hub_slot, int64_t n_rows, int64_t nnz, int64_t f, int feature_tile, int warps,
                          int64_t hub_threshold, unsigned flags, void* workspace, size_t workspace_bytes,
                          cudaStream_t stream) {
  return spmm_entry(crow, col, val, x, hub_y, n_rows, nnz, f, feature_tile, warps, hub_threshold, flags, workspace,
                    workspace_bytes, stream, 0, 0, hub_slot);
}

}  // namespace asg

extern "C" {

int asg_spmm_csr_ex(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* y,
                    int64_t n_rows, int64_t nnz, int64_t f, int feature_tile, int warps_per_block,
                    int64_t hub_threshold, unsigned flags, void* workspace, size_t workspace_bytes, void* stream) {
  return asg::spmm_entry(crow, col, val, x, y, n_rows, nnz, f, feature_tile, warps_per_block, hub_threshold, flags,
                         workspace, workspace_bytes, stream);
}

int asg_spmm_csr_range(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* y,
                       int64_t n_rows, int64_t nnz, int64_t f, int64_t feature_begin, int64_t feature_count,
                       int feature_tile, int warps_per_block, int64_t hub_threshold, unsigned flags, void* workspace,
                       size_t workspace_bytes, void* stream) {
  if (feature_count <= 0) return asg::fail(ASG_EINVAL, "%s", "feature_count must be positive");
  return asg::spmm_entry(crow, col, val, x, y, n_rows, nnz, f, feature_tile, warps_per_block, hub_threshold, flags,
                         workspace, workspace_bytes, stream, feature_begin, feature_count);
}

int asg_spmm_csr_split(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* y,
                       int64_t n_rows, int64_t nnz, int64_t f, int feature_tile, int warps_per_block,
                       int64_t hub_threshold, void* workspace, size_t workspace_bytes, void* stream) {
  if (hub_threshold <= 0) return asg::fail(ASG_EINVAL, "%s", "hub_threshold must be positive");
  return asg::spmm_entry(crow, col, val, x, y, n_rows, nnz, f, feature_tile, warps_per_block, hub_threshold, 0u,
                         workspace, workspace_bytes, stream);
}

int asg_spmm_csr(const int64_t* crow, const int64_t* col, const float* val, const float* x, float* y,
                 int64_t n_rows, int64_t nnz, int64_t f, void* workspace, size_t workspace_bytes, void* stream) {
  // Defaults from the B200 sweeps: 64-float tiles (best or within 4 % of best on every measured graph,
  // 13 % ahead when X is about the size of L2), 4 warps per CTA, hubs from 1024 edges up.
  return asg::spmm_entry(crow, col, val, x, y, n_rows, nnz, f, 64, 4, 1024, 0u, workspace, workspace_bytes,
                         stream);
}

}  // extern "C"
