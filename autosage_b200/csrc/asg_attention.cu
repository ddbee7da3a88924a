// CSR row softmax and the fused SDDMM -> softmax -> SpMM attention row kernel for sm_100a.
//
// Reference behaviour (autosage/_auto.py:744-780): scores = SDDMM(Q, K); per CSR row
// p = exp(s - max) / sum(exp(s - max)); out = SpMM(p, V).  The reference runs this as three passes
// with about ten ATen kernels for the softmax alone and scores/probabilities round-tripping
// through memory.
//
//   csr_softmax_kernel   the standalone softmax: one warp per light row, one CTA per hub row,
//                        three sweeps over the row segment (max, sum, normalise).
//   attention_kernel     the fused pipeline: for each 32-edge batch of a row the warp computes the
//                        32 scores (same code as the SDDMM kernel), folds them into a running
//                        maximum m and running sum l, rescales the output accumulator by
//                        exp(m_old - m_new) and adds exp(s - m_new) * V[col]; hub rows are shared by
//                        the warps of a CTA whose (m, l, acc) triples are merged at the end.
//                        Scores and probabilities never leave registers.
#include <math_constants.h>

#include "asg_tile.cuh"

namespace asg {

// ------------------------------------------------------------------------------------ softmax
struct SoftmaxArgs {
  const int64_t* crow;
  const float* scores;
  float* probs;
  Header* header;
  const int* order;
};

__device__ __forceinline__ void softmax_segment_warp(const float* __restrict__ in, float* __restrict__ out,
                                                     long long s, long long e, int lane) {
  float m = -CUDART_INF_F;
  for (long long p = s + lane; p < e; p += 32) m = fmaxf(m, in[p]);
  m = warp_max(m);
  float sum = 0.f;
  for (long long p = s + lane; p < e; p += 32) sum += expf(in[p] - m);
  sum = warp_sum(sum);
  for (long long p = s + lane; p < e; p += 32) out[p] = expf(in[p] - m) / sum;
}

__global__ void __launch_bounds__(512) csr_softmax_kernel(const SoftmaxArgs a) {
  __shared__ int s_item;
  __shared__ float s_part[16];
  __shared__ float s_bcast;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
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
      const long long e = a.crow[row + 1];
      float m = -CUDART_INF_F;
      for (long long p = s + tid; p < e; p += blockDim.x) m = fmaxf(m, a.scores[p]);
      m = warp_max(m);
      if (lane == 0) s_part[warp] = m;
      __syncthreads();
      if (tid == 0) {
        float t = s_part[0];
        for (int w = 1; w < n_warps; ++w) t = fmaxf(t, s_part[w]);
        s_bcast = t;
      }
      __syncthreads();
      m = s_bcast;
      float sum = 0.f;
      for (long long p = s + tid; p < e; p += blockDim.x) sum += expf(a.scores[p] - m);
      sum = warp_sum(sum);
      __syncthreads();
      if (lane == 0) s_part[warp] = sum;
      __syncthreads();
      if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < n_warps; ++w) t += s_part[w];
        s_bcast = t;
      }
      __syncthreads();
      sum = s_bcast;
      for (long long p = s + tid; p < e; p += blockDim.x) a.probs[p] = expf(a.scores[p] - m) / sum;
    }
  }
  if (n_light > 0) {
    const int* light = a.order + n_hub;
    for (;;) {
      const unsigned long long it = warp_next(&a.header->counter[1]);
      if (it >= static_cast<unsigned long long>(n_light)) break;
      const int row = light[it];
      softmax_segment_warp(a.scores, a.probs, a.crow[row], a.crow[row + 1], lane);
    }
  }
}

// ------------------------------------------------------------------------------ fused attention
// Rows of kSplitDegree edges or more ("mega rows") are not walked by one CTA: they are cut into
// segments of kSegmentEdges edges, every segment is a work item of its own, each CTA leaves its
// segment's (running maximum, running sum, un-normalised accumulator) in the split area, and the CTA
// that finishes a row's last segment merges them (the same merge the warps of one CTA do).  Without
// this the longest row of a power-law graph (13,000 edges on the 169,343-row benchmark graph) keeps one
// CTA busy for most of the launch.  The area lives behind the plan in the workspace and is optional.
constexpr int kSplitDegree = 4096;    // a power of two: such rows are exactly the front of the hub order
constexpr int kSegmentEdges = 1024;
constexpr int kMaxSegments = 512;
constexpr int kMaxSplitRows = 128;
constexpr int kPartialStride = 2 + 512;  // m, l, accumulator of up to 512 features

struct SplitArea {
  int n_split;     // hub rows order[0 .. n_split) are processed in segments
  int n_segments;
  int pad[2];
  int first_segment[kMaxSplitRows];
  int segment_count[kMaxSplitRows];
  int done[kMaxSplitRows];
  int segment_hub[kMaxSegments];    // index into the hub order
  int segment_index[kMaxSegments];  // which segment of that row
  float partial[kMaxSegments][kPartialStride];
};

struct AttentionArgs {
  const int64_t* crow;
  const int64_t* col;
  const float* q;
  const float* k;
  const float* v;
  float* out;
  Header* header;
  const int* order;
  SplitArea* split;  // null: no row is split
  int f;
  float scale;
};

// One warp lists the segments of the mega rows (they lead the hub order: hubs are sorted by descending
// floor(log2 degree)) and clears the per-row completion counters; 32 hub rows per step, their degrees
// read in parallel, segment offsets by a warp scan.
__global__ void __launch_bounds__(32) attention_split_plan(const AttentionArgs a) {
  SplitArea* area = a.split;
  const int lane = threadIdx.x;
  const int n_hub = a.header->n_hub;
  int rows = 0, segments = 0;
  bool more = true;
  for (int base = 0; base < kMaxSplitRows && more; base += 32) {
    const int hub = base + lane;
    int count = 0;
    if (hub < n_hub) {
      const int row = a.order[hub];
      const long long degree = a.crow[row + 1] - a.crow[row];
      if (degree >= kSplitDegree) count = static_cast<int>((degree + kSegmentEdges - 1) / kSegmentEdges);
    }
    int inclusive = count;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(kFull, inclusive, o);
      if (lane >= o) inclusive += up;
    }
    // rows are taken while they are mega rows AND their segments still fit the table
    const bool take = count > 0 && segments + inclusive <= kMaxSegments;
    const unsigned taken = __ballot_sync(kFull, take);
    const int n_taken = __ffs(~taken) - 1 < 0 ? 32 : __ffs(~taken) - 1;  // leading run of taken rows
    if (lane < n_taken) {
      const int first = segments + inclusive - count;
      area->first_segment[hub] = first;
      area->segment_count[hub] = count;
      area->done[hub] = 0;
      for (int s = 0; s < count; ++s) {
        area->segment_hub[first + s] = hub;
        area->segment_index[first + s] = s;
      }
    }
    const int added = n_taken > 0 ? __shfl_sync(kFull, inclusive, n_taken - 1) : 0;
    rows += n_taken;
    segments += added;
    more = n_taken == 32;
  }
  if (lane == 0) {
    area->n_split = rows;
    area->n_segments = segments;
  }
}

// Loads the row of Q a warp works on into registers (lane l of a group owns floats VW*(l+G*v)+i).
template <int VW, int G, int NV>
__device__ __forceinline__ void attention_load_q(const AttentionArgs& a, int row, int lane, uint64_t pol_stream,
                                                 float (&q)[NV][VW], bool (&fvalid)[NV], int (&foff)[NV]) {
  const int l = lane % G;
  const float* qrow = a.q + static_cast<size_t>(row) * a.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    foff[v] = VW * (l + G * v);
    fvalid[v] = foff[v] < a.f;
    if (fvalid[v]) {
      VecIO<VW>::load(q[v], qrow + foff[v], pol_stream);  // read once: must not push K and V out of L2
    } else {
#pragma unroll
      for (int i = 0; i < VW; ++i) q[v][i] = 0.f;
    }
  }
}

// One batch of up to 32 edges (column ids in c_l, one per lane) folded into the online-softmax state
// of the row: running max m, running sum l and the output accumulator (lane-group partial sums).
template <int VW, int G, int NV, int U_REQUESTED>
__device__ __forceinline__ void attention_one_batch(const AttentionArgs& a, int c_l, int cnt, int lane,
                                                    const float (&q)[NV][VW], const bool (&fvalid)[NV],
                                                    const int (&foff)[NV], bool tile_full, uint64_t pol_keep,
                                                    float& m_run, float& l_run, float (&acc)[NV][VW]) {
  constexpr int EPI = 32 / G;
  constexpr int U = U_REQUESTED < G ? U_REQUESTED : G;  // an unrolled batch never exceeds 32 edges
  constexpr int BU = EPI * U;
  const int l = lane % G;
  const int sub = lane / G;
  const int f = a.f;

  // 1. scores of the batch: lane (l, sub) ends with the score of edge l*EPI + sub
  float part[G];
#pragma unroll
  for (int i = 0; i < G; ++i) part[i] = 0.f;
  batch_dots<VW, G, NV, U, true>(a.k, f, c_l, cnt, sub, q, fvalid, foff, pol_keep, part);
  const float dot = group_reduce_scatter<G>(part, l);
  const int my_edge = l * EPI + sub;
  const float score = my_edge < cnt ? dot * a.scale : -CUDART_INF_F;

  // 2. fold into the running max / sum
  const float m_new = fmaxf(m_run, warp_max(score));
  const float rescale = expf(m_run - m_new);  // exp(-inf) = 0 on the first batch
  const float prob = my_edge < cnt ? expf(score - m_new) : 0.f;
  l_run = l_run * rescale + warp_sum(prob);
  m_run = m_new;
#pragma unroll
  for (int v = 0; v < NV; ++v)
#pragma unroll
    for (int i = 0; i < VW; ++i) acc[v][i] *= rescale;

  // 3. acc += sum_j prob_j * V[col_j]; the probability of edge j sits in lane (j/EPI) + G*(j%EPI)
  int j_checked = 0;
  if (tile_full) {
    // whole batches of edges inside a full feature tile: no predicates, no zero fill
    const int whole = cnt & ~(BU - 1);
#pragma unroll 1
    for (int j = 0; j < whole; j += BU) {
      float xv[U][NV][VW];
      float wu[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int src = j + u * EPI + sub;
        const int c = __shfl_sync(kFull, c_l, src);
        wu[u] = __shfl_sync(kFull, prob, (src / EPI) + G * (src % EPI));
        const float* vrow = a.v + static_cast<size_t>(c) * f;
#pragma unroll
        for (int v = 0; v < NV; ++v) VecIO<VW>::load(xv[u][v], vrow + foff[v], pol_keep);
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[v][i] = fmaf(wu[u], xv[u][v][i], acc[v][i]);
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
      const float w = __shfl_sync(kFull, prob, (src / EPI) + G * (src % EPI));
      const bool ok = src < cnt;
      wu[u] = ok ? w : 0.f;
      const float* vrow = a.v + static_cast<size_t>(c) * f;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        if (ok && fvalid[v]) {
          VecIO<VW>::load(xv[u][v], vrow + foff[v], pol_keep);
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

// All batches of one row that this warp is responsible for (first, first+stride, ...).
template <int VW, int G, int NV, int U>
__device__ __forceinline__ void attention_batches(const AttentionArgs& a, int row, long long first, long long e,
                                                  long long stride, int lane, uint64_t pol_keep, uint64_t pol_stream,
                                                  float& m_run, float& l_run, float (&acc)[NV][VW]) {
  float q[NV][VW];
  bool fvalid[NV];
  int foff[NV];
  attention_load_q<VW, G, NV>(a, row, lane, pol_stream, q, fvalid, foff);
  bool lane_full = true;
#pragma unroll
  for (int v = 0; v < NV; ++v) lane_full = lane_full && fvalid[v];
  const bool tile_full = __all_sync(kFull, lane_full);  // every lane inside the row: the V gathers need no predicates
  int c_next = 0;  // the next batch's columns are fetched while the current batch gathers
  if (first + lane < e) c_next = static_cast<int>(ld_index(a.col + first + lane, pol_stream));
  for (long long p = first; p < e; p += stride) {
    const int cnt = e - p < 32 ? static_cast<int>(e - p) : 32;
    const int c_l = c_next;
    if (p + stride + lane < e) c_next = static_cast<int>(ld_index(a.col + p + stride + lane, pol_stream));
    attention_one_batch<VW, G, NV, U>(a, c_l, cnt, lane, q, fvalid, foff, tile_full, pol_keep, m_run, l_run, acc);
  }
}

template <int VW, int G, int NV, int U>
__global__ void __launch_bounds__(512) attention_kernel(const AttentionArgs a) {
  pdl_release_dependents();  // the short-row kernel may move in as CTAs of this one retire
  constexpr int FT = VW * G * NV;
  extern __shared__ __align__(16) unsigned char smem[];
  int* s_item = reinterpret_cast<int*>(smem);
  float* s_m = reinterpret_cast<float*>(smem + 16);   // [16]
  float* s_l = s_m + 16;                               // [16]
  float* s_acc = s_l + 16;                             // [n_warps][FT]
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  const int l = lane % G;
  const int sub = lane / G;
  const uint64_t pol_keep = policy_evict_last();
  const uint64_t pol_stream = policy_evict_first();
  const int n_hub = a.header->n_hub;
  const int n_light = a.header->n_light;
  const int f = a.f;

  if (n_hub > 0) {
    const int n_split = a.split != nullptr ? a.split->n_split : 0;
    const int n_segments = a.split != nullptr ? a.split->n_segments : 0;
    const int n_items = n_segments + (n_hub - n_split);  // segments of the mega rows first, then whole hub rows
    for (;;) {
      __syncthreads();
      if (tid == 0) {
        const unsigned long long it = atomicAdd(&a.header->counter[0], 1ull);
        *s_item = it < static_cast<unsigned long long>(n_items) ? static_cast<int>(it) : -1;
      }
      __syncthreads();
      const int item = *s_item;
      if (item < 0) break;
      const bool segment = item < n_segments;
      const int hub = segment ? a.split->segment_hub[item] : n_split + (item - n_segments);
      const int row = a.order[hub];
      long long begin = a.crow[row], end = a.crow[row + 1];
      if (segment) {
        begin += static_cast<long long>(a.split->segment_index[item]) * kSegmentEdges;
        if (begin + kSegmentEdges < end) end = begin + kSegmentEdges;
      }
      float m_run = -CUDART_INF_F, l_run = 0.f;
      float acc[NV][VW];
#pragma unroll
      for (int v = 0; v < NV; ++v)
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[v][i] = 0.f;
      attention_batches<VW, G, NV, U>(a, row, begin + 32ll * warp, end, 32ll * n_warps, lane, pol_keep, pol_stream,
                                      m_run, l_run, acc);
#pragma unroll
      for (int o = G; o < 32; o <<= 1)
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[v][i] += __shfl_xor_sync(kFull, acc[v][i], o);
      if (lane == 0) {
        s_m[warp] = m_run;
        s_l[warp] = l_run;
      }
      if (sub == 0) {
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) s_acc[warp * FT + VW * (l + G * v) + i] = acc[v][i];
      }
      __syncthreads();
      float m_all = s_m[0];
      for (int w = 1; w < n_warps; ++w) m_all = fmaxf(m_all, s_m[w]);
      float l_all = 0.f;
      for (int w = 0; w < n_warps; ++w) l_all += s_l[w] * expf(s_m[w] - m_all);  // idle warps: 0 * exp(-inf) = 0
      float* partial = segment ? a.split->partial[item] : nullptr;
      for (int i = tid; i < FT; i += blockDim.x) {
        if (i < f) {
          float t = 0.f;
          for (int w = 0; w < n_warps; ++w) {
            const float weight = s_l[w] > 0.f ? expf(s_m[w] - m_all) : 0.f;
            t = fmaf(s_acc[w * FT + i], weight, t);
          }
          if (segment) partial[2 + i] = t;  // un-normalised: the row's merge divides
          else st_stream1(a.out + static_cast<size_t>(row) * f + i, l_all > 0.f ? t / l_all : 0.f);
        }
      }
      if (segment) {
        if (tid == 0) {
          partial[0] = m_all;
          partial[1] = l_all;
        }
        // the CTA that completes the row's last segment merges all of them
        __threadfence();
        __syncthreads();
        if (tid == 0) *s_item = atomicAdd(&a.split->done[hub], 1) == a.split->segment_count[hub] - 1 ? 1 : 0;
        __syncthreads();
        if (*s_item == 1) {
          __threadfence();
          const int first = a.split->first_segment[hub];
          const int count = a.split->segment_count[hub];
          float m_row = -CUDART_INF_F;
          for (int k = 0; k < count; ++k) m_row = fmaxf(m_row, __ldcg(&a.split->partial[first + k][0]));
          float l_row = 0.f;
          for (int k = 0; k < count; ++k) {
            const float l_k = __ldcg(&a.split->partial[first + k][1]);
            if (l_k > 0.f) l_row += l_k * expf(__ldcg(&a.split->partial[first + k][0]) - m_row);
          }
          for (int i = tid; i < f; i += blockDim.x) {
            float t = 0.f;
            for (int k = 0; k < count; ++k) {
              const float l_k = __ldcg(&a.split->partial[first + k][1]);
              const float weight = l_k > 0.f ? expf(__ldcg(&a.split->partial[first + k][0]) - m_row) : 0.f;
              t = fmaf(__ldcg(&a.split->partial[first + k][2 + i]), weight, t);
            }
            st_stream1(a.out + static_cast<size_t>(row) * f + i, l_row > 0.f ? t / l_row : 0.f);
          }
        }
      }
    }
  }
  const int n_short = a.header->n_short;
  const int n_medium = n_light - n_short;  // light rows of 32 edges or more
  if (n_medium > 0) {
    const int* light = a.order + n_hub;
    for (;;) {
      const unsigned long long it = warp_next(&a.header->counter[1]);
      if (it >= static_cast<unsigned long long>(n_medium)) break;
      const int row = light[it];
      float m_run = -CUDART_INF_F, l_run = 0.f;
      float acc[NV][VW];
#pragma unroll
      for (int v = 0; v < NV; ++v)
#pragma unroll
        for (int i = 0; i < VW; ++i) acc[v][i] = 0.f;
      attention_batches<VW, G, NV, U>(a, row, a.crow[row], a.crow[row + 1], 32ll, lane, pol_keep, pol_stream, m_run,
                                      l_run, acc);
#pragma unroll
      for (int o = G; o < 32; o <<= 1)
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[v][i] += __shfl_xor_sync(kFull, acc[v][i], o);
      if (sub == 0) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const int fo = VW * (l + G * v);
          if (fo < f) {
            float r[VW];
#pragma unroll
            for (int i = 0; i < VW; ++i) r[i] = acc[v][i] * inv;
            VecIO<VW>::store(a.out + static_cast<size_t>(row) * f + fo, r);
          }
        }
      }
    }
  }
}

// Queue 2: light rows of fewer than 32 edges - nine rows in ten of a power-law graph, and bound by the
// chain of dependent memory round trips (row pointers -> columns -> K rows -> V rows -> output), not by
// bandwidth.  A warp grabs 32 of them (ids and row pointers with one coalesced load each) and walks
// them 32/G rows at a time: each group of G lanes - the lanes that together hold one feature row - owns
// a row of its own, reads that row's columns itself, and for every edge fetches the K row AND the V
// row in the same step (the V row does not depend on the score), EDGES edges per step; scores, running
// maximum, running sum and the rescaled accumulator then stay inside the group, so nothing is reduced
// across groups and every group stores its own output row.  The columns of the next rows are fetched
// while the current ones are gathered.  A kernel of its own, launched as a programmatic dependent of
// the main kernel: it fills the SMs while the longest hub rows finish.
template <int VW, int G, int NV, int EDGES>
__global__ void __launch_bounds__(512) attention_short_kernel(const AttentionArgs a) {
  constexpr int RPW = 32 / G;                      // rows a warp processes side by side
  constexpr int CREG = (kShortDegree + G - 1) / G;  // column registers per lane: G columns each
  const int lane = threadIdx.x & 31;
  const int l = lane % G;
  const int sub = lane / G;
  const uint64_t pol_keep = policy_evict_last();
  const uint64_t pol_stream = policy_evict_first();
  const int n_hub = a.header->n_hub;
  const int n_short = a.header->n_short;
  const int n_medium = a.header->n_light - n_short;
  const int f = a.f;
  if (n_short > 0) {
    const int* shorts = a.order + n_hub + n_medium;
    const int n_batches = (n_short + 31) / 32;
    bool fvalid[NV];
    int foff[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      foff[v] = VW * (l + G * v);
      fvalid[v] = foff[v] < f;
    }
    for (;;) {
      const unsigned long long it = warp_next(&a.header->counter[2]);
      if (it >= static_cast<unsigned long long>(n_batches)) break;
      const int first = static_cast<int>(it) * 32;
      const int n_here = n_short - first < 32 ? n_short - first : 32;
      int row_l = 0;
      long long s_l = 0;
      int d_l = 0;
      if (lane < n_here) {
        row_l = shorts[first + lane];
        s_l = a.crow[row_l];
        d_l = static_cast<int>(a.crow[row_l + 1] - s_l);
      }
      // columns of the first rows: lane l of a group holds columns l, l + G, ... of the group's row
      int c_next[CREG];
      {
        const long long s0 = __shfl_sync(kFull, s_l, sub);
        const int d0 = __shfl_sync(kFull, d_l, sub);
#pragma unroll
        for (int k = 0; k < CREG; ++k)
          c_next[k] = (l + k * G < d0) ? static_cast<int>(ld_index(a.col + s0 + l + k * G, pol_stream)) : 0;
      }
      for (int r0 = 0; r0 < n_here; r0 += RPW) {
        const int mine = r0 + sub;                      // this group's row of the batch (may be past the end)
        const int src = mine < 32 ? mine : 31;
        const int row = __shfl_sync(kFull, row_l, src);
        const int cnt_any = __shfl_sync(kFull, d_l, src);  // every lane takes part in the shuffle
        const int cnt = mine < n_here ? cnt_any : 0;
        int c_cur[CREG];
#pragma unroll
        for (int k = 0; k < CREG; ++k) c_cur[k] = c_next[k];
        if (r0 + RPW < n_here) {  // warp-uniform
          const int ahead = r0 + RPW + sub < 32 ? r0 + RPW + sub : 31;
          const long long s1 = __shfl_sync(kFull, s_l, ahead);
          const int d1_any = __shfl_sync(kFull, d_l, ahead);
          const int d1 = r0 + RPW + sub < n_here ? d1_any : 0;
#pragma unroll
          for (int k = 0; k < CREG; ++k)
            c_next[k] = (l + k * G < d1) ? static_cast<int>(ld_index(a.col + s1 + l + k * G, pol_stream)) : 0;
        }
        float q[NV][VW];
        if (cnt > 0) {
          const float* qrow = a.q + static_cast<size_t>(row) * f;
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            if (fvalid[v]) {
              VecIO<VW>::load(q[v], qrow + foff[v], pol_stream);
            } else {
#pragma unroll
              for (int i = 0; i < VW; ++i) q[v][i] = 0.f;
            }
          }
        }
        float m_run = -CUDART_INF_F, l_run = 0.f;
        float acc[NV][VW];
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) acc[v][i] = 0.f;
        const int longest = __reduce_max_sync(kFull, cnt);  // the shuffles below need every lane
        for (int j = 0; j < longest; j += EDGES) {
          float kv[EDGES][NV][VW], vv[EDGES][NV][VW];
          bool ok[EDGES];
#pragma unroll
          for (int u = 0; u < EDGES; ++u) {
            const int e = j + u;
            int c = 0;
#pragma unroll
            for (int k = 0; k < CREG; ++k) {
              const int got = __shfl_sync(kFull, c_cur[k], sub * G + ((e - k * G) & (G - 1)));
              if (e >= k * G && e < (k + 1) * G) c = got;
            }
            ok[u] = e < cnt;
            const float* krow = a.k + static_cast<size_t>(c) * f;
            const float* vrow = a.v + static_cast<size_t>(c) * f;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
              if (ok[u] && fvalid[v]) {
                VecIO<VW>::load(kv[u][v], krow + foff[v], pol_keep);
                VecIO<VW>::load(vv[u][v], vrow + foff[v], pol_keep);
              } else {
#pragma unroll
                for (int i = 0; i < VW; ++i) kv[u][v][i] = vv[u][v][i] = 0.f;
              }
            }
          }
          float score[EDGES];
          float m_new = m_run;
#pragma unroll
          for (int u = 0; u < EDGES; ++u) {
            float d = 0.f;
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
              for (int i = 0; i < VW; ++i) d = fmaf(q[v][i], kv[u][v][i], d);
#pragma unroll
            for (int o = G / 2; o >= 1; o >>= 1) d += __shfl_xor_sync(kFull, d, o);  // stays inside the group
            score[u] = ok[u] ? d * a.scale : -CUDART_INF_F;
            m_new = fmaxf(m_new, score[u]);
          }
          if (m_new > -CUDART_INF_F) {  // this group still has edges in the step
            const float rescale = expf(m_run - m_new);  // exp(-inf) = 0 on the first step
            l_run *= rescale;
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
              for (int i = 0; i < VW; ++i) acc[v][i] *= rescale;
#pragma unroll
            for (int u = 0; u < EDGES; ++u) {
              const float p = ok[u] ? expf(score[u] - m_new) : 0.f;
              l_run += p;
#pragma unroll
              for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int i = 0; i < VW; ++i) acc[v][i] = fmaf(p, vv[u][v][i], acc[v][i]);
            }
            m_run = m_new;
          }
        }
        if (mine < n_here) {
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            if (fvalid[v]) {
              float out_v[VW];
#pragma unroll
              for (int i = 0; i < VW; ++i) out_v[i] = acc[v][i] * inv;
              VecIO<VW>::store(a.out + static_cast<size_t>(row) * f + foff[v], out_v);
            }
          }
        }
      }
    }
  }
  pdl_wait_for_primary();  // do not complete before the main kernel has
}

template <int VW, int G, int NV, int U>
static int launch_attention_instance(const AttentionArgs& args, int warps, cudaStream_t stream, int device) {
  constexpr int FT = VW * G * NV;
  auto kernel = attention_kernel<VW, G, NV, U>;
  const int threads = warps * 32;
  const size_t smem = 16 + 128 + size_t(4) * warps * FT;
  if (smem > 48 * 1024)
    ASG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  int per_sm = 0;
  ASG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem));
  if (per_sm < 1) per_sm = 1;
  if (args.split != nullptr) {  // every call: the completion counters start from zero
    attention_split_plan<<<1, 32, 0, stream>>>(args);
    ASG_CUDA(cudaGetLastError());
  }
  kernel<<<sm_count(device) * per_sm, threads, smem, stream>>>(args);
  ASG_CUDA(cudaGetLastError());
  // edges gathered per step in the short-row kernel: K and V rows of 4 edges (2 when a lane already
  // holds more than one vector per row) keep the kernel under 128 registers; 2 edges per step measured
  // 25 % slower on the 169,343-row benchmark graph (0.47 against 0.38 ms)
  auto short_kernel = attention_short_kernel<VW, G, NV, (NV > 1 ? 2 : 4)>;
  int short_per_sm = 0;
  ASG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&short_per_sm, short_kernel, threads, 0));
  if (short_per_sm < 1) short_per_sm = 1;
  ASG_CUDA(launch_overlapped(short_kernel, sm_count(device) * short_per_sm, threads, 0, stream, args));
  return ASG_OK;
}

static bool aligned_to(const void* p, size_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; }

constexpr int kAttentionLoadsInFlight = 8;  // gather instructions issued per lane before their results are used

static int launch_attention(const AttentionArgs& args, int vw, int warps, cudaStream_t stream, int device) {
  constexpr int U = kAttentionLoadsInFlight;
  const int f = args.f;
  if (vw == 8) {
    if (f <= 32) return launch_attention_instance<8, 4, 1, U / 2>(args, warps, stream, device);
    if (f <= 64) return launch_attention_instance<8, 8, 1, U / 2>(args, warps, stream, device);
    if (f <= 128) return launch_attention_instance<8, 16, 1, U / 2>(args, warps, stream, device);
    if (f <= 256) return launch_attention_instance<8, 32, 1, U / 2>(args, warps, stream, device);
    return launch_attention_instance<8, 32, 2, U / 4>(args, warps, stream, device);
  }
  if (vw == 4) {
    if (f <= 32) return launch_attention_instance<4, 8, 1, U>(args, warps, stream, device);
    if (f <= 64) return launch_attention_instance<4, 16, 1, U>(args, warps, stream, device);
    if (f <= 128) return launch_attention_instance<4, 32, 1, U>(args, warps, stream, device);
    if (f <= 256) return launch_attention_instance<4, 32, 2, U / 2>(args, warps, stream, device);
    return launch_attention_instance<4, 32, 4, U / 4>(args, warps, stream, device);
  }
  if (f <= 32) return launch_attention_instance<1, 32, 1, U>(args, warps, stream, device);
  if (f <= 64) return launch_attention_instance<1, 32, 2, U / 2>(args, warps, stream, device);
  if (f <= 128) return launch_attention_instance<1, 32, 4, U / 4>(args, warps, stream, device);
  if (f <= 256) return launch_attention_instance<1, 32, 8, U / 4>(args, warps, stream, device);
  return launch_attention_instance<1, 32, 16, 1>(args, warps, stream, device);
}

}  // namespace asg

extern "C" {

int asg_csr_row_softmax(const int64_t* crow, const float* scores, float* probs, int64_t n_rows, int64_t nnz,
                        int warps_per_block, int64_t hub_threshold, unsigned flags, void* workspace,
                        size_t workspace_bytes, void* stream_ptr) {
  using namespace asg;
  ASG_REQUIRE(n_rows >= 0 && nnz >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(n_rows <= 2147483647ll - 2048, ASG_ERANGE, "n_rows exceeds the kernel index range");
  ASG_REQUIRE(warps_per_block == 2 || warps_per_block == 4 || warps_per_block == 8 || warps_per_block == 16,
              ASG_EINVAL, "warps_per_block must be 2, 4, or 8");
  if (n_rows == 0 || nnz == 0) return ASG_OK;
  ASG_REQUIRE(crow != nullptr && scores != nullptr && probs != nullptr, ASG_EINVAL,
              "crow, scores and probs must not be null");
  if (int rc = check_workspace(workspace, workspace_bytes, n_rows)) return rc;
  DeviceGuard guard(probs);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (flags & ASG_FLAG_PLAN_READY) {
    if (int rc = reset_counters(workspace, stream)) return rc;
  } else {
    if (int rc = plan_build(crow, n_rows, hub_threshold, workspace, stream)) return rc;
  }
  SoftmaxArgs args;
  args.crow = crow;
  args.scores = scores;
  args.probs = probs;
  args.header = static_cast<Header*>(workspace);
  args.order = reinterpret_cast<const int*>(static_cast<const char*>(workspace) + order_offset());
  const int threads = warps_per_block * 32;
  int per_sm = 0;
  ASG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, csr_softmax_kernel, threads, 0));
  if (per_sm < 1) per_sm = 1;
  csr_softmax_kernel<<<sm_count(guard.target) * per_sm, threads, 0, stream>>>(args);
  ASG_CUDA(cudaGetLastError());
  return ASG_OK;
}

size_t asg_attention_workspace_bytes(int64_t n_rows) {
  if (n_rows < 0) n_rows = 0;
  return asg::workspace_bytes(n_rows) + sizeof(asg::SplitArea);
}

int asg_csr_attention(const int64_t* crow, const int64_t* col, const float* q, const float* k, const float* v,
                      float* out, int64_t n_rows, int64_t nnz, int64_t f, float scale, int warps_per_block,
                      int64_t hub_threshold, unsigned flags, void* workspace, size_t workspace_size,
                      void* stream_ptr) {
  using namespace asg;
  ASG_REQUIRE(n_rows >= 0 && nnz >= 0 && f >= 0, ASG_EINVAL, "sizes must be non-negative");
  ASG_REQUIRE(n_rows <= 2147483647ll - 2048, ASG_ERANGE, "n_rows exceeds the kernel index range");
  ASG_REQUIRE(f <= 512, ASG_ERANGE, "the fused attention kernel holds at most 512 features per row");
  ASG_REQUIRE(warps_per_block == 2 || warps_per_block == 4 || warps_per_block == 8 || warps_per_block == 16,
              ASG_EINVAL, "warps_per_block must be 2, 4, or 8");
  if (n_rows == 0 || f == 0) return ASG_OK;
  ASG_REQUIRE(crow != nullptr && q != nullptr && k != nullptr && v != nullptr && out != nullptr, ASG_EINVAL,
              "crow, query, key, value and out must not be null");
  ASG_REQUIRE(nnz == 0 || col != nullptr, ASG_EINVAL, "col must not be null");
  if (int rc = check_workspace(workspace, workspace_size, n_rows)) return rc;
  DeviceGuard guard(out);
  ASG_CUDA(guard.status);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (flags & ASG_FLAG_PLAN_READY) {
    if (int rc = reset_counters(workspace, stream)) return rc;
  } else {
    if (int rc = plan_build(crow, n_rows, hub_threshold, workspace, stream)) return rc;
  }
  int vw = 1;
  if (!(flags & ASG_FLAG_NO_VEC4)) {
    const bool a32 = aligned_to(q, 32) && aligned_to(k, 32) && aligned_to(v, 32) && aligned_to(out, 32);
    const bool a16 = aligned_to(q, 16) && aligned_to(k, 16) && aligned_to(v, 16) && aligned_to(out, 16);
    if (f % 8 == 0 && a32) vw = 8;
    else if (f % 4 == 0 && a16) vw = 4;
  }
  AttentionArgs args;
  args.crow = crow;
  args.col = col;
  args.q = q;
  args.k = k;
  args.v = v;
  args.out = out;
  args.header = static_cast<Header*>(workspace);
  args.order = reinterpret_cast<const int*>(static_cast<const char*>(workspace) + order_offset());
  // the split area is used when the caller's workspace has room for it (asg_attention_workspace_bytes)
  const size_t split_at = workspace_bytes(n_rows);
  args.split = workspace_size >= split_at + sizeof(SplitArea)
                   ? reinterpret_cast<SplitArea*>(static_cast<char*>(workspace) + split_at)
                   : nullptr;
  args.f = static_cast<int>(f);
  args.scale = scale;
  return launch_attention(args, vw, warps_per_block, stream, guard.target);
}

}  // extern "C"
