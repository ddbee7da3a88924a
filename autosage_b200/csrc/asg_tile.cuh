// Feature-tile geometry and vector load/store helpers shared by the SpMM, SDDMM and attention
// kernels.
//
// A warp covers one feature tile of FT = VW*G*NV floats of a dense row per pass:
//   VW  floats per load instruction and lane (1 = scalar, 4 = 128-bit, 8 = 256-bit loads)
//   G   lanes that together cover the tile for one edge ("lane group")
//   NV  vectors each lane of the group owns
// so a warp handles EPI = 32/G edges per load instruction.  Lane l of a group owns the floats
//   tile_base + VW*(l + G*v) + i,   v < NV, i < VW.
#pragma once

#include "asg_common.cuh"

namespace asg {

#ifdef __CUDACC__

template <int VW>
struct VecIO;

template <>
struct VecIO<1> {
  static __device__ __forceinline__ void load(float (&d)[1], const float* p, uint64_t pol) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(d[0]) : "l"(p), "l"(pol));
  }
  static __device__ __forceinline__ void load_plain(float (&d)[1], const float* p) { d[0] = *p; }
  static __device__ __forceinline__ void store(float* p, const float (&d)[1]) { st_stream1(p, d[0]); }
};

template <>
struct VecIO<4> {
  static __device__ __forceinline__ void load(float (&d)[4], const float* p, uint64_t pol) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "l"(p), "l"(pol));
  }
  static __device__ __forceinline__ void load_plain(float (&d)[4], const float* p) {
    float4 t = *reinterpret_cast<const float4*>(p);
    d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&d)[4]) {
    st_stream4(p, make_float4(d[0], d[1], d[2], d[3]));
  }
};

template <>
struct VecIO<8> {
  // 256-bit global load (sm_100): one instruction moves 32 bytes per lane.
  static __device__ __forceinline__ void load(float (&d)[8], const float* p, uint64_t pol) {
    asm volatile(
        "ld.global.nc.L1::no_allocate.L2::cache_hint.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8], %9;"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]), "=f"(d[4]), "=f"(d[5]), "=f"(d[6]), "=f"(d[7])
        : "l"(p), "l"(pol));
  }
  static __device__ __forceinline__ void load_plain(float (&d)[8], const float* p) {
    float4 a = reinterpret_cast<const float4*>(p)[0];
    float4 b = reinterpret_cast<const float4*>(p)[1];
    d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w;
    d[4] = b.x; d[5] = b.y; d[6] = b.z; d[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&d)[8]) {
    st_stream4(p, make_float4(d[0], d[1], d[2], d[3]));
    st_stream4(p + 4, make_float4(d[4], d[5], d[6], d[7]));
  }
};

__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t policy_evict_normal() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ long long ld_index(const int64_t* p, uint64_t pol) {
  long long v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b64 %0, [%1], %2;" : "=l"(v) : "l"(p), "l"(pol));
  return v;
}
__device__ __forceinline__ float ld_weight(const float* p, uint64_t pol) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol));
  return v;
}

#endif  // __CUDACC__

// Host-side choice of the tile geometry for a requested tile width.
struct TileShape {
  int vw, g, nv, ft;
};

inline TileShape make_tile(int vw, int feature_tile) {
  TileShape t;
  t.vw = vw;
  t.ft = feature_tile;
  int lanes = feature_tile / vw;
  t.g = lanes < 32 ? lanes : 32;
  t.nv = feature_tile / (vw * t.g);
  return t;
}

}  // namespace asg

namespace asg {
#ifdef __CUDACC__

// Dot products of one dense row held in registers (q) with up to 32 gathered rows of `mat`.
// Lane `lane` holds in c_l the column index of edge `lane` of the batch; `cnt` edges are valid.
// Load instruction i (0 <= i < G) serves edges i*EPI + sub, one per lane group; its partial dot
// product is added to part[i].  U instructions are issued before their results are used.
// CHECKED = false is the fast form for a full batch (cnt == 32) inside a full feature tile: no
// predicates and no zero fill.
template <int VW, int G, int NV, int U, bool CHECKED>
__device__ __forceinline__ void batch_dots_impl(const float* __restrict__ mat, int f, int c_l, int cnt, int sub,
                                                const float (&q)[NV][VW], const bool (&fvalid)[NV],
                                                const int (&foff)[NV], uint64_t pol, float (&part)[G]) {
  constexpr int EPI = 32 / G;
  constexpr int UU = U < G ? U : G;
#pragma unroll
  for (int i0 = 0; i0 < G; i0 += UU) {
    if (!CHECKED || i0 * EPI < cnt) {
      float kv[UU][NV][VW];
#pragma unroll
      for (int u = 0; u < UU; ++u) {
        const int src = (i0 + u) * EPI + sub;
        const int c = __shfl_sync(kFull, c_l, src);
        const bool ok = !CHECKED || src < cnt;
        const float* krow = mat + static_cast<size_t>(c) * f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          if (!CHECKED || (ok && fvalid[v])) {
            VecIO<VW>::load(kv[u][v], krow + foff[v], pol);
          } else {
#pragma unroll
            for (int i = 0; i < VW; ++i) kv[u][v][i] = 0.f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UU; ++u) {
        float d = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < VW; ++i) d = fmaf(q[v][i], kv[u][v][i], d);
        part[i0 + u] += d;
      }
    }
  }
}

// FAST_PATH adds the unchecked form for full batches; it costs registers (occupancy), which pays
// in the attention kernel but not in the SDDMM kernel (measured), so the caller chooses.
template <int VW, int G, int NV, int U, bool FAST_PATH>
__device__ __forceinline__ void batch_dots(const float* __restrict__ mat, int f, int c_l, int cnt, int sub,
                                           const float (&q)[NV][VW], const bool (&fvalid)[NV],
                                           const int (&foff)[NV], uint64_t pol, float (&part)[G]) {
  if (!FAST_PATH) {
    batch_dots_impl<VW, G, NV, U, true>(mat, f, c_l, cnt, sub, q, fvalid, foff, pol, part);
    return;
  }
  bool lane_full = true;
#pragma unroll
  for (int v = 0; v < NV; ++v) lane_full = lane_full && fvalid[v];
  if (cnt == 32 && __all_sync(kFull, lane_full)) {
    batch_dots_impl<VW, G, NV, U, false>(mat, f, c_l, cnt, sub, q, fvalid, foff, pol, part);
  } else {
    batch_dots_impl<VW, G, NV, U, true>(mat, f, c_l, cnt, sub, q, fvalid, foff, pol, part);
  }
}

// Sum part[i] over the G lanes of a group so that lane l of the group ends with the total of
// part[l] (a reduce-scatter by recursive halving: G-1 shuffles for G values).
template <int G>
__device__ __forceinline__ float group_reduce_scatter(float (&part)[G], int l) {
#pragma unroll
  for (int h = G / 2; h >= 1; h >>= 1) {
    const bool upper = (l & h) != 0;
#pragma unroll
    for (int i = 0; i < h; ++i) {
      const float send = upper ? part[i] : part[i + h];
      const float keep = upper ? part[i + h] : part[i];
      part[i] = keep + __shfl_xor_sync(kFull, send, h);
    }
  }
  return part[0];
}

#endif  // __CUDACC__
}  // namespace asg
