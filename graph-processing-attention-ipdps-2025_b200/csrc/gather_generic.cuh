// FP32 gather path for head dimensions the specialised kernels do not cover: any d in [1, 1024].
//
// The reference accepts every embedded dimension up to its thread count (sp_flatt_csr_kernel.cu:183-184: "does not
// work for sizes greater than number of threads", i.e. d <= 1024; :260-266 rejects only what leaves no room for
// one key in shared memory). The kernels of gather_kernels.cuh are compiled for d in {16, 32, 64, 128}, where a
// key row is split over a power-of-two group of lanes; everything else (48, 80, 96, 256, odd sizes, ...) runs
// here: one warp per query row, the WHOLE warp on one key at a time, each lane holding NC pieces of VW floats of
// the row (piece c of lane l = elements [(c*32 + l)*VW, +VW): consecutive lanes read consecutive memory).
//   VW = 4: 128-bit loads, needs d % 4 == 0        VW = 1: scalar loads, any d
// Same visiting order, same online-softmax recurrence and state merge as the specialised path; rows with more
// than kHeavyRowSlots slots are walked by all warps of the CTA together. Accuracy class: FP32 (1e-5).
#pragma once
#include <type_traits>

#include "gather_kernels.cuh"
#include "gather_kernels_16.cuh"
#include "spfa_common.cuh"

namespace spfa {

constexpr int kGenericMaxD = 1024;

template <int VW, int NC>
struct GenRow {
  float v[NC][VW];
};

// Element type of the tensors in memory: float, __half or __nv_bfloat16 (arithmetic is fp32 throughout).
template <class T> struct Elem {
  static __device__ __forceinline__ float up(T x) { return Cvt16<T>::up1(x); }
  static __device__ __forceinline__ T down(float x) { return Cvt16<T>::down1(x); }
};
template <> struct Elem<float> {
  static __device__ __forceinline__ float up(float x) { return x; }
  static __device__ __forceinline__ float down(float x) { return x; }
};

// VW elements per piece: 4 (fp32) or 8 (16-bit) when the pieces are 128-bit loads, 1 for scalar loads.
template <class T, int VW, int NC>
__device__ __forceinline__ void gen_load(const T* __restrict__ p, int d, int lane, GenRow<VW, NC>& r) {
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * 32 + lane) * VW;
    if (e < d) {
      if (VW == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(p + e));
        r.v[c][0] = t.x;
        r.v[c][1 % VW] = t.y;
        r.v[c][2 % VW] = t.z;
        r.v[c][3 % VW] = t.w;
      } else if (VW == 8) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(p + e));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = Cvt16<typename std::conditional<std::is_same<T, float>::value, __half, T>::type>::up(w[i]);
          r.v[c][(2 * i) % VW] = f.x;
          r.v[c][(2 * i + 1) % VW] = f.y;
        }
      } else {
        r.v[c][0] = Elem<T>::up(__ldg(p + e));
      }
    } else {
#pragma unroll
      for (int i = 0; i < VW; ++i) r.v[c][i] = 0.f;
    }
  }
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(kFullMask, x, o);
  return x;
}

template <int VW, int NC>
struct GenAcc {
  float m, l;
  GenRow<VW, NC> acc;
  __device__ __forceinline__ void clear() {
    m = neg_inf();
    l = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
      for (int i = 0; i < VW; ++i) acc.v[c][i] = 0.f;
  }
};

// Slots [t0, t1) of one row into the warp's state. U keys are in flight at a time (U = 1 for the widest rows, whose
// pieces already fill the register file).
template <class T, int VW, int NC, int U, class Cols>
__device__ __forceinline__ void gen_accumulate(const Cols& cols, const typename Cols::Row& row, int64_t t0, int64_t t1,
                                               const GenRow<VW, NC>& q, const T* __restrict__ K,
                                               const T* __restrict__ V, int d, float scale, int lane,
                                               GenAcc<VW, NC>& st) {
  for (int64_t base = t0; base < t1; base += 32) {
    const int64_t tl = base + lane;
    const int32_t c_lane = (tl < t1) ? cols.slot(row, tl) : -1;
    const int nb = (t1 - base < 32) ? (int)(t1 - base) : 32;
#pragma unroll 1
    for (int j0 = 0; j0 < nb; j0 += U) {
      GenRow<VW, NC> k[U], v[U];
      float s[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int32_t c = (j0 + u < 32) ? __shfl_sync(kFullMask, c_lane, (j0 + u) & 31) : -1;
        if (c >= 0) {  // warp-uniform
          gen_load<T, VW, NC>(K + (size_t)c * d, d, lane, k[u]);
          gen_load<T, VW, NC>(V + (size_t)c * d, d, lane, v[u]);
          float p = 0.f;
#pragma unroll
          for (int cc = 0; cc < NC; ++cc)
#pragma unroll
            for (int i = 0; i < VW; ++i) p = fmaf(q.v[cc][i], k[u].v[cc][i], p);
          s[u] = p;
        } else {
          s[u] = 0.f;
#pragma unroll
          for (int cc = 0; cc < NC; ++cc)
#pragma unroll
            for (int i = 0; i < VW; ++i) v[u].v[cc][i] = 0.f;
        }
        s[u] = (c >= 0) ? warp_sum(s[u]) * scale : neg_inf();
      }
      float mc = s[0];
#pragma unroll
      for (int u = 1; u < U; ++u) mc = fmaxf(mc, s[u]);
      const float m_new = fmaxf(st.m, mc);
      const float m_safe = (m_new == neg_inf()) ? 0.f : m_new;
      const float corr = fast_exp2((st.m - m_safe) * kLog2e);
      float p[U], ps = 0.f;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        p[u] = fast_exp2((s[u] - m_safe) * kLog2e);
        ps += p[u];
      }
#pragma unroll
      for (int cc = 0; cc < NC; ++cc)
#pragma unroll
        for (int i = 0; i < VW; ++i) {
          float a = st.acc.v[cc][i] * corr;
#pragma unroll
          for (int u = 0; u < U; ++u) a = fmaf(p[u], v[u].v[cc][i], a);
          st.acc.v[cc][i] = a;
        }
      st.l = fmaf(st.l, corr, ps);
      st.m = m_new;
    }
  }
}

// Fold (m_loc, l_loc, un-normalised acc) into the caller's state, as store_row of the specialised path
// (sp_flatt_csr_kernel.cu:162-194 applied once to the whole row).
template <class T, int VW, int NC>
__device__ __forceinline__ void gen_store(const GenAcc<VW, NC>& st, T* __restrict__ m, T* __restrict__ l,
                                          T* __restrict__ O, int64_t r, int d, int lane) {
  const float m_in = Elem<T>::up(m[r]), l_in = Elem<T>::up(l[r]);
  const float m_out = fmaxf(m_in, st.m);
  const float a = l_in * fast_exp2((m_in - m_out) * kLog2e);
  const float b = fast_exp2((st.m - m_out) * kLog2e);
  const float l_out = fmaf(st.l, b, a);
  const float inv = 1.0f / l_out;
  T* op = O + (size_t)r * d;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int e = (c * 32 + lane) * VW;
    if (e < d) {
#pragma unroll
      for (int i = 0; i < VW; ++i) op[e + i] = Elem<T>::down((a * Elem<T>::up(op[e + i]) + b * st.acc.v[c][i]) * inv);
    }
  }
  __syncwarp();
  if (lane == 0) {
    m[r] = Elem<T>::down(m_out);
    l[r] = Elem<T>::down(l_out);
  }
}

template <class T, int VW, int NC, class Cols>
__global__ void __launch_bounds__(kRowWarps * 32)
gather_rows_generic_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                           T* __restrict__ m, T* __restrict__ l, T* __restrict__ O, const Cols cols,
                           int64_t row_begin, int64_t n_rows, int use_nan, float scale, int d) {
  constexpr int U = (VW * NC <= 8) ? 4 : 1;
  extern __shared__ float gen_smem[];  // heavy rows: [kRowWarps][d] partial accumulators
  __shared__ float s_ml[kRowWarps][2];
  __shared__ int s_heavy[kRowWarps];
  __shared__ int s_n_heavy;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_n_heavy = 0;
  __syncthreads();
  const int64_t r = (int64_t)blockIdx.x * kRowWarps + warp;
  if (r < n_rows) {
    const typename Cols::Row row = cols.open(r, row_begin + r);
    if (row.n <= 0) {
      if (Cols::kNanFillEmpty && use_nan)
        for (int e = lane; e < d; e += 32) O[(size_t)r * d + e] = Elem<T>::down(__int_as_float(0x7fc00000));
    } else if (row.n > kHeavyRowSlots) {
      if (lane == 0) s_heavy[atomicAdd(&s_n_heavy, 1)] = warp;
    } else {
      GenRow<VW, NC> q;
      gen_load<T, VW, NC>(Q + (size_t)r * d, d, lane, q);
      GenAcc<VW, NC> st;
      st.clear();
      gen_accumulate<T, VW, NC, U, Cols>(cols, row, 0, row.n, q, K, V, d, scale, lane, st);
      if (st.l > 0.f) gen_store<T, VW, NC>(st, m, l, O, r, d, lane);
    }
  }
  __syncthreads();
  const int n_heavy = s_n_heavy;  // uniform over the CTA
  for (int h = 0; h < n_heavy; ++h) {
    const int64_t rh = (int64_t)blockIdx.x * kRowWarps + s_heavy[h];
    const typename Cols::Row row = cols.open(rh, row_begin + rh);
    int64_t per = (row.n + kRowWarps - 1) / kRowWarps;
    per = (per + 31) / 32 * 32;
    const int64_t t0 = (int64_t)warp * per;
    int64_t t1 = t0 + per;
    if (t1 > row.n) t1 = row.n;
    GenAcc<VW, NC> st;
    st.clear();
    if (t0 < t1) {
      GenRow<VW, NC> q;
      gen_load<T, VW, NC>(Q + (size_t)rh * d, d, lane, q);
      gen_accumulate<T, VW, NC, U, Cols>(cols, row, t0, t1, q, K, V, d, scale, lane, st);
    }
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int e = (c * 32 + lane) * VW;
      if (e < d) {
#pragma unroll
        for (int i = 0; i < VW; ++i) gen_smem[(size_t)warp * d + e + i] = st.acc.v[c][i];
      }
    }
    if (lane == 0) {
      s_ml[warp][0] = st.m;
      s_ml[warp][1] = st.l;
    }
    __syncthreads();
    if (warp == 0) {  // fold the warps' states in slot order
      GenAcc<VW, NC> tot;
      tot.clear();
      for (int wv = 0; wv < kRowWarps; ++wv) {
        const float mo = s_ml[wv][0], lo = s_ml[wv][1];
        const float mn = fmaxf(tot.m, mo);
        const float ms = (mn == neg_inf()) ? 0.f : mn;
        const float c1 = fast_exp2((tot.m - ms) * kLog2e), c2 = fast_exp2((mo - ms) * kLog2e);
        tot.l = tot.l * c1 + lo * c2;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int e = (c * 32 + lane) * VW;
          if (e < d) {
#pragma unroll
            for (int i = 0; i < VW; ++i) tot.acc.v[c][i] = tot.acc.v[c][i] * c1 + gen_smem[(size_t)wv * d + e + i] * c2;
          }
        }
        tot.m = mn;
      }
      if (tot.l > 0.f) gen_store<T, VW, NC>(tot, m, l, O, rh, d, lane);
    }
    __syncthreads();
  }
}

// ---- Global-no-local with both row kinds in one functor (the specialised path splits the listed rows over many
//      warps with a scratch buffer; here a listed row is simply a long row walked by its CTA) ----------------------
struct GnlAnyRowCols {
  GnlCols list;            // rows outside the list: listed keys outside the window
  GnlGlobalRowCols strip;  // rows in the list: every key outside the window
  static constexpr bool kNanFillEmpty = false;
  struct Row { bool is_global; GnlCols::Row a; GnlGlobalRowCols::Row b; int64_t n; };
  __device__ __forceinline__ Row open(int64_t r, int64_t i) const {
    Row row;
    row.is_global = (__ldg(list.global_bits + (i >> 5)) >> (i & 31)) & 1u;
    row.b = strip.open(r, i);
    row.a.lo = row.b.lo;
    row.a.hi = row.b.lo + row.b.width;
    row.a.n = list.nG;
    row.n = row.is_global ? row.b.n : list.nG;
    return row;
  }
  __device__ __forceinline__ int32_t slot(const Row& row, int64_t t) const {
    return row.is_global ? strip.slot(row.b, t) : list.slot(row.a, t);
  }
};

}  // namespace spfa
