// Gather path with 16-bit storage: Q, K, V, O, m, l are __half or __nv_bfloat16 in memory, all arithmetic is fp32.
//
// The reference instantiates its kernels for Half as well (AT_DISPATCH_FLOATING_TYPES_AND_HALF,
// sp_flatt_csr_kernel.cu:270) and there accumulates in half; here only the loads and stores are 16-bit, so results
// are at least as accurate as the reference's, and an HBM-bound gather moves half the bytes of the fp32 path.
// Same structure as gather_kernels.cuh: one warp per query row, a key row is covered by LPK = D/8 lanes with one
// 128-bit load each (8 elements), KPS = 32/LPK keys per warp step, four keys in flight per lane group, online
// softmax state per group, groups merged once per row, long rows walked by all warps of the CTA.
// D in {32, 64, 128} (LPK >= 4); other sizes take the generic kernel (gather_generic.cuh) with 16-bit loads.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gather_kernels.cuh"
#include "spfa_common.cuh"

namespace spfa {

template <class T> struct Cvt16;
template <> struct Cvt16<__half> {
  static __device__ __forceinline__ float2 up(uint32_t x) { return __half22float2(*reinterpret_cast<const __half2*>(&x)); }
  static __device__ __forceinline__ uint32_t down(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ float up1(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half down1(float x) { return __float2half_rn(x); }
};
template <> struct Cvt16<__nv_bfloat16> {
  static __device__ __forceinline__ float2 up(uint32_t x) {  // a bfloat16 is the upper half of a float
    return make_float2(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
  }
  static __device__ __forceinline__ uint32_t down(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ float up1(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 down1(float x) { return __float2bfloat16_rn(x); }
};

struct Vec8 {
  float v[8];
};

template <class T>
__device__ __forceinline__ Vec8 ldg8(const T* p) {  // 16 bytes = 8 elements, read-only path
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  Vec8 r;
  float2 f;
  f = Cvt16<T>::up(u.x); r.v[0] = f.x; r.v[1] = f.y;
  f = Cvt16<T>::up(u.y); r.v[2] = f.x; r.v[3] = f.y;
  f = Cvt16<T>::up(u.z); r.v[4] = f.x; r.v[5] = f.y;
  f = Cvt16<T>::up(u.w); r.v[6] = f.x; r.v[7] = f.y;
  return r;
}

__device__ __forceinline__ float dot8(const Vec8& q, const Vec8& k) {
  float p = q.v[0] * k.v[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) p = fmaf(q.v[i], k.v[i], p);
  return p;
}

struct RowAcc8 {
  float m, l;
  Vec8 acc;
  __device__ __forceinline__ void clear() {
    m = neg_inf();
    l = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc.v[i] = 0.f;
  }
};

template <int LPK>
__device__ __forceinline__ void softmax_step4_16(float mine, int grp, const Vec8 (&v)[4], RowAcc8& st) {
  float mc = fmaxf(mine, __shfl_xor_sync(kFullMask, mine, LPK / 2));
  mc = fmaxf(mc, __shfl_xor_sync(kFullMask, mc, LPK / 4));
  const float m_new = fmaxf(st.m, mc);
  const float m_safe = (m_new == neg_inf()) ? 0.f : m_new;
  const float corr = fast_exp2((st.m - m_safe) * kLog2e);
  const float pm = fast_exp2((mine - m_safe) * kLog2e);
  const int base = grp * LPK;
  const float p0 = __shfl_sync(kFullMask, pm, base);
  const float p1 = __shfl_sync(kFullMask, pm, base + LPK / 4);
  const float p2 = __shfl_sync(kFullMask, pm, base + LPK / 2);
  const float p3 = __shfl_sync(kFullMask, pm, base + LPK / 2 + LPK / 4);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float a = st.acc.v[i] * corr;
    a = fmaf(p0, v[0].v[i], a);
    a = fmaf(p1, v[1].v[i], a);
    a = fmaf(p2, v[2].v[i], a);
    a = fmaf(p3, v[3].v[i], a);
    st.acc.v[i] = a;
  }
  st.l = fmaf(st.l, corr, (p0 + p1) + (p2 + p3));
  st.m = m_new;
}

template <int D, class T, class Cols>
__device__ __forceinline__ void accumulate_slots16(const Cols& cols, const typename Cols::Row& row, int64_t t0, int64_t t1,
                                                   const Vec8& q, const T* __restrict__ K, const T* __restrict__ V,
                                                   float scale, int lane, RowAcc8& st) {
  constexpr int LPK = D / 8;
  constexpr int KPS = 32 / LPK;
  static_assert(LPK >= 4 && LPK <= 32, "16-bit rows of 32 to 256 elements");
  const int grp = lane / LPK, sub = lane % LPK;
  const int own = (((sub & (LPK / 2)) != 0) ? 2 : 0) + (((sub & (LPK / 4)) != 0) ? 1 : 0);
  const T* Kl = K + sub * 8;
  const T* Vl = V + sub * 8;
  for (int64_t base = t0; base < t1; base += 32) {
    const int64_t tl = base + lane;
    const int32_t c_lane = (tl < t1) ? cols.slot(row, tl) : -1;
    const int nb = (t1 - base < 32) ? (int)(t1 - base) : 32;
#pragma unroll 1
    for (int j0 = 0; j0 < LPK; j0 += 4) {
      if (j0 * KPS >= nb) break;  // warp-uniform
      Vec8 k[4], v[4];
      int32_t c_own = -1;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int32_t c = __shfl_sync(kFullMask, c_lane, grp + (j0 + u) * KPS);
        if (c >= 0) {
          k[u] = ldg8<T>(Kl + (size_t)c * D);
          v[u] = ldg8<T>(Vl + (size_t)c * D);
        } else {  // a masked key contributes probability 0; zero V keeps 0 * V finite
#pragma unroll
          for (int i = 0; i < 8; ++i) k[u].v[i] = v[u].v[i] = 0.f;
        }
        if (u == own) c_own = c;
      }
      float mine = reduce4_transposed<LPK>(dot8(q, k[0]), dot8(q, k[1]), dot8(q, k[2]), dot8(q, k[3]), sub) * scale;
      if (c_own < 0) mine = neg_inf();
      softmax_step4_16<LPK>(mine, grp, v, st);
    }
  }
}

template <int LPK>
__device__ __forceinline__ void merge_groups16(RowAcc8& st) {
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
    const float mo = __shfl_xor_sync(kFullMask, st.m, o);
    const float lo = __shfl_xor_sync(kFullMask, st.l, o);
    const float mn = fmaxf(st.m, mo);
    const float ms = (mn == neg_inf()) ? 0.f : mn;
    const float c1 = fast_exp2((st.m - ms) * kLog2e);
    const float c2 = fast_exp2((mo - ms) * kLog2e);
    st.l = st.l * c1 + lo * c2;
#pragma unroll
    for (int i = 0; i < 8; ++i) st.acc.v[i] = st.acc.v[i] * c1 + __shfl_xor_sync(kFullMask, st.acc.v[i], o) * c2;
    st.m = mn;
  }
}

// Fold a finished row into the caller's 16-bit state (same recurrence as store_row of the fp32 path).
template <int D, class T>
__device__ __forceinline__ void store_row16(const RowAcc8& st, T* __restrict__ m, T* __restrict__ l, T* __restrict__ O,
                                            int64_t r, int lane) {
  constexpr int LPK = D / 8;
  const float m_in = Cvt16<T>::up1(m[r]), l_in = Cvt16<T>::up1(l[r]);
  const float m_out = fmaxf(m_in, st.m);
  const float a = l_in * fast_exp2((m_in - m_out) * kLog2e);
  const float b = fast_exp2((st.m - m_out) * kLog2e);
  const float l_out = fmaf(st.l, b, a);
  const float inv = 1.0f / l_out;
  if (lane < LPK) {
    T* op = O + (size_t)r * D + lane * 8;
    const Vec8 o = ldg8<T>(op);
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = (a * o.v[i] + b * st.acc.v[i]) * inv;
    uint4 u;
    u.x = Cvt16<T>::down(y[0], y[1]);
    u.y = Cvt16<T>::down(y[2], y[3]);
    u.z = Cvt16<T>::down(y[4], y[5]);
    u.w = Cvt16<T>::down(y[6], y[7]);
    *reinterpret_cast<uint4*>(op) = u;
  }
  if (lane == 0) {
    m[r] = Cvt16<T>::down1(m_out);
    l[r] = Cvt16<T>::down1(l_out);
  }
}

template <int D, class T, class Cols>
__global__ void __launch_bounds__(kRowWarps * 32, 6)
gather_rows16_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V, T* __restrict__ m,
                     T* __restrict__ l, T* __restrict__ O, const Cols cols, int64_t row_begin, int64_t n_rows, int use_nan,
                     float scale) {
  constexpr int LPK = D / 8;
  __shared__ int s_heavy[kRowWarps];
  __shared__ int s_n_heavy;
  __shared__ float s_ml[kRowWarps][2];
  __shared__ float s_acc[kRowWarps][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_n_heavy = 0;
  __syncthreads();
  const int64_t r = (int64_t)blockIdx.x * kRowWarps + warp;
  if (r < n_rows) {
    const typename Cols::Row row = cols.open(r, row_begin + r);
    if (row.n <= 0) {
      if (Cols::kNanFillEmpty && use_nan && lane < LPK) {
        const uint32_t nn = Cvt16<T>::down(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
        *reinterpret_cast<uint4*>(O + (size_t)r * D + lane * 8) = make_uint4(nn, nn, nn, nn);
      }
    } else if (row.n > kHeavyRowSlots) {
      if (lane == 0) s_heavy[atomicAdd(&s_n_heavy, 1)] = warp;
    } else {
      const Vec8 q = ldg8<T>(Q + (size_t)r * D + (lane % LPK) * 8);
      RowAcc8 st;
      st.clear();
      accumulate_slots16<D, T, Cols>(cols, row, 0, row.n, q, K, V, scale, lane, st);
      merge_groups16<LPK>(st);
      if (st.l > 0.f) store_row16<D, T>(st, m, l, O, r, lane);
    }
  }
  __syncthreads();
  const int n_heavy = s_n_heavy;  // uniform over the CTA
  for (int h = 0; h < n_heavy; ++h) {  // long rows: every warp of the CTA takes a share of the slots
    const int64_t rh = (int64_t)blockIdx.x * kRowWarps + s_heavy[h];
    const typename Cols::Row row = cols.open(rh, row_begin + rh);
    int64_t per = (row.n + kRowWarps - 1) / kRowWarps;
    per = (per + 31) / 32 * 32;
    const int64_t t0 = (int64_t)warp * per;
    int64_t t1 = t0 + per;
    if (t1 > row.n) t1 = row.n;
    RowAcc8 st;
    st.clear();
    if (t0 < t1) {
      const Vec8 q = ldg8<T>(Q + (size_t)rh * D + (lane % LPK) * 8);
      accumulate_slots16<D, T, Cols>(cols, row, t0, t1, q, K, V, scale, lane, st);
      merge_groups16<LPK>(st);
    }
    if (lane < LPK) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s_acc[warp][lane * 8 + i] = st.acc.v[i];
    }
    if (lane == 0) {
      s_ml[warp][0] = st.m;
      s_ml[warp][1] = st.l;
    }
    __syncthreads();
    if (warp == 0) {
      RowAcc8 tot;
      tot.clear();
      const int sub = lane % LPK;
      for (int wv = 0; wv < kRowWarps; ++wv) {  // in slot order, like the single-warp walk
        const float mo = s_ml[wv][0], lo = s_ml[wv][1];
        const float mn = fmaxf(tot.m, mo);
        const float ms = (mn == neg_inf()) ? 0.f : mn;
        const float c1 = fast_exp2((tot.m - ms) * kLog2e), c2 = fast_exp2((mo - ms) * kLog2e);
        tot.l = tot.l * c1 + lo * c2;
#pragma unroll
        for (int i = 0; i < 8; ++i) tot.acc.v[i] = tot.acc.v[i] * c1 + s_acc[wv][sub * 8 + i] * c2;
        tot.m = mn;
      }
      if (tot.l > 0.f) store_row16<D, T>(tot, m, l, O, rh, lane);
    }
    __syncthreads();
  }
}

}  // namespace spfa
