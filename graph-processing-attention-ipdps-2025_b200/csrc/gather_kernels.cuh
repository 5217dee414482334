// FP32 gather path: one warp per query row, K/V rows fetched with 128-bit loads.
//
// Layout of a warp: a key row of D floats is D/4 float4s, so LPK = D/4 lanes cover one key and the
// warp works on KPS = 32/LPK keys at once ("key groups"). Each group keeps its own online-softmax
// state (m, l, acc) over the slots it owns; the groups are merged once at the end of the row, then
// merged with the caller's (m, l, O) state. All arithmetic is fp32 FMA; exponentials are ex2.approx.
// The kernel is instruction-issue bound, not bandwidth bound, on cache-friendly masks, so the inner step is
// written to minimise shuffles and special-function work: four keys per lane group are reduced with a
// transposed butterfly and each lane exponentiates one key only.
//
// Replaces the per-row CTA loop of the reference (sp_flatt_csr_kernel.cu:104-205 and its five copies):
// same key visiting order, same state recurrence, no shared memory, no block barriers.
#pragma once
#include "spfa_common.cuh"

namespace spfa {

constexpr int kGatherWarps = 4;  // warps per CTA
constexpr int kGatherUnroll = 4; // keys in flight per group per step

template <int D>
struct RowAcc {
  float m, l;
  float4 acc;
};

// Sum of four per-lane partial dot products over the LPK lanes of a key group, "transposed": instead of
// four full butterflies (4 log2(LPK) shuffles) the first two exchange steps halve the number of live values,
// so each lane ends with the complete sum of ONE of the four keys:
//   key index owned by a lane = 2 * bit(sub, LPK/2) + bit(sub, LPK/4)
// 2 + 1 + (log2(LPK) - 2) shuffles in total.
template <int LPK>
__device__ __forceinline__ float reduce4_transposed(float p0, float p1, float p2, float p3, int sub) {
  static_assert(LPK >= 4, "needs at least four lanes per key");
  const bool hi = (sub & (LPK / 2)) != 0;
  float a0 = hi ? p2 : p0, a1 = hi ? p3 : p1;
  const float b0 = hi ? p0 : p2, b1 = hi ? p1 : p3;
  a0 += __shfl_xor_sync(kFullMask, b0, LPK / 2);
  a1 += __shfl_xor_sync(kFullMask, b1, LPK / 2);
  const bool hi2 = (sub & (LPK / 4)) != 0;
  float c0 = hi2 ? a1 : a0;
  const float d0 = hi2 ? a0 : a1;
  c0 += __shfl_xor_sync(kFullMask, d0, LPK / 4);
#pragma unroll
  for (int o = LPK / 8; o > 0; o >>= 1) c0 += __shfl_xor_sync(kFullMask, c0, o);
  return c0;
}

// One step of the online softmax for the four keys a lane group has in flight. `mine` is the score
// (natural-log units, -inf if masked) of the key this lane owns after reduce4_transposed; the group
// maximum takes two shuffles, each lane exponentiates only its own key, and the four probabilities are
// then broadcast inside the group.
template <int D>
__device__ __forceinline__ void softmax_step4(float mine, int grp, const float4 (&v4)[4], RowAcc<D>& st) {
  constexpr int LPK = D / 4;
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
  float4 a = make_float4(st.acc.x * corr, st.acc.y * corr, st.acc.z * corr, st.acc.w * corr);
  a.x = fmaf(p0, v4[0].x, a.x); a.y = fmaf(p0, v4[0].y, a.y); a.z = fmaf(p0, v4[0].z, a.z); a.w = fmaf(p0, v4[0].w, a.w);
  a.x = fmaf(p1, v4[1].x, a.x); a.y = fmaf(p1, v4[1].y, a.y); a.z = fmaf(p1, v4[1].z, a.z); a.w = fmaf(p1, v4[1].w, a.w);
  a.x = fmaf(p2, v4[2].x, a.x); a.y = fmaf(p2, v4[2].y, a.y); a.z = fmaf(p2, v4[2].z, a.z); a.w = fmaf(p2, v4[2].w, a.w);
  a.x = fmaf(p3, v4[3].x, a.x); a.y = fmaf(p3, v4[3].y, a.y); a.z = fmaf(p3, v4[3].z, a.z); a.w = fmaf(p3, v4[3].w, a.w);
  st.acc = a;
  st.l = fmaf(st.l, corr, (p0 + p1) + (p2 + p3));
  st.m = m_new;
}

__device__ __forceinline__ float dot4(const float4 q, const float4 k) {
  float p = q.x * k.x;
  p = fmaf(q.y, k.y, p);
  p = fmaf(q.z, k.z, p);
  return fmaf(q.w, k.w, p);
}

// Online-softmax accumulation of slots [t0, t1) of one row into the calling lane's group state.
// Slots are taken 32 at a time (one per lane, so explicit column lists are read coalesced); a batch whose
// 32 slots are all valid takes a predicate-free body, ragged or partly masked batches a predicated one.
template <int D, class Cols>
__device__ __forceinline__ void accumulate_slots(const Cols& cols, const typename Cols::Row& row,
                                                 int64_t t0, int64_t t1, const float4 q,
                                                 const float* __restrict__ K, const float* __restrict__ V,
                                                 float scale, int lane, RowAcc<D>& st) {
  constexpr int LPK = D / 4;
  constexpr int KPS = 32 / LPK;
  static_assert(LPK >= 4 && kGatherUnroll == 4, "the step below handles four keys per lane group");
  const int grp = lane / LPK, sub = lane % LPK;
  // which of the four in-flight keys this lane owns after the transposed reduction
  const int own = (((sub & (LPK / 2)) != 0) ? 2 : 0) + (((sub & (LPK / 4)) != 0) ? 1 : 0);
  const float* Kl = K + sub * 4;
  const float* Vl = V + sub * 4;

  for (int64_t base = t0; base < t1; base += 32) {
    const int64_t tl = base + lane;
    const int32_t c_lane = (tl < t1) ? cols.slot(row, tl) : -1;
    const bool full = __all_sync(kFullMask, c_lane >= 0);
    if (full) {
#pragma unroll 1
      for (int j0 = 0; j0 < LPK; j0 += 4) {
        float4 k4[4], v4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t c = (uint32_t)__shfl_sync(kFullMask, c_lane, grp + (j0 + u) * KPS);
          k4[u] = ldg4(Kl + (size_t)c * D);
          v4[u] = ldg4(Vl + (size_t)c * D);
        }
        const float mine = reduce4_transposed<LPK>(dot4(q, k4[0]), dot4(q, k4[1]), dot4(q, k4[2]), dot4(q, k4[3]), sub) * scale;
        softmax_step4<D>(mine, grp, v4, st);
      }
    } else {
      const int nb = (t1 - base < 32) ? (int)(t1 - base) : 32;
#pragma unroll 1
      for (int j0 = 0; j0 < LPK; j0 += 4) {
        if (j0 * KPS >= nb) break;  // warp-uniform
        float4 k4[4], v4[4];
        int32_t c_own = -1;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int32_t c = __shfl_sync(kFullMask, c_lane, grp + (j0 + u) * KPS);
          if (c >= 0) {
            k4[u] = ldg4(Kl + (size_t)c * D);
            v4[u] = ldg4(Vl + (size_t)c * D);
          } else {  // a masked key contributes probability 0; zero V keeps 0 * V finite
            k4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            v4[u] = k4[u];
          }
          if (u == own) c_own = c;
        }
        float mine = reduce4_transposed<LPK>(dot4(q, k4[0]), dot4(q, k4[1]), dot4(q, k4[2]), dot4(q, k4[3]), sub) * scale;
        if (c_own < 0) mine = neg_inf();
        softmax_step4<D>(mine, grp, v4, st);
      }
    }
  }
}

// Merge the KPS key-group states of a warp; afterwards every lane holds the whole-row (m, l) and the
// un-normalised accumulator slice for dims [4*sub, 4*sub+4).
template <int D>
__device__ __forceinline__ void merge_groups(RowAcc<D>& st) {
  constexpr int LPK = D / 4;
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
    const float mo = __shfl_xor_sync(kFullMask, st.m, o);
    const float lo = __shfl_xor_sync(kFullMask, st.l, o);
    float4 ao;
    ao.x = __shfl_xor_sync(kFullMask, st.acc.x, o);
    ao.y = __shfl_xor_sync(kFullMask, st.acc.y, o);
    ao.z = __shfl_xor_sync(kFullMask, st.acc.z, o);
    ao.w = __shfl_xor_sync(kFullMask, st.acc.w, o);
    const float mn = fmaxf(st.m, mo);
    const float ms = (mn == neg_inf()) ? 0.f : mn;
    const float c1 = fast_exp2((st.m - ms) * kLog2e);
    const float c2 = fast_exp2((mo - ms) * kLog2e);
    st.l = st.l * c1 + lo * c2;
    st.acc.x = st.acc.x * c1 + ao.x * c2;
    st.acc.y = st.acc.y * c1 + ao.y * c2;
    st.acc.z = st.acc.z * c1 + ao.z * c2;
    st.acc.w = st.acc.w * c1 + ao.w * c2;
    st.m = mn;
  }
}

// Fold a finished row (m_loc, l_loc, un-normalised acc) into the caller's state and store it.
// O_out = (l_in e^{m_in-m_out} O_in + e^{m_loc-m_out} acc) / l_out -- the recurrence of
// sp_flatt_csr_kernel.cu:162-194 applied once to the whole row. No guard on 0*NaN: a row a previous
// call NaN-filled stays NaN, as it does in the reference.
template <int D>
__device__ __forceinline__ void store_row(const RowAcc<D>& st, float* __restrict__ m, float* __restrict__ l,
                                          float* __restrict__ O, int64_t r, int lane) {
  constexpr int LPK = D / 4;
  const float m_in = m[r], l_in = l[r];
  const float m_out = fmaxf(m_in, st.m);
  const float a = l_in * fast_exp2((m_in - m_out) * kLog2e);
  const float b = fast_exp2((st.m - m_out) * kLog2e);
  const float l_out = fmaf(st.l, b, a);
  const float inv = 1.0f / l_out;
  if (lane < LPK) {
    float4* op = reinterpret_cast<float4*>(O + (size_t)r * D) + lane;
    float4 o = *op;
    o.x = (a * o.x + b * st.acc.x) * inv;
    o.y = (a * o.y + b * st.acc.y) * inv;
    o.z = (a * o.z + b * st.acc.z) * inv;
    o.w = (a * o.w + b * st.acc.w) * inv;
    *op = o;
  }
  if (lane == 0) {
    m[r] = m_out;
    l[r] = l_out;
  }
}

template <int D>
__device__ __forceinline__ void nan_fill_row(float* __restrict__ O, int64_t r, int lane) {
  constexpr int LPK = D / 4;
  if (lane < LPK) {
    const float n = __int_as_float(0x7fc00000);
    reinterpret_cast<float4*>(O + (size_t)r * D)[lane] = make_float4(n, n, n, n);
  }
}

// One warp per row of the shard at a time; a CTA of four warps owns up to kMaxRowsPerCta consecutive rows and its
// warps claim them one by one (gather_rows_cta). Q/m/l/O are indexed by shard-local row; the generator sees the
// absolute row (row_begin + r).
//
// Long rows: a single warp walking thousands of scattered keys is latency bound (one DRAM round trip per
// step of eight keys), so the longest row of a power-law graph would set the duration of the whole launch.
// A row with more than kHeavyRowSlots slots is therefore postponed; once the CTA's ordinary rows are done,
// all warps of the CTA take an equal share of its slots and their partial states are merged through shared
// memory. No scratch memory and no extra launch are involved.
constexpr int kRowWarps = 4;
constexpr int kHeavyRowSlots = 1024;

// All NW warps of a CTA walk one row together: warp w takes the w-th share of the slots (whole 32-slot
// batches), the partial states meet in shared memory and warp 0 folds them in slot order and stores the row.
// Every thread of the CTA must call this (it contains block barriers).
template <int D, class Cols, int NW>
__device__ __forceinline__ void walk_row_with_cta(const Cols& cols, const typename Cols::Row& row, int64_t r,
                                                  const float* __restrict__ Q, const float* __restrict__ K,
                                                  const float* __restrict__ V, float* __restrict__ m,
                                                  float* __restrict__ l, float* __restrict__ O, float scale, int warp,
                                                  int lane, float (*s_ml)[2], float4 (*s_acc)[D / 4]) {
  constexpr int LPK = D / 4;
  int64_t per = (row.n + NW - 1) / NW;
  per = (per + 31) / 32 * 32;  // whole 32-slot batches per warp
  const int64_t t0 = (int64_t)warp * per;
  int64_t t1 = t0 + per;
  if (t1 > row.n) t1 = row.n;
  RowAcc<D> st;
  st.m = neg_inf();
  st.l = 0.f;
  st.acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (t0 < t1) {
    const float4 q = ldg4(Q + (size_t)r * D + (lane % LPK) * 4);
    accumulate_slots<D, Cols>(cols, row, t0, t1, q, K, V, scale, lane, st);
    merge_groups<D>(st);
  }
  if (lane < LPK) s_acc[warp][lane] = st.acc;
  if (lane == 0) {
    s_ml[warp][0] = st.m;
    s_ml[warp][1] = st.l;
  }
  __syncthreads();
  if (warp == 0) {
    RowAcc<D> tot;
    tot.m = neg_inf();
    tot.l = 0.f;
    tot.acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const int sub = lane % LPK;
#pragma unroll 4
    for (int wv = 0; wv < NW; ++wv) {  // in slot order, like the single-warp walk
      const float mo = s_ml[wv][0], lo = s_ml[wv][1];
      const float4 ao = s_acc[wv][sub];
      const float mn = fmaxf(tot.m, mo);
      const float ms = (mn == neg_inf()) ? 0.f : mn;
      const float c1 = fast_exp2((tot.m - ms) * kLog2e);
      const float c2 = fast_exp2((mo - ms) * kLog2e);
      tot.l = tot.l * c1 + lo * c2;
      tot.acc.x = tot.acc.x * c1 + ao.x * c2;
      tot.acc.y = tot.acc.y * c1 + ao.y * c2;
      tot.acc.z = tot.acc.z * c1 + ao.z * c2;
      tot.acc.w = tot.acc.w * c1 + ao.w * c2;
      tot.m = mn;
    }
    if (tot.l > 0.f) store_row<D>(tot, m, l, O, r, lane);
  }
  __syncthreads();
}

// Slots [t_begin, t_end) of one row by all NW warps of a CTA; afterwards warp 0 holds the folded state of the slice in
// `tot` (every lane: m, l; lane sub: its accumulator slice). Every thread of the CTA must call this.
template <int D, class Cols, int NW>
__device__ __forceinline__ void walk_slice_with_cta(const Cols& cols, const typename Cols::Row& row, int64_t r,
                                                    int64_t t_begin, int64_t t_end, const float* __restrict__ Q,
                                                    const float* __restrict__ K, const float* __restrict__ V, float scale,
                                                    int warp, int lane, float (*s_ml)[2], float4 (*s_acc)[D / 4],
                                                    RowAcc<D>& tot) {
  constexpr int LPK = D / 4;
  int64_t per = (t_end - t_begin + NW - 1) / NW;
  per = (per + 31) / 32 * 32;  // whole 32-slot batches per warp
  const int64_t t0 = t_begin + (int64_t)warp * per;
  int64_t t1 = t0 + per;
  if (t1 > t_end) t1 = t_end;
  RowAcc<D> st;
  st.m = neg_inf();
  st.l = 0.f;
  st.acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (t0 < t1) {
    const float4 q = ldg4(Q + (size_t)r * D + (lane % LPK) * 4);
    accumulate_slots<D, Cols>(cols, row, t0, t1, q, K, V, scale, lane, st);
    merge_groups<D>(st);
  }
  if (lane < LPK) s_acc[warp][lane] = st.acc;
  if (lane == 0) {
    s_ml[warp][0] = st.m;
    s_ml[warp][1] = st.l;
  }
  __syncthreads();
  tot.m = neg_inf();
  tot.l = 0.f;
  tot.acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (warp == 0) {
    const int sub = lane % LPK;
#pragma unroll 4
    for (int wv = 0; wv < NW; ++wv) {  // in slot order
      const float mo = s_ml[wv][0], lo = s_ml[wv][1];
      const float4 ao = s_acc[wv][sub];
      const float mn = fmaxf(tot.m, mo);
      const float ms = (mn == neg_inf()) ? 0.f : mn;
      const float c1 = fast_exp2((tot.m - ms) * kLog2e);
      const float c2 = fast_exp2((mo - ms) * kLog2e);
      tot.l = tot.l * c1 + lo * c2;
      tot.acc.x = tot.acc.x * c1 + ao.x * c2;
      tot.acc.y = tot.acc.y * c1 + ao.y * c2;
      tot.acc.z = tot.acc.z * c1 + ao.z * c2;
      tot.acc.w = tot.acc.w * c1 + ao.w * c2;
      tot.m = mn;
    }
  }
  __syncthreads();
}

constexpr int kMaxRowsPerCta = 32;

struct RowCtaShared {
  int heavy[kMaxRowsPerCta];
  int n_heavy;
  int next;  // next unclaimed row of the CTA's range
  float ml[kRowWarps][2];
};

// Rows [block * rows_per_cta, (block + 1) * rows_per_cta) of the shard, by one CTA of kRowWarps warps.
// A warp takes one row at a time and claims the next from a shared counter when it is done: with one fixed row per
// warp a CTA lasts as long as its longest row while the other warps' slots sit idle, which on a mask with skewed row
// lengths left a third of the resident warps waiting. rows_per_cta is at most kMaxRowsPerCta.
template <int D, class Cols>
__device__ __forceinline__ void gather_rows_cta(int64_t block, int rows_per_cta, const float* __restrict__ Q,
                                                const float* __restrict__ K, const float* __restrict__ V,
                                                float* __restrict__ m, float* __restrict__ l, float* __restrict__ O,
                                                const Cols& cols, int64_t row_begin, int64_t n_rows, int use_nan,
                                                float scale, RowCtaShared& sh, float4 (*s_acc)[D / 4]) {
  constexpr int LPK = D / 4;
  int* s_heavy = sh.heavy;
  int& s_n_heavy = sh.n_heavy;
  float (*s_ml)[2] = sh.ml;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    s_n_heavy = 0;
    sh.next = kRowWarps;
  }
  __syncthreads();
  const int64_t first = block * rows_per_cta;
  for (int i = warp; i < rows_per_cta;) {  // warp-uniform
    const int64_t r = first + i;
    if (r >= n_rows) break;
    const typename Cols::Row row = cols.open(r, row_begin + r);
    if (row.n <= 0) {
      if (Cols::kNanFillEmpty && use_nan) nan_fill_row<D>(O, r, lane);
    } else if (row.n > kHeavyRowSlots) {
      if (lane == 0) s_heavy[atomicAdd(&s_n_heavy, 1)] = i;
    } else {
      const float4 q = ldg4(Q + (size_t)r * D + (lane % LPK) * 4);
      RowAcc<D> st;
      st.m = neg_inf();
      st.l = 0.f;
      st.acc = make_float4(0.f, 0.f, 0.f, 0.f);
      accumulate_slots<D, Cols>(cols, row, 0, row.n, q, K, V, scale, lane, st);
      merge_groups<D>(st);
      if (st.l > 0.f) store_row<D>(st, m, l, O, r, lane);
    }
    if (rows_per_cta <= kRowWarps) break;
    int nxt = 0;
    if (lane == 0) nxt = atomicAdd(&sh.next, 1);
    i = __shfl_sync(kFullMask, nxt, 0);
  }
  __syncthreads();
  const int n_heavy = s_n_heavy;  // uniform over the CTA
  for (int h = 0; h < n_heavy; ++h) {
    const int64_t rh = first + s_heavy[h];
    const typename Cols::Row row = cols.open(rh, row_begin + rh);
    walk_row_with_cta<D, Cols, kRowWarps>(cols, row, rh, Q, K, V, m, l, O, scale, warp, lane, s_ml, s_acc);
  }
}

// Rows per CTA for a launch over n_rows rows (times n_slices slices): as many as kMaxRowsPerCta once that still leaves
// several waves of CTAs on the machine, down to one per warp for small shards.
inline int rows_per_cta_for(int64_t n_rows, int64_t n_slices) {
  const int64_t want_ctas = 148LL * 7 * 8;
  int64_t r = n_rows * n_slices / want_ctas;
  r = r / kRowWarps * kRowWarps;
  if (r < kRowWarps) r = kRowWarps;
  if (r > kMaxRowsPerCta) r = kMaxRowsPerCta;
  return (int)r;
}

// Slices of a batched call (batch x heads, one mask for all) ride on blockIdx.y: Q, O advance by n_rows * D elements
// per slice, m, l by n_rows, K, V by kv_slice elements (0 for an unbatched call, whose grid has y = 1).
template <int D, class Cols>
__global__ void __launch_bounds__(kRowWarps * 32, 7)
gather_rows_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                   float* __restrict__ m, float* __restrict__ l, float* __restrict__ O,
                   const Cols cols, int64_t row_begin, int64_t n_rows, int use_nan, float scale, int64_t kv_slice,
                   int rows_per_cta) {
  __shared__ RowCtaShared sh;
  __shared__ float4 s_acc[kRowWarps][D / 4];
  const size_t z = blockIdx.y;
  gather_rows_cta<D, Cols>(blockIdx.x, rows_per_cta, Q + z * n_rows * D, K + z * kv_slice, V + z * kv_slice, m + z * n_rows,
                           l + z * n_rows, O + z * n_rows * D, cols, row_begin, n_rows, use_nan, scale, sh, s_acc);
}

// Same, for a shard whose long rows were listed beforehand (the explicit-mask plan lists the rows whose residual
// part exceeds kHeavyRowSlots; `cols` reports those rows as empty). The first n_list_blocks CTAs stride over the
// list, one listed row at a time with all their warps (`listed` opens the same rows at full length); the other
// CTAs do the ordinary rows. Blocks are dispatched in index order, so the long rows start with the launch
// instead of wherever their row number falls. The list length lives in device memory (it is produced there).
// The lists come from a stored plan: its identity block is compared with the shape the caller passed first.
// Eight CTAs per SM (64 registers, some spills) beat seven here: the residual rows of a split mask are short lists of
// scattered keys, bound by load latency, so resident warps count for more than registers (2.89 -> 2.68 ms on the 1M-row
// graph; nine CTAs: 2.90, ten: 3.45). The plain kernel above is closer to issue bound and loses 3-4 % at eight.
template <int D, class Cols>
__global__ void __launch_bounds__(kRowWarps * 32, 8)
gather_rows_listed_first_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                                float* __restrict__ m, float* __restrict__ l, float* __restrict__ O, const Cols cols,
                                const Cols listed, const int* __restrict__ row_list,
                                const unsigned int* __restrict__ n_listed, int n_list_blocks, int64_t row_begin,
                                int64_t n_rows, int use_nan, float scale, const PlanHeader* __restrict__ hdr,
                                const PlanHeader want, int* __restrict__ err, const int4* __restrict__ split_items,
                                const unsigned int* __restrict__ n_split_items, long long cap_items,
                                unsigned int* __restrict__ split_done, float* __restrict__ split_part,
                                int rows_per_cta) {
  __shared__ RowCtaShared sh;
  __shared__ float4 s_acc[kRowWarps][D / 4];
  __shared__ unsigned int s_last;
  if (!plan_header_matches(hdr, want)) {  // uniform over the grid: the lists belong to a plan of another shape
    if (threadIdx.x == 0) atomicCAS(err, 0, kPlanMismatchCode);
    return;
  }
  if ((int)blockIdx.x >= n_list_blocks) {
    gather_rows_cta<D, Cols>((int64_t)blockIdx.x - n_list_blocks, rows_per_cta, Q, K, V, m, l, O, cols, row_begin, n_rows,
                             use_nan, scale, sh, s_acc);
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // ---- rows cut into slices: one item at a time per CTA; the CTA that finishes a row's last slice folds them ----
  {
    constexpr int LPK = D / 4;
    unsigned int n_items = *n_split_items;
    if ((long long)n_items > cap_items) n_items = (unsigned int)cap_items;
    for (unsigned int it = blockIdx.x; it < n_items; it += (unsigned int)n_list_blocks) {
      const int4 item = split_items[it];
      if (item.x < 0) continue;  // uniform over the CTA
      const int64_t r = item.x;
      const typename Cols::Row row = listed.open(r, row_begin + r);
      int64_t per = (row.n + item.z - 1) / item.z;  // slices are cut from the row's length now (a key-range pass is shorter)
      per = (per + 31) / 32 * 32;
      const int64_t t_begin = (int64_t)item.y * per;
      int64_t t_end = t_begin + per;
      if (t_end > row.n) t_end = row.n;
      RowAcc<D> tot;
      walk_slice_with_cta<D, Cols, kRowWarps>(listed, row, r, t_begin < t_end ? t_begin : t_end, t_end, Q, K, V, scale, warp, lane,
                                              sh.ml, s_acc, tot);
      float* part = split_part + (size_t)it * (D + 4);
      if (warp == 0) {
        if (lane < LPK) reinterpret_cast<float4*>(part)[lane] = tot.acc;
        if (lane == 0) {
          part[D] = tot.m;
          part[D + 1] = tot.l;
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) s_last = (atomicAdd(split_done + item.w, 1u) == (unsigned int)(item.z - 1)) ? 1u : 0u;
      }
      __syncthreads();
      if (s_last && warp == 0) {  // every slice of the row is in scratch: fold them in slice order, store the row
        __threadfence();
        RowAcc<D> all;
        all.m = neg_inf();
        all.l = 0.f;
        all.acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const int sub = lane % LPK;
        for (int sl = 0; sl < item.z; ++sl) {
          const float* p = split_part + (size_t)(item.w + sl) * (D + 4);
          const float mo = __ldcg(p + D), lo = __ldcg(p + D + 1);
          const float4 ao = __ldcg(reinterpret_cast<const float4*>(p) + sub);
          const float mn = fmaxf(all.m, mo);
          const float ms = (mn == neg_inf()) ? 0.f : mn;
          const float c1 = fast_exp2((all.m - ms) * kLog2e), c2 = fast_exp2((mo - ms) * kLog2e);
          all.l = all.l * c1 + lo * c2;
          all.acc.x = all.acc.x * c1 + ao.x * c2;
          all.acc.y = all.acc.y * c1 + ao.y * c2;
          all.acc.z = all.acc.z * c1 + ao.z * c2;
          all.acc.w = all.acc.w * c1 + ao.w * c2;
          all.m = mn;
        }
        if (all.l > 0.f) store_row<D>(all, m, l, O, r, lane);
        if (lane == 0) split_done[item.w] = 0u;  // ready for the next forward call from this plan
      }
      __syncthreads();
    }
  }
  const unsigned int n = *n_listed;
  for (unsigned int e = blockIdx.x; e < n; e += (unsigned int)n_list_blocks) {
    const int64_t r = row_list[e];
    const typename Cols::Row row = listed.open(r, row_begin + r);
    walk_row_with_cta<D, Cols, kRowWarps>(listed, row, r, Q, K, V, m, l, O, scale, warp, lane, sh.ml, s_acc);
  }
}

// Split-row variant for very long rows: entry e of row_list is processed by n_split warps, each
// over a contiguous slot range; partial states go to `partials` ((D+4) floats per (entry, split):
// acc[D], m, l, pad, pad) and are folded into the caller's state by combine_partials_kernel.
template <int D, class Cols>
__global__ void __launch_bounds__(kGatherWarps * 32)
gather_split_rows_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                         const Cols cols, const int32_t* __restrict__ row_list,
                         const uint8_t* __restrict__ entry_live, int n_entries, int64_t row_begin, int64_t row_end,
                         int n_split, int64_t slots_per_split, float* __restrict__ partials, float scale) {
  constexpr int LPK = D / 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // One key range (split) per blockIdx.y, four list entries per CTA: CTAs that are resident together
  // walk the same K/V rows.
  const int e = blockIdx.x * kGatherWarps + warp;
  const int split = blockIdx.y;
  if (e >= n_entries) return;
  float* part = partials + ((size_t)e * n_split + split) * (D + 4);
  RowAcc<D> st;
  st.m = neg_inf();
  st.l = 0.f;
  st.acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const int64_t i = row_list[e];
  const bool live = entry_live[e] && i >= row_begin && i < row_end;
  if (live) {
    const int64_t r = i - row_begin;
    const typename Cols::Row row = cols.open(r, i);
    const int64_t t0 = (int64_t)split * slots_per_split;
    int64_t t1 = t0 + slots_per_split;
    if (t1 > row.n) t1 = row.n;
    if (t0 < t1) {
      const float4 q = ldg4(Q + (size_t)r * D + (lane % LPK) * 4);
      accumulate_slots<D, Cols>(cols, row, t0, t1, q, K, V, scale, lane, st);
      merge_groups<D>(st);
    }
  }
  if (lane < LPK) reinterpret_cast<float4*>(part)[lane] = st.acc;
  if (lane == 0) {
    part[D] = st.m;
    part[D + 1] = st.l;
  }
}

// One CTA (kCombineWarps warps) per list entry: folds that entry's n_split partial states into (m, l, O).
// The partial maxima are reduced first, so the accumulation over splits has no serial dependency: every
// warp takes its share of the splits with several loads in flight, and the warp results are summed through
// shared memory in a fixed order.
constexpr int kCombineWarps = 16;

template <int D>
__global__ void __launch_bounds__(kCombineWarps * 32)
combine_partials_kernel(const float* __restrict__ partials, const int32_t* __restrict__ row_list,
                        const uint8_t* __restrict__ entry_live, int n_entries, int64_t row_begin,
                        int64_t row_end, int n_split, float* __restrict__ m, float* __restrict__ l,
                        float* __restrict__ O) {
  constexpr int LPK = D / 4;
  __shared__ float s_l[kCombineWarps];
  __shared__ float4 s_acc[kCombineWarps][LPK];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = blockIdx.x;
  if (e >= n_entries) return;
  const int64_t i = row_list[e];
  if (!entry_live[e] || i < row_begin || i >= row_end) return;  // uniform over the CTA
  const float* base = partials + (size_t)e * n_split * (D + 4);
  // maximum of the partial maxima (all threads compute the same value)
  float mx = neg_inf();
  for (int sp = lane; sp < n_split; sp += 32) mx = fmaxf(mx, __ldg(base + (size_t)sp * (D + 4) + D));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, o));
  const float ms = (mx == neg_inf()) ? 0.f : mx;
  const int sub = lane % LPK;
  float lsum = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int sp = warp; sp < n_split; sp += kCombineWarps) {
    const float* part = base + (size_t)sp * (D + 4);
    const float w = fast_exp2((__ldg(part + D) - ms) * kLog2e);
    const float4 a = ldg4(part + sub * 4);
    lsum = fmaf(__ldg(part + D + 1), w, lsum);
    acc.x = fmaf(a.x, w, acc.x);
    acc.y = fmaf(a.y, w, acc.y);
    acc.z = fmaf(a.z, w, acc.z);
    acc.w = fmaf(a.w, w, acc.w);
  }
  if (lane < LPK) s_acc[warp][lane] = acc;
  if (lane == 0) s_l[warp] = lsum;
  __syncthreads();
  if (warp == 0) {
    RowAcc<D> st;
    st.m = mx;
    st.l = 0.f;
    st.acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int wv = 0; wv < kCombineWarps; ++wv) {
      const float4 a = s_acc[wv][sub];
      st.l += s_l[wv];
      st.acc.x += a.x;
      st.acc.y += a.y;
      st.acc.z += a.z;
      st.acc.w += a.w;
    }
    if (st.l > 0.f) store_row<D>(st, m, l, O, i - row_begin, lane);
  }
}

// ---- COO row pointers --------------------------------------------------------------------------
// ptr[r] = first k with row_ind[k] >= row_begin + r, for r in [0, n_rows]. One pass over the sorted
// row array: position k writes the pointers of all rows in (row_ind[k-1], row_ind[k]]. The pass is a stream of
// 8-byte (or 4-byte) loads bound by memory latency, so every thread keeps kRowPtrUnroll independent loads in
// flight; the predecessor of a position comes from the neighbouring lane (lane 0 reads it, a cache hit).
constexpr int kRowPtrUnroll = 4;
constexpr int kRowPtrThreads = 256;

template <class IdxT>  // uint64_t (the reference's layout) or int32_t (halves the bytes this pass reads)
__global__ void __launch_bounds__(kRowPtrThreads)
coo_row_pointers_kernel(const IdxT* __restrict__ row_ind, int64_t nnz, int64_t row_begin, int64_t n_rows,
                        uint64_t* __restrict__ ptr) {
  constexpr int64_t span = (int64_t)kRowPtrThreads * kRowPtrUnroll;
  const int lane = threadIdx.x & 31;
  const int64_t end_row = row_begin + n_rows;
  for (int64_t base = (int64_t)blockIdx.x * span; base <= nnz; base += (int64_t)gridDim.x * span) {  // uniform per CTA
    int64_t cur[kRowPtrUnroll];
#pragma unroll
    for (int u = 0; u < kRowPtrUnroll; ++u) {
      const int64_t k = base + u * kRowPtrThreads + threadIdx.x;
      cur[u] = (k < nnz) ? (int64_t)__ldg(row_ind + k) : end_row;  // k == nnz closes the last rows
    }
#pragma unroll
    for (int u = 0; u < kRowPtrUnroll; ++u) {
      const int64_t k = base + u * kRowPtrThreads + threadIdx.x;
      int64_t prev = __shfl_up_sync(kFullMask, cur[u], 1);
      if (lane == 0 && k <= nnz) prev = (k == 0) ? (row_begin - 1) : (int64_t)__ldg(row_ind + k - 1);
      if (k > nnz || cur[u] == prev) continue;
      // rows strictly above `prev` and up to `cur` start at k
      int64_t a = prev + 1 - row_begin, b = cur[u] - row_begin;
      if (a < 0) a = 0;
      if (b > n_rows) b = n_rows;
      for (int64_t r = a; r <= b; ++r) ptr[r] = (uint64_t)k;
    }
  }
}

// 32-bit row offsets widened to the 64-bit offsets the kernels read (n entries; negative values clamp to 0).
static __global__ void widen_offsets_kernel(const int32_t* __restrict__ in, int64_t n, uint64_t* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (uint64_t)(in[i] > 0 ? in[i] : 0);
}

// ---- Global-no-local: mark the listed rows -------------------------------------------------------
// bits must be zero on entry. entry_live[t] = 1 for the first list position naming a row.
static __global__ void gnl_mark_globals_kernel(const int32_t* __restrict__ G, int64_t nG, int64_t L,
                                        uint32_t* __restrict__ bits, uint8_t* __restrict__ entry_live) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nG) return;
  const int64_t g = G[t];
  if (g < 0 || g >= L) { entry_live[t] = 0; return; }
  const uint32_t bit = 1u << (g & 31);
  const uint32_t old = atomicOr(bits + (g >> 5), bit);
  entry_live[t] = (old & bit) ? 0 : 1;
}

// ---- visited-pair dump ----------------------------------------------------------------------------
template <class Cols>
__global__ void mask_count_kernel(const Cols cols, int64_t row_begin, int64_t n_rows, int64_t* __restrict__ counts) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  const typename Cols::Row row = cols.open(r, row_begin + r);
  int64_t n = 0;
  for (int64_t t = 0; t < row.n; ++t) n += (cols.slot(row, t) >= 0);
  counts[r] = n;
}

template <class Cols>
__global__ void mask_fill_kernel(const Cols cols, int64_t row_begin, int64_t n_rows,
                                 const int64_t* __restrict__ row_off, uint32_t* __restrict__ col_out) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  const typename Cols::Row row = cols.open(r, row_begin + r);
  int64_t w = row_off[r];
  for (int64_t t = 0; t < row.n; ++t) {
    const int32_t c = cols.slot(row, t);
    if (c >= 0) col_out[w++] = (uint32_t)c;
  }
}

}  // namespace spfa
