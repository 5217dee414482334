// Shared device helpers and the per-mask column generators.
//
// A "column generator" turns (absolute query row, slot number) into the key row that slot attends to,
// or -1 for a slot that is masked out. Slots are visited in the reference's visiting order, so the
// generators are the single device-side definition of every implicit mask's index set; the gather
// kernels, the split-row kernels and the visited-pair dump all use them.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace spfa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr unsigned kFullMask = 0xffffffffu;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }

__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

// Identity of a filled plan region, written by the inspector into the region's first 256-byte block (behind the
// two counters) and compared by every kernel that consumes the region with the shape its caller passed: a plan
// built for another mask shape would otherwise shift every table behind it and send the tiled kernel to wild
// addresses. On a mismatch the consuming kernels record code kPlanMismatchCode in the error word and do nothing.
struct PlanHeader {
  unsigned long long magic;
  long long n_rows, nnz, n_keys;
  int d, bn;
};
constexpr unsigned long long kPlanMagic = 0x53504641504c414eull;  // "SPFAPLAN"
constexpr int kPlanMismatchCode = 401;
constexpr int kPlanHeaderOffset = 32;  // bytes into the region: [pool_used u64][heavy_count u32][unsorted u32][pad] then this

__device__ __forceinline__ bool plan_header_matches(const PlanHeader* __restrict__ h, const PlanHeader& want) {
  return h->magic == want.magic && h->n_rows == want.n_rows && h->nnz == want.nnz && h->n_keys == want.n_keys &&
         h->d == want.d && h->bn == want.bn;
}

// ---- explicit CSR rows (also used for COO after the row-pointer pass) ---------------------------
// Row r of the shard owns col[row_off[r] .. row_off[r+1])   (reference: sp_flatt_csr_kernel.cu:29-33,117)
struct CsrCols {
  const uint64_t* row_off;
  const uint32_t* col;
  int64_t Lk;
  static constexpr bool kNanFillEmpty = true;
  struct Row { int64_t lo; int64_t n; };
  __device__ __forceinline__ Row open(int64_t r_local, int64_t /*r_abs*/) const {
    Row r;
    r.lo = (int64_t)row_off[r_local];
    r.n = (int64_t)row_off[r_local + 1] - r.lo;
    if (r.n < 0) r.n = 0;
    return r;
  }
  __device__ __forceinline__ int32_t slot(const Row& r, int64_t t) const {
    uint32_t c = __ldg(col + r.lo + t);
    return ((int64_t)c < Lk) ? (int32_t)c : -1;
  }
};

// ---- Local: j in [max(0,i-w), min(L,i+w+1))   (sp_flatt_local_kernel.cu:24-28,101) -----------------
struct LocalCols {
  int64_t L, w;
  static constexpr bool kNanFillEmpty = false;
  struct Row { int64_t lo; int64_t n; };
  __device__ __forceinline__ Row open(int64_t, int64_t i) const {
    Row r;
    r.lo = (i - w > 0) ? (i - w) : 0;
    int64_t hi = (i + w + 1 < L) ? (i + w + 1) : L;
    r.n = hi - r.lo;
    return r;
  }
  __device__ __forceinline__ int32_t slot(const Row& r, int64_t t) const { return (int32_t)(r.lo + t); }
};

// ---- Local 1D dilated: lo=max(i-w s, i mod s), hi=min(i+w s, L-1), n=(hi-lo)/s+1, cols lo+t s
//      (sp_flatt_local_1d_dilated_kernel.cu:25-29,102) ----------------------------------------------
struct Local1dCols {
  int64_t L, w, s;
  static constexpr bool kNanFillEmpty = false;
  struct Row { int64_t lo; int64_t n; };
  __device__ __forceinline__ Row open(int64_t, int64_t i) const {
    Row r;
    int64_t a = i - w * s, b = i % s;
    r.lo = a > b ? a : b;
    int64_t hi = (i + w * s < L - 1) ? (i + w * s) : (L - 1);
    r.n = (hi - r.lo) / s + 1;
    return r;
  }
  __device__ __forceinline__ int32_t slot(const Row& r, int64_t t) const { return (int32_t)(r.lo + t * s); }
};

// ---- Local 2D dilated: start=(i/B)B; live iff (i-start) mod s==0; n=min(B,(B-1)/s+1); cols start+t s
//      (sp_flatt_local_2d_dilated_kernel.cu:26-39,123) ----------------------------------------------
struct Local2dCols {
  int64_t L, B, s;
  static constexpr bool kNanFillEmpty = true;
  struct Row { int64_t lo; int64_t n; };
  __device__ __forceinline__ Row open(int64_t, int64_t i) const {
    Row r;
    r.lo = (i / B) * B;
    if ((i - r.lo) % s != 0) { r.n = 0; return r; }
    int64_t n = (B - 1) / s + 1;
    r.n = n < B ? n : B;
    return r;
  }
  __device__ __forceinline__ int32_t slot(const Row& r, int64_t t) const { return (int32_t)(r.lo + t * s); }
};

// ---- Global-no-local, rows NOT in the global list: listed g outside W(i), list order
//      (sp_flatt_global_no_local_kernel.cu:38-39,58-60,146-162). Rows that ARE global are skipped
//      here (n = 0, flagged) and handled by GnlGlobalRowCols. ------------------------------------------
struct GnlCols {
  const int32_t* G;
  int64_t nG, L, w;
  const uint32_t* global_bits;  // bit i set <=> row i is in the global list
  static constexpr bool kNanFillEmpty = false;
  struct Row { int64_t lo; int64_t hi; int64_t n; };
  __device__ __forceinline__ Row open(int64_t, int64_t i) const {
    Row r;
    r.lo = (i - w > 0) ? (i - w) : 0;
    r.hi = (i + w + 1 < L) ? (i + w + 1) : L;
    bool is_global = (__ldg(global_bits + (i >> 5)) >> (i & 31)) & 1u;
    r.n = is_global ? 0 : nG;
    return r;
  }
  __device__ __forceinline__ int32_t slot(const Row& r, int64_t t) const {
    int64_t g = __ldg(G + t);
    if (g < 0 || g >= L) return -1;
    return (g >= r.lo && g < r.hi) ? -1 : (int32_t)g;
  }
};

// ---- Global-no-local, rows in the global list: every j outside W(i), ascending
//      (sp_flatt_global_no_local_kernel.cu:54-57,135-145) -------------------------------------------
struct GnlGlobalRowCols {
  int64_t L, w;
  static constexpr bool kNanFillEmpty = false;
  struct Row { int64_t lo; int64_t width; int64_t n; };
  __device__ __forceinline__ Row open(int64_t, int64_t i) const {
    Row r;
    r.lo = (i - w > 0) ? (i - w) : 0;
    int64_t hi = (i + w + 1 < L) ? (i + w + 1) : L;
    r.width = hi - r.lo;
    r.n = L - r.width;
    return r;
  }
  __device__ __forceinline__ int32_t slot(const Row& r, int64_t t) const {
    return (int32_t)(t < r.lo ? t : t + r.width);
  }
};

// ---- Global-no-local, both row kinds, membership by scanning the list (visited-pair dump only) -------
struct GnlDumpCols {
  GnlCols list;            // list.global_bits is not used here
  GnlGlobalRowCols strip;
  static constexpr bool kNanFillEmpty = false;
  struct Row { bool is_global; GnlCols::Row a; GnlGlobalRowCols::Row b; int64_t n; };
  __device__ __forceinline__ Row open(int64_t r, int64_t i) const {
    Row row;
    row.is_global = false;
    for (int64_t t = 0; t < list.nG; ++t) row.is_global |= ((int64_t)list.G[t] == i);
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
