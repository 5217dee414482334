// Host side of the tiled tensor-core path: decides whether a banded problem goes to it, builds the TMA
// tensor maps (one set per residue class of a dilated mask) and launches band_forward_kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>

#include "../../include/spfa_b200.h"
#include "gather_kernels.cuh"
#include "tile_kernels_sm100.cuh"

namespace spfa {

constexpr int SPFA_TILE_NOT_TAKEN = 1;
constexpr int64_t kTileMinHalfWidth = 32;  // AUTO: narrower bands stay on the exact FP32 gather path
constexpr int64_t kTileMaxStride = 16;

extern std::atomic<int64_t> g_launches;

// Kernel shape per head dimension. d <= 64: one 128-row sub-tile per CTA, 64-key tiles, two K and two V stages
// (96 KB of shared memory, 256 TMEM columns, 128 registers x 256 threads), so that TWO CTAs share an SM and one
// CTA's prologue, epilogue and softmax phases overlap the other's MMAs. d = 128: the Q tile alone is 64 KB per
// sub-tile, so two CTAs per SM only fit with 32-key tiles and single K/V stages, which measured 5-10 % slower
// than one CTA of two sub-tiles per SM with 64-key tiles, one K and two V stages (224 KB of shared memory): that is
// what d = 128 uses.
// Three CTAs per SM for d <= 64 (32-key tiles, 128 TMEM columns, 80 registers x 256 threads) measured 10-20 %
// slower than two: S MMAs with N = 32 cost as much per instruction as with N = 64.
template <int D>
struct TileCfg {
  static constexpr int BN = 64, NS = (D == 128) ? 1 : 2, NSV = 2, NSUB = (D == 128) ? 2 : 1;
  static constexpr int kRows = 128 * NSUB, kCtasPerSm = (D == 128) ? 1 : 2;
};
// Global-no-local at d = 128 streams: its two launches get shapes of their own (one 128-row sub-tile per CTA).
// Ordinary rows x the few gathered listed keys: the work of a CTA is "Q tile in, O tile out", so it is sized for TWO
// CTAs per SM (32-key tiles, single stages: 97 KB) and one CTA's loads overlap the other's epilogue.
// Listed rows x all keys: one CTA walks a long key range, so it gets two K stages (K tiles were the exposed latency
// with one) and fills the SM alone.
struct GnlRowsCfg128 {
  static constexpr int BN = 32, NS = 1, NSV = 1, NSUB = 1, kRows = 128, kCtasPerSm = 2;
};
struct GnlKeysCfg128 {
  static constexpr int BN = 64, NS = 2, NSV = 2, NSUB = 1, kRows = 128, kCtasPerSm = 1;
};
template <int D> struct GnlRowsCfg { using type = TileCfg<D>; };
template <> struct GnlRowsCfg<128> { using type = GnlRowsCfg128; };
template <int D> struct GnlKeysCfg { using type = TileCfg<D>; };
template <> struct GnlKeysCfg<128> { using type = GnlKeysCfg128; };
inline int tile_bn(int d) { return d == 128 ? TileCfg<128>::BN : TileCfg<64>::BN; }
inline int tile_rows_per_cta(int d) { return d == 128 ? TileCfg<128>::kRows : 128; }
inline int tile_ctas_per_sm(int d) { return d == 128 ? TileCfg<128>::kCtasPerSm : TileCfg<64>::kCtasPerSm; }

// Error word of the tiled kernels (bounded waits record a code here). One per device context.
__device__ int g_tile_error;

typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                           const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                           CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                           CUtensorMapFloatOOBfill);

inline TensorMapEncodeTiledFn tensor_map_encoder() {
  static TensorMapEncodeTiledFn fn = []() -> TensorMapEncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<TensorMapEncodeTiledFn>(p);
  }();
  return fn;
}

// [rows, d] fp32 matrix with a row pitch of `pitch_bytes`, fetched as boxes of box_rows x 32 floats with the
// 128-byte swizzle the MMA descriptors expect (16-byte units for K-major operands, 32-byte units for the
// MN-major V operand). Rows outside [0, rows) read as zeros.
// `slices` such matrices lie `slice_bytes` apart (a batch of heads); the third coordinate of a load picks one.
inline bool make_row_map(CUtensorMap* tm, const float* base, int d, int64_t rows, int64_t pitch_bytes, int box_rows,
                         bool mn_major = false, int64_t slices = 1, int64_t slice_bytes = 0, bool plain_f32 = false) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return false;
  if (slices <= 1 || slice_bytes <= 0) {
    slices = 1;
    slice_bytes = (rows > 0 ? rows : 1) * pitch_bytes;  // never used to address anything: z is 0
  }
  cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)rows, (cuuint64_t)slices};
  cuuint64_t strides[2] = {(cuuint64_t)pitch_bytes, (cuuint64_t)slice_bytes};
  cuuint32_t box[3] = {32u, (cuuint32_t)box_rows, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  // plain_f32: the map of an output tensor (bulk stores of fp32 values); the operand maps are typed tf32
  return enc(tm, plain_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 3,
             const_cast<float*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// setmaxnreg.inc blocks without a timeout when the CTA's register pool cannot satisfy it, so the kernel is only
// launched if the pool the compiler's allocation gives a CTA covers the two budgets of Geo. The answer depends on
// the build alone (a different nvcc may assign fewer registers): it is computed once per instantiation and device.
// Callers on SPFA_PATH_AUTO fall back to the gather path when it is false; a forced tiled call reports
// SPFA_ERR_REGISTER_BUDGET.
template <int D, bool EXPL, class C = TileCfg<D>>
bool band_kernel_usable() {
  using G = tile::Geo<C::NSUB>;
  static std::atomic<int> cached[64];  // per device: 0 unknown, 1 usable, 2 not
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    cudaFuncAttributes attr;
    auto kern = tile::band_forward_kernel<D, C::BN, C::NS, C::NSUB, EXPL, C::NSV>;
    const bool ok = cudaFuncGetAttributes(&attr, kern) == cudaSuccess &&
                    attr.numRegs * G::kThreads >= G::kRegsSoftmax * 128 * C::NSUB + G::kRegsAux * 128;
    v = ok ? 1 : 2;
    cached[dev].store(v, std::memory_order_relaxed);
  }
  return v == 1;
}

// Common launch steps of band_forward_kernel: register-budget guard, shared-memory opt-in, error word.
// tmK2 / tmV2: the second key source of mode 4 (gathered listed keys); every other mode passes null and the first
// pair is handed to the kernel twice.
template <int D, bool EXPL = false, class C = TileCfg<D>>
int launch_band_raw(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, float* m, float* l, float* O,
                    const tile::BandParams& prm_in, dim3 grid, cudaStream_t st, const CUtensorMap* tmK2p = nullptr,
                    const CUtensorMap* tmV2p = nullptr, const CUtensorMap* tmOp = nullptr) {
  const CUtensorMap& tmK2 = tmK2p ? *tmK2p : tmK;
  const CUtensorMap& tmV2 = tmV2p ? *tmV2p : tmV;
  const CUtensorMap& tmO = tmOp ? *tmOp : tmQ;  // O's map (Q's geometry) enables the bulk store of finished tiles
  tile::BandParams prm = prm_in;
  prm.tma_store = tmOp ? 1 : 0;
  constexpr int NSUB = C::NSUB;
  using P = tile::Plan<D, C::BN, C::NS, NSUB, C::NSV>;
  using G = tile::Geo<NSUB>;
  auto kern = tile::band_forward_kernel<D, C::BN, C::NS, NSUB, EXPL, C::NSV>;
  if (!band_kernel_usable<D, EXPL, C>()) return SPFA_ERR_REGISTER_BUDGET;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P::kDynSmem) != cudaSuccess)
    return SPFA_ERR_LAUNCH;
  int* err = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&err), g_tile_error) != cudaSuccess) return SPFA_ERR_LAUNCH;
  if (prm.overlap & 2) {  // may start while the previous launch of the stream is still running (see BandParams)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(G::kThreads);
    cfg.dynamicSmemBytes = P::kDynSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, tmQ, tmK, tmV, tmK2, tmV2, tmO, m, l, O, prm, err) != cudaSuccess)
      return SPFA_ERR_LAUNCH;
  } else {
    kern<<<grid, G::kThreads, P::kDynSmem, st>>>(tmQ, tmK, tmV, tmK2, tmV2, tmO, m, l, O, prm, err);
  }
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? (int)SPFA_OK : (int)SPFA_ERR_LAUNCH;
}

// n_slices > 1: Q, O are [n_slices, rows of the shard, d], K, V [n_slices, L, d], m, l [n_slices, rows]: one launch
// per residue class covers every slice (grid.z).
template <int D>
int launch_band(const float* Q, const float* K, const float* V, float* m, float* l, float* O, int64_t L, int64_t w,
                int64_t s, int64_t row_begin, int64_t row_end, cudaStream_t st, int64_t n_slices = 1) {
  using C = TileCfg<D>;
  constexpr int BN = C::BN;
  bool launched = false;  // residue classes write disjoint rows: consecutive launches may overlap
  for (int64_t r = 0; r < s && r < L; ++r) {
    tile::BandParams prm{};
    prm.n_keys = (L - r + s - 1) / s;
    int64_t u_first = (row_begin > r) ? (row_begin - r + s - 1) / s : 0;
    int64_t u_end = (row_end > r) ? (row_end - r + s - 1) / s : 0;
    if (u_end > prm.n_keys) u_end = prm.n_keys;
    if (u_end <= u_first) continue;
    prm.u_q_first = u_first;
    prm.n_q = u_end - u_first;
    prm.w = w;
    prm.s = s;
    prm.r = r;
    prm.row_begin = row_begin;
    prm.scale_log2e = (1.0f / sqrtf((float)D)) * kLog2e;
    prm.slice_o = (row_end - row_begin) * D;
    prm.slice_ml = row_end - row_begin;
    CUtensorMap tmQ, tmK, tmV, tmO;
    const int64_t pitch = s * D * (int64_t)sizeof(float);
    const int64_t q_slice = (row_end - row_begin) * D * (int64_t)sizeof(float), kv_slice = L * D * (int64_t)sizeof(float);
    if (!make_row_map(&tmQ, Q + (r + u_first * s - row_begin) * D, D, prm.n_q, pitch, 128, false, n_slices, q_slice) ||
        !make_row_map(&tmO, O + (r + u_first * s - row_begin) * D, D, prm.n_q, pitch, 128, false, n_slices, q_slice, true) ||
        !make_row_map(&tmK, K + r * D, D, prm.n_keys, pitch, BN, false, n_slices, kv_slice) ||
        !make_row_map(&tmV, V + r * D, D, prm.n_keys, pitch, BN, /*mn_major=*/true, n_slices, kv_slice))
      return SPFA_ERR_LAUNCH;
    const int64_t grid = (prm.n_q + C::kRows - 1) / C::kRows;
    if (grid > 0x7fffffffLL || n_slices > 65535) return SPFA_ERR_TOO_LARGE;
    prm.overlap = ((r + 1 < s && r + 1 < L) ? 1 : 0) | (launched ? 2 : 0);
    const int rc = launch_band_raw<D>(tmQ, tmK, tmV, m, l, O, prm, dim3((unsigned)grid, 1, (unsigned)n_slices), st, nullptr,
                                      nullptr, &tmO);
    if (rc) return rc;
    launched = true;
  }
  return SPFA_OK;
}

// Band |u_q - u_k| <= w on every residue class of stride s (s = 1: Local; s = dil+1: Local-1D-dilated).
inline int tiled_band_forward(const float* Q, const float* K, const float* V, float* m, float* l, float* O, int64_t L,
                              int d, int64_t w, int64_t s, int64_t row_begin, int64_t row_end, bool forced,
                              cudaStream_t st, int64_t n_slices = 1) {
  const bool shape_ok = (d == 32 || d == 64 || d == 128) && s >= 1 && s <= kTileMaxStride && row_end > row_begin;
  if (!shape_ok) return forced ? (int)SPFA_ERR_BAD_ARG : SPFA_TILE_NOT_TAKEN;
  if (!forced && w < kTileMinHalfWidth) return SPFA_TILE_NOT_TAKEN;
  const bool usable = d == 32 ? band_kernel_usable<32, false>()
                              : (d == 64 ? band_kernel_usable<64, false>() : band_kernel_usable<128, false>());
  if (!usable) return forced ? (int)SPFA_ERR_REGISTER_BUDGET : SPFA_TILE_NOT_TAKEN;
  switch (d) {
    case 32: return launch_band<32>(Q, K, V, m, l, O, L, w, s, row_begin, row_end, st, n_slices);
    case 64: return launch_band<64>(Q, K, V, m, l, O, L, w, s, row_begin, row_end, st, n_slices);
    case 128: return launch_band<128>(Q, K, V, m, l, O, L, w, s, row_begin, row_end, st, n_slices);
  }
  return SPFA_TILE_NOT_TAKEN;
}

// ---- Global-no-local on the tiled path ---------------------------------------------------------------
// The listed global rows are sorted once (<= 1024 of them: one CTA, rank sort) and their Q/K/V rows
// gathered into contiguous scratch. Then two launches of band_forward_kernel in its "every key except an
// interval" modes cover the mask: mode 1, every ordinary row against the gathered global keys; mode 2, the
// gathered global rows against all keys, key range split over the grid, followed by the combine pass.
constexpr int kGnlTiledMaxGlobals = 1024;
// Ordinary rows see at most n_global keys; with very few keys per row the TF32 error of a tile is not
// averaged down, so below this count they stay on the exact FP32 gather kernel (only the global rows, which
// see ~L keys each, go through the tiles).
constexpr int kGnlTiledMinGlobalsForRows = 32;

// One warp per sorted entry: copies the entry's K and V rows (always) and its Q row (if the row belongs to
// this shard) into the contiguous scratch; entries that are invalid get zero rows. live[e] = 1 for the first
// occurrence of a row that lies in the shard (the combine pass writes exactly those rows).
struct GnlGatherArgs {
  const float *Q, *K, *V;
  int d;
  int64_t row_begin, row_end;
  float *QG, *KG, *VG;
  uint8_t* live;
};

__device__ __forceinline__ void gnl_gather_entry(const int32_t* sorted, int e, int lane, const GnlGatherArgs& a) {
  const int32_t g = sorted[e];
  const bool valid = g != 0x7fffffff;
  const bool mine = valid && g >= a.row_begin && g < a.row_end;
  const bool first = (e == 0) || (sorted[e - 1] != g);
  for (int c = lane * 4; c < a.d; c += 128) {
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(a.KG + (size_t)e * a.d + c) = valid ? ldg4(a.K + (size_t)g * a.d + c) : z;
    *reinterpret_cast<float4*>(a.VG + (size_t)e * a.d + c) = valid ? ldg4(a.V + (size_t)g * a.d + c) : z;
    *reinterpret_cast<float4*>(a.QG + (size_t)e * a.d + c) = mine ? ldg4(a.Q + (size_t)(g - a.row_begin) * a.d + c) : z;
  }
  if (lane == 0) a.live[e] = (mine && first) ? 1 : 0;
}

template <bool GATHER>
__global__ void gnl_sort_globals_kernel(const int32_t* __restrict__ G, int nG, int64_t L, int32_t* __restrict__ sorted,
                                        int32_t* __restrict__ n_valid, const GnlGatherArgs ga) {
  __shared__ int32_t g[kGnlTiledMaxGlobals];
  __shared__ int cnt;
  const int t = threadIdx.x;
  if (t == 0) cnt = 0;
  int32_t v = 0x7fffffff;
  if (t < nG) {
    const int32_t x = G[t];
    if (x >= 0 && (int64_t)x < L) v = x;
  }
  g[t] = v;
  __syncthreads();
  if (t < nG) {
    int rank = 0;
    for (int u = 0; u < nG; ++u) rank += (g[u] < v) || (g[u] == v && u < t);
    sorted[rank] = v;  // invalid entries (INT_MAX) end up last
    if (v != 0x7fffffff) atomicAdd(&cnt, 1);
  }
  __syncthreads();
  if (t == 0) *n_valid = cnt;
  if (GATHER)  // the order is complete (the barrier above orders this CTA's writes of `sorted`): copy the rows
    for (int e = t >> 5; e < nG; e += kGnlTiledMaxGlobals / 32) gnl_gather_entry(sorted, e, t & 31, ga);
}

__global__ void gnl_gather_globals_kernel(const int32_t* __restrict__ sorted, int nG, const GnlGatherArgs a) {
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= nG) return;
  gnl_gather_entry(sorted, e, lane, a);
}

// Short lists (the usual case: tens of global tokens) are sorted and gathered by ONE launch: the sorting CTA's 32 warps
// copy the rows themselves once the order is known; a second tiny launch costs more than the copies.
constexpr int kGnlFusedGatherMax = 128;

// Sorts the listed rows and gathers their Q/K/V rows: one launch for short lists, two for long ones.
inline int launch_gnl_sort_gather(const int32_t* G, int64_t nG, int64_t L, int32_t* sorted, int32_t* n_valid,
                                  const GnlGatherArgs& ga, cudaStream_t st) {
  if (nG <= kGnlFusedGatherMax) {
    gnl_sort_globals_kernel<true><<<1, kGnlTiledMaxGlobals, 0, st>>>(G, (int)nG, L, sorted, n_valid, ga);
    g_launches.fetch_add(1);
  } else {
    gnl_sort_globals_kernel<false><<<1, kGnlTiledMaxGlobals, 0, st>>>(G, (int)nG, L, sorted, n_valid, ga);
    g_launches.fetch_add(1);
    gnl_gather_globals_kernel<<<(unsigned)((nG + 3) / 4), 128, 0, st>>>(sorted, (int)nG, ga);
    g_launches.fetch_add(1);
  }
  return cudaGetLastError() == cudaSuccess ? (int)SPFA_OK : (int)SPFA_ERR_LAUNCH;
}

struct GnlTiledPlan {
  int bn, n_split;
  int64_t kv_chunk;
  size_t off_sorted, off_nvalid, off_live, off_qg, off_kg, off_vg, off_part, total;
};

inline GnlTiledPlan gnl_tiled_plan(int64_t L, int d, int64_t nG) {
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  GnlTiledPlan p;
  p.bn = tile_bn(d);  // the listed-rows launch uses 64-key tiles for every d
  const int rows_per_cta = (d == 128) ? GnlKeysCfg128::kRows : 128;
  const int ctas_per_sm = (d == 128) ? GnlKeysCfg128::kCtasPerSm : tile_ctas_per_sm(d);
  const int64_t tiles = (L + p.bn - 1) / p.bn;
  const int64_t q_tiles = (nG + rows_per_cta - 1) / rows_per_cta;
  int64_t ctas = 148 * ctas_per_sm / q_tiles;
  if (ctas < 1) ctas = 1;
  int64_t chunk_tiles = (tiles + ctas - 1) / ctas;
  if (chunk_tiles < 2) chunk_tiles = 2;
  p.kv_chunk = chunk_tiles * p.bn;
  p.n_split = (int)((L + p.kv_chunk - 1) / p.kv_chunk);
  p.off_sorted = 0;
  p.off_nvalid = up((size_t)nG * 4);
  p.off_live = p.off_nvalid + 256;
  p.off_qg = p.off_live + up((size_t)nG);
  p.off_kg = p.off_qg + up((size_t)nG * d * 4);
  p.off_vg = p.off_kg + up((size_t)nG * d * 4);
  p.off_part = p.off_vg + up((size_t)nG * d * 4);
  p.total = p.off_part + up((size_t)nG * p.n_split * (d + 4) * 4);
  return p;
}

inline bool gnl_tiled_shape_ok(int d, int64_t nG) {
  if (!((d == 32 || d == 64 || d == 128) && nG >= 1 && nG <= kGnlTiledMaxGlobals)) return false;
  return d == 32 ? band_kernel_usable<32, false>()
                 : (d == 64 ? band_kernel_usable<64, false>()
                            : (band_kernel_usable<128, false, GnlRowsCfg128>() && band_kernel_usable<128, false, GnlKeysCfg128>()));
}

template <int D>
int launch_gnl_tiled(const float* Q, const float* K, const float* V, float* m, float* l, float* O, const int32_t* G,
                     int64_t nG, int64_t L, int64_t w, int64_t row_begin, int64_t row_end, char* ws,
                     const GnlTiledPlan& plan, bool ordinary_rows_too, cudaStream_t st) {
  int32_t* sorted = reinterpret_cast<int32_t*>(ws + plan.off_sorted);
  int32_t* n_valid = reinterpret_cast<int32_t*>(ws + plan.off_nvalid);
  uint8_t* live = reinterpret_cast<uint8_t*>(ws + plan.off_live);
  float* QG = reinterpret_cast<float*>(ws + plan.off_qg);
  float* KG = reinterpret_cast<float*>(ws + plan.off_kg);
  float* VG = reinterpret_cast<float*>(ws + plan.off_vg);
  float* partials = reinterpret_cast<float*>(ws + plan.off_part);
  if (launch_gnl_sort_gather(G, nG, L, sorted, n_valid, GnlGatherArgs{Q, K, V, D, row_begin, row_end, QG, KG, VG, live}, st))
    return SPFA_ERR_LAUNCH;
  using CR = typename GnlRowsCfg<D>::type;  // ordinary rows x listed keys
  using CK = typename GnlKeysCfg<D>::type;  // listed rows x all keys
  const int64_t pitch = D * (int64_t)sizeof(float);
  const int64_t n_rows = row_end - row_begin;
  tile::BandParams prm{};
  prm.w = w;
  prm.s = 1;
  prm.r = 0;
  prm.row_begin = row_begin;
  prm.scale_log2e = (1.0f / sqrtf((float)D)) * kLog2e;
  prm.sorted = sorted;
  prm.n_valid = n_valid;
  CUtensorMap tmQ, tmK, tmV;
  // mode 1: ordinary rows of the shard against the gathered global keys
  prm.mode = 1;
  prm.n_keys = nG;
  prm.n_listed = nG;
  prm.u_q_first = row_begin;
  prm.n_q = n_rows;
  CUtensorMap tmO;
  if (!make_row_map(&tmQ, Q, D, n_rows, pitch, 128) || !make_row_map(&tmK, KG, D, nG, pitch, CR::BN) ||
      !make_row_map(&tmV, VG, D, nG, pitch, CR::BN, /*mn_major=*/true) ||
      !make_row_map(&tmO, O, D, n_rows, pitch, 128, false, 1, 0, true))
    return SPFA_ERR_LAUNCH;
  int rc = SPFA_OK;
  // the two launches write disjoint things (ordinary rows / partial states of the listed rows): they may overlap
  prm.overlap = 1;
  if (ordinary_rows_too)
    rc = launch_band_raw<D, false, CR>(tmQ, tmK, tmV, m, l, O, prm, dim3((unsigned)((n_rows + CR::kRows - 1) / CR::kRows)),
                                       st, nullptr, nullptr, &tmO);
  if (rc) return rc;
  // mode 2: the gathered global rows against every key, key range split over grid.y
  prm.mode = 2;
  prm.overlap = ordinary_rows_too ? 2 : 0;
  prm.n_keys = L;
  prm.u_q_first = 0;
  prm.n_q = nG;
  prm.row_begin = 0;
  prm.kv_chunk = plan.kv_chunk;
  prm.partials = partials;
  prm.n_split = plan.n_split;
  if (!make_row_map(&tmQ, QG, D, nG, pitch, 128) || !make_row_map(&tmK, K, D, L, pitch, CK::BN) ||
      !make_row_map(&tmV, V, D, L, pitch, CK::BN, /*mn_major=*/true))
    return SPFA_ERR_LAUNCH;
  rc = launch_band_raw<D, false, CK>(tmQ, tmK, tmV, m, l, O, prm,
                                     dim3((unsigned)((nG + CK::kRows - 1) / CK::kRows), (unsigned)plan.n_split), st);
  if (rc) return rc;
  combine_partials_kernel<D><<<(unsigned)nG, kCombineWarps * 32, 0, st>>>(
      partials, sorted, live, (int)nG, row_begin, row_end, plan.n_split, m, l, O);
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? (int)SPFA_OK : (int)SPFA_ERR_LAUNCH;
}

inline int tiled_gnl_forward(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                             const int32_t* G, int64_t nG, int64_t L, int d, int64_t w, int64_t row_begin,
                             int64_t row_end, char* ws, bool ordinary_rows_too, cudaStream_t st) {
  const GnlTiledPlan plan = gnl_tiled_plan(L, d, nG);
  switch (d) {
    case 32: return launch_gnl_tiled<32>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, ws, plan, ordinary_rows_too, st);
    case 64: return launch_gnl_tiled<64>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, ws, plan, ordinary_rows_too, st);
    case 128: return launch_gnl_tiled<128>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, ws, plan, ordinary_rows_too, st);
  }
  return SPFA_ERR_EMBED_DIM;
}

// ---- fused Local + Global-no-local ("BigBird" without its random part) -----------------------------------------
// Mask = { |i - j| <= w }  union  { i or j listed, |i - j| > w }. One pass of band_forward_kernel in mode 4 gives every
// row that is not listed its band tiles and its listed-key tiles (one read of Q, one read-modify-write of O); the
// listed rows attend to every key and run as the split strip of the Global-no-local path with an empty exclusion
// window, followed by the combine pass. Scratch: the Global-no-local tiled plan's.
template <int D>
int launch_bigbird_tiled(const float* Q, const float* K, const float* V, float* m, float* l, float* O, const int32_t* G,
                         int64_t nG, int64_t L, int64_t w, int64_t row_begin, int64_t row_end, char* ws,
                         const GnlTiledPlan& plan, cudaStream_t st) {
  int32_t* sorted = reinterpret_cast<int32_t*>(ws + plan.off_sorted);
  int32_t* n_valid = reinterpret_cast<int32_t*>(ws + plan.off_nvalid);
  uint8_t* live = reinterpret_cast<uint8_t*>(ws + plan.off_live);
  float* QG = reinterpret_cast<float*>(ws + plan.off_qg);
  float* KG = reinterpret_cast<float*>(ws + plan.off_kg);
  float* VG = reinterpret_cast<float*>(ws + plan.off_vg);
  float* partials = reinterpret_cast<float*>(ws + plan.off_part);
  if (launch_gnl_sort_gather(G, nG, L, sorted, n_valid, GnlGatherArgs{Q, K, V, D, row_begin, row_end, QG, KG, VG, live}, st))
    return SPFA_ERR_LAUNCH;
  using CB = TileCfg<D>;                    // band + listed keys, every row of the shard
  using CK = typename GnlKeysCfg<D>::type;  // listed rows x all keys
  const int64_t pitch = D * (int64_t)sizeof(float);
  const int64_t n_rows = row_end - row_begin;
  tile::BandParams prm{};
  prm.mode = 4;
  prm.n_keys = L;
  prm.n_listed = nG;
  prm.u_q_first = row_begin;
  prm.n_q = n_rows;
  prm.w = w;
  prm.s = 1;
  prm.r = 0;
  prm.row_begin = row_begin;
  prm.scale_log2e = (1.0f / sqrtf((float)D)) * kLog2e;
  prm.sorted = sorted;
  prm.n_valid = n_valid;
  prm.overlap = 1;  // the strip launch below writes other things (partial states): it may start beside this one
  CUtensorMap tmQ, tmK, tmV, tmK2, tmV2, tmO;
  if (!make_row_map(&tmQ, Q, D, n_rows, pitch, 128) || !make_row_map(&tmO, O, D, n_rows, pitch, 128, false, 1, 0, true) ||
      !make_row_map(&tmK, K, D, L, pitch, CB::BN) ||
      !make_row_map(&tmV, V, D, L, pitch, CB::BN, /*mn_major=*/true) || !make_row_map(&tmK2, KG, D, nG, pitch, CB::BN) ||
      !make_row_map(&tmV2, VG, D, nG, pitch, CB::BN, /*mn_major=*/true))
    return SPFA_ERR_LAUNCH;
  int rc = launch_band_raw<D, false, CB>(tmQ, tmK, tmV, m, l, O, prm, dim3((unsigned)((n_rows + CB::kRows - 1) / CB::kRows)),
                                         st, &tmK2, &tmV2, &tmO);
  if (rc) return rc;
  prm.mode = 2;
  prm.overlap = 2;
  prm.w = -1;  // an empty exclusion window: the listed rows attend to every key
  prm.n_keys = L;
  prm.u_q_first = 0;
  prm.n_q = nG;
  prm.row_begin = 0;
  prm.kv_chunk = plan.kv_chunk;
  prm.partials = partials;
  prm.n_split = plan.n_split;
  if (!make_row_map(&tmQ, QG, D, nG, pitch, 128) || !make_row_map(&tmK, K, D, L, pitch, CK::BN) ||
      !make_row_map(&tmV, V, D, L, pitch, CK::BN, /*mn_major=*/true))
    return SPFA_ERR_LAUNCH;
  rc = launch_band_raw<D, false, CK>(tmQ, tmK, tmV, m, l, O, prm,
                                     dim3((unsigned)((nG + CK::kRows - 1) / CK::kRows), (unsigned)plan.n_split), st);
  if (rc) return rc;
  combine_partials_kernel<D><<<(unsigned)nG, kCombineWarps * 32, 0, st>>>(partials, sorted, live, (int)nG, row_begin, row_end,
                                                                         plan.n_split, m, l, O);
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? (int)SPFA_OK : (int)SPFA_ERR_LAUNCH;
}

inline int tiled_bigbird_forward(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                 const int32_t* G, int64_t nG, int64_t L, int d, int64_t w, int64_t row_begin,
                                 int64_t row_end, char* ws, cudaStream_t st) {
  const GnlTiledPlan plan = gnl_tiled_plan(L, d, nG);
  switch (d) {
    case 32: return launch_bigbird_tiled<32>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, ws, plan, st);
    case 64: return launch_bigbird_tiled<64>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, ws, plan, st);
    case 128: return launch_bigbird_tiled<128>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, ws, plan, st);
  }
  return SPFA_ERR_EMBED_DIM;
}

// Self-test of the bounded waits: one thread waits on an mbarrier that nothing ever arrives at. After the wait
// limit (tile::kWaitNs) it must give up, record `code` in the error word and return, leaving the context usable.
__global__ void wait_limit_selftest_kernel(int* err, int code) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tile::mbar_init(tile::smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) tile::mbar_wait(tile::smem_u32(&bar), 0, &abort_flag, err, code);
}

inline int launch_wait_limit_selftest(int code, cudaStream_t st) {
  int* err = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&err), g_tile_error) != cudaSuccess) return SPFA_ERR_LAUNCH;
  wait_limit_selftest_kernel<<<1, 32, 0, st>>>(err, code);
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? (int)SPFA_OK : (int)SPFA_ERR_LAUNCH;
}

// Reads and clears the tiled kernels' error word (synchronises the device). 0 = no error.
inline int read_and_clear_tile_error() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_tile_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_tile_error, &zero, sizeof(int));
  return v;
}

}  // namespace spfa
