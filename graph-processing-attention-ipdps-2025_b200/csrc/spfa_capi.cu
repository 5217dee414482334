// C ABI of the library (declared in include/spfa_b200.h): argument validation, workspace carving and
// kernel dispatch. No torch types, no exceptions, no allocation.
#include "../../include/spfa_b200.h"

#include <atomic>
#include <cmath>

#include "block_kernels.cuh"
#include "capi_common.cuh"
#include "explicit_plan.cuh"
#include "gather_generic.cuh"
#include "gather_kernels.cuh"
#include "mask_builders.cuh"
#include "tile_dispatch.cuh"

namespace spfa {

std::atomic<int64_t> g_launches{0};
thread_local PathCell g_path{SPFA_PATH_AUTO};
thread_local PathCell g_last_path{SPFA_PATH_GATHER};

// Head dimensions with specialised kernels; every other d in [1, kGenericMaxD] takes the generic gather kernel.
inline bool specialised_d(int d) { return d == 16 || d == 32 || d == 64 || d == 128; }
inline bool supported_d(int d) { return d >= 1 && d <= kGenericMaxD; }

template <int D, class Cols>
int launch_gather(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                  const Cols& cols, int64_t row_begin, int64_t n_rows, int use_nan, cudaStream_t st, int64_t n_slices = 1,
                  int64_t kv_slice = 0) {
  if (n_rows <= 0) return SPFA_OK;
  const int per_cta = rows_per_cta_for(n_rows, n_slices);
  const int64_t blocks = (n_rows + per_cta - 1) / per_cta;
  if (blocks > 0x7fffffffLL || n_slices > 65535) return SPFA_ERR_TOO_LARGE;
  const float scale = 1.0f / sqrtf((float)D);
  gather_rows_kernel<D, Cols><<<dim3((unsigned)blocks, (unsigned)n_slices), kRowWarps * 32, 0, st>>>(
      Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, scale, kv_slice, per_cta);
  g_launches.fetch_add(1);
  g_last_path.store(SPFA_PATH_GATHER);
  return launch_status();
}

template <int VW, int NC, class Cols>
int launch_gather_generic(const float* Q, const float* K, const float* V, float* m, float* l, float* O, const Cols& cols,
                          int64_t row_begin, int64_t n_rows, int use_nan, int d, cudaStream_t st) {
  if (n_rows <= 0) return SPFA_OK;
  const int64_t blocks = (n_rows + kRowWarps - 1) / kRowWarps;
  if (blocks > 0x7fffffffLL) return SPFA_ERR_TOO_LARGE;
  const float scale = 1.0f / sqrtf((float)d);
  gather_rows_generic_kernel<float, VW, NC, Cols><<<(unsigned)blocks, kRowWarps * 32, (size_t)kRowWarps * d * sizeof(float), st>>>(
      Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, scale, d);
  g_launches.fetch_add(1);
  g_last_path.store(SPFA_PATH_GATHER);
  return launch_status();
}

// Any d in [1, kGenericMaxD]: 128-bit pieces when the rows allow it, scalar pieces otherwise.
template <class Cols>
int dispatch_gather_generic(int d, const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                            const Cols& cols, int64_t row_begin, int64_t n_rows, int use_nan, cudaStream_t st) {
  if (d < 1 || d > kGenericMaxD) return SPFA_ERR_EMBED_DIM;
  if (d % 4 == 0)
    return d <= 256 ? launch_gather_generic<4, 2, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, d, st)
                    : launch_gather_generic<4, 8, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, d, st);
  return d <= 256 ? launch_gather_generic<1, 8, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, d, st)
                  : launch_gather_generic<1, 32, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, d, st);
}

// n_slices > 1 (batched calls): one launch for all slices where a specialised kernel exists, else one per slice.
template <class Cols>
int dispatch_gather(int d, const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                    const Cols& cols, int64_t row_begin, int64_t n_rows, int use_nan, cudaStream_t st, int64_t n_slices = 1,
                    int64_t kv_slice = 0) {
  switch (d) {
    case 16: return launch_gather<16, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st, n_slices, kv_slice);
    case 32: return launch_gather<32, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st, n_slices, kv_slice);
    case 64: return launch_gather<64, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st, n_slices, kv_slice);
    case 128: return launch_gather<128, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st, n_slices, kv_slice);
  }
  for (int64_t z = 0; z < n_slices; ++z) {
    const int rc = dispatch_gather_generic(d, Q + z * n_rows * d, K + z * kv_slice, V + z * kv_slice, m + z * n_rows,
                                           l + z * n_rows, O + z * n_rows * d, cols, row_begin, n_rows, use_nan, st);
    if (rc) return rc;
  }
  return SPFA_OK;
}

inline int check_common(const void* Q, const void* K, const void* V, const void* m, const void* l, const void* O,
                        int d) {
  if (!supported_d(d)) return SPFA_ERR_EMBED_DIM;
  if (!Q || !K || !V || !m || !l || !O) return SPFA_ERR_BAD_ARG;
  if (d % 4 == 0) {  // rows are read and written in 128-bit pieces
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return SPFA_ERR_BAD_ARG;
  } else if (!aligned4(Q) || !aligned4(K) || !aligned4(V) || !aligned4(O)) {
    return SPFA_ERR_BAD_ARG;
  }
  return SPFA_OK;
}

// Split of the global rows' key range: enough warps for a few waves over 148 SMs, ranges a multiple
// of 32 slots.
struct GnlPlan {
  int n_split;
  int64_t slots_per_split;
  size_t off_bits, off_live, off_part, total;
};

inline GnlPlan gnl_plan(int64_t L, int d, int64_t nG) {
  GnlPlan p;
  int64_t want = (148 * 64 + nG - 1) / (nG > 0 ? nG : 1);  // ~64 warps per SM in flight
  int64_t max_split = (L + 255) / 256;
  if (want < 1) want = 1;
  if (want > max_split) want = max_split;
  if (want > 1024) want = 1024;
  int64_t sps = (L + want - 1) / want;
  sps = (sps + 31) / 32 * 32;
  p.slots_per_split = sps;
  p.n_split = (int)((L + sps - 1) / sps);
  p.off_bits = 0;
  p.off_live = align_up((size_t)((L + 31) / 32) * 4);
  p.off_part = p.off_live + align_up((size_t)nG);
  p.total = p.off_part + align_up((size_t)nG * p.n_split * (d + 4) * sizeof(float));
  return p;
}

template <int D>
int launch_gnl_global_rows(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                           const int32_t* G, int64_t nG, int64_t L, int64_t w, int64_t row_begin, int64_t row_end,
                           const GnlPlan& plan, const uint8_t* live, float* partials, cudaStream_t st) {
  GnlGlobalRowCols cols{L, w};
  const float scale = 1.0f / sqrtf((float)D);
  dim3 grid((unsigned)((nG + kGatherWarps - 1) / kGatherWarps), (unsigned)plan.n_split);
  gather_split_rows_kernel<D, GnlGlobalRowCols><<<grid, kGatherWarps * 32, 0, st>>>(
      Q, K, V, cols, G, live, (int)nG, row_begin, row_end, plan.n_split, plan.slots_per_split, partials, scale);
  g_launches.fetch_add(1);
  if (launch_status() != SPFA_OK) return SPFA_ERR_LAUNCH;
  combine_partials_kernel<D><<<(unsigned)nG, kCombineWarps * 32, 0, st>>>(
      partials, G, live, (int)nG, row_begin, row_end, plan.n_split, m, l, O);
  g_launches.fetch_add(1);
  return launch_status();
}

// Local-2D-dilated: one CTA per mask block with the block's key rows staged in shared memory (FP32, exact).
template <int D, int NK>
int launch_local2d_block_nk(const float* Q, const float* K, const float* V, float* m, float* l, float* O, int64_t L,
                         int64_t B, int64_t s, int64_t n, int use_nan, int64_t row_begin, int64_t row_end,
                         cudaStream_t st) {
  const size_t smem = block2d_smem_bytes<D>(n);
  auto kern = local2d_block_kernel<D, NK>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return SPFA_ERR_LAUNCH;
  Block2dParams prm;
  prm.L = L;
  prm.B = B;
  prm.s = s;
  prm.n = n;
  prm.row_begin = row_begin;
  prm.row_end = row_end;
  prm.first_block = row_begin / B;
  prm.use_nan = use_nan;
  prm.scale = 1.0f / sqrtf((float)D);
  const int64_t blocks = (row_end - 1) / B - prm.first_block + 1;
  if (blocks > 0x7fffffffLL) return SPFA_ERR_TOO_LARGE;
  kern<<<(unsigned)blocks, kBlockWarps * 32, smem, st>>>(Q, K, V, m, l, O, prm);
  g_launches.fetch_add(1);
  g_last_path.store(SPFA_PATH_GATHER);  // an FP32 SIMT path, same accuracy class as the gather kernels
  return launch_status();
}

template <int D>
int launch_local2d_block(const float* Q, const float* K, const float* V, float* m, float* l, float* O, int64_t L,
                         int64_t B, int64_t s, int64_t n, int use_nan, int64_t row_begin, int64_t row_end,
                         cudaStream_t st) {
  if (n <= 32) return launch_local2d_block_nk<D, 1>(Q, K, V, m, l, O, L, B, s, n, use_nan, row_begin, row_end, st);
  if (n <= 64) return launch_local2d_block_nk<D, 2>(Q, K, V, m, l, O, L, B, s, n, use_nan, row_begin, row_end, st);
  if (n <= 128) return launch_local2d_block_nk<D, 4>(Q, K, V, m, l, O, L, B, s, n, use_nan, row_begin, row_end, st);
  return launch_local2d_block_nk<D, 8>(Q, K, V, m, l, O, L, B, s, n, use_nan, row_begin, row_end, st);
}

// Blocks with 33..64 keys per live row: the register-tiled kernel.
template <int D>
int launch_local2d_tile(const float* Q, const float* K, const float* V, float* m, float* l, float* O, int64_t L, int64_t B,
                        int64_t s, int64_t n, int use_nan, int64_t row_begin, int64_t row_end, cudaStream_t st) {
  const size_t smem = tile2d_smem_bytes<D>();
  auto kern = local2d_tile_kernel<D>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return SPFA_ERR_LAUNCH;
  Block2dParams prm;
  prm.L = L;
  prm.B = B;
  prm.s = s;
  prm.n = n;
  prm.row_begin = row_begin;
  prm.row_end = row_end;
  prm.first_block = row_begin / B;
  prm.use_nan = use_nan;
  prm.scale = 1.0f / sqrtf((float)D);
  const int64_t blocks = (row_end - 1) / B - prm.first_block + 1;
  if (blocks > 0x7fffffffLL) return SPFA_ERR_TOO_LARGE;
  kern<<<(unsigned)blocks, kTile2dThreads, smem, st>>>(Q, K, V, m, l, O, prm);
  g_launches.fetch_add(1);
  g_last_path.store(SPFA_PATH_GATHER);  // exact FP32, the accuracy class of the gather kernels
  return launch_status();
}

template <class F>
inline int with_mask_cols(int kind, int64_t L, int64_t p0, int64_t p1, const int32_t* G, int64_t nG, F&& f) {
  switch (kind) {
    case 0: return f(LocalCols{L, p0});
    case 1: return f(Local1dCols{L, p0, p1 + 1});
    case 2: return f(Local2dCols{L, p0, p1 + 1});
    case 3: {
      if (!G || nG <= 0) return SPFA_ERR_GLOBAL_COUNT;
      GnlDumpCols c;
      c.list = GnlCols{G, nG, L, p0, nullptr};
      c.strip = GnlGlobalRowCols{L, p0};
      return f(c);
    }
  }
  return SPFA_ERR_BAD_ARG;
}

// ---- explicit masks: dense (row block, key tile) pairs on the tiled kernel, the rest on the gather kernel ----
constexpr int64_t kHybridMinNnz = 1 << 20;  // AUTO: smaller masks are launch bound either way and stay exact FP32
constexpr int kDenseDivisor = 24;           // a tile is dense from 128*BN/24 entries on (~4 % filled)

struct HybridLayout {
  int bn, n_key_tiles, min_entries;
  int64_t n_blocks;
  long long cap_words;
  size_t smem;
  long long cap_items;
  size_t off_pool, off_nt, off_kt, off_moff, off_cnt, off_heavy, off_items, off_done, off_part, off_res, off_masks, total;
};

inline bool hybrid_shape_ok(int d, int64_t n_rows, int64_t nnz, int64_t Lk) {
  if (!(d == 32 || d == 64 || d == 128) || n_rows <= 0 || nnz <= 0 || Lk <= 0) return false;
  const int bn = tile_bn(d);
  return explicit_plan_smem_bytes((Lk + bn - 1) / bn, bn) <= (size_t)kPlanMaxSmem;
}

inline HybridLayout hybrid_layout(int64_t n_rows, int64_t nnz, int64_t Lk, int d) {
  HybridLayout h;
  h.bn = tile_bn(d);
  h.n_key_tiles = (int)((Lk + h.bn - 1) / h.bn);
  h.min_entries = 128 * h.bn / kDenseDivisor;
  h.n_blocks = (n_rows + 127) / 128;
  h.smem = explicit_plan_smem_bytes(h.n_key_tiles, h.bn);
  int64_t cap_tiles = nnz / h.min_entries + 1;  // a dense tile holds at least min_entries entries
  if (cap_tiles > h.n_blocks * tile::kMaxDenseTiles) cap_tiles = h.n_blocks * tile::kMaxDenseTiles;
  h.cap_words = (long long)cap_tiles * (h.bn / 32) * 128;
  h.off_pool = 0;
  h.off_nt = 256;
  h.off_kt = h.off_nt + align_up((size_t)h.n_blocks * 4);
  h.off_moff = h.off_kt + align_up((size_t)h.n_blocks * tile::kMaxDenseTiles * 4);
  h.off_cnt = h.off_moff + align_up((size_t)h.n_blocks * 8);
  h.off_heavy = h.off_cnt + align_up((size_t)n_rows * 4);
  h.cap_items = 2 * (nnz / kSplitRowSlots) + 1;  // a split row has more than kSplitRowSlots entries and ceil(n / that) slices
  h.off_items = h.off_heavy + align_up((size_t)n_rows * 4);
  h.off_done = h.off_items + align_up((size_t)h.cap_items * sizeof(int4));
  h.off_part = h.off_done + align_up((size_t)h.cap_items * 4);
  h.off_res = h.off_part + align_up((size_t)h.cap_items * (d + 4) * 4);
  h.off_masks = h.off_res + align_up((size_t)nnz * 4);
  h.total = h.off_masks + align_up((size_t)h.cap_words * 4);
  return h;
}

// Does this call take the dense-tile split? 1 = yes, 0 = gather path, negative = status to return.
inline int hybrid_decision(int d, int64_t n_rows, int64_t nnz, int64_t Lk, const void* ws, size_t ws_bytes) {
  const int path = g_path.load();
  if (path == SPFA_PATH_GATHER || nnz <= 0) return 0;  // an empty mask has nothing to tile (NaN rows: gather kernel)
  const bool shape = hybrid_shape_ok(d, n_rows, nnz, Lk);
  if (path == SPFA_PATH_TILED && !shape) return SPFA_ERR_BAD_ARG;
  if (!shape || (path == SPFA_PATH_AUTO && nnz < kHybridMinNnz)) return 0;
  if (check_workspace(ws, ws_bytes, hybrid_layout(n_rows, nnz, Lk, d).total) != SPFA_OK)
    return path == SPFA_PATH_TILED ? (int)SPFA_ERR_WORKSPACE : 0;
  const bool usable = d == 32 ? band_kernel_usable<32, true>()
                              : (d == 64 ? band_kernel_usable<64, true>() : band_kernel_usable<128, true>());
  if (!usable) return path == SPFA_PATH_TILED ? (int)SPFA_ERR_REGISTER_BUDGET : 0;
  return 1;
}

inline ExplicitPlan plan_view(const HybridLayout& h, char* ws) {
  ExplicitPlan plan;
  plan.pool_used = reinterpret_cast<unsigned long long*>(ws + h.off_pool);
  plan.heavy_count = reinterpret_cast<unsigned int*>(ws + h.off_pool + 8);
  plan.unsorted = reinterpret_cast<unsigned int*>(ws + h.off_pool + 12);
  plan.header = reinterpret_cast<PlanHeader*>(ws + h.off_pool + kPlanHeaderOffset);
  plan.split_count = reinterpret_cast<unsigned int*>(ws + h.off_pool + 16);
  plan.split_items = reinterpret_cast<int4*>(ws + h.off_items);
  plan.split_done = reinterpret_cast<unsigned int*>(ws + h.off_done);
  plan.split_part = reinterpret_cast<float*>(ws + h.off_part);
  plan.cap_items = h.cap_items;
  plan.rb_nt = reinterpret_cast<int*>(ws + h.off_nt);
  plan.rb_kt = reinterpret_cast<int*>(ws + h.off_kt);
  plan.rb_moff = reinterpret_cast<long long*>(ws + h.off_moff);
  plan.res_cnt = reinterpret_cast<uint32_t*>(ws + h.off_cnt);
  plan.heavy_rows = reinterpret_cast<int*>(ws + h.off_heavy);
  plan.res_col = reinterpret_cast<uint32_t*>(ws + h.off_res);
  plan.masks = reinterpret_cast<uint32_t*>(ws + h.off_masks);
  plan.cap_words = h.cap_words;
  return plan;
}

// The inspector: fills the plan region `ws` for the mask (row_off, col). With use_nan it also NaN-fills the O
// rows of rows without entries (a per-call effect; plans built for later use pass use_nan = 0, O = nullptr).
template <int BN>
int launch_plan(const uint64_t* row_off, const uint32_t* col, int64_t n_rows, int64_t nnz, int64_t Lk, int d,
                const HybridLayout& h, char* ws, int use_nan, float* O, cudaStream_t st) {
  const ExplicitPlan plan = plan_view(h, ws);
  if (cudaMemsetAsync(plan.pool_used, 0, 32, st) != cudaSuccess) return SPFA_ERR_LAUNCH;  // the four counters
  if (cudaMemsetAsync(plan.split_done, 0, (size_t)h.cap_items * 4, st) != cudaSuccess) return SPFA_ERR_LAUNCH;
  auto plan_kern = explicit_plan_kernel<BN>;
  if (cudaFuncSetAttribute(plan_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)h.smem) != cudaSuccess)
    return SPFA_ERR_LAUNCH;
  plan_kern<<<(unsigned)h.n_blocks, kPlanThreads, h.smem, st>>>(row_off, col, n_rows, nnz, Lk, h.n_key_tiles,
                                                                h.min_entries, plan, use_nan, O, d);
  g_launches.fetch_add(1);
  return launch_status();
}

inline int build_plan(int d, const uint64_t* row_off, const uint32_t* col, int64_t n_rows, int64_t nnz, int64_t Lk,
                      char* ws, int use_nan, float* O, cudaStream_t st) {
  const HybridLayout h = hybrid_layout(n_rows, nnz, Lk, d);
  return (h.bn == 64) ? launch_plan<64>(row_off, col, n_rows, nnz, Lk, d, h, ws, use_nan, O, st)
                      : launch_plan<32>(row_off, col, n_rows, nnz, Lk, d, h, ws, use_nan, O, st);
}

// Rows without any mask entry get a NaN output row (what the inspector does in a one-shot call, for calls that
// run from a stored plan).
__global__ void nan_fill_empty_rows_kernel(const uint64_t* __restrict__ row_off, float* __restrict__ O, int64_t n_rows,
                                           int d) {
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= n_rows || row_off[r + 1] > row_off[r]) return;
  const float nn = __int_as_float(0x7fc00000);
  for (int i = lane * 4; i < d; i += 128) *reinterpret_cast<float4*>(O + (size_t)r * d + i) = make_float4(nn, nn, nn, nn);
}

// The two compute launches of the split, from a filled plan region: dense tiles, then everything else.
// [key_begin, key_end) restricts both to a range of keys (whole mask: 0, Lk): a forward split along the key axis
// runs once per range and the passes chain through (m, l, O). key_begin must be a multiple of the key-tile size.
template <int D>
int launch_from_plan(const float* Q, const float* K, const float* V, const uint64_t* row_off, float* m, float* l,
                     float* O, int64_t n_rows, int64_t nnz, int64_t Lk, char* ws, int64_t key_begin, int64_t key_end,
                     cudaStream_t st, int parts = 3) {  // parts: bit 0 the dense tiles, bit 1 the residual entries
  constexpr int BN = TileCfg<D>::BN, kRows = TileCfg<D>::kRows;
  const HybridLayout h = hybrid_layout(n_rows, nnz, Lk, D);
  const ExplicitPlan plan = plan_view(h, ws);
  const bool whole = (key_begin <= 0 && key_end >= Lk);
  const bool cyclic = key_begin > key_end;  // [key_begin, Lk) + [0, key_end)
  PlanHeader want;
  want.magic = kPlanMagic;
  want.n_rows = n_rows;
  want.nnz = nnz;
  want.n_keys = Lk;
  want.d = D;
  want.bn = BN;
  tile::BandParams prm{};
  prm.mode = 3;
  prm.n_keys = Lk;
  prm.u_q_first = 0;
  prm.n_q = n_rows;
  prm.s = 1;
  prm.scale_log2e = (1.0f / sqrtf((float)D)) * kLog2e;
  prm.x_nt = plan.rb_nt;
  prm.x_kt = plan.rb_kt;
  prm.x_moff = plan.rb_moff;
  prm.x_masks = plan.masks;
  prm.x_hdr = plan.header;
  prm.x_want = want;
  prm.x_kt_lo = whole ? 0 : (int)(key_begin / BN);
  prm.x_kt_hi = whole ? 0x7fffffff : (int)((key_end + BN - 1) / BN);
  CUtensorMap tmQ, tmK, tmV, tmO;
  const int64_t pitch = D * (int64_t)sizeof(float);
  if (!make_row_map(&tmQ, Q, D, n_rows, pitch, 128) || !make_row_map(&tmK, K, D, Lk, pitch, BN) ||
      !make_row_map(&tmV, V, D, Lk, pitch, BN, /*mn_major=*/true) ||
      !make_row_map(&tmO, O, D, n_rows, pitch, 128, false, 1, 0, true))
    return SPFA_ERR_LAUNCH;
  if (parts & 1) {
    int rc = launch_band_raw<D, true>(tmQ, tmK, tmV, m, l, O, prm, dim3((unsigned)((n_rows + kRows - 1) / kRows)), st,
                                      nullptr, nullptr, &tmO);
    if (rc) return rc;
    g_last_path.store(SPFA_PATH_TILED);
  }
  if (!(parts & 2)) return SPFA_OK;
  // everything else: one launch whose first CTAs take the long residual rows, the others the ordinary rows
  const float scale = 1.0f / sqrtf((float)D);
  const int per_cta = rows_per_cta_for(n_rows, 1);
  const int64_t row_blocks = (n_rows + per_cta - 1) / per_cta;
  const int list_blocks = (int)(row_blocks < 512 ? row_blocks : 512);
  if (row_blocks + list_blocks > 0x7fffffffLL) return SPFA_ERR_TOO_LARGE;
  int* err = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&err), g_tile_error) != cudaSuccess) return SPFA_ERR_LAUNCH;
  if (whole) {
    ResidualCols listed{row_off, plan.res_cnt, plan.res_col, 0xffffffffu};
    ResidualCols cols{row_off, plan.res_cnt, plan.res_col, (uint32_t)kListedRowSlots};
    gather_rows_listed_first_kernel<D, ResidualCols><<<(unsigned)(row_blocks + list_blocks), kRowWarps * 32, 0, st>>>(
        Q, K, V, m, l, O, cols, listed, plan.heavy_rows, plan.heavy_count, list_blocks, 0, n_rows, 0, scale, plan.header,
        want, err, plan.split_items, plan.split_count, plan.cap_items, plan.split_done, plan.split_part, per_cta);
  } else {
    const uint32_t klo = (uint32_t)key_begin, khi = (uint32_t)(key_end < Lk ? key_end : Lk);
    (void)cyclic;  // klo > khi is the cyclic range for the functor and for the tile filter alike
    ResidualRangeCols listed{row_off, plan.res_cnt, plan.res_col, 0xffffffffu, klo, khi, plan.unsorted};
    ResidualRangeCols cols{row_off, plan.res_cnt, plan.res_col, (uint32_t)kListedRowSlots, klo, khi, plan.unsorted};
    gather_rows_listed_first_kernel<D, ResidualRangeCols>
        <<<(unsigned)(row_blocks + list_blocks), kRowWarps * 32, 0, st>>>(Q, K, V, m, l, O, cols, listed, plan.heavy_rows,
                                                                        plan.heavy_count, list_blocks, 0, n_rows, 0, scale,
                                                                        plan.header, want, err, plan.split_items,
                                                                        plan.split_count, plan.cap_items, plan.split_done,
                                                                        plan.split_part, per_cta);
  }
  g_launches.fetch_add(1);
  g_last_path.store(SPFA_PATH_TILED);
  return launch_status();
}

inline int forward_from_plan(int d, const float* Q, const float* K, const float* V, const uint64_t* row_off, float* m,
                             float* l, float* O, int64_t n_rows, int64_t nnz, int64_t Lk, char* ws, cudaStream_t st,
                             int64_t key_begin = 0, int64_t key_end = INT64_MAX, int parts = 3) {
  switch (d) {
    case 32: return launch_from_plan<32>(Q, K, V, row_off, m, l, O, n_rows, nnz, Lk, ws, key_begin, key_end, st, parts);
    case 64: return launch_from_plan<64>(Q, K, V, row_off, m, l, O, n_rows, nnz, Lk, ws, key_begin, key_end, st, parts);
    case 128: return launch_from_plan<128>(Q, K, V, row_off, m, l, O, n_rows, nnz, Lk, ws, key_begin, key_end, st, parts);
  }
  return SPFA_ERR_EMBED_DIM;
}

// One-shot call: inspector, then the two compute launches.
inline int hybrid_forward(int d, const float* Q, const float* K, const float* V, const uint64_t* row_off,
                          const uint32_t* col, float* m, float* l, float* O, int64_t n_rows, int64_t nnz, int64_t Lk,
                          int use_nan, char* ws, cudaStream_t st) {
  const int rc = build_plan(d, row_off, col, n_rows, nnz, Lk, ws, use_nan, O, st);
  if (rc) return rc;
  return forward_from_plan(d, Q, K, V, row_off, m, l, O, n_rows, nnz, Lk, ws, st);
}

// ---- scratch for the allocation-free COO entry point ---------------------------------------------------
// Row pointers for up to kStaticCooMaxRows query rows, resident in every GPU context that loads this
// library (2 MiB + 8 B) until the process exits. In host code the array's name is only a handle: the
// device address is obtained once per device with cudaGetSymbolAddress and cached here.
constexpr int64_t kStaticCooMaxRows = 1 << 18;
static __device__ __align__(256) unsigned long long g_static_coo_row_ptr[kStaticCooMaxRows + 1];
constexpr int kMaxDevices = 64;
static std::atomic<unsigned long long*> g_static_coo_ptr[kMaxDevices];

inline int static_coo_scratch(unsigned long long** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SPFA_ERR_LAUNCH;
  unsigned long long* p = g_static_coo_ptr[dev].load(std::memory_order_acquire);
  if (!p) {  // first call on this device: resolve the symbol in the current device's context
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_static_coo_row_ptr) != cudaSuccess || !addr) return SPFA_ERR_LAUNCH;
    p = static_cast<unsigned long long*>(addr);
    g_static_coo_ptr[dev].store(p, std::memory_order_release);  // racing first calls resolve the same address
  }
  *out = p;
  return SPFA_OK;
}

template <class IdxT>
int launch_row_pointers(const IdxT* row_ind, int64_t nnz, int64_t row_begin, int64_t n_rows, uint64_t* ptr,
                        cudaStream_t st) {
  constexpr int64_t span = (int64_t)kRowPtrThreads * kRowPtrUnroll;
  int64_t blocks = (nnz + 1 + span - 1) / span;
  if (blocks > 148 * 32) blocks = 148 * 32;
  coo_row_pointers_kernel<IdxT><<<(unsigned)blocks, kRowPtrThreads, 0, st>>>(row_ind, nnz, row_begin, n_rows, ptr);
  g_launches.fetch_add(1);
  return launch_status();
}

}  // namespace spfa

using namespace spfa;

namespace spfa {

template <class IdxT>
int coo_forward_impl(const float* Q, const float* K, const float* V, const IdxT* row_ind, const uint32_t* col_ind,
                     int64_t nnz, float* m, float* l, float* O, int64_t row_begin, int64_t n_rows, int64_t Lk, int d,
                     int use_nan, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  if (nnz < 0 || n_rows < 0 || row_begin < 0 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (nnz > 0 && (!row_ind || !col_ind)) return SPFA_ERR_BAD_ARG;
  if (n_rows == 0) return SPFA_OK;
  const size_t ptr_bytes = spfa_coo_min_workspace_bytes(n_rows);
  rc = check_workspace(workspace, workspace_bytes, ptr_bytes);
  if (rc) return rc;
  char* rest = static_cast<char*>(workspace) + ptr_bytes;
  const int hy = hybrid_decision(d, n_rows, nnz, Lk, rest, workspace_bytes - ptr_bytes);
  if (hy < 0) return hy;
  cudaStream_t st = (cudaStream_t)stream;
  uint64_t* ptr = reinterpret_cast<uint64_t*>(workspace);
  if (launch_row_pointers<IdxT>(row_ind, nnz, row_begin, n_rows, ptr, st) != SPFA_OK) return SPFA_ERR_LAUNCH;
  if (hy == 1) return hybrid_forward(d, Q, K, V, ptr, col_ind, m, l, O, n_rows, nnz, Lk, use_nan, rest, st);
  CsrCols cols{ptr, col_ind, Lk};
  return dispatch_gather(d, Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st);
}

template <class IdxT>
int coo_plan_build_impl(const IdxT* row_ind, const uint32_t* col_ind, int64_t nnz, int64_t row_begin, int64_t n_rows,
                        int64_t Lk, int d, void* plan, size_t plan_bytes, void* stream) {
  if (!row_ind || !col_ind || n_rows <= 0 || nnz <= 0 || row_begin < 0 || Lk <= 0 || Lk >= (1LL << 31))
    return SPFA_ERR_BAD_ARG;
  const size_t need = spfa_explicit_plan_bytes(n_rows, nnz, Lk, d);
  if (need == 0) return supported_d(d) ? (int)SPFA_ERR_BAD_ARG : (int)SPFA_ERR_EMBED_DIM;
  int rc = check_workspace(plan, plan_bytes, need);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  uint64_t* offs = reinterpret_cast<uint64_t*>(plan);
  if (launch_row_pointers<IdxT>(row_ind, nnz, row_begin, n_rows, offs, st) != SPFA_OK) return SPFA_ERR_LAUNCH;
  return build_plan(d, offs, col_ind, n_rows, nnz, Lk, static_cast<char*>(plan) + spfa_coo_min_workspace_bytes(n_rows), 0,
                    nullptr, st);
}

}  // namespace spfa

extern "C" {

const char* spfa_status_string(int s) {
  switch (s) {
    case SPFA_OK: return "ok";
    case SPFA_ERR_BAD_ARG: return "bad argument (null or misaligned pointer, negative size, or row range outside [0, L])";
    case SPFA_ERR_EMBED_DIM: return "The embedded dimension is too large for the amount of shared memory on your GPU.";
    case SPFA_ERR_WORKSPACE: return "workspace missing, not 256-byte aligned, or too small";
    case SPFA_ERR_LAUNCH: return "CUDA reported an error while enqueueing a kernel";
    case SPFA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case SPFA_ERR_LOCAL_SIZE: return "The local size specified is either negative or greater than/equal to (1 - Sequence Length).";
    case SPFA_ERR_DILATION_NEG: return "The dilation factor must be atleast 0.";
    case SPFA_ERR_BLOCK_DIVISOR: return "The block/window size must be a divisor of the whole tensor's size.";
    case SPFA_ERR_DILATION_BLOCK: return "The dilation factor must be less than the block/window size.";
    case SPFA_ERR_GLOBAL_COUNT: return "There are either no global tokens provided or there are more than the sequence length given.";
    case SPFA_ERR_TOO_LARGE: return "size beyond a fixed maximum";
    case SPFA_ERR_REGISTER_BUDGET: return "the tiled kernel of this build cannot run (register allocation below its setmaxnreg budgets)";
  }
  return "unknown status";
}

int spfa_abi_version(void) { return 1100; }

void spfa_set_path(int path) {
  if (path == SPFA_PATH_AUTO || path == SPFA_PATH_GATHER || path == SPFA_PATH_TILED) g_path.store(path);
}
int spfa_get_path(void) { return g_path.load(); }
int spfa_last_path(void) { return g_last_path.load(); }

int64_t spfa_launch_count(void) { return g_launches.load(); }

int spfa_last_device_error(void) { return read_and_clear_tile_error(); }

int spfa_selftest_wait_limit(void* stream) { return launch_wait_limit_selftest(9001, (cudaStream_t)stream); }

// ---- CSR -----------------------------------------------------------------------------------------
size_t spfa_csr_workspace_bytes(int64_t n_rows, int64_t nnz, int64_t Lk, int d) {
  const int path = g_path.load();
  if (path == SPFA_PATH_GATHER || !hybrid_shape_ok(d, n_rows, nnz, Lk)) return 0;
  if (path == SPFA_PATH_AUTO && nnz < kHybridMinNnz) return 0;
  return hybrid_layout(n_rows, nnz, Lk, d).total;
}

int spfa_csr_forward_f32(const float* Q, const float* K, const float* V, const uint64_t* row_off,
                         const uint32_t* col_ind, int64_t nnz, float* m, float* l, float* O, int64_t n_rows,
                         int64_t Lk, int d, int use_nan, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  if (!row_off || n_rows < 0 || nnz < 0 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (n_rows == 0) return SPFA_OK;
  if (!col_ind) return SPFA_ERR_BAD_ARG;
  const int hy = hybrid_decision(d, n_rows, nnz, Lk, workspace, workspace_bytes);
  if (hy < 0) return hy;
  if (hy == 1)
    return hybrid_forward(d, Q, K, V, row_off, col_ind, m, l, O, n_rows, nnz, Lk, use_nan,
                          static_cast<char*>(workspace), (cudaStream_t)stream);
  CsrCols cols{row_off, col_ind, Lk};
  return dispatch_gather(d, Q, K, V, m, l, O, cols, 0, n_rows, use_nan, (cudaStream_t)stream);
}

// ---- COO -----------------------------------------------------------------------------------------
size_t spfa_coo_min_workspace_bytes(int64_t n_rows) {
  return n_rows < 0 ? 0 : align_up((size_t)(n_rows + 1) * sizeof(uint64_t));
}

size_t spfa_coo_workspace_bytes(int64_t n_rows, int64_t nnz, int64_t Lk, int d) {
  return spfa_coo_min_workspace_bytes(n_rows) + spfa_csr_workspace_bytes(n_rows, nnz, Lk, d);
}

int spfa_coo_forward_f32(const float* Q, const float* K, const float* V, const uint64_t* row_ind,
                         const uint32_t* col_ind, int64_t nnz, float* m, float* l, float* O, int64_t row_begin,
                         int64_t n_rows, int64_t Lk, int d, int use_nan, void* workspace, size_t workspace_bytes,
                         void* stream) {
  return coo_forward_impl<uint64_t>(Q, K, V, row_ind, col_ind, nnz, m, l, O, row_begin, n_rows, Lk, d, use_nan, workspace,
                                    workspace_bytes, stream);
}

// ---- 32-bit row offsets / row indices (additive; the reference's tensors are 64-bit) ------------------------
int spfa_coo_forward_f32_idx32(const float* Q, const float* K, const float* V, const int32_t* row_ind,
                               const uint32_t* col_ind, int64_t nnz, float* m, float* l, float* O, int64_t row_begin,
                               int64_t n_rows, int64_t Lk, int d, int use_nan, void* workspace, size_t workspace_bytes,
                               void* stream) {
  return coo_forward_impl<int32_t>(Q, K, V, row_ind, col_ind, nnz, m, l, O, row_begin, n_rows, Lk, d, use_nan, workspace,
                                   workspace_bytes, stream);
}

size_t spfa_csr_workspace_bytes_idx32(int64_t n_rows, int64_t nnz, int64_t Lk, int d) {
  return spfa_coo_min_workspace_bytes(n_rows) + spfa_csr_workspace_bytes(n_rows, nnz, Lk, d);
}

int spfa_csr_forward_f32_idx32(const float* Q, const float* K, const float* V, const int32_t* row_off,
                               const uint32_t* col_ind, int64_t nnz, float* m, float* l, float* O, int64_t n_rows,
                               int64_t Lk, int d, int use_nan, void* workspace, size_t workspace_bytes, void* stream) {
  if (!row_off || n_rows < 0) return SPFA_ERR_BAD_ARG;
  if (n_rows == 0) return SPFA_OK;
  const size_t off_bytes = spfa_coo_min_workspace_bytes(n_rows);
  int rc = check_workspace(workspace, workspace_bytes, off_bytes);
  if (rc) return rc;
  uint64_t* wide = reinterpret_cast<uint64_t*>(workspace);
  widen_offsets_kernel<<<(unsigned)((n_rows + 1 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(row_off, n_rows + 1, wide);
  g_launches.fetch_add(1);
  if (launch_status() != SPFA_OK) return SPFA_ERR_LAUNCH;
  return spfa_csr_forward_f32(Q, K, V, wide, col_ind, nnz, m, l, O, n_rows, Lk, d, use_nan,
                              static_cast<char*>(workspace) + off_bytes, workspace_bytes - off_bytes, stream);
}

// ---- stored plans for explicit masks ---------------------------------------------------------------------
// Plan region = [row offsets: n_rows + 1 x u64][the inspector's output, laid out as in a one-shot call].
size_t spfa_explicit_plan_bytes(int64_t n_rows, int64_t nnz, int64_t Lk, int d) {
  if (!hybrid_shape_ok(d, n_rows, nnz, Lk)) return 0;
  return spfa_coo_min_workspace_bytes(n_rows) + hybrid_layout(n_rows, nnz, Lk, d).total;
}

int spfa_csr_plan_build(const uint64_t* row_off, const uint32_t* col_ind, int64_t nnz, int64_t n_rows, int64_t Lk, int d,
                        void* plan, size_t plan_bytes, void* stream) {
  if (!row_off || !col_ind || n_rows <= 0 || nnz <= 0 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  const size_t need = spfa_explicit_plan_bytes(n_rows, nnz, Lk, d);
  if (need == 0) return supported_d(d) ? (int)SPFA_ERR_BAD_ARG : (int)SPFA_ERR_EMBED_DIM;
  int rc = check_workspace(plan, plan_bytes, need);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  uint64_t* offs = reinterpret_cast<uint64_t*>(plan);
  if (cudaMemcpyAsync(offs, row_off, (size_t)(n_rows + 1) * sizeof(uint64_t), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
    return SPFA_ERR_LAUNCH;
  return build_plan(d, offs, col_ind, n_rows, nnz, Lk, static_cast<char*>(plan) + spfa_coo_min_workspace_bytes(n_rows), 0,
                    nullptr, st);
}

int spfa_coo_plan_build(const uint64_t* row_ind, const uint32_t* col_ind, int64_t nnz, int64_t row_begin, int64_t n_rows,
                        int64_t Lk, int d, void* plan, size_t plan_bytes, void* stream) {
  return coo_plan_build_impl<uint64_t>(row_ind, col_ind, nnz, row_begin, n_rows, Lk, d, plan, plan_bytes, stream);
}

int spfa_coo_plan_build_idx32(const int32_t* row_ind, const uint32_t* col_ind, int64_t nnz, int64_t row_begin,
                              int64_t n_rows, int64_t Lk, int d, void* plan, size_t plan_bytes, void* stream) {
  return coo_plan_build_impl<int32_t>(row_ind, col_ind, nnz, row_begin, n_rows, Lk, d, plan, plan_bytes, stream);
}

int spfa_planned_forward_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                             int64_t n_rows, int64_t nnz, int64_t Lk, int d, int use_nan, const void* plan,
                             size_t plan_bytes, void* stream) {
  return spfa_planned_forward_keys_f32(Q, K, V, m, l, O, n_rows, nnz, Lk, d, use_nan, plan, plan_bytes, 0, Lk, stream);
}

int spfa_planned_forward_keys_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                  int64_t n_rows, int64_t nnz, int64_t Lk, int d, int use_nan, const void* plan,
                                  size_t plan_bytes, int64_t key_begin, int64_t key_end, void* stream) {
  return spfa_planned_forward_parts_f32(Q, K, V, m, l, O, n_rows, nnz, Lk, d, use_nan, plan, plan_bytes, key_begin, key_end,
                                        SPFA_PLAN_DENSE_TILES | SPFA_PLAN_RESIDUAL, stream);
}

int spfa_planned_forward_parts_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                   int64_t n_rows, int64_t nnz, int64_t Lk, int d, int use_nan, const void* plan,
                                   size_t plan_bytes, int64_t key_begin, int64_t key_end, int parts, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  if (parts < 0 || parts > 3) return SPFA_ERR_BAD_ARG;
  if (n_rows <= 0 || nnz <= 0 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (key_begin < 0 || key_end < 0 || key_begin > Lk || (key_begin % 64) != 0) return SPFA_ERR_BAD_ARG;
  if (key_end > Lk) key_end = Lk;
  if (key_end < Lk && (key_end % 64) != 0) return SPFA_ERR_BAD_ARG;  // a dense key tile belongs to exactly one pass
  const size_t need = spfa_explicit_plan_bytes(n_rows, nnz, Lk, d);
  if (need == 0) return SPFA_ERR_BAD_ARG;
  rc = check_workspace(plan, plan_bytes, need);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  char* base = static_cast<char*>(const_cast<void*>(plan));
  const uint64_t* offs = reinterpret_cast<const uint64_t*>(base);
  if (use_nan) {
    nan_fill_empty_rows_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, st>>>(offs, O, n_rows, d);
    g_launches.fetch_add(1);
    if (launch_status() != SPFA_OK) return SPFA_ERR_LAUNCH;
  }
  if (key_end == key_begin || parts == 0) return SPFA_OK;
  return forward_from_plan(d, Q, K, V, offs, m, l, O, n_rows, nnz, Lk, base + spfa_coo_min_workspace_bytes(n_rows), st,
                           key_begin, key_end, parts);
}

int64_t spfa_coo_static_max_rows(void) { return kStaticCooMaxRows; }

// COO forward for callers that may not allocate: same arithmetic and kernels as spfa_coo_forward_f32, with
// the row-pointer scratch taken from the library's own static device array instead of a caller workspace.
int spfa_coo_forward_f32_static(const float* Q, const float* K, const float* V, const uint64_t* row_ind,
                                const uint32_t* col_ind, int64_t nnz, float* m, float* l, float* O,
                                int64_t row_begin, int64_t n_rows, int64_t Lk, int d, int use_nan, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  if (nnz < 0 || n_rows < 0 || row_begin < 0 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (nnz > 0 && (!row_ind || !col_ind)) return SPFA_ERR_BAD_ARG;
  if (n_rows > kStaticCooMaxRows) return SPFA_ERR_TOO_LARGE;  // more rows than the static scratch holds
  if (n_rows == 0) return SPFA_OK;
  unsigned long long* scratch = nullptr;
  rc = static_coo_scratch(&scratch);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  uint64_t* ptr = reinterpret_cast<uint64_t*>(scratch);
  // every entry ptr[0 .. n_rows] is written by this pass, so nothing left by an earlier call is read
  if (launch_row_pointers<uint64_t>(row_ind, nnz, row_begin, n_rows, ptr, st) != SPFA_OK) return SPFA_ERR_LAUNCH;
  CsrCols cols{ptr, col_ind, Lk};
  return dispatch_gather(d, Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st);
}

// ---- Local ---------------------------------------------------------------------------------------
size_t spfa_local_workspace_bytes(int64_t, int64_t, int) { return 0; }

int spfa_local_forward_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O, int64_t L,
                           int d, int64_t w, int64_t row_begin, int64_t row_end, void* ws, size_t ws_bytes, void* stream) {
  return spfa_local_forward_batched_f32(Q, K, V, m, l, O, 1, L, d, w, row_begin, row_end, ws, ws_bytes, stream);
}

int spfa_local_forward_batched_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                   int64_t n_slices, int64_t L, int d, int64_t w, int64_t row_begin, int64_t row_end, void*,
                                   size_t, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (n_slices < 1) return SPFA_ERR_BAD_ARG;
  if (w < 0 || w > L - 1) return SPFA_ERR_LOCAL_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  const int path = g_path.load();
  if (path != SPFA_PATH_GATHER) {
    rc = tiled_band_forward(Q, K, V, m, l, O, L, d, w, /*stride=*/1, row_begin, row_end, path == SPFA_PATH_TILED, st, n_slices);
    if (rc != SPFA_TILE_NOT_TAKEN) {
      if (rc == SPFA_OK) g_last_path.store(SPFA_PATH_TILED);
      return rc;
    }
  }
  LocalCols cols{L, w};
  return dispatch_gather(d, Q, K, V, m, l, O, cols, row_begin, row_end - row_begin, 0, st, n_slices, L * d);
}

// ---- Local 1D dilated ------------------------------------------------------------------------------
size_t spfa_local_1d_dilated_workspace_bytes(int64_t, int64_t, int) { return 0; }

int spfa_local_1d_dilated_forward_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                      int64_t L, int d, int64_t w, int64_t dil, int64_t row_begin, int64_t row_end,
                                      void* ws, size_t ws_bytes, void* stream) {
  return spfa_local_1d_dilated_forward_batched_f32(Q, K, V, m, l, O, 1, L, d, w, dil, row_begin, row_end, ws, ws_bytes, stream);
}

int spfa_local_1d_dilated_forward_batched_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                              int64_t n_slices, int64_t L, int d, int64_t w, int64_t dil, int64_t row_begin,
                                              int64_t row_end, void*, size_t, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (n_slices < 1) return SPFA_ERR_BAD_ARG;
  if (w < 0 || w > L - 1) return SPFA_ERR_LOCAL_SIZE;
  if (dil < 0) return SPFA_ERR_DILATION_NEG;
  if (dil >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int path = g_path.load();
  if (path != SPFA_PATH_GATHER) {
    rc = tiled_band_forward(Q, K, V, m, l, O, L, d, w, dil + 1, row_begin, row_end, path == SPFA_PATH_TILED, st, n_slices);
    if (rc != SPFA_TILE_NOT_TAKEN) {
      if (rc == SPFA_OK) g_last_path.store(SPFA_PATH_TILED);
      return rc;
    }
  }
  Local1dCols cols{L, w, dil + 1};
  return dispatch_gather(d, Q, K, V, m, l, O, cols, row_begin, row_end - row_begin, 0, st, n_slices, L * d);
}

// ---- Local 2D dilated ------------------------------------------------------------------------------
size_t spfa_local_2d_dilated_workspace_bytes(int64_t, int64_t, int) { return 0; }

int spfa_local_2d_dilated_forward_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                      int64_t L, int d, int64_t B, int64_t dil, int use_nan, int64_t row_begin,
                                      int64_t row_end, void*, size_t, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (B <= 0 || L % B != 0) return SPFA_ERR_BLOCK_DIVISOR;
  if (dil < 0) return SPFA_ERR_DILATION_NEG;
  if (dil >= (1LL << 31) || B / (dil + 1) < 1) return SPFA_ERR_DILATION_BLOCK;
  if (row_end == row_begin) return SPFA_OK;
  {
    // block-staged kernel whenever a block's key rows fit in shared memory; else (and when the gather
    // path is forced) one warp per row
    const int64_t s1 = dil + 1;
    const int64_t n = ((B - 1) / s1 + 1 < B) ? ((B - 1) / s1 + 1) : B;
    if (g_path.load() != SPFA_PATH_GATHER && n > kTile2dMinKeys && n <= kTile2dMaxKeys && specialised_d(d)) {
      cudaStream_t st = (cudaStream_t)stream;
      switch (d) {
        case 16: return launch_local2d_tile<16>(Q, K, V, m, l, O, L, B, s1, n, use_nan, row_begin, row_end, st);
        case 32: return launch_local2d_tile<32>(Q, K, V, m, l, O, L, B, s1, n, use_nan, row_begin, row_end, st);
        case 64: return launch_local2d_tile<64>(Q, K, V, m, l, O, L, B, s1, n, use_nan, row_begin, row_end, st);
        case 128: return launch_local2d_tile<128>(Q, K, V, m, l, O, L, B, s1, n, use_nan, row_begin, row_end, st);
      }
    }
    if (g_path.load() != SPFA_PATH_GATHER && n <= 32 * kBlockMaxKeysPerLane) {
      cudaStream_t st = (cudaStream_t)stream;
      switch (d) {
        case 16: if (block2d_smem_bytes<16>(n) <= 200 * 1024) return launch_local2d_block<16>(Q, K, V, m, l, O, L, B, s1, n, use_nan, row_begin, row_end, st); break;
        case 32: if (block2d_smem_bytes<32>(n) <= 200 * 1024) return launch_local2d_block<32>(Q, K, V, m, l, O, L, B, s1, n, use_nan, row_begin, row_end, st); break;
        case 64: if (block2d_smem_bytes<64>(n) <= 200 * 1024) return launch_local2d_block<64>(Q, K, V, m, l, O, L, B, s1, n, use_nan, row_begin, row_end, st); break;
        case 128: if (block2d_smem_bytes<128>(n) <= 200 * 1024) return launch_local2d_block<128>(Q, K, V, m, l, O, L, B, s1, n, use_nan, row_begin, row_end, st); break;
      }
    }
  }
  Local2dCols cols{L, B, dil + 1};
  return dispatch_gather(d, Q, K, V, m, l, O, cols, row_begin, row_end - row_begin, use_nan, (cudaStream_t)stream);
}

// ---- Global-no-local -------------------------------------------------------------------------------
size_t spfa_global_no_local_workspace_bytes(int64_t L, int64_t, int d, int64_t n_global) {
  if (L <= 0 || n_global <= 0 || !supported_d(d)) return 0;
  size_t total = gnl_plan(L, d, n_global).total;  // gather path
  if (gnl_tiled_shape_ok(d, n_global)) total += gnl_tiled_plan(L, d, n_global).total;  // + tiled path scratch
  return total;
}

int spfa_global_no_local_forward_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                     const int32_t* G, int64_t nG, int64_t L, int d, int64_t w, int64_t row_begin,
                                     int64_t row_end, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (nG == 0 || nG > L || nG < 0) return SPFA_ERR_GLOBAL_COUNT;
  if (w < 0 || w > L - 1) return SPFA_ERR_LOCAL_SIZE;
  if (!G) return SPFA_ERR_BAD_ARG;
  if (nG > (1LL << 30)) return SPFA_ERR_TOO_LARGE;
  const GnlPlan plan = gnl_plan(L, d, nG);
  rc = check_workspace(workspace, workspace_bytes, spfa_global_no_local_workspace_bytes(L, row_end - row_begin, d, nG));
  if (rc) return rc;
  if (row_end == row_begin) return SPFA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = reinterpret_cast<char*>(workspace);
  const int path = g_path.load();
  if (path != SPFA_PATH_GATHER) {
    if (gnl_tiled_shape_ok(d, nG)) {
      const bool rows_tiled = (path == SPFA_PATH_TILED) || nG >= kGnlTiledMinGlobalsForRows;
      if (!rows_tiled) {  // few listed keys: ordinary rows on the exact gather kernel, global rows on the tiles
        uint32_t* bits0 = reinterpret_cast<uint32_t*>(ws + plan.off_bits);
        uint8_t* live0 = reinterpret_cast<uint8_t*>(ws + plan.off_live);
        if (cudaMemsetAsync(bits0, 0, (size_t)((L + 31) / 32) * 4, st) != cudaSuccess) return SPFA_ERR_LAUNCH;
        gnl_mark_globals_kernel<<<(unsigned)((nG + 255) / 256), 256, 0, st>>>(G, nG, L, bits0, live0);
        g_launches.fetch_add(1);
        if (launch_status() != SPFA_OK) return SPFA_ERR_LAUNCH;
        GnlCols cols0{G, nG, L, w, bits0};
        rc = dispatch_gather(d, Q, K, V, m, l, O, cols0, row_begin, row_end - row_begin, 0, st);
        if (rc) return rc;
      }
      rc = tiled_gnl_forward(Q, K, V, m, l, O, G, nG, L, d, w, row_begin, row_end, ws + plan.total, rows_tiled, st);
      if (rc == SPFA_OK) g_last_path.store(SPFA_PATH_TILED);
      return rc;
    }
    if (path == SPFA_PATH_TILED) return SPFA_ERR_BAD_ARG;
  }
  uint32_t* bits = reinterpret_cast<uint32_t*>(ws + plan.off_bits);
  uint8_t* live = reinterpret_cast<uint8_t*>(ws + plan.off_live);
  float* partials = reinterpret_cast<float*>(ws + plan.off_part);
  if (cudaMemsetAsync(bits, 0, (size_t)((L + 31) / 32) * 4, st) != cudaSuccess) return SPFA_ERR_LAUNCH;
  gnl_mark_globals_kernel<<<(unsigned)((nG + 255) / 256), 256, 0, st>>>(G, nG, L, bits, live);
  g_launches.fetch_add(1);
  if (launch_status() != SPFA_OK) return SPFA_ERR_LAUNCH;
  if (!specialised_d(d)) {  // one launch: a listed row is a long row walked by its whole CTA
    GnlAnyRowCols any;
    any.list = GnlCols{G, nG, L, w, bits};
    any.strip = GnlGlobalRowCols{L, w};
    return dispatch_gather_generic(d, Q, K, V, m, l, O, any, row_begin, row_end - row_begin, 0, st);
  }
  // rows outside the list: listed keys outside the window
  GnlCols cols{G, nG, L, w, bits};
  rc = dispatch_gather(d, Q, K, V, m, l, O, cols, row_begin, row_end - row_begin, 0, st);
  if (rc) return rc;
  // rows in the list: all keys outside the window, key range split across warps
  switch (d) {
    case 16: return launch_gnl_global_rows<16>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, plan, live, partials, st);
    case 32: return launch_gnl_global_rows<32>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, plan, live, partials, st);
    case 64: return launch_gnl_global_rows<64>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, plan, live, partials, st);
    case 128: return launch_gnl_global_rows<128>(Q, K, V, m, l, O, G, nG, L, w, row_begin, row_end, plan, live, partials, st);
  }
  return SPFA_ERR_EMBED_DIM;
}

// ---- batches of slices (batch x heads sharing one mask) for the operators without a slice dimension in their kernels:
//      one call per slice on the stream; scratch is reused in stream order ------------------------------------------
int spfa_local_2d_dilated_forward_batched_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                              int64_t n_slices, int64_t L, int d, int64_t B, int64_t dil, int use_nan,
                                              int64_t row_begin, int64_t row_end, void* ws, size_t ws_bytes, void* stream) {
  if (n_slices < 1 || row_end < row_begin) return SPFA_ERR_BAD_ARG;
  const int64_t n = row_end - row_begin;
  for (int64_t z = 0; z < n_slices; ++z) {
    const int rc = spfa_local_2d_dilated_forward_f32(Q + z * n * d, K + z * L * d, V + z * L * d, m + z * n, l + z * n,
                                                     O + z * n * d, L, d, B, dil, use_nan, row_begin, row_end, ws, ws_bytes,
                                                     stream);
    if (rc) return rc;
  }
  return SPFA_OK;
}

int spfa_global_no_local_forward_batched_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                             int64_t n_slices, const int32_t* G, int64_t nG, int64_t L, int d, int64_t w,
                                             int64_t row_begin, int64_t row_end, void* ws, size_t ws_bytes, void* stream) {
  if (n_slices < 1 || row_end < row_begin) return SPFA_ERR_BAD_ARG;
  const int64_t n = row_end - row_begin;
  for (int64_t z = 0; z < n_slices; ++z) {
    const int rc = spfa_global_no_local_forward_f32(Q + z * n * d, K + z * L * d, V + z * L * d, m + z * n, l + z * n,
                                                    O + z * n * d, G, nG, L, d, w, row_begin, row_end, ws, ws_bytes, stream);
    if (rc) return rc;
  }
  return SPFA_OK;
}

// Explicit masks: the mask is inspected ONCE (row pointers, dense-tile plan), every slice runs from the result.
static int explicit_batched(const float* Q, const float* K, const float* V, const uint64_t* row_off, const uint32_t* col_ind,
                            int64_t nnz, float* m, float* l, float* O, int64_t n_slices, int64_t row_begin, int64_t n_rows,
                            int64_t Lk, int d, int use_nan, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const int hy = hybrid_decision(d, n_rows, nnz, Lk, workspace, workspace_bytes);
  if (hy < 0) return hy;
  if (hy == 1) {
    char* ws = static_cast<char*>(workspace);
    int rc = build_plan(d, row_off, col_ind, n_rows, nnz, Lk, ws, 0, nullptr, st);
    for (int64_t z = 0; z < n_slices && rc == SPFA_OK; ++z) {
      float* Oz = O + z * n_rows * d;
      if (use_nan) {
        nan_fill_empty_rows_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, st>>>(row_off, Oz, n_rows, d);
        g_launches.fetch_add(1);
      }
      rc = forward_from_plan(d, Q + z * n_rows * d, K + z * Lk * d, V + z * Lk * d, row_off, m + z * n_rows, l + z * n_rows, Oz,
                             n_rows, nnz, Lk, ws, st);
    }
    return rc;
  }
  CsrCols cols{row_off, col_ind, Lk};
  return dispatch_gather(d, Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st, n_slices, Lk * d);
}

int spfa_csr_forward_batched_f32(const float* Q, const float* K, const float* V, const uint64_t* row_off,
                                 const uint32_t* col_ind, int64_t nnz, float* m, float* l, float* O, int64_t n_slices,
                                 int64_t n_rows, int64_t Lk, int d, int use_nan, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  if (!row_off || n_rows < 0 || nnz < 0 || n_slices < 1 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (n_rows == 0) return SPFA_OK;
  if (!col_ind) return SPFA_ERR_BAD_ARG;
  return explicit_batched(Q, K, V, row_off, col_ind, nnz, m, l, O, n_slices, 0, n_rows, Lk, d, use_nan, workspace,
                          workspace_bytes, (cudaStream_t)stream);
}

int spfa_coo_forward_batched_f32(const float* Q, const float* K, const float* V, const uint64_t* row_ind,
                                 const uint32_t* col_ind, int64_t nnz, float* m, float* l, float* O, int64_t n_slices,
                                 int64_t row_begin, int64_t n_rows, int64_t Lk, int d, int use_nan, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  if (nnz < 0 || n_rows < 0 || row_begin < 0 || n_slices < 1 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (nnz > 0 && (!row_ind || !col_ind)) return SPFA_ERR_BAD_ARG;
  if (n_rows == 0) return SPFA_OK;
  const size_t ptr_bytes = spfa_coo_min_workspace_bytes(n_rows);
  rc = check_workspace(workspace, workspace_bytes, ptr_bytes);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  uint64_t* ptr = reinterpret_cast<uint64_t*>(workspace);
  if (launch_row_pointers<uint64_t>(row_ind, nnz, row_begin, n_rows, ptr, st) != SPFA_OK) return SPFA_ERR_LAUNCH;
  return explicit_batched(Q, K, V, ptr, col_ind, nnz, m, l, O, n_slices, row_begin, n_rows, Lk, d, use_nan,
                          static_cast<char*>(workspace) + ptr_bytes, workspace_bytes - ptr_bytes, st);
}

// ---- fused union of masks: Local + Global-no-local + an explicit CSR part -----------------------------------
size_t spfa_bigbird_workspace_bytes(int64_t L, int64_t n_rows, int d, int64_t n_global, int64_t nnz) {
  return align_up(spfa_global_no_local_workspace_bytes(L, n_rows, d, n_global)) + spfa_csr_workspace_bytes(n_rows, nnz, L, d);
}

int spfa_bigbird_forward_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                             const int32_t* G, int64_t nG, const uint64_t* row_off, const uint32_t* col_ind, int64_t nnz,
                             int64_t L, int d, int64_t w, int64_t row_begin, int64_t row_end, void* workspace,
                             size_t workspace_bytes, void* stream) {
  int rc = check_common(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (nG == 0 || nG > L || nG < 0) return SPFA_ERR_GLOBAL_COUNT;
  if (w < 0 || w > L - 1) return SPFA_ERR_LOCAL_SIZE;
  if (!G || nnz < 0 || (nnz > 0 && (!row_off || !col_ind))) return SPFA_ERR_BAD_ARG;
  const int64_t n_rows = row_end - row_begin;
  const size_t gnl_bytes = align_up(spfa_global_no_local_workspace_bytes(L, n_rows, d, nG));
  rc = check_workspace(workspace, workspace_bytes, gnl_bytes + spfa_csr_workspace_bytes(n_rows, nnz, L, d));
  if (rc) return rc;
  if (n_rows == 0) return SPFA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = static_cast<char*>(workspace);
  const int path = g_path.load();
  // one pass over Q and O for the band and the listed keys together, where the tiled kernel serves the shape
  const bool fused = path != SPFA_PATH_GATHER && gnl_tiled_shape_ok(d, nG) && (path == SPFA_PATH_TILED || w >= kTileMinHalfWidth);
  if (fused) {
    rc = tiled_bigbird_forward(Q, K, V, m, l, O, G, nG, L, d, w, row_begin, row_end, ws + gnl_plan(L, d, nG).total, st);
    if (rc == SPFA_OK) g_last_path.store(SPFA_PATH_TILED);
  } else {  // the two operators one after the other on the same state
    rc = spfa_local_forward_f32(Q, K, V, m, l, O, L, d, w, row_begin, row_end, nullptr, 0, stream);
    if (rc == SPFA_OK)
      rc = spfa_global_no_local_forward_f32(Q, K, V, m, l, O, G, nG, L, d, w, row_begin, row_end, ws, gnl_bytes, stream);
  }
  if (rc || nnz == 0) return rc;
  const int taken = g_last_path.load();
  rc = spfa_csr_forward_f32(Q, K, V, row_off, col_ind, nnz, m, l, O, n_rows, L, d, 0, ws + gnl_bytes,
                            workspace_bytes - gnl_bytes, stream);
  if (taken == SPFA_PATH_TILED) g_last_path.store(SPFA_PATH_TILED);
  return rc;
}

// ---- dense mask -> CSR / COO arrays ------------------------------------------------------------------------
int spfa_dense_mask_offsets(const uint8_t* mask, int64_t n_rows, int64_t n_cols, uint64_t* row_off, void* stream) {
  if (!row_off || n_rows < 0 || n_cols < 0 || (n_rows > 0 && n_cols > 0 && !mask)) return SPFA_ERR_BAD_ARG;
  if (n_cols >= (1LL << 32)) return SPFA_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  unsigned long long* off = reinterpret_cast<unsigned long long*>(row_off);
  if (n_rows > 0) {
    const int64_t blocks = (n_rows + 7) / 8;
    if (blocks > 0x7fffffffLL) return SPFA_ERR_TOO_LARGE;
    mask_row_counts_kernel<<<(unsigned)blocks, 256, 0, st>>>(mask, n_rows, n_cols, off);
    g_launches.fetch_add(1);
    if (launch_status() != SPFA_OK) return SPFA_ERR_LAUNCH;
  }
  offsets_scan_kernel<<<1, 1024, 0, st>>>(off, n_rows);
  g_launches.fetch_add(1);
  return launch_status();
}

int spfa_dense_mask_fill(const uint8_t* mask, int64_t n_rows, int64_t n_cols, const uint64_t* row_off, uint32_t* col_ind,
                         uint64_t* row_ind, void* stream) {
  if (n_rows < 0 || n_cols < 0 || !row_off) return SPFA_ERR_BAD_ARG;
  if (n_rows == 0 || n_cols == 0) return SPFA_OK;
  if (!mask || !col_ind) return SPFA_ERR_BAD_ARG;
  const int64_t blocks = (n_rows + 7) / 8;
  if (blocks > 0x7fffffffLL || n_cols >= (1LL << 32)) return SPFA_ERR_TOO_LARGE;
  mask_fill_columns_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      mask, n_rows, n_cols, reinterpret_cast<const unsigned long long*>(row_off), col_ind,
      reinterpret_cast<unsigned long long*>(row_ind));
  g_launches.fetch_add(1);
  return launch_status();
}

// ---- visited-pair dump -----------------------------------------------------------------------------
int spfa_mask_count(int kind, int64_t L, int64_t p0, int64_t p1, const int32_t* G, int64_t nG, int64_t row_begin,
                    int64_t row_end, int64_t* counts, void* stream) {
  int rc = check_rows(L, row_begin, row_end);
  if (rc || !counts) return SPFA_ERR_BAD_ARG;
  const int64_t n_rows = row_end - row_begin;
  if (n_rows == 0) return SPFA_OK;
  return with_mask_cols(kind, L, p0, p1, G, nG, [&](auto cols) {
    mask_count_kernel<<<(unsigned)((n_rows + 127) / 128), 128, 0, (cudaStream_t)stream>>>(cols, row_begin, n_rows, counts);
    g_launches.fetch_add(1);
    return launch_status();
  });
}

int spfa_mask_fill(int kind, int64_t L, int64_t p0, int64_t p1, const int32_t* G, int64_t nG, int64_t row_begin,
                   int64_t row_end, const int64_t* row_off, uint32_t* col_out, void* stream) {
  int rc = check_rows(L, row_begin, row_end);
  if (rc || !row_off || !col_out) return SPFA_ERR_BAD_ARG;
  const int64_t n_rows = row_end - row_begin;
  if (n_rows == 0) return SPFA_OK;
  return with_mask_cols(kind, L, p0, p1, G, nG, [&](auto cols) {
    mask_fill_kernel<<<(unsigned)((n_rows + 127) / 128), 128, 0, (cudaStream_t)stream>>>(cols, row_begin, n_rows, row_off,
                                                                                       col_out);
    g_launches.fetch_add(1);
    return launch_status();
  });
}

}  // extern "C"
