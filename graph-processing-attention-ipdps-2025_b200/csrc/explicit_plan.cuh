// Explicit masks (CSR, and COO after its row-pointer pass) as a hybrid of the two paths.
//
// The query rows are cut into 128-row blocks and the keys into tiles of BN consecutive rows. A (block, tile)
// pair that holds many mask entries is a small dense problem: it goes to the tiled tensor-core kernel with a
// bit mask of its valid (row, key) pairs. Every other entry stays on the FP32 gather path. Both passes merge
// into the caller's (m, l, O) state, so their order does not matter and the result is the union.
//
// explicit_plan_kernel does the split, one CTA per 128-row block:
//   1. histogram of the entries of every 4th row of the block over ALL key tiles (shared memory, one 16-bit
//      counter per tile)
//   2. the tiles with at least a quarter of `min_entries` sampled entries, ascending, at most kMaxDenseTiles,
//      become "dense"
//   3. bit masks of the dense tiles are built in shared memory; a tile in which some (row, key) pair occurs
//      twice is demoted (a bit cannot say "twice", and the reference counts such a key twice)
//   4. space for the masks is taken from a pool in the workspace (one atomicAdd per block); a block that does
//      not get space keeps all its entries on the gather path
//   5. the block's remaining entries are written, in storage order, to a residual column list that keeps the
//      original row offsets (row r: res_col[row_off[r] .. row_off[r] + res_cnt[r])); columns >= Lk are dropped
//      (the ABI skips them); rows without any entry are NaN-filled here when use_nan is set
// Steps 3 and 5 share one walk over the block's entries; the walk of step 5 is repeated only for a block that
// had a tile demoted in step 3 or 4. Shared memory is kept small enough for four CTAs per SM (the histogram of
// step 1 and the masks of step 3 share one region; from step 3 on "is this key tile dense, and which slot" is
// answered by a byte table over the span of the dense tiles, or by a bit per key tile plus a per-word count when
// the dense tiles lie more than 255 tiles apart).
// The walks are bound by instruction issue (the integer pipe), not by memory: a warp takes a row 128 entries at a
// time, every lane FOUR CONSECUTIVE entries from one 16-byte load, so the ascending-order check and the per-lane
// count of residual entries are settled inside the lane; the lanes meet only for the prefix sum that places the
// residual entries (three ballots over the bits of the per-lane counts) and for one shuffle of the order check.
// A dense entry sets its bit with one shared-memory atomic (entries of one warp instruction lie four apart in the
// row, so a band puts about eight lanes on one word and the memory pipe, which has the headroom, serialises them);
// the histogram merges runs of equal key tiles inside a lane first. In blocks whose entries are almost all dense
// (block-structured masks) a step whose lanes each hold four consecutive columns of one 32-key group is settled
// with one lookup and one atomic per lane.
#pragma once
#include "gather_kernels.cuh"
#include "spfa_common.cuh"
#include "tile_kernels_sm100.cuh"

namespace spfa {

// Residual rows longer than this are listed and walked by all warps of a CTA at the start of the gather launch:
// one warp needs about a microsecond per eight scattered keys, so longer rows left to single warps would form
// the launch's tail.
constexpr int kListedRowSlots = 128;
// Residual rows longer than this are cut into slices that different CTAs walk at the same time (partial softmax states
// in scratch, folded by whichever CTA finishes a row's last slice): a row of 8000 scattered keys walked by one CTA takes
// about half a millisecond, which is a fixed tail once the rest of a launch is short (a rank's share of a multi-GPU split).
constexpr int kSplitRowSlots = 1024;
constexpr int kPlanThreads = 512;
constexpr int kPlanSampleStride = 4;  // the histogram looks at every 4th row of a block
constexpr int kPlanWarps = kPlanThreads / 32;
constexpr int kPlanMaxSmem = 200 * 1024;

struct ExplicitPlan {
  // per 128-row block
  int* rb_nt;                       // [n_blocks] dense tiles
  int* rb_kt;                       // [n_blocks][kMaxDenseTiles] key-tile numbers, ascending
  long long* rb_moff;               // [n_blocks] first mask word of the block
  // mask pool
  uint32_t* masks;                  // [cap_words]; tile t of a block: (t*(BN/32) + chunk)*128 + row
  unsigned long long* pool_used;    // words handed out so far (zeroed before the kernel)
  long long cap_words;
  // residual entries for the gather path
  uint32_t* res_cnt;                // [n_rows]
  uint32_t* res_col;                // [nnz], row r at res_col + row_off[r]
  // rows whose residual part is longer than kListedRowSlots get CTAs of their own (gather_rows_listed_first_kernel)
  unsigned int* heavy_count;        // zeroed before the kernel
  int* heavy_rows;                  // [n_rows]
  // set to 1 by any block that meets a row whose kept columns are not ascending (zeroed before the kernel):
  // key-range passes may binary-search the residual rows only while it stays 0
  unsigned int* unsorted;
  PlanHeader* header;
  // rows cut into slices: one item per (row, slice), items of a row adjacent
  unsigned int* split_count;        // zeroed before the kernel
  int4* split_items;                // {row, slice, slices of the row, index of the row's first item}
  unsigned int* split_done;         // per item index of a row's first item: slices finished (zero outside a forward call)
  float* split_part;                // [items][d + 4]: un-normalised accumulator, then m, l
  long long cap_items;
};

// Adds a row of `kept` residual entries to the split list (kept > kSplitRowSlots). Rows that do not fit the list any
// more stay whole on the list of long rows.
__device__ __forceinline__ void list_long_row(const ExplicitPlan& plan, int row, uint32_t kept) {
  if (kept > (uint32_t)kSplitRowSlots) {
    const unsigned int ns = (kept + kSplitRowSlots - 1) / kSplitRowSlots;
    const unsigned int first = atomicAdd(plan.split_count, ns);
    if ((long long)first + ns <= plan.cap_items) {
      for (unsigned int sl = 0; sl < ns; ++sl) plan.split_items[first + sl] = make_int4(row, (int)sl, (int)ns, (int)first);
      return;
    }
    for (unsigned int sl = 0; sl < ns && (long long)first + sl < plan.cap_items; ++sl)  // overflowed: neutral items
      plan.split_items[first + sl] = make_int4(-1, 0, 0, 0);
  }
  plan.heavy_rows[atomicAdd(plan.heavy_count, 1u)] = row;
}

// Residual rows of the hybrid (see above): same offsets as the caller's CSR, fewer entries, all < Lk.
struct ResidualCols {
  const uint64_t* row_off;
  const uint32_t* cnt;
  const uint32_t* col;
  uint32_t skip_above;  // rows with more residual entries than this read as empty (they are on the heavy list)
  static constexpr bool kNanFillEmpty = false;  // the plan kernel has filled the rows that are really empty
  struct Row { int64_t lo; int64_t n; };
  __device__ __forceinline__ Row open(int64_t r_local, int64_t) const {
    Row r;
    r.lo = (int64_t)row_off[r_local];
    const uint32_t n = cnt[r_local];
    r.n = (n > skip_above) ? 0 : (int64_t)n;
    return r;
  }
  __device__ __forceinline__ int32_t slot(const Row& r, int64_t t) const { return (int32_t)__ldg(col + r.lo + t); }
};

// The same rows restricted to the keys [key_lo, key_hi): one pass of a forward that is split along the key axis
// (multi-GPU callers run one pass per K/V chunk as the chunks arrive; the passes chain through (m, l, O)).
// Rows whose columns ascend -- the inspector records whether all do -- are cut by two binary searches;
// otherwise every slot is looked at and the ones outside the range are skipped.
struct ResidualRangeCols {
  const uint64_t* row_off;
  const uint32_t* cnt;
  const uint32_t* col;
  uint32_t skip_above;
  uint32_t key_lo, key_hi;
  const unsigned int* unsorted;  // the plan's flag
  static constexpr bool kNanFillEmpty = false;
  // key_lo > key_hi names the cyclic range [key_lo, inf) + [0, key_hi). A row's share of a range is its ascending
  // list minus one gap: slots [0, gap_at) and [gap_at + gap_len, ...).
  struct Row { int64_t lo; int64_t n; int64_t gap_at; int64_t gap_len; bool filter; };
  __device__ __forceinline__ bool wanted(uint32_t c) const {
    return (key_lo <= key_hi) ? (c >= key_lo && c < key_hi) : (c >= key_lo || c < key_hi);
  }
  // Entries of the ascending list col[lo, lo + n) that are below v1 / below v2, found by the whole warp together
  // (every lane of the warp must call open() for the same row): short rows are loaded once, coalesced, and counted
  // with ballots; long rows take a 33-way search, one memory round trip per level instead of one per halving.
  __device__ __forceinline__ void warp_count_below(int64_t lo, int64_t n, uint32_t v1, uint32_t v2, int64_t* c1,
                                                   int64_t* c2) const {
    const int lane = threadIdx.x & 31;
    if (n <= 128) {
      uint32_t x[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = (k * 32 + lane < n) ? __ldg(col + lo + k * 32 + lane) : 0xffffffffu;
      int a = 0, b = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        a += __popc(__ballot_sync(kFullMask, x[k] < v1));
        b += __popc(__ballot_sync(kFullMask, x[k] < v2));
      }
      *c1 = a;
      *c2 = b;
      return;
    }
    int64_t res[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint32_t v = q ? v2 : v1;
      int64_t a = 0, b = n;  // the count lies in [a, b]
      while (b - a > 32) {
        const int64_t span = b - a;
        const int64_t idx = a + span * (lane + 1) / 33;  // a < idx < b, ascending with the lane
        const int c = __popc(__ballot_sync(kFullMask, __ldg(col + lo + idx) < v));  // lanes 0 .. c-1 saw a smaller entry
        const int64_t na = (c == 0) ? a : (a + span * c / 33 + 1);
        const int64_t nb = (c == 32) ? b : (a + span * (c + 1) / 33);
        a = na;
        b = nb;
      }
      const uint32_t x = (a + lane < b) ? __ldg(col + lo + a + lane) : 0xffffffffu;
      res[q] = a + __popc(__ballot_sync(kFullMask, x < v));
    }
    *c1 = res[0];
    *c2 = res[1];
  }
  __device__ __forceinline__ Row open(int64_t r_local, int64_t) const {
    Row r;
    r.lo = (int64_t)row_off[r_local];
    const uint32_t n = cnt[r_local];
    r.n = (n > skip_above) ? 0 : (int64_t)n;
    r.filter = (*unsorted != 0u);
    r.gap_at = r.n;
    r.gap_len = 0;
    if (!r.filter && r.n > 0) {
      int64_t a, b;  // entries below key_lo / below key_hi
      warp_count_below(r.lo, r.n, key_lo, key_hi, &a, &b);
      if (key_lo <= key_hi) {  // keep [a, b)
        r.lo += a;
        r.n = b - a;
        r.gap_at = r.n;
      } else {                 // keep [0, b) and [a, n)
        r.gap_at = b;
        r.gap_len = a - b;
        r.n -= r.gap_len;
      }
    }
    return r;
  }
  __device__ __forceinline__ int32_t slot(const Row& r, int64_t t) const {
    const uint32_t c = __ldg(col + r.lo + (t < r.gap_at ? t : t + r.gap_len));
    return (!r.filter || wanted(c)) ? (int32_t)c : -1;
  }
};

inline size_t explicit_plan_smem_bytes(int64_t n_key_tiles, int bn) {
  const size_t hist = ((size_t)(n_key_tiles + 1) / 2 + 15) / 16 * 16 * 4;  // 16-bit counters, two per word, whole 64-byte groups
  const size_t masks = (size_t)tile::kMaxDenseTiles * (bn / 32) * 128 * 4;
  const size_t words = (size_t)(n_key_tiles + 31) / 32;
  return (hist > masks ? hist : masks) + words * 4 + (words + 3) / 4 * 4;
}

// Four consecutive entries e .. e+3 of the column array from one 16-byte load; `e` must put the address on a
// 16-byte boundary. Positions outside [0, nnz) (only the array's first and last chunk can have some) read as `none`.
__device__ __forceinline__ void load_four_columns(const uint32_t* __restrict__ col, int64_t e, int64_t nnz, uint32_t none,
                                                  uint32_t (&c)[4]) {
  if (e >= 0 && e + 4 <= nnz) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(col + e));
    c[0] = v.x;
    c[1] = v.y;
    c[2] = v.z;
    c[3] = v.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) c[j] = (e + j >= 0 && e + j < nnz) ? __ldg(col + e + j) : none;
  }
}

// A warp's walk over the entries [a, z) of one row, 128 per step: the step's first entry index (a multiple-of-16-byte
// address at or below a) and, per step, the window [lo, hi) of positions 0..127 that belong to the row.
struct RowSteps {
  int64_t first;
  __device__ __forceinline__ RowSteps(const uint32_t* col, int64_t a) {
    const int mis = (int)((reinterpret_cast<uintptr_t>(col) >> 2) & 3u);  // entries between col and a 16-byte boundary
    first = a - (int64_t)((a + mis) & 3);
  }
};

template <int BN>
__global__ void __launch_bounds__(kPlanThreads, 4)
explicit_plan_kernel(const uint64_t* __restrict__ row_off, const uint32_t* __restrict__ col, int64_t n_rows, int64_t nnz,
                     int64_t Lk, int n_key_tiles, int min_entries, ExplicitPlan plan, int use_nan, float* __restrict__ O,
                     int d) {
  constexpr int NC = BN / 32;
  constexpr int MAXT = tile::kMaxDenseTiles;
  constexpr uint32_t kNoKey = 0xffffffffu;
  extern __shared__ uint32_t plan_smem[];
  const int n_words = (n_key_tiles + 31) / 32;
  const int n_hist_words = ((n_key_tiles + 1) / 2 + 15) / 16 * 16;  // the counters of 32 key tiles are four 16-byte loads
  const int region = (n_hist_words > MAXT * NC * 128) ? n_hist_words : MAXT * NC * 128;
  // Entry counts as 16-bit halves of 32-bit words. A count beyond 65535 (only possible with heavily duplicated
  // entries) carries into its neighbour: that can only change which tiles are CALLED dense, never the result,
  // because masks and residual lists are built from the entries themselves.
  uint32_t* hist = plan_smem;                 // [(n_key_tiles + 1) / 2]               (steps 1-2)
  auto count_of = [&](int k) -> uint32_t { return (hist[k >> 1] >> ((k & 1) * 16)) & 0xffffu; };
  uint32_t* masks = plan_smem;                // [MAXT][NC][128], same storage         (steps 3-4)
  uint32_t* dense_bits = plan_smem + region;  // [n_words] bit k: key tile k is dense
  uint8_t* dense_before = reinterpret_cast<uint8_t*>(dense_bits + n_words);  // [n_words] dense tiles in earlier words
  __shared__ unsigned long long s_off[129];      // the block's row offsets
  __shared__ int s_warp_cnt[kPlanWarps];
  __shared__ int s_sel[MAXT];                    // key tile of slot t
  __shared__ int s_dirty[MAXT];
  __shared__ int s_map[MAXT];                    // slot -> position among the clean slots, or -1
  __shared__ uint8_t s_tab[256];                 // slot + 1 of key tile kt_lo + i while the dense tiles span < 256 tiles
  __shared__ int s_nt, s_nclean, s_redo;
  __shared__ int s_sampled, s_in_dense;  // sampled entries of the block / those that fell into its dense tiles
  __shared__ int s_next_row[2];  // rows are claimed one at a time (row lengths differ widely): step 3, step 5 again
  __shared__ long long s_moff;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t b = blockIdx.x;
  const int64_t r0 = b * 128;
  const int nr = (int)((n_rows - r0 < 128) ? (n_rows - r0) : 128);
  if (tid <= nr) {  // offsets beyond the column array (a malformed mask) are clamped: nothing is read or written past nnz
    unsigned long long o = row_off[r0 + tid];
    s_off[tid] = (o > (unsigned long long)nnz) ? (unsigned long long)nnz : o;
  }
  if (b == 0 && tid == 0) {
    PlanHeader h;
    h.magic = kPlanMagic;
    h.n_rows = n_rows;
    h.nnz = nnz;
    h.n_keys = Lk;
    h.d = d;
    h.bn = BN;
    *plan.header = h;
  }
  for (int k = tid; k < n_hist_words; k += kPlanThreads) hist[k] = 0;
  for (int k = tid; k < n_words; k += kPlanThreads) dense_bits[k] = 0;
  if (tid < MAXT) s_dirty[tid] = 0;
  if (tid < 2) s_next_row[tid] = kPlanWarps;
  if (tid == 0) s_sampled = s_in_dense = 0;
  __syncthreads();

  // ---- 1. histogram over key tiles, from every kPlanSampleStride-th row of the block ----
  // The counts only decide which tiles are CALLED dense (masks and residual lists are built from all entries
  // below), so a sample is enough: a tile is dense if the sampled rows hold their share of min_entries.
  const uint32_t Lk32 = (Lk < 0xffffffffLL) ? (uint32_t)Lk : 0xffffffffu;  // kNoKey is never a valid column
  for (int rl = warp * kPlanSampleStride; rl < nr; rl += kPlanWarps * kPlanSampleStride) {
    const int64_t a = (int64_t)s_off[rl], z = (int64_t)s_off[rl + 1];
    if (lane == 0 && z > a) atomicAdd(&s_sampled, (int)((z - a < (1 << 20)) ? (z - a) : (1 << 20)));
    for (int64_t base = (a < z) ? RowSteps(col, a).first : z; base < z; base += 128) {
      const int lo = (a > base) ? (int)(a - base) : 0, hi = (z - base < 128) ? (int)(z - base) : 128;  // warp-uniform
      uint32_t cu[4];
      if (lane * 4 < hi) load_four_columns(col, base + lane * 4, nnz, kNoKey, cu);
      uint32_t k_run = kNoKey, n_run = 0;  // a run of entries of one key tile inside this lane
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int p = lane * 4 + j;
        if (p < lo || p >= hi || cu[j] >= Lk32) continue;
        const uint32_t kt = cu[j] / BN;
        if (kt != k_run) {
          if (n_run) atomicAdd(&hist[k_run >> 1], n_run << ((k_run & 1) * 16));
          k_run = kt;
          n_run = 0;
        }
        ++n_run;
      }
      if (n_run) atomicAdd(&hist[k_run >> 1], n_run << ((k_run & 1) * 16));
    }
  }
  __syncthreads();
  min_entries = (min_entries + kPlanSampleStride - 1) / kPlanSampleStride;

  // ---- 2. dense tiles, ascending. A lane turns the 32 counters behind one word of dense_bits into that word (SIMD
  //         compares on the 16-bit halves); each warp owns a contiguous range of words, so the ranges are in tile order ----
  {
    const uint32_t thr = (min_entries < 1) ? 1u : (min_entries > 0xffff ? 0xffffu : (uint32_t)min_entries);
    const uint32_t thr2 = thr | (thr << 16);
    auto dense_word = [&](int w) -> uint32_t {
      const uint4* h4 = reinterpret_cast<const uint4*>(hist + (size_t)w * 16);
      auto two = [&](uint32_t x) -> uint32_t {  // bit 0 / 1: low / high counter >= thr
        const uint32_t r = __vcmpgeu2(x, thr2);
        return (r & 1u) | ((r >> 15) & 2u);
      };
      uint32_t bits = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 v = h4[q];
        bits |= (two(v.x) | (two(v.y) << 2) | (two(v.z) << 4) | (two(v.w) << 6)) << (8 * q);
      }
      return bits;
    };
    const int per_w = ((n_words + kPlanWarps - 1) / kPlanWarps + 31) / 32 * 32;
    const int w_lo = warp * per_w, w_hi = (w_lo + per_w < n_words) ? (w_lo + per_w) : n_words;
    int mine = 0;  // dense tiles in this warp's range
    for (int w0 = w_lo; w0 < w_hi; w0 += 32) {
      const int w = w0 + lane;
      if (w < w_hi) {
        const uint32_t dw = dense_word(w);
        dense_bits[w] = dw;
        mine += __popc(dw);
      }
    }
    mine = __reduce_add_sync(kFullMask, mine);
    if (lane == 0) s_warp_cnt[warp] = mine;
    __syncthreads();
    int before = 0, total = 0;
    for (int wv = 0; wv < kPlanWarps; ++wv) {
      before += (wv < warp) ? s_warp_cnt[wv] : 0;
      total += s_warp_cnt[wv];
    }
    if (tid == 0) s_nt = (total < MAXT) ? total : MAXT;
    if (mine > 0)  // number the warp's dense tiles; those beyond the MAXT-th lose their bit
      for (int w0 = w_lo; w0 < w_hi; w0 += 32) {
        const int w = w0 + lane;
        uint32_t dw = (w < w_hi) ? dense_bits[w] : 0u;
        const int cnt = __popc(dw);
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(kFullMask, incl, o);
          if (lane >= o) incl += v;
        }
        int idx = before + incl - cnt;
        if (cnt) {
          uint32_t keep_w = dw;
          for (uint32_t left = dw; left; left &= left - 1u) {
            const int bit = __ffs(left) - 1;
            if (idx < MAXT) s_sel[idx] = w * 32 + bit;
            else keep_w &= ~(1u << bit);
            ++idx;
          }
          if (keep_w != dw) dense_bits[w] = keep_w;
        }
        before += __shfl_sync(kFullMask, incl, 31);
      }
  }
  __syncthreads();
  const int nt = s_nt;
  if (tid < nt) atomicAdd(&s_in_dense, (int)count_of(s_sel[tid]));
  __syncthreads();  // the histogram is dead from here on: its storage becomes the masks
  // A block whose entries lie almost all in dense tiles (block-structured masks) is walked with a warp-level shortcut
  // for runs of consecutive columns; elsewhere the test for it would only cost issue slots.
  const bool dense_heavy = (long long)s_in_dense * 10 >= (long long)s_sampled * 9 && s_in_dense > 0;
  for (int w = tid; w < n_words; w += kPlanThreads) {
    int c = 0;
    for (int t = 0; t < nt; ++t) c += ((s_sel[t] >> 5) < w);
    dense_before[w] = (uint8_t)c;
  }
  // dense tiles lie in [kt_lo, kt_lo + kt_span] (s_sel ascends); a key tile outside is residual without a lookup
  const uint32_t kt_lo = nt ? (uint32_t)s_sel[0] : 1u, kt_span = nt ? (uint32_t)s_sel[nt - 1] - kt_lo : 0u;
  const bool use_tab = kt_span < 256u;  // the usual case (a band, a few clusters): one byte load answers the lookup
  if (tid < 256) {
    uint32_t v = 0;
    for (int t = 0; t < nt; ++t)
      if ((uint32_t)s_sel[t] == kt_lo + (uint32_t)tid) v = (uint32_t)t + 1u;
    s_tab[tid] = (uint8_t)v;
  }
  // slot + 1 of a dense key tile, 0 for any other
  auto slot1_of = [&](uint32_t kt) -> uint32_t {
    const uint32_t w = dense_bits[kt >> 5], bit = 1u << (kt & 31);
    return (w & bit) ? (uint32_t)dense_before[kt >> 5] + __popc(w & (bit - 1u)) + 1u : 0u;
  };

  // ---- 3. bit masks of the dense tiles (duplicates demote a tile) and, in the same walk, 5. the residual list ----
  for (int i = tid; i < nt * NC * 128; i += kPlanThreads) masks[i] = 0;
  __syncthreads();
  const uint32_t lanes_below = (1u << lane) - 1u;
  auto claim_row = [&](int which) -> int {
    int nxt = 0;
    if (lane == 0) nxt = atomicAdd(&s_next_row[which], 1);
    return __shfl_sync(kFullMask, nxt, 0);
  };
  for (int rl = warp; rl < nr; rl = claim_row(0)) {
    const int64_t a = (int64_t)s_off[rl], z = (int64_t)s_off[rl + 1];
    uint32_t kept = 0;
    uint32_t last_col = 0;  // column of the previous step's last entry
    bool row_unsorted = false;
    for (int64_t base = (a < z) ? RowSteps(col, a).first : z; base < z; base += 128) {
      const int lo = (a > base) ? (int)(a - base) : 0, hi = (z - base < 128) ? (int)(z - base) : 128;  // warp-uniform
      uint32_t cu[4] = {kNoKey, kNoKey, kNoKey, kNoKey};
      if (lane * 4 < hi) load_four_columns(col, base + lane * 4, nnz, kNoKey, cu);
      // bit j: entry j of this lane belongs to the row
      const int lo_l = min(max(lo - lane * 4, 0), 4), hi_l = min(max(hi - lane * 4, 0), 4);
      const uint32_t in_row = ((1u << hi_l) - 1u) & ~((1u << lo_l) - 1u);
      if (in_row != 0xfu) {  // positions outside the row take the smallest / largest column: they never break the order
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (!((in_row >> j) & 1u)) cu[j] = (j < lo_l) ? 0u : kNoKey;
      }
      uint32_t keep_bits = 0;  // bit j: entry j of this lane stays on the gather path
      bool done = false;
      if (dense_heavy) {  // every busy lane holds four consecutive columns of one 32-key group: one lookup, one atomic
        const bool run4 = in_row == 0xfu && cu[3] < Lk32 && cu[1] == cu[0] + 1u && cu[2] == cu[0] + 2u &&
                          cu[3] == cu[0] + 3u && ((cu[0] ^ cu[3]) >> 5) == 0u;
        done = __all_sync(kFullMask, run4 || in_row == 0u);
        if (done && run4) {
          const uint32_t kt = cu[0] / BN, dk = kt - kt_lo;
          uint32_t slot1 = 0;
          if (dk <= kt_span) slot1 = use_tab ? (uint32_t)s_tab[dk] : slot1_of(kt);
          if (slot1) {
            const uint32_t kk = cu[0] - kt * BN, bits = 0xfu << (kk & 31);
            const uint32_t old = atomicOr(&masks[((slot1 - 1) * NC + (kk >> 5)) * 128 + rl], bits);
            if (old & bits) s_dirty[slot1 - 1] = 1;
          } else {
            keep_bits = 0xfu;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t c = cu[j];
        if (done || !((in_row >> j) & 1u) || c >= Lk32) continue;
        const uint32_t kt = c / BN, dk = kt - kt_lo;
        uint32_t slot1 = 0;
        if (dk <= kt_span) slot1 = use_tab ? (uint32_t)s_tab[dk] : slot1_of(kt);
        if (!slot1) {
          keep_bits |= 1u << j;
          continue;
        }
        // lanes that hit the same mask word are serialised by the memory pipe; `old` tells a pair that occurs twice
        const uint32_t kk = c - kt * BN, bit = 1u << (kk & 31);
        const uint32_t old = atomicOr(&masks[((slot1 - 1) * NC + (kk >> 5)) * 128 + rl], bit);
        if (old & bit) s_dirty[slot1 - 1] = 1;  // a bit cannot say "twice"
      }
      {  // ascending order of the row's columns (all entries, so the kept ones as well)
        const uint32_t before = __shfl_up_sync(kFullMask, cu[3], 1);
        const uint32_t prev = (lane == 0) ? last_col : before;
        if (prev > cu[0] || cu[0] > cu[1] || cu[1] > cu[2] || cu[2] > cu[3]) row_unsorted = true;
        last_col = __shfl_sync(kFullMask, cu[3], 31);
      }
      // residual entries in storage order: prefix sum of the per-lane counts (0..4) from ballots of their three bits
      const uint32_t cnt = __popc(keep_bits);
      const uint32_t b0 = __ballot_sync(kFullMask, cnt & 1u), b1 = __ballot_sync(kFullMask, cnt & 2u),
                     b2 = __ballot_sync(kFullMask, cnt & 4u);
      if ((b0 | b1 | b2) == 0u) continue;  // warp-uniform
      uint32_t* dst = plan.res_col + a + kept + __popc(b0 & lanes_below) + 2 * __popc(b1 & lanes_below) +
                      4 * __popc(b2 & lanes_below);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (keep_bits & (1u << j)) *dst++ = cu[j];
      kept += __popc(b0) + 2 * __popc(b1) + 4 * __popc(b2);
    }
    if (__any_sync(kFullMask, row_unsorted) && lane == 0) *plan.unsorted = 1u;  // benign race: every writer stores 1
    if (lane == 0) {
      plan.res_cnt[r0 + rl] = kept;
      if (kept > (uint32_t)kListedRowSlots) list_long_row(plan, (int)(r0 + rl), kept);
    }
    if (z <= a && use_nan) {  // a row without any entry
      const float nn = __int_as_float(0x7fc00000);
      for (int i = lane * 4; i < d; i += 128)
        *reinterpret_cast<float4*>(O + (size_t)(r0 + rl) * d + i) = make_float4(nn, nn, nn, nn);
    }
  }
  __syncthreads();

  // ---- 4. drop the demoted tiles, take mask space from the pool, publish the block's tile list ----
  if (tid == 0) {
    int nc = 0;
    for (int t = 0; t < nt; ++t) s_map[t] = s_dirty[t] ? -1 : nc++;
    long long off = 0;
    if (nc > 0) {
      const long long need = (long long)nc * NC * 128;
      off = (long long)atomicAdd(plan.pool_used, (unsigned long long)need);
      if (off + need > plan.cap_words) {  // pool exhausted: this block stays on the gather path
        for (int t = 0; t < nt; ++t) s_map[t] = -1;
        nc = 0;
        off = 0;
      }
    }
    s_nclean = nc;
    s_redo = (nc != nt);
    s_moff = off;
    plan.rb_nt[b] = nc;
    plan.rb_moff[b] = off;
  }
  __syncthreads();
  const int nclean = s_nclean;
  if (tid < nt) {
    const int to = s_map[tid];
    if (to >= 0) plan.rb_kt[b * MAXT + to] = s_sel[tid];
    else atomicAnd(&dense_bits[s_sel[tid] >> 5], ~(1u << (s_sel[tid] & 31)));  // its entries are residual after all
  }
  if (nclean > 0) {
    uint32_t* dst = plan.masks + s_moff;
    for (int i = tid; i < nt * NC * 128; i += kPlanThreads) {
      const int to = s_map[i / (NC * 128)];
      if (to >= 0) dst[(size_t)to * NC * 128 + i % (NC * 128)] = masks[i];
    }
  }
  __syncthreads();

  // ---- 5 again, only if a tile was demoted: membership is all that is asked of the bits now ----
  if (!s_redo) return;
  for (int rl = warp; rl < nr; rl = claim_row(1)) {
    const int64_t a = (int64_t)s_off[rl], z = (int64_t)s_off[rl + 1];
    uint32_t kept = 0;
    for (int64_t base = (a < z) ? RowSteps(col, a).first : z; base < z; base += 128) {
      const int lo = (a > base) ? (int)(a - base) : 0, hi = (z - base < 128) ? (int)(z - base) : 128;  // warp-uniform
      uint32_t cu[4] = {kNoKey, kNoKey, kNoKey, kNoKey};
      if (lane * 4 < hi) load_four_columns(col, base + lane * 4, nnz, kNoKey, cu);
      uint32_t keep_bits = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int p = lane * 4 + j;
        const uint32_t c = cu[j];
        if (p < lo || p >= hi || c >= Lk32) continue;
        const uint32_t kt = c / BN;
        if (((dense_bits[kt >> 5] >> (kt & 31)) & 1u) == 0u) keep_bits |= 1u << j;
      }
      const uint32_t cnt = __popc(keep_bits);
      const uint32_t b0 = __ballot_sync(kFullMask, cnt & 1u), b1 = __ballot_sync(kFullMask, cnt & 2u),
                     b2 = __ballot_sync(kFullMask, cnt & 4u);
      uint32_t* dst = plan.res_col + a + kept + __popc(b0 & lanes_below) + 2 * __popc(b1 & lanes_below) +
                      4 * __popc(b2 & lanes_below);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (keep_bits & (1u << j)) *dst++ = cu[j];
      kept += __popc(b0) + 2 * __popc(b1) + 4 * __popc(b2);
    }
    if (lane == 0) {
      const uint32_t before_cnt = plan.res_cnt[r0 + rl];  // listed already if it was long before the demotion
      plan.res_cnt[r0 + rl] = kept;
      // (a row listed before keeps its place: slices are cut from the row's length at forward time, not from this count)
      if (kept > (uint32_t)kListedRowSlots && before_cnt <= (uint32_t)kListedRowSlots) list_long_row(plan, (int)(r0 + rl), kept);
    }
  }
}

}  // namespace spfa
