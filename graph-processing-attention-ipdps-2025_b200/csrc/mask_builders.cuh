// Dense boolean mask -> CSR / COO index arrays on the GPU.
//
// Callers of the reference build explicit masks from a dense [L, Lk] boolean tensor with torch's
// to_sparse_csr() / to_sparse_coo() followed by dtype casts (verification/verify.py:67-71, 94-98); at 1e8 mask
// entries that conversion costs far more than the attention kernel it feeds. These kernels produce the arrays the
// operators take -- 64-bit row offsets or row indices, 32-bit columns ascending within a row -- in two passes over
// the mask, each at streaming speed:
//   1. mask_row_counts_kernel   entries per row (one warp per row, 128-byte warp loads), then an exclusive scan
//   2. mask_fill_kernel         columns (and, for COO, row numbers) written at the scanned offsets
// The mask is read as bytes (torch.bool / uint8); any non-zero byte is an entry.
#pragma once
#include "spfa_common.cuh"

namespace spfa {

// Word w (4 mask bytes) of the flat mask, with the bytes outside [lo, hi) cleared. `base4` is the mask pointer rounded
// down to 4 bytes and `shift` the number of bytes that rounding skipped.
__device__ __forceinline__ uint32_t mask_word(const uint32_t* __restrict__ base4, int64_t w, int64_t lo, int64_t hi) {
  uint32_t x = __ldg(base4 + w);
  const int64_t b0 = w * 4;  // flat byte index (relative to base4) of the word's first byte
  if (b0 < lo) x &= 0xffffffffu << (8 * (int)(lo - b0));
  if (b0 + 4 > hi) x &= (hi - b0 >= 4) ? 0xffffffffu : (0xffffffffu >> (8 * (int)(b0 + 4 - hi)));
  return __vcmpne4(x, 0u) & 0x01010101u;  // one bit per non-zero byte
}

// counts[r + 1] = entries of row r (counts[0] is set to 0 by the scan).
__global__ void mask_row_counts_kernel(const uint8_t* __restrict__ mask, int64_t n_rows, int64_t n_cols,
                                       unsigned long long* __restrict__ counts) {
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const uintptr_t p = reinterpret_cast<uintptr_t>(mask);
  const int shift = (int)(p & 3u);
  const uint32_t* base4 = reinterpret_cast<const uint32_t*>(p - shift);
  const int64_t lo = shift + r * n_cols, hi = lo + n_cols;
  int n = 0;
  for (int64_t w = lo / 4 + lane; w * 4 < hi; w += 32) n += __popc(mask_word(base4, w, lo, hi));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(kFullMask, n, o);
  if (lane == 0) counts[r + 1] = (unsigned long long)n;
}

// In-place exclusive scan of off[1 .. n] (counts) into offsets, off[0] = 0. One CTA: every thread owns a contiguous
// segment, the segment sums are scanned in shared memory.
__global__ void __launch_bounds__(1024) offsets_scan_kernel(unsigned long long* __restrict__ off, int64_t n) {
  __shared__ unsigned long long s_sum[1024];
  const int t = threadIdx.x;
  const int64_t per = (n + 1023) / 1024;
  const int64_t a = 1 + t * per, b = (a + per < n + 1) ? (a + per) : (n + 1);
  unsigned long long sum = 0;
  for (int64_t i = a; i < b; ++i) sum += off[i];
  s_sum[t] = sum;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {  // Hillis-Steele inclusive scan of the segment sums
    const unsigned long long v = (t >= o) ? s_sum[t - o] : 0ull;
    __syncthreads();
    s_sum[t] += v;
    __syncthreads();
  }
  unsigned long long run = (t > 0) ? s_sum[t - 1] : 0ull;
  if (t == 0) off[0] = 0ull;
  for (int64_t i = a; i < b; ++i) {  // off[i] becomes the sum of counts up to and including row i-1
    run += off[i];
    off[i] = run;
  }
}

// col[off[r] ...] = columns of row r, ascending; row_ind (COO, may be null) gets r for each of them.
__global__ void mask_fill_columns_kernel(const uint8_t* __restrict__ mask, int64_t n_rows, int64_t n_cols,
                                         const unsigned long long* __restrict__ off, uint32_t* __restrict__ col,
                                         unsigned long long* __restrict__ row_ind) {
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const uintptr_t p = reinterpret_cast<uintptr_t>(mask);
  const int shift = (int)(p & 3u);
  const uint32_t* base4 = reinterpret_cast<const uint32_t*>(p - shift);
  const int64_t lo = shift + r * n_cols, hi = lo + n_cols;
  unsigned long long at = off[r];
  for (int64_t w0 = lo / 4; w0 * 4 < hi; w0 += 32) {  // warp-uniform trip count
    const int64_t w = w0 + lane;
    const uint32_t bits = (w * 4 < hi) ? mask_word(base4, w, lo, hi) : 0u;
    const int mine = __popc(bits);
    int before = mine;  // inclusive prefix over the lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(kFullMask, before, o);
      if (lane >= o) before += v;
    }
    const int total = __shfl_sync(kFullMask, before, 31);
    unsigned long long q = at + (unsigned long long)(before - mine);
#pragma unroll
    for (int b = 0; b < 4; ++b)
      if ((bits >> (8 * b)) & 1u) {
        col[q] = (uint32_t)(w * 4 + b - lo);
        if (row_ind) row_ind[q] = (unsigned long long)r;
        ++q;
      }
    at += (unsigned long long)total;
  }
}

}  // namespace spfa
