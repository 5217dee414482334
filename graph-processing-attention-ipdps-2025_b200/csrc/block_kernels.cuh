// Local-2D-dilated (block-diagonal, intra-block dilation) as one CTA per mask block.
//
// Index set (reference: sp_flatt_local_2d_dilated_kernel.cu:26-39,123): with s = dil_factor + 1 and
// start = (i / B) * B, row i is live iff (i - start) mod s == 0 and then attends to start + t*s for
// 0 <= t < n = min(B, (B-1)/s + 1). Every live row of a block therefore attends to the SAME n key rows:
// the block is a small dense problem on a strided subset, and the operator as a whole is bandwidth bound
// (the dead rows' NaN fill is most of the traffic). The gather kernel re-fetches those n K/V rows from
// L1/L2 once per live row; here they are staged in shared memory once per block.
//
// CTA = one mask block, 8 warps. Warp w takes live rows t = w, w+8, ...:
//   scores   lane <-> key (keys lane, lane+32, ...), K rows read from shared memory with a pitch of D+1
//            floats (conflict-free column walks), q broadcast from shared memory
//   softmax  max / sum by warp shuffles, exact FP32 (same recurrence and state merge as the gather path)
//   P V      lane <-> output dims (lane, lane+32, ...), probabilities broadcast from shared memory
// Dead rows of the block are NaN-filled (use_nan) by all threads with 128-bit stores.
#pragma once
#include "spfa_common.cuh"

namespace spfa {

constexpr int kBlockWarps = 8;
constexpr int kBlockMaxKeysPerLane = 8;  // n <= 256 keys per live row; the kernel is compiled for 1, 2, 4, 8

struct Block2dParams {
  int64_t L, B, s, n;            // n = keys per live row
  int64_t row_begin, row_end;    // shard (absolute rows); Q/m/l/O are indexed by row - row_begin
  int64_t first_block;           // mask block handled by CTA 0
  int use_nan;
  float scale;
};

template <int D>
__host__ __device__ constexpr size_t block2d_smem_bytes(int64_t n) {
  // K (pitch D+1, padded so that V starts 16-byte aligned), V (pitch D), per warp: q (D) + p (n rounded up to 32)
  return (size_t)((n * (D + 1) + 3) / 4 * 4 + n * D + kBlockWarps * (D + ((n + 31) / 32) * 32)) * sizeof(float);
}

// Few keys per lane leave room for seven CTAs per SM (36 registers per thread, ~30 KB of shared memory each):
// 1036 slots, so that the 1024 blocks of the 262144-row configuration are one wave instead of one and a bit.
template <int D, int NK>  // NK = keys per lane (n <= 32 NK)
__global__ void __launch_bounds__(kBlockWarps * 32, (NK <= 2) ? 7 : 1)
local2d_block_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                     float* __restrict__ m, float* __restrict__ l, float* __restrict__ O, const Block2dParams prm) {
  extern __shared__ float smem_f[];
  const int n = (int)prm.n;
  const int npad = ((n + 31) / 32) * 32;
  float* Ks = smem_f;                       // [n][D+1]
  float* Vs = Ks + ((size_t)n * (D + 1) + 3) / 4 * 4;  // [n][D], 16-byte aligned for the float4 stores below
  float* Ws = Vs + (size_t)n * D;           // per warp: q[D], p[npad]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = Ws + (size_t)warp * (D + npad);
  float* ps = qs + D;
  const int64_t start = (prm.first_block + blockIdx.x) * prm.B;

  // ---- stage the block's n key rows ----
  constexpr int C4 = D / 4;  // float4 per row
  for (int idx = threadIdx.x; idx < n * C4; idx += blockDim.x) {
    const int j = idx / C4, c = idx % C4;
    const size_t src = (size_t)(start + (int64_t)j * prm.s) * D + c * 4;
    const float4 kv = ldg4(K + src), vv = ldg4(V + src);
    float* kd = Ks + (size_t)j * (D + 1) + c * 4;
    kd[0] = kv.x; kd[1] = kv.y; kd[2] = kv.z; kd[3] = kv.w;
    *reinterpret_cast<float4*>(Vs + (size_t)j * D + c * 4) = vv;
  }
  __syncthreads();

  // ---- live rows ----
  constexpr int DPL = (D + 31) / 32;  // output dims per lane
  for (int t = warp; t < n; t += kBlockWarps) {
    const int64_t i = start + (int64_t)t * prm.s;
    if (i < prm.row_begin || i >= prm.row_end) continue;  // warp-uniform
    const int64_t r = i - prm.row_begin;
    for (int e = lane; e < D; e += 32) qs[e] = __ldg(Q + (size_t)r * D + e);
    __syncwarp();
    float sc[NK];
#pragma unroll
    for (int k = 0; k < NK; ++k) sc[k] = 0.f;
    for (int e = 0; e < D; ++e) {
      const float qv = qs[e];
#pragma unroll
      for (int k = 0; k < NK; ++k) {
        const int j = lane + 32 * k;
        if (j < n) sc[k] = fmaf(qv, Ks[(size_t)j * (D + 1) + e], sc[k]);
      }
    }
    float mx = neg_inf();
#pragma unroll
    for (int k = 0; k < NK; ++k) {
      const int j = lane + 32 * k;
      sc[k] = (j < n) ? sc[k] * prm.scale : neg_inf();
      mx = fmaxf(mx, sc[k]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, o));
    float ls = 0.f;
#pragma unroll
    for (int k = 0; k < NK; ++k) {
      const int j = lane + 32 * k;
      if (j < npad) {
        const float p = (j < n) ? fast_exp2((sc[k] - mx) * kLog2e) : 0.f;
        ps[j] = p;
        ls += p;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(kFullMask, ls, o);
    __syncwarp();
    float acc[DPL];
#pragma unroll
    for (int k = 0; k < DPL; ++k) acc[k] = 0.f;
    for (int j = 0; j < n; ++j) {
      const float p = ps[j];
#pragma unroll
      for (int k = 0; k < DPL; ++k) {
        const int e = lane + 32 * k;
        if (e < D) acc[k] = fmaf(p, Vs[(size_t)j * D + e], acc[k]);
      }
    }
    // merge with the caller's state (same recurrence as store_row of the gather path)
    const float m_in = m[r], l_in = l[r];
    const float m_o = fmaxf(m_in, mx);
    const float a = l_in * fast_exp2((m_in - m_o) * kLog2e);
    const float b = fast_exp2((mx - m_o) * kLog2e);
    const float l_o = fmaf(ls, b, a);
    const float inv = 1.0f / l_o;
#pragma unroll
    for (int k = 0; k < DPL; ++k) {
      const int e = lane + 32 * k;
      if (e < D) {
        float* op = O + (size_t)r * D + e;
        *op = (a * *op + b * acc[k]) * inv;
      }
    }
    __syncwarp();
    if (lane == 0) {
      m[r] = m_o;
      l[r] = l_o;
    }
  }

  // ---- dead rows: NaN fill (32-bit index arithmetic: B < 2^31; one modulo per row, RPI rows per warp store) ----
  if (prm.use_nan && prm.s > 1) {
    const float nn = __int_as_float(0x7fc00000);
    const float4 nan4 = make_float4(nn, nn, nn, nn);
    constexpr int RPI = (C4 >= 32) ? 1 : 32 / C4;  // rows covered by one warp-wide float4 store
    const int B = (int)prm.B, s32 = (int)prm.s;
    for (int r_base = warp * RPI; r_base < B; r_base += kBlockWarps * RPI) {
      const int rr = r_base + lane / C4;
      const int64_t i = start + rr;
      if (rr >= B || rr % s32 == 0 || i < prm.row_begin || i >= prm.row_end) continue;
      float4* row = reinterpret_cast<float4*>(O + (size_t)(i - prm.row_begin) * D);
      for (int c = lane % C4; c < C4; c += 32) row[c] = nan4;
    }
  }
}

}  // namespace spfa
