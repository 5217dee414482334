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


// ---- register-tiled variant for blocks with at most 64 keys per live row --------------------------------------
// The kernel above reads one shared-memory operand per FMA, which makes the shared-memory pipe its limit. Here a
// block is a 64 x 64 (padded) dense problem computed as 4 x 4 register tiles: thread (ig, jg) of 16 x 16 owns
// score rows 4 ig + a and keys jg + 16 b, so one 128-bit shared-memory load feeds 16 FMAs, the q loads of a warp
// are broadcasts (two row groups per warp) and the k loads fall on distinct bank groups (row pitch D + 4 floats).
// The live rows and the key rows of a block are the SAME rows (start + t s, t < n), so Q, K and V rows are staged
// together with 16-byte cp.async copies, all in flight at once; dead rows are NaN-filled while the copies travel.
// P goes through shared memory (over the dead Q tile) for the P V product, which is tiled the same way
// (thread = 4 rows x D/16 output dims). Exact FP32 like the kernel above.
constexpr int kTile2dThreads = 256;
constexpr int kTile2dMaxKeys = 64;
constexpr int kTile2dMinKeys = 32;  // blocks with fewer keys keep the kernel above (little padding there)

template <int D>
__host__ __device__ constexpr size_t tile2d_smem_bytes() {
  constexpr int PQ = D + 4;
  constexpr int region_a = (64 * PQ > 64 * 68) ? 64 * PQ : 64 * 68;  // Q tile, later P (pitch 68)
  return (size_t)(region_a + 64 * PQ + 64 * D) * sizeof(float);
}

// Two fp32 FMAs in one instruction (sm_100: fma.rn.f32x2 on 64-bit register pairs): d = a * b + c, lane-wise.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long ra, rb, rc, rd;
  float2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}

template <int D>
__global__ void __launch_bounds__(kTile2dThreads, (D <= 64) ? 3 : 2)
local2d_tile_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                    float* __restrict__ m, float* __restrict__ l, float* __restrict__ O, const Block2dParams prm) {
  constexpr int PQ = D + 4, PP = 68, C4 = D / 4, DV = D / 16;
  extern __shared__ __align__(16) float smem_t[];
  constexpr int region_a = (64 * PQ > 64 * PP) ? 64 * PQ : 64 * PP;
  float* Qs = smem_t;             // [64][PQ]; reused as P [64][PP] after the scores
  float* Ks = Qs + region_a;      // [64][PQ]
  float* Vs = Ks + 64 * PQ;       // [64][D]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = (int)prm.n;
  const int64_t start = (prm.first_block + blockIdx.x) * prm.B;

  // ---- stage rows start + t s (t < n) of Q, K, V; rows t >= n are zero ----
  for (int idx = tid; idx < 64 * C4; idx += kTile2dThreads) {
    const int t = idx / C4, c = idx % C4;
    float* qd = Qs + t * PQ + c * 4;
    float* kd = Ks + t * PQ + c * 4;
    float* vd = Vs + t * D + c * 4;
    if (t < n) {
      const int64_t i = start + (int64_t)t * prm.s;
      const size_t src = (size_t)i * D + c * 4;
      cp_async16(kd, K + src);
      cp_async16(vd, V + src);
      if (i >= prm.row_begin && i < prm.row_end) {
        cp_async16(qd, Q + (size_t)(i - prm.row_begin) * D + c * 4);
      } else {
        *reinterpret_cast<float4*>(qd) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(qd) = z;
      *reinterpret_cast<float4*>(kd) = z;
      *reinterpret_cast<float4*>(vd) = z;
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  // the caller's state rows are needed only at the end: ask L2 for them now
  if (tid < n) {
    const int64_t i = start + (int64_t)tid * prm.s;
    if (i >= prm.row_begin && i < prm.row_end) {
      const int64_t r = i - prm.row_begin;
      const char* orow = reinterpret_cast<const char*>(O + (size_t)r * D);
#pragma unroll
      for (int b = 0; b < D * 4; b += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(orow + b));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(m + r));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(l + r));
    }
  }

  // ---- dead rows: NaN fill while the copies are in flight ----
  if (prm.use_nan && prm.s > 1) {  // the s - 1 rows behind every live row t (fewer behind the last one)
    const float nn = __int_as_float(0x7fc00000);
    const float4 nan4 = make_float4(nn, nn, nn, nn);
    constexpr int RPI = (C4 >= 32) ? 1 : 32 / C4;  // rows covered by one warp-wide float4 store
    const int B = (int)prm.B, s32 = (int)prm.s;
    for (int t = warp; t < n; t += kTile2dThreads / 32) {
      const int live = t * s32;
      for (int k = 1 + lane / C4; k < s32 && live + k < B; k += RPI) {
        const int64_t i = start + live + k;
        if (i < prm.row_begin || i >= prm.row_end) continue;
        float4* row = reinterpret_cast<float4*>(O + (size_t)(i - prm.row_begin) * D);
        for (int c = lane % C4; c < C4; c += 32) row[c] = nan4;
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // ---- scores: rows 4 ig + a, keys jg + 16 b ----
  const int ig = tid >> 4, jg = tid & 15;
  const bool warp_live = 8 * warp < n;  // a warp owns rows 8 warp .. 8 warp + 7: beyond n there is nothing to compute
  float acc[4][4];
  {
    // even and odd elements of the dot products accumulate side by side (one f32x2 FMA per element pair)
    float2 acc2[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc2[a][b] = make_float2(0.f, 0.f);
    if (warp_live) {
#pragma unroll 2
      for (int e4 = 0; e4 < C4; ++e4) {
        float4 qa[4], kb[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) qa[a] = *reinterpret_cast<const float4*>(Qs + (4 * ig + a) * PQ + 4 * e4);
#pragma unroll
        for (int b = 0; b < 4; ++b) kb[b] = *reinterpret_cast<const float4*>(Ks + (jg + 16 * b) * PQ + 4 * e4);
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            acc2[a][b] = ffma2(make_float2(qa[a].x, qa[a].y), make_float2(kb[b].x, kb[b].y), acc2[a][b]);
            acc2[a][b] = ffma2(make_float2(qa[a].z, qa[a].w), make_float2(kb[b].z, kb[b].w), acc2[a][b]);
          }
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = acc2[a][b].x + acc2[a][b].y;
  }
  // ---- softmax over the row's n keys: 4 local keys, then the 16 lanes that share the row group ----
  float mx[4], ls[4];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    float v = neg_inf();
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      acc[a][b] = (jg + 16 * b < n) ? acc[a][b] * prm.scale : neg_inf();
      v = fmaxf(v, acc[a][b]);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
    mx[a] = v;  // finite: every live row has n >= 1 keys
    float sum = 0.f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      acc[a][b] = (jg + 16 * b < n) ? fast_exp2((acc[a][b] - v) * kLog2e) : 0.f;
      sum += acc[a][b];
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(kFullMask, sum, o);
    ls[a] = sum;
  }
  __syncthreads();  // every warp is done reading the Q tile: P may overwrite it
  float* Pm = Qs;
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) Pm[(4 * ig + a) * PP + jg + 16 * b] = acc[a][b];
  __syncthreads();

  // ---- P V: rows 4 ig + a, output dims dg DV .. dg DV + DV - 1 ----
  const int dg = jg;
  float o[4][DV];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int x = 0; x < DV; ++x) o[a][x] = 0.f;
  const int n4 = warp_live ? (n + 3) / 4 : 0;  // keys beyond n carry probability 0 and zero V rows
#pragma unroll 2
  for (int j4 = 0; j4 < n4; ++j4) {
    float4 pa[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) pa[a] = *reinterpret_cast<const float4*>(Pm + (4 * ig + a) * PP + 4 * j4);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      float vb[DV];
      const float* vrow = Vs + (4 * j4 + b) * D + dg * DV;
      if (DV % 4 == 0) {
#pragma unroll
        for (int x = 0; x < DV; x += 4) {
          const float4 t = *reinterpret_cast<const float4*>(vrow + x);
          vb[x] = t.x;
          vb[(x + 1) % DV] = t.y;
          vb[(x + 2) % DV] = t.z;
          vb[(x + 3) % DV] = t.w;
        }
      } else {
#pragma unroll
        for (int x = 0; x < DV; ++x) vb[x] = vrow[x];
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float p = (b == 0) ? pa[a].x : (b == 1) ? pa[a].y : (b == 2) ? pa[a].z : pa[a].w;
        if (DV % 2 == 0) {  // pairs of output dims per f32x2 FMA
          const float2 pp = make_float2(p, p);
#pragma unroll
          for (int x = 0; x < DV; x += 2) {
            const float2 r = ffma2(pp, make_float2(vb[x], vb[(x + 1) % DV]), make_float2(o[a][x], o[a][(x + 1) % DV]));
            o[a][x] = r.x;
            o[a][(x + 1) % DV] = r.y;
          }
        } else {
#pragma unroll
          for (int x = 0; x < DV; ++x) o[a][x] = fmaf(p, vb[x], o[a][x]);
        }
      }
    }
  }

  // ---- merge with the caller's state (same recurrence as store_row of the gather path) and store: the loads of
  //      all four rows are issued before any of them is used ----
  bool mine[4];
  float m_in[4], l_in[4];
  float4 oin[4][(DV + 3) / 4];
  float* op[4];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int t = 4 * ig + a;
    const int64_t i = start + (int64_t)t * prm.s;
    mine[a] = t < n && i >= prm.row_begin && i < prm.row_end;  // uniform over the 16 lanes of the row group
    const int64_t r = mine[a] ? (i - prm.row_begin) : 0;
    op[a] = O + (size_t)r * D + dg * DV;
    m_in[a] = mine[a] ? m[r] : 0.f;
    l_in[a] = mine[a] ? l[r] : 0.f;
    if (DV % 4 == 0) {
#pragma unroll
      for (int x = 0; x < DV / 4; ++x)
        oin[a][x] = mine[a] ? *reinterpret_cast<const float4*>(op[a] + 4 * x) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    if (!mine[a]) continue;
    const int64_t r = start + (int64_t)(4 * ig + a) * prm.s - prm.row_begin;
    const float m_o = fmaxf(m_in[a], mx[a]);
    const float ca = l_in[a] * fast_exp2((m_in[a] - m_o) * kLog2e);
    const float cb = fast_exp2((mx[a] - m_o) * kLog2e);
    const float l_o = fmaf(ls[a], cb, ca);
    const float inv = 1.0f / l_o;
    if (DV % 4 == 0) {
#pragma unroll
      for (int x = 0; x < DV / 4; ++x) {
        float4 t = oin[a][x];
        t.x = (ca * t.x + cb * o[a][(4 * x) % DV]) * inv;
        t.y = (ca * t.y + cb * o[a][(4 * x + 1) % DV]) * inv;
        t.z = (ca * t.z + cb * o[a][(4 * x + 2) % DV]) * inv;
        t.w = (ca * t.w + cb * o[a][(4 * x + 3) % DV]) * inv;
        *reinterpret_cast<float4*>(op[a] + 4 * x) = t;
      }
    } else {
#pragma unroll
      for (int x = 0; x < DV; ++x) op[a][x] = (ca * op[a][x] + cb * o[a][x]) * inv;
    }
    if (dg == 0) {
      m[r] = m_o;
      l[r] = l_o;
    }
  }
}

}  // namespace spfa
