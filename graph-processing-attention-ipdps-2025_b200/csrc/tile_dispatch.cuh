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
#include "tile_kernels_sm100.cuh"

namespace spfa {

constexpr int SPFA_TILE_NOT_TAKEN = 1;
constexpr int64_t kTileMinHalfWidth = 32;  // AUTO: narrower bands stay on the exact FP32 gather path
constexpr int64_t kTileMaxStride = 16;

extern std::atomic<int64_t> g_launches;

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
inline bool make_row_map(CUtensorMap* tm, const float* base, int d, int64_t rows, int64_t pitch_bytes, int box_rows,
                         bool mn_major = false) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
  cuuint32_t box[2] = {32u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, int BN, int NS, int NSUB>
int launch_band(const float* Q, const float* K, const float* V, float* m, float* l, float* O, int64_t L, int64_t w,
                int64_t s, int64_t row_begin, int64_t row_end, cudaStream_t st) {
  using P = tile::Plan<D, BN, NS, NSUB>;
  using G = tile::Geo<NSUB>;
  auto kern = tile::band_forward_kernel<D, BN, NS, NSUB>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P::kDynSmem) != cudaSuccess)
    return SPFA_ERR_LAUNCH;
  // ask for the largest shared-memory carve-out so that kCtasPerSm CTAs are co-resident
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (const char* dbg = getenv("SPFA_DEBUG_OCCUPANCY")) {
    int nb = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, G::kThreads, P::kDynSmem);
    cudaFuncAttributes fa;
    cudaFuncGetAttributes(&fa, kern);
    int nb_small = 0, smem_sm = 0, regs_sm = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb_small, kern, G::kThreads, 1024);
    cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, 0);
    cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, 0);
    fprintf(stderr, "spfa: band kernel D=%d BN=%d NS=%d NSUB=%d dyn smem=%d B static=%d B regs=%d threads=%d -> %d CTA/SM "
            "(%d with 1 KB smem); SM has %d B smem, %d regs (%s)\n", D, BN, NS, NSUB, (int)P::kDynSmem,
            (int)fa.sharedSizeBytes, fa.numRegs, G::kThreads, nb, nb_small, smem_sm, regs_sm, dbg);
  }
  // The kernel re-balances registers with setmaxnreg, which blocks without timeout if the budgets exceed
  // what the launch allocated: refuse to launch unless the compiled register count covers them.
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, kern) != cudaSuccess) return SPFA_ERR_LAUNCH;
  if (attr.numRegs * G::kThreads < G::kRegsSoftmax * 128 * NSUB + G::kRegsAux * 128) return SPFA_ERR_LAUNCH;
  int* err = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&err), g_tile_error) != cudaSuccess) return SPFA_ERR_LAUNCH;
  for (int64_t r = 0; r < s && r < L; ++r) {
    tile::BandParams prm;
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
    CUtensorMap tmQ, tmK, tmV;
    const int64_t pitch = s * D * (int64_t)sizeof(float);
    if (!make_row_map(&tmQ, Q + (r + u_first * s - row_begin) * D, D, prm.n_q, pitch, 128) ||
        !make_row_map(&tmK, K + r * D, D, prm.n_keys, pitch, BN) || !make_row_map(&tmV, V + r * D, D, prm.n_keys, pitch, BN, /*mn_major=*/true))
      return SPFA_ERR_LAUNCH;
    const int64_t grid = (prm.n_q + G::kQRows - 1) / G::kQRows;
    if (grid > 0x7fffffffLL) return SPFA_ERR_TOO_LARGE;
    kern<<<(unsigned)grid, G::kThreads, P::kDynSmem, st>>>(tmQ, tmK, tmV, m, l, O, prm, err);
    g_launches.fetch_add(1);
    if (cudaGetLastError() != cudaSuccess) return SPFA_ERR_LAUNCH;
  }
  return SPFA_OK;
}

// Band |u_q - u_k| <= w on every residue class of stride s (s = 1: Local; s = dil+1: Local-1D-dilated).
inline int tiled_band_forward(const float* Q, const float* K, const float* V, float* m, float* l, float* O, int64_t L,
                              int d, int64_t w, int64_t s, int64_t row_begin, int64_t row_end, bool forced,
                              cudaStream_t st) {
  const bool shape_ok = (d == 32 || d == 64 || d == 128) && s >= 1 && s <= kTileMaxStride && row_end > row_begin;
  if (!shape_ok) return forced ? (int)SPFA_ERR_BAD_ARG : SPFA_TILE_NOT_TAKEN;
  if (!forced && w < kTileMinHalfWidth) return SPFA_TILE_NOT_TAKEN;
  switch (d) {
    case 32: return launch_band<32, 96, 2, 2>(Q, K, V, m, l, O, L, w, s, row_begin, row_end, st);
    case 64: return launch_band<64, 96, 2, 2>(Q, K, V, m, l, O, L, w, s, row_begin, row_end, st);
    case 128: return launch_band<128, 64, 1, 2>(Q, K, V, m, l, O, L, w, s, row_begin, row_end, st);
  }
  return SPFA_TILE_NOT_TAKEN;
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
