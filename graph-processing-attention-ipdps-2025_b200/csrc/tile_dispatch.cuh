// Entry to the tiled tensor-core path for banded masks (Local, and Local-1D-dilated as a band on each
// residue class). Returns SPFA_TILE_NOT_TAKEN when the shape should go to the gather path instead.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/spfa_b200.h"

namespace spfa {

constexpr int SPFA_TILE_NOT_TAKEN = 1;

inline int tiled_band_forward(const float*, const float*, const float*, float*, float*, float*, int64_t, int, int64_t,
                              int64_t, int64_t, int64_t, bool forced, cudaStream_t) {
  return forced ? (int)SPFA_ERR_BAD_ARG : SPFA_TILE_NOT_TAKEN;
}

}  // namespace spfa
