// Pieces shared by the translation units of the C ABI: launch counter, per-thread path selector, argument checks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/spfa_b200.h"

namespace spfa {

extern std::atomic<int64_t> g_launches;
// Path selector and "path taken" record are per host thread: two threads that force different paths (tests,
// benchmarks) do not see each other's choice, so the forward entry points stay re-entrant.
struct PathCell {
  int v;
  int load() const { return v; }
  void store(int x) { v = x; }
};
extern thread_local PathCell g_path;
extern thread_local PathCell g_last_path;

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }
inline bool aligned2(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 1u) == 0; }

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? SPFA_OK : SPFA_ERR_LAUNCH; }

inline int check_rows(int64_t L, int64_t row_begin, int64_t row_end) {
  if (L <= 0 || L >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (row_begin < 0 || row_end < row_begin || row_end > L) return SPFA_ERR_BAD_ARG;
  return SPFA_OK;
}

inline int check_workspace(const void* ws, size_t have, size_t need) {
  if (need == 0) return SPFA_OK;
  if (!ws || have < need || (reinterpret_cast<uintptr_t>(ws) & 255u)) return SPFA_ERR_WORKSPACE;
  return SPFA_OK;
}

}  // namespace spfa
