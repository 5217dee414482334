// C ABI, 16-bit storage (float16 / bfloat16 Q, K, V, m, l, O): the native gather path for all six mask families.
// Declared in include/spfa_b200.h under "16-bit tensors". Arithmetic is fp32; only loads and stores are 16-bit.
#include <cmath>

#include "capi_common.cuh"
#include "gather_generic.cuh"
#include "gather_kernels.cuh"
#include "gather_kernels_16.cuh"

namespace spfa {

template <int D, class T, class Cols>
int launch_gather16(const T* Q, const T* K, const T* V, T* m, T* l, T* O, const Cols& cols, int64_t row_begin,
                    int64_t n_rows, int use_nan, cudaStream_t st) {
  const int64_t blocks = (n_rows + kRowWarps - 1) / kRowWarps;
  if (blocks > 0x7fffffffLL) return SPFA_ERR_TOO_LARGE;
  gather_rows16_kernel<D, T, Cols><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(Q, K, V, m, l, O, cols, row_begin, n_rows,
                                                                                use_nan, 1.0f / sqrtf((float)D));
  g_launches.fetch_add(1);
  return launch_status();
}

template <class T, int VW, int NC, class Cols>
int launch_generic16(const T* Q, const T* K, const T* V, T* m, T* l, T* O, const Cols& cols, int64_t row_begin,
                     int64_t n_rows, int use_nan, int d, cudaStream_t st) {
  const int64_t blocks = (n_rows + kRowWarps - 1) / kRowWarps;
  if (blocks > 0x7fffffffLL) return SPFA_ERR_TOO_LARGE;
  gather_rows_generic_kernel<T, VW, NC, Cols><<<(unsigned)blocks, kRowWarps * 32, (size_t)kRowWarps * d * sizeof(float), st>>>(
      Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, 1.0f / sqrtf((float)d), d);
  g_launches.fetch_add(1);
  return launch_status();
}

// d in {32, 64, 128}: the specialised kernel; other multiples of 8: 128-bit pieces; anything else: scalar pieces.
template <class T, class Cols>
int dispatch16(int d, const T* Q, const T* K, const T* V, T* m, T* l, T* O, const Cols& cols, int64_t row_begin,
               int64_t n_rows, int use_nan, cudaStream_t st) {
  if (n_rows <= 0) return SPFA_OK;
  g_last_path.store(SPFA_PATH_GATHER);
  switch (d) {
    case 32: return launch_gather16<32, T, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st);
    case 64: return launch_gather16<64, T, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st);
    case 128: return launch_gather16<128, T, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, st);
  }
  if (d % 8 == 0) return launch_generic16<T, 8, 4, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, d, st);
  return launch_generic16<T, 1, 32, Cols>(Q, K, V, m, l, O, cols, row_begin, n_rows, use_nan, d, st);
}

inline int check_common16(const void* Q, const void* K, const void* V, const void* m, const void* l, const void* O, int d) {
  if (d < 1 || d > kGenericMaxD) return SPFA_ERR_EMBED_DIM;
  if (!Q || !K || !V || !m || !l || !O) return SPFA_ERR_BAD_ARG;
  if (d % 8 == 0) {  // rows are read and written in 128-bit pieces
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return SPFA_ERR_BAD_ARG;
  } else if (!aligned2(Q) || !aligned2(K) || !aligned2(V) || !aligned2(O)) {
    return SPFA_ERR_BAD_ARG;
  }
  return SPFA_OK;
}

// f(T*) with T = __half or __nv_bfloat16 according to the ABI's dtype code.
template <class F>
int with_dtype16(int dtype, F&& f) {
  if (dtype == SPFA_DTYPE_F16) return f(static_cast<__half*>(nullptr));
  if (dtype == SPFA_DTYPE_BF16) return f(static_cast<__nv_bfloat16*>(nullptr));
  return SPFA_ERR_BAD_ARG;
}

}  // namespace spfa

using namespace spfa;

extern "C" {

int spfa_csr_forward_16(int dtype, const void* Q, const void* K, const void* V, const uint64_t* row_off,
                        const uint32_t* col_ind, int64_t nnz, void* m, void* l, void* O, int64_t n_rows, int64_t Lk, int d,
                        int use_nan, void* stream) {
  int rc = check_common16(Q, K, V, m, l, O, d);
  if (rc) return rc;
  if (!row_off || n_rows < 0 || nnz < 0 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (n_rows == 0) return SPFA_OK;
  if (!col_ind) return SPFA_ERR_BAD_ARG;
  return with_dtype16(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    CsrCols cols{row_off, col_ind, Lk};
    return dispatch16<T>(d, (const T*)Q, (const T*)K, (const T*)V, (T*)m, (T*)l, (T*)O, cols, 0, n_rows, use_nan,
                         (cudaStream_t)stream);
  });
}

int spfa_coo_forward_16(int dtype, const void* Q, const void* K, const void* V, const uint64_t* row_ind,
                        const uint32_t* col_ind, int64_t nnz, void* m, void* l, void* O, int64_t row_begin, int64_t n_rows,
                        int64_t Lk, int d, int use_nan, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common16(Q, K, V, m, l, O, d);
  if (rc) return rc;
  if (nnz < 0 || n_rows < 0 || row_begin < 0 || Lk <= 0 || Lk >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  if (nnz > 0 && (!row_ind || !col_ind)) return SPFA_ERR_BAD_ARG;
  if (n_rows == 0) return SPFA_OK;
  rc = check_workspace(workspace, workspace_bytes, spfa_coo_min_workspace_bytes(n_rows));
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  uint64_t* ptr = reinterpret_cast<uint64_t*>(workspace);
  constexpr int64_t span = (int64_t)kRowPtrThreads * kRowPtrUnroll;
  int64_t blocks = (nnz + 1 + span - 1) / span;
  if (blocks > 148 * 32) blocks = 148 * 32;
  coo_row_pointers_kernel<uint64_t><<<(unsigned)blocks, kRowPtrThreads, 0, st>>>(row_ind, nnz, row_begin, n_rows, ptr);
  g_launches.fetch_add(1);
  if (launch_status() != SPFA_OK) return SPFA_ERR_LAUNCH;
  return with_dtype16(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    CsrCols cols{ptr, col_ind, Lk};
    return dispatch16<T>(d, (const T*)Q, (const T*)K, (const T*)V, (T*)m, (T*)l, (T*)O, cols, row_begin, n_rows, use_nan, st);
  });
}

int spfa_local_forward_16(int dtype, const void* Q, const void* K, const void* V, void* m, void* l, void* O, int64_t L,
                          int d, int64_t w, int64_t row_begin, int64_t row_end, void* stream) {
  int rc = check_common16(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (w < 0 || w > L - 1) return SPFA_ERR_LOCAL_SIZE;
  return with_dtype16(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    LocalCols cols{L, w};
    return dispatch16<T>(d, (const T*)Q, (const T*)K, (const T*)V, (T*)m, (T*)l, (T*)O, cols, row_begin,
                         row_end - row_begin, 0, (cudaStream_t)stream);
  });
}

int spfa_local_1d_dilated_forward_16(int dtype, const void* Q, const void* K, const void* V, void* m, void* l, void* O,
                                     int64_t L, int d, int64_t w, int64_t dil, int64_t row_begin, int64_t row_end,
                                     void* stream) {
  int rc = check_common16(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (w < 0 || w > L - 1) return SPFA_ERR_LOCAL_SIZE;
  if (dil < 0) return SPFA_ERR_DILATION_NEG;
  if (dil >= (1LL << 31)) return SPFA_ERR_BAD_ARG;
  return with_dtype16(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    Local1dCols cols{L, w, dil + 1};
    return dispatch16<T>(d, (const T*)Q, (const T*)K, (const T*)V, (T*)m, (T*)l, (T*)O, cols, row_begin,
                         row_end - row_begin, 0, (cudaStream_t)stream);
  });
}

int spfa_local_2d_dilated_forward_16(int dtype, const void* Q, const void* K, const void* V, void* m, void* l, void* O,
                                     int64_t L, int d, int64_t B, int64_t dil, int use_nan, int64_t row_begin,
                                     int64_t row_end, void* stream) {
  int rc = check_common16(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (B <= 0 || L % B != 0) return SPFA_ERR_BLOCK_DIVISOR;
  if (dil < 0) return SPFA_ERR_DILATION_NEG;
  if (dil >= (1LL << 31) || B / (dil + 1) < 1) return SPFA_ERR_DILATION_BLOCK;
  return with_dtype16(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    Local2dCols cols{L, B, dil + 1};
    return dispatch16<T>(d, (const T*)Q, (const T*)K, (const T*)V, (T*)m, (T*)l, (T*)O, cols, row_begin,
                         row_end - row_begin, use_nan, (cudaStream_t)stream);
  });
}

size_t spfa_global_no_local_workspace_bytes_16(int64_t L, int64_t n_global) {
  if (L <= 0 || n_global <= 0) return 0;
  return align_up((size_t)((L + 31) / 32) * 4) + align_up((size_t)n_global);
}

int spfa_global_no_local_forward_16(int dtype, const void* Q, const void* K, const void* V, void* m, void* l, void* O,
                                    const int32_t* G, int64_t nG, int64_t L, int d, int64_t w, int64_t row_begin,
                                    int64_t row_end, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common16(Q, K, V, m, l, O, d);
  if (rc) return rc;
  rc = check_rows(L, row_begin, row_end);
  if (rc) return rc;
  if (nG == 0 || nG > L || nG < 0) return SPFA_ERR_GLOBAL_COUNT;
  if (w < 0 || w > L - 1) return SPFA_ERR_LOCAL_SIZE;
  if (!G) return SPFA_ERR_BAD_ARG;
  rc = check_workspace(workspace, workspace_bytes, spfa_global_no_local_workspace_bytes_16(L, nG));
  if (rc) return rc;
  if (row_end == row_begin) return SPFA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* bits = reinterpret_cast<uint32_t*>(workspace);
  uint8_t* live = reinterpret_cast<uint8_t*>(static_cast<char*>(workspace) + align_up((size_t)((L + 31) / 32) * 4));
  if (cudaMemsetAsync(bits, 0, (size_t)((L + 31) / 32) * 4, st) != cudaSuccess) return SPFA_ERR_LAUNCH;
  gnl_mark_globals_kernel<<<(unsigned)((nG + 255) / 256), 256, 0, st>>>(G, nG, L, bits, live);
  g_launches.fetch_add(1);
  if (launch_status() != SPFA_OK) return SPFA_ERR_LAUNCH;
  return with_dtype16(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    GnlAnyRowCols any;  // a listed row is a long row walked by its whole CTA
    any.list = GnlCols{G, nG, L, w, bits};
    any.strip = GnlGlobalRowCols{L, w};
    return dispatch16<T>(d, (const T*)Q, (const T*)K, (const T*)V, (T*)m, (T*)l, (T*)O, any, row_begin, row_end - row_begin,
                         0, st);
  });
}

}  // extern "C"
