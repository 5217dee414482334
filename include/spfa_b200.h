/*
 * spfa_b200.h -- C ABI of the B200 (sm_100a) sparse FlashAttention forward library.
 *
 * One entry point per attention-mask family of KLab-AI3/Graph-Processing-Attention-IPDPS-2025.
 * Each replaces the host dispatch function + CUDA kernel of one reference folder; the reference
 * interface every function stands in for is cited beside it (paths relative to the reference tree).
 *
 * Conventions shared by all entry points
 *   - All pointers are DEVICE pointers on the current CUDA device. Nothing is allocated or freed
 *     by the library: scratch memory comes in through (workspace, workspace_bytes).
 *   - Q, K, V, O are row-major [rows, d] float32; m, l are float32 vectors. K and V hold all
 *     Lk key rows. Q, m, l, O address ONLY the query rows this call works on: element 0 is the
 *     first row of the shard (absolute row `row_begin` for the implicit masks). A single-GPU
 *     caller passes the full tensors with row_begin = 0, row_end = L.
 *   - (m, l, O) are read-modify-write softmax state, exactly as in the reference
 *     (Sparse_FlashAttention_CSR/sp_flatt_csr_kernel.cu:79-92 load, :208-218 store):
 *       m_out = max(m_in, max_j s_ij)               s_ij = q_i . k_j / sqrt(d)
 *       l_out = l_in e^{m_in-m_out} + sum_j e^{s_ij-m_out}
 *       O_out = (l_in e^{m_in-m_out} O_in + sum_j e^{s_ij-m_out} v_j) / l_out
 *     Initial state is m = -inf, l = 0, O = 0. Rows whose key set is empty are left untouched
 *     (or O is NaN-filled where the family has a use_nan flag and it is non-zero).
 *   - `stream` is a cudaStream_t passed as void*. Calls are asynchronous; they return after
 *     enqueueing. The return value is SPFA_OK or a negative spfa_status.
 *   - d (the embedded dimension) may be anything from 1 to 1024, the range the reference's kernels work for
 *     (sp_flatt_csr_kernel.cu:183-184). d in {16, 32, 64, 128} has specialised kernels (and, from 32 on, the tensor-core
 *     path); every other d runs on a generic FP32 gather kernel. Q, K, V, O must be 16-byte aligned when d is a
 *     multiple of 4, 4-byte aligned otherwise.
 */
#ifndef SPFA_B200_H_
#define SPFA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum spfa_status {
  SPFA_OK = 0,
  SPFA_ERR_BAD_ARG = -1,        /* null pointer, negative size, row range outside [0, L] */
  SPFA_ERR_EMBED_DIM = -2,      /* d < 1 or d > 1024 (reference: "embedded dimension is too large", sp_flatt_csr_kernel.cu:264-266) */
  SPFA_ERR_WORKSPACE = -3,      /* workspace missing, misaligned (256 B) or smaller than *_workspace_bytes() */
  SPFA_ERR_LAUNCH = -4,         /* CUDA reported an error when enqueueing */
  SPFA_ERR_DEVICE_TIMEOUT = -5, /* a bounded device-side wait gave up (reported by spfa_last_device_error) */
  SPFA_ERR_LOCAL_SIZE = -6,     /* local_size_each_dir < 0 or > L-1 (sp_flatt_local_kernel.cu:252-254) */
  SPFA_ERR_DILATION_NEG = -7,   /* dil_factor < 0 (sp_flatt_local_1d_dilated_kernel.cu:259-261) */
  SPFA_ERR_BLOCK_DIVISOR = -8,  /* L % block_size != 0 (sp_flatt_local_2d_dilated_kernel.cu:274-276) */
  SPFA_ERR_DILATION_BLOCK = -9, /* block_size / (dil_factor+1) < 1 (sp_flatt_local_2d_dilated_kernel.cu:284-286) */
  SPFA_ERR_GLOBAL_COUNT = -10,  /* n_global == 0 or > L (sp_flatt_global_no_local_kernel.cu:325-327) */
  SPFA_ERR_TOO_LARGE = -11,     /* size beyond a stated fixed maximum */
  SPFA_ERR_REGISTER_BUDGET = -12 /* SPFA_PATH_TILED forced, but this build's tiled kernel got fewer registers than its
                                    setmaxnreg budgets need (AUTO falls back to the gather path instead) */
} spfa_status;

/* Human-readable text for a status code (static storage). */
const char* spfa_status_string(int status);

/* Library/ABI version: major*1000 + minor. */
int spfa_abi_version(void);

/* Execution path selector -- TEST AND BENCHMARK SUPPORT, not part of the drop-in surface (the reference has no
 * counterpart: each of its operators has one kernel).
 *   SPFA_PATH_AUTO   library picks (tiled tensor-core path when the window is wide enough or, for explicit
 *                    masks, when the mask is large and the workspace allows the dense-tile split; else gather)
 *   SPFA_PATH_GATHER FP32 warp-per-row gather path (max-abs error ~1e-6 vs fp64)
 *   SPFA_PATH_TILED  tcgen05 TF32 tiled path (max-abs error <= 2e-3 vs fp64); falls back to
 *                    SPFA_ERR_BAD_ARG if the shape is not supported by that path
 * The selector and the record of the path taken are PER HOST THREAD (thread-local, default AUTO): a thread that
 * never calls spfa_set_path always gets AUTO, and threads forcing different paths do not interfere, so the forward
 * entry points stay stateless and re-entrant for production callers. */
enum { SPFA_PATH_AUTO = 0, SPFA_PATH_GATHER = 1, SPFA_PATH_TILED = 2 };
void spfa_set_path(int path);
int spfa_get_path(void);
/* Path the most recent forward call of the calling thread actually took (SPFA_PATH_GATHER or SPFA_PATH_TILED). */
int spfa_last_path(void);

/* ---- explicit CSR mask ------------------------------------------------------------------------
 * Replaces spfa_csr_cuda_forward + spfa_csr_cuda_forward_kernel
 * (Sparse_FlashAttention_CSR/sp_flatt_csr_kernel.cu:224-288, :14-220).
 * Row r of the shard attends to K/V rows col_ind[row_off[r] .. row_off[r+1]) in storage order.
 * row_off has n_rows+1 entries that index col_ind directly; nnz is the length of col_ind (every offset is
 * <= nnz). Column values >= Lk are skipped.
 * The reference's W_val argument is never read by the reference kernel and is not part of the ABI.
 *
 * Dense-tile split (north of ~1e6 entries under SPFA_PATH_AUTO, always under SPFA_PATH_TILED, d in
 * {32, 64, 128}): the rows are cut into 128-row blocks and the keys into tiles of 64 rows; a
 * (block, tile) pair holding at least 1/24 of its possible entries runs on the tcgen05 tiled kernel under a
 * bit mask (TF32 accuracy class), all other entries on the FP32 gather kernel. It is taken only if the
 * workspace is at least spfa_csr_workspace_bytes(); with a smaller (or no) workspace every entry takes the
 * gather path, which needs none. */
size_t spfa_csr_workspace_bytes(int64_t n_rows, int64_t nnz, int64_t Lk, int d);
int spfa_csr_forward_f32(const float* Q, const float* K, const float* V,
                         const uint64_t* row_off, const uint32_t* col_ind, int64_t nnz,
                         float* m, float* l, float* O,
                         int64_t n_rows, int64_t Lk, int d, int use_nan,
                         void* workspace, size_t workspace_bytes, void* stream);

/* ---- explicit COO mask ------------------------------------------------------------------------
 * Replaces spfa_coo_cuda_forward + spfa_coo_cuda_forward_kernel
 * (Sparse_FlashAttention_COO/sp_flatt_coo_kernel.cu:263-327, :14-259).
 * row_ind (ascending, absolute row numbers) / col_ind hold nnz entries that include every entry of
 * rows [row_begin, row_begin + n_rows); entries of other rows are ignored. The per-row linear scan
 * of the reference (:47-79) is replaced by one pass that writes n_rows+1 row pointers into the
 * workspace, followed by the CSR kernels (including the dense-tile split described above).
 * spfa_coo_workspace_bytes() is the size that allows the split when the shape qualifies; the minimum the
 * entry point accepts is spfa_coo_min_workspace_bytes() (the row pointers only: gather path). */
size_t spfa_coo_workspace_bytes(int64_t n_rows, int64_t nnz, int64_t Lk, int d);
size_t spfa_coo_min_workspace_bytes(int64_t n_rows);
int spfa_coo_forward_f32(const float* Q, const float* K, const float* V,
                         const uint64_t* row_ind, const uint32_t* col_ind, int64_t nnz,
                         float* m, float* l, float* O,
                         int64_t row_begin, int64_t n_rows, int64_t Lk, int d, int use_nan,
                         void* workspace, size_t workspace_bytes, void* stream);

/* ---- explicit masks with 32-bit row offsets / row indices ----------------------------------------------
 * No counterpart in the reference, whose row tensors are 64-bit (sp_flatt_csr_kernel.cu:19,275;
 * sp_flatt_coo_kernel.cu:19). Masks that are stored as int32 CSR / int32 COO (every index below 2^31) can be
 * passed as they are: the COO row-pointer pass then reads half the bytes (4 instead of 8 per mask entry), the CSR
 * offsets are widened into the workspace first (8 (n_rows + 1) bytes more than spfa_csr_workspace_bytes, also for
 * small masks). Everything else -- arguments, results, status codes -- is as in the 64-bit entry points. */
size_t spfa_csr_workspace_bytes_idx32(int64_t n_rows, int64_t nnz, int64_t Lk, int d);
int spfa_csr_forward_f32_idx32(const float* Q, const float* K, const float* V,
                               const int32_t* row_off, const uint32_t* col_ind, int64_t nnz,
                               float* m, float* l, float* O,
                               int64_t n_rows, int64_t Lk, int d, int use_nan,
                               void* workspace, size_t workspace_bytes, void* stream);
int spfa_coo_forward_f32_idx32(const float* Q, const float* K, const float* V,
                               const int32_t* row_ind, const uint32_t* col_ind, int64_t nnz,
                               float* m, float* l, float* O,
                               int64_t row_begin, int64_t n_rows, int64_t Lk, int d, int use_nan,
                               void* workspace, size_t workspace_bytes, void* stream);
int spfa_coo_plan_build_idx32(const int32_t* row_ind, const uint32_t* col_ind, int64_t nnz,
                              int64_t row_begin, int64_t n_rows, int64_t Lk, int d,
                              void* plan, size_t plan_bytes, void* stream);

/* ---- stored plans for explicit masks ---------------------------------------------------------------
 * No counterpart in the reference (its callers rebuild nothing between calls because its kernels inspect
 * nothing). The dense-tile split of a CSR/COO mask depends on the mask only, so a caller that applies one
 * mask many times (layers, heads, training steps) can run the inspector once:
 *
 *   bytes = spfa_explicit_plan_bytes(n_rows, nnz, Lk, d);           0: shape not supported by the split
 *   spfa_csr_plan_build(...) or spfa_coo_plan_build(...)            fills `plan` (device memory, 256-B aligned)
 *   spfa_planned_forward_f32(Q, K, V, m, l, O, ..., plan, bytes)    any number of times, any Q/K/V
 *
 * The plan holds everything the forward call needs of the mask (row offsets, residual column list, tile bit
 * masks); the mask arrays themselves may be freed after the build. n_rows, nnz, Lk and d must be the values
 * the plan was built with. The plan is read-only in spfa_planned_forward_f32, so concurrent calls may share it.
 * Same results as a one-shot call that takes the split (TF32 accuracy class for entries in dense tiles). */
size_t spfa_explicit_plan_bytes(int64_t n_rows, int64_t nnz, int64_t Lk, int d);
int spfa_csr_plan_build(const uint64_t* row_off, const uint32_t* col_ind, int64_t nnz,
                        int64_t n_rows, int64_t Lk, int d,
                        void* plan, size_t plan_bytes, void* stream);
int spfa_coo_plan_build(const uint64_t* row_ind, const uint32_t* col_ind, int64_t nnz,
                        int64_t row_begin, int64_t n_rows, int64_t Lk, int d,
                        void* plan, size_t plan_bytes, void* stream);
int spfa_planned_forward_f32(const float* Q, const float* K, const float* V,
                             float* m, float* l, float* O,
                             int64_t n_rows, int64_t nnz, int64_t Lk, int d, int use_nan,
                             const void* plan, size_t plan_bytes, void* stream);
/* A plan carries the (n_rows, nnz, Lk, d) it was built for. The kernels of spfa_planned_forward_f32 compare them
 * with the arguments of the call before they read any table of the plan; on a mismatch they compute nothing and
 * record code 401, which spfa_last_device_error() returns (the call itself has returned SPFA_OK by then: it is
 * asynchronous). A plan region smaller than spfa_explicit_plan_bytes() is refused at once (SPFA_ERR_WORKSPACE).
 *
 * The same forward restricted to the keys [key_begin, key_end): dense tiles and residual entries whose key lies in
 * the range are applied to (m, l, O), everything else is left for other calls. Calls over disjoint ranges that
 * cover [0, Lk), in any order on one stream, give the result of spfa_planned_forward_f32 (the passes chain through
 * the softmax state like any two calls on disjoint masks). It exists for multi-GPU callers that receive K and V
 * in chunks and want to compute on the chunks that have arrived: only K/V rows inside the range are read.
 * key_begin and key_end must be multiples of 64 (the key-tile size) or, for key_end, >= Lk (clipped to Lk).
 * key_begin > key_end names the cyclic range [key_begin, Lk) + [0, key_end): the complement of [key_end, key_begin),
 * which is what a rank holds after it has received the chunks on both sides of its own. use_nan NaN-fills the rows
 * without any mask entry and belongs on exactly one call of the series, before the others (the first one issued).
 * Residual rows are cut by binary search when every row of the mask stores its columns in ascending order
 * (recorded by the inspector); otherwise each pass walks all residual entries and skips the foreign ones. */
int spfa_planned_forward_keys_f32(const float* Q, const float* K, const float* V,
                                  float* m, float* l, float* O,
                                  int64_t n_rows, int64_t nnz, int64_t Lk, int d, int use_nan,
                                  const void* plan, size_t plan_bytes,
                                  int64_t key_begin, int64_t key_end, void* stream);
/* The same, for one part of the plan only: `parts` is SPFA_PLAN_DENSE_TILES, SPFA_PLAN_RESIDUAL or both. The dense
 * tiles of a banded graph read keys near the diagonal only, i.e. mostly the K/V chunk a rank owns, and their pass
 * costs nothing per row; the residual pass visits every row whatever the key range is. A multi-GPU caller therefore
 * runs the dense tiles of its own key chunk while the other chunks travel, then the dense tiles of the other keys and
 * the residual entries of all keys. No counterpart in the reference. */
enum spfa_plan_parts { SPFA_PLAN_DENSE_TILES = 1, SPFA_PLAN_RESIDUAL = 2 };
int spfa_planned_forward_parts_f32(const float* Q, const float* K, const float* V,
                                   float* m, float* l, float* O,
                                   int64_t n_rows, int64_t nnz, int64_t Lk, int d, int use_nan,
                                   const void* plan, size_t plan_bytes,
                                   int64_t key_begin, int64_t key_end, int parts, void* stream);

/* ---- explicit COO mask, allocation-free variant ---------------------------------------------------
 * No counterpart in the reference (its COO kernel needs no scratch because it re-scans the row array
 * for every row, sp_flatt_coo_kernel.cu:47-79).
 *
 * For callers that cannot hand this library a workspace because they are not allowed to allocate
 * device memory at the point of the call: for example a serving process that gave its whole device
 * budget to its own pool at start-up and forbids plug-ins from touching the CUDA allocator, or a
 * latency-critical section in which the implicit device-wide synchronisation of cudaMalloc/cudaFree
 * is not acceptable. Identical to spfa_coo_forward_f32 except that the n_rows+1 row pointers live in a
 * static device array inside the library (2 MiB per GPU that loads the library, held until exit).
 *
 *   - n_rows may not exceed spfa_coo_static_max_rows() (262144); larger shards return
 *     SPFA_ERR_TOO_LARGE and launch nothing. Shard the rows or use the workspace variant.
 *   - Neither this function nor anything it calls uses cudaMalloc, cudaFree or another allocating
 *     routine. The first call on a device resolves the array's device address
 *     (cudaGetSymbolAddress with that device current) and caches it; make that first call on each
 *     device during set-up, before any stream capture is begun. The cached address belongs to the device's
 *     primary context: it does not survive cudaDeviceReset(), after which this entry point must not be used.
 *   - All calls on a device share the one array. Its previous contents never matter (each call
 *     rewrites every entry it reads), but two calls whose kernels may overlap on the GPU -- different
 *     streams, or different host threads on different streams -- race on it: serialise them. */
int64_t spfa_coo_static_max_rows(void);
int spfa_coo_forward_f32_static(const float* Q, const float* K, const float* V,
                                const uint64_t* row_ind, const uint32_t* col_ind, int64_t nnz,
                                float* m, float* l, float* O,
                                int64_t row_begin, int64_t n_rows, int64_t Lk, int d, int use_nan,
                                void* stream);

/* ---- implicit Local (sliding window) mask -------------------------------------------------------
 * Replaces spfa_local_cuda_forward + kernel (Sparse_FlashAttention_Local/sp_flatt_local_kernel.cu:208-272, :12-204).
 * Row i attends to j in [max(0, i-w), min(L, i+w+1)).  (:24-28) */
size_t spfa_local_workspace_bytes(int64_t L, int64_t n_rows, int d);
int spfa_local_forward_f32(const float* Q, const float* K, const float* V,
                           float* m, float* l, float* O,
                           int64_t L, int d, int64_t local_size_each_dir,
                           int64_t row_begin, int64_t row_end,
                           void* workspace, size_t workspace_bytes, void* stream);

/* ---- implicit Local 1D dilated mask -------------------------------------------------------------
 * Replaces spfa_local_1d_dilated_cuda_forward + kernel
 * (Sparse_FlashAttention_Local_1D_Dilated/sp_flatt_local_1d_dilated_kernel.cu:209-280, :12-205).
 * s = dil_factor+1; lo = max(i - w s, i mod s); hi = min(i + w s, L-1); n = (hi-lo)/s + 1;
 * row i attends to lo + t s, 0 <= t < n.  (:25-29, :102) */
size_t spfa_local_1d_dilated_workspace_bytes(int64_t L, int64_t n_rows, int d);
int spfa_local_1d_dilated_forward_f32(const float* Q, const float* K, const float* V,
                                      float* m, float* l, float* O,
                                      int64_t L, int d, int64_t local_size_each_dir, int64_t dil_factor,
                                      int64_t row_begin, int64_t row_end,
                                      void* workspace, size_t workspace_bytes, void* stream);

/* ---- implicit Local 2D dilated (block-diagonal, intra-block dilation) mask -----------------------
 * Replaces spfa_local_2d_dilated_cuda_forward + kernel
 * (Sparse_FlashAttention_Local_2D_Dilated/sp_flatt_local_2d_dilated_kernel.cu:230-306, :12-226).
 * s = dil_factor+1; start = (i / B) B; rows with (i-start) mod s != 0 have no keys (NaN-filled O if
 * use_nan, else untouched); other rows attend to start + t s, 0 <= t < min(B, (B-1)/s + 1).  (:26-39, :123) */
size_t spfa_local_2d_dilated_workspace_bytes(int64_t L, int64_t n_rows, int d);
int spfa_local_2d_dilated_forward_f32(const float* Q, const float* K, const float* V,
                                      float* m, float* l, float* O,
                                      int64_t L, int d, int64_t block_size, int64_t dil_factor, int use_nan,
                                      int64_t row_begin, int64_t row_end,
                                      void* workspace, size_t workspace_bytes, void* stream);

/* ---- implicit Global-no-local mask --------------------------------------------------------------
 * Replaces spfa_global_no_local_cuda_forward + kernel
 * (Sparse_FlashAttention_Global_No_Local/sp_flatt_global_no_local_kernel.cu:280-353, :12-276).
 * W(i) = [max(0,i-w), min(L,i+w+1)). A row i listed in global_inds attends to every j outside W(i)
 * (:54-57, :135-145); any other row attends to the listed g outside W(i), in list order (:58-60, :146-162).
 * global_inds is int32[n_global]; entries outside [0, L) are ignored. Rows with no key are untouched. */
size_t spfa_global_no_local_workspace_bytes(int64_t L, int64_t n_rows, int d, int64_t n_global);
int spfa_global_no_local_forward_f32(const float* Q, const float* K, const float* V,
                                     float* m, float* l, float* O,
                                     const int32_t* global_inds, int64_t n_global,
                                     int64_t L, int d, int64_t local_size_each_dir,
                                     int64_t row_begin, int64_t row_end,
                                     void* workspace, size_t workspace_bytes, void* stream);

/* ---- batches of slices: batch x heads sharing one mask ------------------------------------------------------
 * No counterpart in the reference, which is "limited to ... single-headed, single-batched attention" (README.md:10).
 * n_slices independent attention problems share the mask and its parameters: Q, O are [n_slices, rows, d], K, V
 * [n_slices, Lk, d], m, l [n_slices, rows], contiguous (a [batch, heads, L, d] tensor viewed as [batch*heads, L, d]).
 * Local and Local-1D-dilated run every slice in ONE launch (the slice is a grid dimension of the tiled and of the
 * gather kernel: many short sequences fill the GPU that one of them would leave idle); CSR / COO inspect the mask
 * once (row pointers, dense-tile plan) and run every slice from the result, or take all slices in one gather launch;
 * Local-2D-dilated and Global-no-local run one call per slice on the stream. Other arguments, workspace sizes (of
 * ONE slice: scratch is reused in stream order) and results are those of the single-slice entry points. */
int spfa_local_forward_batched_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                   int64_t n_slices, int64_t L, int d, int64_t local_size_each_dir,
                                   int64_t row_begin, int64_t row_end, void* workspace, size_t workspace_bytes, void* stream);
int spfa_local_1d_dilated_forward_batched_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                              int64_t n_slices, int64_t L, int d, int64_t local_size_each_dir,
                                              int64_t dil_factor, int64_t row_begin, int64_t row_end,
                                              void* workspace, size_t workspace_bytes, void* stream);
int spfa_local_2d_dilated_forward_batched_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                              int64_t n_slices, int64_t L, int d, int64_t block_size, int64_t dil_factor,
                                              int use_nan, int64_t row_begin, int64_t row_end,
                                              void* workspace, size_t workspace_bytes, void* stream);
int spfa_global_no_local_forward_batched_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                                             int64_t n_slices, const int32_t* global_inds, int64_t n_global, int64_t L,
                                             int d, int64_t local_size_each_dir, int64_t row_begin, int64_t row_end,
                                             void* workspace, size_t workspace_bytes, void* stream);
int spfa_csr_forward_batched_f32(const float* Q, const float* K, const float* V,
                                 const uint64_t* row_off, const uint32_t* col_ind, int64_t nnz,
                                 float* m, float* l, float* O, int64_t n_slices,
                                 int64_t n_rows, int64_t Lk, int d, int use_nan,
                                 void* workspace, size_t workspace_bytes, void* stream);
int spfa_coo_forward_batched_f32(const float* Q, const float* K, const float* V,
                                 const uint64_t* row_ind, const uint32_t* col_ind, int64_t nnz,
                                 float* m, float* l, float* O, int64_t n_slices,
                                 int64_t row_begin, int64_t n_rows, int64_t Lk, int d, int use_nan,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* ---- fused union of masks: Local + Global-no-local + an explicit CSR part ("BigBird") ------------------------
 * No single counterpart in the reference, which composes this mask from three chained launches on one (m, l, O):
 * spfa_local.forward, spfa_global_no_local.forward, spfa_csr.forward (verification/verify.py:337-352). This entry
 * gives the same result -- the attention over
 *     { |i-j| <= w }  +  { i or j in global_inds, |i-j| > w }  +  { (i, col_ind[row_off[i-row_begin] ...]) }
 * with the caller keeping the CSR part disjoint from the other two, as the chained calls need it
 * (verify.py:328) -- with one read of Q and one read-modify-write of (m, l, O) for the band and the global keys
 * together instead of two: where the tiled kernel serves the shape (d in {32, 64, 128}, at most 1024 global tokens,
 * w >= 32 or SPFA_PATH_TILED), every row that is not global gets its band tiles and the gathered global-key tiles in
 * ONE kernel pass; the global rows (which attend to every key) run as a split strip; the CSR part follows on the
 * gather path (or its dense-tile split). Other shapes run the three operators one after the other internally.
 * row_off holds n_rows + 1 offsets into col_ind for the rows [row_begin, row_end); nnz = 0 leaves the CSR part out. */
size_t spfa_bigbird_workspace_bytes(int64_t L, int64_t n_rows, int d, int64_t n_global, int64_t nnz);
int spfa_bigbird_forward_f32(const float* Q, const float* K, const float* V, float* m, float* l, float* O,
                             const int32_t* global_inds, int64_t n_global,
                             const uint64_t* row_off, const uint32_t* col_ind, int64_t nnz,
                             int64_t L, int d, int64_t local_size_each_dir, int64_t row_begin, int64_t row_end,
                             void* workspace, size_t workspace_bytes, void* stream);

/* ---- 16-bit tensors: float16 / bfloat16 Q, K, V, m, l, O ------------------------------------------------------
 * The reference instantiates its kernels for Half too (AT_DISPATCH_FLOATING_TYPES_AND_HALF,
 * Sparse_FlashAttention_CSR/sp_flatt_csr_kernel.cu:270; all floating tensors of a call share one dtype). These entry
 * points read and write such tensors directly -- half the bytes of an fp32 call on the gather path, where HBM traffic
 * is the limit -- and compute in fp32 (the reference accumulates in half), so results are at least as accurate as
 * its own. bfloat16 is additive. They always take the warp-per-row gather path (any d from 1 to 1024; d in
 * {32, 64, 128} has specialised kernels); wide banded masks on 16-bit inputs are better served by converting to fp32
 * and calling the fp32 entry points, which is what the torch modules do. Arguments are those of the fp32 entry
 * points with `dtype` in front and without a path choice; pointers must be 16-byte aligned when d % 8 == 0, 2-byte
 * otherwise. Workspace: COO needs spfa_coo_min_workspace_bytes(n_rows), Global-no-local
 * spfa_global_no_local_workspace_bytes_16(L, n_global), the others none. */
typedef enum spfa_dtype { SPFA_DTYPE_F32 = 0, SPFA_DTYPE_F16 = 1, SPFA_DTYPE_BF16 = 2 } spfa_dtype;
int spfa_csr_forward_16(int dtype, const void* Q, const void* K, const void* V,
                        const uint64_t* row_off, const uint32_t* col_ind, int64_t nnz,
                        void* m, void* l, void* O, int64_t n_rows, int64_t Lk, int d, int use_nan, void* stream);
int spfa_coo_forward_16(int dtype, const void* Q, const void* K, const void* V,
                        const uint64_t* row_ind, const uint32_t* col_ind, int64_t nnz,
                        void* m, void* l, void* O, int64_t row_begin, int64_t n_rows, int64_t Lk, int d, int use_nan,
                        void* workspace, size_t workspace_bytes, void* stream);
int spfa_local_forward_16(int dtype, const void* Q, const void* K, const void* V, void* m, void* l, void* O,
                          int64_t L, int d, int64_t local_size_each_dir, int64_t row_begin, int64_t row_end, void* stream);
int spfa_local_1d_dilated_forward_16(int dtype, const void* Q, const void* K, const void* V, void* m, void* l, void* O,
                                     int64_t L, int d, int64_t local_size_each_dir, int64_t dil_factor,
                                     int64_t row_begin, int64_t row_end, void* stream);
int spfa_local_2d_dilated_forward_16(int dtype, const void* Q, const void* K, const void* V, void* m, void* l, void* O,
                                     int64_t L, int d, int64_t block_size, int64_t dil_factor, int use_nan,
                                     int64_t row_begin, int64_t row_end, void* stream);
size_t spfa_global_no_local_workspace_bytes_16(int64_t L, int64_t n_global);
int spfa_global_no_local_forward_16(int dtype, const void* Q, const void* K, const void* V, void* m, void* l, void* O,
                                    const int32_t* global_inds, int64_t n_global, int64_t L, int d,
                                    int64_t local_size_each_dir, int64_t row_begin, int64_t row_end,
                                    void* workspace, size_t workspace_bytes, void* stream);

/* ---- dense boolean mask -> CSR / COO arrays on the GPU ----------------------------------------------------
 * No counterpart in the reference: its callers convert a dense [n_rows, n_cols] boolean mask with torch's
 * to_sparse_csr() / to_sparse_coo() and cast the index tensors (verification/verify.py:67-71, 94-98). These two
 * calls produce the operators' arrays directly. `mask` holds one byte per (row, column), row-major, non-zero =
 * attend (torch.bool or torch.uint8).
 *   spfa_dense_mask_offsets  writes row_off[n_rows + 1] (exclusive scan of the entries per row); the total number
 *                            of entries is row_off[n_rows], which the caller reads back to size col_ind
 *   spfa_dense_mask_fill     writes col_ind[row_off[r] ...] = the columns of row r in ascending order and, if
 *                            row_ind is not null, row_ind[...] = r for each of them (the COO row array) */
int spfa_dense_mask_offsets(const uint8_t* mask, int64_t n_rows, int64_t n_cols, uint64_t* row_off, void* stream);
int spfa_dense_mask_fill(const uint8_t* mask, int64_t n_rows, int64_t n_cols, const uint64_t* row_off,
                         uint32_t* col_ind, uint64_t* row_ind, void* stream);

/* ---- visited-pair dump (test support) -----------------------------------------------------------
 * Emits the (row, key) set an implicit mask visits, produced by the same device-side column
 * generators the gather kernels use. No counterpart in the reference (its index arithmetic is inlined
 * in each kernel); exists so mask indexing can be compared bit-for-bit with the closed forms.
 *   kind: 0 local(p0=w)  1 local_1d_dilated(p0=w,p1=dil)  2 local_2d_dilated(p0=B,p1=dil)
 *         3 global_no_local(p0=w, global_inds/n_global)
 * Pass 1: spfa_mask_count writes counts[n_rows] (int64). The caller prefix-sums them into
 * row_off[n_rows+1]. Pass 2: spfa_mask_fill writes col_out[row_off[r] ...] in visiting order. */
int spfa_mask_count(int kind, int64_t L, int64_t p0, int64_t p1,
                    const int32_t* global_inds, int64_t n_global,
                    int64_t row_begin, int64_t row_end, int64_t* counts, void* stream);
int spfa_mask_fill(int kind, int64_t L, int64_t p0, int64_t p1,
                   const int32_t* global_inds, int64_t n_global,
                   int64_t row_begin, int64_t row_end, const int64_t* row_off, uint32_t* col_out,
                   void* stream);

/* Reads and clears the error word of the tiled kernels on the current device. Synchronises the device.
 * 0 = no error; a positive code names the bounded wait that gave up (1xx TMA producer, 2xx MMA issuer,
 * 3xx softmax group); -1 = the CUDA runtime reported an error. No counterpart in the reference, whose
 * launches are never checked (sp_flatt_csr_kernel.cu:271). */
int spfa_last_device_error(void);

/* Diagnostics: exercises the time limit of the device-side waits without touching any data. Launches a
 * one-thread kernel that waits on a barrier nothing ever arrives at; after the limit (0.2 s) the wait gives up
 * and records code 9001, which the next spfa_last_device_error() returns (and clears). The context stays
 * usable. No counterpart in the reference. */
int spfa_selftest_wait_limit(void* stream);

/* Number of kernels this library has launched in the calling process since load (monotonic).
 * Benchmarks subtract two readings to report how many launches a timed region contained. */
int64_t spfa_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SPFA_B200_H_ */
