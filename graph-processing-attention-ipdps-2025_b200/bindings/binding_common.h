// Shared helpers of the six torch-extension bindings: input checks with the reference's messages,
// status -> exception mapping, raw pointers, workspace from torch's caching allocator.
//
// The checks mirror the reference bindings (Sparse_FlashAttention_CSR/sp_flatt_csr.cpp:7-9,41-49):
// every tensor must be a CUDA tensor and contiguous, else RuntimeError with
// "<name> must be a CUDA tensor" / "<name> must be contiguous". Parameter-range failures surface as
// std::invalid_argument (ValueError in Python) with the reference's texts
// (e.g. Sparse_FlashAttention_Local/sp_flatt_local_kernel.cu:252-254).
#pragma once
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "spfa_b200.h"

#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) \
  CHECK_CUDA(x);       \
  CHECK_CONTIGUOUS(x)

namespace spfa_binding {

inline void raise_for_status(int rc) {
  if (rc == SPFA_OK) return;
  switch (rc) {
    case SPFA_ERR_EMBED_DIM:
    case SPFA_ERR_LOCAL_SIZE:
    case SPFA_ERR_DILATION_NEG:
    case SPFA_ERR_BLOCK_DIVISOR:
    case SPFA_ERR_DILATION_BLOCK:
    case SPFA_ERR_GLOBAL_COUNT:
      throw std::invalid_argument(spfa_status_string(rc));
    default:
      TORCH_CHECK(false, "spfa_b200: ", spfa_status_string(rc), " (status ", rc, ")");
  }
}

// Q, K, V, O: [rows, d] float32; m, l: [rows]. All on Q's device.
inline void check_qkv_state(const torch::Tensor& Q, const torch::Tensor& K, const torch::Tensor& V,
                            const torch::Tensor& m, const torch::Tensor& l, const torch::Tensor& O) {
  TORCH_CHECK(Q.dim() == 2 && K.dim() == 2 && V.dim() == 2 && O.dim() == 2, "Q, K, V, O must be 2-D [L, d]");
  TORCH_CHECK(m.dim() == 1 && l.dim() == 1, "m and l must be 1-D [L]");
  TORCH_CHECK(Q.scalar_type() == torch::kFloat32, "spfa_b200: internal error, float32 tensors expected here, got ",
              Q.scalar_type());
  for (const torch::Tensor* t : {&K, &V, &m, &l, &O}) {
    TORCH_CHECK(t->scalar_type() == Q.scalar_type(), "expected all floating tensors to share Q's dtype");
    TORCH_CHECK(t->device() == Q.device(), "expected all tensors on Q's device");
  }
  const int64_t L = Q.size(0), d = Q.size(1);
  TORCH_CHECK(K.size(1) == d && V.size(1) == d && O.size(1) == d, "K, V, O must have Q's embedded dimension");
  TORCH_CHECK(K.size(0) == V.size(0), "K and V must have the same number of rows");
  TORCH_CHECK(O.size(0) == L && m.size(0) == L && l.size(0) == L, "O, m, l must have Q's number of rows");
}

// The reference dispatches over double, float and half (AT_DISPATCH_FLOATING_TYPES_AND_HALF,
// Sparse_FlashAttention_CSR/sp_flatt_csr_kernel.cu:270). The kernels here compute in float32 (TF32 on the tiled
// path), so tensors of another floating dtype are converted on the way in and (m, l, O) are written back in their
// own dtype: float16 / bfloat16 results are at least as accurate as arithmetic in that dtype would be, float64
// results carry float32 accuracy (a stated difference from the reference, which computes in double there).
inline bool needs_float32_copy(const torch::Tensor& Q) {
  const auto t = Q.scalar_type();
  if (t == torch::kFloat32) return false;
  TORCH_CHECK(t == torch::kFloat16 || t == torch::kBFloat16 || t == torch::kFloat64,
              "spfa_b200: Q, K, V, m, l, O must be float32, float16, bfloat16 or float64; got ", t);
  return true;
}

// float16 / bfloat16 tensors have native entry points (16-bit loads and stores around fp32 arithmetic, gather path).
// The bindings take them wherever the fp32 call would take the gather path as well; wide bands and long listed-key
// strips, which the fp32 entry points run on the tensor cores, are converted instead (via_float32 below).
inline bool is_16bit(const torch::Tensor& Q) {
  return Q.scalar_type() == torch::kFloat16 || Q.scalar_type() == torch::kBFloat16;
}
inline int dtype_code(const torch::Tensor& Q) { return Q.scalar_type() == torch::kFloat16 ? SPFA_DTYPE_F16 : SPFA_DTYPE_BF16; }
inline void check_same_dtype(const torch::Tensor& Q, std::initializer_list<const torch::Tensor*> ts) {
  for (const torch::Tensor* t : ts) {
    TORCH_CHECK(t->scalar_type() == Q.scalar_type(), "expected all floating tensors to share Q's dtype");
    TORCH_CHECK(t->device() == Q.device(), "expected all tensors on Q's device");
  }
}
// Shape checks of check_qkv_state without its float32 requirement.
inline void check_qkv_state_16(const torch::Tensor& Q, const torch::Tensor& K, const torch::Tensor& V,
                               const torch::Tensor& m, const torch::Tensor& l, const torch::Tensor& O) {
  TORCH_CHECK(Q.dim() == 2 && K.dim() == 2 && V.dim() == 2 && O.dim() == 2, "Q, K, V, O must be 2-D [L, d]");
  TORCH_CHECK(m.dim() == 1 && l.dim() == 1, "m and l must be 1-D [L]");
  check_same_dtype(Q, {&K, &V, &m, &l, &O});
  const int64_t L = Q.size(0), d = Q.size(1);
  TORCH_CHECK(K.size(1) == d && V.size(1) == d && O.size(1) == d, "K, V, O must have Q's embedded dimension");
  TORCH_CHECK(K.size(0) == V.size(0), "K and V must have the same number of rows");
  TORCH_CHECK(O.size(0) == L && m.size(0) == L && l.size(0) == L, "O, m, l must have Q's number of rows");
}
inline bool tiled_d(int64_t d) { return d == 32 || d == 64 || d == 128; }

// f(Q32, K32, V32, m32, l32, O32) runs the float32 path on converted copies; the state is copied back in place.
template <class F>
torch::Tensor via_float32(const torch::Tensor& Q, const torch::Tensor& K, const torch::Tensor& V, torch::Tensor m,
                          torch::Tensor l, torch::Tensor O, F&& f) {
  for (const torch::Tensor* t : std::initializer_list<const torch::Tensor*>{&K, &V, &m, &l, &O})
    TORCH_CHECK(t->scalar_type() == Q.scalar_type(), "expected all floating tensors to share Q's dtype");
  torch::Tensor m32 = m.to(torch::kFloat32), l32 = l.to(torch::kFloat32), O32 = O.to(torch::kFloat32);
  f(Q.to(torch::kFloat32), K.to(torch::kFloat32), V.to(torch::kFloat32), m32, l32, O32);
  m.copy_(m32);
  l.copy_(l32);
  O.copy_(O32);
  return O;
}

inline const uint64_t* u64_ptr(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.scalar_type() == torch::kUInt64 || t.scalar_type() == torch::kInt64, name,
              " must be torch.uint64 (torch.int64 is also accepted)");
  return reinterpret_cast<const uint64_t*>(t.data_ptr());
}

// Row offsets / row indices may also be stored as torch.int32 (additive; the reference's are 64-bit).
inline bool is_idx32(const torch::Tensor& t) { return t.scalar_type() == torch::kInt32; }
inline const int32_t* i32_ptr(const torch::Tensor& t) { return reinterpret_cast<const int32_t*>(t.data_ptr()); }

inline const uint32_t* u32_ptr(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.scalar_type() == torch::kUInt32 || t.scalar_type() == torch::kInt32, name,
              " must be torch.uint32 (torch.int32 is also accepted)");
  return reinterpret_cast<const uint32_t*>(t.data_ptr());
}

struct Workspace {
  torch::Tensor buf;
  void* ptr = nullptr;
  size_t bytes = 0;
  Workspace(size_t need, const torch::Device& dev) {
    if (need == 0) return;
    buf = torch::empty({(int64_t)need + 256}, torch::TensorOptions().dtype(torch::kUInt8).device(dev));
    uintptr_t p = reinterpret_cast<uintptr_t>(buf.data_ptr());
    ptr = reinterpret_cast<void*>((p + 255) & ~uintptr_t(255));
    bytes = need;
  }
};

// ---- stored plans for explicit masks (additive: the reference's modules export `forward` only) ----------
// A plan is a uint8 CUDA tensor whose first byte is 256-byte aligned (a view into a slightly larger buffer).
inline torch::Tensor new_plan_tensor(int64_t n_rows, int64_t nnz, int64_t n_keys, int d, const torch::Device& dev) {
  const size_t need = spfa_explicit_plan_bytes(n_rows, nnz, n_keys, d);
  TORCH_CHECK(need > 0, "spfa_b200: no dense-tile plan for this shape (d must be 32, 64 or 128; the mask non-empty)");
  torch::Tensor buf = torch::empty({(int64_t)need + 256}, torch::TensorOptions().dtype(torch::kUInt8).device(dev));
  const uintptr_t p = reinterpret_cast<uintptr_t>(buf.data_ptr());
  return buf.narrow(0, (int64_t)(((p + 255) & ~uintptr_t(255)) - p), (int64_t)need);
}

// forward_planned(Q, K, V, plan, nnz, m, l, O, use_nan): the forward of the module whose plan() made `plan`.
inline torch::Tensor planned_forward(torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor plan, int64_t nnz,
                                     torch::Tensor m, torch::Tensor l, torch::Tensor O, bool use_nan) {
  CHECK_INPUT(Q);
  CHECK_INPUT(K);
  CHECK_INPUT(V);
  CHECK_INPUT(plan);
  CHECK_INPUT(m);
  CHECK_INPUT(l);
  CHECK_INPUT(O);
  check_qkv_state(Q, K, V, m, l, O);
  TORCH_CHECK(plan.scalar_type() == torch::kUInt8 && plan.dim() == 1, "plan must be the tensor returned by plan()");
  c10::cuda::CUDAGuard guard(Q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  raise_for_status(spfa_planned_forward_f32(Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(),
                                            m.data_ptr<float>(), l.data_ptr<float>(), O.data_ptr<float>(), Q.size(0), nnz,
                                            K.size(0), (int)Q.size(1), use_nan ? 1 : 0, plan.data_ptr(),
                                            (size_t)plan.numel(), stream.stream()));
  return O;
}

// ---- batches (additive): Q, K, V, O with leading batch / head dimensions [..., L, d] and m, l [..., L] ----------------
// The reference is single-head, single-batch (README.md:10) and takes 2-D tensors only. Tensors with more dimensions are
// treated as that many independent problems sharing the mask; the leading dimensions must agree on all six tensors.
// Returns the number of slices (product of the leading dimensions), or 0 for plain 2-D tensors.
inline int64_t batched_slices(const torch::Tensor& Q, const torch::Tensor& K, const torch::Tensor& V,
                              const torch::Tensor& m, const torch::Tensor& l, const torch::Tensor& O) {
  if (Q.dim() <= 2) return 0;
  TORCH_CHECK(Q.scalar_type() == torch::kFloat32, "batched calls take float32 tensors");
  for (const torch::Tensor* t : {&K, &V, &m, &l, &O}) {
    TORCH_CHECK(t->scalar_type() == Q.scalar_type(), "expected all floating tensors to share Q's dtype");
    TORCH_CHECK(t->device() == Q.device(), "expected all tensors on Q's device");
  }
  const int64_t nd = Q.dim();
  TORCH_CHECK(K.dim() == nd && V.dim() == nd && O.dim() == nd && m.dim() == nd - 1 && l.dim() == nd - 1,
              "batched Q, K, V, O must be [..., L, d] and m, l [..., L] with the same leading dimensions");
  int64_t S = 1;
  for (int64_t i = 0; i < nd - 2; ++i) {
    TORCH_CHECK(K.size(i) == Q.size(i) && V.size(i) == Q.size(i) && O.size(i) == Q.size(i) && m.size(i) == Q.size(i) &&
                    l.size(i) == Q.size(i), "leading (batch / head) dimensions differ");
    S *= Q.size(i);
  }
  const int64_t L = Q.size(nd - 2), d = Q.size(nd - 1);
  TORCH_CHECK(K.size(nd - 1) == d && V.size(nd - 1) == d && O.size(nd - 1) == d, "K, V, O must have Q's embedded dimension");
  TORCH_CHECK(K.size(nd - 2) == V.size(nd - 2), "K and V must have the same number of rows");
  TORCH_CHECK(O.size(nd - 2) == L && m.size(nd - 2) == L && l.size(nd - 2) == L, "O, m, l must have Q's number of rows");
  TORCH_CHECK(S >= 1, "empty batch");
  return S;
}

// ---- dense mask -> index tensors (additive: replaces to_sparse_csr()/to_sparse_coo() + casts in caller code) ----
// mask: [n_rows, n_cols] torch.bool or torch.uint8 on the GPU. Returns (row offsets uint64[n_rows+1], columns uint32[nnz])
// or, for COO, (row indices uint64[nnz], columns uint32[nnz]); columns ascend within a row.
inline std::vector<torch::Tensor> dense_mask_to_index_tensors(const torch::Tensor& mask, bool coo) {
  CHECK_INPUT(mask);
  TORCH_CHECK(mask.dim() == 2, "mask must be 2-D [n_rows, n_cols]");
  TORCH_CHECK(mask.scalar_type() == torch::kBool || mask.scalar_type() == torch::kUInt8, "mask must be torch.bool or torch.uint8");
  c10::cuda::CUDAGuard guard(mask.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t n_rows = mask.size(0), n_cols = mask.size(1);
  auto opt = torch::TensorOptions().device(mask.device());
  torch::Tensor row_off = torch::empty({n_rows + 1}, opt.dtype(torch::kUInt64));
  raise_for_status(spfa_dense_mask_offsets(static_cast<const uint8_t*>(mask.data_ptr()), n_rows, n_cols,
                                           static_cast<uint64_t*>(row_off.data_ptr()), stream.stream()));
  const int64_t nnz = row_off.view(torch::kInt64)[n_rows].item<int64_t>();  // synchronises: the sizes of the outputs
  torch::Tensor col = torch::empty({nnz}, opt.dtype(torch::kUInt32));
  torch::Tensor rows = coo ? torch::empty({nnz}, opt.dtype(torch::kUInt64)) : torch::Tensor();
  if (nnz > 0)
    raise_for_status(spfa_dense_mask_fill(static_cast<const uint8_t*>(mask.data_ptr()), n_rows, n_cols,
                                          static_cast<const uint64_t*>(row_off.data_ptr()),
                                          static_cast<uint32_t*>(col.data_ptr()),
                                          coo ? static_cast<uint64_t*>(rows.data_ptr()) : nullptr, stream.stream()));
  if (coo) return {rows, col};
  return {row_off, col};
}

}  // namespace spfa_binding
