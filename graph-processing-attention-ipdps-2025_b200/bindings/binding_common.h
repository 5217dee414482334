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
  TORCH_CHECK(Q.scalar_type() == torch::kFloat32,
              "spfa_b200 computes in float32; got ", Q.scalar_type(), " (float16/float64 I/O is not built)");
  for (const torch::Tensor* t : {&K, &V, &m, &l, &O}) {
    TORCH_CHECK(t->scalar_type() == Q.scalar_type(), "expected all floating tensors to share Q's dtype");
    TORCH_CHECK(t->device() == Q.device(), "expected all tensors on Q's device");
  }
  const int64_t L = Q.size(0), d = Q.size(1);
  TORCH_CHECK(K.size(1) == d && V.size(1) == d && O.size(1) == d, "K, V, O must have Q's embedded dimension");
  TORCH_CHECK(K.size(0) == V.size(0), "K and V must have the same number of rows");
  TORCH_CHECK(O.size(0) == L && m.size(0) == L && l.size(0) == L, "O, m, l must have Q's number of rows");
}

inline const uint64_t* u64_ptr(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.scalar_type() == torch::kUInt64 || t.scalar_type() == torch::kInt64, name,
              " must be torch.uint64 (torch.int64 is also accepted)");
  return reinterpret_cast<const uint64_t*>(t.data_ptr());
}

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

}  // namespace spfa_binding
