// Torch-extension binding `spfa_global_no_local` -- same module name, function name, argument order
// and tensor layouts as the reference
// (Sparse_FlashAttention_Global_No_Local/sp_flatt_global_no_local.cpp:26-53); the reference's
// sp_flatt_global_no_local_kernel.cu is replaced by the sm_100a library behind
// spfa_global_no_local_forward_f32().
#include "binding_common.h"

// Host dispatch: stands in for spfa_global_no_local_cuda_forward (sp_flatt_global_no_local_kernel.cu:280-353).
torch::Tensor spfa_global_no_local_cuda_forward(torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor m,
                                                torch::Tensor l, torch::Tensor O, torch::Tensor global_inds,
                                                int local_size_each_dir) {
  using namespace spfa_binding;
  if (const int64_t S = batched_slices(Q, K, V, m, l, O)) {
    const int64_t L = Q.size(-2), nG = global_inds.size(0);
    TORCH_CHECK(K.size(-2) == L, "implicit masks need K/V with as many rows as Q");
    TORCH_CHECK(global_inds.dim() == 1 && global_inds.scalar_type() == torch::kInt32, "global_inds must be 1-D torch.int32");
    c10::cuda::CUDAGuard guard(Q.device());
    Workspace ws(spfa_global_no_local_workspace_bytes(L, L, (int)Q.size(-1), nG), Q.device());
    raise_for_status(spfa_global_no_local_forward_batched_f32(
        Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(), m.data_ptr<float>(), l.data_ptr<float>(),
        O.data_ptr<float>(), S, nG > 0 ? global_inds.data_ptr<int32_t>() : nullptr, nG, L, (int)Q.size(-1),
        local_size_each_dir, 0, L, ws.ptr, ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    return O;
  }
  // 16-bit tensors: short lists of global tokens (where the float32 call keeps the ordinary rows on the gather path)
  if (is_16bit(Q) && (global_inds.size(0) < 32 || !tiled_d(Q.size(1)))) {
    check_qkv_state_16(Q, K, V, m, l, O);
    TORCH_CHECK(K.size(0) == Q.size(0), "implicit masks need K/V with as many rows as Q");
    TORCH_CHECK(global_inds.dim() == 1, "global_inds must be 1-D");
    TORCH_CHECK(global_inds.scalar_type() == torch::kInt32, "global_inds must be torch.int32");
    c10::cuda::CUDAGuard guard(Q.device());
    const int64_t L16 = Q.size(0), nG16 = global_inds.size(0);
    Workspace ws(spfa_global_no_local_workspace_bytes_16(L16, nG16), Q.device());
    raise_for_status(spfa_global_no_local_forward_16(dtype_code(Q), Q.data_ptr(), K.data_ptr(), V.data_ptr(), m.data_ptr(),
                                                     l.data_ptr(), O.data_ptr(),
                                                     nG16 > 0 ? global_inds.data_ptr<int32_t>() : nullptr, nG16, L16,
                                                     (int)Q.size(1), local_size_each_dir, 0, L16, ws.ptr, ws.bytes,
                                                     at::cuda::getCurrentCUDAStream().stream()));
    return O;
  }
  if (needs_float32_copy(Q)) {
    return via_float32(Q, K, V, m, l, O, [&](torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor mm,
                                             torch::Tensor ll, torch::Tensor oo) {
      spfa_global_no_local_cuda_forward(q, k, v, mm, ll, oo, global_inds, local_size_each_dir);
    });
  }
  check_qkv_state(Q, K, V, m, l, O);
  TORCH_CHECK(K.size(0) == Q.size(0), "implicit masks need K/V with as many rows as Q");
  TORCH_CHECK(global_inds.dim() == 1, "global_inds must be 1-D");
  TORCH_CHECK(global_inds.scalar_type() == torch::kInt32, "global_inds must be torch.int32");
  c10::cuda::CUDAGuard guard(Q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t L = Q.size(0), nG = global_inds.size(0);
  Workspace ws(spfa_global_no_local_workspace_bytes(L, L, (int)Q.size(1), nG), Q.device());
  raise_for_status(spfa_global_no_local_forward_f32(
      Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(), m.data_ptr<float>(), l.data_ptr<float>(),
      O.data_ptr<float>(), nG > 0 ? global_inds.data_ptr<int32_t>() : nullptr, nG, L, (int)Q.size(1),
      local_size_each_dir, 0, L, ws.ptr, ws.bytes, stream.stream()));
  return O;
}

// C++ interface for PyTorch inputs (sp_flatt_global_no_local.cpp:26-47).
torch::Tensor spfa_global_no_local_forward(torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor m,
                                           torch::Tensor l, torch::Tensor O, torch::Tensor global_inds,
                                           int local_size_each_dir) {
  CHECK_INPUT(Q);
  CHECK_INPUT(K);
  CHECK_INPUT(V);
  CHECK_INPUT(m);
  CHECK_INPUT(l);
  CHECK_INPUT(O);
  CHECK_INPUT(global_inds);
  return spfa_global_no_local_cuda_forward(Q, K, V, m, l, O, global_inds, local_size_each_dir);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, mod) {
  mod.def("forward", &spfa_global_no_local_forward, "Sparse-FlashAttention forward (CUDA)");
}
