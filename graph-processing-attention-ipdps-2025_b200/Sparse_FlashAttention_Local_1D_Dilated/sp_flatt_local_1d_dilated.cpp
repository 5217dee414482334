// Torch-extension binding `spfa_local_1d_dilated` -- same module name, function name, argument order
// and tensor layouts as the reference
// (Sparse_FlashAttention_Local_1D_Dilated/sp_flatt_local_1d_dilated.cpp:26-52); the reference's
// sp_flatt_local_1d_dilated_kernel.cu is replaced by the sm_100a library behind
// spfa_local_1d_dilated_forward_f32().
#include "binding_common.h"

// Host dispatch: stands in for spfa_local_1d_dilated_cuda_forward (sp_flatt_local_1d_dilated_kernel.cu:209-280).
torch::Tensor spfa_local_1d_dilated_cuda_forward(torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor m,
                                                 torch::Tensor l, torch::Tensor O, int local_size_each_dir,
                                                 int dil_factor) {
  using namespace spfa_binding;
  if (const int64_t S = batched_slices(Q, K, V, m, l, O)) {  // [..., L, d]: every slice in one launch per residue class
    const int64_t L = Q.size(-2);
    TORCH_CHECK(K.size(-2) == L, "implicit masks need K/V with as many rows as Q");
    c10::cuda::CUDAGuard guard(Q.device());
    raise_for_status(spfa_local_1d_dilated_forward_batched_f32(
        Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(), m.data_ptr<float>(), l.data_ptr<float>(),
        O.data_ptr<float>(), S, L, (int)Q.size(-1), local_size_each_dir, dil_factor, 0, L, nullptr, 0,
        at::cuda::getCurrentCUDAStream().stream()));
    return O;
  }
  // 16-bit tensors: narrow windows (where the float32 call takes the gather path too) run natively in 16 bits
  if (is_16bit(Q) && (local_size_each_dir < 32 || dil_factor >= 16 || !tiled_d(Q.size(1)))) {
    check_qkv_state_16(Q, K, V, m, l, O);
    TORCH_CHECK(K.size(0) == Q.size(0), "implicit masks need K/V with as many rows as Q");
    c10::cuda::CUDAGuard guard(Q.device());
    raise_for_status(spfa_local_1d_dilated_forward_16(dtype_code(Q), Q.data_ptr(), K.data_ptr(), V.data_ptr(), m.data_ptr(),
                                                      l.data_ptr(), O.data_ptr(), Q.size(0), (int)Q.size(1),
                                                      local_size_each_dir, dil_factor, 0, Q.size(0),
                                                      at::cuda::getCurrentCUDAStream().stream()));
    return O;
  }
  if (needs_float32_copy(Q)) {
    return via_float32(Q, K, V, m, l, O, [&](torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor mm,
                                             torch::Tensor ll, torch::Tensor oo) {
      spfa_local_1d_dilated_cuda_forward(q, k, v, mm, ll, oo, local_size_each_dir, dil_factor);
    });
  }
  check_qkv_state(Q, K, V, m, l, O);
  TORCH_CHECK(K.size(0) == Q.size(0), "implicit masks need K/V with as many rows as Q");
  c10::cuda::CUDAGuard guard(Q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t L = Q.size(0);
  Workspace ws(spfa_local_1d_dilated_workspace_bytes(L, L, (int)Q.size(1)), Q.device());
  raise_for_status(spfa_local_1d_dilated_forward_f32(Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(),
                                                     m.data_ptr<float>(), l.data_ptr<float>(), O.data_ptr<float>(), L,
                                                     (int)Q.size(1), local_size_each_dir, dil_factor, 0, L, ws.ptr,
                                                     ws.bytes, stream.stream()));
  return O;
}

// C++ interface for PyTorch inputs (sp_flatt_local_1d_dilated.cpp:26-46).
torch::Tensor spfa_local_1d_dilated_forward(torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor m,
                                            torch::Tensor l, torch::Tensor O, int local_size_each_dir, int dil_factor) {
  CHECK_INPUT(Q);
  CHECK_INPUT(K);
  CHECK_INPUT(V);
  CHECK_INPUT(m);
  CHECK_INPUT(l);
  CHECK_INPUT(O);
  return spfa_local_1d_dilated_cuda_forward(Q, K, V, m, l, O, local_size_each_dir, dil_factor);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, mod) {
  mod.def("forward", &spfa_local_1d_dilated_forward, "Sparse-FlashAttention forward (CUDA)");
}
