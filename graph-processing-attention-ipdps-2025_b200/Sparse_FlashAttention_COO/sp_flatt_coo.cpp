// Torch-extension binding `spfa_coo` -- same module name, function name, argument order and tensor
// layouts as the reference (Sparse_FlashAttention_COO/sp_flatt_coo.cpp:28-59); the reference's
// sp_flatt_coo_kernel.cu is replaced by the sm_100a library behind spfa_coo_forward_f32().
#include "binding_common.h"

// Host dispatch: stands in for spfa_coo_cuda_forward (sp_flatt_coo_kernel.cu:263-327).
torch::Tensor spfa_coo_cuda_forward(torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor W_row_ind,
                                    torch::Tensor W_col_ind, torch::Tensor W_val, torch::Tensor m, torch::Tensor l,
                                    torch::Tensor O, bool use_nan) {
  using namespace spfa_binding;
  if (const int64_t S = batched_slices(Q, K, V, m, l, O)) {  // [..., L, d]: the mask is inspected once for all slices
    const int64_t n_rows = Q.size(-2), Lk = K.size(-2);
    TORCH_CHECK(W_row_ind.dim() == 1 && W_col_ind.dim() == 1 && W_row_ind.size(0) == W_col_ind.size(0),
                "W_row_ind and W_col_ind must be 1-D with one entry per mask non-zero");
    c10::cuda::CUDAGuard guard(Q.device());
    Workspace ws(spfa_coo_workspace_bytes(n_rows, W_row_ind.size(0), Lk, (int)Q.size(-1)), Q.device());
    raise_for_status(spfa_coo_forward_batched_f32(Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(),
                                                  u64_ptr(W_row_ind, "W_row_ind"), u32_ptr(W_col_ind, "W_col_ind"),
                                                  W_row_ind.size(0), m.data_ptr<float>(), l.data_ptr<float>(),
                                                  O.data_ptr<float>(), S, /*row_begin=*/0, n_rows, Lk, (int)Q.size(-1),
                                                  use_nan ? 1 : 0, ws.ptr, ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    return O;
  }
  if (is_16bit(Q)) {  // native 16-bit gather: half the K/V bytes of the float32 call
    check_qkv_state_16(Q, K, V, m, l, O);
    TORCH_CHECK(W_val.scalar_type() == Q.scalar_type(), "expected W_val to share Q's dtype");
    TORCH_CHECK(W_row_ind.dim() == 1 && W_col_ind.dim() == 1 && W_row_ind.size(0) == W_col_ind.size(0),
                "W_row_ind and W_col_ind must be 1-D with one entry per mask non-zero");
    c10::cuda::CUDAGuard guard(Q.device());
    Workspace ws(spfa_coo_min_workspace_bytes(Q.size(0)), Q.device());
    raise_for_status(spfa_coo_forward_16(dtype_code(Q), Q.data_ptr(), K.data_ptr(), V.data_ptr(),
                                         u64_ptr(W_row_ind, "W_row_ind"), u32_ptr(W_col_ind, "W_col_ind"), W_row_ind.size(0),
                                         m.data_ptr(), l.data_ptr(), O.data_ptr(), /*row_begin=*/0, Q.size(0), K.size(0),
                                         (int)Q.size(1), use_nan ? 1 : 0, ws.ptr, ws.bytes,
                                         at::cuda::getCurrentCUDAStream().stream()));
    return O;
  }
  if (needs_float32_copy(Q)) {
    TORCH_CHECK(W_val.scalar_type() == Q.scalar_type(), "expected W_val to share Q's dtype");
    torch::Tensor w32 = W_val.to(torch::kFloat32);
    return via_float32(Q, K, V, m, l, O, [&](torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor mm,
                                             torch::Tensor ll, torch::Tensor oo) {
      spfa_coo_cuda_forward(q, k, v, W_row_ind, W_col_ind, w32, mm, ll, oo, use_nan);
    });
  }
  check_qkv_state(Q, K, V, m, l, O);
  TORCH_CHECK(W_val.scalar_type() == Q.scalar_type(), "expected W_val to share Q's dtype");
  TORCH_CHECK(W_row_ind.dim() == 1 && W_col_ind.dim() == 1 && W_row_ind.size(0) == W_col_ind.size(0),
              "W_row_ind and W_col_ind must be 1-D with one entry per mask non-zero");
  c10::cuda::CUDAGuard guard(Q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  Workspace ws(spfa_coo_workspace_bytes(Q.size(0), W_row_ind.size(0), K.size(0), (int)Q.size(1)), Q.device());
  if (is_idx32(W_row_ind)) {
    raise_for_status(spfa_coo_forward_f32_idx32(Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(),
                                                i32_ptr(W_row_ind), u32_ptr(W_col_ind, "W_col_ind"), W_row_ind.size(0),
                                                m.data_ptr<float>(), l.data_ptr<float>(), O.data_ptr<float>(),
                                                /*row_begin=*/0, Q.size(0), K.size(0), (int)Q.size(1), use_nan ? 1 : 0,
                                                ws.ptr, ws.bytes, stream.stream()));
    return O;
  }
  raise_for_status(spfa_coo_forward_f32(Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(),
                                        u64_ptr(W_row_ind, "W_row_ind"), u32_ptr(W_col_ind, "W_col_ind"),
                                        W_row_ind.size(0), m.data_ptr<float>(), l.data_ptr<float>(),
                                        O.data_ptr<float>(), /*row_begin=*/0, Q.size(0), K.size(0), (int)Q.size(1),
                                        use_nan ? 1 : 0, ws.ptr, ws.bytes, stream.stream()));
  return O;
}

// C++ interface for PyTorch inputs (sp_flatt_coo.cpp:28-53).
torch::Tensor spfa_coo_forward(torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor W_row_ind,
                               torch::Tensor W_col_ind, torch::Tensor W_val, torch::Tensor m, torch::Tensor l,
                               torch::Tensor O, bool use_nan) {
  CHECK_INPUT(Q);
  CHECK_INPUT(K);
  CHECK_INPUT(V);
  CHECK_INPUT(W_row_ind);
  CHECK_INPUT(W_col_ind);
  CHECK_INPUT(W_val);
  CHECK_INPUT(m);
  CHECK_INPUT(l);
  CHECK_INPUT(O);
  return spfa_coo_cuda_forward(Q, K, V, W_row_ind, W_col_ind, W_val, m, l, O, use_nan);
}

// Additive: run the mask inspector once and keep its output. plan(W_row_ind, W_col_ind, n_rows, n_keys, d) -> plan
// tensor for forward_planned(Q, K, V, plan, nnz, m, l, O, use_nan) with nnz = W_col_ind.numel().
torch::Tensor spfa_coo_plan(torch::Tensor W_row_ind, torch::Tensor W_col_ind, int64_t n_rows, int64_t n_keys, int64_t d) {
  using namespace spfa_binding;
  CHECK_INPUT(W_row_ind);
  CHECK_INPUT(W_col_ind);
  TORCH_CHECK(W_row_ind.dim() == 1 && W_col_ind.dim() == 1 && W_row_ind.size(0) == W_col_ind.size(0),
              "W_row_ind and W_col_ind must be 1-D with one entry per mask non-zero");
  c10::cuda::CUDAGuard guard(W_col_ind.device());
  const int64_t nnz = W_col_ind.size(0);
  torch::Tensor plan = new_plan_tensor(n_rows, nnz, n_keys, (int)d, W_col_ind.device());
  if (is_idx32(W_row_ind)) {
    raise_for_status(spfa_coo_plan_build_idx32(i32_ptr(W_row_ind), u32_ptr(W_col_ind, "W_col_ind"), nnz, /*row_begin=*/0,
                                               n_rows, n_keys, (int)d, plan.data_ptr(), (size_t)plan.numel(),
                                               at::cuda::getCurrentCUDAStream().stream()));
    return plan;
  }
  raise_for_status(spfa_coo_plan_build(u64_ptr(W_row_ind, "W_row_ind"), u32_ptr(W_col_ind, "W_col_ind"), nnz,
                                       /*row_begin=*/0, n_rows, n_keys, (int)d, plan.data_ptr(), (size_t)plan.numel(),
                                       at::cuda::getCurrentCUDAStream().stream()));
  return plan;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, mod) {
  mod.def("forward", &spfa_coo_forward, "Sparse-FlashAttention forward (CUDA)");
  mod.def("plan", &spfa_coo_plan, "Dense-tile plan of a COO mask (CUDA)");
  mod.def("mask_to_coo", [](torch::Tensor mask) { return spfa_binding::dense_mask_to_index_tensors(mask, true); },
          "Dense boolean mask -> (row indices uint64, columns uint32) on the GPU");
  mod.def("forward_planned", &spfa_binding::planned_forward, "Sparse-FlashAttention forward from a stored plan (CUDA)");
}
