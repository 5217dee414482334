// Torch-extension module `spfa_bigbird` -- additive, no folder of this name exists in the reference. It fuses what the
// reference composes from three chained calls on one (m, l, O) (verification/verify.py:337-352: spfa_local.forward,
// then spfa_global_no_local.forward, then spfa_csr.forward on the remaining random entries) into one operator with the
// same conventions: float32 CUDA tensors [L, d] / [L], int32 global_inds, uint64 row offsets, uint32 columns, (m, l, O)
// read-modify-write, O returned.
#include "binding_common.h"

// forward(Q, K, V, m, l, O, global_inds, local_size_each_dir, W_row_off, W_col_ind): attention over
//   { |i-j| <= w }  +  { i or j in global_inds, |i-j| > w }  +  the CSR entries (which must not repeat the other two).
// W_col_ind may be empty (then W_row_off is ignored).
torch::Tensor spfa_bigbird_forward(torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor m, torch::Tensor l,
                                   torch::Tensor O, torch::Tensor global_inds, int local_size_each_dir,
                                   torch::Tensor W_row_off, torch::Tensor W_col_ind) {
  using namespace spfa_binding;
  CHECK_INPUT(Q);
  CHECK_INPUT(K);
  CHECK_INPUT(V);
  CHECK_INPUT(m);
  CHECK_INPUT(l);
  CHECK_INPUT(O);
  CHECK_INPUT(global_inds);
  CHECK_INPUT(W_row_off);
  CHECK_INPUT(W_col_ind);
  if (needs_float32_copy(Q))
    return via_float32(Q, K, V, m, l, O, [&](torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor mm,
                                             torch::Tensor ll, torch::Tensor oo) {
      spfa_bigbird_forward(q, k, v, mm, ll, oo, global_inds, local_size_each_dir, W_row_off, W_col_ind);
    });
  check_qkv_state(Q, K, V, m, l, O);
  TORCH_CHECK(K.size(0) == Q.size(0), "implicit masks need K/V with as many rows as Q");
  TORCH_CHECK(global_inds.dim() == 1 && global_inds.scalar_type() == torch::kInt32, "global_inds must be 1-D torch.int32");
  TORCH_CHECK(W_col_ind.dim() == 1 && W_row_off.dim() == 1, "W_row_off and W_col_ind must be 1-D");
  const int64_t L = Q.size(0), nG = global_inds.size(0), nnz = W_col_ind.size(0);
  TORCH_CHECK(nnz == 0 || W_row_off.size(0) == L + 1, "W_row_off must have L+1 entries");
  c10::cuda::CUDAGuard guard(Q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  Workspace ws(spfa_bigbird_workspace_bytes(L, L, (int)Q.size(1), nG, nnz), Q.device());
  raise_for_status(spfa_bigbird_forward_f32(
      Q.data_ptr<float>(), K.data_ptr<float>(), V.data_ptr<float>(), m.data_ptr<float>(), l.data_ptr<float>(),
      O.data_ptr<float>(), nG > 0 ? global_inds.data_ptr<int32_t>() : nullptr, nG,
      nnz ? u64_ptr(W_row_off, "W_row_off") : nullptr, nnz ? u32_ptr(W_col_ind, "W_col_ind") : nullptr, nnz, L,
      (int)Q.size(1), local_size_each_dir, 0, L, ws.ptr, ws.bytes, stream.stream()));
  return O;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, mod) {
  mod.def("forward", &spfa_bigbird_forward, "Fused Local + Global-no-local + CSR forward (CUDA)");
}
