// Force-included (-include) ahead of each UNMODIFIED reference source when it is compiled for sm_100a.
//
// The reference calls AT_DISPATCH_FLOATING_TYPES_AND_HALF(Q.type(), ...) (e.g.
// Sparse_FlashAttention_CSR/sp_flatt_csr_kernel.cu:270); current torch only accepts a ScalarType there.
// Instead of editing the source, the macro is redefined here to convert either argument kind. Every
// other use of Q.type() -- in particular sizeof(Q.type()) in the maskElePerIter formula
// (sp_flatt_csr_kernel.cu:260-261) -- compiles exactly as written.
#pragma once
#include <torch/extension.h>

namespace spfa_ref_shim {
inline c10::ScalarType to_scalar_type(c10::ScalarType t) { return t; }
inline c10::ScalarType to_scalar_type(const at::DeprecatedTypeProperties& t) { return t.scalarType(); }
}  // namespace spfa_ref_shim

#undef AT_DISPATCH_FLOATING_TYPES_AND_HALF
#define AT_DISPATCH_FLOATING_TYPES_AND_HALF(TYPE, NAME, ...) \
  AT_DISPATCH_SWITCH(spfa_ref_shim::to_scalar_type(TYPE), NAME, AT_DISPATCH_CASE_FLOATING_TYPES_AND_HALF(__VA_ARGS__))
