// Force-included (-include) ahead of the reference's own sources when they are
// compiled, unmodified, against a current PyTorch.  TEST INFRASTRUCTURE ONLY.
//
// The reference dispatches with AT_DISPATCH_*(tensor.type(), ...)
// (EPPGCN/GCNConv/EPPGCN_kernel.cu:168,321,426,577).  Current PyTorch resolves
// the dispatch type through ::detail::scalar_type(), which no longer has an
// overload for the deprecated type-properties object; this header supplies it,
// so no reference source line has to change.
#pragma once
#include <torch/extension.h>

namespace detail {
inline at::ScalarType scalar_type(const at::DeprecatedTypeProperties &t) { return t.scalarType(); }
}  // namespace detail
