// Tensor-core kernel of the latent sparse attention (placeholder until the kernel lands: every shape
// goes to the FP32 kernel).
#include "ds_sparse.cuh"

namespace sdb {
bool sparse_mma_supported(const SparseArgs&) { return false; }
void sparse_mma_launch(Device&, const SparseArgs&, const float*, const float*, size_t, size_t, const double2*, const double2*, float*) {
    throw std::runtime_error("the tensor-core sparse attention kernel is not built");
}
}  // namespace sdb
