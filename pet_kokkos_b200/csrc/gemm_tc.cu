// Tensor-core GEMM path (placeholder until the tcgen05 kernel lands).
#include "gemm.h"

namespace petb {
bool gemm_tensor_usable(const GemmArgs&, int) { return false; }
void gemm_tensor(Stream&, Arena&, const GemmArgs&, int) { throw Error(3, "gemm: tensor path not built"); }
bool tensor_gemm_available() { return false; }
}  // namespace petb
