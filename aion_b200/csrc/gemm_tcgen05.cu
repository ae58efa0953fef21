// Prefill GEMM placeholder: reports "not readable by this kernel" so callers route to
// the any-shape path until the tensor-core kernel lands.
#include "common.cuh"
namespace aion {
int32_t gemm_tcgen05(AionCudaDevice*, const MatMulArgs&, bool) { return AION_CUDA_UNSUPPORTED; }
}  // namespace aion
