#include "common.cuh"
namespace aion {
int32_t attention_launch(AionCudaDevice*, const AionCudaAttention*) { return fail(AION_CUDA_UNSUPPORTED, "attention: not built yet"); }
}  // namespace aion
