// Device-side arithmetic shared by the matmul kernels: the activation quantizer and the
// QuantBlockOrder geometry.
#pragma once

#include "common.cuh"

namespace aion {

// The reference's activation block quantizer for one element of a 32-block whose
// absolute maximum is `amax` (src/aion/backend/cpu/kernels/matmul_q_i8.zig:187-203):
//   amax == 0 -> q = 0, scale = 0; else scale = amax/127, q = clamp(round(a * (127/amax)), +-127)
// with round = half away from zero. Divisions and the product are single IEEE
// roundings (the intrinsics keep the compiler from contracting or approximating them).
__device__ __forceinline__ int quantize_activation_value(float a, float amax, float* scale) {
  if (amax == 0.0f) {
    *scale = 0.0f;
    return 0;
  }
  *scale = __fdiv_rn(amax, 127.0f);
  const float inv = __fdiv_rn(127.0f, amax);
  float r = roundf(__fmul_rn(a, inv));
  r = fminf(127.0f, fmaxf(-127.0f, r));
  return (int)r;
}

// The same quantizer split in two for callers that quantize several elements of one
// block: the block's scale and reciprocal once, then each element.
__device__ __forceinline__ void activation_block_scales(float amax, float* scale, float* inv) {
  if (amax == 0.0f) {
    *scale = 0.0f;
    *inv = 0.0f;  // every element of the block is zero, so q = round(0 * 0) = 0
  } else {
    *scale = __fdiv_rn(amax, 127.0f);
    *inv = __fdiv_rn(127.0f, amax);
  }
}
__device__ __forceinline__ int quantize_activation_with_inv(float a, float inv) {
  const float r = fminf(127.0f, fmaxf(-127.0f, roundf(__fmul_rn(a, inv))));
  return (int)r;
}

// Rows per group and bytes per chunk of a QuantBlockOrder
// (src/aion/backend/types.zig:159-176).
__host__ __device__ inline bool block_order_info(uint32_t order, int* group_rows, int* chunk_bytes) {
  switch (order) {
    case AION_CUDA_ORDER_ROW_MAJOR: *group_rows = 1; *chunk_bytes = 4; return true;
    case AION_CUDA_ORDER_LANES4: *group_rows = 4; *chunk_bytes = 4; return true;
    case AION_CUDA_ORDER_LANES8: *group_rows = 8; *chunk_bytes = 4; return true;
    case AION_CUDA_ORDER_LANES16: *group_rows = 16; *chunk_bytes = 4; return true;
    case AION_CUDA_ORDER_LANES32: *group_rows = 32; *chunk_bytes = 4; return true;
    case AION_CUDA_ORDER_LANES32X16: *group_rows = 32; *chunk_bytes = 16; return true;
    default: return false;
  }
}

__device__ __forceinline__ float f16_bits_to_float(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

}  // namespace aion
