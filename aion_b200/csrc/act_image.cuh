// The quantized-activation image: A quantized to int8 per 32-block exactly as the reference
// CPU kernels do (src/aion/backend/cpu/kernels/matmul_q_i8.zig:187-203), stored in the order
// the int8 tensor-core matmul reads it, so that its CTAs bulk-copy slices of it straight into
// shared memory. Any kernel that produces an activation (a norm, the GELU gate, attention) can
// write the image of its output next to the f32 values and spare the matmul that follows a
// quantization pass of its own.
//
// Layout, for A [m, k] and a weight dtype (q4_0 and q8_0 read their codes in different orders):
//   rows are cut into groups of `rows_per_group` (2 for m = 1 — one pad row —, then 8, 16, 32, 64;
//   more than 64 rows: groups of 64); K blocks are padded to a multiple of 8 (`kb_pad`);
//   one group = codes [kb_pad][rows_per_group][32 B], then scales [kb_pad][rows_per_group] f32.
//   Pad rows and pad blocks hold zero codes and zero scales (they then contribute nothing); the
//   one exception is the pad row of a single-row image, which repeats the row's scale (its codes
//   are zero all the same): the single-row kernel reads the two scales as the pair (s, s).
// The 32 code bytes of a block are the 8 words the MMA B fragments read (quad lane j finds its
// two registers at bytes 8j..8j+7):
//   q8: word 2j = codes 4j..4j+3, word 2j+1 = codes 16+4j..16+4j+3
//   q4: word 2j = elements 8j+{0,2,4,6}, word 2j+1 = elements 8j+{1,3,5,7} (the order in which a
//       word of q4 weight nibbles splits into its low and high nibbles); the scale carries an
//       exact 1/16, which undoes the weights' placement in the high nibble of a byte.
//
// From the number of rows at which the tensor-core GEMM takes over (gemm_min_m()), the image is
// what THAT kernel reads instead: row-major bf16 [m][k], every value the bf16 rounding of
// code * scale of the same int8 quantization; for q4 weights the order of K inside every group
// of 8 is e0 e4 e1 e5 e2 e6 e3 e7, the order in which a word of q4 nibbles unpacks two at a time.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"
#include "quant_device.cuh"

namespace aion {

constexpr uint32_t ACT_IMAGE_INT8 = 0, ACT_IMAGE_BF16 = 1;

struct ActImageLayout {
  uint32_t kind;            // ACT_IMAGE_INT8 | ACT_IMAGE_BF16
  uint32_t rows_per_group;  // int8 kind
  uint32_t groups;
  uint32_t kb_pad;
  uint32_t group_bytes;     // bf16 kind: the whole image, m * k * 2
  uint32_t kblocks;
  uint32_t rows_shift;      // log2(rows_per_group): the group sizes are powers of two
};

// Rows of A from which aion_cuda_matmul runs the tensor-core GEMM (AION_CUDA_GEMM_MIN_M, or the
// tuning override from the environment); defined with the routing in api.cu.
uint64_t gemm_min_m();

// The int8 kind whatever m is (the int8 kernel quantizing for itself when it was asked for by flag).
inline ActImageLayout act_image_layout_int8(uint64_t m, uint64_t kblocks);

inline ActImageLayout act_image_layout(uint64_t m, uint64_t kblocks) {
  ActImageLayout L;
  L.kblocks = (uint32_t)kblocks;
  if (m >= gemm_min_m()) {
    L.kind = ACT_IMAGE_BF16;
    L.rows_per_group = 1;
    L.rows_shift = 0;
    L.groups = 1;
    L.kb_pad = (uint32_t)kblocks;
    L.group_bytes = (uint32_t)(m * kblocks * QK * 2);
    return L;
  }
  return act_image_layout_int8(m, kblocks);
}
inline ActImageLayout act_image_layout_int8(uint64_t m, uint64_t kblocks) {
  ActImageLayout L;
  L.kblocks = (uint32_t)kblocks;
  L.kind = ACT_IMAGE_INT8;
  L.rows_per_group = m <= 1 ? 2u : (m <= 8 ? 8u : (m <= 16 ? 16u : (m <= 32 ? 32u : 64u)));
  L.rows_shift = m <= 1 ? 1u : (m <= 8 ? 3u : (m <= 16 ? 4u : (m <= 32 ? 5u : 6u)));
  L.groups = m <= 64 ? 1u : (uint32_t)((m + 63) / 64);
  L.kb_pad = (uint32_t)((kblocks + 7) / 8 * 8);
  L.group_bytes = L.kb_pad * L.rows_per_group * 36u;
  return L;
}
inline size_t act_image_total_bytes(const ActImageLayout& L) { return (size_t)L.groups * L.group_bytes; }

// One 32-block of activations -> its 8 code words and its scale (one thread does the block).
template <int DT>
__device__ __forceinline__ float quantize_act_block(const float* __restrict__ src, bool vec4, uint32_t (&o)[8]) {
  float x[QK];
  if (vec4) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float4 f = reinterpret_cast<const float4*>(src)[i];
      x[4 * i] = f.x; x[4 * i + 1] = f.y; x[4 * i + 2] = f.z; x[4 * i + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < QK; i++) x[i] = src[i];
  }
  float am[8];
#pragma unroll
  for (int i = 0; i < 8; i++) am[i] = fmaxf(fmaxf(fabsf(x[4 * i]), fabsf(x[4 * i + 1])), fmaxf(fabsf(x[4 * i + 2]), fabsf(x[4 * i + 3])));
  const float amax = fmaxf(fmaxf(fmaxf(am[0], am[1]), fmaxf(am[2], am[3])), fmaxf(fmaxf(am[4], am[5]), fmaxf(am[6], am[7])));
  float scale, inv;
  activation_block_scales(amax, &scale, &inv);
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t q0 = (uint32_t)quantize_activation_with_inv(x[4 * i], inv) & 0xFF;
    const uint32_t q1 = (uint32_t)quantize_activation_with_inv(x[4 * i + 1], inv) & 0xFF;
    const uint32_t q2 = (uint32_t)quantize_activation_with_inv(x[4 * i + 2], inv) & 0xFF;
    const uint32_t q3 = (uint32_t)quantize_activation_with_inv(x[4 * i + 3], inv) & 0xFF;
    w[i] = (DT == AION_CUDA_DTYPE_Q8_0) ? (q0 | (q1 << 8) | (q2 << 16) | (q3 << 24))    // elements in order
                                         : (q0 | (q2 << 8) | (q1 << 16) | (q3 << 24));   // (e0, e2 | e1, e3)
  }
#pragma unroll
  for (int jj = 0; jj < 4; jj++) {
    if (DT == AION_CUDA_DTYPE_Q8_0) {
      o[2 * jj] = w[jj];
      o[2 * jj + 1] = w[4 + jj];
    } else {
      o[2 * jj] = (w[2 * jj] & 0xFFFFu) | (w[2 * jj + 1] << 16);
      o[2 * jj + 1] = (w[2 * jj] >> 16) | (w[2 * jj + 1] & 0xFFFF0000u);
    }
  }
  const float fold = (DT == AION_CUDA_DTYPE_Q4_0) ? 0.0625f : 1.0f;  // exact
  return scale * fold;
}

// Where block (row, kb) of the image lives.
__device__ __forceinline__ uint8_t* act_image_codes(uint8_t* image, const ActImageLayout& L, uint32_t row, uint32_t kb) {
  const uint32_t g = row >> L.rows_shift, r = row - (g << L.rows_shift);
  return image + (size_t)g * L.group_bytes + ((size_t)kb * L.rows_per_group + r) * 32;
}
__device__ __forceinline__ void act_image_store_scale(uint8_t* image, const ActImageLayout& L, uint32_t row, uint32_t kb, float scale) {
  const uint32_t g = row >> L.rows_shift, r = row - (g << L.rows_shift);
  float* s = reinterpret_cast<float*>(image + (size_t)g * L.group_bytes + (size_t)L.kb_pad * L.rows_per_group * 32) +
             ((size_t)kb * L.rows_per_group + r);
  *s = scale;
  if (L.rows_per_group == 2 && r == 0) s[1] = scale;  // single-row image: the pad row repeats the scale
}

// The same quantizer for a producer whose threads hold four consecutive elements each: eight
// consecutive lanes of a warp (lane & 7 = i holds elements 4i..4i+3) quantize one block
// together and every lane stores one of its 8 words. All 32 lanes of the warp must call
// (with `store` false where there is no block to write).
template <int DT>
__device__ __forceinline__ void quantize_store_block_8lanes(float4 v, uint32_t i, bool store, uint8_t* image, const ActImageLayout& L,
                                                            uint32_t row, uint32_t kb) {
  float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
  float scale, inv;
  activation_block_scales(amax, &scale, &inv);
  if (L.kind == ACT_IMAGE_BF16) {
    // code * scale, rounded to bf16: what the GEMM's own pre-pass writes.
    const float d0 = __fmul_rn((float)quantize_activation_with_inv(v.x, inv), scale), d1 = __fmul_rn((float)quantize_activation_with_inv(v.y, inv), scale);
    const float d2 = __fmul_rn((float)quantize_activation_with_inv(v.z, inv), scale), d3 = __fmul_rn((float)quantize_activation_with_inv(v.w, inv), scale);
    __nv_bfloat162 lo = __floats2bfloat162_rn(d0, d1), hi = __floats2bfloat162_rn(d2, d3);
    uint2 out = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    if (DT == AION_CUDA_DTYPE_Q4_0) {
      // lanes 2u / 2u+1 hold e0..e3 / e4..e7 of a group of 8; the group is stored e0 e4 e1 e5 | e2 e6 e3 e7
      const uint32_t plo = __shfl_xor_sync(0xFFFFFFFFu, out.x, 1), phi = __shfl_xor_sync(0xFFFFFFFFu, out.y, 1);
      if (i & 1) out = make_uint2(__byte_perm(phi, out.y, 0x5410), __byte_perm(phi, out.y, 0x7632));   // (e2,e6), (e3,e7)
      else out = make_uint2(__byte_perm(out.x, plo, 0x5410), __byte_perm(out.x, plo, 0x7632));          // (e0,e4), (e1,e5)
    }
    if (store) *reinterpret_cast<uint2*>(image + ((size_t)row * L.kblocks * QK + (size_t)kb * QK + 4 * i) * 2) = out;
    return;
  }
  const uint32_t q0 = (uint32_t)quantize_activation_with_inv(v.x, inv) & 0xFF;
  const uint32_t q1 = (uint32_t)quantize_activation_with_inv(v.y, inv) & 0xFF;
  const uint32_t q2 = (uint32_t)quantize_activation_with_inv(v.z, inv) & 0xFF;
  const uint32_t q3 = (uint32_t)quantize_activation_with_inv(v.w, inv) & 0xFF;
  uint32_t word, pos;
  if (DT == AION_CUDA_DTYPE_Q8_0) {
    word = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
    pos = i < 4 ? 2 * i : 2 * (i - 4) + 1;
  } else {
    const uint32_t w = q0 | (q2 << 8) | (q1 << 16) | (q3 << 24);
    const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, w, 1);
    word = (i & 1) ? ((other >> 16) | (w & 0xFFFF0000u)) : ((w & 0xFFFFu) | (other << 16));
    pos = i;
  }
  if (store) {
    reinterpret_cast<uint32_t*>(act_image_codes(image, L, row, kb))[pos] = word;
    if (i == 0) act_image_store_scale(image, L, row, kb, scale * ((DT == AION_CUDA_DTYPE_Q4_0) ? 0.0625f : 1.0f));
  }
}

}  // namespace aion
