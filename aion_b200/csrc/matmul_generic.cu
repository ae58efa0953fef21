// Any-shape quantized matmul: the path for shapes the tiled kernels do not read
// (n not a multiple of 8, unaligned leading dimensions, grouped block orders, ...).
//
// Arithmetic is the reference CPU kernels': the activation is quantized to int8 per
// 32-block (src/aion/backend/cpu/kernels/matmul_q_i8.zig:187-203), each block
// contributes float(int dot) * (a_scale * b_scale), accumulated in f32
// (src/aion/backend/cpu/kernels/matvec_q.zig:124-143), then alpha / beta
// (src/aion/backend/cpu/kernels/matvec_q.zig:32-34).
//
// Launch shape: one warp per output column, lanes stride over the K blocks and a
// shuffle tree folds them; the y grid dimension walks the rows of A. The quantized
// activation comes from device scratch filled by one pre-pass.
#include "common.cuh"
#include "quant_device.cuh"

namespace aion {

struct BlockAddr {
  uint32_t dtype;
  int nt;
  int group, chunk;  // QuantBlockOrder geometry (nt only)
  uint64_t ldb;      // K-major: blocks per block-row; nt: blocks per row
};

// Reads one block's scale and its 32 codes (as 8 packed int8x4 words in K order).
__device__ __forceinline__ void read_block(const uint8_t* __restrict__ b, const BlockAddr& ad, uint64_t kb, uint64_t j,
                                           float* scale, uint32_t q[8]) {
  if (!ad.nt) {
    const int bb = (ad.dtype == AION_CUDA_DTYPE_Q8_0) ? Q8_BYTES : Q4_BYTES;
    const uint8_t* p = b + (kb * ad.ldb + j) * bb;
    const uint16_t* p16 = reinterpret_cast<const uint16_t*>(p);  // blocks are 2-byte aligned
    *scale = f16_bits_to_float(p16[0]);
    if (ad.dtype == AION_CUDA_DTYPE_Q8_0) {
#pragma unroll
      for (int w = 0; w < 8; w++) q[w] = (uint32_t)p16[1 + 2 * w] | ((uint32_t)p16[2 + 2 * w] << 16);
    } else {
      // Byte i holds elements 2i (low nibble) and 2i+1 (high); value = nibble - 8
      // (src/aion/backend/cpu/kernels/matmul_q_i8.zig:362-369).
#pragma unroll
      for (int w = 0; w < 8; w++) {
        const uint32_t two = p16[1 + w];  // bytes 2w, 2w+1 -> elements 4w..4w+3
        uint32_t word = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int nib = (two >> (4 * e)) & 0xF;
          word |= (uint32_t)((nib - 8) & 0xFF) << (8 * e);
        }
        q[w] = word;
      }
    }
  } else {
    // QuantBlockOrder addressing (src/aion/backend/types.zig:185-204).
    const uint64_t seg = ((j / ad.group) * ad.ldb + kb) * (uint64_t)ad.group * Q8_BYTES;
    const int rg = (int)(j % ad.group);
    *scale = f16_bits_to_float(*reinterpret_cast<const uint16_t*>(b + seg + rg * 2));
    const uint8_t* quants = b + seg + 2 * ad.group;
    if (ad.chunk == 4) {
#pragma unroll
      for (int w = 0; w < 8; w++) {
        const uint16_t* c16 = reinterpret_cast<const uint16_t*>(quants + ((uint64_t)w * ad.group + rg) * 4);
        q[w] = (uint32_t)c16[0] | ((uint32_t)c16[1] << 16);
      }
    } else {
#pragma unroll
      for (int ch = 0; ch < 2; ch++) {
        const uint16_t* c16 = reinterpret_cast<const uint16_t*>(quants + ((uint64_t)ch * ad.group + rg) * 16);
#pragma unroll
        for (int w = 0; w < 4; w++) q[ch * 4 + w] = (uint32_t)c16[2 * w] | ((uint32_t)c16[2 * w + 1] << 16);
      }
    }
  }
}

__global__ void matmul_q_generic_kernel(const uint8_t* __restrict__ b, BlockAddr ad, const int8_t* __restrict__ aq,
                                        const float* __restrict__ ascale, float* __restrict__ c, uint64_t n,
                                        uint64_t kblocks, uint64_t ldc, float alpha, float beta) {
  const int lane = threadIdx.x & 31;
  const uint64_t j = blockIdx.x * (uint64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t r = blockIdx.y;
  if (j >= n) return;
  const int8_t* aq_row = aq + r * kblocks * QK;
  const float* as_row = ascale + r * kblocks;
  float acc = 0.0f;
  for (uint64_t kb = lane; kb < kblocks; kb += 32) {
    float bs;
    uint32_t q[8];
    read_block(b, ad, kb, j, &bs, q);
    const uint4* ap = reinterpret_cast<const uint4*>(aq_row + kb * QK);
    const uint4 a0 = ap[0], a1 = ap[1];
    int d = 0;
    d = __dp4a((int)q[0], (int)a0.x, d);
    d = __dp4a((int)q[1], (int)a0.y, d);
    d = __dp4a((int)q[2], (int)a0.z, d);
    d = __dp4a((int)q[3], (int)a0.w, d);
    d = __dp4a((int)q[4], (int)a1.x, d);
    d = __dp4a((int)q[5], (int)a1.y, d);
    d = __dp4a((int)q[6], (int)a1.z, d);
    d = __dp4a((int)q[7], (int)a1.w, d);
    acc += (float)d * (as_row[kb] * bs);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if (lane == 0) {
    float* cp = c + r * ldc + j;
    *cp = (beta == 0.0f) ? alpha * acc : alpha * acc + beta * *cp;
  }
}

int32_t matmul_generic(AionCudaDevice* dev, const MatMulArgs& g) {
  if (g.m == 0 || g.n == 0) return AION_CUDA_OK;
  const uint64_t kblocks = g.k / QK;
  // Scratch: int8 activations (32-byte aligned rows) then their scales.
  const size_t aq_bytes = (g.m * g.k + 255) & ~size_t(255);
  const size_t as_bytes = g.m * kblocks * sizeof(float);
  if (int32_t st = dev->reserve_scratch(aq_bytes + as_bytes)) return st;
  int8_t* aq = static_cast<int8_t*>(dev->lane_scratch());
  float* ascale = reinterpret_cast<float*>(static_cast<uint8_t*>(dev->lane_scratch()) + aq_bytes);
  if (int32_t st = quantize_activation_rows(dev, g.a, g.m, g.k, g.lda, aq, ascale)) return st;

  BlockAddr ad{};
  ad.dtype = g.dtype;
  ad.nt = g.nt ? 1 : 0;
  ad.ldb = g.ldb;
  ad.group = 1;
  ad.chunk = 4;
  if (g.nt && !block_order_info(g.order, &ad.group, &ad.chunk))
    return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_nt: unknown block order %u", g.order);
  const int warps = 8;
  if (g.m > 65535) return fail(AION_CUDA_UNSUPPORTED, "matmul: the any-shape kernel takes at most 65535 rows, got %llu",
                               (unsigned long long)g.m);
  dim3 grid((unsigned)ceil_div(g.n, warps), (unsigned)g.m);
  matmul_q_generic_kernel<<<grid, warps * 32, 0, dev->stream>>>(g.b, ad, aq, ascale, g.c, g.n, kblocks, g.ldc, g.alpha,
                                                                g.beta);
  AION_CUDA_TRY(cudaGetLastError());
  return AION_CUDA_OK;
}

}  // namespace aion
