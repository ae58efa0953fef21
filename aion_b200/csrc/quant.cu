// Block quantizer, dequantizer, q8 re-layout and the activation quantizer.
//
// These are byte-exact with the reference, so this file is compiled with
// -fmad=false: no multiply-add may be contracted into one rounding.
#include "common.cuh"
#include "quant_device.cuh"

namespace aion {

struct QuantGeom {
  int rank;
  int axis;
  uint64_t stride[8];   // element strides, row-major
  uint64_t bshape[8];   // block-space shape
};

// One thread per block. Weight quantization is an offline, once-per-model step in the
// reference (src/aion/storage/quantize.zig:31-79); the placement rule is what matters.
template <int DT>
__global__ void quantize_blocks_kernel(const float* __restrict__ values, uint8_t* __restrict__ out, uint64_t nblocks,
                                       QuantGeom g) {
  const uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
  if (i >= nblocks) return;
  uint64_t rest = i, base = 0;
  for (int d = g.rank - 1; d >= 0; d--) {
    const uint64_t c = rest % g.bshape[d];
    rest /= g.bshape[d];
    base += ((d == g.axis) ? c * QK : c) * g.stride[d];
  }
  const uint64_t st = g.stride[g.axis];
  const float* v = values + base;
  float absmax = 0.0f;
  for (int t = 0; t < QK; t++) absmax = fmaxf(absmax, fabsf(v[t * st]));
  uint8_t* dst = out + i * (DT == AION_CUDA_DTYPE_Q8_0 ? Q8_BYTES : Q4_BYTES);
  if (DT == AION_CUDA_DTYPE_Q8_0) {
    // src/aion/storage/quantize.zig:83-103: codes are chosen against the stored f16 scale.
    const float scale = (absmax == 0.0f) ? 1.0f : __fdiv_rn(absmax, 127.0f);
    const __half sh = __float2half_rn(scale);
    // Blocks are 2-byte aligned (even block sizes on an aligned tensor).
    *reinterpret_cast<__half*>(dst) = sh;
    const float eff = __half2float(sh);
    const float inv = (absmax == 0.0f || eff == 0.0f) ? 0.0f : __fdiv_rn(1.0f, eff);
    for (int t = 0; t < QK; t++) {
      int q = (int)roundf(__fmul_rn(v[t * st], inv));
      q = max(-128, min(127, q));
      dst[2 + t] = (uint8_t)(int8_t)q;
    }
  } else {
    // src/aion/backend/cpu/test_cpu_kernels.zig:490-523: divide by the unrounded scale.
    const float scale = (absmax == 0.0f) ? 1.0f : __fdiv_rn(absmax, 7.0f);
    *reinterpret_cast<__half*>(dst) = __float2half_rn(scale);
    for (int i2 = 0; i2 < 16; i2++) {
      int lo = (int)roundf(__fdiv_rn(v[(2 * i2) * st], scale));
      int hi = (int)roundf(__fdiv_rn(v[(2 * i2 + 1) * st], scale));
      lo = max(-8, min(7, lo)) + 8;
      hi = max(-8, min(7, hi)) + 8;
      dst[2 + i2] = (uint8_t)(lo | (hi << 4));
    }
  }
}

// One thread per weight: w = f32(q) * f32(f16 scale). The product of an integer of at
// most 8 bits and an 11-bit significand is exact in f32.
template <int DT>
__global__ void dequantize_kernel(const uint8_t* __restrict__ blocks, float* __restrict__ out, uint64_t nweights) {
  const uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
  if (i >= nweights) return;
  const uint64_t blk = i / QK;
  const int t = (int)(i % QK);
  const uint8_t* p = blocks + blk * (DT == AION_CUDA_DTYPE_Q8_0 ? Q8_BYTES : Q4_BYTES);
  const float scale = __half2float(__ushort_as_half((uint16_t)(p[0] | (p[1] << 8))));
  int q;
  if (DT == AION_CUDA_DTYPE_Q8_0) {
    q = (int8_t)p[2 + t];
  } else {
    const uint8_t byte = p[2 + (t >> 1)];
    q = (int)((t & 1) ? (byte >> 4) : (byte & 0x0F)) - 8;
  }
  out[i] = __fmul_rn((float)q, scale);
}

// QuantBlockOrder placement (src/aion/backend/types.zig:185-222). One thread per
// (row, block, chunk) moves `chunk_bytes` bytes; thread chunk 0 also moves the scale.
__global__ void relayout_q8_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n,
                                   uint64_t blocks, int group, int chunk_bytes, int inverse) {
  const int chunks = 32 / chunk_bytes;
  const uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
  const uint64_t total = n * blocks * chunks;
  if (i >= total) return;
  const int ch = (int)(i % chunks);
  const uint64_t kb = (i / chunks) % blocks;
  const uint64_t r = i / chunks / blocks;
  const uint64_t rm_blk = (r * blocks + kb) * Q8_BYTES;
  const uint64_t seg = ((r / group) * blocks + kb) * (uint64_t)group * Q8_BYTES;
  const uint64_t g_scale = seg + (r % group) * 2;
  const uint64_t g_chunk = seg + 2 * (uint64_t)group + ((uint64_t)ch * group + r % group) * chunk_bytes;
  const uint8_t* s;
  uint8_t* d;
  if (!inverse) {
    s = src + rm_blk + 2 + ch * chunk_bytes;
    d = dst + g_chunk;
  } else {
    s = src + g_chunk;
    d = dst + rm_blk + 2 + ch * chunk_bytes;
  }
  for (int b = 0; b < chunk_bytes; b++) d[b] = s[b];
  if (ch == 0) {
    const uint8_t* ss = inverse ? src + g_scale : src + rm_blk;
    uint8_t* dd = inverse ? dst + rm_blk : dst + g_scale;
    dd[0] = ss[0];
    dd[1] = ss[1];
  }
}

// One warp per (row, block): lane t owns activation t.
__global__ void quantize_activation_kernel(const float* __restrict__ a, uint64_t m, uint64_t kblocks, uint64_t lda,
                                           int8_t* __restrict__ aq, float* __restrict__ ascale) {
  const uint64_t w = (blockIdx.x * (uint64_t)blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x & 31;
  if (w >= m * kblocks) return;
  const uint64_t r = w / kblocks, kb = w % kblocks;
  const float v = a[r * lda + kb * QK + lane];
  float amax = fabsf(v);
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  float scale;
  const int q = quantize_activation_value(v, amax, &scale);
  aq[(r * kblocks + kb) * QK + lane] = (int8_t)q;
  if (lane == 0) ascale[r * kblocks + kb] = scale;
}

int32_t quantize_activation_rows(AionCudaDevice* dev, const float* a, uint64_t m, uint64_t k, uint64_t lda, int8_t* aq,
                                 float* ascale) {
  const uint64_t warps = m * (k / QK);
  if (warps == 0) return AION_CUDA_OK;
  const int threads = 256;
  const uint64_t grid = ceil_div(warps * 32, threads);
  quantize_activation_kernel<<<(unsigned)grid, threads, 0, dev->stream>>>(a, m, k / QK, lda, aq, ascale);
  AION_CUDA_TRY(cudaGetLastError());
  return AION_CUDA_OK;
}

}  // namespace aion

using namespace aion;

extern "C" {

int32_t aion_cuda_quantize(AionCudaDevice* dev, uint32_t dtype, const AionCudaOperand* values, const uint64_t* shape,
                           uint32_t rank, uint32_t quant_axis, const AionCudaOperand* out) {
  if (!dev || !values || !shape || !out) return fail(AION_CUDA_INVALID_ARGUMENT, "quantize: null argument");
  if (dtype != AION_CUDA_DTYPE_Q8_0 && dtype != AION_CUDA_DTYPE_Q4_0)
    return fail(AION_CUDA_UNSUPPORTED, "quantize: dtype %u is not block-quantized", dtype);
  if (rank == 0 || rank > 8 || quant_axis >= rank) return fail(AION_CUDA_INVALID_ARGUMENT, "quantize: rank %u axis %u", rank, quant_axis);
  if (shape[quant_axis] % QK != 0)
    return fail(AION_CUDA_INVALID_ARGUMENT, "quantize: shape[%u] = %llu is not a multiple of 32", quant_axis,
                (unsigned long long)shape[quant_axis]);
  QuantGeom g{};
  g.rank = (int)rank;
  g.axis = (int)quant_axis;
  uint64_t s = 1, nblocks = 1;
  for (int d = (int)rank - 1; d >= 0; d--) {
    g.stride[d] = s;
    s *= shape[d];
    g.bshape[d] = (d == (int)quant_axis) ? shape[d] / QK : shape[d];
    nblocks *= g.bshape[d];
  }
  if (nblocks == 0) return AION_CUDA_OK;
  const float* v;
  uint8_t* o;
  if (int32_t st = resolve(*values, s * sizeof(float), "quantize.values", &v)) return st;
  if (int32_t st = resolve(*out, nblocks * block_bytes_of(dtype), "quantize.out", &o)) return st;
  if ((reinterpret_cast<uintptr_t>(v) & 3) || (reinterpret_cast<uintptr_t>(o) & 1))
    return fail(AION_CUDA_INVALID_ARGUMENT, "quantize: values must be 4-byte aligned, out 2-byte aligned");
  if (int32_t st = dev->make_current()) return st;
  const int threads = 128;
  const unsigned grid = (unsigned)ceil_div(nblocks, threads);
  if (dtype == AION_CUDA_DTYPE_Q8_0)
    quantize_blocks_kernel<AION_CUDA_DTYPE_Q8_0><<<grid, threads, 0, dev->stream>>>(v, o, nblocks, g);
  else
    quantize_blocks_kernel<AION_CUDA_DTYPE_Q4_0><<<grid, threads, 0, dev->stream>>>(v, o, nblocks, g);
  AION_CUDA_TRY(cudaGetLastError());
  return AION_CUDA_OK;
}

int32_t aion_cuda_dequantize(AionCudaDevice* dev, uint32_t dtype, const AionCudaOperand* blocks, uint64_t nblocks,
                             const AionCudaOperand* out) {
  if (!dev || !blocks || !out) return fail(AION_CUDA_INVALID_ARGUMENT, "dequantize: null argument");
  if (dtype != AION_CUDA_DTYPE_Q8_0 && dtype != AION_CUDA_DTYPE_Q4_0)
    return fail(AION_CUDA_UNSUPPORTED, "dequantize: dtype %u is not block-quantized", dtype);
  if (nblocks == 0) return AION_CUDA_OK;
  const uint8_t* b;
  float* o;
  if (int32_t st = resolve(*blocks, nblocks * block_bytes_of(dtype), "dequantize.blocks", &b)) return st;
  if (int32_t st = resolve(*out, nblocks * QK * sizeof(float), "dequantize.out", &o)) return st;
  if (int32_t st = dev->make_current()) return st;
  const int threads = 256;
  const unsigned grid = (unsigned)ceil_div(nblocks * QK, threads);
  if (dtype == AION_CUDA_DTYPE_Q8_0)
    dequantize_kernel<AION_CUDA_DTYPE_Q8_0><<<grid, threads, 0, dev->stream>>>(b, o, nblocks * QK);
  else
    dequantize_kernel<AION_CUDA_DTYPE_Q4_0><<<grid, threads, 0, dev->stream>>>(b, o, nblocks * QK);
  AION_CUDA_TRY(cudaGetLastError());
  return AION_CUDA_OK;
}

int32_t aion_cuda_relayout_q8(AionCudaDevice* dev, uint32_t order, uint32_t inverse, uint64_t n, uint64_t k,
                              const AionCudaOperand* src, const AionCudaOperand* dst) {
  if (!dev || !src || !dst) return fail(AION_CUDA_INVALID_ARGUMENT, "relayout: null argument");
  int group, chunk;
  if (!block_order_info(order, &group, &chunk)) return fail(AION_CUDA_INVALID_ARGUMENT, "relayout: unknown block order %u", order);
  if (k % QK != 0 || n % group != 0)
    return fail(AION_CUDA_INVALID_ARGUMENT, "relayout: [%llu, %llu] does not tile into groups of %d rows of 32-blocks",
                (unsigned long long)n, (unsigned long long)k, group);
  const uint64_t bytes = n * (k / QK) * Q8_BYTES;
  if (bytes == 0) return AION_CUDA_OK;
  const uint8_t* s;
  uint8_t* d;
  if (int32_t st = resolve(*src, bytes, "relayout.src", &s)) return st;
  if (int32_t st = resolve(*dst, bytes, "relayout.dst", &d)) return st;
  if (s == d) return fail(AION_CUDA_INVALID_ARGUMENT, "relayout: src and dst alias");
  if (int32_t st = dev->make_current()) return st;
  const uint64_t total = n * (k / QK) * (32 / chunk);
  const int threads = 256;
  relayout_q8_kernel<<<(unsigned)ceil_div(total, threads), threads, 0, dev->stream>>>(s, d, n, k / QK, group, chunk,
                                                                                      (int)inverse);
  AION_CUDA_TRY(cudaGetLastError());
  return AION_CUDA_OK;
}


int32_t aion_cuda_derive_kmajor_q8(AionCudaDevice* dev, uint32_t order, uint64_t n, uint64_t k, const AionCudaOperand* src,
                                   const AionCudaOperand* dst) {
  if (!dev || !src || !dst) return fail(AION_CUDA_INVALID_ARGUMENT, "derive_kmajor: null argument");
  int group, chunk;
  if (!block_order_info(order, &group, &chunk)) return fail(AION_CUDA_INVALID_ARGUMENT, "derive_kmajor: unknown block order %u", order);
  if (k % QK != 0 || n % group != 0)
    return fail(AION_CUDA_INVALID_ARGUMENT, "derive_kmajor: [%llu, %llu] does not tile into groups of %d rows of 32-blocks",
                (unsigned long long)n, (unsigned long long)k, group);
  const uint64_t bytes = n * (k / QK) * Q8_BYTES;
  if (bytes == 0) return AION_CUDA_OK;
  const uint8_t* s;
  uint8_t* d;
  if (int32_t st = resolve(*src, bytes, "derive_kmajor.src", &s)) return st;
  if (int32_t st = resolve(*dst, bytes, "derive_kmajor.dst", &d)) return st;
  if (s == d) return fail(AION_CUDA_INVALID_ARGUMENT, "derive_kmajor: src and dst alias");
  if (((uintptr_t)s | (uintptr_t)d) & 1) return fail(AION_CUDA_INVALID_ARGUMENT, "derive_kmajor: blocks must be 2-byte aligned");
  if (int32_t st = dev->make_current()) return st;
  return aion::nt_blocks_to_kmajor(dev, order, s, d, n, k / QK);
}

}  // extern "C"
