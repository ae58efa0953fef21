// Decoder glue steps: RMSNorm (+residual), elementwise add / mul / GELU gate, RoPE,
// f32 <-> f16 cast, SequenceAppend, GatherRows from a q8_0 table, ArgMax.
//
// These are the ops on either side of the matmul / attention path in a decode program
// (src/bench/models.zig:364-540 in the reference shows the graph shape). Each is a small
// HBM-bound pass; what matters is that they run on the device, in the session's stream,
// so a token step never returns to the host. Arithmetic follows the reference CPU
// executors operation by operation; this file is compiled without FMA contraction so a
// multiply followed by an add rounds twice, as it does there.
#include <cfloat>
#include <cmath>

#include "act_image.cuh"
#include "common.cuh"
#include "ptx.cuh"
#include "quant_device.cuh"

namespace aion {

namespace {

// ---- fast_math (src/aion/backend/cpu/kernels/fast_math.zig:53-141) -------------------
__device__ __forceinline__ float clampf(float x, float lo, float hi) { return fmaxf(lo, fminf(hi, x)); }
__device__ __forceinline__ float exp_approx(float x_in) {
  const float x = clampf(x_in, -80.0f, 80.0f);
  const float y = x * 1.4426950408889634f;
  const int n = (int)floorf(y + 0.5f);
  const float r = y - (float)n;
  const float t = r * 0.6931471805599453f;
  const float c4 = 1.0f / 24.0f, c3 = 1.0f / 6.0f, c2 = 0.5f;
  const float poly = 1.0f + t * (1.0f + t * (c2 + t * (c3 + t * c4)));
  return __uint_as_float((uint32_t)(n + 127) << 23) * poly;
}
__device__ __forceinline__ float sigmoid_approx(float x) {
  float y;
  if (x >= 0.0f) {
    const float e = exp_approx(-x);
    y = 1.0f / (1.0f + e);
  } else {
    const float e = exp_approx(x);
    y = e / (1.0f + e);
  }
  return clampf(y, 0.0f, 1.0f);
}
__device__ __forceinline__ float tanh_approx(float x) { return clampf(2.0f * sigmoid_approx(2.0f * x) - 1.0f, -1.0f, 1.0f); }
// src/aion/backend/cpu/kernels/gelu.zig:8-14
__device__ __forceinline__ float gelu_approx(float x) {
  const float x3 = x * x * x;
  const float t = 0.7978845608028654f * (x + 0.044715f * x3);
  return 0.5f * x * (1.0f + tanh_approx(t));
}

// ---- RMSNorm: one block per row -----------------------------------------------------
constexpr int RMS_THREADS = 128;
__global__ void __launch_bounds__(RMS_THREADS) rms_norm_kernel(float* out, const float* x, const float* __restrict__ gamma,
                                                               const float* __restrict__ beta, const float* residual,
                                                               uint64_t cols, float eps, int* fault) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint64_t r = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* xr = x + r * cols;
  float sq = 0.0f;
  for (uint64_t c = threadIdx.x; c < cols; c += RMS_THREADS) {
    const float v = xr[c];
    sq += v * v;
  }
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
  __shared__ float part[RMS_THREADS / 32];
  if (lane == 0) part[warp] = sq;
  __syncthreads();
  sq = 0.0f;
#pragma unroll
  for (int w = 0; w < RMS_THREADS / 32; w++) sq += part[w];  // same order in every thread
  const float d = sq * (1.0f / (float)cols) + eps;
  if (!(d > 0.0f) || !isfinite(d)) {
    if (threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
    return;
  }
  const float inv = 1.0f / sqrtf(d);
  for (uint64_t c = threadIdx.x; c < cols; c += RMS_THREADS) {
    float v = ((xr[c] * inv) * gamma[c]) + beta[c];
    if (residual) v = v + residual[r * cols + c];
    out[r * cols + c] = v;
  }
}

// ---- elementwise ----------------------------------------------------------------------
__global__ void elemwise_kernel(float* out, const float* a, const float* b, uint64_t n, uint32_t op, uint64_t cols, uint64_t ld_out,
                                uint64_t ld_a, uint64_t ld_b) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t io = i, ia = i, ib = i;
    if (cols) {
      const uint64_t r = i / cols, c = i - r * cols;
      io = r * ld_out + c, ia = r * ld_a + c, ib = r * ld_b + c;
    }
    const float av = a[ia], bv = b[ib];
    float v;
    if (op == AION_CUDA_ELEMWISE_ADD) v = av + bv;
    else if (op == AION_CUDA_ELEMWISE_MUL) v = av * bv;
    else v = gelu_approx(av) * bv;
    out[io] = v;
  }
}

// The same over float4s (rows and row strides are multiples of 4 elements, pointers 16-byte
// aligned): a quarter of the index arithmetic and of the load / store instructions per element;
// each element goes through exactly the arithmetic above.
__device__ __forceinline__ float elemwise_one(float av, float bv, uint32_t op) {
  if (op == AION_CUDA_ELEMWISE_ADD) return av + bv;
  if (op == AION_CUDA_ELEMWISE_MUL) return av * bv;
  return gelu_approx(av) * bv;
}
__global__ void elemwise4_kernel(float4* out, const float4* a, const float4* b, uint64_t n4, uint32_t op, uint64_t cols4, uint64_t ld_out4,
                                 uint64_t ld_a4, uint64_t ld_b4) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n4; i += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t io = i, ia = i, ib = i;
    if (cols4) {
      const uint64_t r = i / cols4, c = i - r * cols4;
      io = r * ld_out4 + c, ia = r * ld_a4 + c, ib = r * ld_b4 + c;
    }
    const float4 av = a[ia], bv = b[ib];
    float4 v;
    v.x = elemwise_one(av.x, bv.x, op);
    v.y = elemwise_one(av.y, bv.y, op);
    v.z = elemwise_one(av.z, bv.z, op);
    v.w = elemwise_one(av.w, bv.w, op);
    out[io] = v;
  }
}

// The same, one float4 per thread over [rows, cols] matrices, also writing the quantized image
// of the result for the matmul that consumes it (act_image.cuh): the eight threads that hold
// one 32-block of a row quantize it together. cols % 32 == 0.
__global__ void __launch_bounds__(256) elemwise4_image_kernel(float4* out, const float4* a, const float4* b, uint64_t n4, uint32_t op,
                                                              uint32_t cols4, uint64_t ld_out4, uint64_t ld_a4, uint64_t ld_b4,
                                                              uint8_t* image, ActImageLayout L, uint32_t image_dtype) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
  const bool on = i < n4;
  const uint64_t ii = on ? i : 0;
  const uint32_t r = (uint32_t)(ii / cols4), c = (uint32_t)(ii - (uint64_t)r * cols4);
  float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (on) {
    const float4 av = a[(uint64_t)r * ld_a4 + c], bv = b[(uint64_t)r * ld_b4 + c];
    v.x = elemwise_one(av.x, bv.x, op);
    v.y = elemwise_one(av.y, bv.y, op);
    v.z = elemwise_one(av.z, bv.z, op);
    v.w = elemwise_one(av.w, bv.w, op);
    out[(uint64_t)r * ld_out4 + c] = v;
  }
  if (image_dtype == AION_CUDA_DTYPE_Q8_0) quantize_store_block_8lanes<AION_CUDA_DTYPE_Q8_0>(v, c & 7, on, image, L, r, c >> 3);
  else quantize_store_block_8lanes<AION_CUDA_DTYPE_Q4_0>(v, c & 7, on, image, L, r, c >> 3);
}

// ---- RoPE: one thread per (b, l, pair); the rotation is reused by every head ----------
__global__ void rope_kernel(float* out, const float* x, const int32_t* __restrict__ pos, uint64_t bl,
                            uint32_t heads, uint32_t d, uint32_t rope_pairs, float step, float scale_factor) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint32_t pairs_total = d / 2;
  const uint64_t idx = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
  if (idx >= bl * pairs_total) return;
  const uint64_t row = idx / pairs_total;
  const uint32_t i = (uint32_t)(idx % pairs_total);
  const float* xb = x + row * heads * d;
  float* ob = out + row * heads * d;
  if (i >= rope_pairs) {
    for (uint32_t h = 0; h < heads; h++) {
      const float lo = xb[h * d + i], hi = xb[h * d + pairs_total + i];
      ob[h * d + i] = lo;
      ob[h * d + pairs_total + i] = hi;
    }
    return;
  }
  // Frequency of pair i by repeated f32 multiplies, as the reference builds its table.
  float f = scale_factor;
  for (uint32_t j = 0; j < i; j++) f *= step;
  const float ang = (float)pos[row] * f;
  double sd, cd;
  sincos((double)ang, &sd, &cd);
  const float sn = (float)sd, cs = (float)cd;
  for (uint32_t h = 0; h < heads; h++) {
    const float xl = xb[h * d + i], xr = xb[h * d + pairs_total + i];
    ob[h * d + i] = xl * cs - xr * sn;
    ob[h * d + pairs_total + i] = xl * sn + xr * cs;
  }
}

// ---- cast -----------------------------------------------------------------------------
__global__ void cast_f32_f16_kernel(__half* __restrict__ out, const float* __restrict__ in, uint64_t n) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = __float2half_rn(in[i]);
}
__global__ void cast_f16_f32_kernel(float* __restrict__ out, const __half* __restrict__ in, uint64_t n) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = __half2float(in[i]);
}

// ---- SequenceAppend: one block per (request, new step), 2-byte units ---------------------
__global__ void sequence_append_kernel(uint16_t* __restrict__ cache, const uint16_t* __restrict__ new_kv,
                                       const int32_t* __restrict__ end_index, uint64_t t_cap, uint64_t row_units,
                                       uint64_t new_len, int rolling, int* fault, const int32_t* __restrict__ page_table,
                                       uint64_t page_tokens, uint64_t pages_per_request, uint64_t pool_pages) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint64_t b = blockIdx.x / new_len, t = blockIdx.x % new_len;
  const int32_t e = end_index[b];
  // The whole request is rejected if any of its steps is out of range, like the
  // reference's check loop before the first write.
  if (e < 0 || (!rolling && (uint64_t)e + new_len > t_cap)) {
    if (threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
    return;
  }
  const uint64_t logical = (uint64_t)e + t;
  const uint64_t dst = rolling ? logical % t_cap : logical;
  const uint16_t* src = new_kv + (b * new_len + t) * row_units;
  uint64_t cache_row = b * t_cap + dst;
  if (page_table) {
    // Paged cache: row dst of request b lives in the page its table names.
    const int32_t page = page_table[b * pages_per_request + dst / page_tokens];
    if (page < 0 || (uint64_t)page >= pool_pages) {
      if (threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
      return;
    }
    cache_row = (uint64_t)page * page_tokens + dst % page_tokens;
  }
  uint16_t* dp = cache + cache_row * row_units;
  for (uint64_t i = threadIdx.x; i < row_units; i += blockDim.x) dp[i] = src[i];
}

// ---- GatherRows from a q8_0 table: one block per gathered row --------------------------
__global__ void gather_rows_q8_kernel(float* __restrict__ out, const uint8_t* __restrict__ table,
                                      const int32_t* __restrict__ indices, uint64_t table_rows, uint64_t d, int group, int chunk,
                                      int* fault) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint64_t i = blockIdx.x;
  long long v = indices[i];
  if (v < 0) v += (long long)table_rows;
  if (v < 0 || v >= (long long)table_rows) {
    if (threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
    return;
  }
  const uint64_t r = (uint64_t)v, blocks = d / QK;
  const int rg = (int)(r % group);
  for (uint64_t e = threadIdx.x; e < d; e += blockDim.x) {
    const uint64_t kb = e / QK;
    const int t = (int)(e % QK);
    // QuantBlockOrder addressing (src/aion/backend/types.zig:185-204).
    const uint8_t* seg = table + ((r / group) * blocks + kb) * (uint64_t)group * Q8_BYTES;
    const float scale = f16_bits_to_float(*reinterpret_cast<const uint16_t*>(seg + rg * 2));
    const int8_t q = (int8_t)seg[2 * group + ((uint64_t)(t / chunk) * group + rg) * chunk + (t % chunk)];
    out[i * d + e] = (float)q * scale;
  }
}

// ---- ArgMax: one block per row; first maximum wins ------------------------------------
__device__ __forceinline__ void argmax_take(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) {
    bv = v;
    bi = i;
  }
}
// Block-wide first-maximum of (bv, bi); the result is valid in warp 0, lane 0.
__device__ __forceinline__ void argmax_block_reduce(float& bv, int& bi) {
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
    const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
    argmax_take(bv, bi, ov, oi);
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sv[warp] = bv, si[warp] = bi;
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    bv = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7FFFFFFF;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      argmax_take(bv, bi, ov, oi);
    }
  }
}
// grid (chunks, rows): every block scans one chunk of a row and leaves its candidate in
// scratch; the last block of a row to finish (a ticket) picks among the candidates.
__global__ void argmax_kernel(int32_t* __restrict__ out, const float* __restrict__ in, uint64_t n, uint64_t chunk_len,
                              float* cand_v, int* cand_i, int* tickets) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint64_t rowi = blockIdx.y;
  const float* row = in + rowi * n;
  const uint64_t lo = blockIdx.x * chunk_len, hi = min(n, lo + chunk_len);
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  // Eight independent loads per thread are in flight before the first comparison; the
  // candidates are still taken in index order.
  uint64_t j = lo + threadIdx.x;
  const uint64_t bd = blockDim.x;
  for (; j + 7 * bd < hi; j += 8 * bd) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; u++) v[u] = row[j + u * bd];
#pragma unroll
    for (int u = 0; u < 8; u++) argmax_take(bv, bi, v[u], (int)(j + u * bd));
  }
  for (; j < hi; j += bd) argmax_take(bv, bi, row[j], (int)j);
  argmax_block_reduce(bv, bi);
  __shared__ int last;
  if (threadIdx.x == 0) {
    cand_v[rowi * gridDim.x + blockIdx.x] = bv;
    cand_i[rowi * gridDim.x + blockIdx.x] = bi;
    __threadfence();
    const int prev = atomicAdd(tickets + rowi, 1);
    last = (prev == (int)gridDim.x - 1);
    if (last) tickets[rowi] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  bv = -INFINITY;
  bi = 0x7FFFFFFF;
  for (uint32_t c = threadIdx.x; c < gridDim.x; c += blockDim.x)
    argmax_take(bv, bi, __ldcg(cand_v + rowi * gridDim.x + c), __ldcg(cand_i + rowi * gridDim.x + c));
  __syncthreads();  // the reduction reuses its shared arrays
  argmax_block_reduce(bv, bi);
  // A NaN in front can never be displaced in the reference's scan; a row of nothing but
  // NaN (no candidate taken) answers 0 as well.
  if (threadIdx.x == 0) out[rowi] = (isnan(row[0]) || bi == 0x7FFFFFFF) ? 0 : bi;
}

// ---- RMSNorm(+residual) then RMSNorm of the result: one block per row ------------------
__device__ __forceinline__ float rms_block_sum(float v, float* part) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  __syncthreads();  // `part` may still be read from the previous reduction
  if (lane == 0) part[warp] = v;
  __syncthreads();
  float s = 0.0f;
#pragma unroll
  for (int w = 0; w < RMS_THREADS / 32; w++) s += part[w];
  return s;
}
__global__ void __launch_bounds__(RMS_THREADS) rms_norm_pair_kernel(float* out1, float* out2, const float* x,
                                                                    const float* __restrict__ gamma1, const float* __restrict__ beta1,
                                                                    const float* residual, const float* __restrict__ gamma2,
                                                                    const float* __restrict__ beta2, uint64_t cols, float eps1,
                                                                    float eps2, int* fault) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  __shared__ float part[RMS_THREADS / 32];
  const uint64_t r = blockIdx.x;
  const float* xr = x + r * cols;
  float sq = 0.0f;
  for (uint64_t c = threadIdx.x; c < cols; c += RMS_THREADS) {
    const float v = xr[c];
    sq += v * v;
  }
  const float d1 = rms_block_sum(sq, part) * (1.0f / (float)cols) + eps1;
  if (!(d1 > 0.0f) || !isfinite(d1)) {
    if (threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
    return;
  }
  const float inv1 = 1.0f / sqrtf(d1);
  sq = 0.0f;
  for (uint64_t c = threadIdx.x; c < cols; c += RMS_THREADS) {
    float v = ((xr[c] * inv1) * gamma1[c]) + beta1[c];
    if (residual) v = v + residual[r * cols + c];
    out1[r * cols + c] = v;
    sq += v * v;
  }
  const float d2 = rms_block_sum(sq, part) * (1.0f / (float)cols) + eps2;
  if (!(d2 > 0.0f) || !isfinite(d2)) {
    if (threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
    return;
  }
  const float inv2 = 1.0f / sqrtf(d2);
  for (uint64_t c = threadIdx.x; c < cols; c += RMS_THREADS)  // each thread re-reads what it wrote itself
    out2[r * cols + c] = ((out1[r * cols + c] * inv2) * gamma2[c]) + beta2[c];
}

// ---- RMSNorm (single or pair) for rows that fit registers: one block per row ------------
// The two kernels above walk a row element by element, several dependent cache round trips
// per thread; on a decode step (a handful of rows) that latency is the whole cost. Here every
// operand of the row is fetched up front as float4s (one round trip), the row stays in
// registers between the sum of squares and the scaling, and the element arithmetic keeps
// the reference's order ((x * inv) * gamma) + beta [+ residual].
constexpr int RMSF_THREADS = 256;
__device__ __forceinline__ float rmsf_block_sum(float v, float* part) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  __syncthreads();  // `part` may still be read from the previous reduction
  if (lane == 0) part[warp] = v;
  __syncthreads();
  float s = 0.0f;
#pragma unroll
  for (int w = 0; w < RMSF_THREADS / 32; w++) s += part[w];  // same order in every thread
  return s;
}
// CH: float4 chunks per thread (cols <= CH * 4 * RMSF_THREADS); PAIR: also out2 = RMSNorm(out1).
// out1 may alias x or residual: a thread reads its own elements before it writes them.
// image != null: also the quantized image (act_image.cuh) of the last output (out2 of a pair,
// out1 otherwise) for the matmul that consumes it; cols % 32 == 0 then, so the eight threads
// that hold one 32-block are eight consecutive lanes.
template <int CH, bool PAIR>
__global__ void __launch_bounds__(RMSF_THREADS) rms_norm_regs_kernel(float* out1, float* out2, const float* x,
                                                                     const float* __restrict__ gamma1, const float* __restrict__ beta1,
                                                                     const float* residual, const float* __restrict__ gamma2,
                                                                     const float* __restrict__ beta2, uint32_t cols, float eps1, float eps2,
                                                                     int* fault, uint8_t* image, ActImageLayout L, uint32_t image_dtype) {
  ptx::pdl_launch_dependents();
  __shared__ float part[RMSF_THREADS / 32];
  const uint32_t n4 = cols / 4;
  const uint64_t row4 = (uint64_t)blockIdx.x * n4;
  const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float4 g1[CH], b1[CH], g2[CH], b2[CH], xv[CH], rs[CH];
  ptx::pdl_wait();
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const uint32_t i = threadIdx.x + c * RMSF_THREADS;
    const bool on = i < n4;
    g1[c] = on ? reinterpret_cast<const float4*>(gamma1)[i] : zero;
    b1[c] = on ? reinterpret_cast<const float4*>(beta1)[i] : zero;
    if (PAIR) {
      g2[c] = on ? reinterpret_cast<const float4*>(gamma2)[i] : zero;
      b2[c] = on ? reinterpret_cast<const float4*>(beta2)[i] : zero;
    }
    xv[c] = on ? reinterpret_cast<const float4*>(x)[row4 + i] : zero;
    rs[c] = (on && residual) ? reinterpret_cast<const float4*>(residual)[row4 + i] : zero;
  }
  float sq = 0.0f;
#pragma unroll
  for (int c = 0; c < CH; c++) sq += ((xv[c].x * xv[c].x + xv[c].y * xv[c].y) + xv[c].z * xv[c].z) + xv[c].w * xv[c].w;
  const float d1 = rmsf_block_sum(sq, part) * (1.0f / (float)cols) + eps1;
  if (!(d1 > 0.0f) || !isfinite(d1)) {
    if (threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
    return;
  }
  const float inv1 = 1.0f / sqrtf(d1);
  sq = 0.0f;
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const uint32_t i = threadIdx.x + c * RMSF_THREADS;
    float4 v;
    v.x = ((xv[c].x * inv1) * g1[c].x) + b1[c].x;
    v.y = ((xv[c].y * inv1) * g1[c].y) + b1[c].y;
    v.z = ((xv[c].z * inv1) * g1[c].z) + b1[c].z;
    v.w = ((xv[c].w * inv1) * g1[c].w) + b1[c].w;
    if (residual) v.x = v.x + rs[c].x, v.y = v.y + rs[c].y, v.z = v.z + rs[c].z, v.w = v.w + rs[c].w;
    if (i < n4) reinterpret_cast<float4*>(out1)[row4 + i] = v;
    else v = zero;
    xv[c] = v;
    sq += ((v.x * v.x + v.y * v.y) + v.z * v.z) + v.w * v.w;
  }
  if (!PAIR) {
    if (image) {
#pragma unroll
      for (int c = 0; c < CH; c++) {
        const uint32_t i = threadIdx.x + c * RMSF_THREADS;
        if (image_dtype == AION_CUDA_DTYPE_Q8_0) quantize_store_block_8lanes<AION_CUDA_DTYPE_Q8_0>(xv[c], i & 7, i < n4, image, L, blockIdx.x, i >> 3);
        else quantize_store_block_8lanes<AION_CUDA_DTYPE_Q4_0>(xv[c], i & 7, i < n4, image, L, blockIdx.x, i >> 3);
      }
    }
    return;
  }
  const float d2 = rmsf_block_sum(sq, part) * (1.0f / (float)cols) + eps2;
  if (!(d2 > 0.0f) || !isfinite(d2)) {
    if (threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
    return;
  }
  const float inv2 = 1.0f / sqrtf(d2);
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const uint32_t i = threadIdx.x + c * RMSF_THREADS;
    float4 v;
    v.x = ((xv[c].x * inv2) * g2[c].x) + b2[c].x;
    v.y = ((xv[c].y * inv2) * g2[c].y) + b2[c].y;
    v.z = ((xv[c].z * inv2) * g2[c].z) + b2[c].z;
    v.w = ((xv[c].w * inv2) * g2[c].w) + b2[c].w;
    if (i < n4) reinterpret_cast<float4*>(out2)[row4 + i] = v;
    if (image) {
      if (image_dtype == AION_CUDA_DTYPE_Q8_0) quantize_store_block_8lanes<AION_CUDA_DTYPE_Q8_0>(v, i & 7, i < n4, image, L, blockIdx.x, i >> 3);
      else quantize_store_block_8lanes<AION_CUDA_DTYPE_Q4_0>(v, i & 7, i < n4, image, L, blockIdx.x, i >> 3);
    }
  }
}

// Launches the register-resident kernel when the row fits and everything is float4-readable.
// Returns false when the caller should use the element-wise kernel instead.
template <bool PAIR>
bool launch_rms_regs(AionCudaDevice* dev, cudaError_t* err, unsigned rows, float* out1, float* out2, const float* x, const float* g1,
                     const float* b1, const float* res, const float* g2, const float* b2, uint64_t cols, float eps1, float eps2,
                     uint8_t* image, uint32_t image_dtype) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(out1) | reinterpret_cast<uintptr_t>(out2) | reinterpret_cast<uintptr_t>(x) |
                         reinterpret_cast<uintptr_t>(g1) | reinterpret_cast<uintptr_t>(b1) | reinterpret_cast<uintptr_t>(res) |
                         reinterpret_cast<uintptr_t>(g2) | reinterpret_cast<uintptr_t>(b2);
  if ((bits & 15) != 0 || cols % 4 != 0 || cols > 4ull * 4 * RMSF_THREADS) return false;
  if (image && cols % QK != 0) return false;
  const uint32_t c32 = (uint32_t)cols;
  const ActImageLayout L = act_image_layout(rows, cols / QK);
  if (cols <= 2ull * 4 * RMSF_THREADS)
    *err = launch_pdl(rms_norm_regs_kernel<2, PAIR>, dim3(rows), dim3(RMSF_THREADS), 0, dev->stream, out1, out2, x, g1, b1, res, g2, b2, c32,
                      eps1, eps2, dev->fault_dev, image, L, image_dtype);
  else
    *err = launch_pdl(rms_norm_regs_kernel<4, PAIR>, dim3(rows), dim3(RMSF_THREADS), 0, dev->stream, out1, out2, x, g1, b1, res, g2, b2, c32,
                      eps1, eps2, dev->fault_dev, image, L, image_dtype);
  return true;
}

// ---- RoPE(q), RoPE(k), f16 cast of k and v, append to both caches: one block per (b, l) ----
__global__ void rope_kv_append_kernel(float* __restrict__ q_out, const float* __restrict__ qkv, const int32_t* __restrict__ pos,
                                      const int32_t* __restrict__ end_index, __half* __restrict__ k_cache,
                                      __half* __restrict__ v_cache, uint32_t len, uint32_t h_q, uint32_t h_kv, uint32_t d,
                                      uint64_t ld, uint64_t t_cap, uint32_t rope_pairs, float step, float scale_factor, int rolling,
                                      int* fault) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint64_t row = blockIdx.x;  // (b, l)
  const uint64_t b = row / len, l = row % len;
  const int32_t e = end_index[b];
  const bool bad = e < 0 || (!rolling && (uint64_t)e + len > t_cap);
  if (bad && threadIdx.x == 0) atomicCAS(fault, FAULT_NONE, FAULT_INVALID_ARGUMENT);
  const uint64_t logical = (uint64_t)(e < 0 ? 0 : e) + l;
  const uint64_t dst_t = rolling ? logical % t_cap : logical;
  const float* src = qkv + row * ld;
  const float* ksrc = src + (uint64_t)h_q * d;
  const float* vsrc = ksrc + (uint64_t)h_kv * d;
  float* qo = q_out + row * (uint64_t)h_q * d;
  __half* kd = k_cache + (b * t_cap + dst_t) * (uint64_t)h_kv * d;
  __half* vd = v_cache + (b * t_cap + dst_t) * (uint64_t)h_kv * d;
  const uint32_t pairs_total = d / 2;
  const float p = (float)pos[row];
  // Loads first, eight heads at a time, so that they are all in flight while the angle is
  // computed: on a decode step this kernel is a chain of cache round trips and nothing else.
  constexpr uint32_t HC = 8;
  for (uint32_t i = threadIdx.x; i < pairs_total; i += blockDim.x) {
    const bool rot = i < rope_pairs;
    float xl[HC], xr[HC], kl[HC], kr[HC];
#pragma unroll
    for (uint32_t u = 0; u < HC; u++) {
      const bool on = u < h_q;
      xl[u] = on ? src[u * d + i] : 0.0f;
      xr[u] = on ? src[u * d + pairs_total + i] : 0.0f;
    }
#pragma unroll
    for (uint32_t u = 0; u < HC; u++) {
      const bool on = !bad && u < h_kv;
      kl[u] = on ? ksrc[u * d + i] : 0.0f;
      kr[u] = on ? ksrc[u * d + pairs_total + i] : 0.0f;
    }
    float sn = 0.0f, cs = 1.0f;
    if (rot) {
      float f = scale_factor;
      for (uint32_t j = 0; j < i; j++) f *= step;
      const float ang = p * f;
      double sd, cd;
      sincos((double)ang, &sd, &cd);
      sn = (float)sd, cs = (float)cd;
    }
    for (uint32_t h0q = 0; h0q < h_q; h0q += HC) {
      if (h0q > 0) {
#pragma unroll
        for (uint32_t u = 0; u < HC; u++) {
          const bool on = h0q + u < h_q;
          xl[u] = on ? src[(h0q + u) * d + i] : 0.0f;
          xr[u] = on ? src[(h0q + u) * d + pairs_total + i] : 0.0f;
        }
      }
#pragma unroll
      for (uint32_t u = 0; u < HC; u++) {
        const uint32_t h = h0q + u;
        if (h >= h_q) break;
        qo[h * d + i] = rot ? xl[u] * cs - xr[u] * sn : xl[u];
        qo[h * d + pairs_total + i] = rot ? xl[u] * sn + xr[u] * cs : xr[u];
      }
    }
    if (!bad)
      for (uint32_t h0k = 0; h0k < h_kv; h0k += HC) {
        if (h0k > 0) {
#pragma unroll
          for (uint32_t u = 0; u < HC; u++) {
            const bool on = h0k + u < h_kv;
            kl[u] = on ? ksrc[(h0k + u) * d + i] : 0.0f;
            kr[u] = on ? ksrc[(h0k + u) * d + pairs_total + i] : 0.0f;
          }
        }
#pragma unroll
        for (uint32_t u = 0; u < HC; u++) {
          const uint32_t h = h0k + u;
          if (h >= h_kv) break;
          kd[h * d + i] = __float2half_rn(rot ? kl[u] * cs - kr[u] * sn : kl[u]);
          kd[h * d + pairs_total + i] = __float2half_rn(rot ? kl[u] * sn + kr[u] * cs : kr[u]);
        }
      }
  }
  if (!bad)
    for (uint32_t i = threadIdx.x; i < h_kv * d; i += blockDim.x) vd[i] = __float2half_rn(vsrc[i]);
}

// The optional image operand of a producer step: null when absent.
int32_t resolve_out_image(const AionCudaOperand& op, uint32_t dtype, uint64_t rows, uint64_t cols, const char* name, uint8_t** out) {
  *out = nullptr;
  if (op.handle == 0) return AION_CUDA_OK;
  if (dtype != AION_CUDA_DTYPE_Q8_0 && dtype != AION_CUDA_DTYPE_Q4_0) return fail(AION_CUDA_INVALID_ARGUMENT, "%s: image dtype %u", name, dtype);
  if (cols % QK != 0) return fail(AION_CUDA_INVALID_ARGUMENT, "%s: an image needs rows of whole 32-blocks, got %llu columns", name, (unsigned long long)cols);
  if (rows > (1ull << 22) || cols > (1ull << 26) || rows * cols >= (1ull << 31)) return fail(AION_CUDA_UNSUPPORTED, "%s: shape beyond what the matmul kernels index", name);
  if (int32_t st = resolve(op, act_image_total_bytes(act_image_layout(rows, cols / QK)), name, out)) return st;
  if (reinterpret_cast<uintptr_t>(*out) & 15) return fail(AION_CUDA_INVALID_ARGUMENT, "%s: the image must be 16-byte aligned", name);
  return AION_CUDA_OK;
}

unsigned grid_for(const AionCudaDevice* dev, uint64_t n, unsigned threads) {
  const uint64_t want = ceil_div(n, (uint64_t)threads);
  const uint64_t cap = (uint64_t)dev->sm_count * 16;
  return (unsigned)(want < cap ? (want ? want : 1) : cap);
}

}  // namespace
}  // namespace aion

using namespace aion;

extern "C" {

int32_t aion_cuda_rms_norm(AionCudaDevice* dev, const AionCudaRMSNorm* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "rms_norm: null argument");
  if (!(s->eps > 0.0f) || !std::isfinite(s->eps)) return fail(AION_CUDA_INVALID_ARGUMENT, "rms_norm: eps must be finite and > 0");
  if (s->rows == 0 || s->cols == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  const size_t bytes = s->rows * s->cols * sizeof(float);
  float* out;
  const float *x, *gamma, *beta, *res = nullptr;
  if (int32_t st = resolve(s->out, bytes, "rms_norm.out", &out)) return st;
  if (int32_t st = resolve(s->x, bytes, "rms_norm.x", &x)) return st;
  if (int32_t st = resolve(s->gamma, s->cols * sizeof(float), "rms_norm.gamma", &gamma)) return st;
  if (int32_t st = resolve(s->beta, s->cols * sizeof(float), "rms_norm.beta", &beta)) return st;
  if (s->residual.handle)
    if (int32_t st = resolve(s->residual, bytes, "rms_norm.residual", &res)) return st;
  if (s->rows > 0x7FFFFFFFull) return fail(AION_CUDA_UNSUPPORTED, "rms_norm: too many rows for one launch");
  uint8_t* image;
  if (int32_t st = resolve_out_image(s->image, s->image_dtype, s->rows, s->cols, "rms_norm.image", &image)) return st;
  cudaError_t err = cudaSuccess;
  if (launch_rms_regs<false>(dev, &err, (unsigned)s->rows, out, nullptr, x, gamma, beta, res, nullptr, nullptr, s->cols, s->eps, s->eps, image,
                             s->image_dtype)) {
    AION_CUDA_TRY(err);
    return AION_CUDA_OK;
  }
  if (image) return fail(AION_CUDA_UNSUPPORTED, "rms_norm: an image needs rows of at most 4096 columns and 16-byte aligned operands");
  AION_CUDA_TRY(launch_pdl(rms_norm_kernel, dim3((unsigned)s->rows), dim3(RMS_THREADS), 0, dev->stream, out, x, gamma, beta, res, s->cols, s->eps,
                           dev->fault_dev));
  return AION_CUDA_OK;
}

int32_t aion_cuda_elemwise(AionCudaDevice* dev, const AionCudaElemwise* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "elemwise: null argument");
  if (s->op > AION_CUDA_ELEMWISE_GATE_GELU) return fail(AION_CUDA_INVALID_ARGUMENT, "elemwise: op %u", s->op);
  if (s->count == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  float* out;
  const float *a, *b;
  uint64_t cols = s->cols, ldo = 0, lda = 0, ldb = 0;
  size_t need_o = s->count * sizeof(float), need_a = need_o, need_b = need_o;
  if (cols) {
    if (s->count % cols != 0) return fail(AION_CUDA_INVALID_ARGUMENT, "elemwise: count is not a multiple of cols");
    const uint64_t rows = s->count / cols;
    ldo = s->ld_out ? s->ld_out : cols, lda = s->ld_a ? s->ld_a : cols, ldb = s->ld_b ? s->ld_b : cols;
    if (ldo < cols || lda < cols || ldb < cols) return fail(AION_CUDA_INVALID_ARGUMENT, "elemwise: a row stride is shorter than a row");
    need_o = ((rows - 1) * ldo + cols) * sizeof(float);
    need_a = ((rows - 1) * lda + cols) * sizeof(float);
    need_b = ((rows - 1) * ldb + cols) * sizeof(float);
    if (ldo == cols && lda == cols && ldb == cols) cols = 0;  // dense after all
  }
  if (int32_t st = resolve(s->out, need_o, "elemwise.out", &out)) return st;
  if (int32_t st = resolve(s->a, need_a, "elemwise.a", &a)) return st;
  if (int32_t st = resolve(s->b, need_b, "elemwise.b", &b)) return st;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b);
  if (s->image.handle) {
    // s->cols, not `cols`: a dense matrix still has rows for the image.
    const uint64_t icols = s->cols;
    if (icols == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "elemwise: an image needs cols > 0");
    const uint64_t rows = s->count / icols;
    uint8_t* image;
    if (int32_t st = resolve_out_image(s->image, s->image_dtype, rows, icols, "elemwise.image", &image)) return st;
    const uint64_t lo = ldo ? ldo : icols, la = lda ? lda : icols, lb = ldb ? ldb : icols;
    if ((bits & 15) != 0 || lo % 4 != 0 || la % 4 != 0 || lb % 4 != 0 || s->count / 4 > 0x7FFFFFFFull * 256)
      return fail(AION_CUDA_UNSUPPORTED, "elemwise: an image needs 16-byte aligned operands and row strides that are multiples of 4");
    const uint64_t n4 = s->count / 4;
    AION_CUDA_TRY(launch_pdl(elemwise4_image_kernel, dim3((unsigned)ceil_div(n4, (uint64_t)256)), dim3(256), 0, dev->stream,
                             reinterpret_cast<float4*>(out), reinterpret_cast<const float4*>(a), reinterpret_cast<const float4*>(b), n4, s->op,
                             (uint32_t)(icols / 4), lo / 4, la / 4, lb / 4, image, act_image_layout(rows, icols / QK), s->image_dtype));
    return AION_CUDA_OK;
  }
  // Float4s pay once the element-per-thread grid is saturated anyway (decode of 512 requests:
  // 11.11 -> 10.90 ms); on small steps they only make fewer, longer threads (16 requests:
  // 2.46 -> 2.61 ms), so those stay element by element.
  if (s->count >= (1ull << 20) && (bits & 15) == 0 && s->count % 4 == 0 && cols % 4 == 0 && ldo % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0) {
    AION_CUDA_TRY(launch_pdl(elemwise4_kernel, dim3(grid_for(dev, s->count / 4, 256)), dim3(256), 0, dev->stream, reinterpret_cast<float4*>(out),
                             reinterpret_cast<const float4*>(a), reinterpret_cast<const float4*>(b), s->count / 4, s->op, cols / 4, ldo / 4,
                             lda / 4, ldb / 4));
    return AION_CUDA_OK;
  }
  AION_CUDA_TRY(launch_pdl(elemwise_kernel, dim3(grid_for(dev, s->count, 256)), dim3(256), 0, dev->stream, out, a, b, s->count, s->op, cols,
                           ldo, lda, ldb));
  return AION_CUDA_OK;
}

int32_t aion_cuda_rope(AionCudaDevice* dev, const AionCudaRoPE* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "rope: null argument");
  if (s->head_dim % 2 != 0 || s->head_dim == 0 || s->head_dim > (1u << 20) || s->heads > (1u << 20))
    return fail(AION_CUDA_INVALID_ARGUMENT, "rope: head_dim = %llu", (unsigned long long)s->head_dim);
  const uint64_t bl = s->batch * s->len;
  if (bl == 0 || s->heads == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  // src/aion/backend/cpu/exec/rope.zig:43-50
  const uint64_t pairs_total = s->head_dim / 2;
  const float pf = std::floor(s->proportion * (float)pairs_total);
  if (!(pf >= 0.0f)) return fail(AION_CUDA_INVALID_ARGUMENT, "rope: proportion %g", (double)s->proportion);
  uint64_t rope_pairs = (uint64_t)pf;
  if (rope_pairs > pairs_total) rope_pairs = pairs_total;
  const float head_dim_f = (float)s->head_dim;
  const float step = (float)std::pow((double)s->base_frequency, (double)(-2.0f / head_dim_f));
  const size_t bytes = bl * s->heads * s->head_dim * sizeof(float);
  float* out;
  const float* x;
  const int32_t* pos;
  if (int32_t st = resolve(s->out, bytes, "rope.out", &out)) return st;
  if (int32_t st = resolve(s->x, bytes, "rope.x", &x)) return st;
  if (int32_t st = resolve(s->positions, bl * sizeof(int32_t), "rope.positions", &pos)) return st;
  const uint64_t threads = bl * pairs_total;
  AION_CUDA_TRY(launch_pdl(rope_kernel, dim3((unsigned)ceil_div(threads, (uint64_t)128)), dim3(128), 0, dev->stream, out, x, pos, bl,
                           (uint32_t)s->heads, (uint32_t)s->head_dim, (uint32_t)rope_pairs, step, s->scale_factor));
  return AION_CUDA_OK;
}

int32_t aion_cuda_cast(AionCudaDevice* dev, const AionCudaCast* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "cast: null argument");
  if (s->count == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  if (s->from_dtype == AION_CUDA_DTYPE_F32 && s->to_dtype == AION_CUDA_DTYPE_F16) {
    __half* out;
    const float* in;
    if (int32_t st = resolve(s->out, s->count * 2, "cast.out", &out)) return st;
    if (int32_t st = resolve(s->in, s->count * 4, "cast.in", &in)) return st;
    AION_CUDA_TRY(launch_pdl(cast_f32_f16_kernel, dim3(grid_for(dev, s->count, 256)), dim3(256), 0, dev->stream, out, in, s->count));
  } else if (s->from_dtype == AION_CUDA_DTYPE_F16 && s->to_dtype == AION_CUDA_DTYPE_F32) {
    float* out;
    const __half* in;
    if (int32_t st = resolve(s->out, s->count * 4, "cast.out", &out)) return st;
    if (int32_t st = resolve(s->in, s->count * 2, "cast.in", &in)) return st;
    AION_CUDA_TRY(launch_pdl(cast_f16_f32_kernel, dim3(grid_for(dev, s->count, 256)), dim3(256), 0, dev->stream, out, in, s->count));
  } else {
    return fail(AION_CUDA_UNSUPPORTED, "cast: only f32 <-> f16 is covered (got %u -> %u)", s->from_dtype, s->to_dtype);
  }
  AION_CUDA_TRY(cudaGetLastError());
  return AION_CUDA_OK;
}

int32_t aion_cuda_sequence_append(AionCudaDevice* dev, const AionCudaSequenceAppend* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "sequence_append: null argument");
  if (s->dtype != AION_CUDA_DTYPE_F16 && s->dtype != AION_CUDA_DTYPE_F32)
    return fail(AION_CUDA_INVALID_ARGUMENT, "sequence_append: cache dtype %u", s->dtype);
  if (s->batch == 0 || s->new_len == 0 || s->heads == 0 || s->head_dim == 0) return AION_CUDA_OK;
  if (s->t_cap == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "sequence_append: empty cache");
  if (int32_t st = dev->make_current()) return st;
  const size_t eb = s->dtype == AION_CUDA_DTYPE_F16 ? 2 : 4;
  const size_t row = s->heads * s->head_dim * eb;
  uint16_t* cache;
  const uint16_t* nk;
  const int32_t* idx;
  const int32_t* table = nullptr;
  uint64_t pages_per_request = 0, cache_rows = s->batch * s->t_cap;
  if (s->page_table.handle) {
    if (s->rolling) return fail(AION_CUDA_UNSUPPORTED, "sequence_append: a rolling cache cannot be paged");
    if (s->page_tokens == 0 || s->pool_pages == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "sequence_append: page_tokens and pool_pages must be positive");
    pages_per_request = (s->t_cap + s->page_tokens - 1) / s->page_tokens;
    cache_rows = s->pool_pages * s->page_tokens;
    if (int32_t st = resolve(s->page_table, s->batch * pages_per_request * sizeof(int32_t), "sequence_append.page_table", &table)) return st;
  }
  if (int32_t st = resolve(s->cache, cache_rows * row, "sequence_append.cache", &cache)) return st;
  if (int32_t st = resolve(s->new_kv, s->batch * s->new_len * row, "sequence_append.new_kv", &nk)) return st;
  if (int32_t st = resolve(s->end_index, s->batch * sizeof(int32_t), "sequence_append.end_index", &idx)) return st;
  if (s->batch * s->new_len > 0x7FFFFFFFull) return fail(AION_CUDA_UNSUPPORTED, "sequence_append: too many rows for one launch");
  AION_CUDA_TRY(launch_pdl(sequence_append_kernel, dim3((unsigned)(s->batch * s->new_len)), dim3(128), 0, dev->stream, cache, nk, idx,
                           s->t_cap, (uint64_t)(row / 2), s->new_len, s->rolling ? 1 : 0, dev->fault_dev, table, (uint64_t)s->page_tokens,
                           pages_per_request, (uint64_t)s->pool_pages));
  return AION_CUDA_OK;
}

int32_t aion_cuda_gather_rows(AionCudaDevice* dev, const AionCudaGatherRows* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "gather_rows: null argument");
  if (s->d % QK != 0) return fail(AION_CUDA_INVALID_ARGUMENT, "gather_rows: d = %llu is not a multiple of 32", (unsigned long long)s->d);
  int group = 1, chunk = 4;
  if (!block_order_info(s->block_order, &group, &chunk)) return fail(AION_CUDA_INVALID_ARGUMENT, "gather_rows: unknown block order %u", s->block_order);
  if (s->table_rows % (uint64_t)group != 0)
    return fail(AION_CUDA_INVALID_ARGUMENT, "gather_rows: %llu rows is not a multiple of the order's group of %d",
                (unsigned long long)s->table_rows, group);
  if (s->count == 0 || s->d == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  float* out;
  const uint8_t* table;
  const int32_t* idx;
  if (int32_t st = resolve(s->out, s->count * s->d * sizeof(float), "gather_rows.out", &out)) return st;
  if (int32_t st = resolve(s->table, s->table_rows * (s->d / QK) * Q8_BYTES, "gather_rows.table", &table)) return st;
  if (int32_t st = resolve(s->indices, s->count * sizeof(int32_t), "gather_rows.indices", &idx)) return st;
  if (s->count > 0x7FFFFFFFull) return fail(AION_CUDA_UNSUPPORTED, "gather_rows: too many rows for one launch");
  AION_CUDA_TRY(launch_pdl(gather_rows_q8_kernel, dim3((unsigned)s->count), dim3(256), 0, dev->stream, out, table, idx, s->table_rows,
                           s->d, group, chunk, dev->fault_dev));
  return AION_CUDA_OK;
}

int32_t aion_cuda_argmax(AionCudaDevice* dev, const AionCudaArgMax* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "argmax: null argument");
  if (s->n == 0 || s->n > 0x7FFFFFFEull) return fail(AION_CUDA_INVALID_ARGUMENT, "argmax: n = %llu", (unsigned long long)s->n);
  if (s->outer == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  int32_t* out;
  const float* in;
  if (int32_t st = resolve(s->out, s->outer * sizeof(int32_t), "argmax.out", &out)) return st;
  if (int32_t st = resolve(s->in, s->outer * s->n * sizeof(float), "argmax.in", &in)) return st;
  if (s->outer > 65535) return fail(AION_CUDA_UNSUPPORTED, "argmax: at most 65535 rows per launch, got %llu", (unsigned long long)s->outer);
  // Chunks of at least 4096 elements, enough of them for about eight blocks per SM (a block
  // is one pass of dependent loads, so many small blocks hide the latency better than few).
  uint64_t chunks = ceil_div(8ull * dev->sm_count, s->outer);
  const uint64_t max_chunks = ceil_div(s->n, (uint64_t)4096);
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  const uint64_t chunk_len = ceil_div(s->n, chunks);
  chunks = ceil_div(s->n, chunk_len);
  if (int32_t st = dev->reserve_scratch(s->outer * chunks * 8)) return st;
  if (int32_t st = dev->reserve_tickets(s->outer)) return st;
  float* cand_v = static_cast<float*>(dev->lane_scratch());
  int* cand_i = reinterpret_cast<int*>(cand_v + s->outer * chunks);
  AION_CUDA_TRY(launch_pdl(argmax_kernel, dim3((unsigned)chunks, (unsigned)s->outer), dim3(256), 0, dev->stream, out, in, s->n, chunk_len,
                           cand_v, cand_i, dev->lane_tickets()));
  return AION_CUDA_OK;
}

int32_t aion_cuda_rms_norm_pair(AionCudaDevice* dev, const AionCudaRMSNormPair* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "rms_norm_pair: null argument");
  if (!(s->eps1 > 0.0f) || !std::isfinite(s->eps1) || !(s->eps2 > 0.0f) || !std::isfinite(s->eps2))
    return fail(AION_CUDA_INVALID_ARGUMENT, "rms_norm_pair: eps must be finite and > 0");
  if (s->rows == 0 || s->cols == 0) return AION_CUDA_OK;
  if (s->rows > 0x7FFFFFFFull) return fail(AION_CUDA_UNSUPPORTED, "rms_norm_pair: too many rows for one launch");
  if (int32_t st = dev->make_current()) return st;
  const size_t bytes = s->rows * s->cols * sizeof(float), vec = s->cols * sizeof(float);
  float *out1, *out2;
  const float *x, *g1, *b1, *g2, *b2, *res = nullptr;
  if (int32_t st = resolve(s->out1, bytes, "rms_norm_pair.out1", &out1)) return st;
  if (int32_t st = resolve(s->out2, bytes, "rms_norm_pair.out2", &out2)) return st;
  if (int32_t st = resolve(s->x, bytes, "rms_norm_pair.x", &x)) return st;
  if (int32_t st = resolve(s->gamma1, vec, "rms_norm_pair.gamma1", &g1)) return st;
  if (int32_t st = resolve(s->beta1, vec, "rms_norm_pair.beta1", &b1)) return st;
  if (int32_t st = resolve(s->gamma2, vec, "rms_norm_pair.gamma2", &g2)) return st;
  if (int32_t st = resolve(s->beta2, vec, "rms_norm_pair.beta2", &b2)) return st;
  if (s->residual.handle)
    if (int32_t st = resolve(s->residual, bytes, "rms_norm_pair.residual", &res)) return st;
  uint8_t* image;
  if (int32_t st = resolve_out_image(s->image, s->image_dtype, s->rows, s->cols, "rms_norm_pair.image", &image)) return st;
  cudaError_t err = cudaSuccess;
  if (launch_rms_regs<true>(dev, &err, (unsigned)s->rows, out1, out2, x, g1, b1, res, g2, b2, s->cols, s->eps1, s->eps2, image, s->image_dtype)) {
    AION_CUDA_TRY(err);
    return AION_CUDA_OK;
  }
  if (image) return fail(AION_CUDA_UNSUPPORTED, "rms_norm_pair: an image needs rows of at most 4096 columns and 16-byte aligned operands");
  AION_CUDA_TRY(launch_pdl(rms_norm_pair_kernel, dim3((unsigned)s->rows), dim3(RMS_THREADS), 0, dev->stream, out1, out2, x, g1, b1, res, g2,
                           b2, s->cols, s->eps1, s->eps2, dev->fault_dev));
  return AION_CUDA_OK;
}

int32_t aion_cuda_rope_kv_append(AionCudaDevice* dev, const AionCudaRopeKVAppend* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "rope_kv_append: null argument");
  if (s->head_dim % 2 != 0 || s->head_dim == 0 || s->head_dim > (1u << 16) || s->h_q > (1u << 16) || s->h_kv > (1u << 16))
    return fail(AION_CUDA_INVALID_ARGUMENT, "rope_kv_append: head geometry");
  const uint64_t rows = s->batch * s->len;
  if (rows == 0) return AION_CUDA_OK;
  if (rows > 0x7FFFFFFFull || s->len > 0x7FFFFFFFull) return fail(AION_CUDA_UNSUPPORTED, "rope_kv_append: too many rows for one launch");
  if (s->t_cap == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "rope_kv_append: empty cache");
  const uint64_t width = (s->h_q + 2 * s->h_kv) * s->head_dim;
  const uint64_t ld = s->ld_qkv ? s->ld_qkv : width;
  if (ld < width) return fail(AION_CUDA_INVALID_ARGUMENT, "rope_kv_append: ld_qkv is shorter than q | k | v");
  if (int32_t st = dev->make_current()) return st;
  const uint64_t pairs_total = s->head_dim / 2;
  const float pf = std::floor(s->proportion * (float)pairs_total);
  if (!(pf >= 0.0f)) return fail(AION_CUDA_INVALID_ARGUMENT, "rope_kv_append: proportion %g", (double)s->proportion);
  uint64_t rope_pairs = (uint64_t)pf;
  if (rope_pairs > pairs_total) rope_pairs = pairs_total;
  const float head_dim_f = (float)s->head_dim;
  const float step = (float)std::pow((double)s->base_frequency, (double)(-2.0f / head_dim_f));
  float* q_out;
  const float* qkv;
  const int32_t *pos, *idx;
  __half *kc, *vc;
  const size_t cache_bytes = s->batch * s->t_cap * s->h_kv * s->head_dim * 2;
  if (int32_t st = resolve(s->q_out, rows * s->h_q * s->head_dim * sizeof(float), "rope_kv_append.q_out", &q_out)) return st;
  if (int32_t st = resolve(s->qkv, ((rows - 1) * ld + width) * sizeof(float), "rope_kv_append.qkv", &qkv)) return st;
  if (int32_t st = resolve(s->positions, rows * sizeof(int32_t), "rope_kv_append.positions", &pos)) return st;
  if (int32_t st = resolve(s->end_index, s->batch * sizeof(int32_t), "rope_kv_append.end_index", &idx)) return st;
  if (int32_t st = resolve(s->k_cache, cache_bytes, "rope_kv_append.k_cache", &kc)) return st;
  if (int32_t st = resolve(s->v_cache, cache_bytes, "rope_kv_append.v_cache", &vc)) return st;
  AION_CUDA_TRY(launch_pdl(rope_kv_append_kernel, dim3((unsigned)rows), dim3(128), 0, dev->stream, q_out, qkv, pos, idx, kc, vc,
                           (uint32_t)s->len, (uint32_t)s->h_q, (uint32_t)s->h_kv, (uint32_t)s->head_dim, ld, s->t_cap, (uint32_t)rope_pairs,
                           step, s->scale_factor, s->rolling ? 1 : 0, dev->fault_dev));
  return AION_CUDA_OK;
}

}  // extern "C"
