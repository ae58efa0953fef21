// CPU oracle for aion's quantized-matmul / attention hot path.
//
// TEST INFRASTRUCTURE ONLY. This file restates, in plain C++, the arithmetic of the
// reference's (RubyBit/aion, Zig) CPU kernels so that the CUDA library can be checked
// against it. Nothing in the shipped library links, loads or calls it; only the test
// suite, the smoke check and the benchmark's CPU-baseline leg do.
//
// The reference is Zig and cannot be compiled where this repository is built (no Zig
// toolchain), so this is a restatement ("port"), pinned by regenerating the reference's
// own in-file test fixtures (all of them formulas) and by hand-computed known answers;
// see tests/test_oracle_golden.py.
//
// Zig semantics honoured throughout:
//   @round            -> roundf (half away from zero)
//   @floatCast f32→f16 -> round to nearest even
//   @intFromFloat     -> truncation of an already-rounded, already-clamped value
//
// Each function cites the reference file:line it follows (paths relative to the
// reference project root).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kOk = 0;
constexpr int kInvalid = 1;
constexpr int kUnsupported = 3;

// AionDType codes (include/aion.h:70-77).
constexpr int DT_F32 = 0;
constexpr int DT_F16 = 1;
constexpr int DT_Q4_0 = 3;
constexpr int DT_Q8_0 = 4;

constexpr size_t Q8_BYTES = 34;  // src/aion/backend/types.zig:47
constexpr size_t Q4_BYTES = 18;  // src/aion/backend/types.zig:46
constexpr size_t QK = 32;

// ---------------------------------------------------------------------------------
// f16 <-> f32 (IEEE binary16, round to nearest even), bit level.
// ---------------------------------------------------------------------------------
inline uint16_t f32_to_f16_bits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7FFFFFFFu;
  if (x >= 0x7F800000u) {  // inf / nan
    return static_cast<uint16_t>(sign | 0x7C00u | ((x > 0x7F800000u) ? 0x200u : 0));
  }
  if (x >= 0x477FF000u) {  // rounds to >= 65520 -> inf
    return static_cast<uint16_t>(sign | 0x7C00u);
  }
  if (x < 0x33000001u) {  // < 2^-25 (or exactly 2^-25, ties to even -> 0)
    return static_cast<uint16_t>(sign);
  }
  const int32_t exp = static_cast<int32_t>(x >> 23) - 127;
  uint32_t mant = (x & 0x7FFFFFu) | 0x800000u;
  if (exp < -14) {  // subnormal half
    const int shift = -14 - exp + 13;  // 14..24
    const uint32_t half_ulp = 1u << (shift - 1);
    const uint32_t rem = mant & ((1u << shift) - 1);
    uint32_t m = mant >> shift;
    if (rem > half_ulp || (rem == half_ulp && (m & 1u))) m++;
    return static_cast<uint16_t>(sign | m);
  }
  uint32_t m = mant >> 13;
  const uint32_t rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (m & 1u))) m++;
  // m may have carried into bit 11; adding it to the exponent field handles that.
  const uint32_t h = (static_cast<uint32_t>(exp + 15 - 1) << 10) + m;
  return static_cast<uint16_t>(sign | h);
}

inline float f16_bits_to_f32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t mant = h & 0x3FFu;
  uint32_t out;
  if (exp == 0) {
    if (mant == 0) {
      out = sign;
    } else {
      int e = -1;
      do {
        mant <<= 1;
        e++;
      } while (!(mant & 0x400u));
      out = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((mant & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    out = sign | 0x7F800000u | (mant << 13);
  } else {
    out = sign | ((exp + 127 - 15) << 23) | (mant << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

inline uint16_t load_u16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
inline void store_u16(uint8_t* p, uint16_t v) {
  p[0] = static_cast<uint8_t>(v & 0xFF);
  p[1] = static_cast<uint8_t>(v >> 8);
}

// ---------------------------------------------------------------------------------
// Q1. Production q8_0 block packer: src/aion/storage/quantize.zig:81-103.
//   scale = absmax/127 (1 when the block is all zero), stored as f16; the codes are
//   chosen against the STORED scale: q = clamp(round(v * (1/f32(f16 scale))), -128, 127).
// ---------------------------------------------------------------------------------
void pack_q8_block(const float* values, size_t stride, uint8_t* dst) {
  float absmax = 0.0f;
  for (size_t t = 0; t < QK; t++) absmax = std::max(absmax, std::fabs(values[t * stride]));
  const float scale = (absmax == 0.0f) ? 1.0f : absmax / 127.0f;
  const uint16_t sbits = f32_to_f16_bits(scale);
  store_u16(dst, sbits);
  const float eff = f16_bits_to_f32(sbits);
  const float inv = (absmax == 0.0f || eff == 0.0f) ? 0.0f : 1.0f / eff;
  for (size_t t = 0; t < QK; t++) {
    const float r = std::round(values[t * stride] * inv);
    int32_t q = static_cast<int32_t>(r);
    q = std::max<int32_t>(-128, std::min<int32_t>(127, q));
    dst[2 + t] = static_cast<uint8_t>(static_cast<int8_t>(q));
  }
}

// ---------------------------------------------------------------------------------
// Q2. q4_0 block packer: src/aion/backend/cpu/test_cpu_kernels.zig:490-523
//   (same body at src/aion/backend/cpu/bench_cpu.zig:1916-1947).
//   scale = absmax/7 (1 when zero), stored f16; codes divide by the UNROUNDED f32
//   scale; nibble = q + 8; element t sits in byte t>>1, even t low nibble, odd t high.
// ---------------------------------------------------------------------------------
void pack_q4_block(const float* values, size_t stride, uint8_t* dst) {
  float absmax = 0.0f;
  for (size_t t = 0; t < QK; t++) absmax = std::max(absmax, std::fabs(values[t * stride]));
  const float scale = (absmax == 0.0f) ? 1.0f : absmax / 7.0f;
  store_u16(dst, f32_to_f16_bits(scale));
  for (size_t i = 0; i < 16; i++) dst[2 + i] = 0;
  for (size_t t = 0; t < QK; t++) {
    const float qf = values[t * stride] / scale;
    int32_t qi = static_cast<int32_t>(std::round(qf));
    qi = std::max<int32_t>(-8, std::min<int32_t>(7, qi));
    const uint8_t nib = static_cast<uint8_t>(qi + 8);
    uint8_t& b = dst[2 + (t >> 1)];
    if ((t & 1) == 0) b = static_cast<uint8_t>((b & 0xF0) | (nib & 0x0F));
    else b = static_cast<uint8_t>((b & 0x0F) | (nib << 4));
  }
}

// Nibble decode: src/aion/backend/cpu/kernels/matmul_q_i8.zig:362-369.
inline void unpack_block(int dtype, const uint8_t* blk, int8_t* out32) {
  if (dtype == DT_Q8_0) {
    for (size_t t = 0; t < QK; t++) out32[t] = static_cast<int8_t>(blk[2 + t]);
  } else {
    for (size_t t = 0; t < QK; t++) {
      const uint8_t byte = blk[2 + (t >> 1)];
      const uint8_t nib = ((t & 1) == 0) ? (byte & 0x0F) : (byte >> 4);
      out32[t] = static_cast<int8_t>(static_cast<int>(nib) - 8);
    }
  }
}

inline size_t block_bytes(int dtype) { return dtype == DT_Q8_0 ? Q8_BYTES : Q4_BYTES; }

// ---------------------------------------------------------------------------------
// A1. Activation block quantizer: src/aion/backend/cpu/kernels/matmul_q_i8.zig:187-203.
// ---------------------------------------------------------------------------------
inline float quantize_a_block(const float* a, int8_t* out) {
  float amax = 0.0f;
  for (size_t t = 0; t < QK; t++) amax = std::max(amax, std::fabs(a[t]));
  if (amax == 0.0f) {
    std::memset(out, 0, QK);
    return 0.0f;
  }
  const float scale = amax / 127.0f;
  const float inv = 127.0f / amax;
  for (size_t t = 0; t < QK; t++) {
    float r = std::round(a[t] * inv);
    r = std::max(-127.0f, std::min(127.0f, r));
    out[t] = static_cast<int8_t>(static_cast<int32_t>(r));
  }
  return scale;
}

// The folded four-lane block dot of the matvec / NT kernels, signed ("portable")
// semantics: src/aion/backend/cpu/kernels/matmul_q_i8.zig:213-227 (dotI8Narrow) on top
// of :143-151 (dotI8 .portable). Lane l holds elements 4l..4l+3 and 16+4l..16+4l+3.
inline void dot_narrow(const int8_t* a, const int8_t* b, int32_t lanes[4]) {
  for (int l = 0; l < 4; l++) {
    int32_t s = 0;
    for (int kk = 0; kk < 4; kk++) s += int32_t(a[4 * l + kk]) * int32_t(b[4 * l + kk]);
    for (int kk = 0; kk < 4; kk++) s += int32_t(a[16 + 4 * l + kk]) * int32_t(b[16 + 4 * l + kk]);
    lanes[l] = s;
  }
}

inline float reduce4(const float v[4]) {
  // Zig's @reduce(.Add) on a 4-lane vector lowers to a pairwise tree.
  return (v[0] + v[2]) + (v[1] + v[3]);
}

// Epilogue: src/aion/backend/cpu/kernels/matvec_q.zig:32-34.
inline float store_dot(float c_old, float alpha, float beta, float dot) {
  return beta == 0.0f ? alpha * dot : alpha * dot + beta * c_old;
}

// ---------------------------------------------------------------------------------
// M1. q8_0 K-major matvec (m <= 16): src/aion/backend/cpu/kernels/matvec_q.zig:62-160.
//   Row by row; A quantized in chunks of 8192 K; the first chunk stores through
//   alpha/beta, later chunks add alpha*dot.
// ---------------------------------------------------------------------------------
void matvec_q8_kmajor(size_t m, size_t n, size_t k, size_t lda, size_t ldb, size_t ldc, float alpha,
                      float beta, float* c, const float* a, const uint8_t* b) {
  const size_t blocks = k / QK;
  const size_t chunk_blocks = 8192 / QK;
  std::vector<int8_t> aq(chunk_blocks * QK);
  std::vector<float> ascale(chunk_blocks);
  for (size_t r = 0; r < m; r++) {
    for (size_t kb0 = 0; kb0 < blocks; kb0 += chunk_blocks) {
      const size_t nb = std::min(chunk_blocks, blocks - kb0);
      for (size_t kb = 0; kb < nb; kb++)
        ascale[kb] = quantize_a_block(a + r * lda + (kb0 + kb) * QK, aq.data() + kb * QK);
      const bool first = kb0 == 0;
      for (size_t j = 0; j < n; j++) {
        float acc[4] = {0, 0, 0, 0};
        for (size_t kb = 0; kb < nb; kb++) {
          const uint8_t* bp = b + ((kb0 + kb) * ldb + j) * Q8_BYTES;
          const float bs = f16_bits_to_f32(load_u16(bp));
          int32_t lanes[4];
          dot_narrow(reinterpret_cast<const int8_t*>(bp + 2), aq.data() + kb * QK, lanes);
          const float s = ascale[kb] * bs;
          for (int l = 0; l < 4; l++) acc[l] += float(lanes[l]) * s;
        }
        const float dot = reduce4(acc);
        float& cc = c[r * ldc + j];
        if (first) cc = store_dot(cc, alpha, beta, dot);
        else cc += alpha * dot;
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// M3. Packed int8 GEMM for q8_0 / q4_0 K-major weights:
//   src/aion/backend/cpu/kernels/matmul_q_i8.zig:385-497 (matmulPackedB) driven by
//   src/aion/backend/cpu/exec/matmul.zig:423-463 (gemmTask): K is walked in `kc`
//   chunks; the first applies (alpha, beta), later ones (alpha, 1). Within a chunk:
//   cacc += float(dot) * b_scale * a_scale over kb, then c = alpha*cacc (+ beta*c).
//   The panel/column tiling does not change any value, so it is not restated.
// ---------------------------------------------------------------------------------
void matmul_packed(int dtype, size_t m, size_t n, size_t k, size_t lda, size_t ldb, size_t ldc,
                   float alpha, float beta, float* c, const float* a, const uint8_t* b, size_t kc) {
  const size_t bb = block_bytes(dtype);
  const size_t kcb = kc / QK;
  const size_t blocks = k / QK;
  std::vector<int8_t> aq(blocks * QK);
  std::vector<float> ascale(blocks);
  int8_t wq[QK];
  for (size_t r = 0; r < m; r++) {
    for (size_t kb = 0; kb < blocks; kb++)
      ascale[kb] = quantize_a_block(a + r * lda + kb * QK, aq.data() + kb * QK);
    for (size_t j = 0; j < n; j++) {
      float& cc = c[r * ldc + j];
      for (size_t kb0 = 0; kb0 < blocks; kb0 += kcb) {
        const size_t nb = std::min(kcb, blocks - kb0);
        float cacc = 0.0f;
        for (size_t kb = kb0; kb < kb0 + nb; kb++) {
          const uint8_t* bp = b + (kb * ldb + j) * bb;
          unpack_block(dtype, bp, wq);
          int32_t dot = 0;
          for (size_t t = 0; t < QK; t++) dot += int32_t(aq[kb * QK + t]) * int32_t(wq[t]);
          cacc += float(dot) * f16_bits_to_f32(load_u16(bp)) * ascale[kb];
        }
        const float bt = (kb0 == 0) ? beta : 1.0f;
        const float out = cacc * alpha;
        cc = (bt == 0.0f) ? out : out + bt * cc;
      }
    }
  }
}

// QuantBlockOrder byte placement: src/aion/backend/types.zig:140-223.
struct BlockOrder {
  size_t group_rows;
  size_t chunk_bytes;
};
bool order_info(int order, BlockOrder* o) {
  switch (order) {
    case 0: *o = {1, 4}; return true;    // row_major
    case 1: *o = {4, 4}; return true;    // lanes4
    case 2: *o = {8, 4}; return true;    // lanes8
    case 3: *o = {16, 4}; return true;   // lanes16
    case 4: *o = {32, 4}; return true;   // lanes32
    case 5: *o = {32, 16}; return true;  // lanes32x16
    default: return false;
  }
}
inline size_t seg_off(const BlockOrder& o, size_t blocks, size_t r, size_t kb) {
  return ((r / o.group_rows) * blocks + kb) * o.group_rows * Q8_BYTES;
}
inline size_t scale_at(const BlockOrder& o, size_t blocks, size_t r, size_t kb) {
  return seg_off(o, blocks, r, kb) + (r % o.group_rows) * 2;
}
inline size_t chunk_at(const BlockOrder& o, size_t blocks, size_t r, size_t kb, size_t chunk) {
  return seg_off(o, blocks, r, kb) + 2 * o.group_rows +
         (chunk * o.group_rows + r % o.group_rows) * o.chunk_bytes;
}
void load_block(const BlockOrder& o, const uint8_t* bytes, size_t blocks, size_t r, size_t kb,
                uint8_t* block) {
  std::memcpy(block, bytes + scale_at(o, blocks, r, kb), 2);
  for (size_t ch = 0; ch < 32 / o.chunk_bytes; ch++)
    std::memcpy(block + 2 + ch * o.chunk_bytes, bytes + chunk_at(o, blocks, r, kb, ch), o.chunk_bytes);
}
void store_block(const BlockOrder& o, uint8_t* bytes, size_t blocks, size_t r, size_t kb,
                 const uint8_t* block) {
  std::memcpy(bytes + scale_at(o, blocks, r, kb), block, 2);
  for (size_t ch = 0; ch < 32 / o.chunk_bytes; ch++)
    std::memcpy(bytes + chunk_at(o, blocks, r, kb, ch), block + 2 + ch * o.chunk_bytes, o.chunk_bytes);
}

// ---------------------------------------------------------------------------------
// T3. expApprox / tanhApprox / expSoftmax:
//   src/aion/backend/cpu/kernels/fast_math.zig:53-92, 108-141;
//   src/aion/backend/cpu/kernels/attention.zig:42-48.
// ---------------------------------------------------------------------------------
inline float clampf(float x, float lo, float hi) { return std::max(lo, std::min(hi, x)); }
inline float exp_approx(float x_in) {
  const float x = clampf(x_in, -80.0f, 80.0f);
  const float inv_ln2 = 1.4426950408889634f;
  const float ln2 = 0.6931471805599453f;
  const float y = x * inv_ln2;
  const int32_t n = static_cast<int32_t>(std::floor(y + 0.5f));
  const float r = y - static_cast<float>(n);
  const float t = r * ln2;
  const float c4 = 1.0f / 24.0f, c3 = 1.0f / 6.0f, c2 = 0.5f;
  const float poly = 1.0f + t * (1.0f + t * (c2 + t * (c3 + t * c4)));
  const uint32_t bits = static_cast<uint32_t>(n + 127) << 23;
  float p2;
  std::memcpy(&p2, &bits, 4);
  return p2 * poly;
}
inline float sigmoid_approx(float x) {
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
inline float tanh_approx(float x) { return clampf(2.0f * sigmoid_approx(2.0f * x) - 1.0f, -1.0f, 1.0f); }
inline float exp_softmax(float x) {
  if (!std::isfinite(x)) return x < 0.0f ? 0.0f : std::numeric_limits<float>::infinity();
  return exp_approx(clampf(x, -20.0f, 0.0f));
}

inline float load_elem(const void* p, int dtype, size_t idx) {
  if (dtype == DT_F32) return static_cast<const float*>(p)[idx];
  return f16_bits_to_f32(static_cast<const uint16_t*>(p)[idx]);
}

// Row dot with four independent 8-lane FMA chains:
// src/aion/backend/cpu/exec/attention.zig:202-236 (dotRowsTyped), at the 8-lane width.
float dot_rows(const void* a, int adt, size_t aoff, const void* b, int bdt, size_t boff, size_t n) {
  constexpr size_t L = 8, CH = 4;
  float acc[CH][L] = {};
  size_t i = 0;
  for (; i + L * CH <= n; i += L * CH)
    for (size_t c = 0; c < CH; c++)
      for (size_t l = 0; l < L; l++) {
        const size_t off = i + c * L + l;
        acc[c][l] = std::fmaf(load_elem(a, adt, aoff + off), load_elem(b, bdt, boff + off), acc[c][l]);
      }
  for (; i + L <= n; i += L)
    for (size_t l = 0; l < L; l++)
      acc[0][l] = std::fmaf(load_elem(a, adt, aoff + i + l), load_elem(b, bdt, boff + i + l), acc[0][l]);
  float tot[L];
  for (size_t l = 0; l < L; l++) {
    tot[l] = acc[0][l];
    for (size_t c = 1; c < CH; c++) tot[l] += acc[c][l];
  }
  float sum = ((tot[0] + tot[4]) + (tot[2] + tot[6])) + ((tot[1] + tot[5]) + (tot[3] + tot[7]));
  for (; i < n; i++) sum += load_elem(a, adt, aoff + i) * load_elem(b, bdt, boff + i);
  return sum;
}

}  // namespace

// =================================================================================
// Exported entry points (C ABI, for ctypes).
// =================================================================================

ORC_API uint16_t aion_oracle_f32_to_f16(float f) { return f32_to_f16_bits(f); }
ORC_API float aion_oracle_f16_to_f32(uint16_t h) { return f16_bits_to_f32(h); }
ORC_API float aion_oracle_exp_approx(float x) { return exp_approx(x); }
ORC_API float aion_oracle_tanh_approx(float x) { return tanh_approx(x); }

// Quantize a row-major f32 tensor of `shape[rank]` along `quant_axis` into packed
// blocks, row-major over the block-space shape: src/aion/storage/quantize.zig:31-79.
// dtype q8_0 uses the production packer (Q1); q4_0 uses the reference's q4 helper (Q2)
// under the same placement rule (which for [K,N] axis 0 is buildQuantB_Q4_0,
// src/aion/backend/cpu/bench_cpu.zig:1980-2006).
ORC_API int aion_oracle_quantize(int dtype, const float* values, const uint64_t* shape, int rank,
                                 int quant_axis, uint8_t* out) {
  if (dtype != DT_Q8_0 && dtype != DT_Q4_0) return kUnsupported;
  if (rank <= 0 || rank > 8 || quant_axis < 0 || quant_axis >= rank) return kInvalid;
  if (shape[quant_axis] % QK != 0) return kInvalid;
  size_t strides[8], bshape[8];
  size_t s = 1, nblocks = 1;
  for (int d = rank - 1; d >= 0; d--) {
    strides[d] = s;
    s *= shape[d];
    bshape[d] = (d == quant_axis) ? shape[d] / QK : shape[d];
    nblocks *= bshape[d];
  }
  const size_t bb = block_bytes(dtype);
  for (size_t i = 0; i < nblocks; i++) {
    size_t rest = i, base = 0;
    for (int d = rank - 1; d >= 0; d--) {
      const size_t cidx = rest % bshape[d];
      rest /= bshape[d];
      base += ((d == quant_axis) ? cidx * QK : cidx) * strides[d];
    }
    if (dtype == DT_Q8_0) pack_q8_block(values + base, strides[quant_axis], out + i * bb);
    else pack_q4_block(values + base, strides[quant_axis], out + i * bb);
  }
  return kOk;
}

// Dequantize `nblocks` consecutive blocks: w = f32(q) * f32(f16 scale)
// (src/aion/backend/cpu/kernels/matmul_q_i8.zig:847-862; nibble decode :362-369).
ORC_API int aion_oracle_dequant(int dtype, const uint8_t* blocks, uint64_t nblocks, float* out) {
  if (dtype != DT_Q8_0 && dtype != DT_Q4_0) return kUnsupported;
  const size_t bb = block_bytes(dtype);
  int8_t q[QK];
  for (size_t i = 0; i < nblocks; i++) {
    const float sc = f16_bits_to_f32(load_u16(blocks + i * bb));
    unpack_block(dtype, blocks + i * bb, q);
    for (size_t t = 0; t < QK; t++) out[i * QK + t] = float(q[t]) * sc;
  }
  return kOk;
}

// Re-lay a row-major [n, k] q8_0 tensor into `order` (or back, when `inverse`):
// src/aion/backend/types.zig:206-222; driver src/aion/graph/opt/weight_layout.zig:243-314.
// n must be a multiple of the order's group.
ORC_API int aion_oracle_relayout_q8(int order, int inverse, uint64_t n, uint64_t k, const uint8_t* src,
                                    uint8_t* dst) {
  BlockOrder o, rm = {1, 4};
  if (!order_info(order, &o) || k % QK != 0 || n % o.group_rows != 0) return kInvalid;
  const size_t blocks = k / QK;
  uint8_t blk[Q8_BYTES];
  for (size_t r = 0; r < n; r++)
    for (size_t kb = 0; kb < blocks; kb++) {
      if (!inverse) {
        load_block(rm, src, blocks, r, kb, blk);
        store_block(o, dst, blocks, r, kb, blk);
      } else {
        load_block(o, src, blocks, r, kb, blk);
        store_block(rm, dst, blocks, r, kb, blk);
      }
    }
  return kOk;
}

// A1 exported: quantize K (multiple of 32) activations; out_q[K], out_scale[K/32].
ORC_API int aion_oracle_quantize_activation(const float* a, uint64_t k, int8_t* out_q, float* out_scale) {
  if (k % QK != 0) return kInvalid;
  for (size_t kb = 0; kb < k / QK; kb++) out_scale[kb] = quantize_a_block(a + kb * QK, out_q + kb * QK);
  return kOk;
}

// `MatMul` step with a K-major quantized B ([K/32][ldb] blocks), reference CPU
// arithmetic (int8 activations). route: 0 = the reference's own routing
// (src/aion/backend/cpu/exec/matmul.zig:233-239: q8 with m <= 16 takes the direct
// matvec, everything else the packed GEMM), 1 = force matvec (q8 only), 2 = force
// packed. kc = K chunk of the packed path (the reference's medium tile is 256,
// src/aion/backend/cpu/registry/matmul_q_registry.zig:62-64).
ORC_API int aion_oracle_matmul_q(int dtype, uint64_t m, uint64_t n, uint64_t k, uint64_t lda, uint64_t ldb,
                                 uint64_t ldc, float alpha, float beta, float* c, const float* a,
                                 const uint8_t* b, int route, uint64_t kc) {
  if (dtype != DT_Q8_0 && dtype != DT_Q4_0) return kUnsupported;
  if (k % QK != 0) return kInvalid;
  if (lda == 0) lda = k;
  if (ldb == 0) ldb = n;
  if (ldc == 0) ldc = n;
  if (kc == 0) kc = 256;
  if (kc % QK != 0) return kInvalid;
  if (m == 0 || n == 0) return kOk;
  bool matvec = (dtype == DT_Q8_0 && m <= 16);
  if (route == 1) {
    if (dtype != DT_Q8_0) return kUnsupported;
    matvec = true;
  } else if (route == 2) {
    matvec = false;
  }
  if (matvec) matvec_q8_kmajor(m, n, k, lda, ldb, ldc, alpha, beta, c, a, b);
  else matmul_packed(dtype, m, n, k, lda, ldb, ldc, alpha, beta, c, a, b, kc);
  return kOk;
}

// `MatMulNT` step: C[m,n] = alpha * sum_k A[m,k] B[n,k] + beta C with B q8_0 [n,k] in any
// QuantBlockOrder. src/aion/backend/cpu/kernels/matmul_nt_q.zig:74-95 (row-major: four
// f32 lanes per output, block by block, then a horizontal add) and :173-216 (grouped:
// one f32 sum per output, float(dot) * b_scale * a_scale).
ORC_API int aion_oracle_matmul_nt_q8(int order, uint64_t m, uint64_t n, uint64_t k, uint64_t lda,
                                     uint64_t ldc, float alpha, float beta, float* c, const float* a,
                                     const uint8_t* b) {
  BlockOrder o;
  if (!order_info(order, &o) || k % QK != 0) return kInvalid;
  if (lda == 0) lda = k;
  if (ldc == 0) ldc = n;
  const size_t blocks = k / QK;
  std::vector<int8_t> aq(blocks * QK);
  std::vector<float> ascale(blocks);
  uint8_t blk[Q8_BYTES];
  for (size_t r = 0; r < m; r++) {
    for (size_t kb = 0; kb < blocks; kb++)
      ascale[kb] = quantize_a_block(a + r * lda + kb * QK, aq.data() + kb * QK);
    for (size_t j = 0; j < n; j++) {
      float dot;
      // A row outside a whole group is read row-major by the reference's tail path;
      // the layout contract requires n % group == 0, so that case is not reachable.
      if (o.group_rows == 1) {
        float acc[4] = {0, 0, 0, 0};
        for (size_t kb = 0; kb < blocks; kb++) {
          load_block(o, b, blocks, j, kb, blk);
          int32_t lanes[4];
          dot_narrow(reinterpret_cast<const int8_t*>(blk + 2), aq.data() + kb * QK, lanes);
          const float s = ascale[kb] * f16_bits_to_f32(load_u16(blk));
          for (int l = 0; l < 4; l++) acc[l] += float(lanes[l]) * s;
        }
        dot = reduce4(acc);
      } else {
        float acc = 0.0f;
        for (size_t kb = 0; kb < blocks; kb++) {
          load_block(o, b, blocks, j, kb, blk);
          int32_t d = 0;
          for (size_t t = 0; t < QK; t++) d += int32_t(static_cast<int8_t>(blk[2 + t])) * int32_t(aq[kb * QK + t]);
          acc += float(d) * f16_bits_to_f32(load_u16(blk)) * ascale[kb];
        }
        dot = acc;
      }
      float& cc = c[r * ldc + j];
      cc = store_dot(cc, alpha, beta, dot);
    }
  }
  return kOk;
}

// f32 activation x dequant(B), f32 accumulate in K order: the host reference of the
// reference's GPU tests (src/aion/backend/gpu/test_gpu_backend.zig:1325-1341).
// nt = 0: B K-major [K/32][ldb]; nt = 1: B row-major [n][K/32] (q8_0 or q4_0 bytes).
ORC_API int aion_oracle_matmul_deqf32(int dtype, int nt, uint64_t m, uint64_t n, uint64_t k, uint64_t lda,
                                      uint64_t ldb, uint64_t ldc, float alpha, float beta, float* c,
                                      const float* a, const uint8_t* b) {
  if (dtype != DT_Q8_0 && dtype != DT_Q4_0) return kUnsupported;
  if (k % QK != 0) return kInvalid;
  if (lda == 0) lda = k;
  if (ldb == 0) ldb = nt ? k / QK : n;
  if (ldc == 0) ldc = n;
  const size_t bb = block_bytes(dtype);
  int8_t q[QK];
  for (size_t r = 0; r < m; r++)
    for (size_t j = 0; j < n; j++) {
      float acc = 0.0f;
      for (size_t kb = 0; kb < k / QK; kb++) {
        const uint8_t* bp = b + (nt ? (j * ldb + kb) : (kb * ldb + j)) * bb;
        const float sc = f16_bits_to_f32(load_u16(bp));
        unpack_block(dtype, bp, q);
        for (size_t t = 0; t < QK; t++) acc += a[r * lda + kb * QK + t] * (float(q[t]) * sc);
      }
      float& cc = c[r * ldc + j];
      cc = store_dot(cc, alpha, beta, acc);
    }
  return kOk;
}

// `Attention` step, the generic per-row executor:
// src/aion/backend/cpu/exec/attention.zig:1025-1318. One output row per (b, l, hq);
// key range from the window (src/aion/graph/graph.zig:160-167) clipped by the ring's
// retained span; <= 2048 keys: two-pass softmax, else per-key online softmax.
// q [B,L,Hq,Dk], k [B,T,Hkv,Dk], v [B,T,Hkv,Dv], out f32 [B,L,Hq,Dv].
// positions [B,L] / kv_lengths [B] may be null (position = row; length = T).
// exact != 0 replaces expSoftmax/tanhApprox by f64 exp/tanh with f64 accumulation
// (a mathematical reference, not the reference CPU's arithmetic).
// Returns 1 (InvalidArgument) where the reference fails the step.
ORC_API int aion_oracle_attention(float* out, const void* q, int q_dtype, const void* k, int k_dtype,
                                  const void* v, int v_dtype, const int32_t* positions,
                                  const int32_t* kv_lengths, uint64_t B, uint64_t L, uint64_t Hq,
                                  uint64_t Hkv, uint64_t Dk, uint64_t Dv, uint64_t T, float scale,
                                  uint32_t win_left, uint32_t win_right, uint32_t win_chunk,
                                  float soft_cap, int rolling, int exact) {
  if (!(scale > 0.0f) || !std::isfinite(scale)) return kInvalid;
  if (!std::isfinite(soft_cap) || soft_cap < 0.0f) return kInvalid;
  if (Hkv == 0 || Hq == 0 || Hq % Hkv != 0 || T == 0) return kInvalid;
  for (int dt : {q_dtype, k_dtype, v_dtype})
    if (dt != DT_F32 && dt != DT_F16) return kInvalid;
  const size_t g = Hq / Hkv;
  std::vector<float> logits;
  std::vector<double> acc64(Dv);
  for (size_t b = 0; b < B; b++) {
    size_t valid_end = T;
    if (kv_lengths) {
      if (kv_lengths[b] < 0) return kInvalid;
      valid_end = static_cast<size_t>(kv_lengths[b]);
    }
    if (!rolling && valid_end > T) return kInvalid;
    const size_t avail_start = (rolling && valid_end > T) ? valid_end - T : 0;
    for (size_t l = 0; l < L; l++) {
      size_t q_pos = l;
      if (positions) {
        if (positions[b * L + l] < 0) return kInvalid;
        q_pos = static_cast<size_t>(positions[b * L + l]);
      }
      const size_t anchor = win_chunk > 0 ? (q_pos / win_chunk) * win_chunk : q_pos;
      const size_t span = win_chunk > 0 ? win_chunk : 1;
      const size_t lo_w = anchor - std::min<size_t>(anchor, win_left);
      // Saturating adds in the reference; uint64 cannot overflow with u32 terms here.
      const size_t hi_w = std::min<size_t>(valid_end, anchor + span + static_cast<size_t>(win_right));
      const size_t lower = std::max(lo_w, avail_start);
      const size_t upper = hi_w;
      for (size_t hq = 0; hq < Hq; hq++) {
        float* orow = out + ((b * L + l) * Hq + hq) * Dv;
        for (size_t i = 0; i < Dv; i++) orow[i] = 0.0f;
        if (lower >= upper) continue;
        const size_t hkv = hq / g;
        const size_t qoff = ((b * L + l) * Hq + hq) * Dk;
        const size_t n_keys = upper - lower;
        auto phys = [&](size_t t) { return rolling ? t % T : t; };
        auto logit_of = [&](size_t t) {
          const size_t koff = ((b * T + phys(t)) * Hkv + hkv) * Dk;
          float lg = dot_rows(q, q_dtype, qoff, k, k_dtype, koff, Dk) * scale;
          if (soft_cap > 0.0f) {
            if (exact) lg = soft_cap * static_cast<float>(std::tanh(double(lg) / double(soft_cap)));
            else lg = soft_cap * tanh_approx(lg / soft_cap);
          }
          return lg;
        };
        if (exact) {
          logits.resize(n_keys);
          double mx = -std::numeric_limits<double>::infinity();
          for (size_t i = 0; i < n_keys; i++) {
            logits[i] = logit_of(lower + i);
            mx = std::max(mx, double(logits[i]));
          }
          double lsum = 0.0;
          std::fill(acc64.begin(), acc64.end(), 0.0);
          for (size_t i = 0; i < n_keys; i++) {
            const double p = std::exp(double(logits[i]) - mx);
            lsum += p;
            const size_t voff = ((b * T + phys(lower + i)) * Hkv + hkv) * Dv;
            for (size_t d = 0; d < Dv; d++) acc64[d] += p * double(load_elem(v, v_dtype, voff + d));
          }
          for (size_t d = 0; d < Dv; d++) orow[d] = static_cast<float>(acc64[d] / lsum);
          continue;
        }
        if (n_keys <= 2048) {
          logits.resize(n_keys);
          float m_state = -std::numeric_limits<float>::infinity();
          for (size_t i = 0; i < n_keys; i++) {
            if (!rolling && lower + i >= T) return kInvalid;
            logits[i] = logit_of(lower + i);
            m_state = std::max(m_state, logits[i]);
          }
          float l_state = 0.0f;
          for (size_t i = 0; i < n_keys; i++) {
            const float p = exp_softmax(logits[i] - m_state);
            logits[i] = p;
            l_state += p;
          }
          if (!(l_state > 0.0f) || !std::isfinite(l_state)) return kInvalid;
          const float inv = 1.0f / l_state;
          for (size_t i = 0; i < n_keys; i++) {
            const float alpha = logits[i] * inv;
            const size_t voff = ((b * T + phys(lower + i)) * Hkv + hkv) * Dv;
            for (size_t d = 0; d < Dv; d++) orow[d] += load_elem(v, v_dtype, voff + d) * alpha;
          }
        } else {
          float m_state = -std::numeric_limits<float>::infinity();
          float l_state = 0.0f;
          for (size_t t = lower; t < upper; t++) {
            if (!rolling && t >= T) return kInvalid;
            const float lg = logit_of(t);
            const float m_new = std::max(m_state, lg);
            const float rescale =
                (m_state == -std::numeric_limits<float>::infinity()) ? 0.0f : exp_softmax(m_state - m_new);
            const float p_new = exp_softmax(lg - m_new);
            const size_t voff = ((b * T + phys(t)) * Hkv + hkv) * Dv;
            for (size_t d = 0; d < Dv; d++)
              orow[d] = orow[d] * rescale + load_elem(v, v_dtype, voff + d) * p_new;
            l_state = l_state * rescale + p_new;
            m_state = m_new;
          }
          if (!(l_state > 0.0f) || !std::isfinite(l_state)) return kInvalid;
          const float inv = 1.0f / l_state;
          for (size_t d = 0; d < Dv; d++) orow[d] *= inv;
        }
      }
    }
  }
  return kOk;
}

// =================================================================================
// Decoder glue steps (the ops either side of the matmul / attention path).
// =================================================================================

// RMSNorm with optional residual: src/aion/backend/cpu/exec/layernorm.zig:41-154 and
// src/aion/backend/cpu/kernels/layernorm.zig:7-107. Sum of squares in 16 lane partials
// (the f32 vector width of a 512-bit host) reduced pairwise, tail added serially;
// inv = 1 / sqrt(mean(x^2) + eps); out = (x * inv) * gamma + beta, then + residual.
ORC_API int aion_oracle_rms_norm(float* out, const float* x, const float* gamma, const float* beta, const float* residual,
                                 uint64_t rows, uint64_t cols, float eps) {
  if (!(eps > 0.0f) || !std::isfinite(eps) || cols == 0) return kInvalid;
  const size_t lanes = 16;
  const float inv_denom = 1.0f / static_cast<float>(cols);
  for (uint64_t r = 0; r < rows; r++) {
    const float* xr = x + r * cols;
    float part[16] = {0};
    size_t c = 0;
    const size_t vec_end = cols - (cols % lanes);
    for (; c < vec_end; c += lanes)
      for (size_t l = 0; l < lanes; l++) part[l] += xr[c + l] * xr[c + l];
    for (size_t w = lanes / 2; w > 0; w /= 2)
      for (size_t l = 0; l < w; l++) part[l] += part[l + w];
    float sq = part[0];
    for (; c < cols; c++) sq += xr[c] * xr[c];
    const float d = sq * inv_denom + eps;
    if (!(d > 0.0f) || !std::isfinite(d)) return kInvalid;
    const float inv = 1.0f / std::sqrt(d);
    for (size_t j = 0; j < cols; j++) {
      float v = ((xr[j] * inv) * gamma[j]) + beta[j];
      if (residual) v = v + residual[r * cols + j];
      out[r * cols + j] = v;
    }
  }
  return kOk;
}

// GELU (tanh form over tanhApprox): src/aion/backend/cpu/kernels/gelu.zig:8-14.
inline float gelu_approx(float x) {
  const float c = 0.044715f, k = 0.7978845608028654f;
  const float x3 = x * x * x;
  const float t = k * (x + c * x3);
  return 0.5f * x * (1.0f + tanh_approx(t));
}
// op 0: a + b, 1: a * b, 2: gate = gelu(a) * b (src/aion/backend/cpu/exec/elementwise.zig:25-36).
ORC_API int aion_oracle_elemwise(int op, float* out, const float* a, const float* b, uint64_t n) {
  for (uint64_t i = 0; i < n; i++) {
    switch (op) {
      case 0: out[i] = a[i] + b[i]; break;
      case 1: out[i] = a[i] * b[i]; break;
      case 2: out[i] = gelu_approx(a[i]) * b[i]; break;
      default: return kInvalid;
    }
  }
  return kOk;
}

// RoPE1D over [B, L, H, D] f32 with positions i32 [B, L]:
// src/aion/backend/cpu/exec/rope.zig:43-50 and src/aion/backend/cpu/kernels/rope.zig:20-97.
// Pair i is (x[i], x[D/2 + i]); its frequency is scale * step^i by repeated f32 multiplies,
// step = f32(base^(-2/D)) computed in f64; sin / cos in f64 of the f32 angle.
ORC_API int aion_oracle_rope(float* out, const float* x, const int32_t* pos, uint64_t b, uint64_t l, uint64_t h, uint64_t d,
                             float base_frequency, float scale_factor, float proportion) {
  if (d % 2 != 0) return kInvalid;
  const size_t pairs_total = d / 2;
  const float pf = std::floor(proportion * static_cast<float>(pairs_total));
  if (pf < 0.0f) return kInvalid;
  size_t rope_pairs = static_cast<size_t>(pf);
  if (rope_pairs > pairs_total) rope_pairs = pairs_total;
  const float head_dim_f = static_cast<float>(d);
  const float step = static_cast<float>(std::pow(static_cast<double>(base_frequency), static_cast<double>(-2.0f / head_dim_f)));
  for (uint64_t bl = 0; bl < b * l; bl++) {
    const float p = static_cast<float>(pos[bl]);
    for (uint64_t hh = 0; hh < h; hh++) {
      const float* xr = x + (bl * h + hh) * d;
      float* orow = out + (bl * h + hh) * d;
      std::memcpy(orow, xr, d * sizeof(float));
      float f = scale_factor;
      for (size_t i = 0; i < rope_pairs; i++) {
        const float ang = p * f;
        const float sn = static_cast<float>(std::sin(static_cast<double>(ang)));
        const float cs = static_cast<float>(std::cos(static_cast<double>(ang)));
        const float xl = xr[i], xrr = xr[pairs_total + i];
        orow[i] = xl * cs - xrr * sn;
        orow[pairs_total + i] = xl * sn + xrr * cs;
        f *= step;
      }
    }
  }
  return kOk;
}

// Cast f32 -> f16 (round to nearest even), src/aion/backend/cpu/exec/cast.zig:67-76.
ORC_API int aion_oracle_cast_f32_f16(uint16_t* out, const float* in, uint64_t n) {
  for (uint64_t i = 0; i < n; i++) out[i] = f32_to_f16_bits(in[i]);
  return kOk;
}

// SequenceAppend into a [B, T, H, D] cache at logical step end_index[b] + t:
// src/aion/backend/cpu/exec/sequence_append.zig:12-104. A plain cache maps a logical step
// to itself and rejects steps beyond T; a rolling cache maps it to step % T.
ORC_API int aion_oracle_sequence_append(uint8_t* cache, const uint8_t* new_kv, const int32_t* end_index, uint64_t elem_bytes,
                                        uint64_t b, uint64_t t_cap, uint64_t h, uint64_t d, uint64_t new_len, int rolling) {
  const size_t row = h * d * elem_bytes;
  for (uint64_t bb = 0; bb < b; bb++) {
    if (end_index[bb] < 0) return kInvalid;
    for (uint64_t t = 0; t < new_len; t++) {
      const uint64_t logical = static_cast<uint64_t>(end_index[bb]) + t;
      if (!rolling && logical >= t_cap) return kInvalid;
    }
  }
  for (uint64_t bb = 0; bb < b; bb++)
    for (uint64_t t = 0; t < new_len; t++) {
      const uint64_t logical = static_cast<uint64_t>(end_index[bb]) + t;
      const uint64_t dst = rolling ? logical % t_cap : logical;
      std::memcpy(cache + (bb * t_cap + dst) * row, new_kv + (bb * new_len + t) * row, row);
    }
  return kOk;
}

// GatherRows from a q8_0 [rows, d] table (quant_axis 1, any block order) to f32:
// src/aion/backend/cpu/exec/gather.zig:22-28, 57-87. Index in [-rows, rows-1].
ORC_API int aion_oracle_gather_rows_q8(float* out, const uint8_t* table, int order, uint64_t table_rows, uint64_t d,
                                       const int32_t* indices, uint64_t count) {
  BlockOrder o;
  if (!order_info(order, &o) || d % QK != 0) return kInvalid;
  const size_t blocks = d / QK;
  for (uint64_t i = 0; i < count; i++) {
    int64_t v = indices[i];
    if (v < 0) v += static_cast<int64_t>(table_rows);
    if (v < 0 || v >= static_cast<int64_t>(table_rows)) return kInvalid;
    for (size_t kb = 0; kb < blocks; kb++) {
      uint8_t block[Q8_BYTES];
      load_block(o, table, blocks, static_cast<size_t>(v), kb, block);
      uint16_t sb;
      std::memcpy(&sb, block, 2);
      const float scale = f16_bits_to_f32(sb);
      for (int t = 0; t < 32; t++) out[i * d + kb * QK + t] = static_cast<float>(static_cast<int8_t>(block[2 + t])) * scale;
    }
  }
  return kOk;
}

// ArgMax over the last axis, first maximum wins: src/aion/backend/cpu/exec/argmax.zig:56-82.
ORC_API int aion_oracle_argmax(int32_t* out, const float* in, uint64_t outer, uint64_t n) {
  if (n == 0) return kInvalid;
  for (uint64_t o = 0; o < outer; o++) {
    const float* row = in + o * n;
    size_t best_i = 0;
    float best_v = row[0];
    for (size_t j = 1; j < n; j++)
      if (row[j] > best_v) {
        best_v = row[j];
        best_i = j;
      }
    out[o] = static_cast<int32_t>(best_i);
  }
  return kOk;
}
