// Timed CPU baseline (TEST / BENCHMARK INFRASTRUCTURE ONLY; never linked into the
// shipped library): the reference's CPU kernels restated with the same structure and
// the same x86 byte-dot instruction they use, threaded over all host cores.
//
// The reference (Zig) cannot be built here, so this is a port, labelled "port" wherever
// its numbers are reported. What is mirrored:
//   * q8_0 K-major, m <= 16: the direct register-tile matvec, NT = 4 columns, activation
//     prepared once per row (src/aion/backend/cpu/kernels/matvec_q.zig:62-160), columns
//     split across threads in groups of 16 (src/aion/backend/cpu/exec/matmul.zig:229, 268-293).
//   * q4_0 (any m) and q8_0 m > 16: the packed int8 GEMM — per task, per kc = 256 chunk of
//     K, B is re-packed into 8-column VNNI panels (scales, column sums, 32x8 int8 in groups
//     of 4 K) and multiplied with `vpdpbusd` on MR = 4 rows
//     (src/aion/backend/cpu/kernels/matmul_q_i8.zig:314-497, task grid
//     src/aion/backend/cpu/exec/matmul.zig:381-463). The re-pack per call is part of the
//     reference's cost for q4 at m = 1 and is kept.
//   * q8_0 NT row-major: 2x2 micro-tile over prepared rows
//     (src/aion/backend/cpu/kernels/matmul_nt_q.zig:74-95, 389-461), rows of B split across
//     threads (src/aion/backend/cpu/exec/matmul_nt.zig:132-134).
//   * `Attention`: the generic per-row executor of the scalar oracle, one request per task
//     (the reference threads its per-row executor over rows,
//     src/aion/backend/cpu/exec/attention.zig:1025-1318); same values as the scalar oracle.
// A CPU without AVX-512-VNNI/AVX-VNNI runs the scalar byte dot (same values).
#include <omp.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t QK = 32;
constexpr int DT_Q4_0 = 3, DT_Q8_0 = 4;

inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t mant = h & 0x3FFu;
  uint32_t out;
  if (exp == 0) {
    if (mant == 0) out = sign;
    else {
      int e = -1;
      do { mant <<= 1; e++; } while (!(mant & 0x400u));
      out = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((mant & 0x3FFu) << 13);
    }
  } else if (exp == 31) out = sign | 0x7F800000u | (mant << 13);
  else out = sign | ((exp + 127 - 15) << 23) | (mant << 13);
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

inline float quantize_a_block(const float* a, int8_t* out) {
  float amax = 0.0f;
  for (size_t t = 0; t < QK; t++) amax = std::max(amax, std::fabs(a[t]));
  if (amax == 0.0f) {
    std::memset(out, 0, QK);
    return 0.0f;
  }
  const float inv = 127.0f / amax;
  for (size_t t = 0; t < QK; t++) {
    float r = std::round(a[t] * inv);
    r = std::max(-127.0f, std::min(127.0f, r));
    out[t] = static_cast<int8_t>(static_cast<int32_t>(r));
  }
  return amax / 127.0f;
}

bool g_has_vnni = false;
struct Init {
  Init() {
#if defined(__x86_64__)
    g_has_vnni = __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512vl") &&
                 __builtin_cpu_supports("avx512bw");
#endif
  }
} g_init;

// 32-element signed dot. VNNI: weight ^ 0x80 as the unsigned side, minus 128 * sum(a).
inline int32_t dot32_scalar(const int8_t* w, const int8_t* a) {
  int32_t s = 0;
  for (size_t t = 0; t < QK; t++) s += int32_t(w[t]) * int32_t(a[t]);
  return s;
}
#if defined(__x86_64__)
__attribute__((target("avx512vnni,avx512vl,avx512bw,avx2"))) inline int32_t dot32_vnni(const int8_t* w, const int8_t* a,
                                                                                       int32_t corr128) {
  const __m256i wv = _mm256_xor_si256(_mm256_loadu_si256(reinterpret_cast<const __m256i*>(w)), _mm256_set1_epi8((char)0x80));
  const __m256i av = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(a));
  __m256i acc = _mm256_dpbusd_epi32(_mm256_setzero_si256(), wv, av);
  __m128i lo = _mm_add_epi32(_mm256_castsi256_si128(acc), _mm256_extracti128_si256(acc, 1));
  lo = _mm_add_epi32(lo, _mm_shuffle_epi32(lo, 0x4E));
  lo = _mm_add_epi32(lo, _mm_shuffle_epi32(lo, 0xB1));
  return _mm_cvtsi128_si32(lo) - corr128;
}
#endif

struct Prepared {  // one row of A: int8 codes, scales, 128 * sum per block
  std::vector<int8_t> q;
  std::vector<float> s;
  std::vector<int32_t> c;
  void prepare(const float* a, size_t blocks) {
    q.resize(blocks * QK);
    s.resize(blocks);
    c.resize(blocks);
    for (size_t kb = 0; kb < blocks; kb++) {
      s[kb] = quantize_a_block(a + kb * QK, q.data() + kb * QK);
      int32_t sum = 0;
      for (size_t t = 0; t < QK; t++) sum += q[kb * QK + t];
      c[kb] = 128 * sum;
    }
  }
};

inline int32_t dot32(const int8_t* w, const int8_t* a, int32_t corr) {
#if defined(__x86_64__)
  if (g_has_vnni) return dot32_vnni(w, a, corr);
#endif
  (void)corr;
  return dot32_scalar(w, a);
}

// ---- packed int8 GEMM (q4 / q8), one task = rows x nc block of C over all of K ----------
constexpr size_t NR = 8, MR = 4, KC = 256, NC = 256;
constexpr size_t PB_BLOCK = 32 + 32 + 256;

void pack_tile(int dtype, uint8_t* pb, size_t kblocks, size_t n, size_t ldb, const uint8_t* b) {
  const size_t bb = dtype == DT_Q8_0 ? 34 : 18;
  const size_t panels = (n + NR - 1) / NR;
  for (size_t p = 0; p < panels; p++)
    for (size_t kb = 0; kb < kblocks; kb++) {
      uint8_t* base = pb + (p * kblocks + kb) * PB_BLOCK;
      float* scales = reinterpret_cast<float*>(base);
      int32_t* sumb = reinterpret_cast<int32_t*>(base + 32);
      int8_t* q = reinterpret_cast<int8_t*>(base + 64);
      for (size_t jj = 0; jj < NR; jj++) {
        const size_t col = p * NR + jj;
        if (col >= n) {
          scales[jj] = 0.0f;
          sumb[jj] = 0;
          for (size_t t = 0; t < QK; t++) q[(t >> 2) * (NR * 4) + jj * 4 + (t & 3)] = 0;
          continue;
        }
        const uint8_t* blk = b + (kb * ldb + col) * bb;
        scales[jj] = f16_to_f32(static_cast<uint16_t>(blk[0] | (blk[1] << 8)));
        int32_t sum = 0;
        for (size_t t = 0; t < QK; t++) {
          int8_t v;
          if (dtype == DT_Q8_0) v = static_cast<int8_t>(blk[2 + t]);
          else {
            const uint8_t byte = blk[2 + (t >> 1)];
            v = static_cast<int8_t>(static_cast<int>((t & 1) ? (byte >> 4) : (byte & 0x0F)) - 8);
          }
          sum += v;
          q[(t >> 2) * (NR * 4) + jj * 4 + (t & 3)] = v;
        }
        sumb[jj] = sum;
      }
    }
}

#if defined(__x86_64__)
__attribute__((target("avx512vnni,avx512vl,avx512bw,avx2,fma"))) void packed_rows_vnni(
    const uint8_t* pb, size_t kblocks, size_t panels, size_t n, size_t mr, const int8_t* aq, size_t aq_stride,
    const float* ascale, size_t as_stride, float* c, size_t ldc, float alpha, float beta) {
  for (size_t p = 0; p < panels; p++) {
    __m256 cacc[MR];
    for (size_t r = 0; r < MR; r++) cacc[r] = _mm256_setzero_ps();
    for (size_t kb = 0; kb < kblocks; kb++) {
      const uint8_t* base = pb + (p * kblocks + kb) * PB_BLOCK;
      __m256i acc[MR];
      for (size_t r = 0; r < MR; r++) acc[r] = _mm256_setzero_si256();
      for (size_t g = 0; g < 8; g++) {
        const __m256i bg = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(base + 64 + g * 32));
        for (size_t r = 0; r < mr; r++) {
          int32_t word;
          std::memcpy(&word, aq + r * aq_stride + kb * QK + g * 4, 4);
          const __m256i au = _mm256_xor_si256(_mm256_set1_epi32(word), _mm256_set1_epi8((char)0x80));
          acc[r] = _mm256_dpbusd_epi32(acc[r], au, bg);
        }
      }
      const __m256i sumb = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(base + 32));
      const __m256 bscale = _mm256_loadu_ps(reinterpret_cast<const float*>(base));
      const __m256i corr = _mm256_slli_epi32(sumb, 7);
      for (size_t r = 0; r < mr; r++) {
        const __m256 f = _mm256_cvtepi32_ps(_mm256_sub_epi32(acc[r], corr));
        const __m256 as = _mm256_set1_ps(ascale[r * as_stride + kb]);
        cacc[r] = _mm256_add_ps(cacc[r], _mm256_mul_ps(_mm256_mul_ps(f, bscale), as));
      }
    }
    const size_t rem = std::min(NR, n - p * NR);
    for (size_t r = 0; r < mr; r++) {
      alignas(32) float o[8];
      _mm256_store_ps(o, _mm256_mul_ps(cacc[r], _mm256_set1_ps(alpha)));
      float* cp = c + r * ldc + p * NR;
      for (size_t jj = 0; jj < rem; jj++) cp[jj] = beta == 0.0f ? o[jj] : o[jj] + beta * cp[jj];
    }
  }
}
#endif

void packed_rows_scalar(const uint8_t* pb, size_t kblocks, size_t panels, size_t n, size_t mr, const int8_t* aq,
                        size_t aq_stride, const float* ascale, size_t as_stride, float* c, size_t ldc, float alpha,
                        float beta) {
  for (size_t p = 0; p < panels; p++) {
    float cacc[MR][NR] = {};
    for (size_t kb = 0; kb < kblocks; kb++) {
      const uint8_t* base = pb + (p * kblocks + kb) * PB_BLOCK;
      const float* bscale = reinterpret_cast<const float*>(base);
      const int8_t* q = reinterpret_cast<const int8_t*>(base + 64);
      for (size_t r = 0; r < mr; r++)
        for (size_t jj = 0; jj < NR; jj++) {
          int32_t d = 0;
          for (size_t t = 0; t < QK; t++) d += int32_t(q[(t >> 2) * 32 + jj * 4 + (t & 3)]) * int32_t(aq[r * aq_stride + kb * QK + t]);
          cacc[r][jj] += float(d) * bscale[jj] * ascale[r * as_stride + kb];
        }
    }
    const size_t rem = std::min(NR, n - p * NR);
    for (size_t r = 0; r < mr; r++)
      for (size_t jj = 0; jj < rem; jj++) {
        float* cp = c + r * ldc + p * NR + jj;
        const float o = cacc[r][jj] * alpha;
        *cp = beta == 0.0f ? o : o + beta * *cp;
      }
  }
}

void gemm_packed(int dtype, size_t m, size_t n, size_t k, const float* a, const uint8_t* b, float* c, float alpha,
                 float beta, int threads) {
  const size_t bb = dtype == DT_Q8_0 ? 34 : 18;
  // planGemm (src/aion/backend/cpu/exec/matmul.zig:381-419)
  const double cost = dtype == DT_Q4_0 ? 3.0 : 1.5;
  const double ideal = std::sqrt(double(threads) * double(n) * cost / double(m));
  const size_t max_blocks = (n + 15) / 16;
  const size_t want_blocks = std::min(std::max<size_t>(size_t(std::llround(ideal)), 1), max_blocks);
  size_t nc = ((n + want_blocks - 1) / want_blocks + 15) / 16 * 16;
  nc = std::min(std::max<size_t>(nc, 16), NC);
  const size_t col_blocks = (n + nc - 1) / nc;
  const size_t want_groups = std::max<size_t>(1, size_t(threads) / col_blocks);
  const size_t row_groups_max = std::max<size_t>(1, m / 16);
  size_t rows = (m + std::min(want_groups, row_groups_max) - 1) / std::min(want_groups, row_groups_max);
  rows = std::max<size_t>(rows, 1);
  const size_t row_groups = (m + rows - 1) / rows;
  const size_t tasks = col_blocks * row_groups;
  const size_t kcb = KC / QK;

#pragma omp parallel num_threads(threads)
  {
    std::vector<uint8_t> pb((NC / NR) * kcb * PB_BLOCK);
    std::vector<int8_t> aq(MR * KC);
    std::vector<float> as(MR * kcb);
#pragma omp for schedule(dynamic, 1)
    for (size_t task = 0; task < tasks; task++) {
      const size_t j0 = (task / row_groups) * nc, r0 = (task % row_groups) * rows;
      if (r0 >= m || j0 >= n) continue;
      const size_t nw = std::min(nc, n - j0), rw = std::min(rows, m - r0);
      for (size_t pc = 0; pc < k; pc += KC) {
        const size_t kw = std::min(KC, k - pc), kbs = kw / QK;
        pack_tile(dtype, pb.data(), kbs, nw, n, b + ((pc / QK) * n + j0) * bb);
        const float bt = pc == 0 ? beta : 1.0f;
        for (size_t i0 = 0; i0 < rw; i0 += MR) {
          const size_t mr = std::min(MR, rw - i0);
          for (size_t r = 0; r < mr; r++)
            for (size_t kb = 0; kb < kbs; kb++)
              as[r * kcb + kb] = quantize_a_block(a + (r0 + i0 + r) * k + pc + kb * QK, aq.data() + r * KC + kb * QK);
          float* cblk = c + (r0 + i0) * n + j0;
#if defined(__x86_64__)
          if (g_has_vnni) {
            packed_rows_vnni(pb.data(), kbs, (nw + NR - 1) / NR, nw, mr, aq.data(), KC, as.data(), kcb, cblk, n, alpha, bt);
            continue;
          }
#endif
          packed_rows_scalar(pb.data(), kbs, (nw + NR - 1) / NR, nw, mr, aq.data(), KC, as.data(), kcb, cblk, n, alpha, bt);
        }
      }
    }
  }
}

}  // namespace

ORC_API int aion_oracle_fast_has_vnni() { return g_has_vnni ? 1 : 0; }
ORC_API int aion_oracle_fast_max_threads() { return omp_get_max_threads(); }

// `MatMul` with a K-major quantized B (dense: lda = k, ldb = n, ldc = n), the reference's routing.
ORC_API int aion_oracle_fast_matmul_q(int dtype, uint64_t m, uint64_t n, uint64_t k, float alpha, float beta, float* c,
                                      const float* a, const uint8_t* b, int threads) {
  if ((dtype != DT_Q8_0 && dtype != DT_Q4_0) || k % QK != 0) return 1;
  if (threads <= 0) threads = omp_get_max_threads();
  if (m == 0 || n == 0) return 0;
  const size_t blocks = k / QK;
  if (dtype == DT_Q8_0 && m <= 16) {
    std::vector<Prepared> prep(m);
    for (size_t r = 0; r < m; r++) prep[r].prepare(a + r * k, blocks);
    const size_t groups = (n + 15) / 16;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (size_t gi = 0; gi < groups; gi++) {
      const size_t j0 = gi * 16, j1 = std::min<size_t>(n, j0 + 16);
      for (size_t r = 0; r < m; r++)
        for (size_t jt = j0; jt < j1; jt += 4) {  // NT = 4 register tile
          float acc[4] = {0, 0, 0, 0};
          const size_t nt = std::min<size_t>(4, j1 - jt);
          for (size_t kb = 0; kb < blocks; kb++) {
            const uint8_t* row = b + (kb * n + jt) * 34;
            for (size_t jj = 0; jj < nt; jj++) {
              const uint8_t* bp = row + jj * 34;
              const int32_t d = dot32(reinterpret_cast<const int8_t*>(bp + 2), prep[r].q.data() + kb * QK, prep[r].c[kb]);
              acc[jj] += float(d) * (prep[r].s[kb] * f16_to_f32(static_cast<uint16_t>(bp[0] | (bp[1] << 8))));
            }
          }
          for (size_t jj = 0; jj < nt; jj++) {
            float& cc = c[r * n + jt + jj];
            cc = beta == 0.0f ? alpha * acc[jj] : alpha * acc[jj] + beta * cc;
          }
        }
    }
    return 0;
  }
  gemm_packed(dtype, m, n, k, a, b, c, alpha, beta, threads);
  return 0;
}

// `MatMulNT` with q8_0 row-major [n, k] B.
ORC_API int aion_oracle_fast_matmul_nt_q8(uint64_t m, uint64_t n, uint64_t k, float alpha, float beta, float* c,
                                          const float* a, const uint8_t* b, int threads) {
  if (k % QK != 0) return 1;
  if (threads <= 0) threads = omp_get_max_threads();
  const size_t blocks = k / QK;
  std::vector<Prepared> prep(m);
  for (size_t r = 0; r < m; r++) prep[r].prepare(a + r * k, blocks);
  const size_t chunks = std::max<size_t>(1, std::min<size_t>(size_t(threads) * (m > 1 ? 16 : 4), n * blocks * 34 / 65536));
  const size_t per = (n + chunks - 1) / chunks;
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1)
  for (size_t ch = 0; ch < chunks; ch++) {
    const size_t j0 = ch * per, j1 = std::min<size_t>(n, j0 + per);
    for (size_t j = j0; j < j1; j += 2)      // NR = 2 columns
      for (size_t r = 0; r < m; r += 2) {    // MR = 2 rows
        float acc[2][2] = {};
        const size_t jn = std::min<size_t>(2, j1 - j), rn = std::min<size_t>(2, m - r);
        for (size_t kb = 0; kb < blocks; kb++)
          for (size_t jj = 0; jj < jn; jj++) {
            const uint8_t* bp = b + ((j + jj) * blocks + kb) * 34;
            const float bs = f16_to_f32(static_cast<uint16_t>(bp[0] | (bp[1] << 8)));
            for (size_t rr = 0; rr < rn; rr++) {
              const Prepared& pr = prep[r + rr];
              const int32_t d = dot32(reinterpret_cast<const int8_t*>(bp + 2), pr.q.data() + kb * QK, pr.c[kb]);
              acc[rr][jj] += float(d) * (pr.s[kb] * bs);
            }
          }
        for (size_t rr = 0; rr < rn; rr++)
          for (size_t jj = 0; jj < jn; jj++) {
            float& cc = c[(r + rr) * n + j + jj];
            cc = beta == 0.0f ? alpha * acc[rr][jj] : alpha * acc[rr][jj] + beta * cc;
          }
      }
  }
  return 0;
}


// The scalar oracle's attention (aion_oracle.cpp, same shared object).
extern "C" int aion_oracle_attention(float* out, const void* q, int q_dtype, const void* k, int k_dtype, const void* v, int v_dtype,
                                     const int32_t* positions, const int32_t* kv_lengths, uint64_t B, uint64_t L, uint64_t Hq,
                                     uint64_t Hkv, uint64_t Dk, uint64_t Dv, uint64_t T, float scale, uint32_t win_left,
                                     uint32_t win_right, uint32_t win_chunk, float soft_cap, int rolling, int exact);

// `Attention`, requests in parallel: each task runs the scalar executor on one request.
ORC_API int aion_oracle_fast_attention(float* out, const void* q, int q_dtype, const void* k, int k_dtype, const void* v, int v_dtype,
                                       const int32_t* positions, const int32_t* kv_lengths, uint64_t B, uint64_t L, uint64_t Hq,
                                       uint64_t Hkv, uint64_t Dk, uint64_t Dv, uint64_t T, float scale, uint32_t win_left,
                                       uint32_t win_right, uint32_t win_chunk, float soft_cap, int rolling, int threads) {
  if (threads <= 0) threads = omp_get_max_threads();
  const size_t qe = q_dtype == 0 ? 4 : 2, ke = k_dtype == 0 ? 4 : 2, ve = v_dtype == 0 ? 4 : 2;
  int status = 0;
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1)
  for (uint64_t b = 0; b < B; b++) {
    const int rc = aion_oracle_attention(out + b * L * Hq * Dv, static_cast<const uint8_t*>(q) + b * L * Hq * Dk * qe, q_dtype,
                                         static_cast<const uint8_t*>(k) + b * T * Hkv * Dk * ke, k_dtype,
                                         static_cast<const uint8_t*>(v) + b * T * Hkv * Dv * ve, v_dtype,
                                         positions ? positions + b * L : nullptr, kv_lengths ? kv_lengths + b : nullptr, 1, L, Hq, Hkv, Dk,
                                         Dv, T, scale, win_left, win_right, win_chunk, soft_cap, rolling, 0);
    if (rc != 0) {
#pragma omp atomic write
      status = rc;
    }
  }
  return status;
}
