// Decode GEMV for q4_0 / q8_0 weights: C[m,n] = alpha * A[m,k] . W + beta * C, m <= 16 per
// group of CTAs (blockIdx.y walks further groups of 16 rows over the same weights).
//
// Arithmetic is the reference CPU kernels' (src/aion/backend/cpu/kernels/matvec_q.zig:62-160,
// src/aion/backend/cpu/kernels/matmul_nt_q.zig:74-95, src/aion/backend/cpu/kernels/matmul_q_i8.zig:385-497):
// the activation is quantized to int8 per 32-block inside the kernel, every weight
// block contributes float(exact int dot) * (a_scale * w_scale), accumulated in f32.
//
// The kernel is HBM-bound: each weight byte is read from global memory exactly once.
//   * Work is cut into units of (64 output columns) x (8 K blocks) = one shared-memory
//     stage (9 KB of q4, 17 KB of q8). The grid is persistent — as many CTAs as are
//     resident at once — and CTA c takes the contiguous unit range [c*U/G, (c+1)*U/G)
//     in tile-major order ("stream-K"), so every SM streams the same number of bytes
//     whatever the shape: no tail wave, and narrow matrices split along K for free.
//   * A producer warp fills a 2-stage ring (shallow on purpose: concurrent launches overlap
//     as far as CTAs fit an SM) with ONE tiled TMA load per stage (the weight
//     tensor viewed as bytes in 8-byte elements; one request per stage, because the copy
//     engine takes about 50 ns per request and per-row bulk copies made that the
//     bottleneck), completing on mbarriers. Blocks are 18 / 34 bytes, so nothing inside
//     a stage is aligned except the stage itself.
//   * Four consumer warps drain it, each owning 16 of the tile's 64 columns for all K, so
//     no sums cross warps. They feed the int8 tensor-core MMA (m16n8k32): the 16 "rows"
//     are 16 output columns of one K block, the 8 "columns" are up to 8 activation rows.
//     q4 nibbles become int8 in three logic ops by placing the nibble in the high half of
//     a byte (value 16*(nibble-8)); the 1/16 folds into the activation scale. One block's
//     int32 dot leaves the MMA and is scaled and accumulated in f32 registers with
//     packed f32x2 arithmetic.
//   * Shared-memory reads are one wavefront each: the 8 row groups of a fragment read 8
//     columns that are 8 apart (K-major: 4 words apart modulo the 32 banks) or 8
//     consecutive weight rows 272 bytes apart (NT).
//   * A tile whose K range is shared by several CTAs is finished by the last of them to
//     arrive: each writes its partial sums to scratch, takes a ticket, and the last one
//     adds the parts in CTA order (so results do not depend on timing) and stores C. While
//     independent launches are recorded into parallel lanes and there is about one tile per
//     SM, each CTA takes exactly one whole tile instead and this step is skipped.
//   * With programmatic dependent launch the next kernel's weight stream starts as this
//     one's CTAs retire; only the activation read waits for the previous kernel.
#include "common.cuh"
#include "ptx.cuh"
#include "quant_device.cuh"

namespace aion {


namespace {

constexpr int TN = 64;             // output columns per tile
constexpr int KBT = 8;             // K blocks per stage
constexpr int NS = 2;              // stages in the ring: shallow, so that more CTAs (of concurrent launches) fit an SM
constexpr int CONSUMER_WARPS = 4;  // one per 16 columns
constexpr int CONSUMER_THREADS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMER_THREADS + 32;
constexpr int NT_ROW_PITCH = KBT * Q8_BYTES;  // 272: 16-byte multiple, 4 words mod 32 banks
constexpr size_t ACT_BUDGET_BYTES = 40 * 1024;  // quantized activations kept per CTA


struct GemvParams {
  const float* a;
  float* c;
  uint32_t m, n, kblocks;
  uint32_t mp2;  // activation rows held in shared memory: m rounded up to even
  uint64_t lda, ldc;
  float alpha, beta;
  uint32_t tiles, stages_per_tile;
  uint64_t units;
  float* partials;  // [cta][2][TN * 8*MT]
  int* tickets;     // [tile][warp]
  int* fault;
  uint32_t a_vec4;  // A rows may be read as float4
  // Pre-quantized activations (m >= 2): the shared-memory image of one group of rows,
  // `act_image_bytes` per group, written by gemv_act_image_kernel.
  const uint8_t* act_image;
  uint32_t act_image_bytes;
};

template <int DT, bool NT>
struct Geom {
  static constexpr int BB = (DT == AION_CUDA_DTYPE_Q8_0) ? Q8_BYTES : Q4_BYTES;
  static constexpr int KM_PITCH = TN * BB;
  static constexpr int STAGE_BYTES = NT ? TN * NT_ROW_PITCH : KBT * KM_PITCH;
  static constexpr int RING_BYTES = NS * STAGE_BYTES;
  static constexpr int OFF_BARS = RING_BYTES;
  static constexpr int OFF_ACT = OFF_BARS + 128;
  static_assert(STAGE_BYTES % 128 == 0, "TMA destinations are 128-byte aligned");
};

// Shared-memory bytes of the quantized activations: per K block, mp2 rows of 32 codes,
// then mp2/2 scale quads (s_even, s_even, s_odd, s_odd).
__host__ __device__ inline size_t act_bytes(uint32_t kb_pad, uint32_t mp2, uint32_t mt) {
  return (size_t)kb_pad * (mp2 * 32 + (mp2 == 2 ? 16 : mt * 64));
}

// Shared-memory loads by 32-bit shared address. They are plain (non-volatile) asm so the
// compiler may interleave the loads of independent K blocks; each takes its address from
// a register the mbarrier wait has touched, which keeps it after the wait. Constant
// offsets fold into the instruction.
template <int OFF>
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ float lds_f16(uint32_t addr) {
  unsigned short h;
  asm("ld.shared.u16 %0, [%1+%2];" : "=h"(h) : "r"(addr), "n"(OFF));
  return __half2float(__ushort_as_half(h));
}
template <int OFF>
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ void lds_f32x4(uint32_t addr, uint64_t& lo, uint64_t& hi) {
  asm("ld.shared.v2.b64 {%0, %1}, [%2+%3];" : "=l"(lo), "=l"(hi) : "r"(addr), "n"(OFF));
}

// The two A-fragment registers of one weight block for quad lane j. `aligned` says the
// block's codes start on a 4-byte boundary (they start 2 bytes after the block does).
// `blk` already includes the lane's 4*j.
template <int DT, bool ALIGNED, int OFF>
__device__ __forceinline__ void load_codes(uint32_t blk, uint32_t& r_lo, uint32_t& r_hi) {
  if (DT == AION_CUDA_DTYPE_Q4_0) {
    uint32_t v;
    if (ALIGNED) v = lds_u32<OFF + 2>(blk);
    else v = __funnelshift_r(lds_u32<OFF>(blk), lds_u32<OFF + 4>(blk), 16);
    // nibble -> signed byte 16*(nibble-8): move it to the high half, flip its top bit.
    r_lo = ((v << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
    r_hi = (v & 0xF0F0F0F0u) ^ 0x80808080u;
  } else {
    if (ALIGNED) {
      r_lo = lds_u32<OFF + 2>(blk);
      r_hi = lds_u32<OFF + 18>(blk);
    } else {
      r_lo = __funnelshift_r(lds_u32<OFF>(blk), lds_u32<OFF + 4>(blk), 16);
      r_hi = __funnelshift_r(lds_u32<OFF + 16>(blk), lds_u32<OFF + 20>(blk), 16);
    }
  }
}

// Packed f32x2 helpers (two independent IEEE f32 operations per instruction).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// Everything one K block of a stage needs from shared memory, for one lane.
template <int MT>
struct BlockRegs {
  uint32_t a0, a1, a2, a3;  // weight codes: rows g / g+8, low / high half of K
  uint64_t ws;              // (scale of row g, scale of row g+8)
  uint2 bq[MT];             // activation codes
  uint64_t se[MT], so[MT];  // (s, s) of activation rows 2j and 2j+1
};

// K-major: rows g read an even column (codes 2 bytes past a word boundary), rows g+8 the
// odd column after it (aligned). NT: both rows read block KBL of their weight row, whose
// codes are aligned when KBL is odd.
template <int DT, bool NT, int MT, int KBL, int STEP, int AQ_STRIDE, int AS_STRIDE>
__device__ __forceinline__ void load_block(BlockRegs<MT>& r, uint32_t w0, uint32_t w1, uint32_t b0, uint32_t b1,
                                           const uint32_t (&aq)[MT], const uint32_t (&as)[MT]) {
  constexpr bool AL0 = NT ? (KBL & 1) != 0 : false;
  constexpr bool AL1 = NT ? (KBL & 1) != 0 : true;
  load_codes<DT, AL0, KBL * STEP>(w0, r.a0, r.a2);
  load_codes<DT, AL1, KBL * STEP>(w1, r.a1, r.a3);
  r.ws = pack2(lds_f16<KBL * STEP>(b0), lds_f16<KBL * STEP>(b1));
#pragma unroll
  for (int t = 0; t < MT; t++) {
    r.bq[t] = lds_u64<KBL * AQ_STRIDE>(aq[t]);
    lds_f32x4<KBL * AS_STRIDE>(as[t], r.se[t], r.so[t]);
  }
}

template <int MT, bool M1>
__device__ __forceinline__ void compute_block(const BlockRegs<MT>& r, uint64_t (&acc)[MT][2]) {
#pragma unroll
  for (int t = 0; t < MT; t++) {
    int d[4];
    ptx::mma_s8(d, r.a0, r.a1, r.a2, r.a3, r.bq[t].x, r.bq[t].y);
    // d[0], d[2]: rows g, g+8 against activation row 2j; d[1], d[3]: against row 2j+1.
    acc[t][0] = fma2(mul2(pack2((float)d[0], (float)d[2]), r.ws), r.se[t], acc[t][0]);
    if (!M1) acc[t][1] = fma2(mul2(pack2((float)d[1], (float)d[3]), r.ws), r.so[t], acc[t][1]);
  }
}

// CTA that owns unit u when G CTAs split U units as [c*U/G, (c+1)*U/G).
__device__ __forceinline__ uint32_t unit_owner(uint64_t u, uint64_t U, uint64_t G) { return (uint32_t)(((u + 1) * G - 1) / U); }

// One 32-block of activations -> the 8 words the MMA B fragments read (lane j finds its two
// registers as the 8 bytes at 8j) and the block's scale, with the q4 nibble placement's 16x
// folded in.
//   q8: b0 = k 4j..4j+3, b1 = k 16+4j..16+4j+3            -> word 2j = w[j], word 2j+1 = w[4+j]
//   q4: b0 = elements 8j+{0,2,4,6}, b1 = elements 8j+{1,3,5,7} (low / high nibbles of 4 code bytes)
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
  const float fold = (DT == AION_CUDA_DTYPE_Q4_0) ? 0.0625f : 1.0f;  // undoes the 16x of the nibble placement (exact)
  return scale * fold;
}

// Quantizes A once per launch into the image the GEMV CTAs copy into shared memory: for
// every group of `mpa` rows, per K block `mpa` rows of 32 codes, then per K block `quads`
// scale quads (s_even, s_even, s_odd, s_odd). Rows past m and blocks past kblocks are
// written as zeros (a zero scale contributes nothing). One thread per (group, block, row).
template <int DT>
__global__ void gemv_act_image_kernel(const float* __restrict__ a, uint64_t lda, uint32_t m, uint32_t kblocks, uint32_t kb_pad,
                                      uint32_t mpa, uint32_t quads, uint32_t groups, uint8_t* __restrict__ image,
                                      uint32_t group_bytes, uint32_t a_vec4) {
  // The GEMV that follows may start now: its weight stream does not depend on this kernel,
  // and it waits for this kernel to finish before it copies the image. A comes from the
  // previous kernel, and the image buffer may still be read by an earlier GEMV until then.
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint32_t items = groups * kb_pad * mpa;
  const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= items) return;
  const uint32_t r = item % mpa, kb = (item / mpa) % kb_pad, g = item / (mpa * kb_pad);
  const uint32_t row = g * mpa + r;
  uint32_t o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float sc = 0.0f;
  if (row < m && kb < kblocks) sc = quantize_act_block<DT>(a + (uint64_t)row * lda + (uint64_t)kb * QK, a_vec4 != 0, o);
  uint8_t* base = image + (size_t)g * group_bytes;
  uint4* dst = reinterpret_cast<uint4*>(base + ((size_t)kb * mpa + r) * 32);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  float* act_s = reinterpret_cast<float*>(base + (size_t)kb_pad * mpa * 32);
  *reinterpret_cast<float2*>(act_s + ((size_t)kb * quads + (r >> 1)) * 4 + 2 * (r & 1)) = make_float2(sc, sc);
}

// DT: weight dtype; NT: weights are [n,k] row-major (else K-major); MT: 8-row activation
// tiles (1 or 2); M1: exactly one activation row (skips the odd-row half of the epilogue).
template <int DT, bool NT, int MT, bool M1, bool RG = false, bool PREQ = false>
__global__ void __launch_bounds__(THREADS) gemv_q_mma_kernel(const GemvParams p_in, const __grid_constant__ CUtensorMap tmap) {
  using G = Geom<DT, NT>;
  constexpr int MPA = 8 * MT;  // activation rows of the accumulator tile
  // More than 8 * MT rows of A: blockIdx.y picks a group of 8 * MT rows. Every group streams
  // the same weights (the second and later groups find them in L2), with its own slice of
  // the fix-up scratch.
  // (RG, row groups, is a template parameter so that the usual kernel keeps reading its
  // parameters from the constant bank instead of holding an adjusted copy in registers.)
  GemvParams p_rows;
  if (RG) {
    p_rows = p_in;
    const uint32_t r0 = blockIdx.y * MPA;
    p_rows.a += (uint64_t)r0 * p_in.lda;
    p_rows.c += (uint64_t)r0 * p_in.ldc;
    p_rows.m = min((uint32_t)MPA, p_in.m - r0);
    p_rows.partials += (size_t)blockIdx.y * gridDim.x * 2 * TN * MPA;
    p_rows.tickets += (size_t)blockIdx.y * p_in.tiles * CONSUMER_WARPS;
  }
  const GemvParams& p = RG ? p_rows : p_in;
  constexpr uint32_t MP2 = M1 ? 2 : 8 * MT;  // activation rows held in shared memory
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t smem_base = ptx::smem_u32(smem);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;

  const uint64_t U = p.units, NG = gridDim.x;
  const uint64_t u_begin = U * blockIdx.x / NG, u_end = U * (blockIdx.x + 1) / NG;
  const uint32_t Sg = p.stages_per_tile;

  const uint32_t bar_full = smem_base + G::OFF_BARS;
  const uint32_t bar_empty = bar_full + NS * 8;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + G::OFF_BARS + 2 * NS * 8);
  const uint32_t kb_pad = p.stages_per_tile * KBT;  // K blocks rounded up to whole stages
  uint8_t* act_q = smem + G::OFF_ACT;
  constexpr uint32_t QUADS = M1 ? 1 : 4 * MT;  // scale quads per K block
  float* act_s = reinterpret_cast<float*>(act_q + (size_t)kb_pad * MP2 * 32);  // [kb][QUADS]

  if (warp == CONSUMER_WARPS) {
    // ---------------- producer: one tiled TMA load per stage ----------------
    // It sets the barriers up itself and starts copying at once; the consumers meet it at
    // the CTA barrier below before they first wait on one.
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap);
      for (int s = 0; s < NS; s++) {
        ptx::mbar_init(bar_full + 8 * s, 1);
        ptx::mbar_init(bar_empty + 8 * s, CONSUMER_WARPS);
      }
      *abort_flag = 0;
      ptx::fence_barrier_init();
    }
    __syncwarp();
    const uint64_t n_units = u_end - u_begin;
    uint64_t issued = 0;
    uint32_t tile = (uint32_t)(u_begin / Sg), s = (uint32_t)(u_begin - (uint64_t)tile * Sg);
    // PREQ: every stage also brings its 8 K blocks of the pre-quantized activation image (codes,
    // then scale quads) into the stage's slot of the activation ring. The image comes from the
    // previous kernel, so those copies wait for it; the weight copies of the first NS stages
    // do not, and start at once.
    constexpr uint32_t AQ_SLICE = KBT * (M1 ? 2 : 8 * MT) * 32, AS_SLICE = KBT * (M1 ? 16 : MT * 64);
    const uint8_t* image = PREQ ? p.act_image + (size_t)(RG ? blockIdx.y : 0) * p.act_image_bytes : nullptr;
    auto issue_acts = [&](uint32_t slot_, uint32_t s_) {
      const uint32_t dst = smem_base + G::OFF_ACT + slot_ * (AQ_SLICE + AS_SLICE), full = bar_full + 8 * slot_;
      ptx::bulk_g2s(dst, image + (size_t)s_ * AQ_SLICE, AQ_SLICE, full);
      ptx::bulk_g2s(dst + AQ_SLICE, image + (size_t)kb_pad * (AQ_SLICE / KBT) + (size_t)s_ * AS_SLICE, AS_SLICE, full);
    };
    uint32_t pend_s[NS];
    uint32_t npend = 0;
    bool acts_open = !PREQ;
    for (uint64_t it = 0; it < n_units; it++) {
      const uint32_t slot = (uint32_t)(it % NS);
      if (it == (uint64_t)NS) __syncthreads();  // CTA barrier #1 (see the consumers)
      if (PREQ && !acts_open && it == (uint64_t)NS) {
        ptx::pdl_wait();
        if (lane == 0)
          for (uint32_t i = 0; i < npend; i++) issue_acts(i, pend_s[i]);
        acts_open = true;
      }
      if (it >= (uint64_t)NS) {
        if (*abort_flag) break;
        if (!ptx::mbar_wait_bounded(bar_empty + 8 * slot, (uint32_t)((it / NS) - 1) & 1)) {
          if (lane == 0) {
            atomicExch(p.fault, FAULT_WAIT_EXPIRED);
            *abort_flag = 1;
          }
          break;
        }
      }
      if (lane == 0) {
        const uint32_t full = bar_full + 8 * slot;
        const uint32_t stage = smem_base + slot * G::STAGE_BYTES;
        // Rows or columns past the tensor arrive as zeros (a zero scale), and the whole
        // box counts towards the barrier.
        ptx::mbar_arrive_expect_tx(full, G::STAGE_BYTES + (PREQ ? AQ_SLICE + AS_SLICE : 0));
        if (!NT && DT == AION_CUDA_DTYPE_Q4_0) ptx::tma_load_2d(stage, &tmap, (int32_t)(tile * (TN * G::BB / 8)), (int32_t)(s * KBT), full);
        else if (!NT) ptx::tma_load_3d(stage, &tmap, 0, (int32_t)(tile * (TN / 8)), (int32_t)(s * KBT), full);
        else ptx::tma_load_2d(stage, &tmap, (int32_t)(s * KBT * Q8_BYTES / 8), (int32_t)(tile * TN), full);
        if (PREQ) {
          if (acts_open) issue_acts(slot, s);
          else pend_s[npend] = s;
        }
      }
      if (PREQ && !acts_open) npend++;
      __syncwarp();
      issued = it + 1;
      if (++s == Sg) {
        s = 0;
        tile++;
      }
    }
    if (n_units <= (uint64_t)NS) __syncthreads();  // CTA barrier #1 when the whole range fit the ring
    if (PREQ && !acts_open) {
      ptx::pdl_wait();
      if (lane == 0)
        for (uint32_t i = 0; i < npend; i++) issue_acts(i, pend_s[i]);
    }
    // After a failed wait nobody drains the ring: let the copies still in flight land
    // (bounded) before this CTA's shared memory can be handed to another CTA.
    if (*abort_flag)
      for (uint64_t it = issued > (uint64_t)NS ? issued - NS : 0; it < issued; it++)
        ptx::mbar_wait_bounded(bar_full + 8 * (uint32_t)(it % NS), (uint32_t)(it / NS) & 1, 1u << 16);
    return;
  }

  // ---------------- consumers ----------------
  // Scales start at zero: a pad row (m odd) and rows never written must contribute
  // nothing, whatever their code bytes hold (an integer dot is always finite).
  if (!PREQ) {
    float4* z = reinterpret_cast<float4*>(act_s);
    const uint32_t quads = kb_pad * QUADS;
    for (uint32_t i = tid; i < quads; i += CONSUMER_THREADS) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();  // CTA barrier #1: the producer has initialised the mbarriers
  // The next kernel in the stream may begin: its weight stream does not depend on us.
  ptx::pdl_launch_dependents();
  // Everything below reads what the previous kernel wrote (A, and C when beta != 0).
  ptx::pdl_wait();

  if (PREQ) {
    // A was quantized once for all CTAs; its blocks arrive with the weight stages.
  } else {
    // Quantize all of A, one thread per 32-block (no cross-lane traffic, 32 independent
    // elements of instruction-level parallelism): the block's 128 bytes are one cache line.
    const uint32_t items = p.m * p.kblocks;
    for (uint32_t item = tid; item < items; item += CONSUMER_THREADS) {
      const uint32_t r = item / p.kblocks, kb = item - r * p.kblocks;
      uint32_t o[8];
      const float sc = quantize_act_block<DT>(p.a + (uint64_t)r * p.lda + (uint64_t)kb * QK, p.a_vec4 != 0, o);
      uint4* dst = reinterpret_cast<uint4*>(act_q + ((size_t)kb * MP2 + r) * 32);
      dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
      dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
      float* sq = act_s + ((size_t)kb * QUADS + (r >> 1)) * 4 + 2 * (r & 1);
      *reinterpret_cast<float2*>(sq) = make_float2(sc, sc);
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");

  // Per-lane constants: where this lane's two weight blocks (rows g and g+8 of the
  // fragment) sit inside a stage, and where its activation fragments start. Lanes whose
  // activation row does not exist read a block of zeros instead (no predicates in the loop).
  uint32_t off0, off1;
  if (!NT) {
    off0 = (2 * warp + 8 * g) * G::BB;  // an even column: its codes start 2 bytes past a word boundary
    off1 = off0 + G::BB;                // the odd column after it: codes word aligned
  } else {
    off0 = (16 * warp + g) * NT_ROW_PITCH;
    off1 = off0 + 8 * NT_ROW_PITCH;
  }
  const int col0 = NT ? 16 * warp + g : 2 * warp + 8 * g;
  const int col1 = NT ? col0 + 8 : col0 + 1;
  // Bytes per K block: MP2 rows of codes; 4*MT scale quads (absent rows keep a zero
  // scale, so whatever codes a lane of an absent row reads contribute nothing: such a
  // lane simply reads an existing row).
  // With a single activation row every lane reads the one scale quad: the outputs of the
  // lanes that stand for absent rows are finite and never stored.
  constexpr uint32_t AQ_STRIDE = MP2 * 32, AS_STRIDE = M1 ? 16 : MT * 64;
  const uint32_t act_q_addr = smem_base + G::OFF_ACT;
  const uint32_t act_s_addr = act_q_addr + (PREQ ? KBT : kb_pad) * AQ_STRIDE;  // PREQ: inside a ring slot
  uint32_t aq_lane[MT], as_lane[MT];
#pragma unroll
  for (int t = 0; t < MT; t++) {
    aq_lane[t] = act_q_addr + ((t * 8 + g) % MP2) * 32 + 8 * j;
    as_lane[t] = act_s_addr + (M1 ? 0 : (t * 4 + j) * 16);
  }

  // acc[t][0] = (row g, row g+8) x activation row t*8+2j ; acc[t][1] = the same x row t*8+2j+1.
  uint64_t acc[MT][2];
#pragma unroll
  for (int t = 0; t < MT; t++) acc[t][0] = acc[t][1] = 0ull;

  const uint32_t first_tile = (uint32_t)(u_begin / Sg);
  uint32_t tile = first_tile, s = (uint32_t)(u_begin - (uint64_t)first_tile * Sg);
  bool ok = true;
  uint64_t it = 0;
  for (uint64_t uu = u_begin; uu < u_end; uu++, it++) {
    const uint32_t slot = (uint32_t)(it % NS);
    if (ok && (*abort_flag || !ptx::mbar_wait_bounded(bar_full + 8 * slot, (uint32_t)(it / NS) & 1))) {
      if (lane == 0 && !*abort_flag) {
        atomicExch(p.fault, FAULT_WAIT_EXPIRED);
        *abort_flag = 1;
      }
      ok = false;
    }
    if (ok) {
      // K blocks past the end of K arrive as zero-filled weights against zero-scaled
      // activations, so all 8 blocks of a stage are always processed.
      uint32_t b0 = smem_base + slot * G::STAGE_BYTES + off0, b1 = smem_base + slot * G::STAGE_BYTES + off1;  // block starts
      uint32_t w0 = b0 + 4 * j, w1 = b1 + 4 * j;  // this lane's code words
      uint32_t aq[MT], as[MT];
#pragma unroll
      for (int t = 0; t < MT; t++) {
        aq[t] = aq_lane[t] + (PREQ ? slot * (KBT * (AQ_STRIDE + AS_STRIDE)) : s * (KBT * AQ_STRIDE));
        as[t] = as_lane[t] + (PREQ ? slot * (KBT * (AQ_STRIDE + AS_STRIDE)) : s * (KBT * AS_STRIDE));
      }
      // Ties every load below to this point: they cannot move above the wait.
      asm volatile("" : "+r"(w0), "+r"(w1), "+r"(b0), "+r"(b1)::"memory");
#pragma unroll
      for (int t = 0; t < MT; t++) asm volatile("" : "+r"(aq[t]), "+r"(as[t]));
      constexpr int STEP = NT ? Q8_BYTES : G::KM_PITCH;
      // Loads of four K blocks are issued before their arithmetic (and the next four
      // before the first four finish), so shared-memory and MMA latencies overlap.
      BlockRegs<MT> r[4];
#define AION_LOAD(K, R) load_block<DT, NT, MT, K, STEP, (int)AQ_STRIDE, (int)AS_STRIDE>(r[R], w0, w1, b0, b1, aq, as)
      AION_LOAD(0, 0); AION_LOAD(1, 1); AION_LOAD(2, 2); AION_LOAD(3, 3);
      compute_block<MT, M1>(r[0], acc); AION_LOAD(4, 0);
      compute_block<MT, M1>(r[1], acc); AION_LOAD(5, 1);
      compute_block<MT, M1>(r[2], acc); AION_LOAD(6, 2);
      compute_block<MT, M1>(r[3], acc); AION_LOAD(7, 3);
      compute_block<MT, M1>(r[0], acc);
      compute_block<MT, M1>(r[1], acc);
      compute_block<MT, M1>(r[2], acc);
      compute_block<MT, M1>(r[3], acc);
#undef AION_LOAD
      static_assert(KBT == 8, "eight K blocks per stage are spelled out above");
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(bar_empty + 8 * slot);

    if (s == Sg - 1 || uu == u_end - 1) {
      // ---------------- this CTA's share of `tile` is complete ----------------
      const uint64_t tile_u0 = (uint64_t)tile * Sg;
      const bool whole = (uu + 1 - tile_u0 == Sg) && (tile_u0 >= u_begin);
      const uint32_t n0 = tile * TN;
      float v[MT][4];  // [t][0..3] = (row g, m 2j), (row g+8, m 2j), (row g, m 2j+1), (row g+8, m 2j+1)
#pragma unroll
      for (int t = 0; t < MT; t++) {
        unpack2(acc[t][0], v[t][0], v[t][1]);
        unpack2(acc[t][1], v[t][2], v[t][3]);
        acc[t][0] = acc[t][1] = 0ull;
      }
      bool store = whole;
      if (!whole) {
        const uint32_t c_first = unit_owner(tile_u0, U, NG), c_last = unit_owner(tile_u0 + Sg - 1, U, NG);
        const uint32_t nparts = c_last - c_first + 1;
        float* mine = p.partials + ((size_t)blockIdx.x * 2 + (tile == first_tile ? 0 : 1)) * (TN * MPA);
#pragma unroll
        for (int t = 0; t < MT; t++) {
          *reinterpret_cast<float2*>(mine + col0 * MPA + t * 8 + 2 * j) = make_float2(v[t][0], v[t][2]);
          *reinterpret_cast<float2*>(mine + col1 * MPA + t * 8 + 2 * j) = make_float2(v[t][1], v[t][3]);
        }
        // The warp's stores are ordered before lane 0's release by the warp barrier; the
        // acquire side orders the last arriver's loads after every earlier release.
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          int* tk = p.tickets + (size_t)tile * CONSUMER_WARPS + warp;
          int prev;
          asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(prev) : "l"(tk) : "memory");
          last = (prev == (int)nparts - 1);
          if (last) *tk = 0;  // ready for the next launch
        }
        last = __shfl_sync(0xFFFFFFFFu, last, 0);
        if (last) {
          // The last part to arrive adds all of them in CTA order.
#pragma unroll
          for (int t = 0; t < MT; t++) v[t][0] = v[t][1] = v[t][2] = v[t][3] = 0.0f;
          for (uint32_t part = 0; part < nparts; part++) {
            const uint32_t cc = c_first + part;
            const uint32_t cc_first_tile = (uint32_t)((U * cc / NG) / Sg);
            const float* src = p.partials + ((size_t)cc * 2 + (tile == cc_first_tile ? 0 : 1)) * (TN * MPA);
#pragma unroll
            for (int t = 0; t < MT; t++) {
              const float2 x0 = __ldcg(reinterpret_cast<const float2*>(src + col0 * MPA + t * 8 + 2 * j));
              const float2 x1 = __ldcg(reinterpret_cast<const float2*>(src + col1 * MPA + t * 8 + 2 * j));
              v[t][0] += x0.x; v[t][2] += x0.y;
              v[t][1] += x1.x; v[t][3] += x1.y;
            }
          }
          store = true;
        }
      }
      if (store && !*abort_flag) {
#pragma unroll
        for (int t = 0; t < MT; t++)
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const uint32_t mrow = t * 8 + 2 * j + (e >> 1);
            const uint32_t col = n0 + ((e & 1) ? col1 : col0);
            if (mrow < p.m && col < p.n) {
              float* cp = p.c + (uint64_t)mrow * p.ldc + col;
              *cp = (p.beta == 0.0f) ? p.alpha * v[t][e] : p.alpha * v[t][e] + p.beta * *cp;
            }
          }
      }
    }
    if (++s == Sg) {
      s = 0;
      tile++;
    }
  }
}

template <int DT, bool NT, int MT, bool M1, bool RG = false, bool PREQ = false>
int32_t launch(AionCudaDevice* dev, GemvParams p, const uint8_t* b, uint64_t ldb) {
  using G = Geom<DT, NT>;
  auto kernel = gemv_q_mma_kernel<DT, NT, MT, M1, RG, PREQ>;
  constexpr uint32_t MP2 = M1 ? 2 : 8 * MT;
  const size_t smem = G::OFF_ACT + (PREQ ? (size_t)NS * act_bytes(KBT, MP2, MT) : act_bytes(p.stages_per_tile * KBT, MP2, MT));
  // Kernel attributes and occupancy depend on the device and the dynamic size only.
  static size_t configured_smem[16] = {};
  static size_t occ_smem[16] = {};
  static int occ_blocks[16] = {};
  const int di = dev->ordinal & 15;
  if (smem > configured_smem[di]) {
    AION_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured_smem[di] = smem;
  }
  if (occ_smem[di] != smem) {
    int nb = 0;
    AION_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kernel, THREADS, smem));
    if (nb < 1) return fail(AION_CUDA_INTERNAL_ERROR, "gemv: kernel does not fit an SM with %llu bytes of shared memory", (unsigned long long)smem);
    occ_blocks[di] = nb;
    occ_smem[di] = smem;
  }
  uint64_t grid = (uint64_t)occ_blocks[di] * dev->sm_count;
  if (dev->gemv_split_override) grid = (uint64_t)dev->gemv_split_override * dev->sm_count;  // CTAs per SM, tuning only
  if (grid > p.units) grid = p.units;
  // Small problems: fewer, fuller CTAs — about eight stages each, but never fewer than one
  // CTA per SM. Their launches are latency-bound, and independent ones recorded in
  // parallel lanes then share the GPU (measured on 9 MB q4 matrices: 148 CTAs in 8 lanes
  // stream 3.5 TB/s, 256 or 444 CTAs 2.6 to 3.0 TB/s).
  if (!dev->gemv_split_override) {
    const uint64_t sms = (uint64_t)dev->sm_count;
    uint64_t want = p.units / 8;
    if (want < sms) want = sms;
    if (grid > want) grid = want;
    if (grid > p.units) grid = p.units;
    // Nearly one tile per CTA: give every CTA exactly one whole tile, so that no tile is shared
    // and the partial-sum fix-up (two more L2 round trips at the end of a short kernel) is skipped.
    // Only while independent steps are being recorded into parallel lanes: there other launches
    // fill the idle SMs, whereas a lone launch on a critical path is shortest with every SM busy.
    bool overlapped = false;
    if (dev->recording) {
      overlapped = dev->cur_lane != 0;
      for (int l = 1; l < AionCudaDevice::LANES; l++) overlapped = overlapped || dev->lane_forked[l];
    }
    if (overlapped && (uint64_t)p.tiles <= grid && (uint64_t)p.tiles * 5 >= grid * 4) grid = p.tiles;
  }

  // Scratch for tiles shared by several CTAs: two partial slots per CTA, one ticket per (tile, warp),
  // times the groups of 8 * MT rows.
  constexpr int MPA = 8 * MT;
  const uint64_t groups = RG ? ceil_div((uint64_t)p.m, (uint64_t)MPA) : 1;
  if (groups > 65535) return fail(AION_CUDA_UNSUPPORTED, "gemv: too many rows for one launch");
  if (int32_t st = dev->reserve_gemv_fixup((size_t)groups * grid * 2 * TN * MPA * sizeof(float), (size_t)groups * p.tiles * CONSUMER_WARPS)) return st;
  p.partials = dev->lane_gemv_partials();
  p.tickets = dev->lane_gemv_tickets();

  if (PREQ) {
    // Quantize A once, into lane scratch, in the layout the CTAs copy into shared memory.
    const uint32_t kb_pad = p.stages_per_tile * KBT;
    const size_t image_bytes = act_bytes(kb_pad, MP2, MT);
    if (int32_t st = dev->reserve_scratch(groups * image_bytes)) return st;
    uint8_t* image = static_cast<uint8_t*>(dev->lane_scratch());
    const uint32_t items = (uint32_t)(groups * kb_pad * MP2);
    cudaLaunchConfig_t icfg{};
    icfg.gridDim = dim3((items + 127) / 128);
    icfg.blockDim = dim3(128);
    icfg.stream = dev->stream;
    cudaLaunchAttribute iattrs[1];
    iattrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    iattrs[0].val.programmaticStreamSerializationAllowed = 1;
    icfg.attrs = iattrs;
    static const bool no_pdl_image = std::getenv("AION_CUDA_NO_PDL_MAIN") != nullptr;  // tuning only
    icfg.numAttrs = no_pdl_image ? 0 : 1;
    AION_CUDA_TRY(cudaLaunchKernelEx(&icfg, gemv_act_image_kernel<DT>, p.a, p.lda, p.m, p.kblocks, kb_pad, (uint32_t)MP2, (uint32_t)(M1 ? 1 : 4 * MT),
                                     (uint32_t)groups, image, (uint32_t)image_bytes, p.a_vec4));
    p.act_image = image;
    p.act_image_bytes = (uint32_t)image_bytes;
  }

  // The weight tensor as bytes in 8-byte elements.
  const CUtensorMap* tm = nullptr;
  if (!NT && DT == AION_CUDA_DTYPE_Q4_0) {
    // [kblocks][n*18 bytes]: one box = 8 block rows x 64 blocks (1152 bytes, within the 2048-byte box row).
    const uint64_t dims[2] = {(uint64_t)p.n * G::BB, p.kblocks};
    const uint64_t strides[1] = {ldb * G::BB};
    const uint32_t box[2] = {(uint32_t)TN * G::BB, KBT};
    if (int32_t st = tensor_map_bytes(dev, b, 2, dims, strides, box, &tm)) return st;
  } else if (!NT) {
    // q8: 64 blocks side by side are 2176 bytes, more than a box row holds, so the row is
    // viewed as [n/8 groups][8 blocks]: one box = 8 block rows x 8 groups = 64 columns.
    const uint64_t dims[3] = {8ull * G::BB, p.n / 8, p.kblocks};
    const uint64_t strides[2] = {8ull * G::BB, ldb * G::BB};
    const uint32_t box[3] = {8u * G::BB, TN / 8, KBT};
    if (int32_t st = tensor_map_bytes(dev, b, 3, dims, strides, box, &tm)) return st;
  } else {
    // [n rows][kblocks*34 bytes]: one box = 64 rows x 8 blocks.
    const uint64_t dims[2] = {(uint64_t)p.kblocks * Q8_BYTES, p.n};
    const uint64_t strides[1] = {ldb * Q8_BYTES};
    const uint32_t box[2] = {NT_ROW_PITCH, TN};
    if (int32_t st = tensor_map_bytes(dev, b, 2, dims, strides, box, &tm)) return st;
  }

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid, (unsigned)groups);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  static const bool no_pdl_main = std::getenv("AION_CUDA_NO_PDL_MAIN") != nullptr;  // tuning only
  cfg.numAttrs = no_pdl_main ? 0 : 1;
  AION_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p, *tm));
  return AION_CUDA_OK;
}

template <int DT, bool NT>
int32_t launch_m(AionCudaDevice* dev, const GemvParams& p, const uint8_t* b, uint64_t ldb) {
  // m >= 2: A is quantized once by a small kernel instead of by every CTA.
  // (m = 1 quantizes its one row inside the kernel unless K is deep: past about 3000 the small
  // kernel is cheaper than 148 CTAs each quantizing the whole row.)
  if (p.m == 1) return p.kblocks > 96 ? launch<DT, NT, 1, true, false, true>(dev, p, b, ldb) : launch<DT, NT, 1, true>(dev, p, b, ldb);
  if (p.m <= 8) return launch<DT, NT, 1, false, false, true>(dev, p, b, ldb);
  if (p.m <= 16) return launch<DT, NT, 2, false, false, true>(dev, p, b, ldb);
  return launch<DT, NT, 2, false, true, true>(dev, p, b, ldb);  // groups of 16 rows
}

}  // namespace

int32_t gemv_mma(AionCudaDevice* dev, const MatMulArgs& g, bool probe_only) {
  if (g.m > 16ull * 65535 || g.k == 0) return AION_CUDA_UNSUPPORTED;
  if (g.n > 0x7FFFFFFFull - TN || g.k / QK > 0x7FFFFFFFull) return AION_CUDA_UNSUPPORTED;
  const uint64_t kblocks = g.k / QK;
  const uintptr_t baddr = reinterpret_cast<uintptr_t>(g.b);
  if (baddr & 15) return AION_CUDA_UNSUPPORTED;
  if (!g.nt) {
    // Groups of 8 blocks (144 / 272 bytes) are the tensor map's innermost rows.
    if (g.n % 8 != 0 || g.ldb % 8 != 0) return AION_CUDA_UNSUPPORTED;
  } else {
    if (g.dtype != AION_CUDA_DTYPE_Q8_0 || g.order != AION_CUDA_ORDER_ROW_MAJOR) return AION_CUDA_UNSUPPORTED;
    // A stage takes 8 blocks (272 bytes) of every row; rows are kblocks*34 bytes apart.
    if (kblocks % 8 != 0) return AION_CUDA_UNSUPPORTED;
  }
  if (probe_only) return AION_CUDA_OK;

  const uint32_t mp2 = g.m == 1 ? 2u : (g.m <= 8 ? 8u : 16u);  // activation rows held per CTA (see MP2)
  // K blocks whose quantized activations fit the per-CTA budget; a deeper K is issued as
  // several launches that accumulate into C, like the reference's walk over K in chunks
  // (src/aion/backend/cpu/exec/matmul.zig:431-434).
  uint64_t kb_max = (ACT_BUDGET_BYTES / ((size_t)mp2 * 32 + (g.m == 1 ? 16 : (g.m > 8 ? 128 : 64)))) / KBT * KBT;
  if (kb_max < KBT) kb_max = KBT;
  if (g.m >= 2 || kblocks > 96) kb_max = (kblocks + KBT - 1) / KBT * KBT;  // the activation streams with the weights: any depth in one launch

  for (uint64_t kb0 = 0; kb0 < kblocks; kb0 += kb_max) {
    const uint64_t nkb = kblocks - kb0 < kb_max ? kblocks - kb0 : kb_max;
    GemvParams p{};
    p.a = g.a + kb0 * QK;
    p.c = g.c;
    p.m = (uint32_t)g.m;
    p.n = (uint32_t)g.n;
    p.kblocks = (uint32_t)nkb;
    p.mp2 = mp2;
    p.lda = g.lda;
    p.ldc = g.ldc;
    p.alpha = g.alpha;
    p.beta = kb0 == 0 ? g.beta : 1.0f;
    p.tiles = (uint32_t)((g.n + TN - 1) / TN);
    p.stages_per_tile = (uint32_t)((nkb + KBT - 1) / KBT);
    p.units = (uint64_t)p.tiles * p.stages_per_tile;
    p.fault = dev->fault_dev;
    p.a_vec4 = ((reinterpret_cast<uintptr_t>(p.a) & 15) == 0 && g.lda % 4 == 0) ? 1u : 0u;
    int32_t st;
    if (g.nt) {
      st = launch_m<AION_CUDA_DTYPE_Q8_0, true>(dev, p, g.b + kb0 * Q8_BYTES, g.ldb);
    } else if (g.dtype == AION_CUDA_DTYPE_Q8_0) {
      st = launch_m<AION_CUDA_DTYPE_Q8_0, false>(dev, p, g.b + kb0 * g.ldb * Q8_BYTES, g.ldb);
    } else {
      st = launch_m<AION_CUDA_DTYPE_Q4_0, false>(dev, p, g.b + kb0 * g.ldb * Q4_BYTES, g.ldb);
    }
    if (st != AION_CUDA_OK) return st;
  }
  return AION_CUDA_OK;
}

// ------------------------------------------------------------------------------------
// The same GEMV for callers that must not allocate (see aion_cuda_matmul_static_scratch
// in the header). The split-tile partial sums and their arrival counters live in this
// file-scope array instead of in memory the device object grows on demand. Every GPU that
// loads the library holds the array until the process exits.
// ------------------------------------------------------------------------------------
namespace {

constexpr uint32_t STATIC_MAX_CTAS = 512;    // grid is clamped to this
constexpr uint32_t STATIC_MAX_TILES = 8192;  // n <= 524288
constexpr size_t STATIC_PARTIAL_BYTES = (size_t)STATIC_MAX_CTAS * 2 * TN * 8 * sizeof(float);  // m <= 8
constexpr size_t STATIC_TICKET_BYTES = (size_t)STATIC_MAX_TILES * CONSUMER_WARPS * sizeof(int);

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_PARTIAL_BYTES + STATIC_TICKET_BYTES];

// In host code `g_static_scratch` is only a stand-in for the symbol, not a device
// address: each device's address is looked up once, with that device current.
unsigned char* g_static_scratch_addr[16] = {};

template <int DT, bool NT, bool M1>
int32_t launch_static(AionCudaDevice* dev, GemvParams p, const uint8_t* b, uint64_t ldb, unsigned char* scratch) {
  using G = Geom<DT, NT>;
  auto kernel = gemv_q_mma_kernel<DT, NT, 1, M1>;
  constexpr uint32_t MP2 = M1 ? 2 : 8;
  const size_t smem = G::OFF_ACT + act_bytes(p.stages_per_tile * KBT, MP2, 1);
  AION_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int nb = 0;
  AION_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kernel, THREADS, smem));
  if (nb < 1) return fail(AION_CUDA_INTERNAL_ERROR, "gemv: kernel does not fit an SM with %llu bytes of shared memory", (unsigned long long)smem);
  uint64_t grid = (uint64_t)nb * dev->sm_count;
  if (grid > p.units) grid = p.units;
  if (grid > STATIC_MAX_CTAS) grid = STATIC_MAX_CTAS;
  p.partials = reinterpret_cast<float*>(scratch);
  p.tickets = reinterpret_cast<int*>(scratch + STATIC_PARTIAL_BYTES);
  // The counters must start at zero whatever an earlier call left behind.
  AION_CUDA_TRY(cudaMemsetAsync(p.tickets, 0, (size_t)p.tiles * CONSUMER_WARPS * sizeof(int), dev->stream));

  CUtensorMap tm;
  if (!NT && DT == AION_CUDA_DTYPE_Q4_0) {
    const uint64_t dims[2] = {(uint64_t)p.n * G::BB, p.kblocks};
    const uint64_t strides[1] = {ldb * G::BB};
    const uint32_t box[2] = {(uint32_t)TN * G::BB, KBT};
    if (int32_t st = tensor_map_encode(b, 2, dims, strides, box, &tm)) return st;
  } else if (!NT) {
    const uint64_t dims[3] = {8ull * G::BB, p.n / 8, p.kblocks};
    const uint64_t strides[2] = {8ull * G::BB, ldb * G::BB};
    const uint32_t box[3] = {8u * G::BB, TN / 8, KBT};
    if (int32_t st = tensor_map_encode(b, 3, dims, strides, box, &tm)) return st;
  } else {
    const uint64_t dims[2] = {(uint64_t)p.kblocks * Q8_BYTES, p.n};
    const uint64_t strides[1] = {ldb * Q8_BYTES};
    const uint32_t box[2] = {NT_ROW_PITCH, TN};
    if (int32_t st = tensor_map_encode(b, 2, dims, strides, box, &tm)) return st;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  AION_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p, tm));
  return AION_CUDA_OK;
}

}  // namespace

int32_t gemv_mma_static_scratch(AionCudaDevice* dev, const MatMulArgs& g) {
  if (g.m == 0 || g.n == 0) return AION_CUDA_OK;
  if (g.m > 8)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: m = %llu, the built-in scratch holds at most 8 rows", (unsigned long long)g.m);
  if (g.k == 0 || g.k / QK > 0x7FFFFFFFull || g.n > (uint64_t)STATIC_MAX_TILES * TN)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: n = %llu, k = %llu are outside the built-in scratch (n <= %u, k >= 32)",
                (unsigned long long)g.n, (unsigned long long)g.k, STATIC_MAX_TILES * TN);
  const uint64_t kblocks = g.k / QK;
  bool readable = (reinterpret_cast<uintptr_t>(g.b) & 15) == 0;
  if (!g.nt) readable = readable && g.n % 8 == 0 && g.ldb % 8 == 0;
  else readable = readable && g.dtype == AION_CUDA_DTYPE_Q8_0 && g.order == AION_CUDA_ORDER_ROW_MAJOR && kblocks % 8 == 0;
  if (!readable) return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: the tiled GEMV does not read this shape or alignment");
  const uint32_t mp2 = g.m == 1 ? 2u : 8u;
  const uint64_t kb_max = (ACT_BUDGET_BYTES / ((size_t)mp2 * 32 + (g.m == 1 ? 16 : 64))) / KBT * KBT;
  if (kblocks > kb_max)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: k = %llu with m = %llu exceeds one launch (k <= %llu)",
                (unsigned long long)g.k, (unsigned long long)g.m, (unsigned long long)(kb_max * QK));

  // First call on this device: find where the array lives on it.
  const int di = dev->ordinal & 15;
  if (!g_static_scratch_addr[di]) {
    unsigned char* ptr = nullptr;
    AION_CUDA_TRY(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
    g_static_scratch_addr[di] = ptr;
  }

  GemvParams p{};
  p.a = g.a;
  p.c = g.c;
  p.m = (uint32_t)g.m;
  p.n = (uint32_t)g.n;
  p.kblocks = (uint32_t)kblocks;
  p.mp2 = mp2;
  p.lda = g.lda;
  p.ldc = g.ldc;
  p.alpha = g.alpha;
  p.beta = g.beta;
  p.tiles = (uint32_t)((g.n + TN - 1) / TN);
  p.stages_per_tile = (uint32_t)((kblocks + KBT - 1) / KBT);
  p.units = (uint64_t)p.tiles * p.stages_per_tile;
  p.fault = dev->fault_dev;
  p.a_vec4 = ((reinterpret_cast<uintptr_t>(p.a) & 15) == 0 && g.lda % 4 == 0) ? 1u : 0u;
  unsigned char* scratch = g_static_scratch_addr[di];
  if (g.nt) return g.m == 1 ? launch_static<AION_CUDA_DTYPE_Q8_0, true, true>(dev, p, g.b, g.ldb, scratch)
                            : launch_static<AION_CUDA_DTYPE_Q8_0, true, false>(dev, p, g.b, g.ldb, scratch);
  if (g.dtype == AION_CUDA_DTYPE_Q8_0)
    return g.m == 1 ? launch_static<AION_CUDA_DTYPE_Q8_0, false, true>(dev, p, g.b, g.ldb, scratch)
                    : launch_static<AION_CUDA_DTYPE_Q8_0, false, false>(dev, p, g.b, g.ldb, scratch);
  return g.m == 1 ? launch_static<AION_CUDA_DTYPE_Q4_0, false, true>(dev, p, g.b, g.ldb, scratch)
                  : launch_static<AION_CUDA_DTYPE_Q4_0, false, false>(dev, p, g.b, g.ldb, scratch);
}

}  // namespace aion
