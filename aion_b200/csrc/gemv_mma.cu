// Decode matmul for q4_0 / q8_0 weights with the reference's int8-activation arithmetic:
// C[m,n] = alpha * A[m,k] . W + beta * C for the batch sizes of decoding (one row to a few
// hundred rows of A). The weights are streamed from global memory exactly once per group of
// up to 64 rows of A (further groups of 64 rows are further tiles; they find the weights in L2).
//
// Arithmetic is the reference CPU kernels' (src/aion/backend/cpu/kernels/matvec_q.zig:62-160,
// src/aion/backend/cpu/kernels/matmul_nt_q.zig:74-95, src/aion/backend/cpu/kernels/matmul_q_i8.zig:385-497):
// the activation is quantized to int8 per 32-block, every weight block contributes
// float(exact int dot) * w_scale * a_scale, accumulated in f32 in K order.
//
// The kernel is HBM-bound at small m and bound by instruction issue (the per-block scaling,
// which has to run on the ordinary f32 pipes) at large m:
//   * Work is cut into units of (TN output columns) x (8 K blocks) = one shared-memory stage,
//     TN = 64 (up to 16 rows of A) or 128 (more). The grid is persistent and CTA c takes the
//     contiguous unit range [c*U/G, (c+1)*U/G) in tile-major order ("stream-K"), so every SM
//     streams the same number of bytes whatever the shape; when there are at least as many
//     tiles as CTAs the ranges are rounded to whole tiles and no tile is shared.
//   * A producer warp fills a 2-stage ring with ONE tiled TMA load per stage (the weight tensor
//     viewed as bytes in 8-byte elements: blocks are 18 / 34 bytes, so nothing inside a stage
//     is aligned except the stage itself), completing on mbarriers. With a pre-quantized
//     activation image (m >= 2, deep K, or an image handed in by the producer of A) the
//     stage's 8 K blocks of the image arrive with it as two more bulk copies.
//   * Four consumer warps drain it, each owning 16 (or 2 x 16) of the tile's columns for all K,
//     so no sums cross warps. They feed the int8 tensor-core MMA (m16n8k32): the 16 "rows"
//     are 16 output columns of one K block, the 8 "columns" are 8 activation rows; a weight
//     fragment is unpacked once and used for every group of 8 activation rows.
//     q4 nibbles become int8 in three logic ops by placing the nibble in the high half of
//     a byte (value 16*(nibble-8)); the 1/16 folds into the activation scale.
//   * int32 -> f32 without a conversion instruction: the MMA's accumulator input is the bit
//     pattern of 1.5 * 2^23, so the result read as f32 is 12582912 + dot exactly, and one
//     fused multiply-add (x * w_scale - 12582912 * w_scale, a single rounding of dot * w_scale)
//     removes the offset while applying the weight scale. A second one applies the activation
//     scale and accumulates. Both are packed f32x2 instructions over the MMA's natural
//     register pairs (one weight column, two activation rows).
//   * A tile whose K range is shared by several CTAs is finished by the last of them to
//     arrive: each writes its partial sums to scratch, takes a ticket, and the last one
//     adds the parts in CTA order (so results do not depend on timing) and stores C.
//   * With programmatic dependent launch the next kernel's weight stream starts as this
//     one's CTAs retire; only the activation read waits for the previous kernel.
//   * Launches on a dependent chain (a decode step; up to 16 rows) take the whole-tile variant:
//     one tile per CTA (a deep K: a range of eight stages), a ring that holds all of its stages,
//     the producer warp's lanes issuing them side by side, and four groups of consumer warps
//     taking the stages in turn and adding their sums through shared memory. Every weight byte of
//     the CTA is under way before the previous kernel has finished, and no tile is shared, so
//     there are no partial sums to exchange. Launches recorded into parallel lanes keep the
//     streaming variant above (more CTAs of more launches per SM), except for small matrices.
#include <algorithm>
#include <mutex>

#include "act_image.cuh"
#include "common.cuh"
#include "ptx.cuh"
#include "quant_device.cuh"

namespace aion {

namespace {

constexpr int KBT = 8;             // K blocks per stage
constexpr int NS = 2;              // stages in the ring: shallow, so that more CTAs (of concurrent launches) fit an SM
constexpr int NS_DEEP = 8;         // the ring of the variant that holds a whole tile (up to 64 K blocks) per CTA
constexpr int KW_DEEP = 4;         // and its groups of consumer warps, which take the tile's stages in turn
constexpr int COL_WARPS = 4;                    // consumer warps side by side over a tile's columns
constexpr int threads_of(int rw) { return (COL_WARPS * rw + 1) * 32; }
constexpr int NT_ROW_PITCH = KBT * Q8_BYTES;  // 272: 16-byte multiple, 4 words mod 32 banks
constexpr size_t ACT_BUDGET_BYTES = 40 * 1024;  // quantized activations kept per CTA when it quantizes them itself
constexpr uint32_t MAGIC_BITS = 0x4B400000u;    // 1.5 * 2^23 as f32
constexpr float MAGIC = 12582912.0f;

struct GemvParams {
  const float* a;
  float* c;
  uint32_t m, n, kblocks;
  uint64_t lda, ldc;
  float alpha, beta;
  uint32_t tiles, col_tiles, stages_per_tile;  // tiles = col_tiles x groups of rows, group-major
  uint64_t units;
  uint32_t whole_tiles;  // CTA ranges are rounded to tile boundaries: no tile is shared
  float* partials;       // [cta][2][TN * rows]
  int* tickets;          // [tile][consumer warp]
  int* fault;
  uint32_t a_vec4;       // A rows may be read as float4
  uint32_t c_vec2;       // C may be written as float2 (even ldc, 8-byte aligned base)
  // Pre-quantized activations: `act_image_bytes` per group of rows (see act_image.cuh).
  const uint8_t* act_image;
  uint32_t act_image_bytes;
  uint32_t wait_limit;   // polls a barrier wait makes before it gives up and reports FAULT_WAIT_EXPIRED
  uint32_t drop_first;   // test hook: every CTA leaves out its first weight copy, so that wait runs out
  // Column-split layers over several GPUs (PeerFanout): every output value is also stored into the C
  // of the other ranks, and the last CTA to finish tells every rank that this rank's columns have landed.
  PeerFanout peers;
};

// CG: groups of 16 columns per consumer warp (1: 64-column tiles, 2: 128-column tiles).
template <int DT, bool NT, int CG, int NSK = NS>
struct Geom {
  static constexpr int BB = (DT == AION_CUDA_DTYPE_Q8_0) ? Q8_BYTES : Q4_BYTES;
  static constexpr int TN = 64 * CG;
  static constexpr int KM_PITCH = TN * BB;
  static constexpr int STAGE_BYTES = NT ? TN * NT_ROW_PITCH : KBT * KM_PITCH;
  static constexpr int RING_BYTES = NSK * STAGE_BYTES;
  static constexpr int OFF_BARS = RING_BYTES;
  static constexpr int OFF_ACT = OFF_BARS + (2 * NSK * 8 + 16 + 127) / 128 * 128;   // full / empty barriers, abort flag
  // Distance between a warp's first and second group of 16 columns inside a stage.
  static constexpr int CG_STRIDE = NT ? 64 * NT_ROW_PITCH : 64 * BB;
  static_assert(STAGE_BYTES % 128 == 0, "TMA destinations are 128-byte aligned");
};

// Shared-memory bytes of the quantized activations of `kb` K blocks and `rows` rows:
// 32 code bytes and one f32 scale per (block, row).
__host__ __device__ inline size_t act_bytes(uint32_t kb, uint32_t rows) { return (size_t)kb * rows * 36; }

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
__device__ __forceinline__ uint64_t lds_b64(uint32_t addr) {
  uint64_t v;
  asm("ld.shared.b64 %0, [%1+%2];" : "=l"(v) : "r"(addr), "n"(OFF));
  return v;
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
__device__ __forceinline__ uint64_t pack2i(int lo, int hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// D(16x8, s32) = A(16x32, s8 row) * B(32x8, s8 col) + the bit pattern of 1.5 * 2^23 in every
// element: read as f32 the result is 12582912 + dot, exactly (|dot| <= 32 * 128 * 127 < 2^22).
__device__ __forceinline__ void mma_s8_biased(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(MAGIC_BITS));
}

// The weight side of one K block for one group of 16 columns: the MMA A fragment and, per
// fragment row (column g / column g+8 of the group), the scale pair (s, s) and (-M s, -M s).
struct WeightRegs {
  uint32_t a0, a1, a2, a3;
  uint64_t s0, s1, n0, n1;
};

// K-major: rows g read an even column (codes 2 bytes past a word boundary), rows g+8 the
// odd column after it (aligned). NT: both rows read block KBL of their weight row, whose
// codes are aligned when KBL is odd.
template <int DT, bool NT, int KBL, int STEP, int OFF>
__device__ __forceinline__ void load_weights(WeightRegs& r, uint32_t w0, uint32_t w1, uint32_t b0, uint32_t b1) {
  constexpr bool AL0 = NT ? (KBL & 1) != 0 : false;
  constexpr bool AL1 = NT ? (KBL & 1) != 0 : true;
  load_codes<DT, AL0, KBL * STEP + OFF>(w0, r.a0, r.a2);
  load_codes<DT, AL1, KBL * STEP + OFF>(w1, r.a1, r.a3);
  const float s0 = lds_f16<KBL * STEP + OFF>(b0), s1 = lds_f16<KBL * STEP + OFF>(b1);
  const float m0 = s0 * -MAGIC, m1 = s1 * -MAGIC;  // exact: an f16 value times 3 * 2^22
  r.s0 = pack2(s0, s0);
  r.s1 = pack2(s1, s1);
  r.n0 = pack2(m0, m0);
  r.n1 = pack2(m1, m1);
}

// One K block of a stage: every group of 8 activation rows against every group of 16 columns.
// acc[t][c][0] = (column g of group c) x (activation rows t*8+2j, t*8+2j+1); [1]: column g+8.
template <int DT, bool NT, int MT, int CG, int KBL, int STEP, int CGS, int AQ_STRIDE, int AS_STRIDE>
__device__ __forceinline__ void block_step(uint32_t w0, uint32_t w1, uint32_t b0, uint32_t b1, uint32_t aq, uint32_t as,
                                           uint64_t (&acc)[MT][CG][2]) {
  WeightRegs w[CG];
#pragma unroll
  for (int c = 0; c < CG; c++) load_weights<DT, NT, KBL, STEP, 0>(w[c], w0 + c * CGS, w1 + c * CGS, b0 + c * CGS, b1 + c * CGS);
#pragma unroll
  for (int t = 0; t < MT; t++) {
    // (MT > 1 implies at least 8 rows per K block, so row tile t starts 256 bytes / 8 scales further.)
    const uint2 bq = lds_u64<KBL * AQ_STRIDE>(aq + t * 256);
    const uint64_t sc = lds_b64<KBL * AS_STRIDE>(as + t * 32);
#pragma unroll
    for (int c = 0; c < CG; c++) {
      int d[4];
      mma_s8_biased(d, w[c].a0, w[c].a1, w[c].a2, w[c].a3, bq.x, bq.y);
      acc[t][c][0] = fma2(fma2(pack2i(d[0], d[1]), w[c].s0, w[c].n0), sc, acc[t][c][0]);
      acc[t][c][1] = fma2(fma2(pack2i(d[2], d[3]), w[c].s1, w[c].n1), sc, acc[t][c][1]);
    }
  }
}

// D(16x8, s32) = A(16x32, s8 row) * B(32x8, s8 col), fresh accumulator.
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// ---- up to 16 activation rows, 16 columns per warp: one MMA (or two) per K block -----------------
// Here the weight side is most of the work, and what matters is that the shared-memory loads of
// several K blocks are in flight before the first block's arithmetic needs them: the loads of
// four blocks are issued ahead, spelled out below.
template <int MT>
struct SmallRegs {
  uint32_t a0, a1, a2, a3;  // weight codes: rows g / g+8, low / high half of K
  float s0, s1;             // scales of rows g and g+8
  uint2 bq[MT];             // activation codes
  uint64_t sc[MT];          // activation scales of rows 2j, 2j+1 (a single row: (s, s))
};
template <int DT, bool NT, int MT, int KBL, int STEP, int AQ_STRIDE, int AS_STRIDE>
__device__ __forceinline__ void load_small(SmallRegs<MT>& r, uint32_t w0, uint32_t w1, uint32_t b0, uint32_t b1, uint32_t aq, uint32_t as) {
  constexpr bool AL0 = NT ? (KBL & 1) != 0 : false;
  constexpr bool AL1 = NT ? (KBL & 1) != 0 : true;
  load_codes<DT, AL0, KBL * STEP>(w0, r.a0, r.a2);
  load_codes<DT, AL1, KBL * STEP>(w1, r.a1, r.a3);
  r.s0 = lds_f16<KBL * STEP>(b0);
  r.s1 = lds_f16<KBL * STEP>(b1);
#pragma unroll
  for (int t = 0; t < MT; t++) {
    r.bq[t] = lds_u64<KBL * AQ_STRIDE>(aq + t * 256);
    r.sc[t] = lds_b64<KBL * AS_STRIDE>(as + t * 32);
  }
}
// M1 (a single activation row): acc[0][0][0] holds (column g, column g+8) of that row. Its two useful
// results sit in registers that are not neighbours, so the biased accumulator would cost two moves and a
// multiply more than it saves: two conversion instructions are cheaper here (measured: 2.06 against
// 2.25 us per 9 MB launch).
template <int MT, bool M1>
__device__ __forceinline__ void compute_small(const SmallRegs<MT>& r, uint64_t (&acc)[MT][1][2]) {
  if (M1) {
    int d[4];
    mma_s8(d, r.a0, r.a1, r.a2, r.a3, r.bq[0].x, r.bq[0].y);
    const uint64_t x = pack2((float)d[0], (float)d[2]);
    uint64_t y;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(y) : "l"(x), "l"(pack2(r.s0, r.s1)));
    acc[0][0][0] = fma2(y, r.sc[0], acc[0][0][0]);
    return;
  }
  const float m0 = r.s0 * -MAGIC, m1 = r.s1 * -MAGIC;  // exact: an f16 value times 3 * 2^22
  const uint64_t s0 = pack2(r.s0, r.s0), s1 = pack2(r.s1, r.s1), n0 = pack2(m0, m0), n1 = pack2(m1, m1);
#pragma unroll
  for (int t = 0; t < MT; t++) {
    int d[4];
    mma_s8_biased(d, r.a0, r.a1, r.a2, r.a3, r.bq[t].x, r.bq[t].y);
    acc[t][0][0] = fma2(fma2(pack2i(d[0], d[1]), s0, n0), r.sc[t], acc[t][0][0]);
    acc[t][0][1] = fma2(fma2(pack2i(d[2], d[3]), s1, n1), r.sc[t], acc[t][0][1]);
  }
}

// CTA that owns unit u when G CTAs split U units as [c*U/G, (c+1)*U/G).
__device__ __forceinline__ uint32_t unit_owner(uint64_t u, uint64_t U, uint64_t G) { return (uint32_t)(((u + 1) * G - 1) / U); }

// Quantizes A once per launch into its image (act_image.cuh). Rows past m and blocks past
// kblocks are written as zeros. One thread per (group, block, row).
template <int DT>
__global__ void gemv_act_image_kernel(const float* __restrict__ a, uint64_t lda, uint32_t m, uint32_t kblocks, ActImageLayout L,
                                      uint8_t* __restrict__ image, uint32_t a_vec4) {
  // The matmul that follows may start now: its weight stream does not depend on this kernel,
  // and it waits for this kernel to finish before it copies the image. A comes from the
  // previous kernel, and the image buffer may still be read by an earlier matmul until then.
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint32_t items = L.groups * L.kb_pad * L.rows_per_group;
  const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= items) return;
  const uint32_t r = item % L.rows_per_group, kb = (item / L.rows_per_group) % L.kb_pad, g = item / (L.rows_per_group * L.kb_pad);
  const uint32_t row = g * L.rows_per_group + r;
  uint32_t o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float sc = 0.0f;
  if (row < m && kb < kblocks) sc = quantize_act_block<DT>(a + (uint64_t)row * lda + (uint64_t)kb * QK, a_vec4 != 0, o);
  uint4* dst = reinterpret_cast<uint4*>(act_image_codes(image, L, row, kb));
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  if (row < m || L.rows_per_group != 2) act_image_store_scale(image, L, row, kb, sc);
}

// DT: weight dtype; NT: weights are [n,k] row-major (else K-major); MT: groups of 8 activation
// rows per tile (1, 2, 4, 8); M1: exactly one activation row; RG: A has several groups of
// 8 * MT rows; PREQ: the activation arrives as a pre-quantized image; CG: 16-column groups
// per warp; RW: consumer warps stacked over the activation rows (1: four warps take all MT row
// groups, 2: eight warps, each MT / 2 of them — the warps a scheduler needs to hide the latency
// of the MMA and shared-memory loads once there is this much arithmetic per weight byte).
// Independent small matmuls overlap on an SM, and how many of their CTAs fit decides the
// bandwidth they reach together: the one- and two-MMA variants are held to the registers that
// leave room for seven CTAs per SM (fewer registers measured 4.9 - 5.3 TB/s on 9 MB matrices
// in eight lanes, more 4.6 - 4.8).
constexpr int min_ctas_per_sm(int mt, int cg, int rw, int kw = 1) { return kw > 1 ? 2 : (rw == 2 ? 2 : (mt * cg <= 2 ? 7 : 1)); }

// KW: groups of consumer warps that share a tile's columns and take its stages in turn (stage i goes to group
// i % KW); the groups' sums are added through shared memory when the tile ends. One CTA alone on its tile is
// bound by the latency of a warp's own instruction stream (about 0.6 us per stage with four warps on the SM),
// so the whole-tile variant spreads the stages of a tile over four groups.
template <int DT, bool NT, int MT, bool M1, bool RG, bool PREQ, int CG, int RW, int NSK = NS, int KW = 1>
__global__ void __launch_bounds__(threads_of(RW * KW), min_ctas_per_sm(MT, CG, RW, KW)) gemv_q_mma_kernel(const GemvParams p_in, const __grid_constant__ CUtensorMap tmap) {
  using G = Geom<DT, NT, CG, NSK>;
  constexpr int TN = G::TN;
  constexpr int MPA = 8 * MT;  // activation rows of the accumulator tile
  constexpr int MTW = MT / RW;  // groups of 8 rows per warp
  constexpr int GROUP_WARPS = COL_WARPS * RW;   // the warps that consume one stage together
  constexpr int CONSUMER_WARPS = GROUP_WARPS * KW, CONSUMER_THREADS = CONSUMER_WARPS * 32;
  static_assert(MT % RW == 0, "row groups divide over the row warps");
  static_assert(KW == 1 || (RW == 1 && !RG), "stage groups exist for the variants with a single group of rows");
  // RG: A has more than 8 * MT rows. The tile index then runs over (group of rows, column tile),
  // group-major, and every group streams the weights again (the later ones find them in L2).
  const GemvParams& p = p_in;
  const uint32_t cta = blockIdx.x, n_ctas = gridDim.x;
  constexpr uint32_t MP2 = M1 ? 2 : 8 * MT;  // activation rows held in shared memory
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t smem_base = ptx::smem_u32(smem);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const int wc = warp % COL_WARPS, wr = (warp / COL_WARPS) % RW;  // consumer warp: column position, row half
  const int wk = warp / GROUP_WARPS;                              // its stage group

  const uint64_t U = p.units, NG = n_ctas;
  const uint32_t Sg = p.stages_per_tile;
  uint64_t u_begin, u_end;
  if (p.whole_tiles) {
    u_begin = ((uint64_t)p.tiles * cta / NG) * Sg;
    u_end = ((uint64_t)p.tiles * (cta + 1) / NG) * Sg;
  } else {
    u_begin = U * cta / NG;
    u_end = U * (cta + 1) / NG;
  }

  const uint32_t bar_full = smem_base + G::OFF_BARS;
  const uint32_t bar_empty = bar_full + NSK * 8;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + G::OFF_BARS + 2 * NSK * 8);
  const uint32_t kb_pad = p.stages_per_tile * KBT;  // K blocks rounded up to whole stages
  uint8_t* act_q = smem + G::OFF_ACT;
  float* act_s = reinterpret_cast<float*>(act_q + (size_t)kb_pad * MP2 * 32);  // [kb][MP2] (when the CTA quantizes A itself)
  constexpr uint32_t AQ_SLICE = KBT * MP2 * 32, AS_SLICE = KBT * MP2 * 4;  // one stage's codes / scales of the image

  if (warp == CONSUMER_WARPS) {
    // ---------------- producer: one tiled TMA load per stage ----------------
    // It sets the barriers up itself and starts copying at once; the consumers meet it at
    // the CTA barrier below before they first wait on one.
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap);
      for (int s = 0; s < NSK; s++) {
        ptx::mbar_init(bar_full + 8 * s, 1);
        ptx::mbar_init(bar_empty + 8 * s, GROUP_WARPS);
      }
      *abort_flag = 0;
      ptx::fence_barrier_init();
    }
    __syncwarp();
    const uint64_t n_units = u_end - u_begin;
    uint64_t issued = 0;
    uint32_t tile = (uint32_t)(u_begin / Sg), s = (uint32_t)(u_begin - (uint64_t)tile * Sg);
    // PREQ: every stage also brings its 8 K blocks of the activation image (codes, then scales)
    // into the stage's slot of the activation ring. The image comes from the previous kernel,
    // so those copies wait for it; the weight copies of the first NSK stages do not, and start
    // at once.
    auto issue_acts = [&](uint32_t slot_, uint32_t s_, uint32_t tile_) {
      const uint8_t* image = p.act_image + (RG ? (size_t)(tile_ / p.col_tiles) * p.act_image_bytes : 0);
      const uint32_t dst = smem_base + G::OFF_ACT + slot_ * (AQ_SLICE + AS_SLICE), full = bar_full + 8 * slot_;
      ptx::bulk_g2s(dst, image + (size_t)s_ * AQ_SLICE, AQ_SLICE, full);
      ptx::bulk_g2s(dst + AQ_SLICE, image + (size_t)kb_pad * (MP2 * 32) + (size_t)s_ * AS_SLICE, AS_SLICE, full);
    };
    if (NSK != NS && PREQ && n_units <= (uint64_t)NSK) {
      // Whole-tile variants: the range fits the ring, so nothing is waited for and lane i issues stage i.
      // (One lane issuing eight stages, then their eight pairs of image copies, was 0.1 to 0.2 us per
      // stage on the path every consumer waits on.)
      const uint64_t u = u_begin + lane;
      const uint32_t tile_l = (uint32_t)(u / Sg), s_l = (uint32_t)(u - (uint64_t)tile_l * Sg);
      const bool on = (uint64_t)lane < n_units;
      if (on) {
        const uint32_t full = bar_full + 8 * lane;
        const uint32_t stage = smem_base + lane * G::STAGE_BYTES;
        ptx::mbar_arrive_expect_tx(full, G::STAGE_BYTES + AQ_SLICE + AS_SLICE);
        const uint32_t ct = RG ? tile_l % p.col_tiles : tile_l;
        if (p.drop_first && lane == 0) {
        } else if (!NT && DT == AION_CUDA_DTYPE_Q4_0 && CG == 1) ptx::tma_load_2d(stage, &tmap, (int32_t)(ct * (TN * G::BB / 8)), (int32_t)(s_l * KBT), full);
        else if (!NT) ptx::tma_load_3d(stage, &tmap, 0, (int32_t)(ct * (TN / 8)), (int32_t)(s_l * KBT), full);
        else ptx::tma_load_2d(stage, &tmap, (int32_t)(s_l * KBT * Q8_BYTES / 8), (int32_t)(ct * TN), full);
      }
      __syncwarp();
      __syncthreads();  // CTA barrier #1 (see the consumers)
      ptx::pdl_wait();
      if (on) issue_acts((uint32_t)lane, s_l, tile_l);
      __syncwarp();
      if (*abort_flag)
        for (uint64_t it = 0; it < n_units; it++) ptx::mbar_wait_bounded(bar_full + 8 * (uint32_t)it, 0, min(p.wait_limit, 1u << 16));
      return;
    }
    uint32_t pend_s[NSK], pend_tile[NSK];
    uint32_t npend = 0;
    bool acts_open = !PREQ;
    for (uint64_t it = 0; it < n_units; it++) {
      const uint32_t slot = (uint32_t)(it % NSK);
      if (it == (uint64_t)NSK) __syncthreads();  // CTA barrier #1 (see the consumers)
      if (PREQ && !acts_open && it == (uint64_t)NSK) {
        ptx::pdl_wait();
        if (lane == 0)
          for (uint32_t i = 0; i < npend; i++) issue_acts(i, pend_s[i], pend_tile[i]);
        acts_open = true;
      }
      if (it >= (uint64_t)NSK) {
        if (*abort_flag) break;
        if (!ptx::mbar_wait_bounded(bar_empty + 8 * slot, (uint32_t)((it / NSK) - 1) & 1, p.wait_limit)) {
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
        const uint32_t ct = RG ? tile % p.col_tiles : tile;  // column tile
        // (test hook: the first weight copy is left out, the barrier's byte count never completes, the wait runs out)
        if (p.drop_first && it == 0) {
        } else if (!NT && DT == AION_CUDA_DTYPE_Q4_0 && CG == 1) ptx::tma_load_2d(stage, &tmap, (int32_t)(ct * (TN * G::BB / 8)), (int32_t)(s * KBT), full);
        else if (!NT) ptx::tma_load_3d(stage, &tmap, 0, (int32_t)(ct * (TN / 8)), (int32_t)(s * KBT), full);
        else ptx::tma_load_2d(stage, &tmap, (int32_t)(s * KBT * Q8_BYTES / 8), (int32_t)(ct * TN), full);
        if (PREQ) {
          if (acts_open) issue_acts(slot, s, tile);
          else pend_s[npend] = s, pend_tile[npend] = tile;
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
    if (n_units <= (uint64_t)NSK) __syncthreads();  // CTA barrier #1 when the whole range fit the ring
    if (PREQ && !acts_open) {
      ptx::pdl_wait();
      if (lane == 0)
        for (uint32_t i = 0; i < npend; i++) issue_acts(i, pend_s[i], pend_tile[i]);
    }
    // After a failed wait nobody drains the ring: let the copies still in flight land
    // (bounded) before this CTA's shared memory can be handed to another CTA.
    if (*abort_flag)
      for (uint64_t it = issued > (uint64_t)NSK ? issued - NSK : 0; it < issued; it++)
        ptx::mbar_wait_bounded(bar_full + 8 * (uint32_t)(it % NSK), (uint32_t)(it / NSK) & 1, min(p.wait_limit, 1u << 16));
    return;
  }

  // ---------------- consumers ----------------
  // Scales start at zero: a pad row (m odd) and rows never written must contribute
  // nothing, whatever their code bytes hold (an integer dot is always finite).
  if (!PREQ) {
    float* z = act_s;
    const uint32_t count = kb_pad * MP2;
    for (uint32_t i = tid; i < count; i += CONSUMER_THREADS) z[i] = 0.0f;
  }
  __syncthreads();  // CTA barrier #1: the producer has initialised the mbarriers
  // The next kernel in the stream may begin: its weight stream does not depend on us.
  ptx::pdl_launch_dependents();
  // Everything below reads what the previous kernel wrote (A, and C when beta != 0).
  ptx::pdl_wait();

  if (!PREQ) {
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
      act_s[(size_t)kb * MP2 + r] = sc;
      if (M1) act_s[(size_t)kb * MP2 + 1] = sc;  // the pad row's codes are zero; the lanes read the pair as (s, s)
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");

  // Per-lane constants: where this lane's two weight blocks (rows g and g+8 of the
  // fragment) sit inside a stage, and where its activation fragments start.
  uint32_t off0, off1;
  if (!NT) {
    off0 = (2 * wc + 8 * g) * G::BB;  // an even column: its codes start 2 bytes past a word boundary
    off1 = off0 + G::BB;              // the odd column after it: codes word aligned
  } else {
    off0 = (16 * wc + g) * NT_ROW_PITCH;
    off1 = off0 + 8 * NT_ROW_PITCH;
  }
  const int col0 = NT ? 16 * wc + g : 2 * wc + 8 * g;
  const int col1 = NT ? col0 + 8 : col0 + 1;
  const int row_base = wr * MTW * 8;  // first activation row of this warp's row groups
  // Bytes per K block: MP2 rows of codes, MP2 scales. A lane supplies the codes of activation
  // row t*8+g (absent rows are zero codes with a zero scale) and applies the scales of rows
  // t*8+2j and t*8+2j+1. With a single activation row every lane reads row g % 2 and scale
  // pair 0: the outputs of lanes that stand for absent rows are finite and never stored.
  constexpr uint32_t AQ_STRIDE = MP2 * 32, AS_STRIDE = MP2 * 4;
  const uint32_t act_q_addr = smem_base + G::OFF_ACT;
  const uint32_t act_s_addr = act_q_addr + (PREQ ? KBT : kb_pad) * AQ_STRIDE;  // PREQ: inside a ring slot
  const uint32_t aq_lane = act_q_addr + ((row_base + g) % MP2) * 32 + 8 * j;
  const uint32_t as_lane = act_s_addr + (M1 ? 0 : (row_base + 2 * j) * 4);

  uint64_t acc[MTW][CG][2];
#pragma unroll
  for (int t = 0; t < MTW; t++)
#pragma unroll
    for (int c = 0; c < CG; c++) acc[t][c][0] = acc[t][c][1] = 0ull;

  const uint32_t first_tile = (uint32_t)(u_begin / Sg);
  uint32_t tile = first_tile, s = (uint32_t)(u_begin - (uint64_t)first_tile * Sg);
  bool ok = true;
  uint64_t it = 0;
  for (uint64_t uu = u_begin; uu < u_end; uu++, it++) {
    const uint32_t slot = (uint32_t)(it % NSK);
    const bool my_stage = KW == 1 || (uint32_t)(it % KW) == (uint32_t)wk;
    if (my_stage && ok && (*abort_flag || !ptx::mbar_wait_bounded(bar_full + 8 * slot, (uint32_t)(it / NSK) & 1, p.wait_limit))) {
      if (lane == 0 && !*abort_flag) {
        atomicExch(p.fault, FAULT_WAIT_EXPIRED);
        *abort_flag = 1;
      }
      ok = false;
    }
    if (my_stage && ok) {
      // K blocks past the end of K arrive as zero-filled weights against zero-scaled
      // activations, so all 8 blocks of a stage are always processed.
      uint32_t b0 = smem_base + slot * G::STAGE_BYTES + off0, b1 = smem_base + slot * G::STAGE_BYTES + off1;  // block starts
      uint32_t w0 = b0 + 4 * j, w1 = b1 + 4 * j;  // this lane's code words
      uint32_t aq = aq_lane + (PREQ ? slot * (KBT * (AQ_STRIDE + AS_STRIDE)) : s * (KBT * AQ_STRIDE));
      uint32_t as = as_lane + (PREQ ? slot * (KBT * (AQ_STRIDE + AS_STRIDE)) : s * (KBT * AS_STRIDE));
      // Ties every load below to this point: they cannot move above the wait.
      asm volatile("" : "+r"(w0), "+r"(w1), "+r"(b0), "+r"(b1), "+r"(aq), "+r"(as)::"memory");
      constexpr int STEP = NT ? Q8_BYTES : G::KM_PITCH;
#define AION_BLOCK(K) block_step<DT, NT, MTW, CG, K, STEP, G::CG_STRIDE, (int)AQ_STRIDE, (int)AS_STRIDE>(w0, w1, b0, b1, aq, as, acc)
      if constexpr (MTW * CG <= 2 && RW == 1) {
        SmallRegs<MTW> r[4];
#define AION_LOAD(K, R) load_small<DT, NT, MTW, K, STEP, (int)AQ_STRIDE, (int)AS_STRIDE>(r[R], w0, w1, b0, b1, aq, as)
        AION_LOAD(0, 0); AION_LOAD(1, 1); AION_LOAD(2, 2); AION_LOAD(3, 3);
        compute_small<MTW, M1>(r[0], acc); AION_LOAD(4, 0);
        compute_small<MTW, M1>(r[1], acc); AION_LOAD(5, 1);
        compute_small<MTW, M1>(r[2], acc); AION_LOAD(6, 2);
        compute_small<MTW, M1>(r[3], acc); AION_LOAD(7, 3);
        compute_small<MTW, M1>(r[0], acc);
        compute_small<MTW, M1>(r[1], acc);
        compute_small<MTW, M1>(r[2], acc);
        compute_small<MTW, M1>(r[3], acc);
#undef AION_LOAD
      } else {
        // Many MMAs per K block: two blocks per trip of a real loop, so that the loop body stays
        // inside the instruction cache closest to the schedulers (unrolled eight times it does not,
        // and the warps then stall on instruction fetch more than on anything else).
#pragma unroll 1
        for (int kb2 = 0; kb2 < KBT; kb2 += 2) {
          AION_BLOCK(0); AION_BLOCK(1);
          w0 += 2 * STEP, w1 += 2 * STEP, b0 += 2 * STEP, b1 += 2 * STEP, aq += 2 * AQ_STRIDE, as += 2 * AS_STRIDE;
        }
      }
#undef AION_BLOCK
      static_assert(KBT == 8, "eight K blocks per stage are spelled out above");
    }
    __syncwarp();
    if (my_stage && lane == 0) ptx::mbar_arrive(bar_empty + 8 * slot);

    if (s == Sg - 1 || uu == u_end - 1) {
      if (KW > 1) {
        // The stage groups' sums meet in shared memory; group 0 adds them in group order and carries on alone.
        uint64_t* red = reinterpret_cast<uint64_t*>(smem + G::OFF_ACT + (PREQ ? (size_t)NSK * act_bytes(KBT, MP2) : act_bytes(kb_pad, MP2)));
        constexpr int PER = MTW * CG * 2;
        if (wk > 0) {
#pragma unroll
          for (int t = 0; t < MTW; t++)
#pragma unroll
            for (int c = 0; c < CG; c++) {
              red[((size_t)(wk - 1) * (GROUP_WARPS * 32) + (tid % (GROUP_WARPS * 32))) * PER + (t * CG + c) * 2] = acc[t][c][0];
              red[((size_t)(wk - 1) * (GROUP_WARPS * 32) + (tid % (GROUP_WARPS * 32))) * PER + (t * CG + c) * 2 + 1] = acc[t][c][1];
              acc[t][c][0] = acc[t][c][1] = 0ull;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");
        if (wk == 0) {
          for (int k2 = 0; k2 < KW - 1; k2++)
#pragma unroll
            for (int t = 0; t < MTW; t++)
#pragma unroll
              for (int c = 0; c < CG; c++) {
                const uint64_t x0 = red[((size_t)k2 * (GROUP_WARPS * 32) + tid) * PER + (t * CG + c) * 2];
                const uint64_t x1 = red[((size_t)k2 * (GROUP_WARPS * 32) + tid) * PER + (t * CG + c) * 2 + 1];
                asm("add.rn.f32x2 %0, %0, %1;" : "+l"(acc[t][c][0]) : "l"(x0));
                asm("add.rn.f32x2 %0, %0, %1;" : "+l"(acc[t][c][1]) : "l"(x1));
              }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");   // the buffer is free for the CTA's next tile
      }
      if (KW == 1 || wk == 0) {
      // ---------------- this CTA's share of `tile` is complete ----------------
      const uint64_t tile_u0 = (uint64_t)tile * Sg;
      const bool whole = (uu + 1 - tile_u0 == Sg) && (tile_u0 >= u_begin);
      const uint32_t grp = RG ? tile / p.col_tiles : 0;
      const uint32_t n0 = (RG ? tile - grp * p.col_tiles : tile) * TN, r0 = grp * MPA;  // first column / row of the tile
      // v[t][c][0..3] = (col0, row 2j), (col0, row 2j+1), (col1, row 2j), (col1, row 2j+1)
      float v[MTW][CG][4];
#pragma unroll
      for (int t = 0; t < MTW; t++)
#pragma unroll
        for (int c = 0; c < CG; c++) {
          if (M1) {  // a single row: (column g, column g+8) of row 0 in the first accumulator
            unpack2(acc[t][c][0], v[t][c][0], v[t][c][2]);
            v[t][c][1] = v[t][c][3] = 0.0f;
          } else {
            unpack2(acc[t][c][0], v[t][c][0], v[t][c][1]);
            unpack2(acc[t][c][1], v[t][c][2], v[t][c][3]);
          }
          acc[t][c][0] = acc[t][c][1] = 0ull;
        }
      bool store = whole;
      if (!whole) {
        const uint32_t c_first = unit_owner(tile_u0, U, NG), c_last = unit_owner(tile_u0 + Sg - 1, U, NG);
        const uint32_t nparts = c_last - c_first + 1;
        float* mine = p.partials + ((size_t)cta * 2 + (tile == first_tile ? 0 : 1)) * (TN * MPA);
#pragma unroll
        for (int t = 0; t < MTW; t++)
#pragma unroll
          for (int c = 0; c < CG; c++) {
            *reinterpret_cast<float2*>(mine + (col0 + 64 * c) * MPA + row_base + t * 8 + 2 * j) = make_float2(v[t][c][0], v[t][c][1]);
            *reinterpret_cast<float2*>(mine + (col1 + 64 * c) * MPA + row_base + t * 8 + 2 * j) = make_float2(v[t][c][2], v[t][c][3]);
          }
        // The warp's stores are ordered before lane 0's release by the warp barrier; the
        // acquire side orders the last arriver's loads after every earlier release.
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          int* tk = p.tickets + (size_t)tile * GROUP_WARPS + warp;
          int prev;
          asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(prev) : "l"(tk) : "memory");
          last = (prev == (int)nparts - 1);
          if (last) *tk = 0;  // ready for the next launch
        }
        last = __shfl_sync(0xFFFFFFFFu, last, 0);
        if (last) {
          // The last part to arrive adds all of them in CTA order.
#pragma unroll
          for (int t = 0; t < MTW; t++)
#pragma unroll
            for (int c = 0; c < CG; c++) v[t][c][0] = v[t][c][1] = v[t][c][2] = v[t][c][3] = 0.0f;
          // The loads of several parts are issued before the first is added: taken one part at a time each
          // was a separate trip to L2 (about 0.4 us), and this loop is the tail of the kernel's critical path
          // (a tile of a narrow layer is shared by six or seven CTAs). The sums stay in CTA order.
          constexpr int PB = (MTW * CG == 1) ? 4 : 1;   // parts in flight (the wider variants have no registers to spare: 16 requests ran 2.55 -> 3.16 ms with two in flight)
          for (uint32_t part0 = 0; part0 < nparts; part0 += PB) {
            float2 x0[PB][MTW][CG], x1[PB][MTW][CG];
#pragma unroll
            for (int q = 0; q < PB; q++) {
              const uint32_t cc = min(c_first + part0 + q, c_last);
              const uint32_t cc_first_tile = (uint32_t)((U * cc / NG) / Sg);
              const float* src = p.partials + ((size_t)cc * 2 + (tile == cc_first_tile ? 0 : 1)) * (TN * MPA);
#pragma unroll
              for (int t = 0; t < MTW; t++)
#pragma unroll
                for (int c = 0; c < CG; c++) {
                  x0[q][t][c] = __ldcg(reinterpret_cast<const float2*>(src + (col0 + 64 * c) * MPA + row_base + t * 8 + 2 * j));
                  x1[q][t][c] = __ldcg(reinterpret_cast<const float2*>(src + (col1 + 64 * c) * MPA + row_base + t * 8 + 2 * j));
                }
            }
#pragma unroll
            for (int q = 0; q < PB; q++) {
              if (part0 + q >= nparts) break;
#pragma unroll
              for (int t = 0; t < MTW; t++)
#pragma unroll
                for (int c = 0; c < CG; c++) {
                  v[t][c][0] += x0[q][t][c].x; v[t][c][1] += x0[q][t][c].y;
                  v[t][c][2] += x1[q][t][c].x; v[t][c][3] += x1[q][t][c].y;
                }
            }
          }
          store = true;
        }
      }
      if (store && !*abort_flag) {
#pragma unroll
        for (int t = 0; t < MTW; t++)
#pragma unroll
          for (int c = 0; c < CG; c++)
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
              const uint32_t mrow = r0 + row_base + t * 8 + 2 * j + rr;
              if (mrow >= p.m) continue;
              const uint32_t ca = n0 + col0 + 64 * c, cb = n0 + col1 + 64 * c;
              float* row = p.c + (uint64_t)mrow * p.ldc;
              const float va = v[t][c][rr], vb = v[t][c][2 + rr];
              if (!NT && p.c_vec2 && p.beta == 0.0f && cb < p.n) {
                // K-major tiles: the lane's two columns are neighbours, the first one even.
                const float2 o = make_float2(p.alpha * va, p.alpha * vb);
                *reinterpret_cast<float2*>(row + ca) = o;
                for (uint32_t q = 0; q < p.peers.count; q++) *reinterpret_cast<float2*>(p.peers.c[q] + (uint64_t)mrow * p.ldc + ca) = o;
              } else {
                if (ca < p.n) {
                  const float o = (p.beta == 0.0f) ? p.alpha * va : p.alpha * va + p.beta * row[ca];
                  row[ca] = o;
                  for (uint32_t q = 0; q < p.peers.count; q++) p.peers.c[q][(uint64_t)mrow * p.ldc + ca] = o;
                }
                if (cb < p.n) {
                  const float o = (p.beta == 0.0f) ? p.alpha * vb : p.alpha * vb + p.beta * row[cb];
                  row[cb] = o;
                  for (uint32_t q = 0; q < p.peers.count; q++) p.peers.c[q][(uint64_t)mrow * p.ldc + cb] = o;
                }
              }
            }
      }
      }
    }
    if (++s == Sg) {
      s = 0;
      tile++;
    }
  }
  if (p.peers.world > 1) {
    // Every output of this CTA is stored, here and on the peers. The last CTA of the grid to get here
    // publishes the arrival: flags[this rank] = epoch + 1 in every rank's flag array (the epoch is
    // advanced by the wait kernel that follows in the stream). The CTA barrier orders every thread's
    // stores before thread 0's system-scope fence (fences are cumulative), the fence before the counter;
    // the last CTA's fence after the counter orders every CTA's stores before its flag stores.
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");
    if (tid == 0) {
      __threadfence_system();
      const uint32_t prev = atomicAdd(p.peers.state + 1, 1u);
      if (prev == gridDim.x - 1) {
        __threadfence_system();
        p.peers.state[1] = 0;   // ready for the next launch
        const uint32_t next = *reinterpret_cast<volatile uint32_t*>(p.peers.state) + 1;
        for (uint32_t r = 0; r < p.peers.world; r++)
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peers.flags[r] + p.peers.rank), "r"(next) : "memory");
      }
    }
  }
}

// Waits (bounded) until every rank's arrival word has reached epoch + 1, then advances the epoch.
// One warp; lane r watches rank r. A wait that runs out reports FAULT_WAIT_EXPIRED and leaves the
// epoch where it was.
// Launched with programmatic stream serialization, so its one CTA is resident and its launch off the critical
// path while the matmul that announces this rank's own columns runs; but it reads the epoch only after that
// matmul has completed (griddepcontrol.wait). The matmul's CTAs let their dependents start before they wait
// for their own predecessors, so without that wait this kernel could start while the wait kernel of the step
// before was still polling, read the epoch that kernel was about to advance, pass at once and leave the epoch
// one step behind for good: the peers then wait for an arrival word that never comes (seen on 8 GPUs, where a
// step's wait lasts longest; 2 and 4 GPUs happened to stay clear of it).
__global__ void peer_wait_kernel(const uint32_t* flags, uint32_t* state, uint32_t world, uint32_t poll_limit, int* fault) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint32_t lane = threadIdx.x;
  const uint32_t want = *reinterpret_cast<volatile uint32_t*>(state) + 1;
  bool ok = true;
  if (lane < world) {
    ok = false;
    for (uint32_t i = 0; i < poll_limit; i++) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
      if ((int32_t)(v - want) >= 0) {
        ok = true;
        break;
      }
      __nanosleep(64);
    }
  }
  const bool all = __all_sync(0xFFFFFFFFu, ok);
  if (lane == 0) {
    if (all) *state = want;
    else atomicCAS(fault, FAULT_NONE, FAULT_WAIT_EXPIRED);
  }
}

// Per device and kernel instantiation: the largest dynamic shared-memory size the kernel has
// been allowed so far (the attribute is only ever raised) and the occupancy found for the
// last size asked. Shared by every launch path of the instantiation and safe to call from
// several host threads.
struct KernelSetup {
  std::mutex mu;
  size_t configured_smem[64] = {};
  size_t occ_smem[64] = {};
  int occ_blocks[64] = {};
};

template <typename Kernel>
int32_t kernel_occupancy(KernelSetup& ks, Kernel kernel, AionCudaDevice* dev, int threads, size_t smem, int* blocks_per_sm) {
  if (dev->ordinal < 0 || dev->ordinal >= 64) return fail(AION_CUDA_UNSUPPORTED, "gemv: device ordinal %d is beyond the 64 this library keeps state for", dev->ordinal);
  std::lock_guard<std::mutex> lock(ks.mu);
  const int di = dev->ordinal;
  if (smem > ks.configured_smem[di]) {
    AION_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ks.configured_smem[di] = smem;
  }
  if (ks.occ_smem[di] != smem) {
    int nb = 0;
    AION_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kernel, threads, smem));
    if (nb < 1) return fail(AION_CUDA_INTERNAL_ERROR, "gemv: kernel does not fit an SM with %llu bytes of shared memory", (unsigned long long)smem);
    ks.occ_blocks[di] = nb;
    ks.occ_smem[di] = smem;
  }
  *blocks_per_sm = ks.occ_blocks[di];
  return AION_CUDA_OK;
}

template <int DT, bool NT, int MT, bool M1, bool RG, bool PREQ, int CG, int RW, int NSK = NS, int KW = 1>
KernelSetup& setup_of() {
  static KernelSetup ks;
  return ks;
}

template <int DT, bool NT, int CG>
int32_t encode_weight_map(const uint8_t* b, uint64_t ldb, uint32_t n, uint32_t kblocks, AionCudaDevice* cache_dev, CUtensorMap* local,
                          const CUtensorMap** out) {
  using G = Geom<DT, NT, CG>;
  uint64_t dims[3], strides[2];
  uint32_t box[3], rank;
  if (!NT && DT == AION_CUDA_DTYPE_Q4_0 && CG == 1) {
    // [kblocks][n*18 bytes]: one box = 8 block rows x 64 blocks (1152 bytes, within the 2048-byte box row).
    rank = 2;
    dims[0] = (uint64_t)n * G::BB, dims[1] = kblocks;
    strides[0] = ldb * G::BB;
    box[0] = (uint32_t)G::TN * G::BB, box[1] = KBT;
  } else if (!NT) {
    // A row of TN blocks can exceed what a box row holds (2048 bytes), so the row is viewed as
    // [n/8 groups][8 blocks]: one box = 8 block rows x TN/8 groups.
    rank = 3;
    dims[0] = 8ull * G::BB, dims[1] = n / 8, dims[2] = kblocks;
    strides[0] = 8ull * G::BB, strides[1] = ldb * G::BB;
    box[0] = 8u * G::BB, box[1] = G::TN / 8, box[2] = KBT;
  } else {
    // [n rows][kblocks*34 bytes]: one box = TN rows x 8 blocks.
    rank = 2;
    dims[0] = (uint64_t)kblocks * Q8_BYTES, dims[1] = n;
    strides[0] = ldb * Q8_BYTES;
    box[0] = NT_ROW_PITCH, box[1] = G::TN;
  }
  if (cache_dev) return tensor_map_bytes(cache_dev, b, rank, dims, strides, box, out);
  if (int32_t st = tensor_map_encode(b, rank, dims, strides, box, local)) return st;
  *out = local;
  return AION_CUDA_OK;
}

// Returned by the whole-tile variant when the shape does not suit it; the caller then takes the streaming one.
constexpr int32_t DECLINED = -0x7A11;

template <int DT, bool NT, int MT, bool M1, bool RG, bool PREQ, int CG, int RW, int NSK = NS, int KW = 1>
int32_t launch(AionCudaDevice* dev, GemvParams p, const uint8_t* b, uint64_t ldb, const uint8_t* given_image) {
  using G = Geom<DT, NT, CG, NSK>;
  constexpr int TN = G::TN;
  constexpr int THREADS = threads_of(RW * KW);
  constexpr bool WHOLE = NSK != NS;   // one whole tile per CTA, every stage of it in the ring at once
  auto kernel = gemv_q_mma_kernel<DT, NT, MT, M1, RG, PREQ, CG, RW, NSK, KW>;
  constexpr uint32_t MP2 = M1 ? 2 : 8 * MT;
  constexpr size_t RED_BYTES = (size_t)(KW - 1) * COL_WARPS * RW * 32 * (MT / RW) * CG * 2 * sizeof(uint64_t);   // the stage groups' sums
  const size_t smem = G::OFF_ACT + (PREQ ? (size_t)NSK * act_bytes(KBT, MP2) : act_bytes(p.stages_per_tile * KBT, MP2)) + RED_BYTES;
  int per_sm = 0;
  if (int32_t st = kernel_occupancy(setup_of<DT, NT, MT, M1, RG, PREQ, CG, RW, NSK, KW>(), kernel, dev, THREADS, smem, &per_sm)) return st;
  uint64_t grid = (uint64_t)per_sm * dev->sm_count;
  if (WHOLE) {
    // A deeper K is cut into ranges of NSK stages: still every weight byte of a CTA in flight at once, and the
    // few CTAs that share a tile add their parts up as in the streaming variant.
    const uint64_t want = p.stages_per_tile <= (uint32_t)NSK ? (uint64_t)p.tiles : ceil_div(p.units, (uint64_t)NSK);
    if (want > grid) return DECLINED;
    grid = want;
  }
  if (dev->gemv_split_override && !WHOLE) grid = (uint64_t)dev->gemv_split_override * dev->sm_count;  // CTAs per SM, tuning only
  if (grid > p.units) grid = p.units;
  // Small problems: fewer, fuller CTAs — about eight stages each, but never fewer than one
  // CTA per SM. Their launches are latency-bound, and independent ones recorded in
  // parallel lanes then share the GPU (measured on 9 MB q4 matrices: 148 CTAs in 8 lanes
  // stream 3.5 TB/s, 256 or 444 CTAs 2.6 to 3.0 TB/s).
  if (!dev->gemv_split_override && MT <= 2 && !WHOLE) {
    const uint64_t sms = (uint64_t)dev->sm_count;
    uint64_t want = p.units / 8;
    if (want < sms) want = sms;
    if (grid > want) grid = want;
    if (grid > p.units) grid = p.units;
    // Nearly one tile per CTA while independent steps are being recorded into parallel lanes:
    // give every CTA exactly one whole tile (other launches fill the idle SMs).
    bool overlapped = false;
    if (dev->recording) {
      overlapped = dev->cur_lane != 0;
      for (int l = 1; l < AionCudaDevice::LANES; l++) overlapped = overlapped || dev->lane_forked[l];
    }
    if (overlapped && (uint64_t)p.tiles <= grid && (uint64_t)p.tiles * 5 >= grid * 4) grid = p.tiles;
    // Tiles shared by several CTAs: a grid that cuts every tile into the same number of equal parts, so that
    // no CTA straddles two tiles (one set of partial sums and one ticket per CTA, and the parts of a tile end
    // together). 2048 x 8192 q4 in 8 lanes: 2.16 us per launch with 256 CTAs against 2.47 with 148.
    if (!WHOLE && (uint64_t)p.tiles < grid) {
      const uint64_t cap = (uint64_t)per_sm * dev->sm_count;
      for (uint64_t d = 1; d <= p.stages_per_tile; d++)
        if (p.stages_per_tile % d == 0 && (uint64_t)p.tiles * d >= grid) {
          if ((uint64_t)p.tiles * d <= cap) grid = (uint64_t)p.tiles * d;
          break;
        }
    }
  }
  // At least as many tiles as CTAs: hand out whole tiles, so that no tile is shared and the
  // partial-sum fix-up (two more L2 round trips at the end of a short kernel) is skipped —
  // unless rounding to tiles would leave the busiest CTA more than a fifth above the average.
  p.whole_tiles = 0;
  if ((uint64_t)p.tiles >= grid) {
    const uint64_t most = ceil_div((uint64_t)p.tiles, grid);
    if (most * grid * 5 <= (uint64_t)p.tiles * 6) p.whole_tiles = 1;
  }

  // Scratch for tiles shared by several CTAs: two partial slots per CTA, one ticket per (tile, warp),
  // times the groups of 8 * MT rows.
  constexpr int MPA = 8 * MT;
  const uint64_t groups = p.tiles / p.col_tiles;
  // (The whole-tile variant also reserves what the streaming variant of the same step would ask for: a step
  // run once on its own and then recorded into parallel lanes takes that variant, and a recording cannot grow scratch.)
  uint64_t fix_ctas = grid;
  if (WHOLE) {
    const uint64_t streaming = std::min<uint64_t>(p.units, 7ull * (uint64_t)dev->sm_count);
    if (streaming > fix_ctas) fix_ctas = streaming;
  }
  if (int32_t st = dev->reserve_gemv_fixup((size_t)fix_ctas * 2 * TN * MPA * sizeof(float), (size_t)p.tiles * COL_WARPS * RW)) return st;
  p.partials = dev->lane_gemv_partials();
  p.tickets = dev->lane_gemv_tickets();

  static const bool no_pdl_main = std::getenv("AION_CUDA_NO_PDL_MAIN") != nullptr;  // tuning only
  if (PREQ) {
    const ActImageLayout L = act_image_layout_int8(p.m, p.kblocks);
    if (L.rows_per_group != MP2 || L.groups != groups || L.kb_pad != p.stages_per_tile * KBT)
      return fail(AION_CUDA_INTERNAL_ERROR, "gemv: activation image layout does not match the kernel chosen");
    if (given_image) {
      p.act_image = given_image;
    } else {
      // Quantize A once, into lane scratch, in the layout the CTAs copy into shared memory.
      if (int32_t st = dev->reserve_scratch(act_image_total_bytes(L))) return st;
      uint8_t* image = static_cast<uint8_t*>(dev->lane_scratch());
      const uint32_t items = L.groups * L.kb_pad * L.rows_per_group;
      cudaLaunchConfig_t icfg{};
      icfg.gridDim = dim3((items + 127) / 128);
      icfg.blockDim = dim3(128);
      icfg.stream = dev->stream;
      cudaLaunchAttribute iattrs[1];
      iattrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      iattrs[0].val.programmaticStreamSerializationAllowed = 1;
      icfg.attrs = iattrs;
      icfg.numAttrs = no_pdl_main ? 0 : 1;
      prefer_max_shared(reinterpret_cast<const void*>(gemv_act_image_kernel<DT>));
      AION_CUDA_TRY(cudaLaunchKernelEx(&icfg, gemv_act_image_kernel<DT>, p.a, p.lda, p.m, p.kblocks, L, image, p.a_vec4));
      p.act_image = image;
    }
    p.act_image_bytes = L.group_bytes;
  }

  const CUtensorMap* tm = nullptr;
  if (int32_t st = encode_weight_map<DT, NT, CG>(b, ldb, p.n, p.kblocks, dev, nullptr, &tm)) return st;

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = no_pdl_main ? 0 : 1;
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  AION_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p, *tm));
  return AION_CUDA_OK;
}

template <int DT, bool NT>
int32_t launch_m(AionCudaDevice* dev, const GemvParams& p, const uint8_t* b, uint64_t ldb, const uint8_t* image) {
  // (The streaming variants, which a launch takes when the whole-tile variant below does not apply.)
  // m >= 2: A is quantized once by a small kernel (or by the kernel that produced A) instead of
  // by every CTA. m = 1 quantizes its one row inside the kernel when the launch stands alone on a
  // chain (one kernel less: 10.6 against 11.8 us for a lone 9 MB launch) and K is shallow (past
  // about 3000 the small kernel is cheaper than 148 CTAs each quantizing the whole row). Independent
  // launches recorded into parallel lanes are bound by how soon each CTA starts to consume its
  // weights, and the quantization prologue is a seventh of a CTA's life there: with the small
  // kernel the 9 MB bench shape streams 5.4 - 5.7 TB/s instead of 4.9 - 5.2 (row-major NT weights
  // measured 3 % slower that way and keep the in-kernel prologue).
  bool overlapped = false;
  if (dev->recording) {
    overlapped = dev->cur_lane != 0;
    for (int l = 1; l < AionCudaDevice::LANES; l++) overlapped = overlapped || dev->lane_forked[l];
  }
  // A launch on a dependent chain (a decode step) with a shallow K: one whole tile per CTA and a ring that holds
  // all of its stages. The weights do not depend on the previous kernel, so all of them are on their way (or
  // already in shared memory) before that kernel has finished, and once it has, what is left is the activation
  // image's copy, the arithmetic and the store: no tile is shared, so no partial sums, tickets or second pass.
  // Measured inside a decode step of 8 requests (1536-wide layers): 5.8 to 10 us per matmul after its
  // predecessor has finished with the streaming variant.
  static const bool no_whole = std::getenv("AION_CUDA_GEMV_NO_WHOLE") != nullptr;   // tuning only
  // Recorded into parallel lanes, the streaming variant is the faster one (more CTAs of more launches per SM)
  // except for a small matrix, whose few tiles leave most SMs to the other lanes anyway: 2048 x 2048 q4 in
  // 8 lanes measured 1.04 us per launch with whole tiles against 1.59 us, 8192 x 2048 2.98 against 1.92 us.
  const bool few_tiles = p.stages_per_tile <= (uint32_t)NS_DEEP && (uint64_t)p.tiles * 4 <= (uint64_t)dev->sm_count;
  const bool whole = !no_whole && (!overlapped || few_tiles) && !dev->gemv_split_override && p.m <= 16;
  if (whole) {
    int32_t st;
    // A single row without an image and a K of at most eight stages: the CTA quantizes the row itself while its
    // weights are on their way (one kernel less on the chain than with the image kernel in front).
    if (p.m == 1 && !image && p.stages_per_tile <= (uint32_t)NS_DEEP) st = launch<DT, NT, 1, true, false, false, 1, 1, NS_DEEP, KW_DEEP>(dev, p, b, ldb, nullptr);
    else if (p.m == 1) st = launch<DT, NT, 1, true, false, true, 1, 1, NS_DEEP, KW_DEEP>(dev, p, b, ldb, image);
    else if (p.m <= 8) st = launch<DT, NT, 1, false, false, true, 1, 1, NS_DEEP, KW_DEEP>(dev, p, b, ldb, image);
    else st = launch<DT, NT, 2, false, false, true, 1, 1, NS_DEEP, KW_DEEP>(dev, p, b, ldb, image);
    if (st != DECLINED) return st;
  }
  if (p.m == 1) {
    return (image || p.kblocks > 96 || (overlapped && !NT)) ? launch<DT, NT, 1, true, false, true, 1, 1>(dev, p, b, ldb, image)
                                                            : launch<DT, NT, 1, true, false, false, 1, 1>(dev, p, b, ldb, nullptr);
  }
  if (p.m <= 8) return launch<DT, NT, 1, false, false, true, 1, 1>(dev, p, b, ldb, image);
  if (p.m <= 16) return launch<DT, NT, 2, false, false, true, 1, 1>(dev, p, b, ldb, image);
  if (p.m <= 32) return launch<DT, NT, 4, false, false, true, 2, 2>(dev, p, b, ldb, image);
  if (p.m <= 64) return launch<DT, NT, 8, false, false, true, 2, 2>(dev, p, b, ldb, image);
  return launch<DT, NT, 8, false, true, true, 2, 2>(dev, p, b, ldb, image);  // groups of 64 rows
}

}  // namespace

int32_t gemv_mma(AionCudaDevice* dev, const MatMulArgs& g, bool probe_only) {
  if (g.m > (1ull << 22) || g.k == 0) return AION_CUDA_UNSUPPORTED;
  if (g.n > 0x7FFFFFFFull - 128 || g.k / QK > 0x7FFFFFFFull) return AION_CUDA_UNSUPPORTED;
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

  // m = 1 with a shallow K quantizes its row inside the kernel, in K chunks that fit the per-CTA
  // budget, issued as several launches that accumulate into C, like the reference's walk over
  // K in chunks (src/aion/backend/cpu/exec/matmul.zig:431-434). Every other case streams the
  // activation image with the weights: any depth in one launch.
  // An image laid out for the tensor-core GEMM (this many rows, but the int8 kernel was asked for) is not
  // ours to read: A is quantized here instead.
  const uint8_t* image = (g.a_image && act_image_layout(g.m, kblocks).kind == ACT_IMAGE_INT8) ? g.a_image : nullptr;
  uint64_t kb_max = (ACT_BUDGET_BYTES / 72) / KBT * KBT;
  bool lanes = false;
  if (dev->recording) {
    lanes = dev->cur_lane != 0;
    for (int l = 1; l < AionCudaDevice::LANES; l++) lanes = lanes || dev->lane_forked[l];
  }
  if (g.m >= 2 || kblocks > 96 || image || (lanes && !g.nt)) kb_max = (kblocks + KBT - 1) / KBT * KBT;
  // A single row takes the image kernel only when recorded into parallel lanes: the run before the
  // recording (which quantizes in the kernel) reserves the image's scratch for it.
  if (g.m == 1 && !g.nt && !image && !dev->recording)
    if (int32_t st = dev->reserve_scratch(act_image_total_bytes(act_image_layout_int8(1, kblocks)))) return st;
  if (g.peers && kblocks > kb_max) return AION_CUDA_UNSUPPORTED;   // the fan-out belongs to a single launch

  for (uint64_t kb0 = 0; kb0 < kblocks; kb0 += kb_max) {
    const uint64_t nkb = kblocks - kb0 < kb_max ? kblocks - kb0 : kb_max;
    GemvParams p{};
    p.a = g.a + kb0 * QK;
    p.c = g.c;
    p.m = (uint32_t)g.m;
    p.n = (uint32_t)g.n;
    p.kblocks = (uint32_t)nkb;
    p.lda = g.lda;
    p.ldc = g.ldc;
    p.alpha = g.alpha;
    p.beta = kb0 == 0 ? g.beta : 1.0f;
    const uint32_t tn = g.m > 16 ? 128u : 64u;
    const uint64_t row_groups = g.m <= 64 ? 1 : ceil_div(g.m, (uint64_t)64);
    p.col_tiles = (uint32_t)((g.n + tn - 1) / tn);
    if ((uint64_t)p.col_tiles * row_groups > 0x7FFFFFFFull) return AION_CUDA_UNSUPPORTED;
    p.tiles = (uint32_t)(p.col_tiles * row_groups);
    p.stages_per_tile = (uint32_t)((nkb + KBT - 1) / KBT);
    p.units = (uint64_t)p.tiles * p.stages_per_tile;
    p.fault = dev->fault_dev;
    p.wait_limit = dev->debug_expire_waits ? (1u << 8) : (1u << 20);
    p.drop_first = dev->debug_expire_waits ? 1u : 0u;
    if (g.peers) p.peers = *g.peers;
    p.a_vec4 = (g.a && (reinterpret_cast<uintptr_t>(p.a) & 15) == 0 && g.lda % 4 == 0) ? 1u : 0u;
    p.c_vec2 = ((reinterpret_cast<uintptr_t>(p.c) & 7) == 0 && g.ldc % 2 == 0) ? 1u : 0u;
    int32_t st;
    if (g.nt) {
      st = launch_m<AION_CUDA_DTYPE_Q8_0, true>(dev, p, g.b + kb0 * Q8_BYTES, g.ldb, image);
    } else if (g.dtype == AION_CUDA_DTYPE_Q8_0) {
      st = launch_m<AION_CUDA_DTYPE_Q8_0, false>(dev, p, g.b + kb0 * g.ldb * Q8_BYTES, g.ldb, image);
    } else {
      st = launch_m<AION_CUDA_DTYPE_Q4_0, false>(dev, p, g.b + kb0 * g.ldb * Q4_BYTES, g.ldb, image);
    }
    if (st != AION_CUDA_OK) return st;
  }
  return AION_CUDA_OK;
}

int32_t peer_wait_launch(AionCudaDevice* dev, const uint32_t* flags, uint32_t* state, uint32_t world, uint32_t poll_limit) {
  AION_CUDA_TRY(launch_pdl_main(peer_wait_kernel, dim3(1), dim3(32), 0, dev->stream, flags, state, world, poll_limit, dev->fault_dev));
  return AION_CUDA_OK;
}

// Fills an activation image from f32 rows (the library's own producer of images; the fused
// producers in the other files write the same bytes).
int32_t act_image_from_f32(AionCudaDevice* dev, uint32_t dtype, const float* a, uint64_t m, uint64_t k, uint64_t lda, uint8_t* image) {
  const ActImageLayout L = act_image_layout(m, k / QK);
  if (L.kind == ACT_IMAGE_BF16) return act_image_bf16_from_f32(dev, dtype, a, m, k, lda, image);
  const uint32_t items = L.groups * L.kb_pad * L.rows_per_group;
  const uint32_t vec4 = ((reinterpret_cast<uintptr_t>(a) & 15) == 0 && lda % 4 == 0) ? 1u : 0u;
  if (dtype == AION_CUDA_DTYPE_Q8_0)
    AION_CUDA_TRY(launch_pdl_main(gemv_act_image_kernel<AION_CUDA_DTYPE_Q8_0>, dim3((items + 127) / 128), dim3(128), 0, dev->stream, a, lda,
                                  (uint32_t)m, (uint32_t)(k / QK), L, image, vec4));
  else
    AION_CUDA_TRY(launch_pdl_main(gemv_act_image_kernel<AION_CUDA_DTYPE_Q4_0>, dim3((items + 127) / 128), dim3(128), 0, dev->stream, a, lda,
                                  (uint32_t)m, (uint32_t)(k / QK), L, image, vec4));
  return AION_CUDA_OK;
}

// ------------------------------------------------------------------------------------
// The same matmul for callers that must not allocate (see aion_cuda_matmul_static_scratch
// in the header). The split-tile partial sums and their arrival counters live in this
// file-scope array instead of in memory the device object grows on demand. Every GPU that
// loads the library holds the array until the process exits.
// ------------------------------------------------------------------------------------
namespace {

constexpr uint32_t STATIC_MAX_CTAS = 512;    // grid is clamped to this
constexpr uint32_t STATIC_MAX_TILES = 8192;  // n <= 524288
constexpr size_t STATIC_PARTIAL_BYTES = (size_t)STATIC_MAX_CTAS * 2 * 64 * 8 * sizeof(float);  // m <= 8
constexpr size_t STATIC_TICKET_BYTES = (size_t)STATIC_MAX_TILES * COL_WARPS * sizeof(int);

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_PARTIAL_BYTES + STATIC_TICKET_BYTES];

// In host code `g_static_scratch` is only a stand-in for the symbol, not a device
// address: each device's address is looked up once, with that device current.
std::mutex g_static_scratch_mu;
unsigned char* g_static_scratch_addr[64] = {};

template <int DT, bool M1>
int32_t launch_static(AionCudaDevice* dev, GemvParams p, const uint8_t* b, uint64_t ldb, unsigned char* scratch) {
  using G = Geom<DT, false, 1>;
  // The same instantiation aion_cuda_matmul uses for these shapes: they share its set-up state.
  auto kernel = gemv_q_mma_kernel<DT, false, 1, M1, false, false, 1, 1>;
  constexpr uint32_t MP2 = M1 ? 2 : 8;
  constexpr int THREADS = threads_of(1);
  const size_t smem = G::OFF_ACT + act_bytes(p.stages_per_tile * KBT, MP2);
  int per_sm = 0;
  if (int32_t st = kernel_occupancy(setup_of<DT, false, 1, M1, false, false, 1, 1>(), kernel, dev, THREADS, smem, &per_sm)) return st;
  uint64_t grid = (uint64_t)per_sm * dev->sm_count;
  if (grid > p.units) grid = p.units;
  if (grid > STATIC_MAX_CTAS) grid = STATIC_MAX_CTAS;
  p.whole_tiles = 0;
  p.partials = reinterpret_cast<float*>(scratch);
  p.tickets = reinterpret_cast<int*>(scratch + STATIC_PARTIAL_BYTES);
  // The counters must start at zero whatever an earlier call left behind.
  AION_CUDA_TRY(cudaMemsetAsync(p.tickets, 0, (size_t)p.tiles * COL_WARPS * sizeof(int), dev->stream));
  CUtensorMap local;
  const CUtensorMap* tm = nullptr;
  if (int32_t st = encode_weight_map<DT, false, 1>(b, ldb, p.n, p.kblocks, nullptr, &local, &tm)) return st;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  AION_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p, *tm));
  return AION_CUDA_OK;
}

}  // namespace

int32_t gemv_mma_static_scratch(AionCudaDevice* dev, const MatMulArgs& g) {
  if (g.m == 0 || g.n == 0) return AION_CUDA_OK;
  if (g.m > 8)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: m = %llu, the built-in scratch holds at most 8 rows", (unsigned long long)g.m);
  if (g.k == 0 || g.k / QK > 0x7FFFFFFFull || g.n > (uint64_t)STATIC_MAX_TILES * 64)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: n = %llu, k = %llu are outside the built-in scratch (n <= %u, k >= 32)",
                (unsigned long long)g.n, (unsigned long long)g.k, STATIC_MAX_TILES * 64);
  const uint64_t kblocks = g.k / QK;
  if (g.nt || (reinterpret_cast<uintptr_t>(g.b) & 15) != 0 || g.n % 8 != 0 || g.ldb % 8 != 0)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: the tiled kernel does not read this shape or alignment");
  // One launch holds the whole quantized activation in shared memory: 16384 columns of K for one
  // row, 4096 for up to eight.
  const uint64_t kb_max = g.m == 1 ? 512 : 128;
  static_assert(512 * 2 * 36 <= ACT_BUDGET_BYTES && 128 * 8 * 36 <= ACT_BUDGET_BYTES, "static-scratch K limits fit the activation budget");
  if (kblocks > kb_max)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: k = %llu with m = %llu exceeds one launch (k <= %llu)",
                (unsigned long long)g.k, (unsigned long long)g.m, (unsigned long long)(kb_max * QK));
  if (dev->ordinal < 0 || dev->ordinal >= 64)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: device ordinal %d is beyond the 64 this library keeps state for", dev->ordinal);

  // First call on this device: find where the array lives on it.
  unsigned char* scratch;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (!g_static_scratch_addr[dev->ordinal]) {
      unsigned char* ptr = nullptr;
      AION_CUDA_TRY(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
      g_static_scratch_addr[dev->ordinal] = ptr;
    }
    scratch = g_static_scratch_addr[dev->ordinal];
  }

  GemvParams p{};
  p.a = g.a;
  p.c = g.c;
  p.m = (uint32_t)g.m;
  p.n = (uint32_t)g.n;
  p.kblocks = (uint32_t)kblocks;
  p.lda = g.lda;
  p.ldc = g.ldc;
  p.alpha = g.alpha;
  p.beta = g.beta;
  p.tiles = p.col_tiles = (uint32_t)((g.n + 63) / 64);
  p.stages_per_tile = (uint32_t)((kblocks + KBT - 1) / KBT);
  p.units = (uint64_t)p.tiles * p.stages_per_tile;
  p.fault = dev->fault_dev;
  p.wait_limit = 1u << 20;
  p.a_vec4 = ((reinterpret_cast<uintptr_t>(p.a) & 15) == 0 && g.lda % 4 == 0) ? 1u : 0u;
  p.c_vec2 = ((reinterpret_cast<uintptr_t>(p.c) & 7) == 0 && g.ldc % 2 == 0) ? 1u : 0u;
  if (g.dtype == AION_CUDA_DTYPE_Q8_0)
    return g.m == 1 ? launch_static<AION_CUDA_DTYPE_Q8_0, true>(dev, p, g.b, g.ldb, scratch)
                    : launch_static<AION_CUDA_DTYPE_Q8_0, false>(dev, p, g.b, g.ldb, scratch);
  return g.m == 1 ? launch_static<AION_CUDA_DTYPE_Q4_0, true>(dev, p, g.b, g.ldb, scratch)
                  : launch_static<AION_CUDA_DTYPE_Q4_0, false>(dev, p, g.b, g.ldb, scratch);
}

}  // namespace aion
