// Prefill GEMM for q4_0 / q8_0 K-major weights on the 5th-generation tensor cores:
// C[m,n] = alpha * A[m,k] . dequant(B)[k,n] + beta * C for m beyond the decode GEMV.
//
// This is the one dense contraction of the hot path, so unlike the GEMV it is tensor-pipe
// bound. Arithmetic: A is quantized to int8 per 32-block as the reference does and its
// dequantized value rounded to bf16, B is dequantized to bf16 (w = code * scale), products
// accumulate in f32 in tensor memory; against the reference's int8-activation CPU arithmetic
// (src/aion/backend/cpu/kernels/matmul_q_i8.zig:385-497) that is the same product with both
// factors rounded to bf16, bounded by rel-L2 1e-2 (observed about 2e-3).
//
// Shape of the kernel (one persistent CTA per SM, 128 x 256 output tiles, K in steps of 64):
//   warp 0      TMA producer of bf16 activation tiles (128B-swizzled, straight into the MMA
//               operand layout); warp 2: TMA producer of the packed weight blocks, untouched.
//   warps 3-14  dequantizers: packed blocks -> bf16 -> the 128B-swizzled K-major operand
//               layout in shared memory (one generic-proxy pass; the packed bytes cannot be
//               fed to the tensor core as they are), then a proxy fence and an arrive.
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (M=128 tokens, N=256
//               columns, K=16) four times per stage into one of two TMEM accumulators and
//               commits to the stage's "empty" barrier; it also owns TMEM alloc / dealloc.
//   warps 15-18 epilogue: tcgen05.ld the finished accumulator, alpha / beta in f32, store.
// The activation is converted to bf16 once by a pre-pass (so every column tile re-reads
// 2 bytes per element from L2 instead of converting 4), with the order of K inside each
// group of 8 permuted for q4 to match the order in which a 32-bit word of nibbles
// unpacks; a permutation of K applied to both operands does not change the product.
// Every mbarrier wait is bounded; on expiry the kernel records a fault, stops issuing and
// still frees its tensor memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <mutex>

#include "act_image.cuh"
#include "common.cuh"
#include "ptx.cuh"
#include "quant_device.cuh"

namespace aion {

namespace {

constexpr int BM = 128;      // tokens per MMA (UMMA M); a tile holds MH of these halves (1 or 2)
constexpr int BN = 256;      // output columns per tile (UMMA N)
constexpr int BK = 64;       // K per stage: one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int MAX_A_STAGES = 4, MAX_P_STAGES = 6, MAX_B_STAGES = 3;
constexpr int KB_PER_STAGE = BK / QK;   // 2 quantized blocks of each column per stage
constexpr int DEQ_GROUPS = 3;           // groups of dequantizer warps; group g unpacks k-stages g, g + 3, ...
constexpr int DEQ_WARPS = 4 * DEQ_GROUPS;   // 12: measured against 6 (slower: each warp is a latency chain) and 24 (no faster)
constexpr int DEQ_WARP0 = 3;            // warp 0: activation TMA, warp 1: MMA, warp 2: packed-block TMA
constexpr int EPI_WARP0 = DEQ_WARP0 + DEQ_WARPS;
constexpr int THREADS = (EPI_WARP0 + 4) * 32;
constexpr int A_HALF_BYTES = BM * BK * 2;   // 16 KB: activation rows of one MMA
constexpr int B_TILE_BYTES = BN * BK * 2;   // 32 KB
constexpr uint32_t TMEM_COLS = 512;         // two f32 accumulators of 256 columns

struct GemmParams {
  float* c;
  uint32_t m, n, k;
  uint64_t ldc;
  float alpha, beta;
  uint32_t m_tiles, n_tiles, k_stages;
  uint32_t splits;    // K splits per tile (work unit = tile x split); > 1 goes through `partial`
  float* partial;     // [tile][split][BM * MH][BN] raw accumulators
  uint32_t tile_rows; // BM * MH
  int* fault;
  uint32_t wait_shift;  // poll limits of the bounded waits are shifted right by this much (test hook)
  uint32_t drop_first;  // test hook: every CTA leaves out its first packed-weight copy, so a wait runs out
};

template <int DT, int MH>
struct GemmGeom {
  static constexpr int A_TILE_BYTES = MH * A_HALF_BYTES;
  static constexpr int BB = (DT == AION_CUDA_DTYPE_Q8_0) ? Q8_BYTES : Q4_BYTES;
  static constexpr int PACKED_ROW = BN * BB;                       // one block row of the tile
  static constexpr int PACKED_BYTES = KB_PER_STAGE * PACKED_ROW;   // 9216 (q4) / 17408 (q8)
  static constexpr int PACKED_PAD = (PACKED_BYTES + 16 + 1023) / 1024 * 1024;  // +16: the unpacker reads one word past
  // Three rings, so each resource is released as early as its last reader allows: packed
  // blocks after dequantization, activation tiles and dequantized tiles after their MMAs.
  // B_STAGES equals the number of dequantizer groups and P_STAGES is a multiple of it, so
  // every "free" barrier is waited on by one group only, use after use: a parity wait is
  // only meaningful for a waiter that is at most one phase behind.
  static constexpr int A_STAGES = MH == 1 ? 4 : (DT == AION_CUDA_DTYPE_Q8_0 ? 2 : 3);
  static constexpr int P_STAGES = (DT == AION_CUDA_DTYPE_Q8_0 || MH == 2) ? 3 : 6;
  static constexpr int B_STAGES = DEQ_GROUPS;
  static_assert(P_STAGES % DEQ_GROUPS == 0, "a packed stage belongs to one dequantizer group");
  static constexpr int OFF_BRING = 0;
  static constexpr int OFF_ARING = OFF_BRING + B_STAGES * B_TILE_BYTES;
  static constexpr int OFF_PRING = OFF_ARING + A_STAGES * A_TILE_BYTES;
  static constexpr int OFF_BARS = OFF_PRING + P_STAGES * PACKED_PAD;
  static constexpr int SMEM_BYTES = OFF_BARS + 256 + 1024;  // + slack to align the base to 1024
  static_assert(A_STAGES <= MAX_A_STAGES && P_STAGES <= MAX_P_STAGES && B_STAGES <= MAX_B_STAGES, "barrier block");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

// ---- activation pre-pass: f32 -> the reference's int8 quantization -> bf16 ---------------
// Row-major [m, k] bf16 with k a multiple of 32. Every 32-block of A is quantized to int8 exactly
// as the reference CPU kernels quantize it (src/aion/backend/cpu/kernels/matmul_q_i8.zig:187-203)
// and the value written is code * scale rounded to bf16: the GEMM then multiplies the operands
// the reference multiplies, and differs from it only by the bf16 rounding of both. (Rounding the
// raw activation to bf16 instead leaves the whole int8 quantization error, about 5e-3, between
// the two.) Four consecutive threads hold one block, eight elements each.
// `permute`: inside every group of 8 consecutive k, position p holds element (p >> 1) + 4 * (p & 1),
// i.e. the order e0 e4 e1 e5 e2 e6 e3 e7 in which a word of q4 nibbles unpacks two at a time.
__global__ void __launch_bounds__(256) convert_a_bf16_kernel(const float* __restrict__ a, uint64_t lda, __nv_bfloat16* __restrict__ out, uint32_t m,
                                                             uint32_t k, int permute) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint64_t groups = (uint64_t)m * (k / 8), stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t trips = (groups + stride - 1) / stride;
  uint64_t gi = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
  for (uint64_t trip = 0; trip < trips; trip++, gi += stride) {  // every lane makes every trip: the shuffles need whole warps
    const bool on = gi < groups;
    const uint64_t gq = on ? gi : 0;
    const uint32_t r = (uint32_t)(gq / (k / 8)), g8 = (uint32_t)(gq % (k / 8));
    const float* src = a + (uint64_t)r * lda + (uint64_t)g8 * 8;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = on ? src[i] : 0.0f;
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    float scale, inv;
    activation_block_scales(amax, &scale, &inv);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __fmul_rn((float)quantize_activation_with_inv(v[i], inv), scale);
    __nv_bfloat162 o[4];
    if (permute) {
#pragma unroll
      for (int i = 0; i < 4; i++) o[i] = __floats2bfloat162_rn(v[i], v[i + 4]);
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++) o[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    }
    if (on) *reinterpret_cast<uint4*>(out + (uint64_t)r * k + (uint64_t)g8 * 8) = *reinterpret_cast<const uint4*>(o);
  }
}

// ---- tcgen05 / TMEM wrappers ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem desc] . B[smem desc]^T, bf16 x bf16 -> f32, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major, 128-byte swizzle, rows of 128 bytes, groups of
// 8 rows 1024 bytes apart. (Start address and offsets are in 16-byte units; bit 46 is the
// descriptor version of this architecture; layout type 2 = 128-byte swizzle.)
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// Instruction descriptor: D f32, A and B bf16, both K-major, M = 128, N = 256.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// Byte offset of 16-byte chunk `c` (0..7) of row `r` inside a 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t r, uint32_t c) { return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4); }

__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Barrier block at the end of shared memory.
struct Bars {
  uint64_t a_full[MAX_A_STAGES];   // TMA landed an activation tile
  uint64_t a_empty[MAX_A_STAGES];  // the MMAs that read it are done
  uint64_t p_full[MAX_P_STAGES];   // TMA landed a stage of packed blocks
  uint64_t p_empty[MAX_P_STAGES];  // every dequantizer warp has read it
  uint64_t bready[MAX_B_STAGES];   // a dequantized weight tile is written
  uint64_t bfree[MAX_B_STAGES];    // the MMAs that read it are done
  uint64_t acc_full[2];            // an accumulator holds a finished tile
  uint64_t acc_empty[2];           // the epilogue has drained it
  uint32_t tmem_base;
  uint32_t abort;
};
static_assert(sizeof(Bars) <= 256, "barrier block");

// What a bounded wait needs: the CTA's abort flag, and by how many bits the poll limits are shortened
// (0 in production; the test hook of aion_cuda_debug_expire_waits sets it so a wait that cannot complete
// gives up within milliseconds).
struct WaitCtx {
  volatile uint32_t* abort_flag;
  uint32_t shift;
};
// Bounded wait that also gives up as soon as another role has aborted.
template <bool SPIN = false>
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, const WaitCtx& w) {
  const uint32_t b = ptx::smem_u32(bar);
  const uint32_t limit = (SPIN ? (1u << 24) : (1u << 18)) >> w.shift;
  for (uint32_t i = 0; i < limit; i++) {
    if (SPIN ? ptx::mbar_try_wait_spin(b, parity) : ptx::mbar_try_wait(b, parity)) return true;
    if ((!SPIN || (i & 63) == 63) && *w.abort_flag) return false;
  }
  return false;
}
__device__ __noinline__ void raise_abort(int* fault, volatile uint32_t* abort_flag) {
  *abort_flag = 1;
  atomicCAS(fault, FAULT_NONE, FAULT_WAIT_EXPIRED);
}

// One q4_0 block (scale + 16 code bytes at a 2-byte aligned shared address) -> 32 bf16
// weights, written as four 16-byte chunks of operand row `row`, chunks c0..c0+3. Word i of
// the codes holds elements 8i..8i+7, one per nibble; they leave in the order
// e0 e4 e1 e5 e2 e6 e3 e7 (the activation pre-pass applies the same order).
__device__ __forceinline__ void dequant_q4_block(uint32_t blk, uint8_t* btile, uint32_t row, uint32_t c0) {
  const float s = f16_bits_to_float((uint16_t)ptx::lds16(blk));
  const uint32_t s2 = pack_bf16x2(s, s);
  const uint32_t cb = blk + 2, al = cb & ~3u, sh = (cb & 3u) * 8;
  uint32_t l[5];
#pragma unroll
  for (int i = 0; i < 5; i++) l[i] = ptx::lds32(al + 4 * i);
  constexpr uint32_t MAGIC = 0x43004300u;   // bf16 128.0 twice: OR-ing a nibble gives 128 + nibble exactly
  constexpr uint32_t ONE = 0x3F803F80u;     // 1.0
  constexpr uint32_t NEG136 = 0xC308C308u;  // -(128 + 8)
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t w = __funnelshift_r(l[i], l[i + 1], sh);
    uint4 out;
    out.x = bf16x2_mul(bf16x2_fma((w & 0x000F000Fu) | MAGIC, ONE, NEG136), s2);
    out.y = bf16x2_mul(bf16x2_fma(((w >> 4) & 0x000F000Fu) | MAGIC, ONE, NEG136), s2);
    out.z = bf16x2_mul(bf16x2_fma(((w >> 8) & 0x000F000Fu) | MAGIC, ONE, NEG136), s2);
    out.w = bf16x2_mul(bf16x2_fma(((w >> 12) & 0x000F000Fu) | MAGIC, ONE, NEG136), s2);
    *reinterpret_cast<uint4*>(btile + sw128_offset(row, c0 + i)) = out;
  }
}

// One q8_0 block -> 32 bf16 weights in natural K order. A byte b becomes the f16 value
// 1024 + (b ^ 0x80) by byte permutation, 1152 is subtracted exactly, the scale is applied
// in f32 and the product rounded once to bf16.
__device__ __forceinline__ void dequant_q8_block(uint32_t blk, uint8_t* btile, uint32_t row, uint32_t c0) {
  const float s = f16_bits_to_float((uint16_t)ptx::lds16(blk));
  const uint32_t cb = blk + 2, al = cb & ~3u, sh = (cb & 3u) * 8;
  uint32_t l[9];
#pragma unroll
  for (int i = 0; i < 9; i++) l[i] = ptx::lds32(al + 4 * i);
  const __half2 bias = __float2half2_rn(1152.0f);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t u = __funnelshift_r(l[2 * i + h], l[2 * i + h + 1], sh) ^ 0x80808080u;
      const uint32_t h01 = __byte_perm(u, 0x64646464u, 0x5140);
      const uint32_t h23 = __byte_perm(u, 0x64646464u, 0x7362);
      const __half2 y01 = __hsub2(*reinterpret_cast<const __half2*>(&h01), bias);
      const __half2 y23 = __hsub2(*reinterpret_cast<const __half2*>(&h23), bias);
      o[2 * h] = pack_bf16x2(__low2float(y01) * s, __high2float(y01) * s);
      o[2 * h + 1] = pack_bf16x2(__low2float(y23) * s, __high2float(y23) * s);
    }
    *reinterpret_cast<uint4*>(btile + sw128_offset(row, c0 + i)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Work unit u = tile * splits + split; the splits of a tile walk disjoint, nearly equal
// ranges of the k-stages.
struct Unit {
  uint32_t tile, split, ks0, ks1;
};
__device__ __forceinline__ Unit unit_of(const GemmParams& p, uint32_t u) {
  Unit w;
  w.tile = u / p.splits;
  w.split = u - w.tile * p.splits;
  w.ks0 = (uint32_t)((uint64_t)p.k_stages * w.split / p.splits);
  w.ks1 = (uint32_t)((uint64_t)p.k_stages * (w.split + 1) / p.splits);
  return w;
}

template <int DT, int MH>
__global__ void __launch_bounds__(THREADS, 1)
gemm_q_tcgen05_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b) {
  using G = GemmGeom<DT, MH>;
  // MH == 1: two accumulators of 256 columns, so the epilogue of a tile overlaps the MMAs of
  // the next. MH == 2: the two halves of one 256-token tile fill all 512 columns; one
  // dequantized weight tile then feeds two MMAs, which halves the dequantizer work per flop.
  constexpr uint32_t NACC = MH == 1 ? 2 : 1, ACC_COLS = MH * BN;
  constexpr int A_TILE_BYTES = G::A_TILE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  // Swizzled operand tiles need 1024-byte alignment.
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  Bars* bars = reinterpret_cast<Bars*>(sm + G::OFF_BARS);
  volatile uint32_t* abort_flag = &bars->abort;
  const WaitCtx wctx{abort_flag, p.wait_shift};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t AS = G::A_STAGES, PS = G::P_STAGES, BS = G::B_STAGES;
  if (threadIdx.x == 0) {
    for (int s = 0; s < (int)AS; s++) {
      ptx::mbar_init(ptx::smem_u32(&bars->a_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->a_empty[s]), 1);
    }
    for (int s = 0; s < (int)PS; s++) {
      ptx::mbar_init(ptx::smem_u32(&bars->p_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->p_empty[s]), DEQ_WARPS / DEQ_GROUPS);
    }
    for (int s = 0; s < (int)BS; s++) {
      ptx::mbar_init(ptx::smem_u32(&bars->bready[s]), DEQ_WARPS / DEQ_GROUPS);
      ptx::mbar_init(ptx::smem_u32(&bars->bfree[s]), 1);
    }
    for (int a = 0; a < 2; a++) {
      ptx::mbar_init(ptx::smem_u32(&bars->acc_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->acc_empty[a]), 4);
    }
    bars->abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(ptx::smem_u32(&bars->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Everything above touched only this CTA's shared and tensor memory. The activation (and C, and the scratch
  // of the split partials) belong to earlier kernels: the warp that loads activation tiles and the epilogue
  // warps wait for those (griddepcontrol.wait). The packed weights do not, so their loads and their unpacking
  // start at once: on a decode chain the first dequantized tiles are ready before the activation exists.
  ptx::pdl_launch_dependents();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t units = p.m_tiles * p.n_tiles * p.splits;

  if (warp == 0) {
    // ---- TMA producer of activation tiles ----
    if (lane == 0) {
      ptx::pdl_wait();
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const Unit w = unit_of(p, u);
        const int32_t m0 = (int32_t)((w.tile % p.m_tiles) * (BM * MH));
        for (uint32_t ks = w.ks0; ks < w.ks1; ks++, it++) {
          const uint32_t s = it % AS, use = it / AS;
          if (use > 0 && !wait_or_abort<true>(&bars->a_empty[s], (use - 1) & 1, wctx)) {
            raise_abort(p.fault, abort_flag);
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&bars->a_full[s]);
          ptx::mbar_arrive_expect_tx(full, A_TILE_BYTES);
          ptx::tma_load_2d(base + G::OFF_ARING + s * A_TILE_BYTES, &tmap_a, (int32_t)(ks * BK), m0, full);
        }
      }
    }
  } else if (warp == 2) {
    // ---- TMA producer of packed weight blocks ----
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const Unit w = unit_of(p, u);
        const int32_t n0 = (int32_t)((w.tile / p.m_tiles) * BN);
        for (uint32_t ks = w.ks0; ks < w.ks1; ks++, it++) {
          const uint32_t s = it % PS, use = it / PS;
          if (use > 0 && !wait_or_abort<true>(&bars->p_empty[s], (use - 1) & 1, wctx)) {
            raise_abort(p.fault, abort_flag);
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&bars->p_full[s]);
          ptx::mbar_arrive_expect_tx(full, G::PACKED_BYTES);
          if (p.drop_first && it == 0) continue;   // (test hook: the bytes never arrive, the dequantizers' wait runs out)
          ptx::tma_load_3d(base + G::OFF_PRING + s * G::PACKED_PAD, &tmap_b, 0, n0 / 8, (int32_t)(ks * KB_PER_STAGE), full);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    uint32_t it = 0, tile_iter = 0;
    bool ok = true;
    for (uint32_t u = blockIdx.x; u < units && ok; u += gridDim.x, tile_iter++) {
      const Unit w = unit_of(p, u);
      const uint32_t acc = tile_iter % NACC, acc_use = tile_iter / NACC;
      if (acc_use > 0 && !wait_or_abort<true>(&bars->acc_empty[acc], (acc_use - 1) & 1, wctx)) {
        if (lane == 0) raise_abort(p.fault, abort_flag);
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
      for (uint32_t ks = w.ks0; ks < w.ks1; ks++, it++) {
        const uint32_t sa = it % AS, pha = (it / AS) & 1, sb = it % BS, phb = (it / BS) & 1;
        if (!wait_or_abort<true>(&bars->a_full[sa], pha, wctx) || !wait_or_abort<true>(&bars->bready[sb], phb, wctx)) {
          if (lane == 0) raise_abort(p.fault, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint64_t a_desc = smem_desc_sw128(base + G::OFF_ARING + sa * A_TILE_BYTES);
          const uint64_t b_desc = smem_desc_sw128(base + G::OFF_BRING + sb * B_TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; kk++)
#pragma unroll
            for (int h = 0; h < MH; h++)
              umma_bf16(d_tmem + h * BN, a_desc + (uint64_t)((h * A_HALF_BYTES + kk * UMMA_K * 2) / 16),
                        b_desc + (uint64_t)(kk * UMMA_K * 2 / 16), kInstrDesc, ((ks - w.ks0) | (uint32_t)kk) != 0);
          umma_commit(ptx::smem_u32(&bars->a_empty[sa]));
          umma_commit(ptx::smem_u32(&bars->bfree[sb]));
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(ptx::smem_u32(&bars->acc_full[acc]));
      __syncwarp();
    }
  } else if (warp < EPI_WARP0) {
    // ---- dequantizers: DEQ_GROUPS groups of warps take the k-stages in turn, so that
    // several stages are being unpacked at once and one stage's wait / load / fence
    // latency hides behind another's arithmetic. Thread j of a group owns weight
    // columns (operand rows) j, j + GROUP_THREADS, ... of the tile.
    constexpr uint32_t GROUP_WARPS = DEQ_WARPS / DEQ_GROUPS, GROUP_THREADS = GROUP_WARPS * 32;
    const uint32_t dw = warp - DEQ_WARP0, group = dw / GROUP_WARPS, j0 = (dw % GROUP_WARPS) * 32 + lane;
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const Unit w = unit_of(p, u);
      for (uint32_t ks = w.ks0; ks < w.ks1; ks++, it++) {
        if (it % DEQ_GROUPS != group) continue;
        const uint32_t sp = it % PS, php = (it / PS) & 1, sb = it % BS, buse = it / BS;
        if (!wait_or_abort<true>(&bars->p_full[sp], php, wctx) ||
            (buse > 0 && !wait_or_abort<true>(&bars->bfree[sb], (buse - 1) & 1, wctx))) {
          if (lane == 0) raise_abort(p.fault, abort_flag);
          ok = false;
          break;
        }
        const uint32_t packed = base + G::OFF_PRING + sp * G::PACKED_PAD;
        uint8_t* btile = sm + G::OFF_BRING + sb * B_TILE_BYTES;
#pragma unroll
        for (int rr = 0; rr < BN / (int)GROUP_THREADS; rr++) {
          const uint32_t row = j0 + rr * GROUP_THREADS;
#pragma unroll
          for (int kbl = 0; kbl < KB_PER_STAGE; kbl++) {
            const uint32_t blk = packed + kbl * G::PACKED_ROW + row * G::BB;
            if (DT == AION_CUDA_DTYPE_Q4_0) dequant_q4_block(blk, btile, row, kbl * 4);
            else dequant_q8_block(blk, btile, row, kbl * 4);
          }
        }
        ptx::fence_proxy_async();  // the tensor core reads this tile through the async proxy
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(ptx::smem_u32(&bars->p_empty[sp]));
          ptx::mbar_arrive(ptx::smem_u32(&bars->bready[sb]));
        }
      }
    }
  } else {
    // ---- epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31 ----
    ptx::pdl_wait();
    const uint32_t quarter = warp & 3;
    uint32_t tile_iter = 0;
    for (uint32_t u = blockIdx.x; u < units; u += gridDim.x, tile_iter++) {
      const Unit w = unit_of(p, u);
      const uint32_t acc = tile_iter % NACC, acc_use = tile_iter / NACC;
      if (!wait_or_abort(&bars->acc_full[acc], acc_use & 1, wctx)) {
        if (lane == 0) raise_abort(p.fault, abort_flag);
        break;
      }
      tc_fence_after();
      const uint32_t m0 = (w.tile % p.m_tiles) * (BM * MH), n0 = (w.tile / p.m_tiles) * BN;
#pragma unroll 1
      for (int h = 0; h < MH; h++) {
        const uint32_t trow = h * BM + quarter * 32 + lane, row = m0 + trow;
        float* crow = p.c + (uint64_t)row * p.ldc + n0;
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * ACC_COLS + h * BN;
        // Split K: the raw accumulator goes to this unit's slot; a follow-up kernel adds the slots
        // of every tile in split order, so the sum does not depend on timing.
        float* slot = p.partial + ((size_t)w.tile * p.splits + w.split) * ((size_t)BM * MH * BN) + (size_t)trow * BN;
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
          if (row < p.m) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
              const uint32_t col = n0 + c0 + q * 4;
              if (col >= p.n) continue;  // n is a multiple of 8, so a group of 4 is in or out as a whole
              float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                                     __uint_as_float(r[4 * q + 3]));
              if (p.splits > 1) {
                __stcg(reinterpret_cast<float4*>(slot + c0 + q * 4), v);
                continue;
              }
              v.x *= p.alpha, v.y *= p.alpha, v.z *= p.alpha, v.w *= p.alpha;
              float4* dst = reinterpret_cast<float4*>(crow + c0 + q * 4);
              if (p.beta != 0.0f) {
                const float4 o = *dst;
                v.x += p.beta * o.x, v.y += p.beta * o.y, v.z += p.beta * o.z, v.w += p.beta * o.w;
              }
              *dst = v;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars->acc_empty[acc]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- two-SM variant: a pair of CTAs (a cluster of two) shares every MMA -----------------------
// tcgen05.mma.cta_group::2 multiplies 256 tokens by 256 weight columns per instruction: each CTA
// of the pair holds 128 of the tokens (its A rows, its accumulator lanes) and HALF of the weight
// columns of the B operand. So each SM unpacks, stages and feeds the tensor core half as many
// weight bytes per flop as the one-SM kernel; shared-memory bandwidth, not the tensor pipe, is what
// limits that kernel. The even CTA of the pair (the leader) issues the MMAs for both.
// Signals that cross the pair:
//   * activation tiles: both CTAs' TMA loads complete on the leader's a_full barrier;
//   * dequantized half tiles: the peer's dequantizers arrive on the leader's bready barrier;
//   * MMA completion: one commit arrives on a_empty / bfree / acc_full of both CTAs;
//   * drained accumulators: the peer's epilogue arrives on the leader's acc_empty barrier.
constexpr int BNH = BN / 2;                  // weight columns unpacked per CTA
constexpr int BH_TILE_BYTES = BNH * BK * 2;  // 16 KB
constexpr int PAIR_B_STAGES = 2 * DEQ_GROUPS;

template <int DT, int MH>
struct PairGeom {
  static constexpr int A_TILE_BYTES = MH * A_HALF_BYTES;
  static constexpr int BB = (DT == AION_CUDA_DTYPE_Q8_0) ? Q8_BYTES : Q4_BYTES;
  static constexpr int PACKED_ROW = BNH * BB;
  static constexpr int PACKED_BYTES = KB_PER_STAGE * PACKED_ROW;   // 4608 (q4) / 8704 (q8)
  static constexpr int PACKED_PAD = (PACKED_BYTES + 16 + 1023) / 1024 * 1024;
  static constexpr int A_STAGES = MH == 1 ? 4 : 3;
  static constexpr int P_STAGES = DT == AION_CUDA_DTYPE_Q8_0 ? 3 : 6;
  // Two dequantized half tiles per dequantizer group where the MMAs of a stage are short (one per
  // k-step); one where a stage carries two and the staging buffers below need the room.
  static constexpr int B_STAGES = MH == 1 ? PAIR_B_STAGES : DEQ_GROUPS;
  static_assert(P_STAGES % DEQ_GROUPS == 0 && B_STAGES % DEQ_GROUPS == 0, "a stage belongs to one dequantizer group");
  // Output staging: every epilogue warp has two buffers of 32 rows x 32 columns f32 (one swizzle
  // row per output row), filled from tensor memory and written out by bulk tensor stores.
  static constexpr int OUT_BUF_BYTES = 32 * 128;
  static constexpr int OUT_BYTES = 4 * 2 * OUT_BUF_BYTES;
  static constexpr int OFF_BRING = 0;
  static constexpr int OFF_ARING = OFF_BRING + B_STAGES * BH_TILE_BYTES;
  static constexpr int OFF_PRING = OFF_ARING + A_STAGES * A_TILE_BYTES;
  static constexpr int OFF_OUT = OFF_PRING + P_STAGES * PACKED_PAD;
  static constexpr int OFF_BARS = OFF_OUT + OUT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BARS + 512 + 1024;  // barrier block + slack to align the base to 1024
  static_assert(A_STAGES <= MAX_A_STAGES && P_STAGES <= MAX_P_STAGES && B_STAGES <= PAIR_B_STAGES, "barrier block");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct PairBars {
  uint64_t a_full[MAX_A_STAGES];
  uint64_t a_empty[MAX_A_STAGES];
  uint64_t p_full[MAX_P_STAGES];
  uint64_t p_empty[MAX_P_STAGES];
  uint64_t bready[PAIR_B_STAGES];
  uint64_t bfree[PAIR_B_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
};
static_assert(sizeof(PairBars) <= 512, "barrier block");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier that may live in the other CTA of the cluster. What the arrival publishes is
// this CTA's own shared memory (read by this SM's half of the MMA) or its drained tensor memory, so
// the default CTA-scope release is enough; a cluster-scope release measured about 1900 cycles per
// arrival and made the dequantizers the bottleneck.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on a barrier whose arrivals may come from the other CTA.
__device__ __forceinline__ bool wait_cluster_or_abort(uint64_t* bar, uint32_t parity, const WaitCtx& w) {
  const uint32_t b = ptx::smem_u32(bar);
  const uint32_t limit = (1u << 24) >> w.shift;
  for (uint32_t i = 0; i < limit; i++) {
    if (mbar_try_wait_cluster(b, parity)) return true;
    if ((i & 63) == 63 && *w.abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this offset in BOTH CTAs once every MMA issued so far is done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"((uint16_t)3)
               : "memory");
}
// Tiled load whose completion bytes are counted on a barrier of the pair's leader.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tmap, int32_t x, int32_t y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
      "l"(tmap), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
      "%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// Bulk tensor store of one staged box (shared -> global); out-of-range rows and columns are clipped.
__device__ __forceinline__ void tma_store_2d(const void* tmap, int32_t x, int32_t y, uint32_t src_smem) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tmap), "r"(x), "r"(y), "r"(src_smem)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most `N` of this thread's bulk groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Instruction descriptor of the pair's MMA: D f32, A and B bf16, both K-major, M = 256, N = 256.
constexpr uint32_t kInstrDescPair = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);

template <int DT, int MH>
__global__ void __launch_bounds__(THREADS, 1)
gemm_q_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_c) {
  using G = PairGeom<DT, MH>;
  constexpr uint32_t ACC_COLS = MH * BN;   // all 512 columns when MH == 2: one accumulator set
  constexpr uint32_t NACC = MH == 1 ? 2 : 1;
  constexpr int A_TILE_BYTES = G::A_TILE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  PairBars* bars = reinterpret_cast<PairBars*>(sm + G::OFF_BARS);
  volatile uint32_t* abort_flag = &bars->abort;
  const WaitCtx wctx{abort_flag, p.wait_shift};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0: leader
  const bool leader = rank == 0;
  constexpr uint32_t AS = G::A_STAGES, PS = G::P_STAGES, BS = G::B_STAGES;
  if (threadIdx.x == 0) {
    for (int s = 0; s < (int)AS; s++) {
      ptx::mbar_init(ptx::smem_u32(&bars->a_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->a_empty[s]), 1);
    }
    for (int s = 0; s < (int)PS; s++) {
      ptx::mbar_init(ptx::smem_u32(&bars->p_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->p_empty[s]), DEQ_WARPS / DEQ_GROUPS);
    }
    for (int s = 0; s < (int)BS; s++) {
      ptx::mbar_init(ptx::smem_u32(&bars->bready[s]), 2 * (DEQ_WARPS / DEQ_GROUPS));   // both CTAs' warps
      ptx::mbar_init(ptx::smem_u32(&bars->bfree[s]), 1);
    }
    for (int a = 0; a < 2; a++) {
      ptx::mbar_init(ptx::smem_u32(&bars->acc_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->acc_empty[a]), 8);   // four epilogue warps of each CTA
    }
    bars->abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc2(ptx::smem_u32(&bars->tmem_base), TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the other CTA's barriers and tensor memory exist from here on
  tc_fence_after();
  // (as in the one-SM kernel: only the activation loads and the epilogue wait for the earlier kernels)
  ptx::pdl_launch_dependents();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t units = p.m_tiles * p.n_tiles * p.splits;
  const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ---- TMA producer of this CTA's activation rows ----
    if (lane == 0) {
      ptx::pdl_wait();
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t u = pair; u < units && ok; u += pairs) {
        const Unit w = unit_of(p, u);
        const int32_t m0 = (int32_t)((w.tile % p.m_tiles) * (2 * BM * MH) + rank * BM);
        for (uint32_t ks = w.ks0; ks < w.ks1; ks++, it++) {
          const uint32_t s = it % AS, use = it / AS;
          if (use > 0 && !wait_or_abort<true>(&bars->a_empty[s], (use - 1) & 1, wctx)) {
            raise_abort(p.fault, abort_flag);
            ok = false;
            break;
          }
          const uint32_t full_local = ptx::smem_u32(&bars->a_full[s]);
          if (leader) ptx::mbar_arrive_expect_tx(full_local, 2 * A_TILE_BYTES);
          const uint32_t full = map_to_cta(full_local, 0);
#pragma unroll
          for (int h = 0; h < MH; h++)
            tma_load_2d_pair(base + G::OFF_ARING + s * A_TILE_BYTES + h * A_HALF_BYTES, &tmap_a, (int32_t)(ks * BK), m0 + h * 2 * BM, full);
        }
      }
    }
  } else if (warp == 2) {
    // ---- TMA producer of this CTA's half of the packed weight blocks ----
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t u = pair; u < units && ok; u += pairs) {
        const Unit w = unit_of(p, u);
        const int32_t n0 = (int32_t)((w.tile / p.m_tiles) * BN + rank * BNH);
        for (uint32_t ks = w.ks0; ks < w.ks1; ks++, it++) {
          const uint32_t s = it % PS, use = it / PS;
          if (use > 0 && !wait_or_abort<true>(&bars->p_empty[s], (use - 1) & 1, wctx)) {
            raise_abort(p.fault, abort_flag);
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&bars->p_full[s]);
          ptx::mbar_arrive_expect_tx(full, G::PACKED_BYTES);
          if (p.drop_first && it == 0) continue;   // (test hook: the bytes never arrive, the dequantizers' wait runs out)
          ptx::tma_load_3d(base + G::OFF_PRING + s * G::PACKED_PAD, &tmap_b, 0, n0 / 8, (int32_t)(ks * KB_PER_STAGE), full);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader's, for both CTAs ----
    if (leader) {
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (uint32_t u = pair; u < units && ok; u += pairs, tile_iter++) {
        const Unit w = unit_of(p, u);
        const uint32_t acc = tile_iter % NACC, acc_use = tile_iter / NACC;
        if (acc_use > 0 && !wait_cluster_or_abort(&bars->acc_empty[acc], (acc_use - 1) & 1, wctx)) {
          if (lane == 0) raise_abort(p.fault, abort_flag);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (uint32_t ks = w.ks0; ks < w.ks1; ks++, it++) {
          const uint32_t sa = it % AS, pha = (it / AS) & 1, sb = it % BS, phb = (it / BS) & 1;
          if (!wait_cluster_or_abort(&bars->a_full[sa], pha, wctx) || !wait_cluster_or_abort(&bars->bready[sb], phb, wctx)) {
            if (lane == 0) raise_abort(p.fault, abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint64_t a_desc = smem_desc_sw128(base + G::OFF_ARING + sa * A_TILE_BYTES);
            const uint64_t b_desc = smem_desc_sw128(base + G::OFF_BRING + sb * BH_TILE_BYTES);
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; kk++)
#pragma unroll
              for (int h = 0; h < MH; h++)
                umma_bf16_pair(d_tmem + h * BN, a_desc + (uint64_t)((h * A_HALF_BYTES + kk * UMMA_K * 2) / 16),
                               b_desc + (uint64_t)(kk * UMMA_K * 2 / 16), kInstrDescPair, ((ks - w.ks0) | (uint32_t)kk) != 0);
            umma_commit_pair(ptx::smem_u32(&bars->a_empty[sa]));
            umma_commit_pair(ptx::smem_u32(&bars->bfree[sb]));
          }
          __syncwarp();
        }
        if (ok && lane == 0) umma_commit_pair(ptx::smem_u32(&bars->acc_full[acc]));
        __syncwarp();
      }
    }
  } else if (warp < EPI_WARP0) {
    // ---- dequantizers: thread j of a group owns weight column j of this CTA's half ----
    constexpr uint32_t GROUP_WARPS = DEQ_WARPS / DEQ_GROUPS, GROUP_THREADS = GROUP_WARPS * 32;
    static_assert(GROUP_THREADS == BNH, "one weight column per dequantizer thread");
    const uint32_t dw = warp - DEQ_WARP0, group = dw / GROUP_WARPS, row = (dw % GROUP_WARPS) * 32 + lane;
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t u = pair; u < units && ok; u += pairs) {
      const Unit w = unit_of(p, u);
      for (uint32_t ks = w.ks0; ks < w.ks1; ks++, it++) {
        if (it % DEQ_GROUPS != group) continue;
        const uint32_t sp = it % PS, php = (it / PS) & 1, sb = it % BS, buse = it / BS;
        if (!wait_or_abort<true>(&bars->p_full[sp], php, wctx) ||
            (buse > 0 && !wait_or_abort<true>(&bars->bfree[sb], (buse - 1) & 1, wctx))) {
          if (lane == 0) raise_abort(p.fault, abort_flag);
          ok = false;
          break;
        }
        const uint32_t packed = base + G::OFF_PRING + sp * G::PACKED_PAD;
        uint8_t* btile = sm + G::OFF_BRING + sb * BH_TILE_BYTES;
#pragma unroll
        for (int kbl = 0; kbl < KB_PER_STAGE; kbl++) {
          const uint32_t blk = packed + kbl * G::PACKED_ROW + row * G::BB;
          if (DT == AION_CUDA_DTYPE_Q4_0) dequant_q4_block(blk, btile, row, kbl * 4);
          else dequant_q8_block(blk, btile, row, kbl * 4);
        }
        ptx::fence_proxy_async();  // the tensor core reads this tile through the async proxy
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(ptx::smem_u32(&bars->p_empty[sp]));
          mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&bars->bready[sb]), 0));
        }
      }
    }
  } else {
    // ---- epilogue: this CTA's 128 accumulator lanes = its 128 tokens of every half ----
    ptx::pdl_wait();
    // Plain outputs (no beta, no K split) leave through shared memory: 32 columns of a warp's 32
    // rows at a time are staged (128-byte swizzle, so the stores spread over the banks) and written
    // by one bulk tensor store, which clips the rows past m and the columns past n. A thread
    // storing its own row straight to global memory touches 32 separate sectors per instruction,
    // and that made the epilogue a third of the kernel.
    const uint32_t quarter = warp & 3;
    const bool staged = p.splits == 1 && p.beta == 0.0f;
    const uint32_t out_buf = base + G::OFF_OUT + quarter * 2 * G::OUT_BUF_BYTES;
    uint8_t* out_ptr = sm + G::OFF_OUT + quarter * 2 * G::OUT_BUF_BYTES;
    uint32_t chunk_iter = 0;
    uint32_t tile_iter = 0;
    for (uint32_t u = pair; u < units; u += pairs, tile_iter++) {
      const Unit w = unit_of(p, u);
      const uint32_t acc = tile_iter % NACC, acc_use = tile_iter / NACC;
      if (!wait_or_abort(&bars->acc_full[acc], acc_use & 1, wctx)) {
        if (lane == 0) raise_abort(p.fault, abort_flag);
        break;
      }
      tc_fence_after();
      const uint32_t m0 = (w.tile % p.m_tiles) * (2 * BM * MH), n0 = (w.tile / p.m_tiles) * BN;
#pragma unroll 1
      for (int h = 0; h < MH; h++) {
        const uint32_t trow = h * 2 * BM + rank * BM + quarter * 32 + lane, row = m0 + trow;
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * ACC_COLS + h * BN;
        if (staged) {
          if (row - lane >= p.m) continue;   // none of this warp's rows exist (the same for the whole warp)
#pragma unroll 1
          for (uint32_t c0 = 0; c0 < BN; c0 += 32, chunk_iter++) {
            if (n0 + c0 >= p.n) break;   // the same for the whole warp
            uint32_t r[32];
            tmem_ld32(taddr + c0, r);
            // The buffer about to be filled was the source of the store two chunks ago.
            if (lane == 0) bulk_wait_group_read<1>();
            __syncwarp();
            tmem_ld_wait();
            uint8_t* buf = out_ptr + (chunk_iter & 1) * G::OUT_BUF_BYTES + lane * 128;
#pragma unroll
            for (int q = 0; q < 8; q++)
              *reinterpret_cast<float4*>(buf + ((q ^ (lane & 7)) << 4)) =
                  make_float4(__uint_as_float(r[4 * q]) * p.alpha, __uint_as_float(r[4 * q + 1]) * p.alpha, __uint_as_float(r[4 * q + 2]) * p.alpha,
                              __uint_as_float(r[4 * q + 3]) * p.alpha);
            ptx::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_c, (int32_t)(n0 + c0), (int32_t)(row - lane), out_buf + (chunk_iter & 1) * G::OUT_BUF_BYTES);
              bulk_commit_group();
            }
          }
          continue;
        }
        float* crow = p.c + (uint64_t)row * p.ldc + n0;
        float* slot = p.partial + ((size_t)w.tile * p.splits + w.split) * ((size_t)2 * BM * MH * BN) + (size_t)trow * BN;
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
          if (row < p.m) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
              const uint32_t col = n0 + c0 + q * 4;
              if (col >= p.n) continue;
              float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                                     __uint_as_float(r[4 * q + 3]));
              if (p.splits > 1) {
                __stcg(reinterpret_cast<float4*>(slot + c0 + q * 4), v);
                continue;
              }
              v.x *= p.alpha, v.y *= p.alpha, v.z *= p.alpha, v.w *= p.alpha;
              float4* dst = reinterpret_cast<float4*>(crow + c0 + q * 4);
              if (p.beta != 0.0f) {
                const float4 o = *dst;
                v.x += p.beta * o.x, v.y += p.beta * o.y, v.z += p.beta * o.z, v.w += p.beta * o.w;
              }
              *dst = v;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&bars->acc_empty[acc]), 0));
    }
    if (lane == 0) bulk_wait_group_all();   // this CTA's shared memory and its stores outlive nothing
  }

  // Neither CTA may leave (or free tensor memory) while the other can still signal it or read its
  // shared memory through an MMA in flight: every role of both CTAs is past its last wait here.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

// C = alpha * sum over splits (in split order) + beta * C for the split-K path; one thread per
// four adjacent columns, so both the partial reads and the C accesses are coalesced.
__global__ void splitk_reduce_kernel(const GemmParams p) {
  ptx::pdl_launch_dependents();
  ptx::pdl_wait();
  const uint64_t quads_per_row = p.n / 4, total = (uint64_t)p.m * quads_per_row;
  const size_t slot = (size_t)p.tile_rows * BN;
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t row = (uint32_t)(i / quads_per_row), col = (uint32_t)(i % quads_per_row) * 4;
    const uint32_t tile = (row / p.tile_rows) + (col / BN) * p.m_tiles;
    const float* src = p.partial + (size_t)tile * p.splits * slot + (size_t)(row % p.tile_rows) * BN + (col % BN);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    uint32_t sp = 0;
    for (; sp + 4 <= p.splits; sp += 4) {  // four loads in flight, added in split order
      const float4 x0 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + 0) * slot));
      const float4 x1 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + 1) * slot));
      const float4 x2 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + 2) * slot));
      const float4 x3 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + 3) * slot));
      v.x = (((v.x + x0.x) + x1.x) + x2.x) + x3.x;
      v.y = (((v.y + x0.y) + x1.y) + x2.y) + x3.y;
      v.z = (((v.z + x0.z) + x1.z) + x2.z) + x3.z;
      v.w = (((v.w + x0.w) + x1.w) + x2.w) + x3.w;
    }
    for (; sp < p.splits; sp++) {
      const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * slot));
      v.x += x.x, v.y += x.y, v.z += x.z, v.w += x.w;
    }
    v.x *= p.alpha, v.y *= p.alpha, v.z *= p.alpha, v.w *= p.alpha;
    float4* dst = reinterpret_cast<float4*>(p.c + (uint64_t)row * p.ldc + col);
    if (p.beta != 0.0f) {
      const float4 o = *dst;
      v.x += p.beta * o.x, v.y += p.beta * o.y, v.z += p.beta * o.z, v.w += p.beta * o.w;
    }
    *dst = v;
  }
}

// `MatMulNT` weights, q8_0 [n][k/32] blocks in any QuantBlockOrder (src/aion/backend/types.zig:185-204),
// re-laid as K-major [k/32][n] blocks for the GEMM. Both layouts quantize along K, so a block
// holds the same 34 bytes either way: this is a permutation of blocks. One thread per block,
// n fastest, so the K-major writes are contiguous.
// (It does not release its dependents early: what it writes are WEIGHTS, and the matmul kernels start their
// weight loads without waiting for the kernel before them. Its dependents therefore start when it has completed.)
__global__ void nt_to_kmajor_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n, uint64_t kblocks,
                                    int group, int chunk) {
  ptx::pdl_wait();
  const uint64_t total = n * kblocks;
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t kb = i / n, r = i % n;
    const uint8_t* seg = src + ((r / group) * kblocks + kb) * (uint64_t)group * Q8_BYTES;
    const int rg = (int)(r % group);
    uint16_t* out = reinterpret_cast<uint16_t*>(dst + i * Q8_BYTES);  // blocks are 2-byte aligned
    out[0] = *reinterpret_cast<const uint16_t*>(seg + rg * 2);
    const uint8_t* quants = seg + 2 * group;
#pragma unroll
    for (int t = 0; t < 16; t++) {
      const int e = 2 * t;  // a pair of codes never straddles a chunk (chunks are 4 or 16 bytes)
      out[1 + t] = *reinterpret_cast<const uint16_t*>(quants + ((uint64_t)(e / chunk) * group + rg) * chunk + (e % chunk));
    }
  }
}

// The same permutation for the row-major order, through a shared-memory tile so that both the
// reads (16 blocks of a row are 544 contiguous bytes) and the writes (64 blocks of a block row
// are 2176 contiguous bytes) are coalesced. Tile = 64 rows x 16 blocks, moved as 2-byte units.
constexpr int RT_ROWS = 64, RT_KB = 16, RT_UNITS = Q8_BYTES / 2, RT_PITCH = RT_KB * RT_UNITS + 1;
__global__ void __launch_bounds__(256) nt_rowmajor_to_kmajor_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                                                    uint64_t n, uint64_t kblocks) {
  ptx::pdl_wait();   // (no early release of its dependents, for the same reason)
  __shared__ uint16_t tile[RT_ROWS * RT_PITCH];
  const uint64_t r0 = (uint64_t)blockIdx.x * RT_ROWS, kb0 = (uint64_t)blockIdx.y * RT_KB;
  const uint32_t rows = (uint32_t)min((uint64_t)RT_ROWS, n - r0), kbs = (uint32_t)min((uint64_t)RT_KB, kblocks - kb0);
  const uint32_t row_units = kbs * RT_UNITS;
  for (uint32_t i = threadIdx.x; i < rows * row_units; i += 256) {
    const uint32_t r = i / row_units, u = i - r * row_units;
    tile[r * RT_PITCH + u] = src[((r0 + r) * kblocks + kb0) * RT_UNITS + u];
  }
  __syncthreads();
  const uint32_t col_units = rows * RT_UNITS;
  for (uint32_t i = threadIdx.x; i < kbs * col_units; i += 256) {
    const uint32_t kb = i / col_units, u = i - kb * col_units;
    const uint32_t r = u / RT_UNITS, w = u - r * RT_UNITS;
    dst[((kb0 + kb) * n + r0) * RT_UNITS + u] = tile[r * RT_PITCH + kb * RT_UNITS + w];
  }
}

template <int DT, int MH>
int32_t launch_gemm(AionCudaDevice* dev, const MatMulArgs& g, const __nv_bfloat16* a_bf16, uint32_t splits, float* partial) {
  using G = GemmGeom<DT, MH>;
  auto kernel = gemm_q_tcgen05_kernel<DT, MH>;
  {
    // Once per device and instantiation; several host threads may drive devices at once.
    static std::mutex mu;
    static bool configured[64] = {};
    std::lock_guard<std::mutex> lock(mu);
    if (dev->ordinal < 0 || dev->ordinal >= 64 || !configured[dev->ordinal]) {
      AION_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES));
      if (dev->ordinal >= 0 && dev->ordinal < 64) configured[dev->ordinal] = true;
    }
  }
  const uint64_t kblocks = g.k / QK;
  CUtensorMap tmap_a, tmap_b;
  if (int32_t st = tensor_map_bf16_sw128(a_bf16, g.m, g.k, g.k * 2, BK, BM * MH, &tmap_a)) return st;
  {
    // Packed weights as [K/32][ldb/8][8 blocks]: box = 2 block rows x 32 groups x 8 blocks.
    const uint64_t dims[3] = {8ull * G::BB, g.n / 8, kblocks};
    const uint64_t strides[2] = {8ull * G::BB, g.ldb * G::BB};
    const uint32_t box[3] = {8u * G::BB, BN / 8, KB_PER_STAGE};
    if (int32_t st = tensor_map_encode(g.b, 3, dims, strides, box, &tmap_b)) return st;
  }
  GemmParams p{};
  p.c = g.c;
  p.m = (uint32_t)g.m, p.n = (uint32_t)g.n, p.k = (uint32_t)g.k;
  p.ldc = g.ldc;
  p.alpha = g.alpha, p.beta = g.beta;
  p.m_tiles = (uint32_t)ceil_div(g.m, (uint64_t)(BM * MH));
  p.tile_rows = BM * MH;
  p.n_tiles = (uint32_t)ceil_div(g.n, (uint64_t)BN);
  p.k_stages = (uint32_t)ceil_div(g.k, (uint64_t)BK);
  p.fault = dev->fault_dev;
  p.wait_shift = dev->debug_expire_waits ? 14u : 0u;
  p.drop_first = dev->debug_expire_waits ? 1u : 0u;
  p.splits = splits;
  p.partial = partial;
  const uint32_t units = p.m_tiles * p.n_tiles * splits;
  const uint32_t grid = units < (uint32_t)dev->sm_count ? units : (uint32_t)dev->sm_count;
  AION_CUDA_TRY(launch_pdl_main(kernel, dim3(grid), dim3(THREADS), (size_t)G::SMEM_BYTES, dev->stream, p, tmap_a, tmap_b));
  if (splits > 1) {
    const uint64_t quads = (uint64_t)g.m * (g.n / 4);
    const unsigned blocks = (unsigned)std::min<uint64_t>(ceil_div(quads, (uint64_t)256), (uint64_t)dev->sm_count * 8);
    AION_CUDA_TRY(launch_pdl_main(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, dev->stream, p));
  }
  return AION_CUDA_OK;
}


// Clusters of two CTAs that fit the device at once, per instantiation (0: the launch is not possible).
template <int DT, int MH>
int32_t pair_capacity(AionCudaDevice* dev, int* pairs_out) {
  using G = PairGeom<DT, MH>;
  auto kernel = gemm_q_pair_kernel<DT, MH>;
  static std::mutex mu;
  static int pairs[64] = {};
  static bool configured[64] = {};
  if (dev->ordinal < 0 || dev->ordinal >= 64) {
    *pairs_out = 0;
    return AION_CUDA_OK;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!configured[dev->ordinal]) {
    AION_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * (unsigned)dev->sm_count);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = G::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    pairs[dev->ordinal] = n;
    configured[dev->ordinal] = true;
  }
  *pairs_out = pairs[dev->ordinal];
  return AION_CUDA_OK;
}

template <int DT, int MH>
int32_t launch_gemm_pair(AionCudaDevice* dev, const MatMulArgs& g, const __nv_bfloat16* a_bf16, uint32_t splits, float* partial, uint32_t pairs) {
  using G = PairGeom<DT, MH>;
  auto kernel = gemm_q_pair_kernel<DT, MH>;
  const uint64_t kblocks = g.k / QK;
  CUtensorMap tmap_a, tmap_b;
  if (int32_t st = tensor_map_bf16_sw128(a_bf16, g.m, g.k, g.k * 2, BK, BM, &tmap_a)) return st;
  {
    // Packed weights as [K/32][ldb/8][8 blocks]: box = 2 block rows x 16 groups x 8 blocks (this CTA's 128 columns).
    const uint64_t dims[3] = {8ull * G::BB, g.n / 8, kblocks};
    const uint64_t strides[2] = {8ull * G::BB, g.ldb * G::BB};
    const uint32_t box[3] = {8u * G::BB, BNH / 8, KB_PER_STAGE};
    if (int32_t st = tensor_map_encode(g.b, 3, dims, strides, box, &tmap_b)) return st;
  }
  // C as [m][n] f32 with boxes of 32 x 32 for the staged stores (unused, but valid, when beta or a K split
  // keeps the epilogue on plain stores).
  CUtensorMap tmap_c;
  if (int32_t st = tensor_map_f32_sw128(g.c, g.m, g.n, g.ldc * sizeof(float), 32, 32, &tmap_c)) return st;
  GemmParams p{};
  p.c = g.c;
  p.m = (uint32_t)g.m, p.n = (uint32_t)g.n, p.k = (uint32_t)g.k;
  p.ldc = g.ldc;
  p.alpha = g.alpha, p.beta = g.beta;
  p.tile_rows = 2 * BM * MH;
  p.m_tiles = (uint32_t)ceil_div(g.m, (uint64_t)p.tile_rows);
  p.n_tiles = (uint32_t)ceil_div(g.n, (uint64_t)BN);
  p.k_stages = (uint32_t)ceil_div(g.k, (uint64_t)BK);
  p.fault = dev->fault_dev;
  p.wait_shift = dev->debug_expire_waits ? 14u : 0u;
  p.drop_first = dev->debug_expire_waits ? 1u : 0u;
  p.splits = splits;
  p.partial = partial;
  const uint32_t units = p.m_tiles * p.n_tiles * splits;
  const uint32_t grid = 2 * (units < pairs ? units : pairs);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = G::SMEM_BYTES;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool overlap = std::getenv("AION_CUDA_NO_PDL_MAIN") == nullptr;  // tuning only
  cfg.numAttrs = overlap ? 2 : 1;
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  AION_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p, tmap_a, tmap_b, tmap_c));
  if (splits > 1) {
    const uint64_t quads = (uint64_t)g.m * (g.n / 4);
    const unsigned blocks = (unsigned)std::min<uint64_t>(ceil_div(quads, (uint64_t)256), (uint64_t)dev->sm_count * 8);
    AION_CUDA_TRY(launch_pdl_main(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, dev->stream, p));
  }
  return AION_CUDA_OK;
}

}  // namespace

// q8_0 [n][k/32] blocks in `order` -> K-major [k/32][n] blocks (the layout `MatMul` reads).
int32_t nt_blocks_to_kmajor(AionCudaDevice* dev, uint32_t order, const uint8_t* src, uint8_t* dst, uint64_t n, uint64_t kblocks) {
  int group = 1, chunk = 4;
  if (!block_order_info(order, &group, &chunk)) return AION_CUDA_INVALID_ARGUMENT;
  if (n == 0 || kblocks == 0) return AION_CUDA_OK;
  if (order == AION_CUDA_ORDER_ROW_MAJOR && ceil_div(kblocks, (uint64_t)RT_KB) <= 65535) {
    const dim3 grid((unsigned)ceil_div(n, (uint64_t)RT_ROWS), (unsigned)ceil_div(kblocks, (uint64_t)RT_KB));
    AION_CUDA_TRY(launch_pdl_main(nt_rowmajor_to_kmajor_kernel, grid, dim3(256), 0, dev->stream, reinterpret_cast<const uint16_t*>(src),
                                  reinterpret_cast<uint16_t*>(dst), n, kblocks));
  } else {
    const uint64_t total = n * kblocks;
    const unsigned blocks = (unsigned)std::min<uint64_t>(ceil_div(total, (uint64_t)256), (uint64_t)dev->sm_count * 16);
    AION_CUDA_TRY(launch_pdl_main(nt_to_kmajor_kernel, dim3(blocks), dim3(256), 0, dev->stream, src, dst, n, kblocks, group, chunk));
  }
  return AION_CUDA_OK;
}

// Whether this kernel reads the step's operands, and how it would tile them.
// AION_CUDA_GEMM_PAIR=0 keeps every shape on the one-SM kernel (measurement).
static bool pair_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("AION_CUDA_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

static bool plan_gemm(const AionCudaDevice* dev, const MatMulArgs& g, GemmPlan* out, bool allow_pair = true) {
  if (g.dtype != AION_CUDA_DTYPE_Q4_0 && g.dtype != AION_CUDA_DTYPE_Q8_0) return false;
  if (g.m == 0 || g.n == 0 || g.k == 0) return false;
  if (g.nt) {
    int group, chunk;
    if (g.dtype != AION_CUDA_DTYPE_Q8_0 || !block_order_info(g.order, &group, &chunk)) return false;
    if ((g.n & 7) || ((uintptr_t)g.b & 1)) return false;
  } else if ((g.ldb & 7) || ((uintptr_t)g.b & 15)) {
    return false;
  }
  if ((g.n & 7) || ((uintptr_t)g.c & 15) || (g.ldc & 3)) return false;
  if (g.m > (1u << 24) || g.n > (1u << 24) || g.k > (1u << 24)) return false;
  // Above 128 rows: pairs of CTAs (two-SM MMAs). A pair's tile is 256 tokens, or 512 (two MMAs per
  // dequantized weight tile) once there are enough of those to fill the pairs.
  const bool pair = allow_pair && !g.one_sm && g.m > BM && pair_enabled();
  const uint64_t workers = pair ? (uint64_t)dev->sm_count / 2 : (uint64_t)dev->sm_count;   // CTAs or pairs
  const uint64_t base_rows = pair ? 2 * BM : BM;
  // 1-SM kernel: 256-token tiles (one dequantized weight tile feeds two MMAs) once there are enough
  // of them to fill the SMs; 128-token tiles with a double-buffered accumulator otherwise.
  // (fewer 256-token tiles with a K split to fill the SMs measured slower: m = 512 x 8192 columns
  // took 47 us that way against 39 us with 128-token tiles)
  const uint64_t tiles2 = ceil_div(g.m, 2 * base_rows) * ceil_div(g.n, (uint64_t)BN);
  uint32_t mh = (g.m > base_rows && tiles2 >= workers) ? 2 : 1;
  {
    static const int force = [] { const char* e = std::getenv("AION_CUDA_GEMM_MH"); return e ? atoi(e) : 0; }();   // measurement
    if (force == 1 || (force == 2 && g.m > base_rows)) mh = (uint32_t)force;
  }
  const uint64_t tiles = ceil_div(g.m, base_rows * mh) * ceil_div(g.n, (uint64_t)BN), k_stages = ceil_div(g.k, (uint64_t)BK);
  // Few output tiles (narrow layers): split K so the SMs are covered. A split keeps at least
  // two k-stages; its raw accumulator goes through scratch.
  uint64_t splits = 1;
  if (tiles * 2 <= workers) {
    splits = workers / tiles;
    if (splits > k_stages / 2) splits = k_stages / 2;
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
  }
  out->tile_rows = (uint32_t)(base_rows * mh);
  out->splits = (uint32_t)splits;
  out->pair = pair;
  const uint64_t units = tiles * splits;
  out->grid = (uint32_t)((units < workers ? units : workers) * (pair ? 2 : 1));
  return true;
}

bool gemm_tcgen05_plan(const AionCudaDevice* dev, const MatMulArgs& g, GemmPlan* out) { return plan_gemm(dev, g, out, true); }

// Returns UNSUPPORTED (without setting a message) for shapes this kernel does not read, so
// the caller can route them to the any-shape kernel.
int32_t gemm_tcgen05(AionCudaDevice* dev, const MatMulArgs& g_in) {
  MatMulArgs g = g_in;
  if (g.dtype != AION_CUDA_DTYPE_Q4_0 && g.dtype != AION_CUDA_DTYPE_Q8_0) return AION_CUDA_UNSUPPORTED;
  if (g.m == 0 || g.n == 0) return AION_CUDA_OK;
  GemmPlan plan{};
  if (!plan_gemm(dev, g, &plan)) return AION_CUDA_UNSUPPORTED;
  int pairs = 0;
  if (plan.pair) {
    // Clusters of two that the device can hold at once; none (an SM partition without room for pairs)
    // sends the shape to the one-SM kernel.
    const bool two = plan.tile_rows == 4 * BM;
    int32_t st;
    if (g.dtype == AION_CUDA_DTYPE_Q4_0) st = two ? pair_capacity<AION_CUDA_DTYPE_Q4_0, 2>(dev, &pairs) : pair_capacity<AION_CUDA_DTYPE_Q4_0, 1>(dev, &pairs);
    else st = two ? pair_capacity<AION_CUDA_DTYPE_Q8_0, 2>(dev, &pairs) : pair_capacity<AION_CUDA_DTYPE_Q8_0, 1>(dev, &pairs);
    if (st) return st;
    if (pairs < 1 && !plan_gemm(dev, g, &plan, false)) return AION_CUDA_UNSUPPORTED;
  }
  const int mh = (int)(plan.tile_rows / (plan.pair ? 2 * BM : BM));
  const uint64_t splits = plan.splits;
  const uint64_t tiles = ceil_div(g.m, (uint64_t)plan.tile_rows) * ceil_div(g.n, (uint64_t)BN);
  // `MatMulNT`: the same kernel after a block permutation of the weights into lane scratch
  // (the reference's weight-layout pass does the equivalent once per model).
  size_t relaid_bytes = 0;
  if (g.nt) {
    relaid_bytes = ((size_t)g.n * (g.k / QK) * Q8_BYTES + 1023) & ~size_t(1023);
    g.ldb = g.n;
  }
  // Lane scratch: the bf16 copy of the activation, then the split partials.
  const size_t a_bytes = ((size_t)g.m * g.k * sizeof(__nv_bfloat16) + 1023) & ~size_t(1023);
  const size_t part_bytes = splits > 1 ? (size_t)tiles * splits * plan.tile_rows * BN * sizeof(float) : 0;
  if (int32_t st = dev->reserve_scratch(relaid_bytes + a_bytes + part_bytes)) return st;
  uint8_t* scratch = static_cast<uint8_t*>(dev->lane_scratch());
  if (g.nt) {
    if (int32_t st = nt_blocks_to_kmajor(dev, g.order, g.b, scratch, g.n, g.k / QK)) return st;
    g.b = scratch;
    g.nt = false;
  }
  __nv_bfloat16* a_bf16 = reinterpret_cast<__nv_bfloat16*>(scratch + relaid_bytes);
  float* partial = reinterpret_cast<float*>(scratch + relaid_bytes + a_bytes);
  if (g.a_image && act_image_layout(g.m, g.k / QK).kind == ACT_IMAGE_BF16) {
    // The step that produced A already wrote what the pre-pass would write.
    a_bf16 = reinterpret_cast<__nv_bfloat16*>(const_cast<uint8_t*>(g.a_image));
  } else {
    const uint64_t groups = g.m * (g.k / 8);
    const unsigned blocks = (unsigned)std::min<uint64_t>(ceil_div(groups, (uint64_t)256), (uint64_t)dev->sm_count * 8);
    AION_CUDA_TRY(launch_pdl_main(convert_a_bf16_kernel, dim3(blocks), dim3(256), 0, dev->stream, g.a, g.lda, a_bf16, (uint32_t)g.m, (uint32_t)g.k,
                             g.dtype == AION_CUDA_DTYPE_Q4_0 ? 1 : 0));
  }
  if (plan.pair) {
    if (g.dtype == AION_CUDA_DTYPE_Q4_0)
      return mh == 2 ? launch_gemm_pair<AION_CUDA_DTYPE_Q4_0, 2>(dev, g, a_bf16, (uint32_t)splits, partial, (uint32_t)pairs)
                     : launch_gemm_pair<AION_CUDA_DTYPE_Q4_0, 1>(dev, g, a_bf16, (uint32_t)splits, partial, (uint32_t)pairs);
    return mh == 2 ? launch_gemm_pair<AION_CUDA_DTYPE_Q8_0, 2>(dev, g, a_bf16, (uint32_t)splits, partial, (uint32_t)pairs)
                   : launch_gemm_pair<AION_CUDA_DTYPE_Q8_0, 1>(dev, g, a_bf16, (uint32_t)splits, partial, (uint32_t)pairs);
  }
  if (g.dtype == AION_CUDA_DTYPE_Q4_0)
    return mh == 2 ? launch_gemm<AION_CUDA_DTYPE_Q4_0, 2>(dev, g, a_bf16, (uint32_t)splits, partial)
                   : launch_gemm<AION_CUDA_DTYPE_Q4_0, 1>(dev, g, a_bf16, (uint32_t)splits, partial);
  return mh == 2 ? launch_gemm<AION_CUDA_DTYPE_Q8_0, 2>(dev, g, a_bf16, (uint32_t)splits, partial)
                 : launch_gemm<AION_CUDA_DTYPE_Q8_0, 1>(dev, g, a_bf16, (uint32_t)splits, partial);
}


int32_t act_image_bf16_from_f32(AionCudaDevice* dev, uint32_t dtype, const float* a, uint64_t m, uint64_t k, uint64_t lda, uint8_t* image) {
  const uint64_t groups = m * (k / 8);
  const unsigned blocks = (unsigned)std::min<uint64_t>(ceil_div(groups, (uint64_t)256), (uint64_t)dev->sm_count * 8);
  AION_CUDA_TRY(launch_pdl_main(convert_a_bf16_kernel, dim3(blocks), dim3(256), 0, dev->stream, a, lda, reinterpret_cast<__nv_bfloat16*>(image),
                                (uint32_t)m, (uint32_t)k, dtype == AION_CUDA_DTYPE_Q4_0 ? 1 : 0));
  return AION_CUDA_OK;
}

}  // namespace aion
