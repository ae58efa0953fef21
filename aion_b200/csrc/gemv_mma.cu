// Decode GEMV for q4_0 / q8_0 weights: C[m,n] = alpha * A[m,k] . W + beta * C, m <= 16.
//
// Arithmetic is the reference CPU kernels' (src/aion/backend/cpu/kernels/matvec_q.zig:62-160,
// src/aion/backend/cpu/kernels/matmul_nt_q.zig:74-95, src/aion/backend/cpu/kernels/matmul_q_i8.zig:385-497):
// the activation is quantized to int8 per 32-block inside the kernel, every weight
// block contributes float(exact int dot) * (a_scale * w_scale), accumulated in f32.
//
// The kernel is HBM-bound: each weight byte is read from global memory exactly once.
//   * A CTA owns a tile of 64 output columns and a contiguous range of K blocks. A
//     producer warp streams the packed blocks, untouched, into a 4-stage shared-memory
//     ring with 1-D bulk (TMA) copies that complete on mbarriers; four consumer warps
//     drain it. Blocks are 18 / 34 bytes, so nothing inside a stage is 16-byte aligned
//     except the copies themselves.
//   * Consumers feed the int8 tensor-core MMA (m16n8k32): the 16 "rows" are 16 output
//     columns of one K block, the 8 "columns" are up to 8 activation rows. q4 nibbles
//     become int8 in two logic ops by placing the nibble in the high half of a byte
//     (value 16*(nibble-8)); the 1/16 folds into the weight scale. One block's int32
//     dot leaves the MMA and is scaled and accumulated in f32 registers.
//   * Shared-memory reads are arranged so each load instruction is one wavefront:
//     the 8 row groups of a fragment read 8 columns that are 8 apart (their starts are
//     4 words apart modulo the 32 banks).
//   * K is split across the CTAs of a thread-block cluster when the column tiles alone
//     would not fill the GPU; partial sums meet in distributed shared memory in a fixed
//     order, so results do not depend on scheduling.
//   * With programmatic dependent launch the weight stream of the next GEMV starts
//     while this one drains: only the activation read waits for the previous kernel.
#include "common.cuh"
#include "ptx.cuh"
#include "quant_device.cuh"

namespace aion {

namespace {

constexpr int TN = 64;             // output columns per CTA
constexpr int KBT = 8;             // K blocks per stage
constexpr int NS = 4;              // stages in the ring
constexpr int CONSUMER_WARPS = 4;
constexpr int CONSUMER_THREADS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMER_THREADS + 32;
constexpr int ACT_STAGES = 8;      // stages whose activations are held quantized at once
constexpr int ACT_KB = ACT_STAGES * KBT;
constexpr int NT_ROW_PITCH = KBT * Q8_BYTES;  // 272 bytes: 16-byte multiple, 4 words mod 32 banks

struct GemvParams {
  const uint8_t* b;
  const float* a;
  float* c;
  uint32_t m, n, kblocks;
  uint64_t lda, ldb, ldc;
  float alpha, beta;
  int* fault;
  uint32_t a_vec4;  // A rows may be read as float4
};

template <int DT, bool NT, int MT>
struct Geom {
  static constexpr int BB = (DT == AION_CUDA_DTYPE_Q8_0) ? Q8_BYTES : Q4_BYTES;
  static constexpr int KM_PITCH = TN * BB;
  static constexpr int STAGE_BYTES = NT ? TN * NT_ROW_PITCH : KBT * KM_PITCH;
  static constexpr int MP = 8 * MT;  // padded activation rows
  static constexpr int PARTIAL_BYTES = CONSUMER_WARPS * TN * MP * 4;
  static constexpr int RING_BYTES = NS * STAGE_BYTES;
  static_assert(PARTIAL_BYTES <= RING_BYTES, "partials reuse the ring");
  static constexpr int OFF_ACTQ = RING_BYTES;
  static constexpr int ACTQ_BYTES = ACT_KB * MP * 32;
  static constexpr int OFF_ACTS = OFF_ACTQ + ACTQ_BYTES;
  static constexpr int ACTS_BYTES = ACT_KB * MP * 4;
  static constexpr int OFF_RED = OFF_ACTS + ACTS_BYTES;
  static constexpr int RED_BYTES = TN * MP * 4;
  static constexpr int OFF_BARS = OFF_RED + RED_BYTES;
  static constexpr int SMEM_BYTES = OFF_BARS + 2 * NS * 8 + 16;
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory"); }

// Position, inside the 32-byte quantized row of one K block, of the 4-byte word that
// holds elements 4u..4u+3 (q8) — chosen so that MMA B-fragment lane j finds its two
// registers as the 8 bytes at 8j.
//   q8: b0 = k 4j..4j+3, b1 = k 16+4j..16+4j+3.
//   q4: b0 = elements 8j+{0,2,4,6} (low nibbles of 4 bytes), b1 = 8j+{1,3,5,7}.
template <int DT>
__device__ __forceinline__ void store_act_quad(uint8_t* row32, int u, int q0, int q1, int q2, int q3) {
  if (DT == AION_CUDA_DTYPE_Q8_0) {
    const uint32_t w = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
                       ((uint32_t)(q3 & 0xFF) << 24);
    *reinterpret_cast<uint32_t*>(row32 + 8 * (u & 3) + 4 * (u >> 2)) = w;
  } else {
    const int j = u >> 1, odd = u & 1;
    *reinterpret_cast<uint16_t*>(row32 + 8 * j + 2 * odd) = (uint16_t)((q0 & 0xFF) | ((q2 & 0xFF) << 8));
    *reinterpret_cast<uint16_t*>(row32 + 8 * j + 4 + 2 * odd) = (uint16_t)((q1 & 0xFF) | ((q3 & 0xFF) << 8));
  }
}

// The two A-fragment registers of one weight block for quad lane j. `aligned` says the
// block's codes start on a 4-byte boundary (they start 2 bytes after the block does).
template <int DT>
__device__ __forceinline__ void load_codes(uint32_t blk, bool aligned, int j, uint32_t& r_lo, uint32_t& r_hi) {
  if (DT == AION_CUDA_DTYPE_Q4_0) {
    uint32_t v;
    if (aligned) {
      v = ptx::lds32(blk + 2 + 4 * j);
    } else {
      const uint32_t lo = ptx::lds32(blk + 4 * j), hi = ptx::lds32(blk + 4 * j + 4);
      v = __funnelshift_r(lo, hi, 16);
    }
    // nibble -> signed byte 16*(nibble-8): move it to the high half, flip its top bit.
    r_lo = ((v << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
    r_hi = (v & 0xF0F0F0F0u) ^ 0x80808080u;
  } else {
    if (aligned) {
      r_lo = ptx::lds32(blk + 2 + 4 * j);
      r_hi = ptx::lds32(blk + 18 + 4 * j);
    } else {
      const uint32_t w0 = ptx::lds32(blk + 4 * j), w1 = ptx::lds32(blk + 4 * j + 4);
      const uint32_t w2 = ptx::lds32(blk + 16 + 4 * j), w3 = ptx::lds32(blk + 20 + 4 * j);
      r_lo = __funnelshift_r(w0, w1, 16);
      r_hi = __funnelshift_r(w2, w3, 16);
    }
  }
}

template <int DT>
__device__ __forceinline__ float load_scale(uint32_t blk) {
  const float s = __half2float(__ushort_as_half((unsigned short)ptx::lds16(blk)));
  return DT == AION_CUDA_DTYPE_Q4_0 ? s * 0.0625f : s;  // undo the 16x of the nibble placement (exact)
}

template <int DT, bool NT, int MT>
__global__ void __launch_bounds__(THREADS) gemv_q_mma_kernel(const GemvParams p) {
  using G = Geom<DT, NT, MT>;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t smem_base = ptx::smem_u32(smem);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;

  const uint32_t S = ptx::cluster_nctarank();
  const uint32_t rank = ptx::cluster_ctarank();
  const uint32_t tile = blockIdx.x / S;
  const uint32_t n0 = tile * TN;
  const uint32_t cols = min((uint32_t)TN, p.n - n0);

  const uint32_t stages_total = (p.kblocks + KBT - 1) / KBT;
  const uint32_t s_begin = (uint32_t)((uint64_t)stages_total * rank / S);
  const uint32_t s_end = (uint32_t)((uint64_t)stages_total * (rank + 1) / S);
  const uint32_t my_stages = s_end - s_begin;

  const uint32_t bar_full = smem_base + G::OFF_BARS;
  const uint32_t bar_empty = bar_full + NS * 8;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + G::OFF_BARS + 2 * NS * 8);

  if (tid == 0) {
    for (int s = 0; s < NS; s++) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, CONSUMER_WARPS);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  // The next kernel in the stream may begin (its weight stream does not depend on us).
  ptx::pdl_launch_dependents();

  float acc[4][MT][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[i][t][e] = 0.0f;

  if (warp == CONSUMER_WARPS) {
    // ---------------- producer: stream packed weight blocks into the ring ----------------
    uint32_t issued = 0;
    for (uint32_t it = 0; it < my_stages; it++) {
      const uint32_t slot = it % NS;
      if (*abort_flag) break;
      if (it >= NS) {
        if (!ptx::mbar_wait_bounded(bar_empty + 8 * slot, ((it / NS) - 1) & 1)) {
          if (lane == 0) {
            atomicExch(p.fault, FAULT_WAIT_EXPIRED);
            *abort_flag = 1;
          }
          break;
        }
      }
      const uint32_t kb0 = (s_begin + it) * KBT;
      const uint32_t nkb = min((uint32_t)KBT, p.kblocks - kb0);
      const uint32_t stage = smem_base + slot * G::STAGE_BYTES;
      const uint32_t full = bar_full + 8 * slot;
      if (!NT) {
        const uint32_t seg = cols * G::BB;
        if (lane == 0) ptx::mbar_arrive_expect_tx(full, nkb * seg);
        __syncwarp();
        if ((uint32_t)lane < nkb)
          ptx::bulk_g2s(stage + lane * G::KM_PITCH, p.b + ((uint64_t)(kb0 + lane) * p.ldb + n0) * G::BB, seg, full);
      } else {
        const uint32_t seg = nkb * Q8_BYTES;
        if (lane == 0) ptx::mbar_arrive_expect_tx(full, cols * seg);
        __syncwarp();
        for (uint32_t r = lane; r < cols; r += 32)
          ptx::bulk_g2s(stage + r * NT_ROW_PITCH, p.b + ((uint64_t)(n0 + r) * p.ldb + kb0) * Q8_BYTES, seg, full);
      }
      issued = it + 1;
    }
    // After a failed wait nobody drains the ring: let the copies still in flight land
    // (bounded) before this CTA's shared memory can be handed to another CTA.
    if (*abort_flag)
      for (uint32_t it = issued > NS ? issued - NS : 0; it < issued; it++)
        ptx::mbar_wait_bounded(bar_full + 8 * (it % NS), (it / NS) & 1, 1u << 16);
  } else {
    // ---------------- consumers ----------------
    // Rows of A beyond m are zero activations with zero scale.
    if (p.m < (uint32_t)G::MP) {
      for (int i = tid; i < ACT_KB * G::MP * 8; i += CONSUMER_THREADS) {
        const int row = (i / 8) % G::MP;
        if ((uint32_t)row >= p.m) reinterpret_cast<uint32_t*>(smem + G::OFF_ACTQ)[i] = 0u;
      }
      for (int i = tid; i < ACT_KB * G::MP; i += CONSUMER_THREADS)
        if ((uint32_t)(i % G::MP) >= p.m) reinterpret_cast<float*>(smem + G::OFF_ACTS)[i] = 0.0f;
    }
    // Everything below reads what the previous kernel wrote (A, and C when beta != 0).
    ptx::pdl_wait();

    bool ok = true;
    // A consumer that gives up a wait keeps walking the loops (without waiting or
    // computing) so that every warp meets the same sequence of barriers.
    for (uint32_t c0 = 0; c0 < my_stages; c0 += ACT_STAGES) {
      const uint32_t nst = min((uint32_t)ACT_STAGES, my_stages - c0);
      const uint32_t ckb0 = (s_begin + c0) * KBT;
      const uint32_t cnkb = min(nst * KBT, p.kblocks - ckb0);
      if (c0 > 0) consumer_sync();  // the previous chunk's activations are no longer read
      {
        // Quantize A[:, ckb0*32 .. (ckb0+cnkb)*32) : 8 lanes per 32-block, 4 elements each.
        // The trip count is uniform inside an 8-lane group but not across a warp, so
        // the shuffles name only their own group.
        const int grp = tid >> 3, u = tid & 7;
        const uint32_t gmask = 0xFFu << (lane & 24);
        const uint32_t items = ok ? p.m * cnkb : 0u;
        for (uint32_t item = grp; item < items; item += CONSUMER_THREADS / 8) {
          const uint32_t r = item / cnkb, kb = item % cnkb;
          const float* src = p.a + (uint64_t)r * p.lda + (uint64_t)(ckb0 + kb) * QK + 4 * u;
          float4 v;
          if (p.a_vec4) {
            v = *reinterpret_cast<const float4*>(src);
          } else {
            v.x = src[0]; v.y = src[1]; v.z = src[2]; v.w = src[3];
          }
          float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
          amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 4));
          amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 2));
          amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 1));
          float scale, inv;
          activation_block_scales(amax, &scale, &inv);
          uint8_t* row32 = smem + G::OFF_ACTQ + ((size_t)kb * G::MP + r) * 32;
          store_act_quad<DT>(row32, u, quantize_activation_with_inv(v.x, inv), quantize_activation_with_inv(v.y, inv),
                             quantize_activation_with_inv(v.z, inv), quantize_activation_with_inv(v.w, inv));
          if (u == 0) reinterpret_cast<float*>(smem + G::OFF_ACTS)[kb * G::MP + r] = scale;
        }
        __syncwarp();
      }
      consumer_sync();

      for (uint32_t st = 0; st < nst; st++) {
        const uint32_t it = c0 + st;
        const uint32_t slot = it % NS;
        if (ok && (*abort_flag || !ptx::mbar_wait_bounded(bar_full + 8 * slot, (it / NS) & 1))) {
          if (lane == 0 && !*abort_flag) {
            atomicExch(p.fault, FAULT_WAIT_EXPIRED);
            *abort_flag = 1;
          }
          ok = false;
        }
        const uint32_t kb0 = (s_begin + it) * KBT;
        const uint32_t nkb = ok ? min((uint32_t)KBT, p.kblocks - kb0) : 0u;
        const uint32_t stage = smem_base + slot * G::STAGE_BYTES;
        for (uint32_t kbl = warp; kbl < nkb; kbl += CONSUMER_WARPS) {
          const uint32_t akb = st * KBT + kbl;  // K block index inside the activation chunk
          uint32_t bq[MT][2];
          float as[MT][2];
#pragma unroll
          for (int t = 0; t < MT; t++) {
            const uint2 b2 = *reinterpret_cast<const uint2*>(smem + G::OFF_ACTQ + ((size_t)akb * G::MP + t * 8 + g) * 32 + 8 * j);
            bq[t][0] = b2.x;
            bq[t][1] = b2.y;
            const float2 s2 = *reinterpret_cast<const float2*>(smem + G::OFF_ACTS + ((size_t)akb * G::MP + t * 8 + 2 * j) * 4);
            as[t][0] = s2.x;
            as[t][1] = s2.y;
          }
#pragma unroll
          for (int i = 0; i < 4; i++) {
            uint32_t blk0, blk1;
            bool al0, al1;
            if (!NT) {
              // rows g -> column 2i + 8g (even: codes 2 bytes past a word boundary),
              // rows g+8 -> column 2i + 1 + 8g (odd: codes word aligned).
              blk0 = stage + kbl * G::KM_PITCH + (2 * i + 8 * g) * G::BB;
              blk1 = blk0 + G::BB;
              al0 = false;
              al1 = true;
            } else {
              blk0 = stage + (16 * i + g) * NT_ROW_PITCH + kbl * Q8_BYTES;
              blk1 = blk0 + 8 * NT_ROW_PITCH;
              al0 = al1 = (kbl & 1) != 0;
            }
            uint32_t a0, a1, a2, a3;
            load_codes<DT>(blk0, al0, j, a0, a2);
            load_codes<DT>(blk1, al1, j, a1, a3);
            const float ws0 = load_scale<DT>(blk0), ws1 = load_scale<DT>(blk1);
#pragma unroll
            for (int t = 0; t < MT; t++) {
              int d[4];
              ptx::mma_s8(d, a0, a1, a2, a3, bq[t][0], bq[t][1]);
              acc[i][t][0] += (float)d[0] * (as[t][0] * ws0);
              acc[i][t][1] += (float)d[1] * (as[t][1] * ws0);
              acc[i][t][2] += (float)d[2] * (as[t][0] * ws1);
              acc[i][t][3] += (float)d[3] * (as[t][1] * ws1);
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_empty + 8 * slot);
      }
    }

    // ---------------- fold the four warps' partial sums ----------------
    consumer_sync();  // every consumer is past its last read of the ring
    float* partial = reinterpret_cast<float*>(smem);  // [warp][col][MP], over the drained ring
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int col0 = NT ? 16 * i + g : 2 * i + 8 * g;
      const int col1 = NT ? col0 + 8 : col0 + 1;
#pragma unroll
      for (int t = 0; t < MT; t++) {
        float* p0 = partial + ((size_t)warp * TN + col0) * G::MP + t * 8 + 2 * j;
        float* p1 = partial + ((size_t)warp * TN + col1) * G::MP + t * 8 + 2 * j;
        *reinterpret_cast<float2*>(p0) = make_float2(acc[i][t][0], acc[i][t][1]);
        *reinterpret_cast<float2*>(p1) = make_float2(acc[i][t][2], acc[i][t][3]);
      }
    }
    consumer_sync();
    float* red = reinterpret_cast<float*>(smem + G::OFF_RED);
    for (int idx = tid; idx < TN * G::MP; idx += CONSUMER_THREADS) {
      float s = partial[idx];
#pragma unroll
      for (int w = 1; w < CONSUMER_WARPS; w++) s += partial[(size_t)w * TN * G::MP + idx];
      red[idx] = s;
    }
    consumer_sync();
  }

  // ---------------- meet the other K slices of the cluster, store ----------------
  if (S > 1) ptx::cluster_sync_all();
  if (warp < CONSUMER_WARPS && !*abort_flag) {
    const uint32_t cpr = TN / S;  // columns this rank finishes
    const uint32_t red_addr = smem_base + G::OFF_RED;
    for (uint32_t idx = tid; idx < cpr * p.m; idx += CONSUMER_THREADS) {
      const uint32_t col = rank * cpr + idx % cpr;
      const uint32_t r = idx / cpr;
      if (col >= cols) continue;
      float s = 0.0f;
      if (S == 1) {
        s = reinterpret_cast<const float*>(smem + G::OFF_RED)[col * G::MP + r];
      } else {
        for (uint32_t q = 0; q < S; q++) s += ptx::ld_cluster_f32(ptx::map_to_rank(red_addr + (col * G::MP + r) * 4, q));
      }
      float* cp = p.c + (uint64_t)r * p.ldc + n0 + col;
      *cp = (p.beta == 0.0f) ? p.alpha * s : p.alpha * s + p.beta * *cp;
    }
  }
  // No CTA may exit while a peer still reads its shared memory.
  if (S > 1) ptx::cluster_sync_all();
}

template <int DT, bool NT, int MT>
int32_t launch(AionCudaDevice* dev, const GemvParams& p, uint32_t split) {
  using G = Geom<DT, NT, MT>;
  auto kernel = gemv_q_mma_kernel<DT, NT, MT>;
  static bool configured[16] = {};
  if (!configured[dev->ordinal & 15]) {
    AION_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES));
    configured[dev->ordinal & 15] = true;
  }
  const uint32_t tiles = (p.n + TN - 1) / TN;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(tiles * split);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = G::SMEM_BYTES;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = split;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 2;
  AION_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p));
  return AION_CUDA_OK;
}

}  // namespace

int32_t gemv_mma(AionCudaDevice* dev, const MatMulArgs& g, bool probe_only) {
  if (g.m > 16 || g.k == 0) return AION_CUDA_UNSUPPORTED;
  if (g.n > 0xFFFFFFFFull - TN || g.k / QK > 0xFFFFFFFFull) return AION_CUDA_UNSUPPORTED;
  const uint64_t kblocks = g.k / QK;
  const uintptr_t baddr = reinterpret_cast<uintptr_t>(g.b);
  if (baddr & 15) return AION_CUDA_UNSUPPORTED;
  if (!g.nt) {
    // Every 64-column segment of a block row must start and end on 16 bytes.
    if (g.n % 8 != 0 || g.ldb % 8 != 0) return AION_CUDA_UNSUPPORTED;
  } else {
    if (g.dtype != AION_CUDA_DTYPE_Q8_0 || g.order != AION_CUDA_ORDER_ROW_MAJOR) return AION_CUDA_UNSUPPORTED;
    // A stage takes 8 blocks (272 bytes) of every row; rows are kblocks*34 bytes apart.
    if (kblocks % 8 != 0) return AION_CUDA_UNSUPPORTED;
  }
  if (probe_only) return AION_CUDA_OK;

  GemvParams p{};
  p.a = g.a;
  p.b = g.b;
  p.c = g.c;
  p.m = (uint32_t)g.m;
  p.n = (uint32_t)g.n;
  p.kblocks = (uint32_t)kblocks;
  p.lda = g.lda;
  p.ldb = g.ldb;
  p.ldc = g.ldc;
  p.alpha = g.alpha;
  p.beta = g.beta;
  p.fault = dev->fault_dev;
  p.a_vec4 = ((reinterpret_cast<uintptr_t>(g.a) & 15) == 0 && g.lda % 4 == 0) ? 1u : 0u;

  // Split K over a cluster until the grid covers the SMs about twice, as far as the
  // stage count allows.
  const uint32_t tiles = (p.n + TN - 1) / TN;
  const uint32_t stages = (p.kblocks + KBT - 1) / KBT;
  uint32_t split = 1;
  while (split < 8 && tiles * split < (uint32_t)dev->sm_count * 3 / 2 && split * 2 <= stages) split *= 2;
  if (dev->gemv_split_override) {
    split = dev->gemv_split_override;
    while (split > 1 && split > stages) split /= 2;
  }

  const bool two = g.m > 8;
  if (g.nt) return two ? launch<AION_CUDA_DTYPE_Q8_0, true, 2>(dev, p, split) : launch<AION_CUDA_DTYPE_Q8_0, true, 1>(dev, p, split);
  if (g.dtype == AION_CUDA_DTYPE_Q8_0)
    return two ? launch<AION_CUDA_DTYPE_Q8_0, false, 2>(dev, p, split) : launch<AION_CUDA_DTYPE_Q8_0, false, 1>(dev, p, split);
  return two ? launch<AION_CUDA_DTYPE_Q4_0, false, 2>(dev, p, split) : launch<AION_CUDA_DTYPE_Q4_0, false, 1>(dev, p, split);
}

}  // namespace aion
