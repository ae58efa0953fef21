// Grouped-query `Attention` step (src/aion/backend/cpu/exec/attention.zig:1444-1608).
//
// Semantics per output row (b, l, hq): keys [lo, hi) from the window
// (src/aion/graph/graph.zig:160-167) clipped to the ring's retained span
// (exec/attention.zig:1072-1075), logit = (q . k) * scale with optional soft cap,
// softmax, out = sum p v / sum p, zeros for an empty range. The reference's softmax uses
// a polynomial exp (kernels/fast_math.zig:79-92); this kernel uses the hardware exp2,
// which is closer to the exact value than the polynomial is.
//
// Two kernels:
//  * attn_decode_kernel — f16 K/V with Dk = Dv in {64, 128, 256}: the decode hot path.
//    HBM-bound: K and V are read from global memory once per (b, l, kv head); the up to
//    eight query heads of the group share them. With several query rows per request (prefill,
//    the reference's 32-row block kernel, exec/attention.zig:546-963) a CTA takes a block of
//    up to 64 (position, head) columns instead and streams K / V once for all of them, each
//    column masked to its own key range. K / V may live in a pool of pages behind a page table. A producer warp brings 64-key stages
//    of K and V rows into shared memory with 1-D bulk (TMA) copies (row pitch padded by
//    16 bytes so ldmatrix is conflict free); four consumer warps take 16 keys each.
//    Both contractions run on the tensor cores in transposed form so that no
//    accumulator row is padding: S^T[16 keys x 8 heads] = K . Q^T, then
//    O^T[Dv x 8 heads] += V^T . P^T, with P^T obtained from the S^T fragment by one
//    movmatrix transpose. An f32 q is split into two f16 terms so the logits keep f32
//    accuracy. The context is split across CTAs (split-K); each writes an
//    (unnormalised O, running max, sum) partial and the last CTA of a row to finish
//    merges them by log-sum-exp — no second launch.
//  * attn_generic_kernel — every other dtype / head size: one warp per key slice of a
//    row, f32 arithmetic, same merge inside the CTA.
#include <cfloat>
#include <cmath>
#include <mutex>

#include "act_image.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace aion {

namespace {

constexpr int KT = 64;              // keys per stage
constexpr int CONSUMER_WARPS = 4;   // 16 keys each
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
  const void* q;
  const void* k;
  const void* v;
  float* out;
  const int32_t* positions;
  const int32_t* lengths;
  uint32_t B, L, Hq, Hkv, Dk, Dv, T;
  uint32_t q_dtype, k_dtype, v_dtype;
  uint32_t rolling;
  uint32_t win_left, win_right, win_chunk;
  float scale, soft_cap;
  uint32_t splits;
  uint32_t head_groups;  // ceil((Hq/Hkv) / 8)
  uint32_t col_heads;    // query heads of a head group: min(Hq/Hkv, 8)
  uint32_t pos_per_tile; // query positions sharing one 8-column MMA tile
  uint32_t l_blocks;     // blocks of positions per request
  const int32_t* page_table;  // [B][pages_per_request] page numbers, or null: K / V are [B, T, ...]
  uint32_t page_tokens, pages_per_request, pool_pages;
  float* partial;        // [unit][split][columns][Dv + 4]: sums, max, sum of weights, pad
  int* tickets;          // [unit]
  int* fault;
  // Optional: the quantized image of `out` as [B*L, Hq*Dv] rows (act_image.cuh), for the matmul
  // that consumes the attention output.
  uint8_t* image;
  ActImageLayout image_layout;
  uint32_t image_dtype;
  uint32_t wait_limit;   // polls a barrier wait makes before it gives up and reports FAULT_WAIT_EXPIRED
  uint32_t drop_first;   // test hook: every CTA leaves out the copies of its first stage, so that wait runs out
};

struct KeyRange {
  uint32_t lo, hi;
  bool bad;
};

// Window and ring clipping of one query row; flags inputs the reference rejects.
__device__ __forceinline__ KeyRange key_range(const AttnParams& p, uint32_t b, uint32_t l) {
  KeyRange r{0, 0, false};
  int64_t valid_end = p.T;
  if (p.lengths) {
    const int32_t e = p.lengths[b];
    if (e < 0) { r.bad = true; return r; }
    valid_end = e;
  }
  if (!p.rolling && valid_end > (int64_t)p.T) { r.bad = true; return r; }
  int64_t q_pos = l;
  if (p.positions) {
    const int32_t qp = p.positions[(uint64_t)b * p.L + l];
    if (qp < 0) { r.bad = true; return r; }
    q_pos = qp;
  }
  const int64_t anchor = p.win_chunk > 0 ? (q_pos / p.win_chunk) * p.win_chunk : q_pos;
  const int64_t span = p.win_chunk > 0 ? p.win_chunk : 1;
  int64_t lo = anchor - min(anchor, (int64_t)p.win_left);
  int64_t hi = min(valid_end, anchor + span + (int64_t)p.win_right);
  if (p.rolling && valid_end > (int64_t)p.T) lo = max(lo, valid_end - (int64_t)p.T);
  if (hi > lo) {
    r.lo = (uint32_t)lo;
    r.hi = (uint32_t)hi;
  }
  return r;
}

__device__ __forceinline__ float soft_cap_logit(float x, float cap) { return cap > 0.0f ? cap * tanhf(x / cap) : x; }

// ------------------------------------------------------------------------------------
// tensor-core decode kernel
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Two shared-memory layouts of a K / V tile of KT rows:
//  * tiled (the usual case): the tile arrives as D/64 TMA boxes of 64 columns x KT rows with
//    the 128-byte swizzle, so 16-byte chunk c of row r sits in column block c/8 at
//    r*128 + ((c%8) ^ (r&7))*16 and ldmatrix is conflict free;
//  * padded rows (rolling caches, whose rows wrap and so cannot be one box): one bulk copy
//    per row at a pitch of D*2 + 16 bytes.
template <int D, bool TILED>
__device__ __forceinline__ uint32_t tile_off(uint32_t row, uint32_t chunk) {
  if (TILED) return (chunk >> 3) * (KT * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
  return row * (D * 2 + 16) + (chunk << 4);
}

// A CTA serves COLS "query columns" of one kv head: column = (query position, query head of the
// group). The MMAs run in transposed form, so a column is one of the 8 columns (n) of an MMA and
// NTT is the number of such 8-column tiles per CTA.
//  * decode (BLOCK = false): NT tiles, every consumer warp works on all of them and takes 16 of
//    a stage's 64 keys; the four warps are folded at the end.
//  * query blocks (BLOCK = true, l_q > 1): each warp owns NT tiles of its own and walks all 64
//    keys of every stage, so K and V are read once per block of positions and nothing is folded.
template <int D, bool QF32, bool BLOCK, int NT>
struct DecodeGeom {
  static constexpr int NTT = BLOCK ? CONSUMER_WARPS * NT : NT;
  static constexpr int COLS = 8 * NTT;
  static constexpr int PITCH = D * 2 + 16;            // bytes per K / V row in shared memory (padded layout)
  static constexpr int TILE_BYTES = KT * PITCH;       // one of K, V
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;  // K then V
  static constexpr int QFRAG_BYTES = (D / 16) * 32 * 8;  // one tile, one of hi, lo
  static constexpr int Q_BYTES = NTT * QFRAG_BYTES * (QF32 ? 2 : 1);
  static constexpr int STAGING_BUFS = BLOCK ? 1 : CONSUMER_WARPS;
  static constexpr int WS = COLS * D + 2 * COLS;      // floats per staging buffer: sums, then max and weight per column
  static constexpr int MERGE_BYTES = STAGING_BUFS * WS * 4;
  static constexpr int META_BYTES = COLS * 20;        // per column: output row x head, first key, key end, row of the [B*L] view, head
  static constexpr int NS_MAX = (220 * 1024 - Q_BYTES - META_BYTES - 256) / STAGE_BYTES;
  static constexpr int NS = NS_MAX > 4 ? 4 : NS_MAX;
  static_assert(NS >= 2, "ring too small");
  static_assert(MERGE_BYTES <= NS * STAGE_BYTES, "merge buffer reuses the ring");
  static constexpr int OFF_QHI = NS * STAGE_BYTES;
  static constexpr int OFF_QLO = OFF_QHI + NTT * QFRAG_BYTES;
  static constexpr int OFF_META = OFF_QHI + Q_BYTES;
  static constexpr int OFF_BARS = OFF_META + META_BYTES;
  static constexpr int SMEM_BYTES = OFF_BARS + 2 * NS * 8 + 32;
  // The merge of split partials keeps (max, weight) of every column and split at the start of the drained
  // ring and the merged sums ([COLS][D] floats) at its end.
  static constexpr int OFF_SUMS = NS * STAGE_BYTES - COLS * D * 4;
  static constexpr int MAX_SPLITS = (OFF_SUMS / 4 - COLS) / (2 * COLS);
  static_assert(OFF_SUMS % 16 == 0 && MAX_SPLITS >= 16, "room for the merge");
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory"); }

constexpr uint32_t NO_ROW = 0xFFFFFFFFu;

// The last step of one float4 of an output column: o / lsum (zeros for a column without keys), the store, and
// the quantized image of the output. All 32 lanes of a warp call it together (a column that does not exist
// passes on = false). Callers run it in a loop that is NOT unrolled: this code runs once per CTA, at the very
// end, on the CTA every other one is waiting for, and run once it costs what fetching its instructions costs
// (four columns spelled out side by side took 4 to 5 us, most of it in the quantizer).
template <int D>
__device__ __forceinline__ void finish_column(const AttnParams& p, float4 o, float lsum, bool on, bool has_keys, uint32_t col, uint32_t d4,
                                              const uint32_t* col_row, const uint32_t* col_orow, const uint32_t* col_head, bool report) {
  const bool good = lsum > 0.0f && isfinite(lsum);
  const float inv = good ? __frcp_rn(lsum) : 0.0f;
  float4 r = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
  if (!good) r = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (!good && on && has_keys && report) atomicCAS(p.fault, FAULT_NONE, FAULT_NONFINITE);
  if (on) *reinterpret_cast<float4*>(p.out + (uint64_t)col_row[col] * D + 4 * d4) = r;
  if (p.image) {
    const uint32_t irow = on ? col_orow[col] : 0, kb = on ? (col_head[col] * (D / 4) + d4) >> 3 : 0;
    if (p.image_dtype == AION_CUDA_DTYPE_Q8_0) quantize_store_block_8lanes<AION_CUDA_DTYPE_Q8_0>(r, d4 & 7, on, p.image, p.image_layout, irow, kb);
    else quantize_store_block_8lanes<AION_CUDA_DTYPE_Q4_0>(r, d4 & 7, on, p.image, p.image_layout, irow, kb);
  }
}

template <int D, bool QF32, bool TILED, bool BLOCK, int NT>
__global__ void __launch_bounds__(THREADS, 1) attn_decode_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tmap_k,
                                                                 const __grid_constant__ CUtensorMap tmap_v) {
  using G = DecodeGeom<D, QF32, BLOCK, NT>;
  constexpr int NS = G::NS, COLS = G::COLS, NTT = G::NTT;
  extern __shared__ __align__(1024) uint8_t smem[];  // swizzled TMA tiles need 1024-byte alignment
  const uint32_t smem_base = ptx::smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;

  // unit = (b, block of positions, hkv, head group); split = blockIdx.y
  const uint32_t unit = blockIdx.x;
  const uint32_t hg = unit % p.head_groups;
  const uint32_t hkv = (unit / p.head_groups) % p.Hkv;
  const uint32_t bl = unit / (p.head_groups * p.Hkv);
  // Later positions see more keys under a causal window: the blocks are handed out last first, so
  // the long ones start early and the short ones fill the tail.
  const uint32_t lb = p.l_blocks - 1 - bl % p.l_blocks, b = bl / p.l_blocks;
  const uint32_t split = blockIdx.y;
  const uint32_t group = p.Hq / p.Hkv;
  const uint32_t h0 = hkv * group + hg * 8;
  const uint32_t nh = min(8u, group - hg * 8);
  const uint32_t l0 = lb * (NTT * p.pos_per_tile);

  const uint32_t bar_full = smem_base + G::OFF_BARS;
  const uint32_t bar_empty = bar_full + NS * 8;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + G::OFF_BARS + 2 * NS * 8);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  uint32_t* union_range = reinterpret_cast<uint32_t*>(const_cast<int*>(abort_flag) + 2);  // lo, hi, bad
  uint32_t* col_row = reinterpret_cast<uint32_t*>(smem + G::OFF_META);  // (b*L + l)*Hq + head, NO_ROW for a column that is padding
  uint32_t* col_lo = col_row + COLS;
  uint32_t* col_hi = col_lo + COLS;
  uint32_t* col_orow = col_hi + COLS;   // b*L + l: the row of the output seen as [B*L, Hq*Dv]
  uint32_t* col_head = col_orow + COLS;

  if (tid == 0) {
    for (int s = 0; s < NS; s++) {
      ptx::mbar_init(bar_full + 8 * s, 1);
      ptx::mbar_init(bar_empty + 8 * s, CONSUMER_WARPS);
    }
    *abort_flag = 0;
    *last_flag = 0;
    union_range[0] = 0xFFFFFFFFu;
    union_range[1] = 0;
    union_range[2] = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  ptx::pdl_launch_dependents();
  // q, K, V, positions and lengths may all come from the previous kernel.
  ptx::pdl_wait();

  // Every column's row and key range; the CTA walks the union of the ranges and masks per column.
  for (uint32_t c = tid; c < (uint32_t)COLS; c += THREADS) {
    const uint32_t tile = c >> 3, cc = c & 7;
    const uint32_t pl = cc / p.col_heads, hh = cc - pl * p.col_heads;
    const uint32_t l = l0 + tile * p.pos_per_tile + pl;
    uint32_t row = NO_ROW, lo = 0, hi = 0;
    if (pl < p.pos_per_tile && hh < nh && l < p.L) {
      const KeyRange kr = key_range(p, b, l);
      if (kr.bad) atomicOr(union_range + 2, 1u);
      row = (b * p.L + l) * p.Hq + h0 + hh;
      lo = kr.lo, hi = kr.hi;
      if (hi > lo) {
        atomicMin(union_range, lo);
        atomicMax(union_range + 1, hi);
      }
    }
    col_row[c] = row, col_lo[c] = lo, col_hi[c] = hi;
    col_orow[c] = b * p.L + l, col_head[c] = h0 + hh;
  }
  __syncthreads();
  const bool bad = union_range[2] != 0;
  if (bad && tid == 0) atomicExch(p.fault, FAULT_INVALID_ARGUMENT);
  const uint32_t u_hi = union_range[1], u_lo = min(union_range[0], u_hi);
  // Splits walk disjoint slices of the union. With a page table a stage must not straddle a
  // page, so slices then start on multiples of a stage (the keys before a column's range are
  // masked like any others).
  const uint32_t base = p.page_tokens ? (u_lo / KT) * KT : u_lo;
  uint32_t per = (u_hi - base + p.splits - 1) / p.splits;
  per = p.page_tokens ? (per + KT - 1) / KT * KT : (per + 15) & ~15u;
  const uint32_t my_lo = min(u_hi, base + split * per);
  const uint32_t my_hi = min(u_hi, my_lo + per);
  const uint32_t ntiles = (my_hi - my_lo + KT - 1) / KT;

  // running state of this lane's two columns (2j, 2j+1) of every tile, log2 domain
  float m_run[NT][2], l_run[NT][2];
  float acc[D / 16][NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.0f;
#pragma unroll
    for (int t = 0; t < D / 16; t++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[t][nt][e] = 0.0f;
  }

  if (warp == CONSUMER_WARPS) {
    // ---------------- producer ----------------
    const __half* kbase = static_cast<const __half*>(p.k);
    const __half* vbase = static_cast<const __half*>(p.v);
    uint32_t issued = 0;
    for (uint32_t it = 0; it < ntiles; it++) {
      const uint32_t slot = it % NS;
      if (*abort_flag) break;
      if (it >= (uint32_t)NS && !ptx::mbar_wait_bounded(bar_empty + 8 * slot, ((it / NS) - 1) & 1, p.wait_limit)) {
        if (lane == 0) {
          atomicExch(p.fault, FAULT_WAIT_EXPIRED);
          *abort_flag = 1;
        }
        break;
      }
      const uint32_t t0 = my_lo + it * KT;
      const uint32_t cnt = min((uint32_t)KT, my_hi - t0);
      const uint32_t full = bar_full + 8 * slot;
      const uint32_t stage = smem_base + slot * G::STAGE_BYTES;
      if (TILED) {
        // Whole boxes always: rows past the range arrive too (later keys, the next request's
        // rows or zeros past the tensor) and are cleared by the consumers before use.
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(full, 2u * KT * D * 2);
          if (p.drop_first && it == 0) continue;   // (test hook: the bytes never arrive, the consumers' wait runs out)
          int32_t y;
          if (p.page_tokens) {
            // t0 is a multiple of a stage and a page is a whole number of stages.
            const int32_t page = p.page_table[(uint64_t)b * p.pages_per_request + t0 / p.page_tokens];
            y = (int32_t)((uint32_t)page * p.page_tokens + t0 % p.page_tokens);
          } else {
            y = (int32_t)(b * p.T + t0);
          }
#pragma unroll
          for (int cb = 0; cb < D / 64; cb++) {
            ptx::tma_load_2d(stage + cb * (KT * 128), &tmap_k, (int32_t)(hkv * D + cb * 64), y, full);
            ptx::tma_load_2d(stage + G::TILE_BYTES + cb * (KT * 128), &tmap_v, (int32_t)(hkv * D + cb * 64), y, full);
          }
        }
      } else {
        if (lane == 0) ptx::mbar_arrive_expect_tx(full, cnt * (uint32_t)(D * 2) * 2u);
        __syncwarp();
        for (uint32_t r = lane; r < cnt; r += 32) {
          const uint32_t t = t0 + r;
          const uint64_t row = ((uint64_t)b * p.T + (p.rolling ? t % p.T : t)) * p.Hkv + hkv;
          ptx::bulk_g2s(stage + r * G::PITCH, kbase + row * D, D * 2, full);
          ptx::bulk_g2s(stage + G::TILE_BYTES + r * G::PITCH, vbase + row * D, D * 2, full);
        }
      }
      issued = it + 1;
    }
    if (*abort_flag)
      for (uint32_t it = issued > (uint32_t)NS ? issued - NS : 0; it < issued; it++)
        ptx::mbar_wait_bounded(bar_full + 8 * (it % NS), (it / NS) & 1, min(p.wait_limit, 1u << 16));
  } else {
    // ---------------- consumers ----------------
    // Q^T fragments: for tile n and k-step s, lane (g, j) needs (q[column g][16s+2j], q[..][16s+2j+1])
    // and the same at +8; padding columns are zero. An f32 q is split hi + lo.
    {
      uint2* qhi = reinterpret_cast<uint2*>(smem + G::OFF_QHI);
      uint2* qlo = reinterpret_cast<uint2*>(smem + G::OFF_QLO);
      // Every thread builds ITEMS fragment words. The loads of a batch of them are all issued before the
      // first is used: taken one item at a time, each item's loads were a separate trip to L2 and this loop
      // was a quarter of a short kernel.
      constexpr int ITEMS = NTT * (D / 16) * 32 / (CONSUMER_WARPS * 32);
      constexpr int BATCH = ITEMS < 8 ? ITEMS : 8;
      static_assert(ITEMS >= 1 && ITEMS % BATCH == 0, "whole batches of fragment words per thread");
#pragma unroll 1
      for (int i0 = 0; i0 < ITEMS; i0 += BATCH) {
        float v[BATCH][4];
#pragma unroll
        for (int u = 0; u < BATCH; u++) {
          const int i = tid + (i0 + u) * (CONSUMER_WARPS * 32);
          const int tile = i / ((D / 16) * 32), s = (i >> 5) % (D / 16), ln = i & 31, gg = ln >> 2, jj = ln & 3;
          v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.0f;
          const uint32_t row = col_row[tile * 8 + gg];
          if (row != NO_ROW) {
            const uint64_t off = (uint64_t)row * D + 16 * s + 2 * jj;
            if (QF32) {
              const float* qp = static_cast<const float*>(p.q) + off;
              v[u][0] = qp[0]; v[u][1] = qp[1]; v[u][2] = qp[8]; v[u][3] = qp[9];
            } else {
              const __half* qp = static_cast<const __half*>(p.q) + off;
              v[u][0] = __half2float(qp[0]); v[u][1] = __half2float(qp[1]);
              v[u][2] = __half2float(qp[8]); v[u][3] = __half2float(qp[9]);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < BATCH; u++) {
          const int i = tid + (i0 + u) * (CONSUMER_WARPS * 32);
          const __half h0a = __float2half_rn(v[u][0]), h1a = __float2half_rn(v[u][1]), h2a = __float2half_rn(v[u][2]), h3a = __float2half_rn(v[u][3]);
          qhi[i] = make_uint2(pack_half2(__half2float(h0a), __half2float(h1a)), pack_half2(__half2float(h2a), __half2float(h3a)));
          if (QF32)
            qlo[i] = make_uint2(pack_half2(v[u][0] - __half2float(h0a), v[u][1] - __half2float(h1a)),
                                pack_half2(v[u][2] - __half2float(h2a), v[u][3] - __half2float(h3a)));
        }
      }
    }
    // This lane's columns and their key ranges clipped to this CTA's slice (lo, length).
    const uint32_t tile0 = BLOCK ? warp * NT : 0;
    uint32_t c_lo[NT][2], c_len[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int hh = 0; hh < 2; hh++) {
        const uint32_t c = (tile0 + nt) * 8 + 2 * j + hh;
        const uint32_t lo = max(col_lo[c], my_lo), hi = min(col_hi[c], my_hi);
        c_lo[nt][hh] = lo;
        c_len[nt][hh] = hi > lo ? hi - lo : 0;
      }
    consumer_sync();

    const float sc = (p.soft_cap > 0.0f) ? p.scale : p.scale * LOG2E;
    const uint2* qhi = reinterpret_cast<const uint2*>(smem + G::OFF_QHI) + tile0 * (D / 16) * 32;
    const uint2* qlo = reinterpret_cast<const uint2*>(smem + G::OFF_QLO) + tile0 * (D / 16) * 32;
    bool ok = true;
    for (uint32_t it = 0; it < ntiles; it++) {
      const uint32_t slot = it % NS;
      if (ok && (*abort_flag || !ptx::mbar_wait_bounded(bar_full + 8 * slot, (it / NS) & 1, p.wait_limit))) {
        if (lane == 0 && !*abort_flag) {
          atomicExch(p.fault, FAULT_WAIT_EXPIRED);
          *abort_flag = 1;
        }
        ok = false;
      }
      const uint32_t t0 = my_lo + it * KT;
      const uint32_t cnt = min((uint32_t)KT, my_hi - t0);
      const uint32_t kst = smem_base + slot * G::STAGE_BYTES;
      const uint32_t vst = kst + G::TILE_BYTES;
#pragma unroll 1
      for (uint32_t r0 = BLOCK ? 0 : 16 * warp; r0 < (BLOCK ? (uint32_t)KT : 16 * warp + 16); r0 += 16) {
        if (!ok || r0 >= cnt) break;
        const uint32_t valid = min(16u, cnt - r0);
        if (valid < 16) {
          // Rows past the slice were not copied (or hold other rows): clear them so stale bits cannot
          // reach an MMA. (With query blocks every warp clears the same rows with the same zeros.)
          uint8_t* kt = smem + slot * G::STAGE_BYTES;
          for (uint32_t i = lane; i < (16 - valid) * (D * 2 / 16); i += 32) {
            const uint32_t rr = r0 + valid + i / (D * 2 / 16), cc = i % (D * 2 / 16);
            *reinterpret_cast<uint4*>(kt + tile_off<D, TILED>(rr, cc)) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(kt + G::TILE_BYTES + tile_off<D, TILED>(rr, cc)) = make_uint4(0, 0, 0, 0);
          }
          __syncwarp();
        }
        // ---- S^T[16 keys x 8 columns] = K . Q^T per tile ----
        // Separate accumulators (even / odd k-steps when there is one tile, high / low half of an
        // f32 q) keep the chains of dependent MMAs short.
        constexpr int CH = NT == 1 ? 2 : 1;
        float s_hi[NT][CH][4], s_lo[NT][CH][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int c = 0; c < CH; c++)
#pragma unroll
            for (int e = 0; e < 4; e++) s_hi[nt][c][e] = s_lo[nt][c][e] = 0.0f;
        {
          const uint32_t a_row = r0 + (lane & 7) + 8 * ((lane >> 3) & 1);
          const uint32_t a_chunk = lane >> 4;
#pragma unroll
          for (int ks = 0; ks < D / 16; ks++) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(kst + tile_off<D, TILED>(a_row, 2 * ks + a_chunk), a0, a1, a2, a3);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
              const uint2 bh = qhi[(nt * (D / 16) + ks) * 32 + lane];
              mma_f16(s_hi[nt][ks % CH], a0, a1, a2, a3, bh.x, bh.y);
              if (QF32) {
                const uint2 bl2 = qlo[(nt * (D / 16) + ks) * 32 + lane];
                mma_f16(s_lo[nt][ks % CH], a0, a1, a2, a3, bl2.x, bl2.y);
              }
            }
          }
        }
        // s[0], s[1]: key g, columns 2j, 2j+1;  s[2], s[3]: key g+8.
        const uint32_t key0 = t0 + r0 + g, key1 = key0 + 8;
        float alpha[NT][2];
        uint32_t pb0[NT], pb1[NT];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          float lg[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            float x = (CH == 2 ? (s_hi[nt][0][e] + s_hi[nt][CH - 1][e]) + (s_lo[nt][0][e] + s_lo[nt][CH - 1][e])
                               : s_hi[nt][0][e] + s_lo[nt][0][e]) * sc;
            if (p.soft_cap > 0.0f) x = soft_cap_logit(x, p.soft_cap) * LOG2E;
            const uint32_t key = e < 2 ? key0 : key1;
            lg[e] = (key - c_lo[nt][e & 1] < c_len[nt][e & 1]) ? x : -INFINITY;
          }
          float mx[2] = {fmaxf(lg[0], lg[2]), fmaxf(lg[1], lg[3])};
#pragma unroll
          for (int o = 4; o < 32; o <<= 1) {
            mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xFFFFFFFFu, mx[0], o));
            mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xFFFFFFFFu, mx[1], o));
          }
          float mu[2];
#pragma unroll
          for (int hh = 0; hh < 2; hh++) {
            const float m_new = fmaxf(m_run[nt][hh], mx[hh]);
            mu[hh] = m_new == -INFINITY ? 0.0f : m_new;   // a column that has seen no key yet
            alpha[nt][hh] = exp2f(m_run[nt][hh] - mu[hh]);  // exp2(-inf) = 0 on the first keys
            m_run[nt][hh] = m_new;
          }
          const float pr0 = exp2f(lg[0] - mu[0]), pr1 = exp2f(lg[1] - mu[1]), pr2 = exp2f(lg[2] - mu[0]), pr3 = exp2f(lg[3] - mu[1]);
          l_run[nt][0] = l_run[nt][0] * alpha[nt][0] + pr0 + pr2;
          l_run[nt][1] = l_run[nt][1] * alpha[nt][1] + pr1 + pr3;
          // P^T fragments (k = key, n = column) from the S^T accumulator layout by an 8x8 transpose.
          pb0[nt] = movmatrix_trans(pack_half2(pr0, pr1));
          pb1[nt] = movmatrix_trans(pack_half2(pr2, pr3));
        }
        // ---- O^T[Dv x 8 columns] = alpha * O^T + V^T . P^T per tile ----
        const uint32_t v_row = r0 + (lane & 7) + 8 * (lane >> 4);
        const uint32_t v_chunk = (lane >> 3) & 1;
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
          uint32_t a0, a1, a2, a3;
          ldmatrix_x4_trans(vst + tile_off<D, TILED>(v_row, 2 * mt + v_chunk), a0, a1, a2, a3);
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            acc[mt][nt][0] *= alpha[nt][0];
            acc[mt][nt][1] *= alpha[nt][1];
            acc[mt][nt][2] *= alpha[nt][0];
            acc[mt][nt][3] *= alpha[nt][1];
            mma_f16(acc[mt][nt], a0, a1, a2, a3, pb0[nt], pb1[nt]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_empty + 8 * slot);
    }

    // ---------------- stage the warps' results in the drained ring; fold them (decode) ----------------
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l_run[nt][0] += __shfl_xor_sync(0xFFFFFFFFu, l_run[nt][0], o);
        l_run[nt][1] += __shfl_xor_sync(0xFFFFFFFFu, l_run[nt][1], o);
      }
    consumer_sync();
    constexpr int WS = G::WS, NB = G::STAGING_BUFS;
    {
      float* mb = reinterpret_cast<float*>(smem) + (BLOCK ? 0 : (size_t)warp * WS);  // [COLS][D], then max[COLS], weight[COLS]
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        const uint32_t c0 = (tile0 + nt) * 8 + 2 * j;
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
          mb[c0 * D + mt * 16 + g] = acc[mt][nt][0];
          mb[(c0 + 1) * D + mt * 16 + g] = acc[mt][nt][1];
          mb[c0 * D + mt * 16 + g + 8] = acc[mt][nt][2];
          mb[(c0 + 1) * D + mt * 16 + g + 8] = acc[mt][nt][3];
        }
        if (g == 0) {
          mb[COLS * D + c0] = m_run[nt][0];
          mb[COLS * D + c0 + 1] = m_run[nt][1];
          mb[COLS * D + COLS + c0] = l_run[nt][0];
          mb[COLS * D + COLS + c0 + 1] = l_run[nt][1];
        }
      }
    }
    consumer_sync();
    const float* all = reinterpret_cast<const float*>(smem);
    // A partial row is D sums, then (max, sum of weights), padded to a 16-byte multiple so
    // that the merge reads it in float4s.
    constexpr int PP = D + 4;
    float* part = p.partial + ((uint64_t)unit * p.splits + split) * COLS * PP;
    const bool direct = p.splits == 1;
    // Thread t owns the float4s t, t + 128, ... of the CTA's [COLS][D] outputs: eight consecutive
    // lanes hold one 32-block of an output row.
    constexpr int C4 = (COLS * D / 4) / (CONSUMER_WARPS * 32);
    static_assert(C4 >= 1 && C4 * CONSUMER_WARPS * 32 * 4 == COLS * D, "whole float4 columns per thread");
    constexpr int CHK = C4 < 4 ? C4 : 4;
    static_assert(C4 % CHK == 0, "whole chunks");
    const uint32_t d4 = tid % (D / 4);   // the same for every column of this thread: 128 threads are a multiple of D/4
#pragma unroll 1
    for (int c = 0; c < C4; c++) {
      const uint32_t idx4 = tid + c * (CONSUMER_WARPS * 32), col = idx4 / (D / 4);
      const bool on = col_row[col] != NO_ROW;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NB; w++) M = fmaxf(M, all[w * WS + COLS * D + col]);
      float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      float lsum = 0.0f;
#pragma unroll
      for (int w = 0; w < NB; w++) {
        const float mw = all[w * WS + COLS * D + col];
        const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
        const float4 x = *reinterpret_cast<const float4*>(all + w * WS + 4 * idx4);
        o.x += x.x * f; o.y += x.y * f; o.z += x.z * f; o.w += x.w * f;
        lsum += all[w * WS + COLS * D + COLS + col] * f;
      }
      if (direct) {
        finish_column<D>(p, o, lsum, on, col_hi[col] > col_lo[col], col, d4, col_row, col_orow, col_head, !bad && !*abort_flag);
      } else if (on) {
        *reinterpret_cast<float4*>(part + col * PP + 4 * d4) = o;
        if (d4 == 0) *reinterpret_cast<float2*>(part + col * PP + D) = make_float2(M, lsum);
      }
    }
    if (!direct) {
      // The last CTA of this unit to arrive merges every split's partial.
      __threadfence();
      consumer_sync();
      if (tid == 0) {
        const int prev = atomicAdd(p.tickets + unit, 1);
        const int last = (prev == (int)p.splits - 1);
        if (last) p.tickets[unit] = 0;  // ready for the next launch
        *last_flag = last;
      }
      consumer_sync();
      if (*last_flag) {
        __threadfence();
        // The merge is a chain of L2 round trips on one CTA, so it keeps them few: one pass
        // fetches every split's (max, sum) pair into shared memory (the ring is drained, its
        // space is free), the factors come from there, and the weighted sums then run over
        // float4 loads issued sixteen at a time per thread.
        const float* pu = p.partial + (uint64_t)unit * p.splits * COLS * PP;
        float* fac = reinterpret_cast<float*>(smem);  // [COLS][splits]: max, then factor
        float* wsum = fac + COLS * p.splits;          // [COLS][splits]: sum of weights
        float* lsums = wsum + COLS * p.splits;        // [COLS]
        float4* sums = reinterpret_cast<float4*>(smem + G::OFF_SUMS);   // [C4][128]: the merged sums
        for (uint32_t idx = tid; idx < COLS * p.splits; idx += CONSUMER_WARPS * 32) {
          const uint32_t h = idx / p.splits, s2 = idx % p.splits;
          float2 ml = make_float2(-INFINITY, 0.0f);
          if (col_row[h] != NO_ROW) ml = __ldcg(reinterpret_cast<const float2*>(pu + (size_t)(s2 * COLS + h) * PP + D));
          fac[idx] = ml.x;
          wsum[idx] = ml.y;
        }
        consumer_sync();
        for (uint32_t h = warp; h < (uint32_t)COLS; h += CONSUMER_WARPS) {
          float M = -INFINITY;
          for (uint32_t s2 = lane; s2 < p.splits; s2 += 32) M = fmaxf(M, fac[h * p.splits + s2]);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
          float lsum = 0.0f;
          for (uint32_t s2 = lane; s2 < p.splits; s2 += 32) {
            const float ms = fac[h * p.splits + s2];
            const float f = (ms == -INFINITY) ? 0.0f : exp2f(ms - M);
            fac[h * p.splits + s2] = f;
            lsum += wsum[h * p.splits + s2] * f;
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xFFFFFFFFu, lsum, o);
          if (lane == 0) lsums[h] = lsum;
        }
        consumer_sync();
#pragma unroll 1
        for (int cb = 0; cb < C4; cb += CHK) {
          const float* colp[CHK];
          const float* fh[CHK];
          bool live[CHK], has_keys[CHK];
          uint32_t col[CHK];
          float4 o[CHK];
          float lsum[CHK];
#pragma unroll
          for (int c = 0; c < CHK; c++) {
            const uint32_t idx4 = tid + (cb + c) * (CONSUMER_WARPS * 32);
            col[c] = idx4 / (D / 4);
            live[c] = col_row[col[c]] != NO_ROW;
            has_keys[c] = col_hi[col[c]] > col_lo[col[c]];
            colp[c] = pu + (size_t)col[c] * PP + 4 * d4;
            fh[c] = fac + col[c] * p.splits;
            lsum[c] = lsums[col[c]];
            o[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          }
          for (uint32_t s2 = 0; s2 < p.splits; s2 += 4) {
            float4 v[CHK][4];
            float f[CHK][4];
#pragma unroll
            for (int c = 0; c < CHK; c++)
#pragma unroll
              for (int k = 0; k < 4; k++) {
                const uint32_t ss = s2 + k;
                const bool on = live[c] && ss < p.splits;
                v[c][k] = on ? __ldcg(reinterpret_cast<const float4*>(colp[c] + (size_t)ss * COLS * PP)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                f[c][k] = on ? fh[c][ss] : 0.0f;
              }
#pragma unroll
            for (int c = 0; c < CHK; c++)
#pragma unroll
              for (int k = 0; k < 4; k++) {  // splits in order
                o[c].x += v[c][k].x * f[c][k];
                o[c].y += v[c][k].y * f[c][k];
                o[c].z += v[c][k].z * f[c][k];
                o[c].w += v[c][k].w * f[c][k];
              }
          }
          // The sums go through shared memory (this thread's own slots) so that the loop below can stay rolled.
#pragma unroll
          for (int c = 0; c < CHK; c++) sums[(cb + c) * (CONSUMER_WARPS * 32) + tid] = o[c];
        }
#pragma unroll 1
        for (int c = 0; c < C4; c++) {
          const uint32_t col = (tid + c * (CONSUMER_WARPS * 32)) / (D / 4);
          finish_column<D>(p, sums[c * (CONSUMER_WARPS * 32) + tid], lsums[col], col_row[col] != NO_ROW, col_hi[col] > col_lo[col], col, d4,
                           col_row, col_orow, col_head, !bad);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// any-dtype, any-head-size kernel: one CTA per output row (b, l, hq), 4 warps stride the
// keys, lanes stride the head dimension; per-warp online softmax, merged in shared memory.
// ------------------------------------------------------------------------------------
constexpr int GEN_WARPS = 4;
constexpr int GEN_MAX_DV_PER_LANE = 32;  // Dv <= 1024

__device__ __forceinline__ float load_as_float(const void* base, uint32_t dtype, uint64_t idx) {
  return dtype == AION_CUDA_DTYPE_F32 ? static_cast<const float*>(base)[idx]
                                      : __half2float(static_cast<const __half*>(base)[idx]);
}

__global__ void __launch_bounds__(GEN_WARPS * 32) attn_generic_kernel(const AttnParams p) {
  extern __shared__ float gsm[];  // q[Dk], then per warp: acc[Dv], m, l
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t row = blockIdx.x;
  const uint32_t hq = row % p.Hq;
  const uint32_t l = (row / p.Hq) % p.L;
  const uint32_t b = row / (p.Hq * p.L);
  const uint32_t hkv = hq / (p.Hq / p.Hkv);
  float* qs = gsm;
  float* wbuf = gsm + p.Dk + (size_t)warp * (p.Dv + 2);

  const KeyRange kr = key_range(p, b, l);
  if (kr.bad && tid == 0) atomicExch(p.fault, FAULT_INVALID_ARGUMENT);
  for (uint32_t i = tid; i < p.Dk; i += blockDim.x)
    qs[i] = load_as_float(p.q, p.q_dtype, (((uint64_t)b * p.L + l) * p.Hq + hq) * p.Dk + i);
  __syncthreads();

  float m_run = -INFINITY, l_run = 0.0f;
  float acc[GEN_MAX_DV_PER_LANE];
#pragma unroll
  for (int i = 0; i < GEN_MAX_DV_PER_LANE; i++) acc[i] = 0.0f;

  for (uint32_t t = kr.lo + warp; t < kr.hi; t += GEN_WARPS) {
    const uint64_t krow = ((uint64_t)b * p.T + (p.rolling ? t % p.T : t)) * p.Hkv + hkv;
    float dot = 0.0f;
    for (uint32_t i = lane; i < p.Dk; i += 32) dot = fmaf(qs[i], load_as_float(p.k, p.k_dtype, krow * p.Dk + i), dot);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
    const float lg = soft_cap_logit(dot * p.scale, p.soft_cap) * LOG2E;
    const float m_new = fmaxf(m_run, lg);
    const float alpha = exp2f(m_run - m_new);
    const float pr = exp2f(lg - m_new);
    l_run = l_run * alpha + pr;
    m_run = m_new;
#pragma unroll
    for (int i = 0; i < GEN_MAX_DV_PER_LANE; i++) {
      const uint32_t d = lane + 32 * i;
      if (d < p.Dv) acc[i] = acc[i] * alpha + pr * load_as_float(p.v, p.v_dtype, krow * p.Dv + d);
    }
  }
#pragma unroll
  for (int i = 0; i < GEN_MAX_DV_PER_LANE; i++) {
    const uint32_t d = lane + 32 * i;
    if (d < p.Dv) wbuf[d] = acc[i];
  }
  if (lane == 0) {
    wbuf[p.Dv] = m_run;
    wbuf[p.Dv + 1] = l_run;
  }
  __syncthreads();
  float* orow = p.out + (((uint64_t)b * p.L + l) * p.Hq + hq) * p.Dv;
  const float* base = gsm + p.Dk;
  float M = -INFINITY;
  for (int w = 0; w < GEN_WARPS; w++) M = fmaxf(M, base[(size_t)w * (p.Dv + 2) + p.Dv]);
  float lsum = 0.0f;
  for (int w = 0; w < GEN_WARPS; w++) {
    const float mw = base[(size_t)w * (p.Dv + 2) + p.Dv];
    lsum += (mw == -INFINITY) ? 0.0f : base[(size_t)w * (p.Dv + 2) + p.Dv + 1] * exp2f(mw - M);
  }
  const bool good = lsum > 0.0f && isfinite(lsum);
  if (!good && kr.hi > kr.lo && !kr.bad && tid == 0) atomicCAS(p.fault, FAULT_NONE, FAULT_NONFINITE);
  for (uint32_t d = tid; d < p.Dv; d += blockDim.x) {
    float o = 0.0f;
    for (int w = 0; w < GEN_WARPS; w++) {
      const float mw = base[(size_t)w * (p.Dv + 2) + p.Dv];
      if (mw != -INFINITY) o += base[(size_t)w * (p.Dv + 2) + d] * exp2f(mw - M);
    }
    orow[d] = good ? o / lsum : 0.0f;
  }
}

template <int D, bool QF32, bool TILED, bool BLOCK, int NT>
int32_t launch_decode_as(AionCudaDevice* dev, const AttnParams& p, uint32_t units, const CUtensorMap& tk, const CUtensorMap& tv) {
  using G = DecodeGeom<D, QF32, BLOCK, NT>;
  auto kernel = attn_decode_kernel<D, QF32, TILED, BLOCK, NT>;
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
  if (p.splits > (uint32_t)G::MAX_SPLITS) return fail(AION_CUDA_INTERNAL_ERROR, "attention: %u splits exceed the merge buffer", p.splits);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(units, p.splits);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = G::SMEM_BYTES;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl_main = std::getenv("AION_CUDA_NO_PDL_MAIN") != nullptr;  // tuning only
  cfg.numAttrs = no_pdl_main ? 0 : 1;
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  AION_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p, tk, tv));
  return AION_CUDA_OK;
}

template <int D, bool QF32, bool BLOCK, int NT>
int32_t launch_decode(AionCudaDevice* dev, const AttnParams& p, uint32_t units) {
  CUtensorMap tk{}, tv{};
  // K and V as [rows][Hkv*D columns] f16, rows = B*T (or every row of the page pool); a rolling
  // cache's rows wrap, so it keeps row copies.
  const uint64_t rows = p.page_tokens ? (uint64_t)p.pool_pages * p.page_tokens : (uint64_t)p.B * p.T;
  if (!p.rolling && rows < (1ull << 31)) {
    const uint64_t cols = (uint64_t)p.Hkv * D;
    if (int32_t st = tensor_map_16bit_sw128(p.k, false, rows, cols, cols * 2, 64, KT, &tk)) return st;
    if (int32_t st = tensor_map_16bit_sw128(p.v, false, rows, cols, cols * 2, 64, KT, &tv)) return st;
    return launch_decode_as<D, QF32, true, BLOCK, NT>(dev, p, units, tk, tv);
  }
  if (p.page_tokens) return fail(AION_CUDA_UNSUPPORTED, "attention: a paged cache needs the tiled path (no rolling, fewer than 2^31 pool rows)");
  return launch_decode_as<D, QF32, false, BLOCK, NT>(dev, p, units, tk, tv);
}

}  // namespace

int32_t attention_launch(AionCudaDevice* dev, const AionCudaAttention* s) {
  AttnParams p{};
  const uint64_t B = s->batch, L = s->l_q, Hq = s->h_q, Hkv = s->h_kv, Dk = s->d_k, Dv = s->d_v, T = s->t_cap;
  if (B > 0x7FFFFFFF || L > 0x7FFFFFFF || Hq > 65535 || Dk > 65535 || Dv > 65535 || T > 0x7FFFFFFF || B * L * Hq > 0x7FFFFFFF)
    return fail(AION_CUDA_UNSUPPORTED, "attention: a dimension is beyond what the kernels index");
  auto esz = [](uint32_t dt) { return dt == AION_CUDA_DTYPE_F32 ? 4u : 2u; };
  const bool paged = s->page_table.handle != 0;
  const uint64_t page_tokens = s->page_tokens, pool_pages = s->pool_pages;
  uint64_t pages_per_request = 0;
  if (paged) {
    if (page_tokens == 0 || page_tokens % KT != 0 || page_tokens > (1u << 20))
      return fail(AION_CUDA_INVALID_ARGUMENT, "attention: page_tokens %llu must be a positive multiple of %d", (unsigned long long)page_tokens, KT);
    if (pool_pages == 0 || pool_pages * page_tokens > 0x7FFFFFFFull)
      return fail(AION_CUDA_INVALID_ARGUMENT, "attention: pool of %llu pages", (unsigned long long)pool_pages);
    if (s->rolling) return fail(AION_CUDA_UNSUPPORTED, "attention: a rolling cache cannot be paged");
    pages_per_request = (T + page_tokens - 1) / page_tokens;
  }
  const uint64_t kv_rows = paged ? pool_pages * page_tokens : B * T;
  const uint8_t *q, *k, *v;
  float* out;
  if (int32_t st = resolve(s->q, B * L * Hq * Dk * esz(s->q_dtype), "attention.q", &q)) return st;
  if (int32_t st = resolve(s->k, kv_rows * Hkv * Dk * esz(s->k_dtype), "attention.k", &k)) return st;
  if (int32_t st = resolve(s->v, kv_rows * Hkv * Dv * esz(s->v_dtype), "attention.v", &v)) return st;
  if (int32_t st = resolve(s->out, B * L * Hq * Dv * sizeof(float), "attention.out", &out)) return st;
  p.q = q;
  p.k = k;
  p.v = v;
  p.out = out;
  if (s->query_positions.handle) {
    if (int32_t st = resolve(s->query_positions, B * L * 4, "attention.query_positions", &p.positions)) return st;
  }
  if (s->kv_lengths.handle) {
    if (int32_t st = resolve(s->kv_lengths, B * 4, "attention.kv_lengths", &p.lengths)) return st;
  }
  if (paged) {
    if (int32_t st = resolve(s->page_table, B * pages_per_request * 4, "attention.page_table", &p.page_table)) return st;
    p.page_tokens = (uint32_t)page_tokens;
    p.pages_per_request = (uint32_t)pages_per_request;
    p.pool_pages = (uint32_t)pool_pages;
  }
  p.B = (uint32_t)B; p.L = (uint32_t)L; p.Hq = (uint32_t)Hq; p.Hkv = (uint32_t)Hkv;
  p.Dk = (uint32_t)Dk; p.Dv = (uint32_t)Dv; p.T = (uint32_t)T;
  p.q_dtype = s->q_dtype; p.k_dtype = s->k_dtype; p.v_dtype = s->v_dtype;
  p.rolling = s->rolling ? 1u : 0u;
  p.win_left = s->window_left; p.win_right = s->window_right; p.win_chunk = s->window_chunk;
  p.scale = s->scale;
  p.soft_cap = s->soft_cap;
  p.fault = dev->fault_dev;
  p.wait_limit = dev->debug_expire_waits ? (1u << 6) : (1u << 20);
  p.drop_first = dev->debug_expire_waits ? 1u : 0u;

  const bool f16kv = s->k_dtype == AION_CUDA_DTYPE_F16 && s->v_dtype == AION_CUDA_DTYPE_F16;
  const bool aligned = ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(q) & 3) == 0;
  const bool tensor_path = f16kv && aligned && Dk == Dv && (Dk == 64 || Dk == 128 || Dk == 256) && !(s->flags & AION_CUDA_ATTENTION_GENERIC);
  if (paged && !tensor_path)
    return fail(AION_CUDA_UNSUPPORTED, "attention: the page table is read by the f16 tensor-core kernel only (Dk = Dv in {64, 128, 256}, aligned operands)");
  if (s->image.handle) {
    if (!tensor_path) return fail(AION_CUDA_UNSUPPORTED, "attention: the output image is written by the f16 tensor-core kernel only (Dk = Dv in {64, 128, 256}, aligned operands)");
    if (s->image_dtype != AION_CUDA_DTYPE_Q8_0 && s->image_dtype != AION_CUDA_DTYPE_Q4_0)
      return fail(AION_CUDA_INVALID_ARGUMENT, "attention: image dtype %u", s->image_dtype);
    p.image_layout = act_image_layout(B * L, Hq * Dv / QK);
    if (int32_t st = resolve(s->image, act_image_total_bytes(p.image_layout), "attention.image", &p.image)) return st;
    if (reinterpret_cast<uintptr_t>(p.image) & 15) return fail(AION_CUDA_INVALID_ARGUMENT, "attention.image: the image must be 16-byte aligned");
    p.image_dtype = s->image_dtype;
  }
  if (tensor_path) {
    const uint32_t group = p.Hq / p.Hkv;
    p.head_groups = (group + 7) / 8;
    p.col_heads = group < 8 ? group : 8;
    // One query position per CTA (the four warps split the keys) for a single-row step; blocks of
    // positions (each warp owns some, all walk every key) when a request brings several rows, so that
    // K and V are streamed once per block instead of once per row.
    bool block = L > 1 && !(s->flags & AION_CUDA_ATTENTION_ROW_UNITS);
    uint32_t nt = 1;
    if (block) {
      p.pos_per_tile = 8 / p.col_heads;
      if (L > (uint64_t)CONSUMER_WARPS * p.pos_per_tile) nt = 2;
      const uint64_t per_unit = (uint64_t)CONSUMER_WARPS * nt * p.pos_per_tile;
      p.l_blocks = (uint32_t)((L + per_unit - 1) / per_unit);
      // Eight heads already share a row's keys; blocks of eight such rows pay once they cover half the
      // SMs (one kv head: 2048 rows 0.130 ms in blocks against 0.233 ms as rows, 8 x 256 rows 0.061
      // against 0.091; 512 rows, 64 blocks: 0.049 against 0.033).
      if (p.col_heads == 8 && 2 * B * p.l_blocks * Hkv * p.head_groups < (uint64_t)dev->sm_count && !(s->flags & AION_CUDA_ATTENTION_BLOCKS))
        block = false;
    }
    if (!block) {
      nt = 1;
      p.pos_per_tile = 1;
      p.l_blocks = (uint32_t)L;
    }
    const uint64_t units = B * p.l_blocks * Hkv * p.head_groups;
    if (units > 0x7FFFFFFF) return fail(AION_CUDA_UNSUPPORTED, "attention: too many rows");
    const uint32_t cols = 8 * (block ? CONSUMER_WARPS * nt : 1);
    // Split the context until the grid covers the SMs about twice; a split is at least 64 keys.
    // Upper bound of any row's keys: the window span clipped to the cache (or ring) length.
    uint64_t max_keys = T;
    const uint64_t span = (uint64_t)(s->window_chunk ? s->window_chunk : 1) + s->window_left + s->window_right;
    if (s->window_left != AION_CUDA_WINDOW_UNBOUNDED && s->window_right != AION_CUDA_WINDOW_UNBOUNDED && span < max_keys)
      max_keys = span;
    // Choose the number of context splits by a small cost model: CTAs run in waves of one per
    // SM (the ring fills shared memory), a CTA costs its 64-key stages plus a fixed ramp
    // (first TMA round trip, fold, output) of about four stages, two more when it leaves a partial
    // behind (write, fence, ticket), and the merge of a
    // row's partials by one CTA grows with the splits (so they are capped near sqrt(keys / 5),
    // where split work and merge cost balance). The merge's weight per split comes from a decode step of
    // 8 requests at 2048 keys: 16 splits 1.65 ms, 12 1.57, 8 1.56, 4 1.63.
    const uint64_t sms = (uint64_t)dev->sm_count;
    const uint64_t stages_total = (max_keys + KT - 1) / KT;
    uint64_t cap = (uint64_t)std::sqrt(0.2 * (double)max_keys) + 1;
    if (cap > stages_total) cap = stages_total;
    if (cap > 256) cap = 256;
    if (block && cap > 32) cap = 32;   // a block's partial is `cols` rows: keep the merge short
    if (cap < 1) cap = 1;
    uint64_t splits = 1;
    double best = 1e30;
    const double stage_cost = block ? (double)(CONSUMER_WARPS * nt) : 1.0;  // a block's warps walk every key of a stage for their own tiles
    for (uint64_t sp = 1; sp <= cap; sp++) {
      const uint64_t waves = (units * sp + sms - 1) / sms;
      const double per_cta = stage_cost * (double)((stages_total + sp - 1) / sp) + 4.0 + (sp > 1 ? 2.0 + 0.35 * (double)sp * (cols / 8) : 0.0);
      const double cost = (double)waves * per_cta;
      if (cost < best * 0.999) {
        best = cost;
        splits = sp;
      }
    }
    // Blocks of positions: a split leaves a partial of every column of the block behind (64 rows of Dv floats)
    // and a causal prompt's blocks are uneven anyway, so the context is split only while the blocks alone
    // cannot cover the SMs (2048 causal rows of one request: 0.133 ms unsplit against 0.28 ms in four splits).
    if (block) {
      splits = 1;
      if (units < sms) splits = std::min<uint64_t>(cap, sms / units);
      if (splits < 1) splits = 1;
    }
    if (dev->attn_split_override) splits = dev->attn_split_override;
    p.splits = (uint32_t)splits;
    if (splits > 1) {
      const size_t part_bytes = (size_t)units * splits * cols * (Dk + 4) * sizeof(float);
      if (int32_t st = dev->reserve_scratch(part_bytes)) return st;
      if (int32_t st = dev->reserve_tickets(units)) return st;
      p.partial = static_cast<float*>(dev->lane_scratch());
      p.tickets = dev->lane_tickets();
    }
    const bool qf32 = s->q_dtype == AION_CUDA_DTYPE_F32;
    const uint32_t u = (uint32_t)units;
#define AION_ATTN(DD)                                                                                              \
  if (!block) return qf32 ? launch_decode<DD, true, false, 1>(dev, p, u) : launch_decode<DD, false, false, 1>(dev, p, u); \
  if (nt == 1) return qf32 ? launch_decode<DD, true, true, 1>(dev, p, u) : launch_decode<DD, false, true, 1>(dev, p, u);  \
  return qf32 ? launch_decode<DD, true, true, 2>(dev, p, u) : launch_decode<DD, false, true, 2>(dev, p, u);
    switch (Dk) {
      case 64: AION_ATTN(64)
      case 128: AION_ATTN(128)
      default: AION_ATTN(256)
    }
#undef AION_ATTN
  }
  if (Dv > 32 * GEN_MAX_DV_PER_LANE) return fail(AION_CUDA_UNSUPPORTED, "attention: Dv = %llu (any-shape kernel takes <= 1024)", (unsigned long long)Dv);
  const size_t smem = (Dk + GEN_WARPS * (Dv + 2)) * sizeof(float);
  if (smem > 48 * 1024) return fail(AION_CUDA_UNSUPPORTED, "attention: head dimensions %llu / %llu exceed the any-shape kernel", (unsigned long long)Dk, (unsigned long long)Dv);
  p.splits = 1;
  attn_generic_kernel<<<(unsigned)(B * L * Hq), GEN_WARPS * 32, smem, dev->stream>>>(p);
  AION_CUDA_TRY(cudaGetLastError());
  return AION_CUDA_OK;
}

}  // namespace aion
