// Step entry points: argument checks and routing to a kernel family.
#include <cmath>
#include <cstdlib>

#include "act_image.cuh"
#include <cstring>

#include "common.cuh"

using namespace aion;

namespace aion {
// Rows of A from which the step is a dense contraction for the tensor cores (bf16 operands);
// below, the int8 kernel streams the weights with the reference CPU kernels' arithmetic.
uint64_t gemm_min_m() {
  static const uint64_t v = [] {
    const char* e = std::getenv("AION_CUDA_GEMM_MIN_M");  // tuning: where the int8 kernel hands over to the bf16 GEMM
    const long x = e ? std::atol(e) : 0;
    return x > 0 ? (uint64_t)x : (uint64_t)AION_CUDA_GEMM_MIN_M;
  }();
  return v;
}

}  // namespace aion

namespace {

// Bytes a K-major quantized B of `kblocks` block-rows must hold
// (src/aion/backend/cpu/kernels/matvec_q.zig:85).
uint64_t kmajor_bytes(uint64_t kblocks, uint64_t ldb, uint64_t n, size_t bb) {
  return kblocks == 0 ? 0 : ((kblocks - 1) * ldb + n) * bb;
}

int32_t route(AionCudaDevice* dev, const MatMulArgs& g, uint32_t flags, const char* what) {
  if (flags & AION_CUDA_MATMUL_FORCE_GENERIC) return matmul_generic(dev, g);
  if (flags & AION_CUDA_MATMUL_FORCE_GEMV) {
    const int32_t st = gemv_mma(dev, g, false);
    if (st == AION_CUDA_UNSUPPORTED) return fail(st, "%s: the tiled int8 kernel does not read this shape or alignment", what);
    return st;
  }
  if (flags & AION_CUDA_MATMUL_FORCE_GEMM) {
    const int32_t st = gemm_tcgen05(dev, g);
    if (st == AION_CUDA_UNSUPPORTED) return fail(st, "%s: the tensor-core GEMM does not read this shape or alignment", what);
    return st;
  }
  // Either family falls back to the any-shape kernel (still on the device) when the tiled
  // kernel cannot read the operands.
  if (g.m < gemm_min_m()) {
    const int32_t st = gemv_mma(dev, g, false);
    if (st != AION_CUDA_UNSUPPORTED) return st;
  } else {
    const int32_t st = gemm_tcgen05(dev, g);
    if (st != AION_CUDA_UNSUPPORTED) return st;
  }
  return matmul_generic(dev, g);
}

// Resolves the optional activation image of a matmul step.
int32_t resolve_image(const AionCudaOperand& op, uint64_t m, uint64_t k, const char* name, const uint8_t** out) {
  *out = nullptr;
  if (op.handle == 0) return AION_CUDA_OK;
  if (m * k >= (1ull << 31)) return fail(AION_CUDA_UNSUPPORTED, "%s: shape beyond what an activation image holds", name);
  const size_t need = act_image_total_bytes(act_image_layout(m, k / QK));
  if (int32_t st = resolve(op, need, name, out)) return st;
  if (reinterpret_cast<uintptr_t>(*out) & 15) return fail(AION_CUDA_INVALID_ARGUMENT, "%s: the image must be 16-byte aligned", name);
  return AION_CUDA_OK;
}

// Fills MatMulArgs from a `MatMul` step after checking it. *empty: nothing to do.
int32_t matmul_args(const AionCudaMatMul* s, MatMulArgs* out, bool* empty) {
  *empty = false;
  if (s->b_dtype == AION_CUDA_DTYPE_F32 || s->b_dtype == AION_CUDA_DTYPE_F16)
    return fail(AION_CUDA_UNSUPPORTED, "matmul: float B is outside this backend (quantized q8_0 / q4_0 only)");
  if (s->b_dtype != AION_CUDA_DTYPE_Q8_0 && s->b_dtype != AION_CUDA_DTYPE_Q4_0)
    return fail(AION_CUDA_INVALID_ARGUMENT, "matmul: B dtype %u", s->b_dtype);
  // Quantized B: K must be whole blocks (src/aion/graph/program/compiler.zig:189-239).
  if (s->k % QK != 0) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul: k = %llu is not a multiple of 32", (unsigned long long)s->k);
  if (s->m == 0 || s->n == 0) {
    *empty = true;
    return AION_CUDA_OK;
  }
  MatMulArgs g{};
  g.dtype = s->b_dtype;
  g.nt = false;
  g.order = AION_CUDA_ORDER_ROW_MAJOR;
  g.m = s->m;
  g.n = s->n;
  g.k = s->k;
  g.lda = s->lda ? s->lda : s->k;
  g.ldb = s->ldb ? s->ldb : s->n;
  g.ldc = s->ldc ? s->ldc : s->n;
  g.alpha = s->alpha;
  g.one_sm = (s->flags & AION_CUDA_MATMUL_ONE_SM) != 0;
  g.beta = s->beta;
  if (g.lda < g.k || g.ldb < g.n || g.ldc < g.n) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul: a leading dimension is shorter than its row");
  const size_t bb = block_bytes_of(g.dtype);
  if (int32_t st = resolve(s->a, ((g.m - 1) * g.lda + g.k) * sizeof(float), "matmul.a", &g.a)) return st;
  if (int32_t st = resolve(s->c, ((g.m - 1) * g.ldc + g.n) * sizeof(float), "matmul.c", &g.c)) return st;
  if (g.k == 0) {
    // An empty contraction still applies beta; the any-shape kernel handles it.
    g.b = nullptr;
  } else if (int32_t st = resolve(s->b, kmajor_bytes(g.k / QK, g.ldb, g.n, bb), "matmul.b", &g.b)) {
    return st;
  }
  if ((reinterpret_cast<uintptr_t>(g.a) & 3) || (reinterpret_cast<uintptr_t>(g.c) & 3) || (reinterpret_cast<uintptr_t>(g.b) & 1))
    return fail(AION_CUDA_INVALID_ARGUMENT, "matmul: A and C must be 4-byte aligned, B 2-byte aligned");
  if (g.k > 0)
    if (int32_t st = resolve_image(s->a_image, g.m, g.k, "matmul.a_image", &g.a_image)) return st;
  *out = g;
  return AION_CUDA_OK;
}

}  // namespace

extern "C" {

int32_t aion_cuda_matmul(AionCudaDevice* dev, const AionCudaMatMul* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul: null argument");
  MatMulArgs g{};
  bool empty = false;
  if (int32_t st = matmul_args(s, &g, &empty)) return st;
  if (empty) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  return route(dev, g, s->flags, "matmul");
}

int32_t aion_cuda_matmul_peers(AionCudaDevice* dev, const AionCudaMatMul* s, const AionCudaPeerFanout* fan) {
  if (!dev || !s || !fan) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_peers: null argument");
  if (fan->world < 1 || fan->world > 8 || fan->rank >= fan->world)
    return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_peers: rank %u of %u (at most 8 ranks)", fan->rank, fan->world);
  MatMulArgs g{};
  bool empty = false;
  if (int32_t st = matmul_args(s, &g, &empty)) return st;
  if (empty) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_peers: an empty matmul has nothing to announce");
  if (g.m > 32) return fail(AION_CUDA_UNSUPPORTED, "matmul_peers: m = %llu (the fan-out is part of the int8 kernel, m <= 32)", (unsigned long long)g.m);
  PeerFanout pf{};
  pf.world = fan->world;
  pf.rank = fan->rank;
  const uint64_t c_bytes = ((g.m - 1) * g.ldc + g.n) * sizeof(float);
  for (uint32_t r = 0; r < fan->world; r++) {
    if (int32_t st = resolve(fan->flags[r], 8 * sizeof(uint32_t), "matmul_peers.flags", &pf.flags[r])) return st;
    if (r == fan->rank) continue;
    if (int32_t st = resolve(fan->c[r], c_bytes, "matmul_peers.c", &pf.c[pf.count])) return st;
    if (reinterpret_cast<uintptr_t>(pf.c[pf.count]) & 7) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_peers.c: 8-byte alignment");
    pf.count++;
  }
  if (int32_t st = resolve(fan->state, 2 * sizeof(uint32_t), "matmul_peers.state", &pf.state)) return st;
  g.peers = &pf;
  if (int32_t st = dev->make_current()) return st;
  const int32_t st = gemv_mma(dev, g, false);
  if (st == AION_CUDA_UNSUPPORTED) return fail(AION_CUDA_UNSUPPORTED, "matmul_peers: this shape or alignment is outside the tiled int8 kernel");
  return st;
}

int32_t aion_cuda_peer_wait(AionCudaDevice* dev, const AionCudaOperand* flags, const AionCudaOperand* state, uint32_t world,
                            uint32_t poll_limit) {
  if (!dev || !flags || !state) return fail(AION_CUDA_INVALID_ARGUMENT, "peer_wait: null argument");
  if (world < 1 || world > 8) return fail(AION_CUDA_INVALID_ARGUMENT, "peer_wait: %u ranks", world);
  const uint32_t* f;
  uint32_t* st_ptr;
  if (int32_t st = resolve(*flags, 8 * sizeof(uint32_t), "peer_wait.flags", &f)) return st;
  if (int32_t st = resolve(*state, 2 * sizeof(uint32_t), "peer_wait.state", &st_ptr)) return st;
  if (int32_t st = dev->make_current()) return st;
  return peer_wait_launch(dev, f, st_ptr, world, poll_limit ? poll_limit : (1u << 23));
}

int32_t aion_cuda_ipc_export(AionCudaDevice* dev, uint64_t handle, uint8_t out[64]) {
  if (!dev || !handle || !out) return fail(AION_CUDA_INVALID_ARGUMENT, "ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (int32_t st = dev->make_current()) return st;
  cudaIpcMemHandle_t h;
  AION_CUDA_TRY(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(handle))));
  memcpy(out, &h, 64);
  return AION_CUDA_OK;
}

int32_t aion_cuda_ipc_import(AionCudaDevice* dev, const uint8_t in[64], uint64_t* handle) {
  if (!dev || !in || !handle) return fail(AION_CUDA_INVALID_ARGUMENT, "ipc_import: null argument");
  if (int32_t st = dev->make_current()) return st;
  cudaIpcMemHandle_t h;
  memcpy(&h, in, 64);
  void* p = nullptr;
  AION_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *handle = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(p));
  return AION_CUDA_OK;
}

int32_t aion_cuda_ipc_close(AionCudaDevice* dev, uint64_t handle) {
  if (!dev || !handle) return fail(AION_CUDA_INVALID_ARGUMENT, "ipc_close: null argument");
  if (int32_t st = dev->make_current()) return st;
  AION_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  AION_CUDA_TRY(cudaIpcCloseMemHandle(reinterpret_cast<void*>(static_cast<uintptr_t>(handle))));
  return AION_CUDA_OK;
}

int32_t aion_cuda_matmul_plan(AionCudaDevice* dev, const AionCudaMatMul* s, AionCudaMatMulPlan* out) {
  if (!dev || !s || !out) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_plan: null argument");
  *out = AionCudaMatMulPlan{};
  MatMulArgs g{};
  bool empty = false;
  if (int32_t st = matmul_args(s, &g, &empty)) return st;
  if (empty) return AION_CUDA_OK;
  const bool want_gemm = (s->flags & AION_CUDA_MATMUL_FORCE_GEMM) || (!(s->flags & (AION_CUDA_MATMUL_FORCE_GEMV | AION_CUDA_MATMUL_FORCE_GENERIC)) && g.m >= gemm_min_m());
  GemmPlan gp{};
  if (s->flags & AION_CUDA_MATMUL_FORCE_GENERIC) {
    out->kernel = AION_CUDA_KERNEL_GENERIC;
  } else if (want_gemm && gemm_tcgen05_plan(dev, g, &gp)) {
    out->kernel = AION_CUDA_KERNEL_GEMM;
    out->tile_rows = gp.tile_rows;
    out->tile_cols = 256;
    out->k_splits = gp.splits;
    out->grid = gp.grid;
    out->cta_pairs = gp.pair ? 1u : 0u;
  } else if (!want_gemm && g.k > 0 && gemv_mma(dev, g, true) == AION_CUDA_OK) {
    out->kernel = AION_CUDA_KERNEL_INT8;
    out->tile_rows = g.m <= 8 ? 8u : (g.m <= 16 ? 16u : (g.m <= 32 ? 32u : (uint32_t)AION_CUDA_INT8_GROUP_ROWS));
    out->tile_cols = g.m <= 16 ? 64u : 128u;
    out->k_splits = 1;
  } else {
    out->kernel = AION_CUDA_KERNEL_GENERIC;
  }
  return AION_CUDA_OK;
}

int32_t aion_cuda_act_image_bytes(uint64_t m, uint64_t k, uint64_t* out_bytes) {
  if (!out_bytes) return fail(AION_CUDA_INVALID_ARGUMENT, "act_image_bytes: null out");
  if (k % QK != 0) return fail(AION_CUDA_INVALID_ARGUMENT, "act_image_bytes: k = %llu is not a multiple of 32", (unsigned long long)k);
  if (m > (1ull << 22) || k > (1ull << 26) || m * k >= (1ull << 31)) return fail(AION_CUDA_UNSUPPORTED, "act_image_bytes: shape beyond what the matmul kernels index");
  *out_bytes = m == 0 ? 0 : act_image_total_bytes(act_image_layout(m, k / QK));
  return AION_CUDA_OK;
}

int32_t aion_cuda_act_image(AionCudaDevice* dev, uint32_t b_dtype, const AionCudaOperand* a, uint64_t m, uint64_t k, uint64_t lda,
                            const AionCudaOperand* image) {
  if (!dev || !a || !image) return fail(AION_CUDA_INVALID_ARGUMENT, "act_image: null argument");
  if (b_dtype != AION_CUDA_DTYPE_Q8_0 && b_dtype != AION_CUDA_DTYPE_Q4_0) return fail(AION_CUDA_INVALID_ARGUMENT, "act_image: weight dtype %u", b_dtype);
  if (k % QK != 0 || k == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "act_image: k = %llu must be a positive multiple of 32", (unsigned long long)k);
  if (m == 0) return AION_CUDA_OK;
  if (m > (1ull << 22) || k > (1ull << 26) || m * k >= (1ull << 31)) return fail(AION_CUDA_UNSUPPORTED, "act_image: shape beyond what the matmul kernels index");
  const uint64_t ld = lda ? lda : k;
  if (ld < k) return fail(AION_CUDA_INVALID_ARGUMENT, "act_image: lda is shorter than a row");
  const float* ap;
  const uint8_t* ip;
  if (int32_t st = resolve(*a, ((m - 1) * ld + k) * sizeof(float), "act_image.a", &ap)) return st;
  if (int32_t st = resolve_image(*image, m, k, "act_image.image", &ip)) return st;
  if (int32_t st = dev->make_current()) return st;
  return act_image_from_f32(dev, b_dtype, ap, m, k, ld, const_cast<uint8_t*>(ip));
}

// The `MatMul` step for a caller that cannot allocate: same arguments and results as
// aion_cuda_matmul for decode-sized m, with the kernel's scratch taken from an array
// built into the library. See the header for who needs it and its limits.
int32_t aion_cuda_matmul_static_scratch(AionCudaDevice* dev, const AionCudaMatMul* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_static_scratch: null argument");
  if (s->b_dtype != AION_CUDA_DTYPE_Q8_0 && s->b_dtype != AION_CUDA_DTYPE_Q4_0)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: B must be q8_0 or q4_0");
  if (s->k % QK != 0) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_static_scratch: k = %llu is not a multiple of 32", (unsigned long long)s->k);
  if (s->m == 0 || s->n == 0) return AION_CUDA_OK;
  MatMulArgs g{};
  g.dtype = s->b_dtype;
  g.nt = false;
  g.order = AION_CUDA_ORDER_ROW_MAJOR;
  g.m = s->m;
  g.n = s->n;
  g.k = s->k;
  g.lda = s->lda ? s->lda : s->k;
  g.ldb = s->ldb ? s->ldb : s->n;
  g.ldc = s->ldc ? s->ldc : s->n;
  g.alpha = s->alpha;
  g.beta = s->beta;
  if (g.lda < g.k || g.ldb < g.n || g.ldc < g.n) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_static_scratch: a leading dimension is shorter than its row");
  if (g.k == 0) return fail(AION_CUDA_UNSUPPORTED, "matmul_static_scratch: k = 0");
  if (int32_t st = resolve(s->a, ((g.m - 1) * g.lda + g.k) * sizeof(float), "matmul_static_scratch.a", &g.a)) return st;
  if (int32_t st = resolve(s->c, ((g.m - 1) * g.ldc + g.n) * sizeof(float), "matmul_static_scratch.c", &g.c)) return st;
  if (int32_t st = resolve(s->b, kmajor_bytes(g.k / QK, g.ldb, g.n, block_bytes_of(g.dtype)), "matmul_static_scratch.b", &g.b)) return st;
  if ((reinterpret_cast<uintptr_t>(g.a) & 3) || (reinterpret_cast<uintptr_t>(g.c) & 3))
    return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_static_scratch: A and C must be 4-byte aligned");
  if (int32_t st = dev->make_current()) return st;
  return gemv_mma_static_scratch(dev, g);
}

int32_t aion_cuda_matmul_nt(AionCudaDevice* dev, const AionCudaMatMulNT* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_nt: null argument");
  if (s->b_dtype == AION_CUDA_DTYPE_F32)
    return fail(AION_CUDA_UNSUPPORTED, "matmul_nt: f32 B is outside this backend (q8_0 only)");
  // The NT lowering exists for q8_0 and f32 only (src/aion/graph/program/matmul_rows.zig:89-100).
  if (s->b_dtype != AION_CUDA_DTYPE_Q8_0) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_nt: B dtype %u", s->b_dtype);
  if (s->block_order > AION_CUDA_ORDER_LANES32X16) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_nt: block order %u", s->block_order);
  if (s->k % QK != 0) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_nt: k = %llu is not a multiple of 32", (unsigned long long)s->k);
  static const int group_of[6] = {1, 4, 8, 16, 32, 32};
  if (s->n % group_of[s->block_order] != 0)
    return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_nt: n = %llu does not fill groups of %d rows", (unsigned long long)s->n,
                group_of[s->block_order]);
  if (s->m == 0 || s->n == 0) return AION_CUDA_OK;
  MatMulArgs g{};
  g.dtype = s->b_dtype;
  g.nt = true;
  g.one_sm = (s->flags & AION_CUDA_MATMUL_ONE_SM) != 0;
  g.order = s->block_order;
  g.m = s->m;
  g.n = s->n;
  g.k = s->k;
  g.lda = s->lda ? s->lda : s->k;
  g.ldb = s->k / QK;
  g.ldc = s->ldc ? s->ldc : s->n;
  g.alpha = s->alpha;
  g.beta = s->beta;
  if (g.lda < g.k || g.ldc < s->c_off + g.n) return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_nt: a leading dimension is shorter than its row");
  if (int32_t st = resolve(s->a, ((g.m - 1) * g.lda + g.k) * sizeof(float), "matmul_nt.a", &g.a)) return st;
  float* c0;
  if (int32_t st = resolve(s->c, ((g.m - 1) * g.ldc + s->c_off + g.n) * sizeof(float), "matmul_nt.c", &c0)) return st;
  g.c = c0 + s->c_off;
  if (g.k == 0) g.b = nullptr;
  else if (int32_t st = resolve(s->b, g.n * (g.k / QK) * Q8_BYTES, "matmul_nt.b", &g.b)) return st;
  if ((reinterpret_cast<uintptr_t>(g.a) & 3) || (reinterpret_cast<uintptr_t>(g.c) & 3) || (reinterpret_cast<uintptr_t>(g.b) & 1))
    return fail(AION_CUDA_INVALID_ARGUMENT, "matmul_nt: A and C must be 4-byte aligned, B 2-byte aligned");
  if (g.k > 0)
    if (int32_t st = resolve_image(s->a_image, g.m, g.k, "matmul_nt.a_image", &g.a_image)) return st;
  if (int32_t st = dev->make_current()) return st;
  return route(dev, g, s->flags, "matmul_nt");
}

int32_t aion_cuda_attention(AionCudaDevice* dev, const AionCudaAttention* s) {
  if (!dev || !s) return fail(AION_CUDA_INVALID_ARGUMENT, "attention: null argument");
  // src/aion/backend/cpu/exec/attention.zig:1452-1500.
  if (!(s->scale > 0.0f) || !std::isfinite(s->scale)) return fail(AION_CUDA_INVALID_ARGUMENT, "attention: scale must be finite and positive");
  if (!std::isfinite(s->soft_cap) || s->soft_cap < 0.0f) return fail(AION_CUDA_INVALID_ARGUMENT, "attention: soft cap must be finite and >= 0");
  for (uint32_t dt : {s->q_dtype, s->k_dtype, s->v_dtype})
    if (dt != AION_CUDA_DTYPE_F16 && dt != AION_CUDA_DTYPE_F32) return fail(AION_CUDA_INVALID_ARGUMENT, "attention: q/k/v dtype %u", dt);
  if (s->h_kv == 0 || s->h_q == 0 || s->h_q % s->h_kv != 0)
    return fail(AION_CUDA_INVALID_ARGUMENT, "attention: %llu query heads over %llu kv heads", (unsigned long long)s->h_q,
                (unsigned long long)s->h_kv);
  if (s->t_cap == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "attention: empty K/V");
  if (s->batch * s->l_q * s->h_q == 0) return AION_CUDA_OK;
  if (s->d_k == 0 || s->d_v == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "attention: zero head dimension");
  if (int32_t st = dev->make_current()) return st;
  return attention_launch(dev, s);
}

}  // extern "C"
