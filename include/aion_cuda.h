/* aion_cuda.h — C ABI of libaion_cuda, a B200 (sm_100a) device backend for aion's
 * inference hot path: the q4_0 / q8_0 block-quantized `MatMul` / `MatMulNT` steps and
 * the grouped-query `Attention` step.
 *
 * The header sits beside aion's own `include/aion.h`. aion has no C plugin ABI for
 * backends: its seam is three Zig vtables (`Backend`, `Session`, `DeviceMemory`). Every
 * entry point here is what a Zig `CudaBackend` implementing those vtables binds; the
 * comment on each one names the reference interface it stands behind (paths relative
 * to the aion project root).
 *
 * Conventions
 *  - Every function returns an `AionStatus` value (aion `include/aion.h:62-68`):
 *    0 OK, 1 INVALID_ARGUMENT, 2 OUT_OF_MEMORY, 3 UNSUPPORTED, 4 INTERNAL_ERROR.
 *    Nothing throws. The only global state is a per-thread last-error string.
 *  - A device handle (`uint64_t`) is a raw device address; 0 means "none"
 *    (aion `src/aion/runtime/device_memory.zig:14`). An operand is (handle, byte
 *    offset, byte length), exactly what `DeviceStore` resolves a `TensorId` chunk to
 *    (aion `src/aion/runtime/device_store.zig:24-93`).
 *  - Work is enqueued on the device's stream and is asynchronous; `aion_cuda_d2h` and
 *    `aion_cuda_sync` wait for it. One thread drives a device at a time
 *    (aion `src/aion/backend/backend.zig:28-40`: one `execute` per session at a time).
 *  - There is no CPU path. A dtype / layout this library has no kernel for returns
 *    UNSUPPORTED, never a host fallback (aion `src/aion/runtime/executable.zig:355-357`).
 */
#ifndef AION_CUDA_H
#define AION_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define AION_CUDA_API __declspec(dllexport)
#else
#define AION_CUDA_API __attribute__((visibility("default")))
#endif

/* AionStatus values (aion include/aion.h:62-68). */
#define AION_CUDA_OK 0
#define AION_CUDA_INVALID_ARGUMENT 1
#define AION_CUDA_OUT_OF_MEMORY 2
#define AION_CUDA_UNSUPPORTED 3
#define AION_CUDA_INTERNAL_ERROR 4

/* AionDType values (aion include/aion.h:70-77; src/aion/backend/types.zig:29-41). */
#define AION_CUDA_DTYPE_F32 0
#define AION_CUDA_DTYPE_F16 1
#define AION_CUDA_DTYPE_I8 2
#define AION_CUDA_DTYPE_Q4_0 3 /* 18-byte blocks: f16 scale + 16 nibble bytes, 32 weights */
#define AION_CUDA_DTYPE_Q8_0 4 /* 34-byte blocks: f16 scale + 32 int8, 32 weights */
#define AION_CUDA_DTYPE_I32 5

/* QuantBlockOrder values (aion src/aion/backend/types.zig:150-157). */
#define AION_CUDA_ORDER_ROW_MAJOR 0
#define AION_CUDA_ORDER_LANES4 1
#define AION_CUDA_ORDER_LANES8 2
#define AION_CUDA_ORDER_LANES16 3
#define AION_CUDA_ORDER_LANES32 4
#define AION_CUDA_ORDER_LANES32X16 5

/* AttentionWindow "no limit" (aion src/aion/graph/graph.zig:134). */
#define AION_CUDA_WINDOW_UNBOUNDED 0xFFFFFFFFu

typedef struct AionCudaDevice AionCudaDevice;

/* One resolved tensor chunk: `DeviceStore` Chunk{handle, offset, len}
 * (aion src/aion/runtime/device_store.zig:24-37). */
typedef struct AionCudaOperand {
  uint64_t handle; /* device address of the buffer, 0 = absent */
  uint64_t offset; /* byte offset of the tensor inside the buffer */
  uint64_t len;    /* bytes of the tensor available from `offset` */
} AionCudaOperand;

typedef struct AionCudaDeviceInfo {
  char name[128];
  int32_t ordinal;
  int32_t sm_count;
  int32_t cc_major;
  int32_t cc_minor;
  uint64_t total_bytes;
  uint64_t l2_bytes;
} AionCudaDeviceInfo;

/* ---------------------------------------------------------------------------------
 * Backend lifetime. Stands behind `Backend.VTable` {kind, name, caps, deinit,
 * createSession} (aion src/aion/backend/backend.zig:59-72) the way `GpuBackend.init`
 * stands behind it for wgpu (aion src/aion/backend/gpu/backend.zig:85-268).
 * A device owns one stream, its kernel scratch and nothing else.
 * --------------------------------------------------------------------------------- */
AION_CUDA_API int32_t aion_cuda_device_count(int32_t* out_count);
AION_CUDA_API int32_t aion_cuda_device_create(int32_t ordinal, AionCudaDevice** out);
AION_CUDA_API void aion_cuda_device_destroy(AionCudaDevice* dev);
AION_CUDA_API int32_t aion_cuda_device_info(AionCudaDevice* dev, AionCudaDeviceInfo* out);
/* The QuantBlockOrder this backend's NT q8 kernel reads fastest; the compile pass
 * re-lays q8 weights into it (aion src/aion/backend/gpu/backend.zig:86-87,
 * src/aion/graph/target.zig:33-35). Row-major: weights are read in place. */
AION_CUDA_API uint8_t aion_cuda_quant_block_order(AionCudaDevice* dev);
/* Run on a caller-owned CUDA stream (a `cudaStream_t` passed as void*) instead of the
 * device's own; NULL restores the device's stream. No counterpart in the reference:
 * it lets a host that already owns a stream (PyTorch, a graph capture) order work. */
AION_CUDA_API int32_t aion_cuda_set_stream(AionCudaDevice* dev, void* cuda_stream);
AION_CUDA_API void* aion_cuda_get_stream(AionCudaDevice* dev);
/* `Session.retireResources` (aion src/aion/backend/backend.zig:34-36): wait for all
 * submitted work. */
AION_CUDA_API int32_t aion_cuda_sync(AionCudaDevice* dev);
/* Record the steps issued between begin and end into a replayable device program (a
 * CUDA graph) instead of running them, then replay it with one call. The reference's
 * device path likewise records steps into a frame and submits them in bulk
 * (aion src/aion/backend/gpu/backend.zig:551-662, src/aion/backend/gpu/frame.zig); here the
 * recording also removes the per-launch host cost that decode-sized kernels cannot hide.
 * Every buffer a recorded step names must stay allocated while the program is replayed.
 * Steps that would allocate scratch must have run once before recording. */
typedef struct AionCudaProgram AionCudaProgram;
AION_CUDA_API int32_t aion_cuda_record_begin(AionCudaDevice* dev);
/* While recording, steps that do not depend on one another may be issued into different
 * lanes (0..7; lane 0 is the default): lanes become parallel branches of the recorded
 * program and their kernels may overlap on the device. A lane starts after everything
 * recorded on lane 0 before its first use; aion_cuda_record_join orders everything
 * recorded so far before what follows (record_end joins too). The caller owns the
 * dependency analysis, as the reference's compiler owns step order
 * (aion src/aion/graph/program/compiler.zig:1052-1153). Each lane has its own kernel scratch. */
AION_CUDA_API int32_t aion_cuda_record_lane(AionCudaDevice* dev, uint32_t lane);
AION_CUDA_API int32_t aion_cuda_record_join(AionCudaDevice* dev);
AION_CUDA_API int32_t aion_cuda_record_end(AionCudaDevice* dev, AionCudaProgram** out);
AION_CUDA_API int32_t aion_cuda_program_launch(AionCudaDevice* dev, AionCudaProgram* prog);
AION_CUDA_API void aion_cuda_program_destroy(AionCudaDevice* dev, AionCudaProgram* prog);
/* Test hook, no counterpart in the reference. Every wait a kernel of this library makes on a copy
 * barrier is bounded: when it runs out, the kernel records a fault, lets the copies still in flight
 * land and returns, and the next aion_cuda_sync / aion_cuda_d2h reports INTERNAL_ERROR; the device
 * stays usable. While this switch is on, the tiled matmul kernels leave out their first weight copy
 * and poll a few hundred times instead of a million, so that exactly this happens within
 * milliseconds (the result of such a matmul is meaningless). For tests of the fault path. */
AION_CUDA_API int32_t aion_cuda_debug_expire_waits(AionCudaDevice* dev, int32_t on);
/* Per-thread diagnostic text of the last failing call on this thread
 * (aion src/aion/diagnostic.zig:8-44; include/aion.h:117-140). Copies at most `cap`
 * bytes, NUL-terminates when cap > 0, stores the full length in *len when non-NULL. */
AION_CUDA_API int32_t aion_cuda_last_error(char* buf, size_t cap, size_t* len);

/* ---------------------------------------------------------------------------------
 * DeviceMemory.VTable (aion src/aion/runtime/device_memory.zig:40-73).
 * model() is `.discrete`; maxBindingBytes() is unbounded, so no tensor is dim-0
 * chunked (aion src/aion/storage/layout.zig:22-25); importHost is absent.
 * --------------------------------------------------------------------------------- */
AION_CUDA_API int32_t aion_cuda_memory_model(AionCudaDevice* dev); /* 0 = discrete */
AION_CUDA_API uint64_t aion_cuda_max_binding_bytes(AionCudaDevice* dev);
AION_CUDA_API int32_t aion_cuda_alloc(AionCudaDevice* dev, size_t bytes, size_t alignment, uint64_t* out_handle);
AION_CUDA_API int32_t aion_cuda_free(AionCudaDevice* dev, uint64_t handle);
AION_CUDA_API int32_t aion_cuda_h2d(AionCudaDevice* dev, uint64_t handle, size_t dst_offset, const void* src, size_t bytes);
/* Waits for the stream, like the reference's readback (aion src/aion/backend/gpu/backend.zig:296-308). */
AION_CUDA_API int32_t aion_cuda_d2h(AionCudaDevice* dev, void* dst, uint64_t handle, size_t src_offset, size_t bytes);
AION_CUDA_API int32_t aion_cuda_d2d(AionCudaDevice* dev, uint64_t dst, size_t dst_offset, uint64_t src, size_t src_offset, size_t bytes);
AION_CUDA_API int32_t aion_cuda_memset(AionCudaDevice* dev, uint64_t handle, size_t offset, int32_t byte_value, size_t bytes);

/* ---------------------------------------------------------------------------------
 * `MatMul` step: C[m,n] = alpha * A[m,k] @ B[k,n] + beta * C.
 * `StepMatMul` (aion src/aion/runtime/executable.zig:27) executed by `execMatMul` /
 * `gemm2D` (aion src/aion/backend/cpu/exec/matmul.zig:48-108, 243-296) with
 * `MatMulParams` (aion src/aion/backend/types.zig:225-241).
 *   A f32 row-major, row stride lda elements (0 = k); leading dims folded into m.
 *   B q8_0 or q4_0, quant_axis 0: block (kb, j) at byte ((kb*ldb + j) * block_bytes),
 *     ldb in blocks (0 = n); k % 32 == 0.
 *   C f32, row stride ldc elements (0 = n).
 * The activation is quantized to int8 per 32-block exactly as the reference CPU
 * kernels do (aion src/aion/backend/cpu/kernels/matmul_q_i8.zig:187-203) for
 * m < AION_CUDA_GEMM_MIN_M (one launch streams the weights once per AION_CUDA_INT8_GROUP_ROWS rows
 * of A); from there on the tensor-core GEMM runs: it quantizes A to int8 per 32-block in the
 * same way, then multiplies the dequantized activation and the dequantized weights, both
 * rounded to bf16 (results within rel-L2 1e-2 of the int8 arithmetic instead of 1e-3; about
 * 2e-3 in practice). AION_CUDA_MATMUL_FORCE_GEMV keeps the int8 kernel at any m: exact
 * integer dots, at a quarter to a third of the GEMM's speed once m reaches the hundreds.
 * f32 / f16 B return UNSUPPORTED.
 *   a_image (handle 0 = absent): the quantized image of A that the step producing A wrote
 *     (see aion_cuda_act_image_bytes); the kernel then reads it instead of quantizing A.
 *     Ignored by the any-shape kernel, and by a kernel forced through `flags` onto a number of
 *     rows whose image is laid out for the other one: those read A itself.
 * --------------------------------------------------------------------------------- */
#define AION_CUDA_INT8_GROUP_ROWS 64 /* rows of A that share one pass over the weights */
#define AION_CUDA_GEMM_MIN_M 33      /* from this many rows on, the tensor-core GEMM (bf16 operands) runs */

typedef struct AionCudaMatMul {
  AionCudaOperand c, a, b;
  uint32_t b_dtype; /* AION_CUDA_DTYPE_Q8_0 | AION_CUDA_DTYPE_Q4_0 */
  uint32_t flags;   /* AION_CUDA_MATMUL_* */
  uint64_t m, n, k;
  uint64_t lda, ldb, ldc;
  float alpha, beta;
  AionCudaOperand a_image; /* handle 0 = absent */
} AionCudaMatMul;

/* Force a kernel family regardless of m; tests use these the way the reference's GPU
 * tests pin a pipeline (aion src/aion/backend/gpu/test_gpu_backend.zig:403-422). */
#define AION_CUDA_MATMUL_AUTO 0u
#define AION_CUDA_MATMUL_FORCE_GENERIC 1u /* any-shape scalar kernel */
#define AION_CUDA_MATMUL_FORCE_GEMV 2u    /* tiled int8 tensor-core kernel (decode) */
#define AION_CUDA_MATMUL_FORCE_GEMM 4u    /* tcgen05 prefill GEMM */
#define AION_CUDA_MATMUL_ONE_SM 8u        /* the prefill GEMM stays on its one-SM kernel (no pairs of CTAs sharing an MMA) */

AION_CUDA_API int32_t aion_cuda_matmul(AionCudaDevice* dev, const AionCudaMatMul* step);

/* Which kernel aion_cuda_matmul would run for this step and how it would tile it, without
 * running anything. No counterpart in the reference; the tests use it to show that a case
 * reaches the kernel variant it is meant to cover, the way the reference's device tests pin
 * a pipeline (aion src/aion/backend/gpu/test_gpu_backend.zig:403-422). */
#define AION_CUDA_KERNEL_GENERIC 1u /* any-shape scalar kernel */
#define AION_CUDA_KERNEL_INT8 2u    /* tiled int8 tensor-core kernel */
#define AION_CUDA_KERNEL_GEMM 3u    /* tcgen05 prefill GEMM */
typedef struct AionCudaMatMulPlan {
  uint32_t kernel;    /* AION_CUDA_KERNEL_* */
  uint32_t tile_rows; /* rows of A per tile (GEMM: 128 or 256) or per pass over the weights (int8) */
  uint32_t tile_cols; /* output columns per tile */
  uint32_t k_splits;  /* GEMM: CTAs that share one tile's K range (1 = none) */
  uint32_t grid;      /* GEMM: CTAs launched; 0 where the choice is made at launch */
  uint32_t cta_pairs; /* GEMM: 1 = clusters of two CTAs share every MMA (tile_rows is the pair's: 256 or 512) */
  uint32_t reserved[2];
} AionCudaMatMulPlan;
AION_CUDA_API int32_t aion_cuda_matmul_plan(AionCudaDevice* dev, const AionCudaMatMul* step, AionCudaMatMulPlan* out);

/* The quantized-activation image. No counterpart in the reference, whose CPU kernels quantize
 * A at the start of every matmul (aion src/aion/backend/cpu/kernels/matmul_q_i8.zig:237-246):
 * here the step that PRODUCES an activation (RMSNorm, the GELU gate, Attention) can write, next
 * to its f32 output, the int8 codes and block scales of that output in the order the int8
 * matmul kernel reads them, and the matmul that consumes it takes the image through `a_image`.
 * A decode layer then runs without a quantization kernel between its steps. The codes and
 * scales are exactly those the matmul would compute from the f32 values. What an image holds
 * follows the kernel that will read it, which the number of rows decides: below
 * AION_CUDA_GEMM_MIN_M rows the int8 codes and f32 block scales in the int8 kernel's fragment
 * order; from there on the same quantization dequantized and rounded to bf16, row-major, which is
 * what the tensor-core GEMM's own pre-pass produces.
 *   aion_cuda_act_image_bytes: size of the image of an [m, k] activation (k % 32 == 0).
 *   aion_cuda_act_image: writes the image of f32 rows (row stride lda elements, 0 = k) for
 *     weights of `b_dtype` (q4_0 and q8_0 weights read their codes in different orders).
 * A producer writes only the blocks of rows < m and K blocks < k/32: zero the image buffer
 * once (aion_cuda_memset) before its first use with a given shape, the padding must read as zeros. */
AION_CUDA_API int32_t aion_cuda_act_image_bytes(uint64_t m, uint64_t k, uint64_t* out_bytes);
AION_CUDA_API int32_t aion_cuda_act_image(AionCudaDevice* dev, uint32_t b_dtype, const AionCudaOperand* a, uint64_t m, uint64_t k,
                                          uint64_t lda, const AionCudaOperand* image);

/* No counterpart in the reference. The decode `MatMul` step (m <= 8, K-major q8_0 /
 * q4_0 B) for callers that are not allowed to allocate device memory: code running
 * inside someone else's memory pool or allocator callback, inside a region where the
 * CUDA context's allocator must not be entered (a stream capture owned by the caller,
 * a real-time audio or control loop that pre-allocates everything), or in a process
 * whose device memory budget is fixed up front. aion_cuda_matmul grows the device's
 * scratch with cudaMalloc the first time a shape needs it; this entry point never calls
 * cudaMalloc, cudaFree or any allocating routine, on the host or on the device. The
 * kernel's scratch (split-tile partial sums and their arrival counters) is a 2.23 MB
 * array compiled into the library; every GPU that loads the library holds it until the
 * process exits.
 *  - Same arguments, arithmetic and results as aion_cuda_matmul (bitwise when both pick
 *    the same grid; within f32 rounding otherwise).
 *  - Limits: m <= 8; n <= 524288; n and ldb multiples of 8; B 16-byte aligned; k small
 *    enough for one launch (k <= 16384 at m = 1, k <= 4096 at m = 2..8). Anything beyond
 *    returns UNSUPPORTED with a message naming the limit.
 *  - The first call on a device looks up where the array lives on that device
 *    (cudaGetSymbolAddress); make that first call before beginning any stream capture.
 *  - All calls share the one array: two calls whose kernels overlap on the GPU (different
 *    streams, parallel recording lanes, several host threads) race on it. Issue them on
 *    one stream, one at a time. The arrival counters are cleared by every call. */
AION_CUDA_API int32_t aion_cuda_matmul_static_scratch(AionCudaDevice* dev, const AionCudaMatMul* step);

/* ---------------------------------------------------------------------------------
 * `MatMulNT` step: C[m,n] = alpha * sum_k A[m,k] * B[n,k] + beta * C.
 * `StepMatMulNT` (aion src/aion/runtime/executable.zig:217-223) executed by
 * `execMatMulNT` (aion src/aion/backend/cpu/exec/matmul_nt.zig:87-174) over
 * `matmulNtQ8_0(order)` (aion src/aion/backend/cpu/kernels/matmul_nt_q.zig:560-579).
 *   B q8_0 [n,k], quant_axis 1, in `block_order`; a row is k/32 blocks.
 *   c_off / ldc let one weight be issued as several N-chunks of one C, as the
 *   reference's device path does (aion src/aion/backend/gpu/exec/matmul_nt.zig:151-160):
 *   C element (r, j) is at c + (r*ldc + c_off + j) * 4.
 * --------------------------------------------------------------------------------- */
typedef struct AionCudaMatMulNT {
  AionCudaOperand c, a, b;
  uint32_t b_dtype;     /* AION_CUDA_DTYPE_Q8_0 */
  uint32_t block_order; /* AION_CUDA_ORDER_* */
  uint32_t flags;       /* AION_CUDA_MATMUL_* */
  uint32_t reserved;
  uint64_t m, n, k;
  uint64_t lda, ldc, c_off;
  float alpha, beta;
  AionCudaOperand a_image; /* as in AionCudaMatMul; handle 0 = absent */
} AionCudaMatMulNT;

AION_CUDA_API int32_t aion_cuda_matmul_nt(AionCudaDevice* dev, const AionCudaMatMulNT* step);

/* ---------------------------------------------------------------------------------
 * `Attention` step. `StepAttention` (aion src/aion/runtime/executable.zig:105-115)
 * executed by `execAttention` (aion src/aion/backend/cpu/exec/attention.zig:1444-1608).
 *   q   [B, L, Hq, Dk]   f16 or f32
 *   k   [B, T, Hkv, Dk]  f16 or f32       v [B, T, Hkv, Dv] f16 or f32
 *   out [B, L, Hq, Dv]   f32
 *   query_positions i32 [B, L] (absent: position = row l)
 *   kv_lengths      i32 [B]    (absent: T)
 *   window {left, right, chunk} (aion src/aion/graph/graph.zig:130-167), soft cap
 *   (0 = off), rolling: K/V are a ring of T rows addressed t % T and only the last T
 *   logical keys are visible (aion src/aion/backend/cpu/exec/attention.zig:1072-1075).
 * With l_q > 1 (prefill, or several new rows per request) the f16 kernel works on blocks of up to
 * 32 positions that share one pass over K / V, as the reference's block kernel does
 * (aion src/aion/backend/cpu/exec/attention.zig:546-963).
 * Empty key range writes zeros. A negative position / length, or a length beyond T on
 * a non-rolling cache, is detected on the device and reported by the next
 * aion_cuda_sync / aion_cuda_d2h as INVALID_ARGUMENT.
 * --------------------------------------------------------------------------------- */
#define AION_CUDA_ATTENTION_GENERIC 1u   /* flags: take the any-shape f32 kernel */
#define AION_CUDA_ATTENTION_ROW_UNITS 2u /* flags: one CTA per query row even when l_q > 1 (measurement) */
#define AION_CUDA_ATTENTION_BLOCKS 4u    /* flags: blocks of positions whenever l_q > 1 (measurement) */
typedef struct AionCudaAttention {
  AionCudaOperand out, q, k, v;
  AionCudaOperand query_positions; /* handle 0 = absent */
  AionCudaOperand kv_lengths;      /* handle 0 = absent */
  uint32_t q_dtype, k_dtype, v_dtype;
  uint32_t rolling;
  uint64_t batch, l_q, h_q, h_kv, d_k, d_v, t_cap;
  float scale;
  float soft_cap;
  uint32_t window_left, window_right, window_chunk;
  uint32_t flags;
  /* Optional (handle 0 = absent): the quantized image of `out` seen as [B*L, Hq*Dv] rows, for the
   * matmul against weights of image_dtype that consumes it (aion_cuda_act_image_bytes). Written
   * by the tensor-core decode kernel; other shapes return UNSUPPORTED when it is asked for. */
  AionCudaOperand image;
  uint32_t image_dtype;
  /* Paged K / V (handle 0 = absent: K / V are the contiguous [B, T, ...] tensors above). With a
   * page table, k and v are pools [pool_pages, page_tokens, Hkv, D] f16 and key t of request b is
   * row t % page_tokens of page page_table[b][t / page_tokens]; page_table is i32
   * [B, ceil(t_cap / page_tokens)], page_tokens a multiple of 64. Entries past a request's
   * kv_length are not read. Tensor-core kernel only; not with `rolling`. */
  uint32_t page_tokens;
  AionCudaOperand page_table;
  uint64_t pool_pages;
} AionCudaAttention;

AION_CUDA_API int32_t aion_cuda_attention(AionCudaDevice* dev, const AionCudaAttention* step);

/* ---------------------------------------------------------------------------------
 * Decoder glue steps: the ops on either side of the matmul / attention path in a decode
 * program, so a whole token step stays on the device. All f32 unless stated.
 * --------------------------------------------------------------------------------- */

/* `RMSNorm` step with optional residual: `StepRMSNorm` executed by `execRMSNorm`
 * (aion src/aion/backend/cpu/exec/layernorm.zig:41-154).
 *   out[r, :] = (x[r, :] * inv_r) * gamma + beta (+ residual[r, :]),
 *   inv_r = 1 / sqrt(mean(x[r, :]^2) + eps); eps must be finite and > 0.
 * residual.handle == 0: absent. out may alias x or residual.
 * image (handle 0 = absent): also write the quantized image of `out` for a matmul against
 * weights of image_dtype (cols % 32 == 0, cols <= 4096 and 16-byte aligned operands). */
typedef struct AionCudaRMSNorm {
  AionCudaOperand out, x, gamma, beta, residual;
  uint64_t rows, cols;
  float eps;
  uint32_t image_dtype;
  AionCudaOperand image;
} AionCudaRMSNorm;
AION_CUDA_API int32_t aion_cuda_rms_norm(AionCudaDevice* dev, const AionCudaRMSNorm* step);

/* `ElemwiseBinary` step over identical shapes (aion
 * src/aion/backend/cpu/exec/elementwise.zig:18-45): add, mul, and `gate` = gelu(a) * b with
 * the tanh-form GELU over the reference's tanhApprox (aion
 * src/aion/backend/cpu/kernels/gelu.zig:8-14). out may alias a or b. */
#define AION_CUDA_ELEMWISE_ADD 0u
#define AION_CUDA_ELEMWISE_MUL 1u
#define AION_CUDA_ELEMWISE_GATE_GELU 2u
typedef struct AionCudaElemwise {
  AionCudaOperand out, a, b;
  uint64_t count;
  uint32_t op;
  uint32_t reserved;
  /* cols > 0: the operands are [count / cols, cols] matrices with these row strides in
   * elements (0 = cols), e.g. the two halves of a [gate | up] matmul output. */
  uint64_t cols, ld_out, ld_a, ld_b;
  /* Optional (handle 0 = absent): the quantized image of `out` as [count / cols, cols] rows for a
   * matmul against weights of image_dtype; needs cols > 0, cols % 32 == 0 and 16-byte aligned rows. */
  AionCudaOperand image;
  uint32_t image_dtype;
  uint32_t reserved2;
} AionCudaElemwise;
AION_CUDA_API int32_t aion_cuda_elemwise(AionCudaDevice* dev, const AionCudaElemwise* step);

/* `RoPE1D` step: x, out [B, L, H, D] f32, positions i32 [B, L]; pair i of a head is
 * (x[i], x[D/2 + i]); the first floor(proportion * D/2) pairs rotate, the rest copy
 * (aion src/aion/backend/cpu/exec/rope.zig:43-50, src/aion/backend/cpu/kernels/rope.zig:20-97).
 * out may alias x. */
typedef struct AionCudaRoPE {
  AionCudaOperand out, x, positions;
  uint64_t batch, len, heads, head_dim;
  float base_frequency, scale_factor, proportion;
  uint32_t reserved;
} AionCudaRoPE;
AION_CUDA_API int32_t aion_cuda_rope(AionCudaDevice* dev, const AionCudaRoPE* step);

/* `Cast` step, f32 -> f16 (round to nearest even) or f16 -> f32 (aion
 * src/aion/backend/cpu/exec/cast.zig:60-90). */
typedef struct AionCudaCast {
  AionCudaOperand out, in;
  uint64_t count;
  uint32_t from_dtype, to_dtype; /* AION_CUDA_DTYPE_F32 / AION_CUDA_DTYPE_F16 */
} AionCudaCast;
AION_CUDA_API int32_t aion_cuda_cast(AionCudaDevice* dev, const AionCudaCast* step);

/* `SequenceAppend` step: writes new_kv [B, Ln, H, D] into cache [B, T, H, D] (same dtype,
 * f16 or f32) at logical steps end_index[b] + t (aion
 * src/aion/backend/cpu/exec/sequence_append.zig:12-104). rolling = 0: a step >= T is an
 * error; rolling = 1: the step lands in row step % T. A negative index or an out-of-range
 * step is detected on the device, nothing of that request is written, and the next
 * aion_cuda_sync / aion_cuda_d2h reports INVALID_ARGUMENT. */
typedef struct AionCudaSequenceAppend {
  AionCudaOperand cache, new_kv, end_index;
  uint64_t batch, t_cap, heads, head_dim, new_len;
  uint32_t dtype;
  uint32_t rolling;
  /* Paged cache (handle 0 = absent), as in AionCudaAttention: cache is the pool
   * [pool_pages, page_tokens, H, D], page_table i32 [B, ceil(t_cap / page_tokens)]; a page number
   * outside the pool is reported like a bad index. */
  AionCudaOperand page_table;
  uint64_t page_tokens, pool_pages;
} AionCudaSequenceAppend;
AION_CUDA_API int32_t aion_cuda_sequence_append(AionCudaDevice* dev, const AionCudaSequenceAppend* step);

/* `GatherRows` step from a q8_0 [table_rows, d] table (quant_axis 1, any block order) to
 * f32 [count, d] (aion src/aion/backend/cpu/exec/gather.zig:22-28, 57-87). Indices follow
 * the ONNX rule: [-table_rows, table_rows - 1], negative counts from the end; anything else
 * is reported like SequenceAppend's range error. */
typedef struct AionCudaGatherRows {
  AionCudaOperand out, table, indices;
  uint64_t table_rows, d, count;
  uint32_t block_order;
  uint32_t reserved;
} AionCudaGatherRows;
AION_CUDA_API int32_t aion_cuda_gather_rows(AionCudaDevice* dev, const AionCudaGatherRows* step);

/* `ArgMax` step over the last axis of f32 [outer, n] -> i32 [outer]; the first maximum
 * wins, a NaN never beats a number, a row whose first element is NaN answers 0 (aion
 * src/aion/backend/cpu/exec/argmax.zig:56-82). */
typedef struct AionCudaArgMax {
  AionCudaOperand out, in;
  uint64_t outer, n;
} AionCudaArgMax;
AION_CUDA_API int32_t aion_cuda_argmax(AionCudaDevice* dev, const AionCudaArgMax* step);

/* ---------------------------------------------------------------------------------
 * Fused decoder steps. No counterpart step in the reference: each is the exact composition
 * of reference steps that always follow one another in a decode program, issued as one
 * kernel so a token step is fewer, fuller launches (the reference fuses in the same spirit:
 * RMSNorm + residual, gate). Results equal the unfused sequences bit for bit (RoPE, cast,
 * append) or to f32 summation order (norms).
 * --------------------------------------------------------------------------------- */

/* RMSNorm(+residual) followed by the RMSNorm of its result:
 *   out1 = rms(x; gamma1, beta1, eps1) + residual     (residual.handle == 0: absent)
 *   out2 = rms(out1; gamma2, beta2, eps2)
 * out1 may alias x or residual. */
typedef struct AionCudaRMSNormPair {
  AionCudaOperand out1, out2, x, gamma1, beta1, residual, gamma2, beta2;
  uint64_t rows, cols;
  float eps1, eps2;
  AionCudaOperand image; /* optional: the quantized image of out2, as in AionCudaRMSNorm */
  uint32_t image_dtype;
  uint32_t reserved;
} AionCudaRMSNormPair;
AION_CUDA_API int32_t aion_cuda_rms_norm_pair(AionCudaDevice* dev, const AionCudaRMSNormPair* step);

/* RoPE1D of q and k, Cast f32 -> f16 of k and v, SequenceAppend of both into their caches.
 * qkv is one f32 row of ld_qkv elements per (b, l): q (h_q * head_dim) then k then v
 * (h_kv * head_dim each) — the output of one matmul against [Wq | Wk | Wv].
 *   q_out [B, L, h_q, head_dim] f32 = RoPE(q)
 *   k_cache / v_cache [B, t_cap, h_kv, head_dim] f16: rows end_index[b] + l receive
 *   f16(RoPE(k)) and f16(v); range rules and rolling as in aion_cuda_sequence_append. */
typedef struct AionCudaRopeKVAppend {
  AionCudaOperand q_out, qkv, positions, end_index, k_cache, v_cache;
  uint64_t batch, len, h_q, h_kv, head_dim, ld_qkv, t_cap;
  float base_frequency, scale_factor, proportion;
  uint32_t rolling;
} AionCudaRopeKVAppend;
AION_CUDA_API int32_t aion_cuda_rope_kv_append(AionCudaDevice* dev, const AionCudaRopeKVAppend* step);

/* ---------------------------------------------------------------------------------
 * Block quantizer on the device. `quantizeBlocks` (aion src/aion/storage/quantize.zig:31-103)
 * for q8_0; for q4_0 the reference's only q4 packer (aion
 * src/aion/backend/cpu/test_cpu_kernels.zig:490-523) under the same placement rule.
 * `values` f32 row-major of `shape[rank]`; blocks along `quant_axis`; `out` row-major
 * over the block-space shape. Byte-exact with the reference.
 * --------------------------------------------------------------------------------- */
AION_CUDA_API int32_t aion_cuda_quantize(AionCudaDevice* dev, uint32_t dtype, const AionCudaOperand* values,
                                         const uint64_t* shape, uint32_t rank, uint32_t quant_axis,
                                         const AionCudaOperand* out);
/* w = f32(q) * f32(f16 scale) for `nblocks` consecutive blocks, 32 f32 per block
 * (aion src/aion/backend/cpu/kernels/matmul_q_i8.zig:847-862, nibble decode :362-369).
 * Bit-exact in f32. */
AION_CUDA_API int32_t aion_cuda_dequantize(AionCudaDevice* dev, uint32_t dtype, const AionCudaOperand* blocks,
                                           uint64_t nblocks, const AionCudaOperand* out);
/* Re-lay a row-major q8_0 [n,k] tensor into `order` (inverse != 0: back to row-major).
 * `QuantBlockOrder.storeBlock/loadBlock` (aion src/aion/backend/types.zig:206-222) as
 * driven by the weight_layout pass (aion src/aion/graph/opt/weight_layout.zig:243-314),
 * which creates the derived tensor directly on the device (:270-275). */
AION_CUDA_API int32_t aion_cuda_relayout_q8(AionCudaDevice* dev, uint32_t order, uint32_t inverse, uint64_t n,
                                            uint64_t k, const AionCudaOperand* src, const AionCudaOperand* dst);
/* ---------------------------------------------------------------------------------
 * Column-split layers over the GPUs of one node (one process per GPU). No counterpart in
 * the reference, which runs on one device. Rank r holds the columns [n0_r, n1_r) of a K-major
 * weight and computes y[:, n0_r:n1_r]; with a fan-out the int8 matmul kernel (m <= 32) stores
 * every output value into the C of every other rank as well (plain peer stores over NVLink from
 * the kernel's epilogue) and, when its last CTA is done, writes its arrival into every rank's
 * flag array. aion_cuda_peer_wait, next in the stream, waits (bounded) until all ranks have
 * arrived: y is then complete on this GPU without a collective call.
 *   Buffers another rank writes (C, flags) come from aion_cuda_alloc, are exported with
 *   aion_cuda_ipc_export, and opened in the other processes with aion_cuda_ipc_import.
 *   flags: u32[8] per rank, zero-filled once; state: u32[2] per rank (epoch, CTA counter),
 *   zero-filled once. Every rank must run the same sequence of fan-out matmuls and waits.
 *   A rank may run one step ahead of a peer, so consecutive steps alternate between two C
 *   buffers (a peer still reading step s is never overwritten by step s + 1).
 *   A wait that runs out (a rank that never arrives) is reported by the next
 *   aion_cuda_sync / aion_cuda_d2h as EXECUTION_FAILED; the device stays usable.
 * --------------------------------------------------------------------------------- */
typedef struct AionCudaPeerFanout {
  uint32_t world, rank;
  AionCudaOperand c[8];     /* C of every rank, laid out like the step's own c (entry `rank` is ignored) */
  AionCudaOperand flags[8]; /* u32[8] arrival words of every rank (entry `rank`: this rank's own) */
  AionCudaOperand state;    /* this rank's u32[2] */
} AionCudaPeerFanout;
AION_CUDA_API int32_t aion_cuda_matmul_peers(AionCudaDevice* dev, const AionCudaMatMul* step, const AionCudaPeerFanout* fan);
/* poll_limit: polls (about 0.1 us apart) before the wait gives up; 0 = the default (about a second). */
AION_CUDA_API int32_t aion_cuda_peer_wait(AionCudaDevice* dev, const AionCudaOperand* flags, const AionCudaOperand* state,
                                          uint32_t world, uint32_t poll_limit);
/* 64 opaque bytes that name an aion_cuda_alloc allocation to the other processes of the node, and back. */
AION_CUDA_API int32_t aion_cuda_ipc_export(AionCudaDevice* dev, uint64_t handle, uint8_t out[64]);
AION_CUDA_API int32_t aion_cuda_ipc_import(AionCudaDevice* dev, const uint8_t in[64], uint64_t* handle);
AION_CUDA_API int32_t aion_cuda_ipc_close(AionCudaDevice* dev, uint64_t handle);

/* The derived weight of this backend: a q8_0 [n,k] tensor in `order` re-laid as K-major
 * [k/32][n] blocks, the layout `aion_cuda_matmul` streams. Both layouts quantize along K, so
 * this is a permutation of 34-byte blocks and C = A . B^T of the `MatMulNT` step equals
 * `MatMul` over the derived tensor bit for bit. A binder calls it once per weight from its
 * weight-layout pass (aion src/aion/graph/opt/weight_layout.zig:243-314 memoises the derived
 * tensor per model) and then issues the step as `aion_cuda_matmul`; `aion_cuda_matmul_nt`
 * stays available for weights that were not derived. */
AION_CUDA_API int32_t aion_cuda_derive_kmajor_q8(AionCudaDevice* dev, uint32_t order, uint64_t n, uint64_t k,
                                                 const AionCudaOperand* src, const AionCudaOperand* dst);

#ifdef __cplusplus
}
#endif
#endif /* AION_CUDA_H */
