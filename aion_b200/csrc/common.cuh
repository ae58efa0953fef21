// Shared declarations of libaion_cuda: the device object, status plumbing and the
// block-format helpers every kernel file uses.
#pragma once

#include <cstdlib>

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <mutex>
#include <set>
#include <utility>
#include <cstdio>

#include "../../include/aion_cuda.h"

namespace aion {

constexpr int QK = 32;          // weights per quantized block
constexpr int Q8_BYTES = 34;    // f16 scale + 32 int8
constexpr int Q4_BYTES = 18;    // f16 scale + 16 nibble bytes

// Codes a kernel can leave in the device status word; the host maps them to AionStatus.
enum DeviceFault : int {
  FAULT_NONE = 0,
  FAULT_INVALID_ARGUMENT = 1,  // a negative position / length, a length beyond the cache
  FAULT_WAIT_EXPIRED = 2,      // a bounded wait on an mbarrier gave up
  FAULT_NONFINITE = 3,         // softmax denominator not finite and positive
};

void set_error(const char* fmt, ...);
int32_t fail(int32_t status, const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what);

#define AION_CUDA_TRY(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::aion::cuda_fail(_e, #expr); \
  } while (0)

inline __host__ __device__ size_t block_bytes_of(uint32_t dtype) {
  return dtype == AION_CUDA_DTYPE_Q8_0 ? Q8_BYTES : Q4_BYTES;
}

inline uint64_t ceil_div(uint64_t a, uint64_t b) { return (a + b - 1) / b; }

}  // namespace aion

// The device object behind the C handle.
struct AionCudaDevice {
  int ordinal = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  cudaDeviceProp prop{};
  int sm_count = 0;
  // Device status word kernels write a DeviceFault into, and its pinned host mirror.
  int* fault_dev = nullptr;
  int* fault_host = nullptr;
  // While recording, independent steps may be issued into parallel lanes (branches of the
  // recorded graph). Lane 0 is the device's stream; `stream` is always the lane in use.
  static constexpr int LANES = 8;
  cudaStream_t main_stream = nullptr;       // `stream` outside lanes
  cudaStream_t lane_streams[LANES] = {};    // [0] unused
  cudaEvent_t lane_events[LANES] = {};
  cudaEvent_t fork_event = nullptr;
  bool lane_forked[LANES] = {};
  int cur_lane = 0;
  // Kernel scratch (quantized activations of the any-shape path, split partials);
  // grown on demand, never shrunk, freed with the device. Every scratch buffer holds one
  // slice per lane (`*_bytes` / `*_cap` are the size of one slice), so steps recorded in
  // different lanes never share scratch.
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // Tuning override (environment AION_CUDA_GEMV_SPLIT): K-split of the tiled GEMV, 0 = automatic.
  uint32_t gemv_split_override = 0;
  // Same for the decode attention's context split (AION_CUDA_ATTN_SPLIT), 0 = automatic.
  uint32_t attn_split_override = 0;
  // One arrival counter per attention row for the split-K merge; zero between launches.
  int* tickets = nullptr;
  size_t tickets_cap = 0;
  // The GEMV's split-tile partial sums and their arrival counters (same discipline).
  float* gemv_partials = nullptr;
  size_t gemv_partials_bytes = 0;
  int* gemv_tickets = nullptr;
  size_t gemv_tickets_cap = 0;

  // Between aion_cuda_record_begin and aion_cuda_record_end.
  bool recording = false;
  // Test hook (aion_cuda_debug_expire_waits): matmul launches leave out a copy and poll briefly,
  // so that a bounded wait runs out and the fault path can be observed.
  bool debug_expire_waits = false;

  // Tensor maps (TMA descriptors) already encoded for this device, keyed by view geometry.
  struct TmapCache;
  TmapCache* tmaps = nullptr;

  int32_t make_current() const;
  // Recorded programs hold the addresses of the scratch buffers they were recorded with, so
  // the buffers may not be re-allocated while one is alive.
  int live_programs = 0;
  int32_t reserve_scratch(size_t bytes);
  int32_t reserve_tickets(size_t count);
  int32_t reserve_gemv_fixup(size_t partial_bytes, size_t tickets);
  void* lane_scratch() const { return static_cast<uint8_t*>(scratch) + (size_t)cur_lane * scratch_bytes; }
  int* lane_tickets() const { return tickets + (size_t)cur_lane * tickets_cap; }
  float* lane_gemv_partials() const { return reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(gemv_partials) + (size_t)cur_lane * gemv_partials_bytes); }
  int* lane_gemv_tickets() const { return gemv_tickets + (size_t)cur_lane * gemv_tickets_cap; }
  // Reads the status word back (call after the stream has been synchronized).
  int32_t check_fault();
};

namespace aion {

// Resolve an operand to a typed device pointer after checking it covers `need` bytes.
template <class T>
inline int32_t resolve(const AionCudaOperand& op, size_t need, const char* name, T** out) {
  if (op.handle == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "%s: null handle", name);
  if (op.len < need) return fail(AION_CUDA_INVALID_ARGUMENT, "%s: operand holds %llu bytes, step needs %llu", name,
                                 (unsigned long long)op.len, (unsigned long long)need);
  *out = reinterpret_cast<T*>(static_cast<uintptr_t>(op.handle + op.offset));
  return AION_CUDA_OK;
}

// A rank-2 or rank-3 byte view of device memory for tiled TMA loads. dims[0] is the
// innermost extent in BYTES (a multiple of 8), dims[1..] are counts; strides[i] is the
// byte distance between consecutive indices of dimension i+1 (multiples of 16); box[0] is
// the innermost box extent in bytes (a multiple of 16, at most 2048), box[1..] counts
// (at most 256). The descriptor is cached on the device.
int32_t tensor_map_bytes(AionCudaDevice* dev, const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides,
                         const uint32_t* box, const CUtensorMap** out);

// The same descriptor written into caller storage, with no cache and no allocation of
// any kind (for the entry point that must not allocate).
int32_t tensor_map_encode(const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                          CUtensorMap* out);

// Row-major bf16 [rows, cols] view with a 128-byte swizzled box (tensor-core operand tiles).
int32_t tensor_map_bf16_sw128(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                              uint32_t box_rows, CUtensorMap* out);
// The same for either 16-bit float type (bf16 or f16).
int32_t tensor_map_16bit_sw128(const void* base, bool bf16, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                               uint32_t box_rows, CUtensorMap* out);

// Row-major f32 [rows, cols] view with a 128-byte swizzled box of 32 columns (bulk stores of output tiles).
int32_t tensor_map_f32_sw128(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows,
                             CUtensorMap* out);

// Launch with programmatic stream serialization: the kernel may be scheduled while its
// predecessor in the stream is still draining, which hides the launch latency of the chains
// of small kernels a decode step is made of. Such a kernel calls ptx::pdl_wait() before it
// reads anything an earlier kernel wrote (the wait returns when the predecessors have
// completed and their writes are visible) and ptx::pdl_launch_dependents() to let its own
// successor start early.
// Every kernel of the library asks for the largest shared-memory carve-out, whatever it uses itself. An SM
// changes its split between L1 and shared memory only while no CTA runs on it, so a kernel that needs a
// different split from the one running cannot start under it: with programmatic dependent launch that cost
// a matmul its head start (its CTAs, and with them its weight copies, began only when the small kernel before
// it had finished: measured 3 us later). Once per kernel and device.
inline void prefer_max_shared(const void* func) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> done;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return;
  std::lock_guard<std::mutex> lock(mu);
  if (done.insert({device, func}).second)
    cudaFuncSetAttribute(func, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_if(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// The small glue kernels: in stream order unless AION_CUDA_PDL_GLUE is set (with every kernel
// of a decode step scheduled early, the waiting ones hold SM resources the running ones
// need: measured slower at 8 requests, 2.59 ms against 2.28 ms).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  static const bool overlap = std::getenv("AION_CUDA_PDL_GLUE") != nullptr;  // tuning only
  return launch_pdl_if(overlap, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}
// The matmul kernels and their pre- and post-passes: overlapped unless AION_CUDA_NO_PDL_MAIN is
// set (the GEMM's set-up runs under the bf16 conversion, the reduction's launch under the GEMM).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_main(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  static const bool overlap = std::getenv("AION_CUDA_NO_PDL_MAIN") == nullptr;  // tuning only
  return launch_pdl_if(overlap, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

// ---- step implementations, one per kernel file ------------------------------------
int32_t quantize_activation_rows(AionCudaDevice* dev, const float* a, uint64_t m, uint64_t k, uint64_t lda,
                                 int8_t* aq, float* ascale);

// Column-split layers over several GPUs of a node: where a matmul also stores its outputs, and whom
// it tells when they have landed (aion_cuda_matmul_peers).
struct PeerFanout {
  float* c[7];          // C of the other ranks, laid out like this rank's
  uint32_t* flags[8];   // arrival words [8] of every rank, this one included
  uint32_t* state;      // this rank's: [0] epoch, [1] CTAs done
  uint32_t count;       // entries of c
  uint32_t world, rank;
};

struct MatMulArgs {
  const float* a;
  const uint8_t* b;
  float* c;
  uint32_t dtype;
  bool nt;            // B is [n, k] (quant_axis 1) rather than K-major
  uint32_t order;     // QuantBlockOrder, nt only
  uint64_t m, n, k, lda, ldb, ldc;
  float alpha, beta;
  // The quantized image of A written by the kernel that produced A (act_image.cuh), or null:
  // the int8 matmul then reads it instead of quantizing A itself.
  const uint8_t* a_image = nullptr;
  bool one_sm = false;   // keep the prefill GEMM on its one-SM kernel (no CTA pairs)
  const PeerFanout* peers = nullptr;   // int8 kernel only
};
int32_t matmul_generic(AionCudaDevice* dev, const MatMulArgs& g);
// Returns AION_CUDA_UNSUPPORTED (without setting an error) when the shape or the
// alignment is outside what the tiled kernel reads; the caller then routes elsewhere.
int32_t gemv_mma(AionCudaDevice* dev, const MatMulArgs& g, bool probe_only);
int32_t gemm_tcgen05(AionCudaDevice* dev, const MatMulArgs& g);
int32_t gemv_mma_static_scratch(AionCudaDevice* dev, const MatMulArgs& g);
// Quantizes f32 rows into an activation image (act_image.cuh) for weights of `dtype`.
int32_t act_image_from_f32(AionCudaDevice* dev, uint32_t dtype, const float* a, uint64_t m, uint64_t k, uint64_t lda, uint8_t* image);
// The bf16 kind of image (what the tensor-core GEMM reads), written by that kernel's own pre-pass.
int32_t nt_blocks_to_kmajor(AionCudaDevice* dev, uint32_t order, const uint8_t* src, uint8_t* dst, uint64_t n, uint64_t kblocks);
int32_t act_image_bf16_from_f32(AionCudaDevice* dev, uint32_t dtype, const float* a, uint64_t m, uint64_t k, uint64_t lda, uint8_t* image);
// What the prefill GEMM would do with this shape: rows per tile (128 or 256), K splits, CTAs.
struct GemmPlan {
  uint32_t tile_rows, splits, grid;
  bool pair;   // pairs of CTAs (two-SM MMAs); tile_rows is then the pair's
};
bool gemm_tcgen05_plan(const AionCudaDevice* dev, const MatMulArgs& g, GemmPlan* out);
int32_t attention_launch(AionCudaDevice* dev, const AionCudaAttention* s);
int32_t peer_wait_launch(AionCudaDevice* dev, const uint32_t* flags, uint32_t* state, uint32_t world, uint32_t poll_limit);

}  // namespace aion
