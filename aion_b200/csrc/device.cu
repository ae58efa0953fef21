// Device lifetime, the DeviceMemory entry points and the per-thread diagnostic.
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <unordered_map>

#include "common.cuh"

namespace aion {

static thread_local std::string g_last_error;

void set_error(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

int32_t fail(int32_t status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return status;
}

int32_t cuda_fail(cudaError_t e, const char* what) {
  const int32_t st = (e == cudaErrorMemoryAllocation) ? AION_CUDA_OUT_OF_MEMORY : AION_CUDA_INTERNAL_ERROR;
  return fail(st, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

}  // namespace aion

struct AionCudaDevice::TmapCache {
  struct Key {
    uint64_t v[10];  // base, rank, dims[3], box[3], strides[2]
    bool operator==(const Key& o) const {
      for (int i = 0; i < 10; i++)
        if (v[i] != o.v[i]) return false;
      return true;
    }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      uint64_t h = 0xCBF29CE484222325ull;
      for (int i = 0; i < 10; i++) h = (h ^ k.v[i]) * 0x100000001B3ull;
      return (size_t)(h ^ (h >> 29));
    }
  };
  std::unordered_map<Key, CUtensorMap, Hash> map;
};

namespace aion {

int32_t tensor_map_bytes(AionCudaDevice* dev, const void* base, uint32_t rank, const uint64_t* dim_bytes0_then_counts,
                         const uint64_t* stride_bytes, const uint32_t* box, const CUtensorMap** out) {
  if (!dev->tmaps) {
    dev->tmaps = new (std::nothrow) AionCudaDevice::TmapCache();
    if (!dev->tmaps) return fail(AION_CUDA_OUT_OF_MEMORY, "tensor map cache: host allocation failed");
  }
  AionCudaDevice::TmapCache::Key key{};
  key.v[0] = (uint64_t)(uintptr_t)base;
  key.v[1] = rank;
  for (uint32_t i = 0; i < rank; i++) {
    key.v[2 + i] = dim_bytes0_then_counts[i];
    key.v[5 + i] = box[i];
    if (i + 1 < rank) key.v[8 + i] = stride_bytes[i];
  }
  auto& m = dev->tmaps->map;
  auto it = m.find(key);
  if (it == m.end()) {
    if (m.size() > 8192) m.clear();  // descriptors are cheap to rebuild; keep the table bounded
    // Elements are 8-byte words so that a box row may hold up to 2048 bytes.
    if (rank < 2 || rank > 3 || (dim_bytes0_then_counts[0] & 7) || (box[0] & 15) || box[0] / 8 > 256 || ((uintptr_t)base & 15))
      return fail(AION_CUDA_INTERNAL_ERROR, "tensor map: view geometry is not TMA-addressable");
    cuuint64_t gdim[3] = {dim_bytes0_then_counts[0] / 8, 1, 1};
    cuuint64_t gstride[2] = {0, 0};
    cuuint32_t bx[3] = {box[0] / 8, 1, 1};
    const cuuint32_t estride[3] = {1, 1, 1};
    for (uint32_t i = 1; i < rank; i++) {
      gdim[i] = dim_bytes0_then_counts[i];
      bx[i] = box[i];
      gstride[i - 1] = stride_bytes[i - 1];
      if ((stride_bytes[i - 1] & 15) || box[i] > 256)
        return fail(AION_CUDA_INTERNAL_ERROR, "tensor map: view geometry is not TMA-addressable");
    }
    // The driver entry point is looked up through the runtime, so the library does not
    // link libcuda and still loads on a machine without a driver.
    typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      AION_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (!fn || qres != cudaDriverEntryPointSuccess) return fail(AION_CUDA_INTERNAL_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
      encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    CUtensorMap tm;
    const CUresult r = encode(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT64, rank, const_cast<void*>(base), gdim, gstride, bx,
                                              estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AION_CUDA_INTERNAL_ERROR, "cuTensorMapEncodeTiled failed with %d", (int)r);
    it = m.emplace(key, tm).first;
  }
  *out = &it->second;
  return AION_CUDA_OK;
}

int32_t tensor_map_encode(const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                          CUtensorMap* out) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    AION_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess) return fail(AION_CUDA_INTERNAL_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if (rank < 2 || rank > 3 || (dims[0] & 7) || (box[0] & 15) || box[0] / 8 > 256 || ((uintptr_t)base & 15))
    return fail(AION_CUDA_INTERNAL_ERROR, "tensor map: view geometry is not TMA-addressable");
  cuuint64_t gdim[3] = {dims[0] / 8, 1, 1};
  cuuint64_t gstride[2] = {0, 0};
  cuuint32_t bx[3] = {box[0] / 8, 1, 1};
  const cuuint32_t estride[3] = {1, 1, 1};
  for (uint32_t i = 1; i < rank; i++) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    gstride[i - 1] = strides[i - 1];
    if ((strides[i - 1] & 15) || box[i] > 256) return fail(AION_CUDA_INTERNAL_ERROR, "tensor map: view geometry is not TMA-addressable");
  }
  const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, rank, const_cast<void*>(base), gdim, gstride, bx, estride,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AION_CUDA_INTERNAL_ERROR, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return AION_CUDA_OK;
}

// Row-major bf16 matrix [rows, cols] (row pitch in bytes, a multiple of 16) with a
// 128-byte swizzled box of box_cols (= 64) x box_rows: the layout tcgen05 K-major operand
// descriptors read. Out-of-range rows and columns arrive as zeros.
int32_t tensor_map_bf16_sw128(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                              uint32_t box_rows, CUtensorMap* out) {
  return tensor_map_16bit_sw128(base, true, rows, cols, pitch_bytes, box_cols, box_rows, out);
}

// Row-major 2-D view with a 128-byte swizzled box: the box's inner extent is exactly one swizzle row.
static int32_t tensor_map_2d_sw128(const void* base, CUtensorMapDataType type, uint32_t elem_bytes, uint64_t rows, uint64_t cols,
                                   uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, CUtensorMap* out) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    AION_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess) return fail(AION_CUDA_INTERNAL_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if (((uintptr_t)base & 15) || (pitch_bytes & 15) || box_cols * elem_bytes != 128 || box_rows > 256)
    return fail(AION_CUDA_INTERNAL_ERROR, "tensor map: swizzled view geometry is not TMA-addressable");
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {pitch_bytes};
  const cuuint32_t bx[2] = {box_cols, box_rows};
  const cuuint32_t estride[2] = {1, 1};
  const CUresult r = encode(out, type, 2, const_cast<void*>(base), gdim, gstride, bx, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AION_CUDA_INTERNAL_ERROR, "cuTensorMapEncodeTiled (swizzled) failed with %d", (int)r);
  return AION_CUDA_OK;
}

int32_t tensor_map_16bit_sw128(const void* base, bool bf16, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                               uint32_t box_rows, CUtensorMap* out) {
  return tensor_map_2d_sw128(base, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, rows, cols, pitch_bytes,
                             box_cols, box_rows, out);
}

int32_t tensor_map_f32_sw128(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows,
                             CUtensorMap* out) {
  return tensor_map_2d_sw128(base, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, rows, cols, pitch_bytes, box_cols, box_rows, out);
}

}  // namespace aion

using namespace aion;

int32_t AionCudaDevice::make_current() const {
  int cur = -1;
  AION_CUDA_TRY(cudaGetDevice(&cur));
  if (cur != ordinal) AION_CUDA_TRY(cudaSetDevice(ordinal));
  return AION_CUDA_OK;
}

int32_t AionCudaDevice::reserve_scratch(size_t bytes) {
  if (bytes <= scratch_bytes) return AION_CUDA_OK;
  if (recording) return fail(AION_CUDA_INVALID_ARGUMENT, "a recorded step needs %llu bytes of scratch that are not reserved yet: run it once before recording", (unsigned long long)bytes);
  if (live_programs > 0) return fail(AION_CUDA_INVALID_ARGUMENT, "this step needs more device scratch than is reserved, and a recorded program still uses the current buffers: destroy the program, or run the largest step once before recording");
  // Earlier launches may still read the old buffer.
  AION_CUDA_TRY(cudaStreamSynchronize(stream));
  if (scratch) AION_CUDA_TRY(cudaFree(scratch));
  scratch = nullptr;
  scratch_bytes = 0;
  size_t want = bytes + (bytes >> 2);
  want = (want + 255) & ~size_t(255);
  AION_CUDA_TRY(cudaMalloc(&scratch, want * LANES));
  scratch_bytes = want;
  return AION_CUDA_OK;
}

int32_t AionCudaDevice::reserve_tickets(size_t count) {
  if (count <= tickets_cap) return AION_CUDA_OK;
  if (recording) return fail(AION_CUDA_INVALID_ARGUMENT, "a recorded attention step needs arrival counters that are not reserved yet: run it once before recording");
  if (live_programs > 0) return fail(AION_CUDA_INVALID_ARGUMENT, "this step needs more device scratch than is reserved, and a recorded program still uses the current buffers: destroy the program, or run the largest step once before recording");
  AION_CUDA_TRY(cudaStreamSynchronize(stream));
  if (tickets) AION_CUDA_TRY(cudaFree(tickets));
  tickets = nullptr;
  tickets_cap = 0;
  size_t want = count < 1024 ? 1024 : count + (count >> 1);
  AION_CUDA_TRY(cudaMalloc(&tickets, want * sizeof(int) * LANES));
  AION_CUDA_TRY(cudaMemsetAsync(tickets, 0, want * sizeof(int) * LANES, stream));
  tickets_cap = want;
  return AION_CUDA_OK;
}

int32_t AionCudaDevice::reserve_gemv_fixup(size_t partial_bytes, size_t ticket_count) {
  if (partial_bytes > gemv_partials_bytes) {
    if (recording) return fail(AION_CUDA_INVALID_ARGUMENT, "a recorded matmul step needs split-tile scratch that is not reserved yet: run it once before recording");
    if (live_programs > 0) return fail(AION_CUDA_INVALID_ARGUMENT, "this step needs more device scratch than is reserved, and a recorded program still uses the current buffers: destroy the program, or run the largest step once before recording");
    AION_CUDA_TRY(cudaStreamSynchronize(stream));
    if (gemv_partials) AION_CUDA_TRY(cudaFree(gemv_partials));
    gemv_partials = nullptr;
    gemv_partials_bytes = 0;
    const size_t want = (partial_bytes + (partial_bytes >> 2) + 255) & ~size_t(255);
    AION_CUDA_TRY(cudaMalloc(&gemv_partials, want * LANES));
    gemv_partials_bytes = want;
  }
  if (ticket_count > gemv_tickets_cap) {
    if (recording) return fail(AION_CUDA_INVALID_ARGUMENT, "a recorded matmul step needs arrival counters that are not reserved yet: run it once before recording");
    if (live_programs > 0) return fail(AION_CUDA_INVALID_ARGUMENT, "this step needs more device scratch than is reserved, and a recorded program still uses the current buffers: destroy the program, or run the largest step once before recording");
    AION_CUDA_TRY(cudaStreamSynchronize(stream));
    if (gemv_tickets) AION_CUDA_TRY(cudaFree(gemv_tickets));
    gemv_tickets = nullptr;
    gemv_tickets_cap = 0;
    const size_t want = ticket_count < 4096 ? 4096 : ticket_count + (ticket_count >> 1);
    AION_CUDA_TRY(cudaMalloc(&gemv_tickets, want * sizeof(int) * LANES));
    AION_CUDA_TRY(cudaMemsetAsync(gemv_tickets, 0, want * sizeof(int) * LANES, stream));
    gemv_tickets_cap = want;
  }
  return AION_CUDA_OK;
}

int32_t AionCudaDevice::check_fault() {
  // The stream is idle here, so a plain copy of one word is enough.
  AION_CUDA_TRY(cudaMemcpy(fault_host, fault_dev, sizeof(int), cudaMemcpyDeviceToHost));
  const int f = *fault_host;
  if (f == FAULT_NONE) return AION_CUDA_OK;
  AION_CUDA_TRY(cudaMemset(fault_dev, 0, sizeof(int)));
  switch (f) {
    case FAULT_INVALID_ARGUMENT:
      return fail(AION_CUDA_INVALID_ARGUMENT,
                  "a kernel rejected its inputs (a negative or out-of-range position, length or index, or a non-finite norm)");
    case FAULT_WAIT_EXPIRED:
      return fail(AION_CUDA_INTERNAL_ERROR, "a kernel gave up a bounded wait on a copy barrier");
    case FAULT_NONFINITE:
      return fail(AION_CUDA_INVALID_ARGUMENT, "attention: softmax denominator is not finite and positive");
    default:
      return fail(AION_CUDA_INTERNAL_ERROR, "kernel fault code %d", f);
  }
}

extern "C" {

int32_t aion_cuda_device_count(int32_t* out_count) {
  if (!out_count) return fail(AION_CUDA_INVALID_ARGUMENT, "device_count: null out");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    *out_count = 0;
    return cuda_fail(e, "cudaGetDeviceCount");
  }
  *out_count = n;
  return AION_CUDA_OK;
}

int32_t aion_cuda_device_create(int32_t ordinal, AionCudaDevice** out) {
  if (!out) return fail(AION_CUDA_INVALID_ARGUMENT, "device_create: null out");
  *out = nullptr;
  int n = 0;
  AION_CUDA_TRY(cudaGetDeviceCount(&n));
  if (ordinal < 0 || ordinal >= n) return fail(AION_CUDA_INVALID_ARGUMENT, "device_create: ordinal %d of %d", ordinal, n);
  AionCudaDevice* d = new (std::nothrow) AionCudaDevice();
  if (!d) return fail(AION_CUDA_OUT_OF_MEMORY, "device_create: host allocation failed");
  d->ordinal = ordinal;
  cudaError_t e = cudaSetDevice(ordinal);
  if (e == cudaSuccess) e = cudaGetDeviceProperties(&d->prop, ordinal);
  if (e == cudaSuccess && d->prop.major != 10) {
    const int major = d->prop.major, minor = d->prop.minor;
    delete d;
    return fail(AION_CUDA_UNSUPPORTED, "device_create: device %d is sm_%d%d; this library holds sm_100a code only",
                ordinal, major, minor);
  }
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&d->own_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(&d->fault_dev, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(d->fault_dev, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost(&d->fault_host, sizeof(int));
  if (e != cudaSuccess) {
    const int32_t st = cuda_fail(e, "device_create");
    aion_cuda_device_destroy(d);
    return st;
  }
  d->stream = d->own_stream;
  d->main_stream = d->own_stream;
  d->sm_count = d->prop.multiProcessorCount;
  if (const char* e2 = std::getenv("AION_CUDA_GEMV_SPLIT")) {
    const int v = std::atoi(e2);
    if (v == 1 || v == 2 || v == 4 || v == 8) d->gemv_split_override = (uint32_t)v;
  }
  if (const char* e3 = std::getenv("AION_CUDA_ATTN_SPLIT")) {
    const int v = std::atoi(e3);
    if (v >= 1 && v <= 256) d->attn_split_override = (uint32_t)v;
  }
  *out = d;
  return AION_CUDA_OK;
}

void aion_cuda_device_destroy(AionCudaDevice* dev) {
  if (!dev) return;
  cudaSetDevice(dev->ordinal);
  if (dev->own_stream) {
    cudaStreamSynchronize(dev->own_stream);
    cudaStreamDestroy(dev->own_stream);
  }
  for (int l = 1; l < AionCudaDevice::LANES; l++) {
    if (dev->lane_streams[l]) cudaStreamDestroy(dev->lane_streams[l]);
    if (dev->lane_events[l]) cudaEventDestroy(dev->lane_events[l]);
  }
  if (dev->fork_event) cudaEventDestroy(dev->fork_event);
  if (dev->scratch) cudaFree(dev->scratch);
  if (dev->tickets) cudaFree(dev->tickets);
  if (dev->gemv_partials) cudaFree(dev->gemv_partials);
  if (dev->gemv_tickets) cudaFree(dev->gemv_tickets);
  delete dev->tmaps;
  if (dev->fault_dev) cudaFree(dev->fault_dev);
  if (dev->fault_host) cudaFreeHost(dev->fault_host);
  delete dev;
}

int32_t aion_cuda_device_info(AionCudaDevice* dev, AionCudaDeviceInfo* out) {
  if (!dev || !out) return fail(AION_CUDA_INVALID_ARGUMENT, "device_info: null argument");
  std::memset(out, 0, sizeof *out);
  std::strncpy(out->name, dev->prop.name, sizeof(out->name) - 1);
  out->ordinal = dev->ordinal;
  out->sm_count = dev->prop.multiProcessorCount;
  out->cc_major = dev->prop.major;
  out->cc_minor = dev->prop.minor;
  out->total_bytes = dev->prop.totalGlobalMem;
  out->l2_bytes = (uint64_t)dev->prop.l2CacheSize;
  return AION_CUDA_OK;
}

uint8_t aion_cuda_quant_block_order(AionCudaDevice*) { return AION_CUDA_ORDER_ROW_MAJOR; }

int32_t aion_cuda_set_stream(AionCudaDevice* dev, void* cuda_stream) {
  if (!dev) return fail(AION_CUDA_INVALID_ARGUMENT, "set_stream: null device");
  if (dev->recording) return fail(AION_CUDA_INVALID_ARGUMENT, "set_stream: not while recording");
  dev->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : dev->own_stream;
  dev->main_stream = dev->stream;
  return AION_CUDA_OK;
}

void* aion_cuda_get_stream(AionCudaDevice* dev) { return dev ? (void*)dev->stream : nullptr; }

int32_t aion_cuda_sync(AionCudaDevice* dev) {
  if (!dev) return fail(AION_CUDA_INVALID_ARGUMENT, "sync: null device");
  if (int32_t st = dev->make_current()) return st;
  AION_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  return dev->check_fault();
}

struct AionCudaProgram {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
};

int32_t aion_cuda_record_begin(AionCudaDevice* dev) {
  if (!dev) return fail(AION_CUDA_INVALID_ARGUMENT, "record_begin: null device");
  if (dev->recording) return fail(AION_CUDA_INVALID_ARGUMENT, "record_begin: already recording");
  if (int32_t st = dev->make_current()) return st;
  // Lane streams and events are created on first use (outside any capture).
  for (int l = 1; l < AionCudaDevice::LANES; l++) {
    if (!dev->lane_streams[l]) AION_CUDA_TRY(cudaStreamCreateWithFlags(&dev->lane_streams[l], cudaStreamNonBlocking));
    if (!dev->lane_events[l]) AION_CUDA_TRY(cudaEventCreateWithFlags(&dev->lane_events[l], cudaEventDisableTiming));
  }
  if (!dev->fork_event) AION_CUDA_TRY(cudaEventCreateWithFlags(&dev->fork_event, cudaEventDisableTiming));
  AION_CUDA_TRY(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
  dev->recording = true;
  return AION_CUDA_OK;
}

static int32_t join_lanes(AionCudaDevice* dev) {
  for (int l = 1; l < AionCudaDevice::LANES; l++) {
    if (!dev->lane_forked[l]) continue;
    AION_CUDA_TRY(cudaEventRecord(dev->lane_events[l], dev->lane_streams[l]));
    AION_CUDA_TRY(cudaStreamWaitEvent(dev->main_stream, dev->lane_events[l], 0));
    dev->lane_forked[l] = false;
  }
  dev->cur_lane = 0;
  dev->stream = dev->main_stream;
  return AION_CUDA_OK;
}

int32_t aion_cuda_record_lane(AionCudaDevice* dev, uint32_t lane) {
  if (!dev) return fail(AION_CUDA_INVALID_ARGUMENT, "record_lane: null device");
  if (!dev->recording) return fail(AION_CUDA_INVALID_ARGUMENT, "record_lane: not recording");
  if (lane >= (uint32_t)AionCudaDevice::LANES) return fail(AION_CUDA_INVALID_ARGUMENT, "record_lane: lane %u of %d", lane, AionCudaDevice::LANES);
  if (lane != 0 && !dev->lane_forked[lane]) {
    // The lane starts after everything recorded so far on the device's own stream.
    AION_CUDA_TRY(cudaEventRecord(dev->fork_event, dev->main_stream));
    AION_CUDA_TRY(cudaStreamWaitEvent(dev->lane_streams[lane], dev->fork_event, 0));
    dev->lane_forked[lane] = true;
  }
  dev->cur_lane = (int)lane;
  dev->stream = lane == 0 ? dev->main_stream : dev->lane_streams[lane];
  return AION_CUDA_OK;
}

int32_t aion_cuda_record_join(AionCudaDevice* dev) {
  if (!dev) return fail(AION_CUDA_INVALID_ARGUMENT, "record_join: null device");
  if (!dev->recording) return fail(AION_CUDA_INVALID_ARGUMENT, "record_join: not recording");
  return join_lanes(dev);
}

int32_t aion_cuda_record_end(AionCudaDevice* dev, AionCudaProgram** out) {
  if (!dev || !out) return fail(AION_CUDA_INVALID_ARGUMENT, "record_end: null argument");
  *out = nullptr;
  if (!dev->recording) return fail(AION_CUDA_INVALID_ARGUMENT, "record_end: not recording");
  const int32_t jst = join_lanes(dev);
  dev->recording = false;
  if (jst != AION_CUDA_OK) {
    cudaGraph_t dead = nullptr;
    cudaStreamEndCapture(dev->main_stream, &dead);
    if (dead) cudaGraphDestroy(dead);
    cudaGetLastError();
    return jst;
  }
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(dev->stream, &graph);
  if (e != cudaSuccess || !graph) {
    cudaGetLastError();
    return fail(AION_CUDA_INTERNAL_ERROR, "record_end: the recording was invalidated (%s); a recorded step may have "
                "allocated or synchronized", cudaGetErrorString(e));
  }
  AionCudaProgram* p = new (std::nothrow) AionCudaProgram();
  if (!p) {
    cudaGraphDestroy(graph);
    return fail(AION_CUDA_OUT_OF_MEMORY, "record_end: host allocation failed");
  }
  p->graph = graph;
  e = cudaGraphInstantiate(&p->exec, graph, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(graph);
    delete p;
    return cuda_fail(e, "cudaGraphInstantiate");
  }
  dev->live_programs++;
  *out = p;
  return AION_CUDA_OK;
}

int32_t aion_cuda_program_launch(AionCudaDevice* dev, AionCudaProgram* prog) {
  if (!dev || !prog || !prog->exec) return fail(AION_CUDA_INVALID_ARGUMENT, "program_launch: null argument");
  if (int32_t st = dev->make_current()) return st;
  AION_CUDA_TRY(cudaGraphLaunch(prog->exec, dev->stream));
  return AION_CUDA_OK;
}

void aion_cuda_program_destroy(AionCudaDevice* dev, AionCudaProgram* prog) {
  if (!prog) return;
  if (dev) {
    cudaSetDevice(dev->ordinal);
    cudaStreamSynchronize(dev->stream);
    if (dev->live_programs > 0) dev->live_programs--;
  }
  if (prog->exec) cudaGraphExecDestroy(prog->exec);
  if (prog->graph) cudaGraphDestroy(prog->graph);
  delete prog;
}

int32_t aion_cuda_debug_expire_waits(AionCudaDevice* dev, int32_t on) {
  if (!dev) return fail(AION_CUDA_INVALID_ARGUMENT, "debug_expire_waits: null device");
  dev->debug_expire_waits = on != 0;
  return AION_CUDA_OK;
}

int32_t aion_cuda_last_error(char* buf, size_t cap, size_t* len) {
  const std::string& s = g_last_error;
  if (len) *len = s.size();
  if (buf && cap > 0) {
    const size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
    std::memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return AION_CUDA_OK;
}

int32_t aion_cuda_memory_model(AionCudaDevice*) { return 0; }
uint64_t aion_cuda_max_binding_bytes(AionCudaDevice*) { return UINT64_MAX; }

int32_t aion_cuda_alloc(AionCudaDevice* dev, size_t bytes, size_t alignment, uint64_t* out_handle) {
  if (!dev || !out_handle) return fail(AION_CUDA_INVALID_ARGUMENT, "alloc: null argument");
  *out_handle = 0;
  // cudaMalloc returns 256-byte aligned addresses.
  if (alignment > 256 || (alignment & (alignment - 1)) != 0)
    return fail(AION_CUDA_INVALID_ARGUMENT, "alloc: alignment %llu is not a power of two <= 256", (unsigned long long)alignment);
  if (int32_t st = dev->make_current()) return st;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(AION_CUDA_OUT_OF_MEMORY, "alloc: %llu bytes: %s", (unsigned long long)bytes, cudaGetErrorString(e));
  }
  *out_handle = (uint64_t)(uintptr_t)p;
  return AION_CUDA_OK;
}

int32_t aion_cuda_free(AionCudaDevice* dev, uint64_t handle) {
  if (!dev) return fail(AION_CUDA_INVALID_ARGUMENT, "free: null device");
  if (handle == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  // Work that still reads the buffer must finish first (cudaFree also synchronizes,
  // but only implicitly).
  AION_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  AION_CUDA_TRY(cudaFree((void*)(uintptr_t)handle));
  return AION_CUDA_OK;
}

int32_t aion_cuda_h2d(AionCudaDevice* dev, uint64_t handle, size_t dst_offset, const void* src, size_t bytes) {
  if (!dev || handle == 0 || (!src && bytes)) return fail(AION_CUDA_INVALID_ARGUMENT, "h2d: null argument");
  if (bytes == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  AION_CUDA_TRY(cudaMemcpyAsync((void*)(uintptr_t)(handle + dst_offset), src, bytes, cudaMemcpyHostToDevice, dev->stream));
  // The source may be pageable and reused by the caller right after return.
  AION_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  return AION_CUDA_OK;
}

int32_t aion_cuda_d2h(AionCudaDevice* dev, void* dst, uint64_t handle, size_t src_offset, size_t bytes) {
  if (!dev || handle == 0 || (!dst && bytes)) return fail(AION_CUDA_INVALID_ARGUMENT, "d2h: null argument");
  if (int32_t st = dev->make_current()) return st;
  if (bytes) AION_CUDA_TRY(cudaMemcpyAsync(dst, (const void*)(uintptr_t)(handle + src_offset), bytes, cudaMemcpyDeviceToHost, dev->stream));
  AION_CUDA_TRY(cudaStreamSynchronize(dev->stream));
  return dev->check_fault();
}

int32_t aion_cuda_d2d(AionCudaDevice* dev, uint64_t dst, size_t dst_offset, uint64_t src, size_t src_offset, size_t bytes) {
  if (!dev || dst == 0 || src == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "d2d: null argument");
  if (bytes == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  AION_CUDA_TRY(cudaMemcpyAsync((void*)(uintptr_t)(dst + dst_offset), (const void*)(uintptr_t)(src + src_offset), bytes,
                                cudaMemcpyDeviceToDevice, dev->stream));
  return AION_CUDA_OK;
}

int32_t aion_cuda_memset(AionCudaDevice* dev, uint64_t handle, size_t offset, int32_t byte_value, size_t bytes) {
  if (!dev || handle == 0) return fail(AION_CUDA_INVALID_ARGUMENT, "memset: null argument");
  if (bytes == 0) return AION_CUDA_OK;
  if (int32_t st = dev->make_current()) return st;
  AION_CUDA_TRY(cudaMemsetAsync((void*)(uintptr_t)(handle + offset), byte_value, bytes, dev->stream));
  return AION_CUDA_OK;
}

}  // extern "C"
