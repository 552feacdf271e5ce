// Host runtime shared by all kernels: error strings, per-device status words for bounded waits,
// TMA descriptor encoding through the driver entry point (no link-time dependency on libcuda).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace ajb {

static thread_local char g_error[1024] = {0};

void set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

const char* last_error() { return g_error; }

static constexpr int kMaxDevices = 16;
static DeviceStatus* g_status[kMaxDevices] = {nullptr};
static int g_sm_count[kMaxDevices] = {0};
static std::mutex g_mutex;

DeviceStatus* device_status_buffer() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status[dev] == nullptr) {
    DeviceStatus* buf = nullptr;
    if (cudaMalloc(&buf, sizeof(DeviceStatus) * kNumKernelIds) != cudaSuccess) return nullptr;
    cudaMemset(buf, 0, sizeof(DeviceStatus) * kNumKernelIds);
    g_status[dev] = buf;
  }
  return g_status[dev];
}

// First non-zero status word of this device (0 = none), cleared once read. One copy covers every kernel's word, so a
// caller that has just synchronised (a serving step after its token read-back) pays a few microseconds.
int check_device_status_all() {
  DeviceStatus* buf = device_status_buffer();
  if (buf == nullptr) return 0;
  DeviceStatus host[kNumKernelIds];
  if (cudaMemcpy(host, buf, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  for (int k = 0; k < kNumKernelIds; ++k) {
    if (host[k].code == 0) continue;
    set_error("kernel %d gave up waiting (stage %u, block %u, detail %u/%u)", k, host[k].code >> 8, host[k].block,
              host[k].detail0, host[k].detail1);
    cudaMemset(buf + k, 0, sizeof(DeviceStatus));
    return (int)host[k].code;
  }
  return 0;
}

int sm_count_physical() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

// SM budget of the calling host thread: kernels that size their grid from sm_count() (the persistent GEMMs, the
// tensor-parallel GEMMs, the grid-stride pointwise kernels) then occupy at most that many SMs, so that a kernel
// launched on another stream finds the rest of the device free at once instead of queueing behind a full wave.
static thread_local int g_sm_budget = 0;

int sm_count() {
  const int physical = sm_count_physical();
  return (g_sm_budget > 0 && g_sm_budget < physical) ? g_sm_budget : physical;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Descriptor encoding is a driver call and needs the primary context current on the calling thread.
// Threads that have only ever used the runtime lazily (autograd worker threads, for one) may not have
// it bound yet; one cudaFree(nullptr) per thread binds it.
static void bind_context_once() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

static EncodeTiledFn encode_fn() {
  bind_context_once();
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) == cudaSuccess &&
        query == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

int make_tensor_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t rows,
                       uint64_t cols, uint64_t row_pitch_bytes, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  AJB_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  AJB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base address must be 16-byte aligned");
  AJB_REQUIRE((row_pitch_bytes & 15) == 0, "TMA row pitch (%llu bytes) must be a multiple of 16",
              (unsigned long long)row_pitch_bytes);
  AJB_REQUIRE(box_cols * elem_bytes <= 128 && box_rows <= 256, "TMA box %ux%u is too large", box_rows, box_cols);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult res = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  AJB_REQUIRE(res == CUDA_SUCCESS, "cuTensorMapEncodeTiled(2d) failed with code %d (rows=%llu cols=%llu pitch=%llu)",
              (int)res, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)row_pitch_bytes);
  return 0;
}

int make_tensor_map_3d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t d2,
                       uint64_t rows, uint64_t cols, uint64_t d2_pitch_bytes, uint64_t row_pitch_bytes,
                       uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  AJB_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  AJB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base address must be 16-byte aligned");
  AJB_REQUIRE((row_pitch_bytes & 15) == 0 && (d2_pitch_bytes & 15) == 0, "TMA pitches must be multiples of 16");
  AJB_REQUIRE(box_cols * elem_bytes <= 128 && box_rows <= 256, "TMA box %ux%u is too large", box_rows, box_cols);
  cuuint64_t dims[3] = {cols, rows, d2};
  cuuint64_t strides[2] = {row_pitch_bytes, d2_pitch_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult res = fn(map, dtype, 3, const_cast<void*>(base), dims, strides, box, elem_strides,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  AJB_REQUIRE(res == CUDA_SUCCESS, "cuTensorMapEncodeTiled(3d) failed with code %d", (int)res);
  return 0;
}

}  // namespace ajb

extern "C" const char* ajb_last_error() { return ajb::last_error(); }

// 0 (or a value >= the device's SM count) lifts the budget. Returns the previous budget of this thread.
extern "C" int ajb_set_sm_budget(int sms) {
  const int previous = ajb::g_sm_budget;
  ajb::g_sm_budget = sms > 0 ? sms : 0;
  return previous;
}
extern "C" int ajb_sm_count() { return ajb::sm_count_physical(); }

// Returns 0 when no kernel has reported an expired wait since the last call; otherwise the status
// code of the first one found (and clears it). Synchronises the device.
extern "C" int ajb_check_status() {
  if (cudaDeviceSynchronize() != cudaSuccess) {
    ajb::set_error("device synchronize failed: %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  return ajb::check_device_status_all();
}
