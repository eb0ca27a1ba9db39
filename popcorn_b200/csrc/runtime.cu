// Host-side plumbing of the C ABI: status strings, per-thread error text,
// launch accounting and the per-device capability check.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace b200 {

namespace {
thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};

constexpr int kMaxDevices = 64;
// 0 = not probed yet, otherwise (cc_major << 16 | sm_count) + 1
std::atomic<uint32_t> g_device_info[kMaxDevices];

uint32_t device_info() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return 0;
  }
  uint32_t cached = g_device_info[dev].load(std::memory_order_acquire);
  if (cached != 0) return cached;
  int major = 0, sms = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  uint32_t info = ((static_cast<uint32_t>(major) << 16) | static_cast<uint32_t>(sms & 0xffff)) + 1;
  g_device_info[dev].store(info, std::memory_order_release);
  return info;
}
}  // namespace

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

int after_launch(const char* kernel) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(B200_ERR_LAUNCH, "%s: launch failed: %s", kernel, cudaGetErrorString(err));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200_OK;
}

int check_device() {
  uint32_t info = device_info();
  if (info == 0) return fail(B200_ERR_DEVICE, "no usable CUDA device is current");
  int major = static_cast<int>((info - 1) >> 16);
  if (major != 10)
    return fail(B200_ERR_DEVICE, "libpopcorn_b200 is built for sm_100a only; current device is compute capability %d.x", major);
  return B200_OK;
}

bool pdl_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("B200_PDL");
    return v == nullptr || v[0] != '0';
  }();
  return enabled;
}

int sm_count() {
  uint32_t info = device_info();
  return info == 0 ? 1 : static_cast<int>((info - 1) & 0xffff);
}

}  // namespace b200

extern "C" {

int b200_version(void) { return B200_ABI_VERSION; }

const char* b200_status_string(int status) {
  switch (status) {
    case B200_OK: return "B200_OK";
    case B200_ERR_NULL_POINTER: return "B200_ERR_NULL_POINTER";
    case B200_ERR_DTYPE: return "B200_ERR_DTYPE";
    case B200_ERR_SHAPE: return "B200_ERR_SHAPE";
    case B200_ERR_ALIGNMENT: return "B200_ERR_ALIGNMENT";
    case B200_ERR_LAUNCH: return "B200_ERR_LAUNCH";
    case B200_ERR_SCRATCH: return "B200_ERR_SCRATCH";
    case B200_ERR_DEVICE: return "B200_ERR_DEVICE";
    default: return "B200_ERR_UNKNOWN";
  }
}

const char* b200_last_error(void) { return b200::g_error; }

uint64_t b200_launch_count(void) { return b200::g_launches.load(std::memory_order_relaxed); }

uint64_t b200_wait_timeouts(void) {
  return static_cast<uint64_t>(b200::rope_wait_timeouts()) + static_cast<uint64_t>(b200::norm_wait_timeouts()) +
         static_cast<uint64_t>(b200::gemm_wait_timeouts());
}

}  // extern "C"
