// Status text, version and per-device facts behind the C ABI.
#include <cstdarg>
#include <mutex>

#include "common.cuh"

namespace rl {
bool g_launch_overlap = false;
namespace {
thread_local char g_error[512] = "";
constexpr int kMaxDevices = 64;
DeviceFacts g_facts[kMaxDevices];
std::mutex g_facts_mutex;
}  // namespace

int Fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}

int LaunchStatus(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return RL_OK;
  return Fail(static_cast<int>(e), "%s: %s", what, cudaGetErrorString(e));
}

int CurrentDeviceIndex() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  return dev;
}

const DeviceFacts& CurrentDeviceFacts() {
  const int dev = CurrentDeviceIndex();
  DeviceFacts& f = g_facts[dev];
  if (f.ready) return f;
  std::lock_guard<std::mutex> lock(g_facts_mutex);
  if (!f.ready) {
    cudaDeviceGetAttribute(&f.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&f.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (f.sm_count <= 0) f.sm_count = 148;
    f.ready = true;
  }
  return f;
}
}  // namespace rl

extern "C" const char* rl_version(void) { return "0.1.0"; }
extern "C" const char* rl_last_error(void) { return rl::g_error; }
