// Error channel and build identification of the kernel library.
#include "common.cuh"
#include <cstring>

namespace lb {
static thread_local char g_error[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
int g_pdl_enabled = 1;
static unsigned long long g_launches = 0;
void count_launch() { __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED); }
}  // namespace lb

// Kernels this library has launched so far in this process (launches recorded into a CUDA graph
// count once, when they are recorded).
LB_EXPORT unsigned long long lb_launch_count() { return __atomic_load_n(&lb::g_launches, __ATOMIC_RELAXED); }

// Switches programmatic dependent launch on (default) or off for all later launches.
LB_EXPORT void lb_set_pdl(int on) { lb::g_pdl_enabled = on ? 1 : 0; }

// One asynchronous copy of a step's integers from pinned host memory to the device, in stream order.
LB_EXPORT int lb_upload(void* dst, const void* src, long long bytes, cudaStream_t stream) {
  LB_CHECK_ARG(dst && src && bytes >= 0, "upload: bad arguments");
  const cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) { lb::set_error("upload: %s", cudaGetErrorString(e)); return 2; }
  return 0;
}

// Message of the last failed call on this thread.
LB_EXPORT const char* lb_last_error() { return lb::g_error; }

// Interface version; the Python side refuses a library of another version.
LB_EXPORT int lb_abi_version() { return 3; }

// Compute capability of the current device as major*10+minor, or a negative
// CUDA error code.
LB_EXPORT int lb_device_arch() {
  int dev = 0, major = 0, minor = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -(int)e;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return -(int)e;
  e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  if (e != cudaSuccess) return -(int)e;
  return major * 10 + minor;
}
