// Shared helpers of the kernel library: element types, conversions, warp and
// block reductions, the error channel of the C interface.
//
// Every exported function has C linkage, takes raw device pointers and a
// stream, validates its arguments on the host and returns 0 on success.  On
// failure it returns a non-zero code and leaves a message that
// lb_last_error() hands out; nothing is launched in that case.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#define LB_EXPORT extern "C" __attribute__((visibility("default")))

// Element type codes of the C interface.
enum LbDType : int { LB_F32 = 0, LB_BF16 = 1 };

namespace lb {

typedef __nv_bfloat16 bf16;

void set_error(const char* fmt, ...);
void count_launch();   // every kernel launch of the library is counted (lb_launch_count)

#define LB_CHECK_ARG(cond, ...)          \
  do {                                   \
    if (!(cond)) {                       \
      lb::set_error(__VA_ARGS__);        \
      return 1;                          \
    }                                    \
  } while (0)

// Called after a launch: reports a bad launch configuration at once.
#define LB_CHECK_LAUNCH(name)                                              \
  do {                                                                     \
    cudaError_t e__ = cudaGetLastError();                                  \
    if (e__ != cudaSuccess) {                                              \
      lb::set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
      return 2;                                                            \
    }                                                                      \
    lb::count_launch();                                                    \
  } while (0)

// Programmatic dependent launch.  Every kernel of the library is launched with the attribute that
// lets it start while the kernel before it on the stream is still running, calls pdl_trigger() at its
// start (so that its own successor may be scheduled early) and pdl_wait() before it reads anything
// another kernel wrote or writes anything at all.  pdl_wait() returns when the kernel before has
// completed and its writes are visible; in a kernel launched without the attribute both are no-ops.
// lb_set_pdl(0) switches the attribute off for all later launches.
extern int g_pdl_enabled;

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

// 2^x in one instruction (relative error about 2^-22, denormal results flushed to zero; 2^-inf = 0):
// for softmax weights that are rounded to bfloat16 afterwards.
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 33 floats of shared memory.  The order of the additions is
// fixed by the thread layout, so a row's sum does not depend on the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Dispatch on a (fp32 | bf16) element type code.
#define LB_DISPATCH_DTYPE(code, T, ...)                \
  if ((code) == LB_F32) { typedef float T; __VA_ARGS__ } \
  else { typedef lb::bf16 T; __VA_ARGS__ }

inline bool valid_dtype(int d) { return d == LB_F32 || d == LB_BF16; }

}  // namespace lb
