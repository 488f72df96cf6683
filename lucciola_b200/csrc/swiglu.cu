// SwiGLU: out = silu(gate) * up with silu(x) = x / (1 + exp(-x)), computed in
// 32-bit and rounded once (src/kernels/swiglu.cu:8,30-36 of lucciola).  gate
// and up are two column ranges of one matrix row (the fused gate|up product)
// or two separate matrices; `in_stride` is the distance between their rows.
#include "common.cuh"

namespace lb {

template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gate,
                              const T* __restrict__ up, long long in_stride, int inter,
                              long long total) {
  pdl_trigger();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / inter;
    const int c = (int)(idx - t * inter);
    const float g = to_f32(gate[t * in_stride + c]);
    const float u = to_f32(up[t * in_stride + c]);
    out[idx] = from_f32<T>(g / (1.f + expf(-g)) * u);
  }
}

// Eight bfloat16 values a thread (16-byte accesses).
__global__ void swiglu_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gate,
                                     const bf16* __restrict__ up, long long in_stride, int inter,
                                     long long total8) {
  pdl_trigger();
  pdl_wait();
  const int per_row = inter >> 3;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total8;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / per_row;
    const int c = (int)(idx - t * per_row) << 3;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gate + t * in_stride + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(up + t * in_stride + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 g = __bfloat1622float2(g2[i]);
      const float2 u = __bfloat1622float2(u2[i]);
      o2[i] = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = o4;
  }
}

}  // namespace lb

LB_EXPORT int lb_swiglu(int dtype, void* out, const void* gate, const void* up, long long in_stride,
                        int num_tokens, int inter, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "swiglu: bad dtype %d", dtype);
  LB_CHECK_ARG(num_tokens >= 0 && inter > 0 && in_stride >= inter, "swiglu: bad sizes");
  if (num_tokens == 0) return 0;
  const long long total = (long long)num_tokens * inter;
  const bool vec = dtype == LB_BF16 && inter % 8 == 0 && in_stride % 8 == 0 &&
                   ((uintptr_t)gate % 16 == 0) && ((uintptr_t)up % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (vec) {
    const long long total8 = total >> 3;
    const int blocks = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
    lb::launch(lb::swiglu_bf16x8_kernel, dim3(blocks), dim3(256), 0, stream, (lb::bf16*)out, (const lb::bf16*)gate,
               (const lb::bf16*)up, in_stride, inter, total8);
  } else {
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    LB_DISPATCH_DTYPE(dtype, T, {
      lb::launch(lb::swiglu_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out, (const T*)gate, (const T*)up,
                 in_stride, inter, total);
    })
  }
  LB_CHECK_LAUNCH("swiglu");
  return 0;
}
