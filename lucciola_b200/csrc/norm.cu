// Residual add fused with RMSNorm.
//
//   v      = residual[src] + delta[src]          (delta optional)
//   residual[src] = v                            (only when rows == nullptr)
//   out[i] = v * rsqrt(mean(v^2) + eps) * weight
//
// with src = rows ? rows[i] : i.  The residual stream and the norm weight are
// 32-bit; the statistics, the normalisation and the product with the weight
// are computed in 32-bit and rounded once, as src/kernels/rmsnorm.cu:57-97 of
// lucciola does (weight multiplied inside the single rounding, no 1+w).  The
// reference runs add (src/kernels/add.cu:11-14), a copy and the norm as three
// launches; this is one pass over the row.
#include "common.cuh"

namespace lb {

template <typename TD, typename TO, int VEC>
__global__ void add_rmsnorm_kernel(TO* __restrict__ out, float* __restrict__ residual,
                                   const TD* __restrict__ delta, const float* __restrict__ weight,
                                   const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  float* r = residual + (size_t)src * hidden;
  const TD* d = delta ? delta + (size_t)src * hidden : nullptr;
  TO* o = out + (size_t)i * hidden;
  const bool update = (rows == nullptr) && (delta != nullptr);

  float ss = 0.f;
  if (VEC == 4) {
    const int n4 = hidden >> 2;
    for (int j = threadIdx.x; j < n4; j += blockDim.x) {
      float4 v = reinterpret_cast<const float4*>(r)[j];
      if (d) {
        v.x += to_f32(d[4 * j + 0]); v.y += to_f32(d[4 * j + 1]);
        v.z += to_f32(d[4 * j + 2]); v.w += to_f32(d[4 * j + 3]);
        if (update) reinterpret_cast<float4*>(r)[j] = v;
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
      float v = r[j];
      if (d) { v += to_f32(d[j]); if (update) r[j] = v; }
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  // Second pass: the row is in L1/L2.  When the residual was not updated the
  // sum has to be formed again.
  const bool readd = d && !update;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
    float v = r[j];
    if (readd) v += to_f32(d[j]);
    o[j] = from_f32<TO>(v * inv * weight[j]);
  }
}

// Four consecutive elements as one access.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

// The same for rows that fit the CTA's registers (hidden = PER * threads, PER a multiple of 4): one pass.  Every
// load of a thread is issued before any is used, the norm weights even before the kernel ahead has finished (they do
// not depend on it); the row is read once, kept in registers across the sum, and written with 8- or 16-byte stores.
template <typename TD, typename TO, int PER>
__global__ void add_rmsnorm_row_kernel(TO* __restrict__ out, float* __restrict__ residual, const TD* __restrict__ delta,
                                       const float* __restrict__ weight, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  const int tid = threadIdx.x, nt = blockDim.x;
  float4 w[PER / 4], v[PER / 4];
#pragma unroll
  for (int q = 0; q < PER / 4; ++q) w[q] = load4(weight + 4 * (q * nt + tid));
  pdl_wait();
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  float* r = residual + (size_t)src * hidden;
  const bool update = (rows == nullptr) && (delta != nullptr);
#pragma unroll
  for (int q = 0; q < PER / 4; ++q) v[q] = load4(r + 4 * (q * nt + tid));
  if (delta) {
    const TD* d = delta + (size_t)src * hidden;
    float4 dv[PER / 4];
#pragma unroll
    for (int q = 0; q < PER / 4; ++q) dv[q] = load4(d + 4 * (q * nt + tid));
#pragma unroll
    for (int q = 0; q < PER / 4; ++q) { v[q].x += dv[q].x; v[q].y += dv[q].y; v[q].z += dv[q].z; v[q].w += dv[q].w; }
  }
  float ss = 0.f;
#pragma unroll
  for (int q = 0; q < PER / 4; ++q) {
    if (update) store4(r + 4 * (q * nt + tid), v[q]);
    ss += v[q].x * v[q].x + v[q].y * v[q].y + v[q].z * v[q].z + v[q].w * v[q].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TO* o = out + (size_t)i * hidden;
#pragma unroll
  for (int q = 0; q < PER / 4; ++q)
    store4(o + 4 * (q * nt + tid), make_float4(v[q].x * inv * w[q].x, v[q].y * inv * w[q].y, v[q].z * inv * w[q].z, v[q].w * inv * w[q].w));
}

}  // namespace lb

LB_EXPORT int lb_add_rmsnorm(void* out, int out_dtype, float* residual, const void* delta,
                             int delta_dtype, const float* weight, const int* rows, int num_rows,
                             int hidden, float eps, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && lb::valid_dtype(delta_dtype), "add_rmsnorm: bad dtype");
  LB_CHECK_ARG(num_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", num_rows, hidden);
  if (num_rows == 0) return 0;
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const bool vec4 = (hidden % 4 == 0);
  // rows of 4, 8 or 16 elements a thread (a whole number of warps, 64 to 1024 threads), 16-byte aligned operands:
  // the one-pass kernel.  8 elements a thread where that works (4096 -> 512 threads, 5120 -> 640), else 4, else 16.
  int per = 0;
  for (int cand : {8, 4, 16}) {
    if (hidden % cand == 0 && (hidden / cand) % 32 == 0 && hidden / cand >= 64 && hidden / cand <= 1024) { per = cand; threads = hidden / cand; break; }
  }
  const bool aligned = ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)weight % 16 == 0);
  LB_DISPATCH_DTYPE(delta_dtype, TD, {
    LB_DISPATCH_DTYPE(out_dtype, TO, {
      if (aligned && (per == 4 || per == 8 || per == 16)) {
        if (per == 4)
          lb::launch(lb::add_rmsnorm_row_kernel<TD, TO, 4>, dim3(num_rows), dim3(threads), 0, stream,
                     (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
        else if (per == 8)
          lb::launch(lb::add_rmsnorm_row_kernel<TD, TO, 8>, dim3(num_rows), dim3(threads), 0, stream,
                     (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
        else
          lb::launch(lb::add_rmsnorm_row_kernel<TD, TO, 16>, dim3(num_rows), dim3(threads), 0, stream,
                     (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
      } else if (vec4)
        lb::launch(lb::add_rmsnorm_kernel<TD, TO, 4>, dim3(num_rows), dim3(threads), 0, stream,
                   (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
      else
        lb::launch(lb::add_rmsnorm_kernel<TD, TO, 1>, dim3(num_rows), dim3(threads), 0, stream,
                   (TO*)out, residual, (const TD*)delta, weight, rows, hidden, eps);
    })
  })
  LB_CHECK_LAUNCH("add_rmsnorm");
  return 0;
}
