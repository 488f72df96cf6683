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

}  // namespace lb

LB_EXPORT int lb_add_rmsnorm(void* out, int out_dtype, float* residual, const void* delta,
                             int delta_dtype, const float* weight, const int* rows, int num_rows,
                             int hidden, float eps, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && lb::valid_dtype(delta_dtype), "add_rmsnorm: bad dtype");
  LB_CHECK_ARG(num_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", num_rows, hidden);
  if (num_rows == 0) return 0;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const bool vec4 = (hidden % 4 == 0);
  LB_DISPATCH_DTYPE(delta_dtype, TD, {
    LB_DISPATCH_DTYPE(out_dtype, TO, {
      if (vec4)
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
