// Plain matrix product Y[M,N] = X[M,K] . W[N,K]^T on the ordinary 32-bit
// pipes: weights in the layout of the checkpoint ([out, in], row-major), one
// 32-bit accumulator per output element, k visited in increasing order by a
// single thread (include/kernels/linear.h:8-16 and src/kernels/linear.cu:24-55
// of lucciola define the same contraction, one thread per element without
// tiling).  Because of the fixed order an element's value does not depend on
// how many rows the batch has or where its row lies.  It is the product of
// the 32-bit path (no reduced-precision matrix mode: FFMA only) and the
// fallback for shapes the tensor-core kernel refuses.  X, W and Y may each be
// 32-bit or bfloat16.
#include "common.cuh"

namespace lb {

constexpr int PG_BM = 64, PG_BN = 64, PG_BK = 16;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(TY* __restrict__ y, const TX* __restrict__ x, const TW* __restrict__ w, int M, int N,
                  int K, long long ldx, long long ldy) {
  __shared__ float xs[PG_BK][PG_BM + 4];
  __shared__ float ws[PG_BK][PG_BN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * PG_BM, n0 = blockIdx.x * PG_BN;
  const int tr = tid / 16, tc = tid % 16;  // thread owns rows tr*4.., cols tc*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += PG_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;     // 0..1023
      const int r = idx / PG_BK, c = idx % PG_BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      xs[c][r] = (gm < M && gk < K) ? to_f32(x[(size_t)gm * ldx + gk]) : 0.f;
      ws[c][r] = (gn < N && gk < K) ? to_f32(w[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < PG_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][tr * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tc * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + tr * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tc * 4 + j;
      if (gn < N) y[(size_t)gm * ldy + gn] = from_f32<TY>(acc[i][j]);
    }
  }
}

template <typename TX, typename TW, typename TY>
void launch_gemm_plain(void* y, const void* x, const void* w, int M, int N, int K, long long ldx,
                       long long ldy, cudaStream_t stream) {
  dim3 grid((N + PG_BN - 1) / PG_BN, (M + PG_BM - 1) / PG_BM);
  launch(gemm_plain_kernel<TX, TW, TY>, grid, dim3(256), 0, stream, (TY*)y, (const TX*)x, (const TW*)w, M, N, K, ldx, ldy);
}

}  // namespace lb

LB_EXPORT int lb_gemm_plain(void* y, int y_dtype, const void* x, int x_dtype, const void* w,
                            int w_dtype, int M, int N, int K, long long ldx, long long ldy,
                            cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(y_dtype) && lb::valid_dtype(x_dtype) && lb::valid_dtype(w_dtype),
               "gemm_plain: bad dtype");
  LB_CHECK_ARG(M >= 0 && N > 0 && K > 0 && ldx >= K && ldy >= N, "gemm_plain: bad sizes M=%d N=%d K=%d", M, N, K);
  LB_CHECK_ARG((M + lb::PG_BM - 1) / lb::PG_BM <= 65535, "gemm_plain: too many rows (%d)", M);
  if (M == 0) return 0;
  LB_DISPATCH_DTYPE(x_dtype, TX, {
    LB_DISPATCH_DTYPE(w_dtype, TW, {
      LB_DISPATCH_DTYPE(y_dtype, TY, {
        lb::launch_gemm_plain<TX, TW, TY>(y, x, w, M, N, K, ldx, ldy, stream);
      })
    })
  })
  LB_CHECK_LAUNCH("gemm_plain");
  return 0;
}
