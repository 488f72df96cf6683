// Samplers over 32-bit logits [R, V]: greedy (lowest index wins a tie;
// src/kernels/argmax.cu:8-59 of lucciola takes the maximum of bfloat16 logits
// with a tie rule that depends on the thread layout) and temperature sampling.
//
// Temperature sampling draws from softmax(logits / T) by the Gumbel-max rule:
// token = argmax_i (logits[i] / T - log(-log(u_i))).  u_i comes from a
// counter-based hash of (key of the request, index of the generated token, i),
// so the token does not depend on what else is in the batch or on how the
// prompt was cut.  T == 0 is greedy.
#include "common.cuh"

namespace lb {

__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

// The top 23 bits of a hash as a number strictly inside (0, 1): (b + 0.5) / 2^23.  b + 0.5 has at most 24
// significant bits, so every value is exact in float32; the smallest is 2^-24 and the largest 1 - 2^-24.  (With
// 24 bits the largest sum, 16777215.5, would round to 2^24 and give exactly 1, whose score is +infinity.)
__host__ __device__ __forceinline__ float bits_to_uniform(unsigned int bits23) {
  return ((float)bits23 + 0.5f) * (1.0f / 8388608.0f);
}

// Uniform in (0, 1) with 23 bits.
__host__ __device__ __forceinline__ float hash_uniform(unsigned long long key, unsigned int counter,
                                                       unsigned int i) {
  unsigned long long x = mix64(key + 0x9E3779B97F4A7C15ull * (unsigned long long)(counter + 1u));
  x = mix64(x ^ (0xD6E8FEB86659FD93ull * (unsigned long long)(i + 1u)));
  return bits_to_uniform((unsigned int)(x >> 41));
}

__global__ void sample_kernel(int* __restrict__ tokens, const float* __restrict__ logits,
                              const float* __restrict__ temperature,
                              const unsigned long long* __restrict__ keys,
                              const int* __restrict__ counters, int vocab) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const float temp = temperature ? temperature[r] : 0.f;
  const bool greedy = !(temp > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / temp;
  const unsigned long long key = keys ? keys[r] : 0ull;
  const unsigned int counter = counters ? (unsigned int)counters[r] : 0u;

  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float s = row[i];
    if (!greedy) s = s * inv_t - logf(-logf(hash_uniform(key, counter, (unsigned int)i)));
    if (s > bv || (s == bv && i < bi)) { bv = s; bi = i; }
  }
  // A NaN never compares greater, so a row of NaNs yields index 0x7fffffff;
  // map it to 0 at the end.
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = blockDim.x >> 5;
    bv = lane < nwarps ? best_v[lane] : -INFINITY;
    bi = lane < nwarps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) tokens[r] = bi == 0x7fffffff ? 0 : bi;
  }
}

}  // namespace lb

LB_EXPORT int lb_sample(int* tokens, const float* logits, const float* temperature,
                        const unsigned long long* keys, const int* counters, int num_rows, int vocab,
                        cudaStream_t stream) {
  LB_CHECK_ARG(num_rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", num_rows, vocab);
  if (num_rows == 0) return 0;
  const int threads = vocab >= 8192 ? 1024 : (vocab >= 1024 ? 256 : 64);
  lb::launch(lb::sample_kernel, dim3(num_rows), dim3(threads), 0, stream, tokens, logits, temperature, keys, counters, vocab);
  LB_CHECK_LAUNCH("sample");
  return 0;
}

// The same hash on the host, for tests and for a plain restatement.
LB_EXPORT float lb_hash_uniform(unsigned long long key, unsigned int counter, unsigned int i) {
  return lb::hash_uniform(key, counter, i);
}

LB_EXPORT float lb_bits_to_uniform(unsigned int bits23) { return lb::bits_to_uniform(bits23 & 0x7FFFFFu); }
