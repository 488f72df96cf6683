// Embedding gather: out[t, :] = table[ids[t], :], written in the type of the
// residual stream (32-bit).  Reference behaviour: src/kernels/embedding.cu:22-38
// of lucciola copies the row unchanged, without scaling; an id outside the
// table reads row 0 there.  Here ids are validated on the host before a step;
// the clamp below only keeps a bad id from reading outside the table.
#include "common.cuh"

namespace lb {

template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const int* __restrict__ ids,
                                 const TW* __restrict__ table, int hidden, int vocab) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const TW* row = table + (size_t)id * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(row[i]);
}

}  // namespace lb

LB_EXPORT int lb_embedding(float* out, const int* ids, const void* table, int table_dtype,
                           int num_tokens, int hidden, int vocab, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(table_dtype), "embedding: bad table dtype %d", table_dtype);
  LB_CHECK_ARG(num_tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes T=%d H=%d V=%d",
               num_tokens, hidden, vocab);
  if (num_tokens == 0) return 0;
  int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
  LB_DISPATCH_DTYPE(table_dtype, TW, {
    lb::launch(lb::embedding_kernel<TW>, dim3(num_tokens), dim3(threads), 0, stream, out, ids, (const TW*)table, hidden, vocab);
  })
  LB_CHECK_LAUNCH("embedding");
  return 0;
}
