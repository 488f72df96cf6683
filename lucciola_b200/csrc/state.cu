// Per-request state of fixed size (the slots beside the paged cache): clearing the rows of requests
// that a step admits.  lucciola has no such state (its only per-request memory is the block table,
// include/sequence.h:41); mixers with a recurrent state need it zeroed when a request starts.
//
// The list of slots comes from device memory, so that the launch is the same whatever the list holds and
// can be part of a recorded CUDA graph: entry i names the row to clear, a negative entry names none.
#include "common.cuh"

namespace lb {

__global__ void zero_rows_kernel(unsigned char* __restrict__ base, long long row_bytes,
                                 const int* __restrict__ slots, int num_rows) {
  pdl_trigger();
  pdl_wait();
  const int slot = slots[blockIdx.x];
  if (slot < 0 || slot >= num_rows) return;
  unsigned char* row = base + (size_t)slot * (size_t)row_bytes;
  if ((row_bytes & 15) == 0 && ((uintptr_t)base & 15) == 0) {
    uint4* r16 = reinterpret_cast<uint4*>(row);
    const long long n = row_bytes >> 4;
    for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.y * blockDim.x)
      r16[i] = make_uint4(0u, 0u, 0u, 0u);
  } else {
    for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < row_bytes; i += (long long)gridDim.y * blockDim.x)
      row[i] = 0;
  }
}

}  // namespace lb

// base: [num_rows, row_bytes] bytes; slots: int32 [count] on the device, negative entries are skipped.
LB_EXPORT int lb_zero_rows(void* base, long long row_bytes, int num_rows, const int* slots, int count,
                           cudaStream_t stream) {
  LB_CHECK_ARG(base && slots && row_bytes > 0 && num_rows > 0 && count >= 0, "zero_rows: bad arguments");
  if (count == 0) return 0;
  LB_CHECK_ARG(count <= 65535 * 32, "zero_rows: too many slots (%d)", count);
  const long long units = (row_bytes & 15) == 0 ? row_bytes >> 4 : row_bytes;
  long long by = (units + 256 * 8 - 1) / (256 * 8);
  if (by < 1) by = 1;
  if (by > 64) by = 64;
  lb::launch(lb::zero_rows_kernel, dim3(count, (unsigned)by), dim3(256), 0, stream, (unsigned char*)base, row_bytes, slots,
             num_rows);
  LB_CHECK_LAUNCH("zero_rows");
  return 0;
}
