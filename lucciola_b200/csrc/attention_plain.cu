// Plain paged attention: one warp per (query token, query head), keys visited
// in their order in the sequence, everything in 32-bit.  It serves the 32-bit
// path of the engine and is the kernel beside which the fast bfloat16 kernels
// are tested.  It takes any head size up to 512, any head counts and group
// sizes, any page size, whole prompts, portions and single decoded tokens alike.
//
// Formulas as in lucciola: kv head = q head / (nq / nkv)
// (src/kernels/attention_paged.cu:68), score = (q . k) * scale, key j allowed
// iff j <= pos (src/kernels/flash_attention.cu:183-225), online softmax with
// m, l, o and out = o / l (src/kernels/flash_attention.cu:246-298, 311-347).
// A sliding window, which lucciola does not have, adds j > pos - window.
// Keys outside the allowed range are never read, so what a reused page still
// holds cannot reach a sum.
#include "common.cuh"

namespace lb {

struct PlainAttnParams {
  const void* q; void* out; const void* k_cache; const void* v_cache;
  const int* positions; const int* token_seq; const int* block_table;
  int num_q_heads, num_kv_heads, head_dim, page_size, max_pages, window;
  float scale;
};

template <typename T, int DPL>
__global__ void plain_attention_kernel(PlainAttnParams p) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int t = blockIdx.y;
  const int h = blockIdx.x * nwarps + warp;
  if (h >= p.num_q_heads) return;
  const int d = p.head_dim;
  const int kvh = h / (p.num_q_heads / p.num_kv_heads);
  float* qs = smem + (size_t)warp * d;
  const T* q = (const T*)p.q + ((size_t)t * p.num_q_heads + h) * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_f32(q[i]);
  __syncwarp();

  const int pos = p.positions[t];
  const int* bt = p.block_table + (size_t)p.token_seq[t] * p.max_pages;
  const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const T* kc = (const T*)p.k_cache;
  const T* vc = (const T*)p.v_cache;

  float m = -INFINITY, l = 0.f;
  float o[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = 0.f;

  for (int base = lo; base <= pos; base += 32) {
    const int j = base + lane;
    const bool valid = j <= pos;
    long long off = -1;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[j / p.page_size];
      if (page >= 0) {
        off = (((long long)page * p.num_kv_heads + kvh) * p.page_size + (j % p.page_size)) * d;
        const T* k = kc + off;
        float acc = 0.f;
        for (int i = 0; i < d; ++i) acc += qs[i] * to_f32(k[i]);
        s = acc * p.scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float pj = (off >= 0) ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] *= alpha;
    const int n = min(32, pos - base + 1);
    for (int jj = 0; jj < n; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const long long voff = __shfl_sync(0xffffffffu, off, jj);
      if (voff < 0) continue;  // uniform over the warp
      const T* v = vc + voff;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int dim = lane + 32 * i;
        if (dim < d) o[i] += pv * to_f32(v[dim]);
      }
    }
    m = m_new;
  }
  T* out = (T*)p.out + ((size_t)t * p.num_q_heads + h) * d;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int dim = lane + 32 * i;
    if (dim < d) out[dim] = from_f32<T>(o[i] * inv);
  }
}

template <typename T>
int launch_plain(const PlainAttnParams& p, int num_tokens, cudaStream_t stream) {
  const int warps = 4;
  dim3 grid((p.num_q_heads + warps - 1) / warps, num_tokens);
  const size_t smem = (size_t)warps * p.head_dim * sizeof(float);
  const int dpl = (p.head_dim + 31) / 32;
  if (dpl <= 1) launch(plain_attention_kernel<T, 1>, grid, dim3(warps * 32), smem, stream, p);
  else if (dpl <= 2) launch(plain_attention_kernel<T, 2>, grid, dim3(warps * 32), smem, stream, p);
  else if (dpl <= 4) launch(plain_attention_kernel<T, 4>, grid, dim3(warps * 32), smem, stream, p);
  else if (dpl <= 8) launch(plain_attention_kernel<T, 8>, grid, dim3(warps * 32), smem, stream, p);
  else launch(plain_attention_kernel<T, 16>, grid, dim3(warps * 32), smem, stream, p);
  return 0;
}

}  // namespace lb

LB_EXPORT int lb_attention_plain(int dtype, const void* q, void* out, const void* k_cache,
                                 const void* v_cache, const int* positions, const int* token_seq,
                                 const int* block_table, int num_tokens, int num_q_heads,
                                 int num_kv_heads, int head_dim, int page_size, int max_pages,
                                 int window, float scale, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "attention_plain: bad dtype %d", dtype);
  LB_CHECK_ARG(head_dim > 0 && head_dim <= 512, "attention_plain: head_dim %d not in 1..512", head_dim);
  LB_CHECK_ARG(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0,
               "attention_plain: %d query heads are not a multiple of %d kv heads", num_q_heads,
               num_kv_heads);
  LB_CHECK_ARG(page_size > 0 && max_pages > 0 && window >= 0, "attention_plain: bad page size or window");
  LB_CHECK_ARG(num_tokens <= 65535, "attention_plain: at most 65535 tokens a step, got %d", num_tokens);
  if (num_tokens == 0) return 0;
  lb::PlainAttnParams p;
  p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.token_seq = token_seq; p.block_table = block_table;
  p.num_q_heads = num_q_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim;
  p.page_size = page_size; p.max_pages = max_pages; p.window = window; p.scale = scale;
  LB_DISPATCH_DTYPE(dtype, T, { lb::launch_plain<T>(p, num_tokens, stream); })
  LB_CHECK_LAUNCH("attention_plain");
  return 0;
}
