// Per-head RMSNorm of q and k, rotary position encoding, and the write of the
// new keys and values into their pages: one launch for what lucciola runs as
// two norms (src/qwen.cc:617-632), two rotations (src/qwen.cc:635-644,
// src/kernels/rope.cu:28-60) and the cache append
// (src/kernels/attention_paged.cu:26-44).
//
// Order as in the reference: norm over the head (weight [d] shared by all
// heads), then the rotation of the pairs (i, i + rot/2) by pos * inv_freq[i]
// ("NeoX" halves), then the write.  v is copied unchanged.  All arithmetic is
// 32-bit; the angle is one 32-bit product of the position and a host-made
// table entry, so a plain implementation that uses the same table gets the
// same angle.
//
// Page layout of one cache layer: [page][kv_head][slot][d].
#include "common.cuh"

#include <type_traits>

namespace lb {

struct RopeKvParams {
  const void* q_in; const void* k_in; const void* v_in;
  long long q_stride, k_stride, v_stride;   // elements between token rows
  void* q_out;                               // [T, nq, d]
  void* k_out; void* v_out;                  // optional [T, nkv, d] (when no cache is given)
  void* k_cache; void* v_cache;              // optional pools
  const int* positions; const int* token_seq; const int* block_table;
  const float* q_norm_w; const float* k_norm_w; const float* inv_freq;
  int num_q_heads, num_kv_heads, head_dim, rot_dim, page_size, max_pages;
  float eps;
};

template <typename T>
__global__ void rope_kv_kernel(RopeKvParams p) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int d = p.head_dim, half = p.rot_dim >> 1;
  float* buf = smem + (size_t)warp * d;
  const int pos = p.positions[t];
  const int total_heads = p.num_q_heads + 2 * p.num_kv_heads;

  // One head per warp: the grid's second dimension covers the heads.
  for (int h = blockIdx.y * nwarps + warp; h < total_heads; h += gridDim.y * nwarps) {
    const int kind = h < p.num_q_heads ? 0 : (h < p.num_q_heads + p.num_kv_heads ? 1 : 2);
    const int hh = kind == 0 ? h : (kind == 1 ? h - p.num_q_heads : h - p.num_q_heads - p.num_kv_heads);
    const T* src = kind == 0 ? (const T*)p.q_in + (size_t)t * p.q_stride + (size_t)hh * d
                 : kind == 1 ? (const T*)p.k_in + (size_t)t * p.k_stride + (size_t)hh * d
                             : (const T*)p.v_in + (size_t)t * p.v_stride + (size_t)hh * d;
    T* dst = nullptr;
    if (kind == 0) {
      dst = (T*)p.q_out + ((size_t)t * p.num_q_heads + hh) * d;
    } else if (p.k_cache) {
      const int seq = p.token_seq[t];
      const int page = p.block_table[(size_t)seq * p.max_pages + pos / p.page_size];
      const int slot = pos % p.page_size;
      if (page >= 0) {
        T* pool = (T*)(kind == 1 ? p.k_cache : p.v_cache);
        dst = pool + (((size_t)page * p.num_kv_heads + hh) * p.page_size + slot) * d;
      }
    } else {
      T* o = (T*)(kind == 1 ? p.k_out : p.v_out);
      if (o) dst = o + ((size_t)t * p.num_kv_heads + hh) * d;
    }
    if (dst == nullptr) continue;  // uniform over the warp

    if (kind == 2) {
      for (int i = lane; i < d; i += 32) dst[i] = src[i];
      continue;
    }
    const float* w = kind == 0 ? p.q_norm_w : p.k_norm_w;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float x = to_f32(src[i]);
      buf[i] = x;
      ss += x * x;
    }
    __syncwarp();
    if (w) {
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)d + p.eps);
      // No rounding between norm and rotation: one rounding at the store.
      for (int i = lane; i < d; i += 32) buf[i] = buf[i] * inv * w[i];
      __syncwarp();
    }
    if (p.inv_freq) {
      for (int i = lane; i < half; i += 32) {
        const float angle = (float)pos * p.inv_freq[i];
        float s, c;
        sincosf(angle, &s, &c);
        const float x = buf[i], y = buf[i + half];
        dst[i] = from_f32<T>(x * c - y * s);
        dst[i + half] = from_f32<T>(x * s + y * c);
      }
      for (int i = p.rot_dim + lane; i < d; i += 32) dst[i] = from_f32<T>(buf[i]);
    } else {
      for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(buf[i]);
    }
    __syncwarp();
  }
}

// The same for bfloat16 heads of 64, 128 or 256 elements with the whole head rotated: a lane holds
// VEC = d / 32 consecutive elements in registers (one 4-, 8- or 16-byte access), lanes 0..15 the first
// half of the head and lanes 16..31 the second, so the partner of a pair is the lane 16 further on.
template <int VEC>
__global__ void rope_kv_vec_kernel(RopeKvParams p) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  constexpr int d = VEC * 32;
  const int pos = p.positions[t];
  const int total_heads = p.num_q_heads + 2 * p.num_kv_heads;
  typedef typename std::conditional<VEC == 2, uint32_t, typename std::conditional<VEC == 4, uint2, uint4>::type>::type Word;
  // The angles depend on the token and the lane only: one sine and cosine per element for all heads
  // this warp walks over.
  float cs[VEC], sn[VEC];
  if (p.inv_freq) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) sincosf((float)pos * p.inv_freq[(lane & 15) * VEC + i], &sn[i], &cs[i]);
  }
  // The token's page does not depend on the kernel ahead either (positions and block tables are the step's inputs).
  int page = -1;
  if (p.k_cache) page = p.block_table[(size_t)p.token_seq[t] * p.max_pages + pos / p.page_size];
  pdl_wait();                                   // what follows reads the q|k|v product
  // Four heads at a time: their loads are issued together, so that a warp keeps a kilobyte in flight
  // instead of 256 bytes.
  constexpr int UNR = 4;
  const int hstep = gridDim.y * nwarps;
  for (int h0 = blockIdx.y * nwarps + warp; h0 < total_heads; h0 += UNR * hstep) {
    Word raw[UNR];
    bf16* dsts[UNR];
    int kinds[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int h = h0 + u * hstep;
      dsts[u] = nullptr; kinds[u] = 2;
      if (h >= total_heads) continue;
      const int kind = h < p.num_q_heads ? 0 : (h < p.num_q_heads + p.num_kv_heads ? 1 : 2);
      const int hh = kind == 0 ? h : (kind == 1 ? h - p.num_q_heads : h - p.num_q_heads - p.num_kv_heads);
      const bf16* src = kind == 0 ? (const bf16*)p.q_in + (size_t)t * p.q_stride + (size_t)hh * d
                      : kind == 1 ? (const bf16*)p.k_in + (size_t)t * p.k_stride + (size_t)hh * d
                                  : (const bf16*)p.v_in + (size_t)t * p.v_stride + (size_t)hh * d;
      bf16* dst = nullptr;
      if (kind == 0) {
        dst = (bf16*)p.q_out + ((size_t)t * p.num_q_heads + hh) * d;
      } else if (p.k_cache) {
        if (page >= 0) {
          bf16* pool = (bf16*)(kind == 1 ? p.k_cache : p.v_cache);
          dst = pool + (((size_t)page * p.num_kv_heads + hh) * p.page_size + pos % p.page_size) * d;
        }
      } else {
        bf16* o = (bf16*)(kind == 1 ? p.k_out : p.v_out);
        if (o) dst = o + ((size_t)t * p.num_kv_heads + hh) * d;
      }
      dsts[u] = dst; kinds[u] = kind;
      if (dst) raw[u] = reinterpret_cast<const Word*>(src)[lane];
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      bf16* dst = dsts[u];
      if (dst == nullptr) continue;
      const int kind = kinds[u];
      if (kind == 2) { reinterpret_cast<Word*>(dst)[lane] = raw[u]; continue; }
      const bf16* e = reinterpret_cast<const bf16*>(&raw[u]);
      float x[VEC];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) { x[i] = __bfloat162float(e[i]); ss += x[i] * x[i]; }
      const float* w = kind == 0 ? p.q_norm_w : p.k_norm_w;
      if (w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)d + p.eps);
#pragma unroll
        for (int i = 0; i < VEC; ++i) x[i] = x[i] * inv * w[lane * VEC + i];
      }
      if (p.inv_freq) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
          // first half: x cos - y sin with y the partner; second half: x' sin + y' cos with x' the partner
          x[i] = lane < 16 ? x[i] * cs[i] - other * sn[i] : other * sn[i] + x[i] * cs[i];
        }
      }
      Word outw;
      bf16* o = reinterpret_cast<bf16*>(&outw);
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = __float2bfloat16_rn(x[i]);
      reinterpret_cast<Word*>(dst)[lane] = outw;
    }
  }
}

}  // namespace lb

LB_EXPORT int lb_rope_kv(int dtype, const void* q_in, const void* k_in, const void* v_in,
                         long long q_stride, long long k_stride, long long v_stride, void* q_out,
                         void* k_out, void* v_out, void* k_cache, void* v_cache,
                         const int* positions, const int* token_seq, const int* block_table,
                         const float* q_norm_w, const float* k_norm_w, const float* inv_freq,
                         int num_tokens, int num_q_heads, int num_kv_heads, int head_dim,
                         int rot_dim, int page_size, int max_pages, float eps,
                         cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "rope_kv: bad dtype %d", dtype);
  LB_CHECK_ARG(head_dim > 0 && head_dim <= 1024, "rope_kv: head_dim %d not in 1..1024", head_dim);
  LB_CHECK_ARG(rot_dim >= 0 && rot_dim <= head_dim && rot_dim % 2 == 0,
               "rope_kv: rotary size %d must be even and at most head_dim %d", rot_dim, head_dim);
  LB_CHECK_ARG(num_q_heads >= 0 && num_kv_heads >= 0, "rope_kv: bad head counts");
  LB_CHECK_ARG(k_cache == nullptr || (v_cache && block_table && token_seq && page_size > 0 && max_pages > 0),
               "rope_kv: a cache needs v pool, block table, token map and page size");
  if (num_tokens == 0) return 0;
  lb::RopeKvParams p;
  p.q_in = q_in; p.k_in = k_in; p.v_in = v_in;
  p.q_stride = q_stride; p.k_stride = k_stride; p.v_stride = v_stride;
  p.q_out = q_out; p.k_out = k_out; p.v_out = v_out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.positions = positions; p.token_seq = token_seq; p.block_table = block_table;
  p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.inv_freq = rot_dim > 0 ? inv_freq : nullptr;
  p.num_q_heads = num_q_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim;
  p.rot_dim = rot_dim; p.page_size = page_size; p.max_pages = max_pages; p.eps = eps;
  const int warps = 4;
  const size_t smem = (size_t)warps * head_dim * sizeof(float);
  // The register version: bfloat16, heads of 64 / 128 / 256, whole head rotated, every row 16-byte aligned.
  const int vec = head_dim / 32;
  const size_t word = (size_t)vec * 2;
  auto aligned = [&](const void* ptr, long long stride) { return ptr == nullptr || ((uintptr_t)ptr % word == 0 && (stride * 2) % (long long)word == 0); };
  const bool fast = dtype == LB_BF16 && (head_dim == 64 || head_dim == 128 || head_dim == 256) &&
                    (p.inv_freq == nullptr || rot_dim == head_dim) && aligned(q_in, q_stride) && aligned(k_in, k_stride) &&
                    aligned(v_in, v_stride) && aligned(q_out, head_dim) && aligned(k_out, head_dim) && aligned(v_out, head_dim) &&
                    aligned(k_cache, head_dim) && aligned(v_cache, head_dim);
  if (fast) {
    // With few tokens every head gets a warp of its own; with many a warp walks over several heads,
    // so that the grid stays near eight blocks per SM instead of tens of thousands of tiny ones.
    const int total_heads = num_q_heads + 2 * num_kv_heads;
    int head_blocks = (total_heads + warps - 1) / warps;
    const int wanted = (1184 + num_tokens - 1) / num_tokens;
    if (head_blocks > wanted) head_blocks = wanted;
    if (head_blocks < 1) head_blocks = 1;
    dim3 grid(num_tokens, head_blocks);
    if (vec == 2) lb::launch(lb::rope_kv_vec_kernel<2>, grid, dim3(warps * 32), 0, stream, p);
    else if (vec == 4) lb::launch(lb::rope_kv_vec_kernel<4>, grid, dim3(warps * 32), 0, stream, p);
    else lb::launch(lb::rope_kv_vec_kernel<8>, grid, dim3(warps * 32), 0, stream, p);
    LB_CHECK_LAUNCH("rope_kv");
    return 0;
  }
  LB_DISPATCH_DTYPE(dtype, T, {
    const int total_heads = num_q_heads + 2 * num_kv_heads;
    int head_blocks = (total_heads + warps - 1) / warps;
    if (head_blocks > 65535) head_blocks = 65535;
    if (head_blocks < 1) head_blocks = 1;
    lb::launch(lb::rope_kv_kernel<T>, dim3(num_tokens, head_blocks), dim3(warps * 32), smem, stream, p);
  })
  LB_CHECK_LAUNCH("rope_kv");
  return 0;
}
