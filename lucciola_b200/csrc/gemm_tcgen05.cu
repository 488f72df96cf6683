// Matrix product on the 5th-generation tensor cores: Y[M,N] = X[M,K] . W[N,K]^T, bfloat16 in,
// 32-bit accumulation in tensor memory, bfloat16 or 32-bit out.  This is the product behind every
// linear map of the bfloat16 path (q|k|v, o, gate|up, down, the output head); lucciola computes
// the same contraction with one thread per output element (src/kernels/linear.cu:24-55).
//
// Orientation.  Weight rows go on the 128 lanes of the accumulator (the M side of tcgen05.mma),
// tokens on its columns (the N side, 16..256).  One kernel therefore serves decode (a handful of
// tokens: a 128 x 16 tile, the weights stream through once) and prefill (128 x 256 tiles).
//
// Pipeline of one CTA (192 threads):
//   warp 0      producer: one thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle)
//               of a 128 x 64 weight tile and a BT x 64 token tile per stage into a ring of stages
//   warp 1      one thread issues tcgen05.mma (kind::f16, M=128, N=BT, K=16) four times per stage on
//               shared-memory descriptors; tcgen05.commit frees the stage, and at the end signals
//               the epilogue; this warp also allocates and frees tensor memory
//   warps 2..5  epilogue: tcgen05.ld (32 lanes x 32 bit) of the accumulator, conversion, stores
// K may be split over gridDim.z.  With up to 8 splits the CTAs of a tile form a thread-block cluster:
// each leaves its 32-bit partial tile in its own shared memory, and after a cluster barrier every CTA
// adds, for its share of the tile's columns, the partials of all CTAs in the order of the splits,
// reading its peers' shared memory directly (ld.shared::cluster).  With more splits (or when asked
// to) the partials go through a workspace in global memory and the CTA that finishes last for a
// tile adds them, again in the order of the splits.  Either way the result does not depend on timing.
//
// With more than 256 tokens (and from 65 or 129 tokens on for products with many features, see lb_gemm_tcgen05) a second
// kernel takes over (gemm_tcgen05_prefill_kernel): tokens on the lanes, features on
// the columns, persistent CTAs over tiles of 128 tokens x up to 256 features with two accumulators, so that the epilogue
// of a tile runs under the MMAs of the next; from 1024 tokens on as pairs of CTAs on tiles of 256 x 256 (tcgen05
// cta_group::2: each CTA stages its 128 tokens and half of the weight rows, the first CTA issues the MMAs for both).
//
// Every wait on an mbarrier is bounded: when a wait gives up the CTA records a code in a device
// flag, stops, waits (bounded) for its loads in flight, frees its tensor memory and returns.
// K must be a multiple of 8 and X, W 16-byte aligned (TMA strides); M, N, K tails are handled by
// TMA's zero fill on loads and by bounds checks on stores.
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace lb {

// ---- device error flag (shared by kernels with bounded waits) ---------------------------------
__device__ int g_device_error = 0;

constexpr int BM = 128;          // weight rows of a tile (lanes of the accumulator)
constexpr int BK = 64;           // k extent of a stage: 64 bfloat16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr unsigned long long WAIT_CYCLES = 4000000000ull;   // about two seconds

enum : int { ERR_FULL_WAIT = 101, ERR_EMPTY_WAIT = 102, ERR_ACCUM_WAIT = 103 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the limit (in clock cycles) passed or another role of the CTA gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          unsigned long long limit = WAIT_CYCLES) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag) return false;
      if ((unsigned long long)(clock64() - t0) > limit) {
        *abort_flag = code;
        atomicCAS(&g_device_error, 0, code);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// The same from a CTA of a pair (cta_group::2): the barrier may lie in the other CTA of the pair (a shared::cluster
// address), which is how both CTAs' bytes are counted on the barrier of the CTA that issues the pair's MMAs.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, groups
// of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// One MMA of a CTA pair: 256 rows (128 from each CTA's shared memory), n columns (half of the B rows from each CTA).
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The commit of a pair arrives on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__host__ __device__ constexpr uint32_t umma_idesc_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// What the epilogue of the q|k|v product does instead of storing its tile when the tile is one head (128 weight
// rows = a head of 128): per-head RMSNorm of query and key heads, the rotation, queries into the attention layout,
// keys and values into their cache page.  The formulas are those of rope_kv.cu (src/qwen.cc:600-663 of lucciola),
// taken from the 32-bit accumulator instead of a rounded bfloat16 copy.  The layout mirrors LbHeadEpilogue in ops.py.
struct HeadEpilogue {
  int on;
  int num_q_heads, num_kv_heads, page_size, max_pages;
  float eps;
  const int* positions;       // [M]
  const int* token_seq;       // [M] row of the block table
  const int* block_table;     // [S, max_pages]; a negative page: the token's key and value are written nowhere
  const float* q_norm_w;      // [128] or null
  const float* k_norm_w;      // [128] or null
  const float* inv_freq;      // [64] or null (no rotation)
  bf16* q_out;                // [M, num_q_heads, 128]
  bf16* k_cache;              // [pages, num_kv_heads, page_size, 128]
  bf16* v_cache;
};

// The sum over the cluster's CTAs of the float at `addr` of each one's shared memory, in the order of their ranks.
// All loads are issued before the first is used (a load from another SM's shared memory takes several hundred cycles).
__device__ __forceinline__ float cluster_sum_f32(uint32_t addr, int splits) {
  float v[8];
#pragma unroll
  for (int z = 0; z < 8; ++z) v[z] = z < splits ? ld_cluster_f32(addr, (uint32_t)z) : 0.f;
  float acc = 0.f;
#pragma unroll
  for (int z = 0; z < 8; ++z) acc += v[z];
  return acc;
}

// What the epilogue of the o and down products does instead of storing their tile: the residual add and the first
// half of the RMSNorm that follows (lucciola: add_kernel, a copy and rmsnorm_forward_kernel, src/qwen.cc:731-759).
// residual += y; out = residual * norm_w, rounded, WITHOUT the row's factor rsqrt(mean(residual^2) + eps); and the sum
// of squares of the new residual over this tile's features goes to sumsq[row][tile].  The product that reads `out`
// multiplies its 32-bit sums by the row's factor (RowScale): a row's factor commutes with a linear map.
struct AddNormEpilogue {
  int on;
  int tiles;                  // 128-feature tiles of a row (columns of sumsq)
  float* residual;            // [M, N] float32
  const float* norm_w;        // [N]
  bf16* out;                  // [M, N]
  float* sumsq;               // [M, tiles]
};

// The input rows of this product lack their norm's factor: row m of the result is multiplied by
// rsqrt(sum_t sumsq[m][t] * inv_width + eps) (the tiles are added in their order).  Mirrors LbRowScale in ops.py.
struct RowScale {
  int on;
  int tiles;
  const float* sumsq;         // [M, tiles]
  float inv_width, eps;
};

__device__ __forceinline__ float row_factor(const RowScale& rs, int m) {
  const float* src = rs.sumsq + (size_t)m * rs.tiles;
  float total = 0.f;
  for (int t0 = 0; t0 < rs.tiles; t0 += 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = t0 + u < rs.tiles ? __ldcg(src + t0 + u) : 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) total += v[u];
  }
  return rsqrtf(total * rs.inv_width + rs.eps);
}

// The same by a whole warp: lane l adds the tiles l, l + 32, ..., then the lanes add up in a fixed pattern.
__device__ __forceinline__ float row_factor_warp(const RowScale& rs, int m, int lane) {
  const float* src = rs.sumsq + (size_t)m * rs.tiles;
  float part = 0.f;
  for (int t = lane; t < rs.tiles; t += 32) part += __ldcg(src + t);
  return rsqrtf(warp_sum(part) * rs.inv_width + rs.eps);
}

struct GemmParams {
  HeadEpilogue he = {};   // off unless a caller fills it in
  AddNormEpilogue an = {};
  RowScale rs = {};
  void* y;              // [M, N] output, row stride ldy
  float* workspace;     // [splits, M, N] partials (split-K only)
  int* counters;        // one per output tile, zero between launches (split-K only)
  int M, N, K;
  long long ldy;
  int out_dtype;        // LB_F32 or LB_BF16
  int cluster;          // > 0: the splits of a tile form a thread-block cluster of this size and add
                        // their partials through distributed shared memory (no workspace, no counters)
  int swiglu;           // 1: the weight rows alternate in blocks of 64 between "gate" and "up" rows of the same 64
                        // features; the output has N/2 columns and holds silu(gate) * up (computed in 32-bit)
  unsigned long long wait_cycles = WAIT_CYCLES;   // after this many clock cycles a wait on a barrier gives up
  int skip_loads = 0;   // tests of the give-up path only: the producer requests nothing, so the first wait runs out
};

// silu(g) * u; the quotient by the fast division (2 ulp), the result is rounded to bfloat16 or summed with like terms afterwards
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

template <int BT>
__host__ __device__ constexpr int tmem_cols() { return BT < 32 ? 32 : BT; }

template <int BT, int STAGES>
struct SmemLayout {
  static constexpr int W_BYTES = BM * BK * 2;
  static constexpr int X_BYTES = BT * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16;
};

template <int BT, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
  using L = SmemLayout<BT, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // The swizzled tiles need 1024-byte alignment.
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t accum_bar = bar_base + 8u * (2 * STAGES);
  uint32_t* tmem_slot = (uint32_t*)(smem + L::BAR_OFFSET + (2 * STAGES + 1) * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* last_flag = (int*)(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BT;
  const int splits = gridDim.z, split = blockIdx.z;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_begin = (int)((long long)kb_total * split / splits);
  const int kb_end = (int)((long long)kb_total * (split + 1) / splits);
  const int num_kb = kb_end - kb_begin;

  pdl_trigger();
  const int early = num_kb < STAGES ? num_kb : STAGES;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // This thread is also the producer.  The weights do not depend on the kernel before this one:
    // the first ring of weight tiles is requested at once, before the rest of the CTA is even set up.
    for (int i = 0; i < early && !p.skip_loads; ++i) {
      mbar_expect_tx(full_bar(i), L::STAGE_BYTES);
      tma_load_2d(smem_base + i * L::STAGE_BYTES, &map_w, (kb_begin + i) * BK, n0, full_bar(i));
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols<BT>()) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;
  float an_w = 0.f, an_before[4] = {0.f, 0.f, 0.f, 0.f};       // of the epilogue that adds to the residual stream
  float he_w = 1.f, he_freq = 0.f;                             // of the epilogue that finishes heads

  if (warp == 0) {
    // ---- producer --------------------------------------------------------------------------
    if (lane == 0 && !p.skip_loads) {
      int issued = 0;
      // The token tiles follow the early weight tiles when the kernel before this one has completed.
      pdl_wait();
      for (int i = 0; i < early; ++i)
        tma_load_2d(smem_base + i * L::STAGE_BYTES + L::W_BYTES, &map_x, (kb_begin + i) * BK, m0, full_bar(i));
      issued = early;
      for (int i = early; i < num_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t parity = ((i / STAGES) & 1) ^ 1;          // the stage's earlier use has been consumed
        if (!mbar_wait(empty_bar(s), parity, abort_flag, ERR_EMPTY_WAIT, p.wait_cycles)) break;
        mbar_expect_tx(full_bar(s), L::STAGE_BYTES);
        const uint32_t dst = smem_base + s * L::STAGE_BYTES;
        const int k = (kb_begin + i) * BK;
        tma_load_2d(dst, &map_w, k, n0, full_bar(s));
        tma_load_2d(dst + L::W_BYTES, &map_x, k, m0, full_bar(s));
        issued = i + 1;
      }
      if (*abort_flag) {
        // Give the loads in flight time to land before this CTA's shared memory is given away.
        for (int i = max(0, issued - STAGES); i < issued; ++i) {
          const long long t0 = clock64();
          while (!mbar_try_wait(full_bar(i % STAGES), (i / STAGES) & 1) &&
                 (unsigned long long)(clock64() - t0) < WAIT_CYCLES / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---- tensor-core issue ---------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BT);
      bool ok = true;
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(full_bar(s), (i / STAGES) & 1, abort_flag, ERR_FULL_WAIT, p.wait_cycles);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_base + s * L::STAGE_BYTES;
        const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + L::W_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // 16 bfloat16 = 32 bytes further along k inside the swizzled row: +2 in the address field
          umma_f16(tmem_acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (i | k) != 0);
        }
        umma_commit(empty_bar(s));
      }
      if (ok) umma_commit(accum_bar);
    }
  } else {
    // ---- epilogue: warps 2..5, lanes (warp % 4) * 32 .. + 31 of the accumulator ----------------
    const int quarter = warp & 3;
    const int n = n0 + quarter * 32 + lane;
    // A norm weight is read once a step: a miss all the way to memory.  Asked for here, it has arrived when the
    // reduction at the end wants it.
    if (p.an.on) an_w = n < p.N ? p.an.norm_w[n] : 0.f;
    if (p.he.on) {
      const int head = n0 / BM, nl = quarter * 32 + lane;
      const float* w = head < p.he.num_q_heads ? p.he.q_norm_w : (head < p.he.num_q_heads + p.he.num_kv_heads ? p.he.k_norm_w : nullptr);
      const bool rotated = head < p.he.num_q_heads + p.he.num_kv_heads;
      he_w = w ? w[nl] : 1.f;
      he_freq = (rotated && p.he.inv_freq) ? p.he.inv_freq[nl & 63] : 0.f;
    }
    // The accumulator is ready when the whole main loop is through: twice the limit of one of its waits, so that a
    // wait of the main loop that runs out is what gets reported.
    mbar_wait(accum_bar, 0, abort_flag, ERR_ACCUM_WAIT, 2 * p.wait_cycles);
    // All four epilogue warps take the same path: agree on the outcome before any of them goes on.
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool ok = (*abort_flag == 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && p.an.on && p.cluster > 0) {
      // The residual values of the first tokens this CTA finishes, on their way while the tile goes to shared memory.
      pdl_wait();
      const int per = (BT + p.cluster - 1) / p.cluster, j0 = split * per, j1 = min(min((split + 1) * per, BT), p.M - m0);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        an_before[u] = (j0 + u < j1 && n < p.N) ? p.an.residual[(size_t)(m0 + j0 + u) * p.N + n] : 0.f;
    }
    if (ok) {
      const uint32_t taddr = tmem_acc + ((uint32_t)(quarter * 32) << 16);
      const bool direct = splits == 1;
      const bool via_cluster = (!direct && p.cluster > 0) || (direct && p.swiglu);   // the tile goes to shared memory first
      float* part = (direct || via_cluster) ? nullptr : p.workspace + (size_t)split * p.M * p.N;
      float* part_smem = reinterpret_cast<float*>(smem);          // [BT][128]; the stages are drained by now
      float* row_f = part_smem + BT * BM;                         // the rows' norm factors, when the input lacks them
      if (p.rs.on && direct) {
        // Eight threads a token, each adds every eighth block of the row (its loads are in flight together), then the
        // eight add up in a fixed pattern: one round trip to the L2 for 16 tokens.  (Waiting for the kernel before this
        // one any earlier, while the main loop runs, made the step slower, not faster: see the residual-add epilogue.)
        pdl_wait();
        const int t = threadIdx.x - 64, sub = t & 7;
        for (int jb = 0; jb < BT && m0 + jb < p.M; jb += 16) {
          const int j = jb + (t >> 3);
          float part_sum = 0.f;
          if (m0 + j < p.M) {
            const float* src = p.rs.sumsq + (size_t)(m0 + j) * p.rs.tiles;
            for (int i = sub; i < p.rs.tiles; i += 8) part_sum += __ldcg(src + i);
          }
          part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 4);
          part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 2);
          part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 1);
          if (sub == 0 && j < BT) row_f[j] = m0 + j < p.M ? rsqrtf(part_sum * p.rs.inv_width + p.rs.eps) : 0.f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
#pragma unroll 1
      for (int c = 0; c < BT; c += 16) {
        uint32_t r[16];
        tmem_ld16(taddr + c, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (via_cluster) {
#pragma unroll
          for (int j = 0; j < 16; ++j) part_smem[(c + j) * BM + quarter * 32 + lane] = __uint_as_float(r[j]);
        } else if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c + j;
            if (m < p.M) {
              const float v = (p.rs.on && direct) ? __uint_as_float(r[j]) * row_f[c + j] : __uint_as_float(r[j]);
              if (!direct) part[(size_t)m * p.N + n] = v;
              else if (p.out_dtype == LB_F32) ((float*)p.y)[(size_t)m * p.ldy + n] = v;
              else ((bf16*)p.y)[(size_t)m * p.ldy + n] = __float2bfloat16_rn(v);
            }
          }
        }
      }
      if (direct && p.swiglu) {
        // gate and up of a feature sit 64 lanes apart: pair them through shared memory
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int t = threadIdx.x - 64, f = t & 63;
        const int feature = (n0 >> 1) + f;
        if (feature < (p.N >> 1)) {
          for (int j = t >> 6; j < BT && m0 + j < p.M; j += 2) {
            const float rf = p.rs.on ? row_f[j] : 1.f;
            const float v = silu_mul(part_smem[j * BM + f] * rf, part_smem[j * BM + f + 64] * rf);
            if (p.out_dtype == LB_F32) ((float*)p.y)[(size_t)(m0 + j) * p.ldy + feature] = v;
            else ((bf16*)p.y)[(size_t)(m0 + j) * p.ldy + feature] = __float2bfloat16_rn(v);
          }
        }
      }
      if (!direct && !via_cluster) {
        // The CTA that arrives last for this tile adds the partials in the order of the splits.
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        if (threadIdx.x == 64) {
          const int prev = atomicAdd(&p.counters[tile], 1);
          *last_flag = (prev == splits - 1);
          if (prev == splits - 1) p.counters[tile] = 0;           // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          if (n < p.N) {
            // All partials of a few rows are requested before any is added (the loads are independent;
            // the additions keep the order of the splits).
            const int m_end = min(m0 + BT, p.M);
            const size_t zstride = (size_t)p.M * p.N;
            for (int m = m0; m < m_end; m += 4) {
              float v[4][16];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float* src = p.workspace + (size_t)min(m + i, m_end - 1) * p.N + n;
#pragma unroll
                for (int z = 0; z < 16; ++z) v[i][z] = z < splits ? __ldcg(src + z * zstride) : 0.f;
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (m + i >= m_end) break;
                float acc = 0.f;
#pragma unroll
                for (int z = 0; z < 16; ++z) acc += v[i][z];
                if (p.out_dtype == LB_F32) ((float*)p.y)[(size_t)(m + i) * p.ldy + n] = acc;
                else ((bf16*)p.y)[(size_t)(m + i) * p.ldy + n] = __float2bfloat16_rn(acc);
              }
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (p.cluster > 0 && splits > 1) {
    // Every thread of every CTA of the cluster passes both barriers, whatever happened before.
    cluster_sync_all();                               // all partial tiles are in place
    if (warp >= 2 && *abort_flag == 0) {
      const int quarter = warp & 3;
      const int nl = quarter * 32 + lane;
      const int n = n0 + nl;
      const int per = (BT + p.cluster - 1) / p.cluster;   // columns (tokens) of the tile this CTA adds up
      const int jend = min((split + 1) * per, BT);
      const uint32_t base = smem_base + (uint32_t)nl * 4u;
      if (p.swiglu) {
        if (p.rs.on) pdl_wait();
        const int f = nl & 63, feature = (n0 >> 1) + f;
        if (feature < (p.N >> 1)) {
          for (int j = split * per + (nl >> 6); j < jend; j += 2) {
            const int m = m0 + j;
            if (m >= p.M) break;
            const uint32_t a = smem_base + (uint32_t)j * (BM * 4u) + (uint32_t)f * 4u;
            const float rf = p.rs.on ? row_factor(p.rs, m) : 1.f;
            const float g = cluster_sum_f32(a, splits) * rf, u = cluster_sum_f32(a + 256u, splits) * rf;
            const float v = silu_mul(g, u);
            if (p.out_dtype == LB_F32) ((float*)p.y)[(size_t)m * p.ldy + feature] = v;
            else ((bf16*)p.y)[(size_t)m * p.ldy + feature] = __float2bfloat16_rn(v);
          }
        }
      } else if (p.he.on) {
        // The tile is one head; this CTA finishes `per` tokens of it, all 128 threads together (thread = feature).
        const HeadEpilogue& he = p.he;
        const int head = n0 / BM;
        const int kind = head < he.num_q_heads ? 0 : (head < he.num_q_heads + he.num_kv_heads ? 1 : 2);
        const int hh = kind == 0 ? head : (kind == 1 ? head - he.num_q_heads : head - he.num_q_heads - he.num_kv_heads);
        float* scratch = reinterpret_cast<float*>(smem) + BT * BM;      // behind the partial tile: 128 values, 4 sums,
        int* tok_pos = reinterpret_cast<int*>(scratch + BM + 4);        // then position and page of this CTA's tokens
        int* tok_page = tok_pos + BT;
        float* tok_rf = reinterpret_cast<float*>(tok_page + BT);        // and the factor its input row lacks
        if (p.rs.on) pdl_wait();
        const float* w = kind == 0 ? he.q_norm_w : he.k_norm_w;
        // What does not depend on the sums is fetched first, all at once: the loop below then waits for nothing but
        // its own barriers.
        const float w_n = he_w, freq = he_freq;                        // asked for at the kernel's start
        if (nl < per && m0 + split * per + nl < p.M) {
          const int m = m0 + split * per + nl;
          const int pos = he.positions[m];
          tok_pos[nl] = pos;
          tok_page[nl] = kind == 0 ? 0 : he.block_table[(size_t)he.token_seq[m] * he.max_pages + pos / he.page_size];
        }
        // the factors that the input rows lack: a warp a token, a lane a tile, so that a token's loads are one round trip
        for (int t = quarter; t < per && m0 + split * per + t < p.M; t += 4) {
          const float f = p.rs.on ? row_factor_warp(p.rs, m0 + split * per + t, lane) : 1.f;
          if (lane == 0) tok_rf[t] = f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        for (int j = split * per; j < jend; ++j) {
          const int m = m0 + j;
          if (m >= p.M) break;                                        // the same for every thread
          float v = cluster_sum_f32(base + (uint32_t)j * (BM * 4u), splits) * tok_rf[j - split * per];
          const int pos = tok_pos[j - split * per];
          if (kind != 2) {
            if (w) {
              const float ss = warp_sum(v * v);
              if (lane == 0) scratch[BM + quarter] = ss;
              asm volatile("bar.sync 1, 128;" ::: "memory");
              const float total = scratch[BM] + scratch[BM + 1] + scratch[BM + 2] + scratch[BM + 3];
              v = v * rsqrtf(total / (float)BM + he.eps) * w_n;
            }
            if (he.inv_freq) {
              scratch[nl] = v;
              asm volatile("bar.sync 1, 128;" ::: "memory");
              const float other = scratch[nl ^ 64];
              float sn, cs;
              sincosf((float)pos * freq, &sn, &cs);
              // first half: x cos - y sin with y the partner; second half: x' sin + y' cos with x' the partner
              v = nl < 64 ? v * cs - other * sn : other * sn + v * cs;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");              // the scratch is free for the next token
          }
          if (kind == 0) {
            he.q_out[((size_t)m * he.num_q_heads + hh) * BM + nl] = __float2bfloat16_rn(v);
          } else {
            const int page = tok_page[j - split * per];
            if (page >= 0) {
              bf16* pool = kind == 1 ? he.k_cache : he.v_cache;
              pool[(((size_t)page * he.num_kv_heads + hh) * he.page_size + pos % he.page_size) * BM + nl] = __float2bfloat16_rn(v);
            }
          }
        }
      } else if (p.an.on) {
        // The residual add and the first half of the norm that follows; this CTA finishes `per` tokens of the tile,
        // four at a time so that their loads (the residual, the peers' partial sums) are in flight together.
        const AddNormEpilogue& an = p.an;
        float* scratch = reinterpret_cast<float*>(smem) + BT * BM;      // behind the partial tile: 4 warp sums a token
        const float w_n = an_w;
        const int j0 = split * per, j1 = min(jend, p.M - m0);
        for (int jb = j0; jb < j1; jb += 4) {
          float before[4], acc[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            before[u] = jb == j0 ? an_before[u]
                                 : ((jb + u < j1 && n < p.N) ? an.residual[(size_t)(m0 + jb + u) * p.N + n] : 0.f);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            acc[u] = jb + u < j1 ? cluster_sum_f32(base + (uint32_t)(jb + u) * (BM * 4u), splits) : 0.f;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (jb + u >= j1) break;                                   // the same for every thread
            const float r = before[u] + acc[u];
            if (n < p.N) {
              const size_t at = (size_t)(m0 + jb + u) * p.N + n;
              an.residual[at] = r;
              an.out[at] = __float2bfloat16_rn(r * w_n);
            }
            const float sq = warp_sum(n < p.N ? r * r : 0.f);
            if (lane == 0) scratch[(jb + u - j0) * 4 + quarter] = sq;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (nl < j1 - j0) {
          const float* sl = scratch + nl * 4;
          an.sumsq[(size_t)(m0 + j0 + nl) * an.tiles + blockIdx.x] = sl[0] + sl[1] + sl[2] + sl[3];
        }
      } else {
        float* tok_rf = reinterpret_cast<float*>(smem) + BT * BM;       // behind the partial tile
        if (p.rs.on) {                                                  // the factors the input rows lack: a warp a token
          pdl_wait();
          for (int t = quarter; split * per + t < jend && m0 + split * per + t < p.M; t += 4) {
            const float f = row_factor_warp(p.rs, m0 + split * per + t, lane);
            if (lane == 0) tok_rf[t] = f;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (n < p.N)
        for (int j = split * per; j < jend; ++j) {
          const int m = m0 + j;
          if (m >= p.M) break;
          float acc = cluster_sum_f32(base + (uint32_t)j * (BM * 4u), splits);
          if (p.rs.on) acc *= tok_rf[j - split * per];
          if (p.out_dtype == LB_F32) ((float*)p.y)[(size_t)m * p.ldy + n] = acc;
          else ((bf16*)p.y)[(size_t)m * p.ldy + n] = __float2bfloat16_rn(acc);
        }
      }
    }
    cluster_sync_all();                               // no CTA leaves while a peer still reads its memory
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(tmem_cols<BT>()) : "memory");
  }
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

// A [rows, K] bfloat16 matrix, row stride ld elements, read in boxes of box_rows x 64.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapKey {
  const void* base; long long rows, K, ld; int box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.K;
    h = h * 1000003u ^ (size_t)k.ld; h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

static bool cached_map(CUtensorMap* out, const void* base, long long rows, long long K, long long ld, int box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{base, rows, K, ld, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  if (cache.size() > 8192) cache.clear();
  if (!make_map(out, base, rows, K, ld, box_rows)) return false;
  cache.emplace(key, *out);
  return true;
}

template <int BT, int STAGES>
int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, int splits, cudaStream_t stream) {
  using L = SmemLayout<BT, STAGES>;
  const int smem = L::TOTAL + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { set_error("gemm_tcgen05: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e)); return 2; }
    configured = true;
  }
  dim3 grid((p.N + BM - 1) / BM, (p.M + BT - 1) / BT, splits);
  if (p.cluster > 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 2 : 1;
    cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BT, STAGES>, mw, mx, p);
  } else {
    launch(gemm_tcgen05_kernel<BT, STAGES>, grid, dim3(192), smem, stream, mw, mx, p);
  }
  return 0;
}

// ---- many tokens: persistent CTAs, tokens on the lanes, two accumulators -----------------------------------
// With many tokens the product is bound by the tensor cores, and the kernel is arranged for that:
// one CTA per SM walks over output tiles of 128 tokens x 256 features; tokens sit on the 128 lanes of the
// accumulator, so an epilogue thread holds one token's row and stores 16 consecutive features as whole
// 16-byte words; tensor memory holds two accumulators (2 x 256 columns), so the epilogue of one tile runs
// while the tensor cores work on the next.  Tiles are visited with the token tile running fastest, so that
// CTAs working at the same time share weight tiles in L2.
//
// The feature width of a tile is a launch parameter (a multiple of 16 up to 256; 128 or 256 with the fused
// SwiGLU): with few token tiles, 256 features a tile can leave most SMs without a tile (512 tokens x 4096 features:
// 64 tiles for 148 SMs), and the launcher picks the width with the smallest waves x width.
constexpr int PF_BM = 128;       // tokens of a tile (lanes)
constexpr int PF_BN = 256;       // the most features of a tile (columns of an accumulator)
constexpr int PF_STAGES = 4;

// The feature tiles of a launch: `cols1` columns of tiles `bn1` wide, then the features from cols1 * bn1 on in tiles
// `bn2` wide (their weight boxes come through a second tensor map).  Tiles are numbered column by column, the token
// tile running fastest, the second kind after the first.
struct PrefillPlan { int bn1, cols1, bn2; int mb = 16; };     // mb: token tiles of a block (the order of the tiles, see tile_of)

// PAIR: two CTAs of a cluster work on one tile of 256 tokens x up to 256 features (tcgen05 cta_group::2): each holds its
// own 128 tokens and half of the tile's weight rows in shared memory (two thirds of the bytes a stage of one CTA holds:
// six stages instead of four), the first CTA of the pair issues the MMAs for both, and each CTA finds its 128 tokens x
// all features of the tile in its own tensor memory.
template <bool PAIR>
struct PrefillSmemT {
  static constexpr int STAGES = PAIR ? 6 : PF_STAGES;
  static constexpr int A_BYTES = PF_BM * BK * 2;
  static constexpr int B_BYTES = (PAIR ? PF_BN / 2 : PF_BN) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16;
};
using PrefillSmem = PrefillSmemT<false>;

// With PAIR, m_tiles counts pairs of token tiles, num_tiles tiles of 256 tokens, and the grid holds two CTAs a tile slot.
template <bool PAIR>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_prefill_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                            const __grid_constant__ CUtensorMap map_w2, GemmParams p, int m_tiles, int num_tiles,
                            PrefillPlan plan, int vec_store) {
  using L = PrefillSmemT<PAIR>;
  constexpr int PF_STAGES = L::STAGES;
  const uint32_t rank = PAIR ? cluster_rank() : 0u;          // 0: the CTA that issues the pair's MMAs
  const int slot_id = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, num_slots = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (PF_STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * PF_STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * PF_STAGES + 2 + b); };
  uint32_t* tmem_slot = (uint32_t*)(smem + L::BAR_OFFSET + L::NUM_BARS * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  const int my_tiles = slot_id < num_tiles ? (num_tiles - 1 - slot_id) / num_slots + 1 : 0;
  const int tiles1 = plan.cols1 * m_tiles;
  constexpr int M_STEP = PAIR ? 2 * PF_BM : PF_BM;
  // first token (of this CTA), first feature and feature width of a tile; second: whether its weights come through the second map
  // Inside a kind of tiles the token tiles run fastest, in blocks of MB token tiles: the tiles that are worked on at a time
  // (one a CTA or pair) then share MB token tiles and slots / MB feature tiles, which is what L2 has to hold; with all token
  // tiles in one block, 8192 tokens x 4096 are 67 MB of tokens read again for every two columns of feature tiles.  The
  // launcher sizes a block to about 24 MB of tokens (at most 8 pairs or 16 single token tiles, at least 2).
  const int MB = plan.mb;
  auto place = [&](int idx, int cols, int& mt, int& col) {
    const int per_block = MB * cols;
    const int b = idx / per_block, r = idx - b * per_block;
    const int mb = min(MB, m_tiles - b * MB);
    col = r / mb;
    mt = b * MB + (r - col * mb);
  };
  auto tile_of = [&](int tile, int& m0, int& n0, int& bn) -> bool {
    int mt, col;
    if (tile < tiles1) {
      place(tile, plan.cols1, mt, col);
      m0 = mt * M_STEP + (int)rank * PF_BM; n0 = col * plan.bn1; bn = plan.bn1;
      return false;
    }
    const int cols2 = (p.N - plan.cols1 * plan.bn1 + plan.bn2 - 1) / plan.bn2;
    place(tile - tiles1, cols2, mt, col);
    m0 = mt * M_STEP + (int)rank * PF_BM; n0 = plan.cols1 * plan.bn1 + col * plan.bn2; bn = plan.bn2;
    return true;
  };
  // bytes a stage's barrier expects (of a pair: both CTAs' bytes on the first CTA's barrier), the first weight row this CTA loads
  auto stage_bytes = [&](int bn) { return (uint32_t)(PAIR ? 2 * (L::A_BYTES + (bn / 2) * BK * 2) : L::A_BYTES + bn * BK * 2); };
  auto w_row = [&](int n0, int bn) { return PAIR ? n0 + (int)rank * (bn / 2) : n0; };
  auto load = [&](uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    if (PAIR) tma_load_2d_pair(dst, map, x, y, map_to_rank(bar, 0));
    else tma_load_2d(dst, map, x, y, bar);
  };

  pdl_trigger();
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w2) : "memory");
    for (int s = 0; s < PF_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    // an accumulator is free again when the four epilogue warps (of both CTAs of a pair) have read it
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), PAIR ? 8 : 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();          // the other CTA's barriers are set up before anything of this CTA signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer: one ring of stages across all tiles of this CTA -------------------------------------
    if (lane == 0 && my_tiles > 0) {
      long long it = 0;                       // stage uses so far
      bool ok = true;
      // The weights of the first tile do not depend on the kernel before this one.
      const int early = num_kb < PF_STAGES ? num_kb : PF_STAGES;
      {
        int m0, n0, bn;
        const CUtensorMap* mw = tile_of(slot_id, m0, n0, bn) ? &map_w2 : &map_w;
        for (int i = 0; i < early; ++i) {
          if (rank == 0) mbar_expect_tx(full_bar(i), stage_bytes(bn));
          load(smem_base + i * L::STAGE_BYTES + L::A_BYTES, mw, i * BK, w_row(n0, bn), full_bar(i));
        }
        pdl_wait();
        for (int i = 0; i < early; ++i)
          load(smem_base + i * L::STAGE_BYTES, &map_x, i * BK, m0, full_bar(i));
      }
      for (int t = 0; t < my_tiles && ok; ++t) {
        int m0, n0, bn;
        const CUtensorMap* mw = tile_of(slot_id + t * num_slots, m0, n0, bn) ? &map_w2 : &map_w;
        const uint32_t stage_tx = stage_bytes(bn);
        for (int kb = (t == 0 ? early : 0); kb < num_kb; ++kb) {
          const long long use = (long long)t * num_kb + kb;
          const int s = (int)(use % PF_STAGES);
          const uint32_t parity = (uint32_t)((use / PF_STAGES) & 1) ^ 1u;
          if (!mbar_wait(empty_bar(s), parity, abort_flag, ERR_EMPTY_WAIT)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(s), stage_tx);
          const uint32_t dst = smem_base + s * L::STAGE_BYTES;
          load(dst, &map_x, kb * BK, m0, full_bar(s));
          load(dst + L::A_BYTES, mw, kb * BK, w_row(n0, bn), full_bar(s));
          it = use + 1;
        }
        if (t == 0 && it < early) it = early;
      }
      if (*abort_flag) {
        for (long long u = it > PF_STAGES ? it - PF_STAGES : 0; u < it; ++u) {
          const long long t0 = clock64();
          while (!mbar_try_wait(full_bar((int)(u % PF_STAGES)), (uint32_t)((u / PF_STAGES) & 1)) &&
                 (unsigned long long)(clock64() - t0) < WAIT_CYCLES / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---- tensor-core issue -----------------------------------------------------------------------------------
    if (lane == 0 && rank == 0) {
      bool ok = true;
      for (int t = 0; t < my_tiles && ok; ++t) {
        const int b = t & 1;
        int m0, n0, bn;
        tile_of(slot_id + t * num_slots, m0, n0, bn);
        const uint32_t idesc = PAIR ? umma_idesc_pair(bn) : umma_idesc(bn);
        // the epilogue has drained this accumulator (its use two tiles ago)
        ok = mbar_wait(acc_empty(b), (uint32_t)((t >> 1) & 1) ^ 1u, abort_flag, ERR_ACCUM_WAIT);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + (uint32_t)b * PF_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long use = (long long)t * num_kb + kb;
          const int s = (int)(use % PF_STAGES);
          ok = mbar_wait(full_bar(s), (uint32_t)((use / PF_STAGES) & 1), abort_flag, ERR_FULL_WAIT);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_base + s * L::STAGE_BYTES;
          const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + L::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (PAIR) umma_f16_pair(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
            else umma_f16(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          }
          if (PAIR) umma_commit_pair(empty_bar(s)); else umma_commit(empty_bar(s));
        }
        if (ok) { if (PAIR) umma_commit_pair(acc_full(b)); else umma_commit(acc_full(b)); }
      }
    }
  } else {
    // ---- epilogue: warp w reads lanes (w % 4) * 32 .. + 31, i.e. 32 tokens, 16 features at a time -------------
    const int quarter = warp & 3;
    bool ok = true;
    for (int t = 0; t < my_tiles && ok; ++t) {
      int m0, n0, bn;
      tile_of(slot_id + t * num_slots, m0, n0, bn);
      const int m = m0 + quarter * 32 + lane;
      const int b = t & 1;
      ok = mbar_wait(acc_full(b), (uint32_t)((t >> 1) & 1), abort_flag, ERR_ACCUM_WAIT);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)b * PF_BN;
      // The factor this thread's token lacks (RowScale): its partial sums are asked for together, one round trip a tile.
      float rf = 1.f;
      if (p.rs.on) {
        pdl_wait();
        rf = m < p.M ? row_factor(p.rs, m) : 0.f;
      }
      if (p.an.on) {
        // The residual add and the first half of the norm that follows (AddNormEpilogue): this thread holds one token's
        // part of the tile; the residual values of the next 16 features are asked for while these 16 are finished.
        pdl_wait();
        const AddNormEpilogue& an = p.an;
        const bool second = n0 >= plan.cols1 * plan.bn1 && plan.cols1 * plan.bn1 < p.N;
        const int tile_col = second ? plan.cols1 + (n0 - plan.cols1 * plan.bn1) / plan.bn2 : n0 / plan.bn1;
        const bool row_ok = m < p.M;
        const bool vec = (p.N & 7) == 0;
        float* res_row = an.residual + (size_t)(row_ok ? m : 0) * p.N;
        bf16* out_row = an.out + (size_t)(row_ok ? m : 0) * p.N;
        float ss = 0.f;
        // Two chunks of 16 features are asked for while the two before them are finished: four in flight.
        float4 nxt[8];
        auto fetch = [&](int n, float4* dst) {
          if (row_ok && vec && n + 16 <= p.N) {
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = *reinterpret_cast<const float4*>(res_row + n + 4 * j);
          } else {
            float* f = reinterpret_cast<float*>(dst);
#pragma unroll
            for (int j = 0; j < 16; ++j) f[j] = (row_ok && n + j < p.N) ? res_row[n + j] : 0.f;
          }
        };
        fetch(n0, nxt);
        if (16 < bn) fetch(n0 + 16, nxt + 4);
#pragma unroll 1
        for (int c0 = 0; c0 < bn; c0 += 32) {
          float4 cur[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
          if (c0 + 32 < bn) fetch(n0 + c0 + 32, nxt);
          if (c0 + 48 < bn) fetch(n0 + c0 + 48, nxt + 4);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int c = c0 + 16 * h;
            if (c >= bn) break;
            uint32_t r[16];
            tmem_ld16(taddr + c, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int n = n0 + c;
            if (row_ok && n < p.N) {
              const float* before = reinterpret_cast<const float*>(cur + 4 * h);
              float v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                v[j] = before[j] + __uint_as_float(r[j]);
                if (n + j < p.N) ss += v[j] * v[j];
              }
              if (vec && n + 16 <= p.N) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  *reinterpret_cast<float4*>(res_row + n + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float4 nw = *reinterpret_cast<const float4*>(an.norm_w + n + 4 * j);
                  __nv_bfloat162 lo = __floats2bfloat162_rn(v[4 * j] * nw.x, v[4 * j + 1] * nw.y);
                  __nv_bfloat162 hi = __floats2bfloat162_rn(v[4 * j + 2] * nw.z, v[4 * j + 3] * nw.w);
                  w[2 * j] = *reinterpret_cast<uint32_t*>(&lo); w[2 * j + 1] = *reinterpret_cast<uint32_t*>(&hi);
                }
                uint4* dst = reinterpret_cast<uint4*>(out_row + n);
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  if (n + j < p.N) {
                    res_row[n + j] = v[j];
                    out_row[n + j] = __float2bfloat16_rn(v[j] * an.norm_w[n + j]);
                  }
                }
              }
            }
          }
        }
        if (row_ok) an.sumsq[(size_t)m * an.tiles + tile_col] = ss;
      } else if (p.swiglu) {
        // columns [128b, 128b+64) are gate rows, [128b+64, 128b+128) the up rows of the same 64 features
#pragma unroll 1
        for (int cc = 0; cc < bn / 2; cc += 16) {
          const int c = (cc >> 6) * 128 + (cc & 63);
          uint32_t g[16], u[16];
          tmem_ld16(taddr + c, g);
          tmem_ld16(taddr + c + 64, u);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const int feature = (n0 >> 1) + cc;
          if (m < p.M && feature < (p.N >> 1)) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = silu_mul(__uint_as_float(g[j]) * rf, __uint_as_float(u[j]) * rf);
            if (vec_store && feature + 16 <= (p.N >> 1)) {
              if (p.out_dtype == LB_F32) {
                float4* dst = reinterpret_cast<float4*>((float*)p.y + (size_t)m * p.ldy + feature);
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              } else {
                uint4* dst = reinterpret_cast<uint4*>((bf16*)p.y + (size_t)m * p.ldy + feature);
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                  w[j] = *reinterpret_cast<uint32_t*>(&b2);
                }
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (feature + j < (p.N >> 1)) {
                  if (p.out_dtype == LB_F32) ((float*)p.y)[(size_t)m * p.ldy + feature + j] = v[j];
                  else ((bf16*)p.y)[(size_t)m * p.ldy + feature + j] = __float2bfloat16_rn(v[j]);
                }
              }
            }
          }
        }
      } else
#pragma unroll 2
      for (int c = 0; c < bn; c += 16) {
        uint32_t r[16];
        tmem_ld16(taddr + c, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int n = n0 + c;
        if (p.rs.on) {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * rf);
        }
        if (m < p.M && n < p.N) {
          if (vec_store && n + 16 <= p.N) {
            if (p.out_dtype == LB_F32) {
              float4* dst = reinterpret_cast<float4*>((float*)p.y + (size_t)m * p.ldy + n);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            } else {
              uint4* dst = reinterpret_cast<uint4*>((bf16*)p.y + (size_t)m * p.ldy + n);
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                w[j] = *reinterpret_cast<uint32_t*>(&v);
              }
              dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
              dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (n + j < p.N) {
                const float v = __uint_as_float(r[j]);
                if (p.out_dtype == LB_F32) ((float*)p.y)[(size_t)m * p.ldy + n + j] = v;
                else ((bf16*)p.y)[(size_t)m * p.ldy + n + j] = __float2bfloat16_rn(v);
              }
            }
          }
        }
      }
      // this accumulator may be overwritten: one arrival per epilogue warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (PAIR) asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(map_to_rank(acc_empty(b), 0)) : "memory");
        else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(b)) : "memory");
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();          // nothing of the other CTA is on its way to this CTA's barriers or tensor memory any more
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// The feature tiles of a launch.  CTA i of G = min(tiles, SMs) takes tiles i, i + G, ...; a tile costs its width + 64
// (the 64 stand for what a tile costs whatever its width: its token tile is loaded again for every feature tile, and
// narrow MMAs use the tensor cores less well), and the launch takes as long as its busiest CTA.  Candidates: one width
// for all tiles (256, or a narrower multiple of 16, of 128 with the fused SwiGLU, whose gate and up rows come in blocks
// of 64), or columns of 256 followed by narrower tiles for the rest, so that the last round of tiles fits the SMs (2048
// tokens x 4096 features: 9 columns of 256 and 9 of 208 are two rounds of 144 tiles instead of 148 + 108 tiles of 256).
// Measured at 8B sizes: 512 x 4096 x 4096 27.6 -> 23.4 us (width 144), 2048 x 6144 x 4096 81.3 -> 80.0 (240); with
// ten waves and more a narrower tile for all only lost (2048 x 24576 x 4096, width 224: 305 -> 314 us), hence the margin
// a narrower plan has to win by.
static long long prefill_plan_cost(const PrefillPlan& pl, int m_tiles, int N, int num_sms) {
  const long long t1 = (long long)pl.cols1 * m_tiles;
  const int rest = N - pl.cols1 * pl.bn1;
  const long long t2 = rest > 0 ? (long long)m_tiles * ((rest + pl.bn2 - 1) / pl.bn2) : 0;
  const long long tiles = t1 + t2;
  const long long G = tiles < num_sms ? tiles : num_sms;
  if (G <= 0) return 0;
  // CTA 0 takes the most tiles; CTA i's tiles i, i + G, ... of the first kind number ceil((t1 - i) / G)
  long long worst = 0;
  for (long long i = 0; i < G; ++i) {
    const long long n1 = i < t1 ? (t1 - 1 - i) / G + 1 : 0;
    const long long first2 = t1 + ((i - t1) % G + G) % G;                  // its first tile index >= t1
    const long long n2 = first2 < tiles ? (tiles - 1 - first2) / G + 1 : 0;
    const long long c = n1 * (pl.bn1 + 64) + n2 * (pl.bn2 + 64);
    if (c > worst) worst = c;
  }
  return worst;
}

static PrefillPlan prefill_plan_search(int m_tiles, int N, int step, int num_sms);

// The search costs a few hundred microseconds: its result is kept per (token tiles, features, step of the widths, SMs).
// step: 16, 32 for CTA pairs (each CTA loads half of a tile's weight rows), 128 with the fused SwiGLU.
static PrefillPlan prefill_plan(int m_tiles, int N, int step, int num_sms) {
  static std::unordered_map<unsigned long long, PrefillPlan> cache;
  static std::mutex mu;
  const unsigned long long key = ((unsigned long long)m_tiles << 44) ^ ((unsigned long long)N << 20) ^ ((unsigned long long)num_sms << 8) ^ (unsigned long long)step;
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 4096) cache.clear();
  const PrefillPlan pl = prefill_plan_search(m_tiles, N, step, num_sms);
  cache.emplace(key, pl);
  return pl;
}

static PrefillPlan prefill_plan_search(int m_tiles, int N, int step, int num_sms) {
  const int full_cols = (N + PF_BN - 1) / PF_BN;
  PrefillPlan best{PF_BN, full_cols, PF_BN};
  const long long base = prefill_plan_cost(best, m_tiles, N, num_sms);
  long long best_cost = base * 93 / 100;                   // one narrower width for all has to win by 7 %
  for (int bn = PF_BN - step; bn >= 64; bn -= step) {
    PrefillPlan pl{bn, (N + bn - 1) / bn, bn};
    const long long c = prefill_plan_cost(pl, m_tiles, N, num_sms);
    if (c < best_cost) { best = pl; best_cost = c; }
  }
  if (best.bn1 == PF_BN) best_cost = base * 97 / 100;      // columns of 256 and a narrower rest: by 3 %
  for (int cols1 = N / PF_BN - 1; cols1 >= 0 && cols1 >= N / PF_BN - 24; --cols1) {
    for (int bn2 = PF_BN - step; bn2 >= 64; bn2 -= step) {
      PrefillPlan pl{PF_BN, cols1, bn2};
      const long long c = prefill_plan_cost(pl, m_tiles, N, num_sms);
      if (c < best_cost) { best = pl; best_cost = c; }
    }
  }
  return best;
}

static int g_pair_slots_seen = -1;

// Which kind of tiles a many-token product uses: pairs of CTAs or single ones, how many token tiles, how many run at a
// time, and the feature tiles.  force_bn: 0 choose, else the feature width of the tiles (tests); pair: 0 choose, 1 never,
// 2 always.
static void prefill_choose(int M, int N, int K, int swiglu, int force_bn, int pair, bool* use_pair_out, int* m_tiles_out,
                           int* slots_out, PrefillPlan* plan_out) {
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  // Pairs of CTAs on tiles of 256 tokens when there are at least two token tiles (pair: 0 choose, 1 never, 2 always);
  // their widths are multiples of 32, each CTA loading half of a tile's weight rows.
  int forced_width = force_bn < 0 ? (-force_bn) & 1023 : force_bn;
  // Measured at 8B sizes: pairs are 3 to 8 % faster from 1024 tokens on (2048 x 4096 x 12288: 155.7 -> 147.3 us; with
  // SwiGLU 2048 x 24576 x 4096: 293.6 -> 275.9 us; whole steps of 2048 tokens, many in a row: 28.3 -> 27.3 ms); they
  // compute whole tiles of 256 tokens, so they are left alone where that adds more than 4 % of rows.
  const int rows_pair = (M + 2 * PF_BM - 1) / (2 * PF_BM) * 2 * PF_BM, rows_single = (M + PF_BM - 1) / PF_BM * PF_BM;
  // Below 1024 tokens only products with at least two rounds of such tiles gain (512 x 24576 x 4096 with SwiGLU: 87.9 ->
  // 79.9 us; 512 x 4096 x 4096, 32 tiles of 256 x 256 instead of 64 of 128 x 256: 24.8 -> 27.2 us).
  const long long tiles256 = (long long)(rows_pair / (2 * PF_BM)) * ((N + PF_BN - 1) / PF_BN);
  const bool use_pair = pair == 2 || (pair == 0 && (M >= 1024 || tiles256 >= num_sms) && rows_pair * 100 <= rows_single * 104 &&
                                      num_sms >= 2 && (forced_width % 32) == 0);
  const int m_tiles = use_pair ? (M + 2 * PF_BM - 1) / (2 * PF_BM) : (M + PF_BM - 1) / PF_BM;
  // The pairs of a launch all have to be resident at once (each walks its own list of tiles): as many as the GPU takes.
  static int pair_slots = -1;
  if (use_pair && pair_slots < 0) {
    const int smem_pair = PrefillSmemT<true>::TOTAL + 1024;
    pair_slots = num_sms / 2;
    if (cudaFuncSetAttribute(gemm_tcgen05_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pair) == cudaSuccess) {
      cudaLaunchConfig_t qc = {};
      qc.gridDim = dim3(2 * (num_sms / 2)); qc.blockDim = dim3(192); qc.dynamicSmemBytes = smem_pair;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      qc.attrs = qa; qc.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_prefill_kernel<true>, &qc) == cudaSuccess && n > 0 && n < pair_slots) pair_slots = n;
    }
    cudaGetLastError();
  }
  if (use_pair) g_pair_slots_seen = pair_slots;
  const int slots = use_pair ? pair_slots : num_sms;
  PrefillPlan plan;
  if (force_bn > 0) plan = PrefillPlan{force_bn, (N + force_bn - 1) / force_bn, force_bn};
  else if (force_bn < 0) plan = PrefillPlan{PF_BN, (-force_bn) >> 10, (-force_bn) & 1023};   // tests: columns of 256, then a width
  else plan = prefill_plan(m_tiles, N, swiglu ? 128 : use_pair ? 32 : 16, slots);
  if (plan.cols1 * plan.bn1 >= N) plan = PrefillPlan{plan.bn1, (N + plan.bn1 - 1) / plan.bn1, plan.bn1};
  {
    const long long tile_bytes = (long long)(use_pair ? 2 * PF_BM : PF_BM) * K * 2;
    long long mb = (24ll << 20) / (tile_bytes > 0 ? tile_bytes : 1);
    const int top = use_pair ? 8 : 16;
    plan.mb = (int)(mb < 2 ? 2 : mb > top ? top : mb);
  }
  *use_pair_out = use_pair; *m_tiles_out = m_tiles; *slots_out = slots; *plan_out = plan;
}

// Feature tiles of a row in that plan: the columns of AddNormEpilogue::sumsq.
static int prefill_feature_tiles(const PrefillPlan& plan, int N) {
  const int rest = N - plan.cols1 * plan.bn1;
  return plan.cols1 + (rest > 0 ? (rest + plan.bn2 - 1) / plan.bn2 : 0);
}

static int launch_prefill(const void* y, int y_dtype, const void* x, const void* w, int M, int N, int K, long long ldx,
                          long long ldy, int swiglu, int force_bn, int pair, cudaStream_t stream,
                          const AddNormEpilogue* an = nullptr, const RowScale* rs = nullptr) {
  bool use_pair; int m_tiles, slots; PrefillPlan plan;
  prefill_choose(M, N, K, swiglu, force_bn, pair, &use_pair, &m_tiles, &slots, &plan);
  if (use_pair && (plan.bn1 % 32 || plan.bn2 % 32)) { set_error("gemm_tcgen05: pairs of CTAs take tile widths that are multiples of 32"); return 1; }
  const int box1 = use_pair ? plan.bn1 / 2 : plan.bn1, box2 = use_pair ? plan.bn2 / 2 : plan.bn2;
  CUtensorMap mx, mw, mw2;
  if (!cached_map(&mx, x, M, K, ldx, PF_BM) || !cached_map(&mw, w, N, K, K, box1) || !cached_map(&mw2, w, N, K, K, box2)) {
    set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%lld)", M, N, K, ldx);
    return 3;
  }
  GemmParams p;
  p.y = const_cast<void*>(y); p.workspace = nullptr; p.counters = nullptr; p.M = M; p.N = N; p.K = K; p.ldy = ldy;
  p.out_dtype = y_dtype; p.cluster = 0; p.swiglu = swiglu;
  if (an) {
    p.an = *an; p.an.on = 1;
    if (p.an.tiles != prefill_feature_tiles(plan, N)) { set_error("gemm_tcgen05: %d columns of partial sums, the plan has %d feature tiles", p.an.tiles, prefill_feature_tiles(plan, N)); return 1; }
  }
  if (rs) { p.rs = *rs; p.rs.on = 1; }
  const int rest = N - plan.cols1 * plan.bn1;
  const int num_tiles = m_tiles * (plan.cols1 + (rest > 0 ? (rest + plan.bn2 - 1) / plan.bn2 : 0));
  const int el = y_dtype == LB_F32 ? 4 : 2;
  const int vec_store = ((uintptr_t)y % 16 == 0) && ((ldy * el) % 16 == 0);
  const int smem = (use_pair ? PrefillSmemT<true>::TOTAL : PrefillSmemT<false>::TOTAL) + 1024;
  static bool configured[2] = {false, false};
  if (!configured[use_pair]) {
    cudaError_t e = use_pair ? cudaFuncSetAttribute(gemm_tcgen05_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
                             : cudaFuncSetAttribute(gemm_tcgen05_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { set_error("gemm_tcgen05: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e)); return 2; }
    configured[use_pair] = true;
  }
  const int grid = num_tiles < slots ? num_tiles : slots;
  if (!use_pair) {
    launch(gemm_tcgen05_prefill_kernel<false>, dim3(grid), dim3(192), smem, stream, mx, mw, mw2, p, m_tiles, num_tiles, plan, vec_store);
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * grid); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = g_pdl_enabled ? 2 : 1;
  cudaLaunchKernelEx(&cfg, gemm_tcgen05_prefill_kernel<true>, mx, mw, mw2, p, m_tiles, num_tiles, plan, vec_store);
  return 0;
}

// Stages per token tile: up to 128 tokens the ring is sized so that two CTAs share an SM (about 100 KB
// each): the product is bound by memory there and a second CTA hides the first one's start and end.
static int launch_for_tile(int bt, const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, int splits,
                           cudaStream_t stream) {
  switch (bt) {
    case 16: return launch_tc<16, 6>(mw, mx, p, splits, stream);
    case 32: return launch_tc<32, 5>(mw, mx, p, splits, stream);
    case 64: return launch_tc<64, 4>(mw, mx, p, splits, stream);
    case 128: return launch_tc<128, 3>(mw, mx, p, splits, stream);
    default: return launch_tc<256, 4>(mw, mx, p, splits, stream);
  }
}

}  // namespace lb

// How many pairs of CTAs of the many-token kernel run at a time (-1: no launch has asked yet).
LB_EXPORT int lb_gemm_tcgen05_pair_slots() { return lb::g_pair_slots_seen; }

// The feature tiles the many-token kernel would use for M tokens and N features: out[0] columns of tiles out[1] wide,
// then tiles out[2] wide (out[0] * out[1] >= N: one width for all).
LB_EXPORT void lb_gemm_tcgen05_prefill_plan(int M, int N, int swiglu, int num_sms, int* out) {
  const lb::PrefillPlan pl = lb::prefill_plan((M + lb::PF_BM - 1) / lb::PF_BM, N, swiglu ? 128 : 16, num_sms > 0 ? num_sms : 148);
  out[0] = pl.cols1; out[1] = pl.bn1; out[2] = pl.bn2;
}

// Which (token tile, splits) the launcher would choose; exposed so that callers can size the workspace
// and tests can force a choice.  Returns splits; *bt receives the token tile.
LB_EXPORT int lb_gemm_tcgen05_plan(int M, int N, int K, int* bt) {
  int t = 16;
  if (M > 128) {
    t = (((M + 255) / 256) * 256 <= ((M + 127) / 128) * 128) ? 256 : 128;
    if (t == 256 && ((N + lb::BM - 1) / lb::BM) * ((M + 255) / 256) < 148) t = 128;   // more, smaller tiles to fill the SMs
  }
  else if (M > 64) t = 128;
  else if (M > 32) t = 64;
  else if (M > 16) t = 32;
  if (bt) *bt = t;
  const int tiles = ((N + lb::BM - 1) / lb::BM) * ((M + t - 1) / t);
  const int kb = (K + lb::BK - 1) / lb::BK;
  int splits = 1;
  if (tiles < 148 && M <= 256) {       // splitting pays only while the weights are what is streamed
    // The splits of a tile form a thread-block cluster that adds up through shared memory: any count up to 8.  As many
    // as keep the launch within 256 CTAs: clusters are placed inside a GPC (18 or 20 SMs, two CTAs an SM), and
    // beyond about 240-256 CTAs some of them wait for a second round (measured at 8 tokens, back to back, us: q|k|v of the
    // 8B shape, 48 tiles: 4 splits 13.1, 5 splits 11.8, 6 splits 17.3; o, 32 tiles: 4 splits 10.9, 7 splits 8.8, 8
    // splits 8.9; o of the 14B shape, 40 tiles: 4 splits 13.2, 6 splits 11.9, 7 splits 17.6).
    for (int s = 2; s <= 8; ++s)
      if (tiles * s <= 256 && s <= kb / 4) splits = s;
    if (splits == 1) {                   // more than 128 tiles: two splits where they still fit one round of two CTAs an SM
      splits = 296 / tiles;
      if (splits > kb / 4) splits = kb / 4;
      splits = splits >= 2 ? 2 : 1;
    }
  }
  return splits;
}

// y[M,N] = x[M,K] . w[N,K]^T.  x: bfloat16, row stride ldx; w: bfloat16, contiguous; y: bfloat16 or float32,
// row stride ldy.  workspace (float32, workspace_elems elements) and counters (int32, zero, counters_len
// entries) are needed when K is split; with too little of either the product runs unsplit.
// force_bt / force_splits (0: choose) are for tests.
// row_scale (may be null): the rows of x lack their norm's factor (see RowScale); taken by the few-token product with
// the fused SwiGLU only.
LB_EXPORT int lb_gemm_tcgen05(void* y, int y_dtype, const void* x, const void* w, int M, int N, int K, long long ldx,
                              long long ldy, float* workspace, long long workspace_elems, int* counters,
                              int counters_len, int force_bt, int force_splits, int swiglu, const lb::RowScale* row_scale,
                              cudaStream_t stream) {
  LB_CHECK_ARG(!row_scale || (row_scale->sumsq && row_scale->tiles > 0), "gemm_tcgen05: a row scale without partial sums");
  LB_CHECK_ARG(lb::valid_dtype(y_dtype), "gemm_tcgen05: bad output dtype %d", y_dtype);
  LB_CHECK_ARG(M >= 0 && N > 0 && K > 0 && ldx >= K && ldy >= (swiglu ? N / 2 : N), "gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
  LB_CHECK_ARG(!swiglu || N % 128 == 0, "gemm_tcgen05: the fused SwiGLU needs gate and up rows in blocks of 64 (N=%d is no multiple of 128)", N);
  LB_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0, "gemm_tcgen05: K=%d and the row stride %lld must be multiples of 8 (TMA strides are multiples of 16 bytes)", K, ldx);
  LB_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tcgen05: operands must be 16-byte aligned");
  if (M == 0) return 0;
  // Which kernel: above 256 tokens the one with tokens on the lanes.  Below, it still wins where the product has many
  // features for its inner size, so that its tiles fill the SMs without any cut along K: the gate|up product from 65
  // tokens on (8B sizes, 128 tokens: 39 us against 46; 256 tokens: 58 against 92), other products with more features
  // than inner size (q|k|v) from 129 tokens on (256 tokens: 26 us against 37).  The o and down products, few features
  // and a long inner size, stay with the kernel that cuts K over a cluster (256 tokens, down: 37 us against 64).  The
  // same at the sizes of every model of the family from 0.6B to 32B.  force_bt < 0 asks for the kernel with tokens on the
  // lanes at any size; force_bt > 0 or a given split count for the other one.
  const bool many = M > 256 ? force_bt <= 0
                            : force_bt < 0 || (force_bt == 0 && force_splits == 0 && (swiglu ? M > 64 : (M > 128 && N > K)));
  if (many) {
    // force_bt: 0 chooses between one CTA a tile of 128 tokens and a pair of CTAs a tile of 256, -1 asks for the former,
    // -2 for the latter
    // with many tokens force_splits stands for the feature width of the tiles (0: choose; -(c * 1024 + w): c columns of
    // tiles 256 wide, then tiles w wide)
    const int fw = force_splits < 0 ? (-force_splits) & 1023 : force_splits;
    LB_CHECK_ARG(force_splits == 0 || (fw >= 16 && fw <= lb::PF_BN && fw % 16 == 0 && (!swiglu || fw % 128 == 0)),
                 "gemm_tcgen05: tile width %d is no multiple of 16 (128 with SwiGLU) up to 256", fw);
    LB_CHECK_ARG(force_bt >= -2, "gemm_tcgen05: token tile %d is not one of 16, 32, 64, 128, 256", force_bt);
    if (int rc = lb::launch_prefill(y, y_dtype, x, w, M, N, K, ldx, ldy, swiglu, force_splits, -force_bt, stream, nullptr, row_scale)) return rc;
    LB_CHECK_LAUNCH("gemm_tcgen05 (many tokens)");
    return 0;
  }
  int bt = 16;
  int splits = lb_gemm_tcgen05_plan(M, N, K, &bt);
  if (force_bt) {
    LB_CHECK_ARG(force_bt == 16 || force_bt == 32 || force_bt == 64 || force_bt == 128 || force_bt == 256,
                 "gemm_tcgen05: token tile %d is not one of 16, 32, 64, 128, 256", force_bt);
    bt = force_bt;
  }
  const bool workspace_path = force_splits < 0;
  if (force_splits) splits = force_splits < 0 ? -force_splits : force_splits;
  const int kb = (K + lb::BK - 1) / lb::BK;
  if (splits > kb) splits = kb;
  if (splits > 16) splits = 16;            // the reduction holds at most 16 partials of an element at a time
  const long long tiles = (long long)((N + lb::BM - 1) / lb::BM) * ((M + bt - 1) / bt);
  const bool cluster_ok = !workspace_path && splits <= 8;
  if (swiglu && splits > 1 && !cluster_ok) splits = 1;       // the pairing of gate and up is done in shared memory
  if (splits > 1 && !cluster_ok && (workspace == nullptr || counters == nullptr || (long long)splits * M * N > workspace_elems ||
                                    tiles > counters_len))
    splits = 1;
  LB_CHECK_ARG((M + bt - 1) / bt <= 65535 && splits <= 65535, "gemm_tcgen05: grid too large");

  CUtensorMap mw, mx;
  if (!lb::cached_map(&mw, w, N, K, K, lb::BM) || !lb::cached_map(&mx, x, M, K, ldx, bt)) {
    lb::set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%lld)", M, N, K, ldx);
    return 3;
  }
  lb::GemmParams p;
  p.y = y; p.workspace = workspace; p.counters = counters; p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.out_dtype = y_dtype;
  // Clusters when the split count allows it and the caller did not ask for the workspace path
  // (force_splits < 0 asks for -force_splits splits through the workspace).
  p.cluster = (!workspace_path && splits > 1 && splits <= 8) ? splits : 0;
  p.swiglu = swiglu;
  LB_CHECK_ARG(!row_scale || splits == 1 || p.cluster > 0,
               "gemm_tcgen05: a row scale is not taken by a product that is split through the workspace (M=%d, %d splits)", M, splits);
  if (row_scale) { p.rs = *row_scale; p.rs.on = 1; }
  if (int rc = lb::launch_for_tile(bt, mw, mx, p, splits, stream)) return rc;
  LB_CHECK_LAUNCH("gemm_tcgen05");
  return 0;
}

// The plan of a product whose epilogue adds to the residual stream (AddNormEpilogue): token tile and splits with few
// tokens, -1 for the many-token product, 0 when the sizes do not allow it or would not gain.  With few tokens the
// epilogue lives in the reduction over a cluster, so the product has to be one that is split over a cluster (fewer
// tiles than SMs).  With many tokens it runs under the main loop of the CTA's next tile; a product with no more tiles
// than CTAs has no next tile, its epilogues are the end of the kernel, and there the add and the norm as a kernel of
// their own, spread over all SMs, are the faster (measured at the 8B sizes: 512 tokens 9.2 ms a step against 9.8 with
// the epilogue, 1024 tokens 14.9 against 15.3; 2048 tokens 27.1 against 26.9, 4096 tokens 56.7 against 55.4).
static int addnorm_plan(int M, int N, int K, int* bt) {
  if (M > 256 && K % 8 == 0) {
    bool use_pair; int m_tiles, slots; lb::PrefillPlan pl;
    lb::prefill_choose(M, N, K, 0, 0, 0, &use_pair, &m_tiles, &slots, &pl);
    return (long long)m_tiles * lb::prefill_feature_tiles(pl, N) > slots ? -1 : 0;
  }
  if (M <= 0 || M > 256 || K % 8) return 0;
  int t = 16;
  int splits = lb_gemm_tcgen05_plan(M, N, K, &t);
  const int kb = (K + lb::BK - 1) / lb::BK;
  if (splits > kb) splits = kb;
  if (splits < 2 || splits > 8) return 0;
  if (bt) *bt = t;
  return splits;
}

LB_EXPORT int lb_gemm_tcgen05_addnorm_ok(int M, int N, int K) { return addnorm_plan(M, N, K, nullptr) != 0; }

// Columns of the partial sums of squares that lb_gemm_tcgen05_addnorm writes for these sizes (0: sizes it does not
// take): blocks of 128 features with few tokens, the feature tiles of the plan with many.
LB_EXPORT int lb_gemm_tcgen05_addnorm_tiles(int M, int N, int K) {
  const int plan = addnorm_plan(M, N, K, nullptr);
  if (plan == 0) return 0;
  if (plan > 0) return (N + lb::BM - 1) / lb::BM;
  bool use_pair; int m_tiles, slots; lb::PrefillPlan pl;
  lb::prefill_choose(M, N, K, 0, 0, 0, &use_pair, &m_tiles, &slots, &pl);
  return lb::prefill_feature_tiles(pl, N);
}

// x[M,K] . w[N,K]^T added to residual [M,N] (float32, in place); out [M,N] (bfloat16) receives residual * norm_w
// without the row's norm factor, sumsq [M, ceil(N/128)] the partial sums of squares of the new residual from which
// the reader of `out` forms that factor (see AddNormEpilogue, RowScale).
LB_EXPORT int lb_gemm_tcgen05_addnorm(const void* x, const void* w, int M, int N, int K, long long ldx, float* residual,
                                      const float* norm_w, void* out, float* sumsq, int sumsq_tiles, cudaStream_t stream) {
  int bt = 16;
  const int splits = addnorm_plan(M, N, K, &bt);
  LB_CHECK_ARG(splits != 0, "gemm_tcgen05_addnorm: sizes M=%d N=%d K=%d are not taken (many tokens, or a product that is split over a cluster)", M, N, K);
  LB_CHECK_ARG(residual && norm_w && out && sumsq, "gemm_tcgen05_addnorm: null argument");
  LB_CHECK_ARG(ldx >= K && ldx % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tcgen05_addnorm: operands must be 16-byte aligned");
  LB_CHECK_ARG(sumsq_tiles == lb_gemm_tcgen05_addnorm_tiles(M, N, K), "gemm_tcgen05_addnorm: %d columns of partial sums, these sizes write %d",
               sumsq_tiles, lb_gemm_tcgen05_addnorm_tiles(M, N, K));
  if (splits < 0) {
    LB_CHECK_ARG(((uintptr_t)residual % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)norm_w % 16 == 0),
                 "gemm_tcgen05_addnorm: residual, output and norm weight must be 16-byte aligned");
    lb::AddNormEpilogue an = {};
    an.on = 1; an.tiles = sumsq_tiles; an.residual = residual; an.norm_w = norm_w; an.out = (lb::bf16*)out; an.sumsq = sumsq;
    if (int rc = lb::launch_prefill(nullptr, LB_BF16, x, w, M, N, K, ldx, N, 0, 0, 0, stream, &an, nullptr)) return rc;
    LB_CHECK_LAUNCH("gemm_tcgen05_addnorm (many tokens)");
    return 0;
  }
  CUtensorMap mw, mx;
  if (!lb::cached_map(&mw, w, N, K, K, lb::BM) || !lb::cached_map(&mx, x, M, K, ldx, bt)) {
    lb::set_error("gemm_tcgen05_addnorm: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%lld)", M, N, K, ldx);
    return 3;
  }
  lb::GemmParams p;
  p.an.on = 1; p.an.tiles = (N + lb::BM - 1) / lb::BM; p.an.residual = residual; p.an.norm_w = norm_w;
  p.an.out = (lb::bf16*)out; p.an.sumsq = sumsq;
  p.y = nullptr; p.workspace = nullptr; p.counters = nullptr; p.M = M; p.N = N; p.K = K; p.ldy = N; p.out_dtype = LB_BF16;
  p.cluster = splits; p.swiglu = 0;
  if (int rc = lb::launch_for_tile(bt, mw, mx, p, splits, stream)) return rc;
  LB_CHECK_LAUNCH("gemm_tcgen05_addnorm");
  return 0;
}

// The plan of the q|k|v product with the head epilogue: token tile and splits, or 0 splits when the sizes do not
// allow it (it needs heads of 128, at most 32 tokens, and a split count whose CTAs form a cluster: the epilogue
// lives in the cluster's reduction).
static int heads_plan(int M, int N, int K, int head_dim, int* bt) {
  // Up to 32 tokens: there a CTA finishes at most 8 tokens one after the other.  With 64 tokens the separate kernel,
  // which spreads the heads over the whole GPU, was the faster of the two (decode step of 64 requests 19.3 against 19.7 ms).
  if (head_dim != lb::BM || N % lb::BM || M <= 0 || M > 32 || K % 8) return 0;
  int t = 16;
  int splits = lb_gemm_tcgen05_plan(M, N, K, &t);
  const int kb = (K + lb::BK - 1) / lb::BK;
  if (splits > kb) splits = kb;
  if (splits < 2 || splits > 8) return 0;
  if (bt) *bt = t;
  return splits;
}

// 1 when lb_gemm_tcgen05_heads takes these sizes.
LB_EXPORT int lb_gemm_tcgen05_heads_ok(int M, int N, int K, int head_dim) { return heads_plan(M, N, K, head_dim, nullptr) > 0; }

// The q|k|v product x[M,K] . w[N,K]^T with N = (num_q_heads + 2 num_kv_heads) * 128, whose epilogue norms and rotates
// the heads and writes queries to he->q_out and keys and values into their cache pages (see HeadEpilogue): the
// product's output is never stored as such.
LB_EXPORT int lb_gemm_tcgen05_heads(const void* x, const void* w, int M, int N, int K, long long ldx, const lb::HeadEpilogue* he,
                                    const lb::RowScale* row_scale, cudaStream_t stream) {
  int bt = 16;
  const int splits = heads_plan(M, N, K, lb::BM, &bt);
  LB_CHECK_ARG(splits > 0, "gemm_tcgen05_heads: sizes M=%d N=%d K=%d are not taken (heads of 128, up to 32 tokens, a split product)", M, N, K);
  LB_CHECK_ARG(he && he->positions && he->token_seq && he->block_table && he->q_out && he->k_cache && he->v_cache, "gemm_tcgen05_heads: null argument");
  LB_CHECK_ARG(N == (he->num_q_heads + 2 * he->num_kv_heads) * lb::BM && he->page_size > 0 && he->max_pages > 0,
               "gemm_tcgen05_heads: %d output features for %d + 2 x %d heads of 128", N, he->num_q_heads, he->num_kv_heads);
  LB_CHECK_ARG(ldx >= K && ldx % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tcgen05_heads: operands must be 16-byte aligned");
  CUtensorMap mw, mx;
  if (!lb::cached_map(&mw, w, N, K, K, lb::BM) || !lb::cached_map(&mx, x, M, K, ldx, bt)) {
    lb::set_error("gemm_tcgen05_heads: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%lld)", M, N, K, ldx);
    return 3;
  }
  lb::GemmParams p;
  p.he = *he; p.he.on = 1;
  if (row_scale) { p.rs = *row_scale; p.rs.on = 1; }
  p.y = nullptr; p.workspace = nullptr; p.counters = nullptr; p.M = M; p.N = N; p.K = K; p.ldy = N; p.out_dtype = LB_BF16;
  p.cluster = splits; p.swiglu = 0;
  if (int rc = lb::launch_for_tile(bt, mw, mx, p, splits, stream)) return rc;
  LB_CHECK_LAUNCH("gemm_tcgen05_heads");
  return 0;
}

// For tests of the give-up path.  The smallest launch of the few-token kernel (one CTA: up to 16 tokens x up to 128
// features, K not split, no cluster) with a producer that requests no tile at all and a wait limit of `wait_cycles`
// clock cycles: the issuing thread's first wait runs out, it records ERR_FULL_WAIT (101) in the device error flag, the
// other roles see the CTA's abort flag, nothing is stored to y, tensor memory is freed and the kernel returns.
// Nothing is in flight when the wait gives up, and the context stays usable.
LB_EXPORT int lb_gemm_tcgen05_wait_test(void* y, const void* x, const void* w, int M, int N, int K,
                                        unsigned long long wait_cycles, cudaStream_t stream) {
  LB_CHECK_ARG(M > 0 && M <= 16 && N > 0 && N <= lb::BM && K > 0 && K % 8 == 0, "gemm_tcgen05_wait_test: one tile only (M <= 16, N <= 128), K a multiple of 8");
  LB_CHECK_ARG(wait_cycles > 0 && wait_cycles <= lb::WAIT_CYCLES, "gemm_tcgen05_wait_test: the limit must be positive and at most the ordinary one");
  LB_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tcgen05_wait_test: operands must be 16-byte aligned");
  CUtensorMap mw, mx;
  if (!lb::make_map(&mw, w, N, K, K, lb::BM) || !lb::make_map(&mx, x, M, K, K, 16)) {
    lb::set_error("gemm_tcgen05_wait_test: cuTensorMapEncodeTiled failed");
    return 3;
  }
  lb::GemmParams p;
  p.y = y; p.workspace = nullptr; p.counters = nullptr; p.M = M; p.N = N; p.K = K; p.ldy = N; p.out_dtype = LB_BF16;
  p.cluster = 0; p.swiglu = 0; p.wait_cycles = wait_cycles; p.skip_loads = 1;
  if (int rc = lb::launch_for_tile(16, mw, mx, p, 1, stream)) return rc;
  LB_CHECK_LAUNCH("gemm_tcgen05_wait_test");
  return 0;
}

// Reads and clears the device error flag that kernels with bounded waits set when a wait gave up.
// Synchronises the device.  0: no error.
LB_EXPORT int lb_device_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, lb::g_device_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(lb::g_device_error, &zero, sizeof(int));
  return v;
}

// ---- the same product for callers that cannot allocate (see no_alloc.h) ---------------------------------
#include "no_alloc.h"

namespace lb {

// Scratch of the static-scratch entry point: tile counters first, then the float32 partial sums.
// One copy per device, held from the moment the library's code is loaded there until the process ends.
static __device__ __align__(256) unsigned char g_static_scratch[LB_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on each device, resolved at the first call there.
constexpr int MAX_DEVICES = 64;
static unsigned char* g_static_scratch_addr[MAX_DEVICES] = {};
static std::mutex g_static_scratch_mu;

// In host code `g_static_scratch` names a host-side handle; a kernel given that would read the wrong
// memory.  The runtime translates it for the device that is current.
static int static_scratch_address(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_error("gemm_tcgen05_static_scratch: cudaGetDevice failed: %s", cudaGetErrorString(e)); return 4; }
  if (dev < 0 || dev >= MAX_DEVICES) { set_error("gemm_tcgen05_static_scratch: device %d is beyond the %d this table holds", dev, MAX_DEVICES); return 4; }
  std::lock_guard<std::mutex> g(g_static_scratch_mu);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("gemm_tcgen05_static_scratch: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return 4;
    }
    g_static_scratch_addr[dev] = (unsigned char*)p;
  }
  *out = g_static_scratch_addr[dev];
  return 0;
}

}  // namespace lb

LB_EXPORT int lb_gemm_tcgen05_static_scratch(void* y, int y_dtype, const void* x, const void* w, int M, int N, int K,
                                             long long ldx, long long ldy, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(y_dtype), "gemm_tcgen05_static_scratch: bad output dtype %d", y_dtype);
  LB_CHECK_ARG(M >= 0 && N > 0 && K > 0 && ldx >= K && ldy >= N, "gemm_tcgen05_static_scratch: bad sizes M=%d N=%d K=%d", M, N, K);
  LB_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0, "gemm_tcgen05_static_scratch: K=%d and the row stride %lld must be multiples of 8", K, ldx);
  LB_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tcgen05_static_scratch: operands must be 16-byte aligned");
  if (M == 0) return 0;
  int bt = 16;
  int splits = lb_gemm_tcgen05_plan(M, N, K, &bt);
  const int kb = (K + lb::BK - 1) / lb::BK;
  if (splits > kb) splits = kb;
  const long long tiles = (long long)((N + lb::BM - 1) / lb::BM) * ((M + bt - 1) / bt);
  LB_CHECK_ARG((M + bt - 1) / bt <= 65535, "gemm_tcgen05_static_scratch: too many rows (%d)", M);
  float* partials = nullptr;
  int* counters = nullptr;
  if (splits > 1) {
    const long long need = (long long)splits * M * N;
    LB_CHECK_ARG(need <= LB_STATIC_SCRATCH_PARTIALS && tiles <= LB_STATIC_SCRATCH_COUNTERS,
                 "gemm_tcgen05_static_scratch: M=%d N=%d K=%d is split %d ways and needs %lld partial sums and %lld tile "
                 "counters; the built-in scratch holds %d and %d",
                 M, N, K, splits, need, tiles, LB_STATIC_SCRATCH_PARTIALS, LB_STATIC_SCRATCH_COUNTERS);
    unsigned char* base = nullptr;
    if (int rc = lb::static_scratch_address(&base)) return rc;
    counters = (int*)base;
    partials = (float*)(base + LB_STATIC_SCRATCH_COUNTERS * 4);
    // The counters must start at zero whatever an earlier call left behind.
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)tiles * sizeof(int), stream);
    if (e != cudaSuccess) { lb::set_error("gemm_tcgen05_static_scratch: clearing the counters failed: %s", cudaGetErrorString(e)); return 4; }
  }
  CUtensorMap mw, mx;                      // built for this call, on the stack
  if (!lb::make_map(&mw, w, N, K, K, lb::BM) || !lb::make_map(&mx, x, M, K, ldx, bt)) {
    lb::set_error("gemm_tcgen05_static_scratch: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%lld)", M, N, K, ldx);
    return 3;
  }
  lb::GemmParams p;
  p.y = y; p.workspace = partials; p.counters = counters; p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.out_dtype = y_dtype;
  p.cluster = 0;                           // this entry point is the workspace path, with the workspace built in
  p.swiglu = 0;
  if (int rc = lb::launch_for_tile(bt, mw, mx, p, splits, stream)) return rc;
  LB_CHECK_LAUNCH("gemm_tcgen05_static_scratch");
  return 0;
}
