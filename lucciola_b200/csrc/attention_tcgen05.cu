// Causal grouped-query attention for portions of prompts on the 5th-generation tensor cores
// (bfloat16, head size 128, page sizes 8..128 that divide 128).
//
// A work item is a run of up to 128/G consecutive tokens of one request and one kv head (G = query
// heads per kv head): its G*tokens query rows form a 128-row tile.  Keys and values are visited in
// blocks of 128 keys.  Per block
//     S = Q K^T          tcgen05.mma, both operands K-major from shared memory, S (128 x 128 float32) in
//                        tensor memory, two S buffers
//     P = softmax part   eight warps, TWO THREADS PER QUERY ROW (64 keys each): a thread reads its half of the
//                        row of S with one tcgen05.ld into registers, gives the S buffer back at once, needs
//                        no shuffles, exchanges the row's maximum with the other thread through shared
//                        memory, and writes its half of the row of P (bfloat16) into shared memory in the
//                        swizzled layout the tensor core reads
//     O_blk = P V        tcgen05.mma, P K-major, V MN-major (as it lies in the pages), two O buffers
//     O = O alpha + O_blk in registers of the row's threads (64 float32 columns each)
// The formulas are the online softmax of src/kernels/flash_attention.cu:246-298 of lucciola (m, l, o per
// row in 32-bit).  Keys and values come through TMA, one box per page and half of the head
// (cp.async.bulk.tensor.2d, 128-byte swizzle) into rings of two blocks, keys and values apart; the queries through one
// three-dimensional box per half (head size, heads of the group, tokens).
//
// Warp roles (320 threads): warp 0 producer (one thread), warp 1 tensor-core issue (one thread) and
// tensor-memory allocation, warps 2..9 softmax.  The softmax of block i+1 is computed before O_blk of
// block i is added, so that the tensor cores work on P V of block i and Q K^T of block i+2 meanwhile.
// Every wait on an mbarrier is bounded; when one gives up the CTA records it and leaves.
//
// Value rows outside the range a tile may see (past the last key, before the window, pages that were
// given back) are set to zero in shared memory before they are multiplied, so that whatever a reused
// page holds cannot reach a sum; scores there are set to -inf by assignment.
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace lb {

__device__ int g_attention_tc_error = 0;

constexpr int TA_D = 128;                 // head size
constexpr int TA_ROWS = 128;              // query rows of a tile
constexpr int TA_KEYS = 128;              // keys of a block
constexpr int TA_HALF_BYTES = 128 * 128;  // 128 rows of 128 bytes (64 bfloat16): one half of a 128-wide tile
constexpr int TA_TILE_BYTES = 2 * TA_HALF_BYTES;
constexpr unsigned long long TA_WAIT_CYCLES = 4000000000ull;

struct TcAttnParams {
  bf16* out;                                // [T, nq, d]
  const int* positions;                     // [T]
  const int* block_table; int max_pages;    // [S, max_pages]
  const int4* tiles;                        // {first token, tokens, request index, unused}
  int num_q_heads, num_kv_heads, group, page_size, page_shift, window;
  float scale_log2;
};

__device__ __forceinline__ uint32_t ta_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ta_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void ta_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ta_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool ta_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool ta_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (ta_mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    if (ta_mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag) return false;
      if ((unsigned long long)(clock64() - t0) > TA_WAIT_CYCLES) {
        *abort_flag = code;
        atomicCAS(&g_attention_tc_error, 0, code);
        return false;
      }
    }
  }
}
// The same for the single producer and issue threads: they sleep between polls, so that their spinning
// does not take issue slots from the softmax warps that share their schedulers.
__device__ __forceinline__ bool ta_mbar_wait_idle(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (ta_mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    __nanosleep(40);
    if (ta_mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if ((unsigned long long)(clock64() - t0) > TA_WAIT_CYCLES) {
        *abort_flag = code;
        atomicCAS(&g_attention_tc_error, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void ta_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void ta_tma_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t ta_desc_kmajor(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand, 128-byte swizzle: 64 contiguous elements of the N side per 128-byte row, the next 64
// `lbo` bytes further; rows are the K side, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t ta_desc_mnmajor(uint32_t addr, uint32_t lbo) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// D float32, A and B bfloat16, A K-major, B K-major (b_mn = 0) or MN-major (1), M = 128, N = 128.
__host__ __device__ constexpr uint32_t ta_idesc(int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void ta_umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ta_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ta_tmem_ld64(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}

enum : int { TA_ERR_Q = 301, TA_ERR_KV_FULL = 302, TA_ERR_KV_EMPTY = 303, TA_ERR_S_FULL = 304, TA_ERR_S_EMPTY = 305,
             TA_ERR_P_FULL = 306, TA_ERR_P_EMPTY = 307, TA_ERR_O_FULL = 308, TA_ERR_O_EMPTY = 309, TA_ERR_EXCHANGE = 310 };

// Shared memory: Q (2 halves) | K,V ring of 2 blocks (each K 2 halves, V 2 halves) | P (2 halves) | barriers
constexpr int TA_Q_OFF = 0;
constexpr int TA_KV_OFF = TA_TILE_BYTES;                       // 32 KB
constexpr int TA_KV_STAGE = 2 * TA_TILE_BYTES;                 // K then V: 64 KB
constexpr int TA_P_OFF = TA_KV_OFF + 2 * TA_KV_STAGE;          // 160 KB
constexpr int TA_BAR_OFF = TA_P_OFF + TA_TILE_BYTES;           // 192 KB
constexpr int TA_NUM_BARS = 20;
constexpr int TA_MAX_TILE_PAGES = 4096;                        // pages a tile's keys may span (32 K keys of 8-token pages)
constexpr int TA_PAGES_OFF = TA_BAR_OFF + TA_NUM_BARS * 8 + 16;
constexpr int TA_XCH_OFF = TA_PAGES_OFF + TA_MAX_TILE_PAGES * 4;   // maxima and sums that the two threads of a row exchange
constexpr int TA_SMEM_BYTES = TA_XCH_OFF + 2 * 2 * 128 * 4;
constexpr int TA_THREADS = 320;

__global__ void __launch_bounds__(TA_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = ta_smem_u32(smem);
  const uint32_t bars = sbase + TA_BAR_OFF;
  const uint32_t q_full = bars;
  auto k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bars + 8u * (3 + s); };
  auto v_full = [&](int s) { return bars + 8u * (16 + s); };
  auto v_empty = [&](int s) { return bars + 8u * (18 + s); };
  auto s_full = [&](int b) { return bars + 8u * (5 + b); };
  auto s_empty = [&](int b) { return bars + 8u * (7 + b); };
  const uint32_t p_full = bars + 8u * 9, p_empty = bars + 8u * 10;
  auto o_full = [&](int b) { return bars + 8u * (11 + b); };
  auto o_empty = [&](int b) { return bars + 8u * (13 + b); };
  const uint32_t x_bar = bars + 8u * 15;
  uint32_t* tmem_slot = (uint32_t*)(smem + TA_BAR_OFF + TA_NUM_BARS * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int4 tile = p.tiles[blockIdx.x];
  const int t0 = tile.x, ntok = tile.y, seq = tile.z;
  const int kvh = blockIdx.y, G = p.group;
  const int rows = ntok * G;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    ta_mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ta_mbar_init(k_full(i), 1); ta_mbar_init(k_empty(i), 1);
      ta_mbar_init(v_full(i), 1); ta_mbar_init(v_empty(i), 1);
      ta_mbar_init(s_full(i), 1); ta_mbar_init(s_empty(i), 8);
      ta_mbar_init(o_full(i), 1); ta_mbar_init(o_empty(i), 8);
    }
    ta_mbar_init(p_full, 8); ta_mbar_init(p_empty, 1);
    ta_mbar_init(x_bar, 8);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ta_smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;            // S0: +0, S1: +128, O0: +256, O1: +384 (columns)

  pdl_wait();                                   // everything below reads what earlier kernels wrote
  const int pos0 = p.positions[t0];
  const int pos_last = pos0 + ntok - 1;
  const int lo_tile = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kbeg = (lo_tile / TA_KEYS) * TA_KEYS;
  const int kend = pos_last + 1;                // exclusive
  const int nblocks = (kend - kbeg + TA_KEYS - 1) / TA_KEYS;
  const int* bt = p.block_table + (size_t)seq * p.max_pages;
  // The page ids of the keys this tile visits, copied once into shared memory for the producer.
  int* spages = reinterpret_cast<int*>(smem + TA_PAGES_OFF);
  const int first_page = kbeg >> p.page_shift;
  const int num_tile_pages = min(((kend - 1) >> p.page_shift) - first_page + 1, TA_MAX_TILE_PAGES);
  for (int i = threadIdx.x; i < num_tile_pages; i += blockDim.x) spages[i] = bt[first_page + i];
  __syncthreads();

  if (warp == 0) {
    // ---- producer: the whole warp; lane 0 waits and announces the bytes, every lane issues its share of the
    // boxes (a page and a half of the head, keys or values) -------------------------------------------------
    if (lane == 0) {
      ta_mbar_expect_tx(q_full, TA_TILE_BYTES);
      ta_tma_3d(sbase + TA_Q_OFF, &map_q, 0, kvh * G, t0, q_full);
      ta_tma_3d(sbase + TA_Q_OFF + TA_HALF_BYTES, &map_q, 64, kvh * G, t0, q_full);
    }
    const int pages_per_block = TA_KEYS / p.page_size;
    const uint32_t page_bytes = (uint32_t)p.page_size * 128u;       // one half of one page
    // Keys and values have rings and barriers of their own: the keys of block i+2 may come as soon as Q K^T of
    // block i is done, which is a whole block earlier than P V of block i gives the values' buffer back.
    for (int step = 0; step < 2 * nblocks; ++step) {
      const int i = step >> 1, is_v = step & 1, s = i & 1;
      int go = 1;
      if (lane == 0)
        go = ta_mbar_wait_idle(is_v ? v_empty(s) : k_empty(s), (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag, TA_ERR_KV_EMPTY) ? 1 : 0;
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go) break;
      const int kb = kbeg + i * TA_KEYS;
      const int* blk_pages = spages + ((kb - kbeg) >> p.page_shift);
      const uint32_t full = is_v ? v_full(s) : k_full(s);
      // pages of this block that exist and hold keys the tile may see
      int npages = 0;
      for (int pg = lane; pg < pages_per_block; pg += 32) {
        const bool seen = (kb + (pg + 1) * p.page_size > lo_tile) && (kb + pg * p.page_size < kend);
        npages += (seen && blk_pages[pg] >= 0) ? 1 : 0;
      }
      npages = __reduce_add_sync(0xffffffffu, npages);
      if (lane == 0) ta_mbar_expect_tx(full, (uint32_t)npages * page_bytes * 2u);
      __syncwarp();
      const uint32_t dst0 = sbase + TA_KV_OFF + s * TA_KV_STAGE + (is_v ? TA_TILE_BYTES : 0);
      const CUtensorMap* map = is_v ? &map_v : &map_k;
      for (int b = lane; b < pages_per_block * 2; b += 32) {
        const int pg = b >> 1, hf = b & 1;
        const bool seen = (kb + (pg + 1) * p.page_size > lo_tile) && (kb + pg * p.page_size < kend);
        const int page = seen ? blk_pages[pg] : -1;
        if (page < 0) continue;
        const int y = (page * p.num_kv_heads + kvh) * p.page_size;
        ta_tma_2d(dst0 + (uint32_t)hf * TA_HALF_BYTES + (uint32_t)pg * page_bytes, map, hf * 64, y, full);
      }
    }
  } else if (warp == 1) {
    // ---- tensor-core issue ---------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = ta_idesc(0), idesc_pv = ta_idesc(1);
      bool ok = ta_mbar_wait(q_full, 0, abort_flag, TA_ERR_Q);
      auto issue_qk = [&](int i) -> bool {
        const int s = i & 1;
        if (!ta_mbar_wait(k_full(s), (uint32_t)((i >> 1) & 1), abort_flag, TA_ERR_KV_FULL)) return false;
        if (!ta_mbar_wait(s_empty(s), (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag, TA_ERR_S_EMPTY)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t qa = sbase + TA_Q_OFF, ka = sbase + TA_KV_OFF + s * TA_KV_STAGE;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t o = (uint32_t)(k >> 2) * TA_HALF_BYTES + (uint32_t)(k & 3) * 32u;
          ta_umma(tmem + (uint32_t)s * 128u, ta_desc_kmajor(qa + o), ta_desc_kmajor(ka + o), idesc_qk, k != 0);
        }
        ta_commit(s_full(s));
        ta_commit(k_empty(s));
        return true;
      };
      if (ok && nblocks > 0) ok = issue_qk(0);
      for (int i = 0; i < nblocks && ok; ++i) {
        const int s = i & 1;
        if (i + 1 < nblocks) { ok = issue_qk(i + 1); if (!ok) break; }
        // O_blk(i) = P(i) V(i)
        ok = ta_mbar_wait(p_full, (uint32_t)(i & 1), abort_flag, TA_ERR_P_FULL);
        if (!ok) break;
        ok = ta_mbar_wait(o_empty(s), (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag, TA_ERR_O_EMPTY);
        if (!ok) break;
        ok = ta_mbar_wait(v_full(s), (uint32_t)((i >> 1) & 1), abort_flag, TA_ERR_KV_FULL);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t pa = sbase + TA_P_OFF, va = sbase + TA_KV_OFF + s * TA_KV_STAGE + TA_TILE_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t po = (uint32_t)(k >> 2) * TA_HALF_BYTES + (uint32_t)(k & 3) * 32u;     // 16 keys further in P's rows
          const uint32_t vo = (uint32_t)k * 16u * 128u;                                           // 16 key rows further in V
          ta_umma(tmem + 256u + (uint32_t)s * 128u, ta_desc_kmajor(pa + po), ta_desc_mnmajor(va + vo, TA_HALF_BYTES), idesc_pv, k != 0);
        }
        ta_commit(o_full(s));
        ta_commit(p_empty);
        ta_commit(v_empty(s));
      }
    }
  } else {
    // ---- softmax: eight warps; warp w reads lanes (w % 4) * 32 .. + 31 of tensor memory, so two warps share a
    // quarter of the rows: the first four warps take keys 0..63 of a block and columns 0..63 of O, the other four
    // the upper halves.  The two threads of a row exchange their maxima through shared memory once a block and
    // their sums once at the end; everything else they do alone. ------------------------------------------------
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;                       // row of the tile
    const uint32_t tlane = (uint32_t)(quarter * 32) << 16;
    const uint32_t tcol = (uint32_t)half * 64u;
    const int row_pos = r < rows ? pos0 + r / G : -1;
    const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
    float* xch = reinterpret_cast<float*>(smem + TA_XCH_OFF);          // [2 block parities][2 halves][128 rows]
    float o_acc[TA_D / 2];
#pragma unroll
    for (int i = 0; i < TA_D / 2; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    bool ok = true;

    // gives this thread's value to the row's other thread and returns that thread's value (exchange number i)
    auto exchange = [&](int i, float mine, float& other) -> bool {
      float* slot = xch + (i & 1) * 256;
      slot[half * 128 + r] = mine;
      __syncwarp();
      if (lane == 0) ta_mbar_arrive(x_bar);
      if (!ta_mbar_wait(x_bar, (uint32_t)(i & 1), abort_flag, TA_ERR_EXCHANGE)) return false;
      other = slot[(half ^ 1) * 128 + r];
      return true;
    };

    auto accumulate = [&](int i, float alpha) -> bool {      // O = O * alpha + O_blk(i), this thread's 64 columns
      const int s = i & 1;
      if (!ta_mbar_wait(o_full(s), (uint32_t)((i >> 1) & 1), abort_flag, TA_ERR_O_FULL)) return false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t v[64];
      ta_tmem_ld64(tmem + tlane + 256u + (uint32_t)s * 128u + tcol, v);
#pragma unroll
      for (int j = 0; j < 64; ++j) o_acc[j] = fmaf(o_acc[j], alpha, __uint_as_float(v[j]));
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) ta_mbar_arrive(o_empty(s));
      return true;
    };

    // Iteration i: the softmax of block i (if there is one), then the addition of block i-1's O_blk.
    for (int i = 0; i <= nblocks && ok; ++i) {
      float alpha = 1.f;
      if (i < nblocks) do {
      const int s = i & 1;
      const int kb = kbeg + i * TA_KEYS;
      ok = ta_mbar_wait(s_full(s), (uint32_t)((i >> 1) & 1), abort_flag, TA_ERR_S_FULL);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool need_mask = (kb + TA_KEYS - 1 > pos0) || (p.window > 0) || (kb < lo_tile) || (kb + TA_KEYS > kend);
      // this thread's 64 scores into registers; the S buffer goes back to the tensor cores at once
      float x[64];
      {
        uint32_t v[64];
        ta_tmem_ld64(tmem + tlane + (uint32_t)s * 128u + tcol, v);
#pragma unroll
        for (int j = 0; j < 64; ++j) x[j] = __uint_as_float(v[j]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) ta_mbar_arrive(s_empty(s));
      float mx = -INFINITY;
      if (need_mask) {
        const int key0 = kb + half * 64;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int key = key0 + j;
          if (key > row_pos || key < row_lo) x[j] = -INFINITY;
        }
      }
#pragma unroll
      for (int j = 0; j < 64; ++j) mx = fmaxf(mx, x[j]);
      float other;
      ok = exchange(i, mx, other);
      if (!ok) break;
      const float m_new = fmaxf(m_run, fmaxf(mx, other));
      const float m_use = m_new == -INFINITY ? 0.f : m_new * p.scale_log2;
      alpha = m_run == -INFINITY ? 0.f : exp2f(m_run * p.scale_log2 - m_use);
      m_run = m_new;
      // the P buffer is free once P V of the previous block has been read by the tensor cores
      if (i > 0) { ok = ta_mbar_wait(p_empty, (uint32_t)((i - 1) & 1), abort_flag, TA_ERR_P_EMPTY); if (!ok) break; }
      // p = 2^(s * scale - m), the sum over this thread's keys, its half of the row of P into shared memory
      // (K-major, swizzled: the 16-byte chunk index within the 128-byte row is permuted by the row)
      float sum = 0.f;
      uint8_t* prow = smem + TA_P_OFF + half * TA_HALF_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float p0 = exp2_approx(fmaf(x[8 * c + 2 * j], p.scale_log2, -m_use));
          const float p1 = exp2_approx(fmaf(x[8 * c + 2 * j + 1], p.scale_log2, -m_use));
          sum += p0 + p1;
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
          w[j] = *reinterpret_cast<uint32_t*>(&b2);
        }
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_run = l_run * alpha + sum;
      // value rows the tile may not see hold whatever the page or the shared memory held: zero them
      // (keys before the window's first key and keys past the last one; 16 threads a row)
      if ((kb < lo_tile) || (kb + TA_KEYS > kend)) {
        ok = ta_mbar_wait(v_full(s), (uint32_t)((i >> 1) & 1), abort_flag, TA_ERR_KV_FULL);     // the values have landed
        if (!ok) break;
        uint8_t* vb = smem + TA_KV_OFF + s * TA_KV_STAGE + TA_TILE_BYTES;
        const int head_rows = min(max(lo_tile - kb, 0), TA_KEYS), tail_from = min(max(kend - kb, 0), TA_KEYS);
        const int idx = (warp - 2) * 32 + lane, chunk = idx & 15;
        for (int key = idx >> 4; key < TA_KEYS; key += 16) {
          if (key < head_rows || key >= tail_from)
            *reinterpret_cast<uint4*>(vb + (chunk >> 3) * TA_HALF_BYTES + key * 128 + ((chunk & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      // hand P (and the cleaned V) to the tensor cores
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) ta_mbar_arrive(p_full);
      } while (0);
      if (!ok) break;
      // add the previous block's O_blk while the tensor cores work on this one
      if (i > 0) ok = accumulate(i - 1, alpha_prev);
      alpha_prev = alpha;
    }
    float l_other = 0.f;
    if (ok) ok = exchange(nblocks, l_run, l_other);
    if (ok && r < rows) {
      const float l = l_run + l_other;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int token = t0 + r / G, head = kvh * G + r % G;
      uint4* dst = reinterpret_cast<uint4*>(p.out + ((size_t)token * p.num_q_heads + head) * TA_D + half * 64);
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 b2 = __floats2bfloat162_rn(o_acc[c + 2 * j] * inv, o_acc[c + 2 * j + 1] * inv);
          w[j] = *reinterpret_cast<uint32_t*>(&b2);
        }
        dst[c >> 3] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------------------------
typedef CUresult (*TaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TaEncodeFn ta_encode_fn() {
  static TaEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (TaEncodeFn)sym;
  });
  return fn;
}

struct TaMapKey {
  const void* base; long long a, b, c; int kind;
  bool operator==(const TaMapKey& o) const { return base == o.base && a == o.a && b == o.b && c == o.c && kind == o.kind; }
};
struct TaMapKeyHash {
  size_t operator()(const TaMapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    h = h * 1000003u ^ (size_t)k.a; h = h * 1000003u ^ (size_t)k.b; h = h * 1000003u ^ (size_t)k.c; h = h * 1000003u ^ (size_t)k.kind;
    return h;
  }
};
static std::unordered_map<TaMapKey, CUtensorMap, TaMapKeyHash> g_ta_maps;
static std::mutex g_ta_mu;

// Keys or values of one cache layer: [pages * kv_heads * page_size, 128] bfloat16, boxes of page_size rows x 64.
static bool ta_pool_map(CUtensorMap* out, const void* pool, long long rows, int page_size) {
  TaMapKey key{pool, rows, page_size, 0, 1};
  std::lock_guard<std::mutex> g(g_ta_mu);
  auto it = g_ta_maps.find(key);
  if (it != g_ta_maps.end()) { *out = it->second; return true; }
  TaEncodeFn fn = ta_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {128, (cuuint64_t)rows};
  cuuint64_t strides[1] = {256};
  cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  cuuint32_t estr[2] = {1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (g_ta_maps.size() > 4096) g_ta_maps.clear();
  g_ta_maps.emplace(key, *out);
  return true;
}

// Queries [T, nq, 128]: boxes of 64 x G heads x (128 / G) tokens; rows of a box are (token, head of the group).
static bool ta_q_map(CUtensorMap* out, const void* q, long long tokens, int num_q_heads, int group) {
  TaMapKey key{q, tokens, num_q_heads, group, 2};
  std::lock_guard<std::mutex> g(g_ta_mu);
  auto it = g_ta_maps.find(key);
  if (it != g_ta_maps.end()) { *out = it->second; return true; }
  TaEncodeFn fn = ta_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {128, (cuuint64_t)num_q_heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {256, (cuuint64_t)num_q_heads * 256};
  cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(128 / group)};
  cuuint32_t estr[3] = {1, 1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (g_ta_maps.size() > 4096) g_ta_maps.clear();
  g_ta_maps.emplace(key, *out);
  return true;
}

}  // namespace lb

// 1 when lb_attention_tcgen05 takes these sizes.
LB_EXPORT int lb_attention_tcgen05_ok(int num_q_heads, int num_kv_heads, int head_dim, int page_size) {
  if (head_dim != 128 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return 0;
  const int g = num_q_heads / num_kv_heads;
  if (g > 128 || 128 % g) return 0;                          // the query box is G heads x 128/G tokens
  if (page_size < 8 || page_size > 128 || 128 % page_size || (page_size & (page_size - 1))) return 0;
  return 1;
}

// q, out: [T, nq, 128] bfloat16.  k_cache, v_cache: [pages, nkv, page_size, 128].  tiles: {first token,
// tokens, request index, 0} with tokens * (nq / nkv) <= 128.
LB_EXPORT int lb_attention_tcgen05(const void* q, void* out, const void* k_cache, const void* v_cache, const int* positions,
                                   const int* block_table, const void* tiles, int num_tiles, int num_tokens,
                                   int num_q_heads, int num_kv_heads, int head_dim, int page_size, int num_pages,
                                   int max_pages, int window, float scale, cudaStream_t stream) {
  LB_CHECK_ARG(lb_attention_tcgen05_ok(num_q_heads, num_kv_heads, head_dim, page_size),
               "attention_tcgen05: needs head_dim 128, a group size that divides 128 and a page size among 8, 16, 32, 64, 128 "
               "(got head_dim %d, %d/%d heads, pages of %d)", head_dim, num_q_heads, num_kv_heads, page_size);
  LB_CHECK_ARG(max_pages > 0 && window >= 0 && num_tokens > 0 && num_pages > 0, "attention_tcgen05: bad sizes");
  LB_CHECK_ARG(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) && ((uintptr_t)out % 16 == 0),
               "attention_tcgen05: operands must be 16-byte aligned");
  if (num_tiles == 0) return 0;
  LB_CHECK_ARG(max_pages <= lb::TA_MAX_TILE_PAGES, "attention_tcgen05: a request may span %d pages, at most %d", max_pages, lb::TA_MAX_TILE_PAGES);
  const int group = num_q_heads / num_kv_heads;
  CUtensorMap mq, mk, mv;
  const long long pool_rows = (long long)num_pages * num_kv_heads * page_size;
  if (!lb::ta_q_map(&mq, q, num_tokens, num_q_heads, group) || !lb::ta_pool_map(&mk, k_cache, pool_rows, page_size) ||
      !lb::ta_pool_map(&mv, v_cache, pool_rows, page_size)) {
    lb::set_error("attention_tcgen05: cuTensorMapEncodeTiled failed");
    return 3;
  }
  lb::TcAttnParams p;
  p.out = (lb::bf16*)out; p.positions = positions; p.block_table = block_table; p.max_pages = max_pages;
  p.tiles = (const int4*)tiles; p.num_q_heads = num_q_heads; p.num_kv_heads = num_kv_heads; p.group = group;
  p.page_size = page_size; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  const int smem = lb::TA_SMEM_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(lb::attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { lb::set_error("attention_tcgen05: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e)); return 2; }
    configured = true;
  }
  lb::launch(lb::attention_tcgen05_kernel, dim3(num_tiles, num_kv_heads), dim3(lb::TA_THREADS), smem, stream, mq, mk, mv, p);
  LB_CHECK_LAUNCH("attention_tcgen05");
  return 0;
}

// Reads and clears the flag a bounded wait of this kernel sets when it gives up (0: none).
LB_EXPORT int lb_attention_tcgen05_device_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, lb::g_attention_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(lb::g_attention_tc_error, &zero, sizeof(int));
  return v;
}
