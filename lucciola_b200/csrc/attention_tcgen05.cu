// Causal grouped-query attention for portions of prompts on the 5th-generation tensor cores
// (bfloat16, head size 128, page sizes 8..128 that are powers of two).
//
// A work item is a run of up to 2 * floor(128/G) consecutive tokens of one request and one kv head (G = query
// heads per kv head): its G*tokens query rows form TWO tiles of up to 128 rows, A and B, that share the keys
// and values the CTA loads (half the traffic from L2 per query row).  Keys and values are visited in
// blocks of 64 keys.  Per block and tile
//     S = Q K^T          tcgen05.mma, both operands K-major from shared memory, S (128 x 64 float32) in
//                        tensor memory, TWO S buffers a tile: Q K^T of block i+1 is done while the softmax
//                        of block i runs
//     P = softmax part   four warps, ONE THREAD PER QUERY ROW: the thread reads its row of S with tcgen05.ld,
//                        needs no shuffles for the row's maximum and sum, and writes its row of P (bfloat16,
//                        two keys a column) with tcgen05.st over the first 32 columns of that S buffer
//     O += P V           tcgen05.mma, P from TENSOR MEMORY, V MN-major from shared memory (as it lies in the
//                        pages), O (128 x 128 float32) accumulated in tensor memory over all blocks
// The formulas are the online softmax of src/kernels/flash_attention.cu:246-298 of lucciola (m, l, o per
// row in 32-bit), with one change of bookkeeping: the reference value m that the exponentials are taken
// against follows the row's maximum only when that has grown by more than 2^8, so that O in tensor memory
// is rescaled (tcgen05.ld, multiply, tcgen05.st by the row's thread) a few times per row instead of once
// per block; p <= 2^8 then, and O / l is the same quotient whatever m was.
// The queries come through TMA, one three-dimensional box per tile and half (head size, heads of the
// group, tokens).  Keys and values come through cp.async, 16 bytes a thread and instruction, written in the
// 128-byte swizzle the tensor cores read, into rings of four blocks, keys and values apart, one warp each
// with three blocks in flight: with pages of 16 tokens a TMA box is 2 KB, a CTA issues a box in about 125
// cycles, and the boxes alone took longer than the tensor cores need for a block.
//
// Warp roles (384 threads): warp 0 loads the queries and the keys, warp 10 the values; warp 1 issues tile A's
// products to the tensor cores (one thread) and owns the tensor memory, warp 11 issues tile B's; warps 2..5
// softmax of tile A, warps 6..9 of tile B.  One issuing thread per tile, because between two products of a
// tile stand three waits and as many commits: with one thread for both tiles those alone filled the time the
// tensor cores need for a block.  The tensor cores execute what one thread issues in order, which is what
// orders P V of block i before Q K^T of block i+2 overwrites the columns P lies in.
// Every wait on an mbarrier is bounded; when one gives up the CTA records it and leaves.
//
// Key and value rows outside the range a work item may see (past the last key, before the window, pages
// that were given back) are filled with zeros instead of being read, so that whatever a reused page holds
// cannot reach a sum; scores there are set to -inf by assignment.
//
// A CTA takes a whole SM, and a work item walks all the keys its tokens see: a portion of a few hundred tokens
// behind a long context makes fewer items than the GPU has SMs, each as long as the context.  Such a launch cuts
// the blocks of every item into gridDim.z ranges, one CTA each; a CTA then leaves its rows unnormalised, with
// their reference value and sum, in a float32 workspace, and ta_combine_kernel weighs the ranges of a row by
// 2^(m - M) in the ranges' order.  A range may be empty (an item that sees few keys): it leaves (-inf, 0) and no
// rows, and the combining kernel does not read what it did not write.
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace lb {

__device__ int g_attention_tc_error = 0;

constexpr int TA_D = 128;                 // head size
constexpr int TA_ROWS = 128;              // query rows of a tile
constexpr int TA_KEYS = 64;               // keys of a block
constexpr int TA_HALF_BYTES = 128 * 128;  // 128 rows of 128 bytes (64 bfloat16): one half of a 128-wide tile
constexpr int TA_TILE_BYTES = 2 * TA_HALF_BYTES;
constexpr unsigned long long TA_WAIT_CYCLES = 4000000000ull;

struct TcAttnParams {
  bf16* out;                                // [T, nq, d]
  const uint8_t* k_cache; const uint8_t* v_cache;   // [pages, nkv, page_size, d] bfloat16
  const int* positions;                     // [T]
  const int* block_table; int max_pages;    // [S, max_pages]
  const int4* tiles;                        // {first token, tokens, request index, unused}
  int num_q_heads, num_kv_heads, group, page_size, page_shift, window;
  float scale_log2;
  // With gridDim.z > 1 the keys of every work item are cut into gridDim.z ranges of whole blocks, one CTA each; a CTA
  // then leaves its rows unnormalised, with their reference value and sum, for ta_combine_kernel:
  float* part_o;                            // [(item * kv heads + kv head) * ranges + range][TA_PART_ROWS][d] float32
  float* part_ml;                           // [...][TA_PART_ROWS][2]: reference value (log2 domain, -inf: no key seen), sum
};
constexpr int TA_PART_ROWS = 256;           // rows of a work item in the partial results: (token of the item, head of the group)

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
// D float32, A and B bfloat16, A K-major, B K-major (b_mn = 0) or MN-major (1), M = 128, N = n.
__host__ __device__ constexpr uint32_t ta_idesc(int b_mn, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
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

__device__ __forceinline__ void ta_tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// The caller waits with ta_tmem_wait_st() before it tells anyone.
__device__ __forceinline__ void ta_tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      :: "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void ta_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// A from tensor memory (rows on lanes, two bfloat16 of the K side a column), B from shared memory.
__device__ __forceinline__ void ta_umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

// Two float32 in one 64-bit register for the packed instructions of sm_100 (one issue slot for two elements).
__device__ __forceinline__ uint64_t ta_pack2(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void ta_unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t ta_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d;
}
__device__ __forceinline__ uint64_t ta_add2(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ float ta_max3(float a, float b, float c) { float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
// Which wait gave up (what lb_attention_tcgen05_device_error reports).
enum : int { TA_ERR_Q = 301, TA_ERR_KV_FULL = 302, TA_ERR_KV_EMPTY = 303, TA_ERR_S_FULL = 304, TA_ERR_P_FULL = 306, TA_ERR_O_FULL = 308 };

// Shared memory: Q of tile A, Q of tile B | K ring of 4 blocks | V ring of 4 blocks | barriers | page ids.
// A tile of R rows x 128 bfloat16 is two halves of R rows x 128 bytes (64 elements); within a half the 16-byte
// chunk c of row r lies at r * 128 + ((c ^ (r & 7)) << 4).  R = 128 for Q, 64 for a block of keys or values.
constexpr int TA_STAGES = 4;
constexpr int TA_KV_HALF = TA_KEYS * 128;                      // one half of a block of keys: 8 KB
constexpr int TA_KV_TILE = 2 * TA_KV_HALF;                     // 16 KB
constexpr int TA_Q_OFF = 0;
constexpr int TA_K_OFF = 2 * TA_TILE_BYTES;                    // 64 KB
constexpr int TA_V_OFF = TA_K_OFF + TA_STAGES * TA_KV_TILE;    // 128 KB
constexpr int TA_BAR_OFF = TA_V_OFF + TA_STAGES * TA_KV_TILE;  // 192 KB
constexpr int TA_NUM_BARS = 1 + 4 * TA_STAGES + 2 * 6;
constexpr int TA_MAX_TILE_PAGES = 4096;                        // pages a tile's keys may span (32 K keys of 8-token pages)
constexpr int TA_PAGES_OFF = TA_BAR_OFF + TA_NUM_BARS * 8 + 16;
constexpr int TA_SMEM_BYTES = TA_PAGES_OFF + TA_MAX_TILE_PAGES * 4;
constexpr int TA_THREADS = 384;
constexpr int TA_IN_FLIGHT = 2;                                // blocks a producer warp has requested beyond the one it waits for
constexpr float TA_RESCALE_STEP = 8.f;                         // log2 of the growth of a row's maximum that moves its reference

// One block of 64 keys (or values) of one kv head from the pages into a stage of the ring, by one warp.  A lane
// copies chunk c (16 bytes) of every second row: rows rp, rp + 2, ...  `ring_lane` is the stage's address plus the
// lane's fixed part (its half of the head and row rp); xr[u] the swizzled chunk offset of the rows rp + 2u (mod 8).
// Rows the work item may not see, and pages that are not there, are filled with zeros.  PS: tokens of a page, at
// most 64 here (a page of 128 is walked as two of 64: `sub` is the half the block lies in).
template <int PS>
__device__ __forceinline__ void ta_copy_block(uint32_t ring_lane, const uint32_t (&xr)[4], const uint8_t* pool_lane, const int* blk_pages,
                                              int kb, int lo_tile, int kend, size_t page_stride, size_t head_off, int rp, int sub) {
  const bool inner = kb >= lo_tile && kb + TA_KEYS <= kend;           // every key of the block may be seen
  uint32_t dst_u[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) dst_u[u] = ring_lane + xr[u];
#pragma unroll
  for (int pg = 0; pg < TA_KEYS / PS; ++pg) {
    const int key0 = kb + pg * PS;
    const int page = (inner || (key0 + PS > lo_tile && key0 < kend)) ? blk_pages[pg] : -1;
    const uint8_t* src = pool_lane + (size_t)max(page, 0) * page_stride + head_off + (size_t)sub * (64 * 256);
#pragma unroll
    for (int j = 0; j < PS / 2; ++j) {
      const int key = key0 + rp + 2 * j;
      const uint32_t bytes = (page >= 0 && (inner || (key >= lo_tile && key < kend))) ? 16u : 0u;       // 0: sixteen zeros
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                   ::"r"(dst_u[j & 3] + (uint32_t)(pg * PS * 128 + j * 256)), "l"(src + (size_t)j * 512u), "r"(bytes) : "memory");
    }
  }
}

__global__ void __launch_bounds__(TA_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = ta_smem_u32(smem);
  const uint32_t bars = sbase + TA_BAR_OFF;
  const uint32_t q_full = bars;
  auto k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bars + 8u * (1 + TA_STAGES + s); };
  auto v_full = [&](int s) { return bars + 8u * (1 + 2 * TA_STAGES + s); };
  auto v_empty = [&](int s) { return bars + 8u * (1 + 3 * TA_STAGES + s); };
  // per tile t and S buffer b: S complete, P written, P V complete
  auto s_full = [&](int t, int b) { return bars + 8u * (1 + 4 * TA_STAGES + t * 6 + b); };
  auto p_full = [&](int t, int b) { return bars + 8u * (1 + 4 * TA_STAGES + t * 6 + 2 + b); };
  auto pv_done = [&](int t, int b) { return bars + 8u * (1 + 4 * TA_STAGES + t * 6 + 4 + b); };
  uint32_t* tmem_slot = (uint32_t*)(smem + TA_BAR_OFF + TA_NUM_BARS * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int4 tile = p.tiles[blockIdx.y];        // kv heads run fastest: the tiles come heaviest first over the whole grid
  const int t0 = tile.x, ntok = tile.y, seq = tile.z;
  const int kvh = blockIdx.x, G = p.group;
  const int per = TA_ROWS / G;                  // tokens of a 128-row tile
  const bool two = ntok > per;                  // is there a tile B
  const int ntiles = two ? 2 : 1;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    ta_mbar_init(q_full, 1);
    for (int i = 0; i < TA_STAGES; ++i) {
      ta_mbar_init(k_full(i), 1); ta_mbar_init(k_empty(i), ntiles);       // a stage goes back when every tile's product has read it
      ta_mbar_init(v_full(i), 1); ta_mbar_init(v_empty(i), ntiles);
    }
    for (int t = 0; t < 2; ++t)
      for (int b = 0; b < 2; ++b) { ta_mbar_init(s_full(t, b), 1); ta_mbar_init(p_full(t, b), 4); ta_mbar_init(pv_done(t, b), 1); }
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
  const uint32_t tmem = *tmem_slot;            // columns: tile t's S buffers at t * 128 and t * 128 + 64 (P over their first 32), O at 256 + t * 128

  // Positions and block tables were written before the step began: they are read while the kernel ahead may still run.
  const int pos0 = p.positions[t0];
  const int pos_last = pos0 + ntok - 1;
  const int lo_tile = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int kbeg_all = (lo_tile / TA_KEYS) * TA_KEYS;
  const int kend_all = pos_last + 1;            // exclusive
  const int nblocks_all = (kend_all - kbeg_all + TA_KEYS - 1) / TA_KEYS;
  // This CTA's range of blocks (all of them unless the keys are split; a range may be empty when the item sees few keys).
  const int nsplit = gridDim.z, isplit = blockIdx.z;
  const int blk0 = (int)((long long)nblocks_all * isplit / nsplit), blk1 = (int)((long long)nblocks_all * (isplit + 1) / nsplit);
  const int kbeg = kbeg_all + blk0 * TA_KEYS;
  const int kend = min(kend_all, kbeg_all + blk1 * TA_KEYS);       // keys from here on belong to the next range, or are not there
  const int nblocks = blk1 - blk0;
  const int* bt = p.block_table + (size_t)seq * p.max_pages;
  // The page ids of the keys this work item visits, copied once into shared memory for the producers.
  int* spages = reinterpret_cast<int*>(smem + TA_PAGES_OFF);
  const int first_page = kbeg >> p.page_shift;
  const int num_tile_pages = min(((kend - 1) >> p.page_shift) - first_page + 1, TA_MAX_TILE_PAGES);
  for (int i = threadIdx.x; i < num_tile_pages; i += blockDim.x) spages[i] = bt[first_page + i];
  __syncthreads();
  pdl_wait();                                   // the queries, keys and values below are what earlier kernels wrote

  if (nblocks <= 0) {
    // ---- an empty range of a split item: its rows weigh nothing in the combination -------------------------------
    if (warp >= 2 && warp < 10) {
      const int t = (warp - 2) >> 2, r = (warp & 3) * 32 + lane;
      const int tok_in_item = t * per + r / G;
      if (r < per * G && tok_in_item < ntok) {
        const size_t prow = (((size_t)blockIdx.y * p.num_kv_heads + kvh) * nsplit + isplit) * TA_PART_ROWS + tok_in_item * G + r % G;
        p.part_ml[prow * 2] = -INFINITY;
        p.part_ml[prow * 2 + 1] = 0.f;
      }
    }
  } else if (warp == 0 || warp == 10) {
    // ---- producers: warp 0 the queries (TMA) and the keys, warp 10 the values ---------------------------------
    const bool is_v = warp == 10;
    if (!is_v && lane == 0) {
      ta_mbar_expect_tx(q_full, (uint32_t)(ntiles * G * per) * 256u);      // a tile's box: G * per rows of 256 bytes, in two halves
      for (int t = 0; t < ntiles; ++t) {
        ta_tma_3d(sbase + TA_Q_OFF + t * TA_TILE_BYTES, &map_q, 0, kvh * G, t0 + t * per, q_full);
        ta_tma_3d(sbase + TA_Q_OFF + t * TA_TILE_BYTES + TA_HALF_BYTES, &map_q, 64, kvh * G, t0 + t * per, q_full);
      }
    }
    const int ps = p.page_size;
    const int c = lane & 15, rp = lane >> 4;
    const uint8_t* pool_lane = (is_v ? p.v_cache : p.k_cache) + c * 16 + rp * 256;
    const size_t page_stride = (size_t)p.num_kv_heads * ps * 256u, head_off = (size_t)kvh * ps * 256u;
    uint32_t xr[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) xr[u] = (uint32_t)(((c & 7) ^ ((rp + 2 * u) & 7)) << 4);
    const uint32_t ring = sbase + (is_v ? TA_V_OFF : TA_K_OFF) + (uint32_t)(c >> 3) * TA_KV_HALF + (uint32_t)rp * 128u;
    // Block i is requested, then block i - TA_IN_FLIGHT is waited for and handed over: three blocks in flight.
    bool go_on = true;
    for (int i = 0; i < nblocks + TA_IN_FLIGHT && go_on; ++i) {
      if (i < nblocks) {
        const int s = i % TA_STAGES;
        int go = 1;
        if (lane == 0)
          go = ta_mbar_wait_idle(is_v ? v_empty(s) : k_empty(s), (uint32_t)((i / TA_STAGES) & 1) ^ 1u, abort_flag, TA_ERR_KV_EMPTY) ? 1 : 0;
        go = __shfl_sync(0xffffffffu, go, 0);
        if (!go) { go_on = false; break; }
        const int kb = kbeg + i * TA_KEYS;
        const int* blk_pages = spages + ((kb >> p.page_shift) - first_page);
        const uint32_t stage = ring + (uint32_t)s * TA_KV_TILE;
        switch (ps) {
          case 8: ta_copy_block<8>(stage, xr, pool_lane, blk_pages, kb, lo_tile, kend, page_stride, head_off, rp, 0); break;
          case 16: ta_copy_block<16>(stage, xr, pool_lane, blk_pages, kb, lo_tile, kend, page_stride, head_off, rp, 0); break;
          case 32: ta_copy_block<32>(stage, xr, pool_lane, blk_pages, kb, lo_tile, kend, page_stride, head_off, rp, 0); break;
          default: ta_copy_block<64>(stage, xr, pool_lane, blk_pages, kb, lo_tile, kend, page_stride, head_off, rp, ps == 128 ? (kb >> 6) & 1 : 0); break;
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");          // (an empty group past the last block)
      if (i >= TA_IN_FLIGHT) {
        // block i - TA_IN_FLIGHT has landed: make it visible to the tensor cores' reads, then say so
        asm volatile("cp.async.wait_group %0;" ::"n"(TA_IN_FLIGHT) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        const int s = (i - TA_IN_FLIGHT) % TA_STAGES;
        if (lane == 0) ta_mbar_arrive(is_v ? v_full(s) : k_full(s));
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == 1 || warp == 11) {
    // ---- tensor-core issue, one thread per tile --------------------------------------------------------------
    const int t = warp == 1 ? 0 : 1;
    if (lane == 0 && t < ntiles) {
      constexpr uint32_t idesc_qk = ta_idesc(0, TA_KEYS), idesc_pv = ta_idesc(1, TA_D);
      const uint32_t s_col = tmem + (uint32_t)t * 128u, o_col = tmem + 256u + (uint32_t)t * 128u;
      const uint32_t qa = sbase + TA_Q_OFF + t * TA_TILE_BYTES;
      bool ok = ta_mbar_wait(q_full, 0, abort_flag, TA_ERR_Q);
      // S(j) = Q K(j)^T into S buffer j & 1; the keys' stage goes back when every tile's product is done
      auto issue_qk = [&](int j) -> bool {
        const int s = j % TA_STAGES;
        if (!ta_mbar_wait(k_full(s), (uint32_t)((j / TA_STAGES) & 1), abort_flag, TA_ERR_KV_FULL)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t ka = sbase + TA_K_OFF + s * TA_KV_TILE;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          ta_umma(s_col + (uint32_t)(j & 1) * 64u, ta_desc_kmajor(qa + (uint32_t)(k >> 2) * TA_HALF_BYTES + (uint32_t)(k & 3) * 32u),
                  ta_desc_kmajor(ka + (uint32_t)(k >> 2) * TA_KV_HALF + (uint32_t)(k & 3) * 32u), idesc_qk, k != 0);
        ta_commit(s_full(t, j & 1));
        ta_commit(k_empty(s));
        return true;
      };
      for (int j = 0; j < 2 && j < nblocks && ok; ++j) ok = issue_qk(j);
      for (int i = 0; i < nblocks && ok; ++i) {
        const int s = i % TA_STAGES, b = i & 1;
        // O += P(i) V(i)
        ok = ta_mbar_wait(p_full(t, b), (uint32_t)((i >> 1) & 1), abort_flag, TA_ERR_P_FULL);
        if (!ok) break;
        ok = ta_mbar_wait(v_full(s), (uint32_t)((i / TA_STAGES) & 1), abort_flag, TA_ERR_KV_FULL);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t va = sbase + TA_V_OFF + s * TA_KV_TILE;
#pragma unroll
        for (int k = 0; k < TA_KEYS / 16; ++k)            // 16 keys a step: 8 columns of P, 16 rows of V
          ta_umma_ts(o_col, s_col + (uint32_t)b * 64u + (uint32_t)k * 8u, ta_desc_mnmajor(va + (uint32_t)k * 16u * 128u, TA_KV_HALF),
                     idesc_pv, (i | k) != 0);
        ta_commit(pv_done(t, b));
        ta_commit(v_empty(s));
        // S(i+2) goes where P(i) lies: issued behind P V(i), which the tensor cores finish first
        if (i + 2 < nblocks) ok = issue_qk(i + 2);
      }
    }
  } else if (warp < 6 || (two && warp < 10)) {
    // ---- softmax: warps 2..5 tile A, warps 6..9 tile B; warp w reads lanes (w % 4) * 32 .. + 31 of tensor memory;
    // thread = query row -------------------------------------------------------------------------------------
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                       // row of the tile
    const uint32_t tlane = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr = tmem + tlane + (uint32_t)t * 128u, o_addr = tmem + tlane + 256u + (uint32_t)t * 128u;
    const int tok_in_item = t * per + r / G;
    const bool row_valid = r < per * G && tok_in_item < ntok;       // (128 - per * G rows of a tile stay unused when G does not divide 128)
    const int row_pos = row_valid ? pos0 + tok_in_item : -1;
    const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
    const int tile_pos0 = pos0 + t * per;                    // the smallest position among the tile's rows
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int i = 0; i < nblocks; ++i) {
      const int b = i & 1;
      const int kb = kbeg + i * TA_KEYS;
      ok = ta_mbar_wait(s_full(t, b), (uint32_t)((i >> 1) & 1), abort_flag, TA_ERR_S_FULL);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool need_mask = (kb + TA_KEYS - 1 > tile_pos0) || (p.window > 0) || (kb < lo_tile) || (kb + TA_KEYS > kend);
      float x[TA_KEYS];
      {
        uint32_t v[64];
        ta_tmem_ld64(s_addr + (uint32_t)b * 64u, v);
#pragma unroll
        for (int j = 0; j < 64; ++j) x[j] = __uint_as_float(v[j]);
      }
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < TA_KEYS; ++j) {
          const int key = kb + j;
          if (key > row_pos || key < row_lo) x[j] = -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains of three-input maxima
#pragma unroll
      for (int j = 0; j < TA_KEYS; j += 8) {
#pragma unroll
        for (int u = 0; u < 4; ++u) mx4[u] = ta_max3(mx4[u], x[j + 2 * u], x[j + 2 * u + 1]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The reference follows the maximum only when that has grown much; then O is rescaled, once P V of the block
      // before is complete.  The warp goes together: tcgen05.ld and st are warp-wide.
      const float m_loc = mx * p.scale_log2;
      const bool grow = m_loc > m_ref + TA_RESCALE_STEP;      // also true for the first finite maximum (m_ref = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        float f = 1.f;
        if (grow) {
          if (m_ref != -INFINITY) f = exp2f(m_ref - m_loc);
          m_ref = m_loc;
          l_run *= f;
        }
        if (i > 0) {
          ok = ta_mbar_wait(pv_done(t, b ^ 1), (uint32_t)(((i - 1) >> 1) & 1), abort_flag, TA_ERR_O_FULL);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
          for (int c = 0; c < TA_D; c += 32) {
            uint32_t v[32];
            ta_tmem_ld32(o_addr + (uint32_t)c, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * f);
            ta_tmem_st32(o_addr + (uint32_t)c, v);
          }
          ta_tmem_wait_st();
        }
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      // p = 2^(s * scale - m), the row's sum, P (two keys a column) over the first 32 columns of this S buffer.
      // Pairs of keys in packed instructions.  (Tried: a cubic for 2^f on the FMA pipe for half or a quarter of the
      // pairs, to take load off the special-function unit.  Slower: the softmax warps are short of issue slots, not
      // of that unit.)
      const uint64_t scale2 = ta_pack2(p.scale_log2, p.scale_log2), negm2 = ta_pack2(-m_use, -m_use);
      uint64_t sum2 = ta_pack2(0.f, 0.f);
      uint32_t w[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float y0, y1;
        ta_unpack2(ta_fma2(ta_pack2(x[2 * j], x[2 * j + 1]), scale2, negm2), y0, y1);
        const float p0 = exp2_approx(y0), p1 = exp2_approx(y1);          // 2^-inf = 0 for masked keys
        sum2 = ta_add2(sum2, ta_pack2(p0, p1));
        __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
        w[j] = *reinterpret_cast<uint32_t*>(&b2);
      }
      ta_tmem_st32(s_addr + (uint32_t)b * 64u, w);
      ta_tmem_wait_st();
      {
        float s0, s1;
        ta_unpack2(sum2, s0, s1);
        l_run += s0 + s1;
      }
      // hand P to the tensor cores
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) ta_mbar_arrive(p_full(t, b));
    }
    if (ok) ok = ta_mbar_wait(pv_done(t, (nblocks - 1) & 1), (uint32_t)(((nblocks - 1) >> 1) & 1), abort_flag, TA_ERR_O_FULL);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int token = t0 + tok_in_item, head = kvh * G + r % G;
      uint4* dst = reinterpret_cast<uint4*>(p.out + ((size_t)token * p.num_q_heads + head) * TA_D);
      const size_t prow = (((size_t)blockIdx.y * p.num_kv_heads + kvh) * nsplit + isplit) * TA_PART_ROWS + tok_in_item * G + r % G;
      if (nsplit > 1 && row_valid) {
        p.part_ml[prow * 2] = m_ref;
        p.part_ml[prow * 2 + 1] = l_run;
      }
#pragma unroll 1
      for (int c = 0; c < TA_D; c += 32) {
        uint32_t v[32];
        ta_tmem_ld32(o_addr + (uint32_t)c, v);              // warp-wide: rows without a token take part and write nothing
        if (nsplit > 1) {
          if (row_valid) {
            uint4* pdst = reinterpret_cast<uint4*>(p.part_o + prow * TA_D + c);
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) pdst[q4] = make_uint4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
          }
        } else if (row_valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[8 * q4 + 2 * j]) * inv, __uint_as_float(v[8 * q4 + 2 * j + 1]) * inv);
              w[j] = *reinterpret_cast<uint32_t*>(&b2);
            }
            dst[(c >> 3) + q4] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
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

// The rows of work items whose keys were cut into ranges: out = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z with
// M = max_z m_z.  One warp a row (a lane adds up four dimensions), the rows of an item spread over gridDim.z blocks.
// A range without keys for a row (m_z = -inf) is left out: its o_z may never have been written.
constexpr int TA_MAX_SPLITS = 8;
__global__ void __launch_bounds__(256) ta_combine_kernel(TcAttnParams p, int nsplit) {
  pdl_trigger();
  pdl_wait();
  const int4 tile = p.tiles[blockIdx.x];
  const int kvh = blockIdx.y, G = p.group;
  const int rows = tile.y * G;
  const int lane = threadIdx.x, warp = threadIdx.y;
  const size_t base = ((size_t)blockIdx.x * p.num_kv_heads + kvh) * nsplit;
  for (int r = blockIdx.z * blockDim.y + warp; r < rows; r += blockDim.y * gridDim.z) {
    float w[TA_MAX_SPLITS];
    float M = -INFINITY;
#pragma unroll
    for (int z = 0; z < TA_MAX_SPLITS; ++z) {
      w[z] = z < nsplit ? __ldcg(p.part_ml + ((base + z) * TA_PART_ROWS + r) * 2) : -INFINITY;
      M = fmaxf(M, w[z]);
    }
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int z = 0; z < TA_MAX_SPLITS; ++z) {
      if (z < nsplit && w[z] != -INFINITY) {
        const float wz = exp2f(w[z] - M);
        L += __ldcg(p.part_ml + ((base + z) * TA_PART_ROWS + r) * 2 + 1) * wz;
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p.part_o + ((base + z) * TA_PART_ROWS + r) * TA_D) + lane);
        acc.x += a.x * wz; acc.y += a.y * wz; acc.z += a.z * wz; acc.w += a.w * wz;
      }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int token = tile.x + r / G, head = kvh * G + r % G;
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(p.out + ((size_t)token * p.num_q_heads + head) * TA_D + lane * 4) =
        make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
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
  if (g > 128) return 0;                                     // the query box is G heads x floor(128/G) tokens
  if (page_size < 8 || page_size > 128 || 128 % page_size || (page_size & (page_size - 1))) return 0;
  return 1;
}

// Floats of workspace a launch with `key_splits` ranges needs (0 for one range).
LB_EXPORT long long lb_attention_tcgen05_workspace(int num_tiles, int num_kv_heads, int key_splits) {
  if (key_splits <= 1) return 0;
  return (long long)num_tiles * num_kv_heads * key_splits * lb::TA_PART_ROWS * (lb::TA_D + 2);
}

// q, out: [T, nq, 128] bfloat16.  k_cache, v_cache: [pages, nkv, page_size, 128].  tiles: {first token,
// tokens, request index, 0} with tokens <= 2 * floor(128 / (nq / nkv)); the tokens of a tile are consecutive tokens of one
// request at consecutive positions.  key_splits > 1 (at most 8): the keys of every tile are cut into that many ranges, a CTA
// each, whose results a second kernel combines through `workspace` (float32, lb_attention_tcgen05_workspace elements).
LB_EXPORT int lb_attention_tcgen05(const void* q, void* out, const void* k_cache, const void* v_cache, const int* positions,
                                   const int* block_table, const void* tiles, int num_tiles, int num_tokens,
                                   int num_q_heads, int num_kv_heads, int head_dim, int page_size, int num_pages,
                                   int max_pages, int window, float scale, int key_splits, float* workspace,
                                   long long workspace_elems, cudaStream_t stream) {
  LB_CHECK_ARG(lb_attention_tcgen05_ok(num_q_heads, num_kv_heads, head_dim, page_size),
               "attention_tcgen05: needs head_dim 128, at most 128 query heads per kv head and a page size among 8, 16, 32, 64, 128 "
               "(got head_dim %d, %d/%d heads, pages of %d)", head_dim, num_q_heads, num_kv_heads, page_size);
  LB_CHECK_ARG(max_pages > 0 && window >= 0 && num_tokens > 0 && num_pages > 0, "attention_tcgen05: bad sizes");
  LB_CHECK_ARG(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) && ((uintptr_t)out % 16 == 0),
               "attention_tcgen05: operands must be 16-byte aligned");
  if (num_tiles == 0) return 0;
  LB_CHECK_ARG(num_tiles <= 65535, "attention_tcgen05: %d tiles, at most 65535 a launch", num_tiles);
  LB_CHECK_ARG(max_pages <= lb::TA_MAX_TILE_PAGES, "attention_tcgen05: a request may span %d pages, at most %d", max_pages, lb::TA_MAX_TILE_PAGES);
  const int group = num_q_heads / num_kv_heads;
  CUtensorMap mq;
  if (!lb::ta_q_map(&mq, q, num_tokens, num_q_heads, group)) {
    lb::set_error("attention_tcgen05: cuTensorMapEncodeTiled failed");
    return 3;
  }
  LB_CHECK_ARG(key_splits >= 1 && key_splits <= lb::TA_MAX_SPLITS, "attention_tcgen05: %d key ranges, at most %d", key_splits, lb::TA_MAX_SPLITS);
  LB_CHECK_ARG(key_splits == 1 || (workspace && ((uintptr_t)workspace % 16 == 0) &&
                                   workspace_elems >= lb_attention_tcgen05_workspace(num_tiles, num_kv_heads, key_splits)),
               "attention_tcgen05: %d key ranges of %d tiles need a 16-byte aligned workspace of %lld floats (got %lld)", key_splits,
               num_tiles, lb_attention_tcgen05_workspace(num_tiles, num_kv_heads, key_splits), workspace_elems);
  lb::TcAttnParams p;
  p.part_o = workspace;
  p.part_ml = key_splits > 1 ? workspace + (size_t)num_tiles * num_kv_heads * key_splits * lb::TA_PART_ROWS * lb::TA_D : nullptr;
  p.out = (lb::bf16*)out; p.k_cache = (const uint8_t*)k_cache; p.v_cache = (const uint8_t*)v_cache; p.positions = positions; p.block_table = block_table; p.max_pages = max_pages;
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
  lb::launch(lb::attention_tcgen05_kernel, dim3(num_kv_heads, num_tiles, key_splits), dim3(lb::TA_THREADS), smem, stream, mq, p);
  LB_CHECK_LAUNCH("attention_tcgen05");
  if (key_splits > 1) {
    lb::launch(lb::ta_combine_kernel, dim3(num_tiles, num_kv_heads, lb::TA_PART_ROWS / 8), dim3(32, 8), 0, stream, p, key_splits);   // a row a warp: one round of loads
    LB_CHECK_LAUNCH("attention_tcgen05 combine");
  }
  return 0;
}

// Reads and clears the flag a bounded wait of this kernel sets when it gives up (0: none).
LB_EXPORT int lb_attention_tcgen05_device_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, lb::g_attention_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(lb::g_attention_tc_error, &zero, sizeof(int));
  return v;
}
