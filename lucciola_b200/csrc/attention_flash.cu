// Causal grouped-query attention over paged keys and values on the tensor cores (bfloat16),
// for portions of prompts and for decoded tokens alike.
//
// A work item ("tile") is a run of up to 64/G consecutive tokens of one request (G = query heads per
// kv head) and one kv head: its G*tokens query rows are stacked into a 64-row tile, so that the keys
// and values of a kv head are read once for all query heads that share them.  A decoded token is a
// tile with one token.  The keys a tile sees may be cut into `splits` ranges (grid z): each range
// produces an unnormalised partial (m, l, o) in 32-bit, and a second kernel combines the partials in
// the order of the ranges.  That is what keeps all SMs busy when few tokens attend to long contexts.
//
// Per CTA (4 warps, 16 query rows each): keys and values stream through a ring of shared-memory
// stages of 64 keys, fetched with 16-byte cp.async copies through the block table (any page size);
// scores S = Q K^T and the product P V run on mma.sync.m16n8k16 with ldmatrix-fed fragments; the
// softmax is the online form of src/kernels/flash_attention.cu:246-298 of lucciola (m, l, o per row,
// 32-bit), with P rounded to bfloat16 for the second product.  Keys outside a row's range (after its
// position, before its window, past the end) are masked, and their rows in shared memory are zeros,
// so whatever a reused page still holds cannot reach a sum (lucciola zero-fills the tail of the last
// page for the same reason, src/kernels/flash_attention.cu:142-154).
//
// Two arrangements of the four warps.  When tiles have more than 16 query rows (portions of prompts)
// each warp owns 16 rows and visits all 64 keys of a stage.  When no tile has more than 16 rows
// (decoded tokens) all warps share the rows and each visits 16 of the 64 keys, keeping its own
// (m, l, o); the four are merged through shared memory, in the order of the warps, at the end.
//
// Head sizes: any multiple of 8 up to 128 (padded with zeros to 64 or 128 in shared memory).
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace lb {

constexpr int FA_ROWS = 64;      // query rows of a tile
constexpr int FA_KEYS = 64;      // keys of a stage
constexpr int FA_STAGES = 3;
constexpr int FA_THREADS = 128;

struct FlashParams {
  const bf16* q; bf16* out;                 // [T, nq, d]
  const bf16* k_cache; const bf16* v_cache; // [pages, nkv, page_size, d]
  const int* positions;                     // [T]
  const int* block_table; int max_pages;    // [S, max_pages]
  const int4* tiles;                        // {first token, tokens, request index, unused}
  float* part_o;                            // [tiles, nkv, splits, part_rows, d]
  float* part_ml;                           // [tiles, nkv, splits, part_rows, 2]
  int part_rows;                            // most query rows of any tile
  int cluster;                              // > 0: the splits of a tile form a cluster of this size and combine through shared memory
  int num_q_heads, num_kv_heads, head_dim, group, page_size, page_shift, window, splits;   // page_shift: log2(page_size) or -1
  float scale_log2;                         // scale * log2(e)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;             // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void fa_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float fa_ld_cluster(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold DP bfloat16.
// Chunks are permuted by the row's low bits so that ldmatrix reads hit all banks.
template <int DP>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return (uint32_t)(row * (DP * 2) + ((chunk ^ (row & 7)) << 4));
}

// What the four warps that shared a tile's rows do when the keys are through: merge their (m, l, o) through shared
// memory in the order of the warps, then write the result, hand it to the combining kernel, or combine it with the
// other splits of the cluster.  scratch: keysplit_scratch_floats(DP) floats, fin: 16 * (DP + 2) floats, both free by now;
// with NAMED only the 128 computing threads of a larger CTA take part in the barriers.  Rows of the partial results are
// DP + 8 floats apart, so that the eight rows a warp stores at a time fall into different banks.
__host__ __device__ constexpr int keysplit_scratch_floats(int dp) { return 4 * 16 * (dp + 8) + 4 * 16 * 2; }
template <bool NAMED>
__device__ __forceinline__ void keysplit_sync() {
  if (NAMED) asm volatile("bar.sync 1, 128;" ::: "memory");
  else __syncthreads();
}
template <int DP, bool NAMED>
__device__ __forceinline__ void keysplit_finish(const FlashParams& p, float* scratch, float* fin, const float (&o)[DP / 8][4],
                                                const float (&m_run)[2], const float (&l_run)[2], int t0, int rows, int kvh, int split) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.group, d = p.head_dim;
  // Merge the four warps' (m, l, o) through shared memory (the stages are no longer needed).
  keysplit_sync<NAMED>();
  constexpr int MS = DP + 8;
  float* mo = scratch;                                                       // [4][16][MS]
  float* mml = mo + 4 * 16 * MS;                                             // [4][16][2]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + 8 * h;
    if (r >= rows) continue;                                                 // rows past the tile's last are never read
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      const int dim = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(mo + ((warp * 16 + r) * MS + dim)) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
    }
    if ((lane & 3) == 0) {
      mml[(warp * 16 + r) * 2 + 0] = m_run[h] == -INFINITY ? -INFINITY : m_run[h] * p.scale_log2;
      mml[(warp * 16 + r) * 2 + 1] = l_run[h];
    }
  }
  keysplit_sync<NAMED>();
  // With a cluster the merged (M, L, O) of this CTA stay in shared memory (in the value stages, free by
  // now) for the combination across the cluster; otherwise they go straight out.
  float* fin_o = fin;                                                        // [16][DP]
  float* fin_ml = fin_o + 16 * DP;                                                               // [16][2]
  for (int r = 0; r < rows; ++r) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
    float L = 0.f, wgt[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mml[(w * 16 + r) * 2];
      wgt[w] = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += mml[(w * 16 + r) * 2 + 1] * wgt[w];
    }
    const int token = t0 + r / G, head = kvh * G + r % G;
    if (p.cluster > 0 && tid == 0) { fin_ml[r * 2] = M; fin_ml[r * 2 + 1] = L; }
    for (int dim = tid; dim < d; dim += FA_THREADS) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) acc += mo[(w * 16 + r) * MS + dim] * wgt[w];
      if (p.cluster > 0) {
        fin_o[r * DP + dim] = acc;
      } else if (p.splits == 1) {
        p.out[((size_t)token * p.num_q_heads + head) * d + dim] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      } else {
        const size_t slot = (((size_t)blockIdx.x * p.num_kv_heads + kvh) * p.splits + split) * p.part_rows + r;
        p.part_o[slot * d + dim] = acc;
        if (dim == 0) { p.part_ml[slot * 2] = M; p.part_ml[slot * 2 + 1] = L; }
      }
    }
  }
  if (p.cluster > 0) {
    // Every CTA of the cluster combines its share of the head's dimensions over all splits, in their
    // order, reading the peers' shared memory.
    fa_cluster_sync();
    const int per = (d + p.cluster - 1) / p.cluster;
    for (int item = tid; item < rows * per; item += FA_THREADS) {
      const int r = item / per, dim = split * per + item % per;
      if (dim >= d) continue;
      // All loads from the peers' shared memory first (each takes several hundred cycles), then the arithmetic.
      float mz[16], lz[16], oz[16];
#pragma unroll
      for (int z = 0; z < 16; ++z) {
        const bool in = z < p.splits;
        mz[z] = in ? fa_ld_cluster(fin_ml + r * 2, z) : -INFINITY;
        lz[z] = in ? fa_ld_cluster(fin_ml + r * 2 + 1, z) : 0.f;
        oz[z] = in ? fa_ld_cluster(fin_o + r * DP + dim, z) : 0.f;
      }
      float M = -INFINITY;
#pragma unroll
      for (int z = 0; z < 16; ++z) M = fmaxf(M, mz[z]);
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int z = 0; z < 16; ++z) {
        if (mz[z] == -INFINITY) continue;
        const float wz = exp2f(mz[z] - M);
        L += lz[z] * wz;
        acc += oz[z] * wz;
      }
      const int token = t0 + r / G, head = kvh * G + r % G;
      p.out[((size_t)token * p.num_q_heads + head) * d + dim] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
    fa_cluster_sync();                        // nobody leaves while a peer still reads its memory
  }
}

template <int DP, bool KEYSPLIT>
__global__ void __launch_bounds__(FA_THREADS, KEYSPLIT ? 2 : 3)
flash_attention_kernel(FlashParams p) {
  constexpr int CHUNKS = DP / 8;                  // 16-byte chunks of a row
  constexpr int NB = KEYSPLIT ? 2 : FA_KEYS / 8;  // blocks of 8 keys a warp visits in a stage
  constexpr int LOADS = FA_KEYS * CHUNKS / FA_THREADS;      // 16-byte copies a thread makes per stage and matrix
  constexpr int ROW_STEP = FA_THREADS / CHUNKS;             // rows between two copies of one thread
  constexpr int TILE_BYTES = FA_KEYS * DP * 2;
  // Decoded tokens: three stages, bound by memory.  Portions of prompts: two stages, and the query tile
  // lies on the second stage's keys (it is in registers before that stage is first filled), so that a CTA
  // needs 64 KB and three of them share an SM.
  constexpr int STAGES = KEYSPLIT ? FA_STAGES : 2;
  constexpr int Q_BYTES = KEYSPLIT ? FA_ROWS * DP * 2 : 0;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t k_smem = (uint32_t)__cvta_generic_to_shared(smem) + Q_BYTES;
  const uint32_t v_smem = k_smem + STAGES * TILE_BYTES;
  const uint32_t q_smem = KEYSPLIT ? k_smem - Q_BYTES : k_smem + TILE_BYTES;

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int4 tile = p.tiles[blockIdx.x];
  const int t0 = tile.x, ntok = tile.y, seq = tile.z;
  const int kvh = blockIdx.y, split = blockIdx.z;
  const int G = p.group, d = p.head_dim;
  const int rows = ntok * G;
  const int pos0 = p.positions[t0];
  const int pos_last = pos0 + ntok - 1;
  const int* bt = p.block_table + (size_t)seq * p.max_pages;

  // Keys this tile can see, and the part of them this split handles (multiples of a stage).
  const int lo_tile = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int span = pos_last - lo_tile + 1;
  const int per_split = ((span + p.splits - 1) / p.splits + FA_KEYS - 1) / FA_KEYS * FA_KEYS;
  const int kbeg = lo_tile + split * per_split;
  const int kend = min(pos_last + 1, kbeg + per_split);      // exclusive
  const int num_stages = kend > kbeg ? (kend - kbeg + FA_KEYS - 1) / FA_KEYS : 0;
  // Tiles, positions and block tables were written before the step began: they are read, and the lines of the block
  // table this CTA will need are fetched, while the kernel ahead may still run.  Queries, and the keys and values that
  // kernel wrote, only after the wait.
  if (num_stages > 0) {
    const int first = p.page_shift >= 0 ? (kbeg >> p.page_shift) : (kbeg / p.page_size);
    const int last = p.page_shift >= 0 ? ((kend - 1) >> p.page_shift) : ((kend - 1) / p.page_size);
    for (int i = first + tid * 32; i <= last; i += FA_THREADS * 32) asm volatile("prefetch.global.L1 [%0];" ::"l"(bt + i));
  }
  pdl_wait();

  // ---- Q: global -> shared (zero padded), then into A fragments ------------------------------
  for (int idx = tid; idx < FA_ROWS * CHUNKS; idx += FA_THREADS) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool valid = r < rows && c * 8 < d;
    const bf16* src = p.q;
    if (valid) src = p.q + ((size_t)(t0 + r / G) * p.num_q_heads + kvh * G + r % G) * d + c * 8;
    cp_async16(q_smem + tile_offset<DP>(r, c), src, valid);
  }
  cp_async_commit();

  // A thread copies the same 16-byte column of rows ld_row, ld_row + ROW_STEP, ...: the swizzled
  // column is the same for all of them because ROW_STEP is a multiple of 8.
  const int ld_row = tid / CHUNKS, ld_chunk = tid % CHUNKS;
  const bool ld_col_valid = ld_chunk * 8 < d;
  const uint32_t ld_smem = tile_offset<DP>(ld_row, ld_chunk);
  const size_t head_off = (size_t)kvh * p.page_size * d + ld_chunk * 8;
  const size_t page_stride = (size_t)p.num_kv_heads * p.page_size * d;
  auto load_stage = [&](int stage_idx) {
    const int buf = stage_idx % STAGES;
    const int kbase = kbeg + stage_idx * FA_KEYS + ld_row;
    int page[LOADS], slot[LOADS];
#pragma unroll
    for (int i = 0; i < LOADS; ++i) {           // all page lookups first: they are independent loads
      const int j = kbase + i * ROW_STEP;
      const int pi = p.page_shift >= 0 ? (j >> p.page_shift) : (j / p.page_size);
      slot[i] = j - pi * p.page_size;
      page[i] = (j < kend && ld_col_valid) ? bt[pi] : -1;
    }
#pragma unroll
    for (int i = 0; i < LOADS; ++i) {
      const bool valid = page[i] >= 0;
      const size_t off = valid ? (size_t)page[i] * page_stride + head_off + (size_t)slot[i] * d : 0;
      const uint32_t so = buf * TILE_BYTES + ld_smem + i * ROW_STEP * (DP * 2);
      cp_async16(k_smem + so, p.k_cache + off, valid);
      cp_async16(v_smem + so, p.v_cache + off, valid);
    }
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_stages) load_stage(s);
    cp_async_commit();
  }

  // Rows of this thread: r0 = (first row of the warp) + lane/4 and r0 + 8.
  const int warp_row0 = KEYSPLIT ? 0 : warp * 16;
  const int r0 = warp_row0 + (lane >> 2);
  int row_pos[2], row_lo[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = r0 + 8 * h;
    row_pos[h] = r < rows ? pos0 + r / G : -1;                  // -1: no key passes the mask
    row_lo[h] = p.window > 0 ? max(0, row_pos[h] - p.window + 1) : 0;
  }
  const bool warp_active = warp_row0 < rows;

  cp_async_wait<STAGES - 1>();        // Q has landed (the stage loads may still be in flight)
  __syncthreads();
  uint32_t qf[DP / 16][4];
  if (warp_active) {
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
      const int r = warp_row0 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int c = kk * 2 + (lane >> 4);
      ldmatrix_x4(q_smem + tile_offset<DP>(r, c), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
  }

  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int st = 0; st < num_stages; ++st) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();                   // stage st is visible; the buffer of stage st-1 is free
    if (st + STAGES - 1 < num_stages) load_stage(st + STAGES - 1);
    cp_async_commit();
    if (!warp_active) continue;

    const int buf = st % STAGES;
    const uint32_t kb = k_smem + buf * TILE_BYTES, vb = v_smem + buf * TILE_BYTES;
    const int kbase = kbeg + st * FA_KEYS;

    // ---- S = Q K^T: 16 rows x (64 or, with shared rows, this warp's 16) keys -----------------------
    const int key0 = KEYSPLIT ? warp * 16 : 0;       // first key of the stage this warp visits
    float s[NB][4];
#pragma unroll
    for (int i = 0; i < NB; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
#pragma unroll
      for (int nb = 0; nb < NB; nb += 2) {
        // matrices: (keys nb, dims lo), (keys nb, dims hi), (keys nb+1, dims lo), (keys nb+1, dims hi)
        const int key = key0 + nb * 8 + (lane & 7) + (lane >> 4) * 8;
        const int c = kk * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kb + tile_offset<DP>(key, c), b0, b1, b2, b3);
        mma_bf16(s[nb], qf[kk], b0, b1);
        mma_bf16(s[nb + 1], qf[kk], b2, b3);
      }
    }

    // ---- mask, online softmax ----------------------------------------------------------------
    // Rows past the tile's last (zero queries, positions -1) need no mask of their own: what they gather is never
    // written, and it is finite, because keys and values of slots that hold nothing lie at or past kend.
    const bool need_mask = (kbase + FA_KEYS - 1 > pos0) || (p.window > 0) || (kbase + FA_KEYS > kend);
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        if (need_mask) {
          const int j = kbase + key0 + nb * 8 + (lane & 3) * 2 + (e & 1);
          if (j > row_pos[h] || j < row_lo[h] || j >= kend) s[nb][e] = -INFINITY;
        }
        m_new[h] = fmaxf(m_new[h], s[nb][e]);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
      m_use[h] = m_new[h] == -INFINITY ? 0.f : m_new[h] * p.scale_log2;
      alpha[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] * p.scale_log2 - m_use[h]);
      m_run[h] = m_new[h];
    }
    float row_sum[2] = {0.f, 0.f};
    uint32_t pf[NB / 2][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        pv[e] = exp2_approx(fmaf(s[nb][e], p.scale_log2, -m_use[h]));   // 2^-inf = 0 for masked keys
        row_sum[h] += pv[e];
      }
      // C fragments of two key blocks become one A fragment of 16 keys
      pf[nb >> 1][(nb & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
      pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + row_sum[h];
    // Once the maxima have settled the factors are exactly 1 for stage after stage: skip the multiplications then.
    if (!__all_sync(0xffffffffu, alpha[0] == 1.f && alpha[1] == 1.f)) {
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
    }

    // ---- O += P V ----------------------------------------------------------------------------------
#pragma unroll
    for (int ks = 0; ks < NB / 2; ++ks) {
#pragma unroll
      for (int db = 0; db < DP / 8; db += 2) {
        // matrices (transposed on load): (keys lo, dims db), (keys hi, dims db), (keys lo, dims db+1), (keys hi, dims db+1)
        const int key = key0 + ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = db + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vb + tile_offset<DP>(key, c), b0, b1, b2, b3);
        mma_bf16(o[db], pf[ks], b0, b1);
        mma_bf16(o[db + 1], pf[ks], b2, b3);
      }
    }
  }
  cp_async_wait<0>();

  // ---- write: the row sums live in four lanes each ------------------------------------------------
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  if (KEYSPLIT) {
    keysplit_finish<DP, false>(p, reinterpret_cast<float*>(smem + FA_ROWS * DP * 2),
                               reinterpret_cast<float*>(smem + FA_ROWS * DP * 2 + STAGES * TILE_BYTES), o, m_run, l_run, t0, rows, kvh, split);
    return;
  }
  if (!warp_active) return;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = r0 + 8 * h;
    if (r >= rows) continue;
    const int token = t0 + r / G, head = kvh * G + r % G;
    if (p.splits == 1) {
      const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
      bf16* dst = p.out + ((size_t)token * p.num_q_heads + head) * d;
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        const int dim = i * 8 + (lane & 3) * 2;
        if (dim < d) *reinterpret_cast<__nv_bfloat162*>(dst + dim) = __floats2bfloat162_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      }
    } else {
      const size_t slot = (((size_t)blockIdx.x * p.num_kv_heads + kvh) * p.splits + split) * p.part_rows + r;
      float* dst = p.part_o + slot * d;
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        const int dim = i * 8 + (lane & 3) * 2;
        if (dim < d) *reinterpret_cast<float2*>(dst + dim) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
      }
      if ((lane & 3) == 0) {
        p.part_ml[slot * 2 + 0] = m_run[h] == -INFINITY ? -INFINITY : m_run[h] * p.scale_log2;
        p.part_ml[slot * 2 + 1] = l_run[h];
      }
    }
  }
}

// ---- decoded tokens, keys and values fetched by TMA -----------------------------------------------------------------------
// The kernel above spends most of its instructions on fetching: every thread computes the addresses of sixteen 16-byte
// copies a stage and looks their pages up, and with two CTAs of four warps on an SM nothing hides the latency of that
// chain, so the warps, not the memory, set the pace.  Here a fifth warp fetches: each of its lanes looks one page up and
// issues one TMA copy (a box of 64 dimensions x the page's keys, up to 64, in the 128-byte swizzle, 32 KB a stage in at most
// 32 copies), and the four computing warps only wait on the stage's barrier, multiply and give the stage back.
// Needs a page size among 8, 16, 32, 64, 128 and tiles of at most 16 query rows.  Keys before the window's start down to
// a multiple of 64 are fetched as well and masked; a page that the table no longer holds (behind the window, or past the
// end) is replaced by page 0, whose keys are masked all the same.
constexpr int FD_THREADS = 160;
constexpr int FD_STAGES = 3;
constexpr unsigned long long FD_WAIT_CYCLES = 4000000000ull;
enum { FD_ERR_FULL = 401, FD_ERR_EMPTY = 402 };
__device__ int g_flash_decode_error = 0;

__device__ __forceinline__ void fd_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fd_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fd_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool fd_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded: gives up after about two seconds, leaves a code for the host and tells the rest of the CTA.
template <bool SLEEP>
__device__ __forceinline__ bool fd_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (fd_mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned it = 1;; ++it) {
    if (SLEEP) __nanosleep(64);
    if (fd_mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag) return false;
      if ((unsigned long long)(clock64() - t0) > FD_WAIT_CYCLES) {
        *abort_flag = code;
        atomicCAS(&g_flash_decode_error, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void fd_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Byte offset of 16-byte chunk `chunk` (of DP / 8) of key `key` in a stage's keys or values: halves of 64 dimensions,
// each [64 keys][128 bytes] in the 128-byte swizzle that the copies write.
__device__ __forceinline__ uint32_t fd_offset(int key, int chunk) {
  return (uint32_t)((chunk >> 3) * 8192 + key * 128 + (((chunk & 7) ^ (key & 7)) << 4));
}

template <int DP>
__global__ void __launch_bounds__(FD_THREADS, 2)
flash_decode_tma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, FlashParams p) {
  constexpr int CHUNKS = DP / 8;
  constexpr int NH = DP / 64;                       // halves of 64 dimensions
  constexpr int MAT_BYTES = NH * 8192;              // a stage's keys (or values)
  constexpr int STAGE_BYTES = 2 * MAT_BYTES;
  extern __shared__ uint8_t fd_smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * FD_STAGES];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const uint32_t base = ((uint32_t)__cvta_generic_to_shared(fd_smem_raw) + 1023u) & ~1023u;     // the swizzle wants 1024
  uint8_t* base_ptr = fd_smem_raw + (base - (uint32_t)__cvta_generic_to_shared(fd_smem_raw));
  const uint32_t q_smem = base + FD_STAGES * STAGE_BYTES;                                         // [16][DP] bfloat16
  auto full = [&](int s) { return (uint32_t)__cvta_generic_to_shared(&bars[s]); };
  auto empty = [&](int s) { return (uint32_t)__cvta_generic_to_shared(&bars[FD_STAGES + s]); };

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int4 tile = p.tiles[blockIdx.x];
  const int t0 = tile.x, ntok = tile.y, seq = tile.z;
  const int kvh = blockIdx.y, split = blockIdx.z;
  const int G = p.group, d = p.head_dim;
  const int rows = ntok * G;
  const int pos0 = p.positions[t0];
  const int pos_last = pos0 + ntok - 1;
  const int* bt = p.block_table + (size_t)seq * p.max_pages;

  // Keys this tile can see, from a multiple of a stage, and the part of them this split handles.
  const int lo_tile = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int lo_al = lo_tile & ~(FA_KEYS - 1);
  const int span = pos_last - lo_al + 1;
  const int per_split = ((span + p.splits - 1) / p.splits + FA_KEYS - 1) / FA_KEYS * FA_KEYS;
  const int kbeg = lo_al + split * per_split;
  const int kend = min(pos_last + 1, kbeg + per_split);      // exclusive
  const int num_stages = kend > kbeg ? (kend - kbeg + FA_KEYS - 1) / FA_KEYS : 0;

  if (tid == 0) {
    for (int s = 0; s < FD_STAGES; ++s) { fd_mbar_init(full(s), 1); fd_mbar_init(empty(s), 4); }
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 4) {
    // ---- the fetching warp: lane = (box of keys, half of the dimensions, keys or values) ----------------------------------
    const int box_keys = min(p.page_size, FA_KEYS);
    const int nops = 2 * NH * (FA_KEYS / box_keys);
    const int kv = lane & 1, half = (lane >> 1) % NH, box = (lane >> 1) / NH;
    const bool active = lane < nops;
    const CUtensorMap* map = kv ? &vmap : &kmap;
    const uint32_t dst_off = (uint32_t)(kv * MAT_BYTES + half * 8192 + box * box_keys * 128);
    auto row_of = [&](int st) -> int {            // first row of this lane's box in the pool's [pages * kv heads * page size, d]
      const int key0 = kbeg + st * FA_KEYS + box * box_keys;
      int page = -1;
      if (active && st < num_stages && key0 < kend) page = bt[key0 >> p.page_shift];
      if (page < 0) return kvh * p.page_size;                                        // page 0: masked whatever it holds
      return (page * p.num_kv_heads + kvh) * p.page_size + (key0 & (p.page_size - 1));
    };
    int row = row_of(0);                            // the tables were written before the step began
    auto fetch = [&](int st) {
      const int b = st % FD_STAGES;
      if (lane == 0) fd_mbar_expect_tx(full(b), STAGE_BYTES);
      __syncwarp();
      if (active) fd_tma_2d(base + b * STAGE_BYTES + dst_off, map, half * 64, row, full(b));
      row = row_of(st + 1);                         // looked up while the stage is awaited
    };
    // Keys before this step's first token were written by earlier steps: the first stages of them are requested while
    // the kernel ahead (which writes this step's keys and values) may still run.
    int st = 0;
    for (; st < min(num_stages, FD_STAGES) && kbeg + (st + 1) * FA_KEYS <= pos0; ++st) fetch(st);
    pdl_wait();
    for (; st < num_stages; ++st) {
      if (!fd_mbar_wait<true>(empty(st % FD_STAGES), (uint32_t)((st / FD_STAGES) & 1) ^ 1u, abort_flag, FD_ERR_EMPTY)) break;
      fetch(st);
    }
    if (p.cluster > 0) { fa_cluster_sync(); fa_cluster_sync(); }      // the cluster's barriers count every thread
    return;
  }

  // ---- the computing warps ----------------------------------------------------------------------------------------------------
  pdl_wait();
  for (int idx = tid; idx < 16 * CHUNKS; idx += 128) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool valid = r < rows && c * 8 < d;
    const bf16* src = p.q;
    if (valid) src = p.q + ((size_t)(t0 + r / G) * p.num_q_heads + kvh * G + r % G) * d + c * 8;
    cp_async16(q_smem + tile_offset<DP>(r, c), src, valid);
  }
  cp_async_commit();

  const int r0 = lane >> 2;
  int row_pos[2], row_lo[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = r0 + 8 * h;
    row_pos[h] = r < rows ? pos0 + r / G : -1;                  // -1: no key passes the mask
    row_lo[h] = p.window > 0 ? max(0, row_pos[h] - p.window + 1) : 0;
  }
  cp_async_wait<0>();
  keysplit_sync<true>();
  uint32_t qf[DP / 16][4];
#pragma unroll
  for (int kk = 0; kk < DP / 16; ++kk) {
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = kk * 2 + (lane >> 4);
    ldmatrix_x4(q_smem + tile_offset<DP>(r, c), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }

  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int key0 = warp * 16;                        // the 16 keys of a stage this warp visits

  for (int st = 0; st < num_stages; ++st) {
    const int b = st % FD_STAGES;
    if (!fd_mbar_wait<false>(full(b), (uint32_t)((st / FD_STAGES) & 1), abort_flag, FD_ERR_FULL)) break;
    const uint32_t kb = base + b * STAGE_BYTES, vb = kb + MAT_BYTES;
    const int kbase = kbeg + st * FA_KEYS;

    // ---- S = Q K^T: 16 rows x this warp's 16 keys -----------------------------------------------------------------------
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
      // matrices: (keys lo, dims lo), (keys lo, dims hi), (keys hi, dims lo), (keys hi, dims hi)
      const int key = key0 + (lane & 7) + (lane >> 4) * 8;
      const int c = kk * 2 + ((lane >> 3) & 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(kb + fd_offset(key, c), b0, b1, b2, b3);
      mma_bf16(s[0], qf[kk], b0, b1);
      mma_bf16(s[1], qf[kk], b2, b3);
    }
    // The values of keys past the end, or before the first key any row of the tile sees, are whatever a page still
    // holds: zeros instead, so that nothing a reused page holds can reach a sum (their weights are zeros, but zero
    // times a NaN is not).
    if (kbase + FA_KEYS > kend || kbase < lo_tile) {
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      for (int idx = lane; idx < 16 * CHUNKS; idx += 32) {
        const int key = key0 + idx / CHUNKS, c = idx % CHUNKS;
        if (kbase + key >= kend || kbase + key < lo_tile)
          *reinterpret_cast<uint4*>(base_ptr + b * STAGE_BYTES + MAT_BYTES + fd_offset(key, c)) = zero;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // a later copy into this stage comes after these stores
      __syncwarp();
    }

    // ---- mask, online softmax ---------------------------------------------------------------------------------------------
    const bool need_mask = (kbase + FA_KEYS - 1 > pos0) || (p.window > 0) || (kbase + FA_KEYS > kend);
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        if (need_mask) {
          const int j = kbase + key0 + nb * 8 + (lane & 3) * 2 + (e & 1);
          if (j > row_pos[h] || j < row_lo[h] || j >= kend) s[nb][e] = -INFINITY;
        }
        m_new[h] = fmaxf(m_new[h], s[nb][e]);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
      m_use[h] = m_new[h] == -INFINITY ? 0.f : m_new[h] * p.scale_log2;
      alpha[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] * p.scale_log2 - m_use[h]);
      m_run[h] = m_new[h];
    }
    float row_sum[2] = {0.f, 0.f};
    uint32_t pf[4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        pv[e] = exp2_approx(fmaf(s[nb][e], p.scale_log2, -m_use[h]));   // 2^-inf = 0 for masked keys
        row_sum[h] += pv[e];
      }
      pf[nb * 2 + 0] = pack_bf16(pv[0], pv[1]);       // C fragments of two key blocks become one A fragment of 16 keys
      pf[nb * 2 + 1] = pack_bf16(pv[2], pv[3]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + row_sum[h];
    if (!__all_sync(0xffffffffu, alpha[0] == 1.f && alpha[1] == 1.f)) {
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
    }

    // ---- O += P V ------------------------------------------------------------------------------------------------------------
#pragma unroll
    for (int db = 0; db < DP / 8; db += 2) {
      // matrices (transposed on load): (keys lo, dims db), (keys hi, dims db), (keys lo, dims db+1), (keys hi, dims db+1)
      const int key = key0 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int c = db + (lane >> 4);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(vb + fd_offset(key, c), b0, b1, b2, b3);
      mma_bf16(o[db], pf, b0, b1);
      mma_bf16(o[db + 1], pf, b2, b3);
    }
    __syncwarp();
    if (lane == 0) fd_mbar_arrive(empty(b));          // this warp has read the stage
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  // the stages are free now (every copy that was issued has been waited for): the merge uses them
  float* scratch = reinterpret_cast<float*>(base_ptr);
  keysplit_finish<DP, true>(p, scratch, scratch + keysplit_scratch_floats(DP), o, m_run, l_run, t0, rows, kvh, split);
}

// Combines the partials of the splits, in their order: out = sum_z o_z 2^(m_z - M) / sum_z l_z 2^(m_z - M).
// One warp per query row: the lanes first share the work of the weights 2^(m_z - M) (kept in shared
// memory), then each lane adds up four dimensions over the splits, eight independent 16-byte loads at a time.
// The rows of a tile are spread over gridDim.z blocks of four warps: a launch with few tiles (one portion of a few
// tokens beside decoded tokens) would otherwise walk its rows one after the other in a handful of warps, each row
// a chain of dependent loads (32 rows x 31 splits: 122 us in 8 blocks, as long as the attention of the whole step).
__global__ void flash_combine_kernel(FlashParams p) {
  extern __shared__ float wsm[];                      // [warps][splits]
  pdl_trigger();
  pdl_wait();
  const int4 tile = p.tiles[blockIdx.x];
  const int kvh = blockIdx.y;
  const int rows = tile.y * p.group, d = p.head_dim;
  const int lane = threadIdx.x, warp = threadIdx.y, nwarps = blockDim.y;
  float* wz = wsm + warp * p.splits;
  const size_t base = ((size_t)blockIdx.x * p.num_kv_heads + kvh) * p.splits;
  for (int r = blockIdx.z * nwarps + warp; r < rows; r += nwarps * gridDim.z) {
    float M = -INFINITY;
    for (int z = lane; z < p.splits; z += 32) M = fmaxf(M, p.part_ml[((base + z) * p.part_rows + r) * 2]);
    M = warp_max(M);
    float L = 0.f;
    for (int z = lane; z < p.splits; z += 32) {
      const float mz = p.part_ml[((base + z) * p.part_rows + r) * 2];
      const float w = mz == -INFINITY ? 0.f : exp2f(mz - M);
      wz[z] = w;
      L += p.part_ml[((base + z) * p.part_rows + r) * 2 + 1] * w;
    }
    // Sum over the lanes in a fixed pattern; then every lane holds the same L.
    L = warp_sum(L);
    __syncwarp();
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int token = tile.x + r / p.group, head = kvh * p.group + r % p.group;
    bf16* dst = p.out + ((size_t)token * p.num_q_heads + head) * d;
    const size_t zstride = (size_t)p.part_rows * d;
    // a lane adds up four neighbouring dimensions (one 16-byte load a split), eight splits in flight at a time
    for (int dim = lane * 4; dim < d; dim += 128) {
      const float* src = p.part_o + ((base * p.part_rows) + r) * d + dim;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int z0 = 0; z0 < p.splits; z0 += 8) {
        float4 a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          a[u] = z0 + u < p.splits ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(z0 + u) * zstride)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float w = z0 + u < p.splits ? wz[z0 + u] : 0.f;
          acc[0] += a[u].x * w; acc[1] += a[u].y * w; acc[2] += a[u].z * w; acc[3] += a[u].w * w;
        }
      }
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv), hi = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
      *reinterpret_cast<uint2*>(dst + dim) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
    __syncwarp();
  }
}

static int log2_exact(int v) {          // log2 of a power of two, else -1
  for (int b = 0; b < 31; ++b) if ((1 << b) == v) return b;
  return -1;
}

// ---- host side of the TMA kernel: tensor maps of the pools, made once per pool ----------------------------------------------------
typedef CUresult (*FdEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static FdEncodeFn fd_encode_fn() {
  static FdEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (FdEncodeFn)sym;
  });
  return fn;
}
struct FdMapKey {
  const void* base; long long rows; int d, box;
  bool operator==(const FdMapKey& o) const { return base == o.base && rows == o.rows && d == o.d && box == o.box; }
};
struct FdMapKeyHash {
  size_t operator()(const FdMapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.d; h = h * 1000003u ^ (size_t)k.box;
    return h;
  }
};
static std::unordered_map<FdMapKey, CUtensorMap, FdMapKeyHash> g_fd_maps;
static std::mutex g_fd_mu;

// A pool [pages, kv heads, page size, d] as rows of d: boxes of 64 dimensions x `box` rows, 128-byte swizzle; what lies past
// d reads as zeros.
static bool fd_pool_map(CUtensorMap* out, const void* pool, long long rows, int d, int box) {
  FdMapKey key{pool, rows, d, box};
  std::lock_guard<std::mutex> g(g_fd_mu);
  auto it = g_fd_maps.find(key);
  if (it != g_fd_maps.end()) { *out = it->second; return true; }
  FdEncodeFn fn = fd_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  cuuint32_t bx[2] = {64, (cuuint32_t)box};
  cuuint32_t estr[2] = {1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (g_fd_maps.size() > 4096) g_fd_maps.clear();
  g_fd_maps.emplace(key, *out);
  return true;
}

}  // namespace lb

// Reads and clears the flag a bounded wait of the TMA kernel sets when it gives up (0: none).
LB_EXPORT int lb_attention_flash_device_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, lb::g_flash_decode_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(lb::g_flash_decode_error, &zero, sizeof(int));
  return v;
}

// How many clusters of 16 CTAs of the TMA kernel the GPU keeps resident at a time (0: it does not schedule them).
// Callers use clusters of 16 only for launches of at most this many clusters.
LB_EXPORT int lb_attention_flash_wide_clusters(int head_dim) {
  static int cached[2] = {-1, -1};
  const int dp = head_dim <= 64 ? 64 : 128;
  int& c = cached[dp == 64];
  if (c >= 0) return c;
  void (*kern)(CUtensorMap, CUtensorMap, lb::FlashParams) = dp == 64 ? lb::flash_decode_tma_kernel<64> : lb::flash_decode_tma_kernel<128>;
  const int fd_smem = 1024 + lb::FD_STAGES * 2 * (dp / 64) * 8192 + 16 * dp * 2;
  c = 0;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess ||
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fd_smem) != cudaSuccess) {
    cudaGetLastError();
    return c;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, 1, 16); cfg.blockDim = dim3(lb::FD_THREADS); cfg.dynamicSmemBytes = fd_smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 16;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) c = n;
  else cudaGetLastError();
  return c;
}

// Floats of workspace a launch with these sizes needs (partials of o, then of m and l).
LB_EXPORT long long lb_attention_flash_workspace(int num_tiles, int num_kv_heads, int splits, int part_rows, int head_dim) {
  if (splits <= 1) return 0;
  return (long long)num_tiles * num_kv_heads * splits * part_rows * (head_dim + 2);
}

// q, out: [T, nq, d] bfloat16.  tiles: [num_tiles] of {first token, tokens, request index, 0} with
// tokens * (nq / nkv) <= part_rows <= 64.  workspace: float32, needed when splits > 1.
LB_EXPORT int lb_attention_flash(const void* q, void* out, const void* k_cache, const void* v_cache,
                                 const int* positions, const int* block_table, const void* tiles, int num_tiles,
                                 int num_q_heads, int num_kv_heads, int head_dim, int page_size, int max_pages,
                                 int num_pages, int window, float scale, int splits, int part_rows, float* workspace,
                                 long long workspace_elems, cudaStream_t stream) {
  LB_CHECK_ARG(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0,
               "attention_flash: %d query heads are not a multiple of %d kv heads", num_q_heads, num_kv_heads);
  const int group = num_q_heads / num_kv_heads;
  LB_CHECK_ARG(group <= lb::FA_ROWS, "attention_flash: %d query heads per kv head, at most %d", group, lb::FA_ROWS);
  LB_CHECK_ARG(head_dim >= 8 && head_dim <= 128 && head_dim % 8 == 0,
               "attention_flash: head_dim %d must be a multiple of 8 between 8 and 128", head_dim);
  const bool force_workspace = splits < 0;     // a negative count asks for the path through the workspace
  if (splits < 0) splits = -splits;
  LB_CHECK_ARG(page_size > 0 && max_pages > 0 && window >= 0 && splits >= 1 && splits <= 65535, "attention_flash: bad sizes");
  LB_CHECK_ARG(num_kv_heads <= 65535, "attention_flash: too many kv heads");
  LB_CHECK_ARG(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) &&
               ((uintptr_t)out % 4 == 0), "attention_flash: operands must be 16-byte aligned");
  if (num_tiles == 0) return 0;
  LB_CHECK_ARG(part_rows >= group && part_rows <= lb::FA_ROWS, "attention_flash: rows of a tile must be in %d..%d, got %d", group, lb::FA_ROWS, part_rows);
  const int page_shift = lb::log2_exact(page_size);
  // Decoded tokens over pages of 8 to 128 keys: the kernel whose fifth warp fetches by TMA.  num_pages <= 0 keeps it off.
  const bool by_tma = part_rows <= 16 && num_pages > 0 && page_shift >= 3 && page_size <= 128 &&
                      (long long)num_pages * num_kv_heads * page_size < (1ll << 31);
  // Up to 8 splits (a power of two) of tiles of at most 16 rows combine inside a thread-block cluster; the TMA kernel
  // also takes clusters of 16 (a size the launch has to ask for: not every GPU schedules it).
  const bool may_cluster = part_rows <= 16 && splits <= (by_tma ? 16 : 8) && !force_workspace;
  LB_CHECK_ARG(splits == 1 || may_cluster || (workspace && workspace_elems >= lb_attention_flash_workspace(num_tiles, num_kv_heads, splits, part_rows, head_dim)),
               "attention_flash: the workspace is too small for %d splits", splits);
  lb::FlashParams p;
  p.q = (const lb::bf16*)q; p.out = (lb::bf16*)out; p.k_cache = (const lb::bf16*)k_cache; p.v_cache = (const lb::bf16*)v_cache;
  p.positions = positions; p.block_table = block_table; p.max_pages = max_pages; p.tiles = (const int4*)tiles;
  p.part_o = workspace;
  p.part_ml = workspace ? workspace + (long long)num_tiles * num_kv_heads * splits * part_rows * head_dim : nullptr;
  p.part_rows = part_rows;
  p.num_q_heads = num_q_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim; p.group = group;
  p.page_size = page_size; p.window = window; p.splits = splits;
  p.page_shift = page_shift;
  p.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(num_tiles, num_kv_heads, splits);
  const int dp = head_dim <= 64 ? 64 : 128;
  const int smem = part_rows <= 16 ? (lb::FA_ROWS + 2 * lb::FA_STAGES * lb::FA_KEYS) * dp * 2   // query tile + 3 stages
                                   : 2 * 2 * lb::FA_KEYS * dp * 2;                             // 2 stages, query tile aliased
  const bool keysplit = part_rows <= 16;      // no tile has more than 16 query rows: the warps share them
  const bool clustered = splits > 1 && may_cluster;
  p.cluster = clustered ? splits : 0;
  if (by_tma) {
    CUtensorMap mk, mv;
    const long long pool_rows = (long long)num_pages * num_kv_heads * page_size;
    const int box = page_size < lb::FA_KEYS ? page_size : lb::FA_KEYS;
    if (!lb::fd_pool_map(&mk, k_cache, pool_rows, head_dim, box) || !lb::fd_pool_map(&mv, v_cache, pool_rows, head_dim, box)) {
      lb::set_error("attention_flash: cuTensorMapEncodeTiled failed (pool of %lld rows of %d)", pool_rows, head_dim);
      return 3;
    }
    const int fd_smem = 1024 + lb::FD_STAGES * 2 * (dp / 64) * 8192 + 16 * dp * 2;
    static bool fd_cfg[2] = {false, false};
    void (*kern)(CUtensorMap, CUtensorMap, lb::FlashParams) = dp == 64 ? lb::flash_decode_tma_kernel<64> : lb::flash_decode_tma_kernel<128>;
    if (!fd_cfg[dp == 64]) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fd_smem);
      if (e != cudaSuccess) { lb::set_error("attention_flash: cannot reserve %d bytes of shared memory: %s", fd_smem, cudaGetErrorString(e)); return 2; }
      fd_cfg[dp == 64] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(lb::FD_THREADS); cfg.dynamicSmemBytes = fd_smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (clustered) {
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 1; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = splits;
      ++na;
    }
    if (lb::g_pdl_enabled) {
      attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    cfg.attrs = attr; cfg.numAttrs = na;
    cudaLaunchKernelEx(&cfg, kern, mk, mv, p);
    LB_CHECK_LAUNCH("attention_flash (tma)");
    if (splits > 1 && !clustered) {
      dim3 cgrid(num_tiles, num_kv_heads, (part_rows + 3) / 4), cblock(32, 4);
      lb::launch(lb::flash_combine_kernel, cgrid, cblock, (size_t)4 * splits * sizeof(float), stream, p);
      LB_CHECK_LAUNCH("attention_flash combine");
    }
    return 0;
  }
#define LB_FLASH_LAUNCH(DP, KS)                                                                                 \
  do {                                                                                                          \
    static bool cfg = false;                                                                                    \
    if (!cfg) {                                                                                                 \
      cudaFuncSetAttribute(lb::flash_attention_kernel<DP, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
      cfg = true;                                                                                               \
    }                                                                                                           \
    if (clustered) {                                                                                            \
      cudaLaunchConfig_t cfg = {};                                                                              \
      cfg.gridDim = grid; cfg.blockDim = dim3(lb::FA_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream; \
      cudaLaunchAttribute attr[2];                                                                              \
      attr[0].id = cudaLaunchAttributeClusterDimension;                                                         \
      attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = splits;            \
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                          \
      attr[1].val.programmaticStreamSerializationAllowed = 1;                                                   \
      cfg.attrs = attr; cfg.numAttrs = lb::g_pdl_enabled ? 2 : 1;                                               \
      cudaLaunchKernelEx(&cfg, lb::flash_attention_kernel<DP, KS>, p);                                          \
    } else {                                                                                                    \
      lb::launch(lb::flash_attention_kernel<DP, KS>, grid, dim3(lb::FA_THREADS), smem, stream, p);              \
    }                                                                                                           \
  } while (0)
  if (dp == 64) { if (keysplit) LB_FLASH_LAUNCH(64, true); else LB_FLASH_LAUNCH(64, false); }
  else { if (keysplit) LB_FLASH_LAUNCH(128, true); else LB_FLASH_LAUNCH(128, false); }
#undef LB_FLASH_LAUNCH
  LB_CHECK_LAUNCH("attention_flash");
  if (splits > 1 && !clustered) {
    dim3 cgrid(num_tiles, num_kv_heads, (part_rows + 3) / 4), cblock(32, 4);
    lb::launch(lb::flash_combine_kernel, cgrid, cblock, (size_t)4 * splits * sizeof(float), stream, p);
    LB_CHECK_LAUNCH("attention_flash combine");
  }
  return 0;
}
