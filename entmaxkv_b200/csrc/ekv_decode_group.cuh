// Paged entmax decode for GQA groups of four or eight query heads per KV head (GS below): the shared (union)
// page table with membership masks and the group-shared K pass that fetches every row once and scores it against
// the group's queries with tensor-core tiles.
#pragma once

#include <cooperative_groups.h>

#include "ekv_decode_args.cuh"

namespace ekv {

// ---- shared page table of a GQA group ---------------------------------------------------------

constexpr int kUnionThreads = 512;

// grid: B*H_kv blocks.  Merges the ascending page tables of the group's GS query heads into
// one ascending table (written to the rows of all GS heads, so every later stage can keep
// indexing by query head), with a GS-bit membership mask per entry, the token count of the
// union, and the K pass's work list over groups: fixed slots (group, chunk), empty past the end.
template <int GS>
__global__ void __launch_bounds__(kUnionThreads)
group_union_kernel(ekv_cache_desc c, int q_heads, const int* __restrict__ page_indices, int64_t pi_stride,
                   const int* __restrict__ num_selected, int max_tokens, int* __restrict__ u_pages,
                   int64_t u_stride, unsigned char* __restrict__ member, int64_t m_stride,
                   int* __restrict__ u_tok_heads, unsigned long long* __restrict__ g_items, int cph,
                   unsigned long long* __restrict__ h_items) {
  extern __shared__ uint32_t s_bits[];      // [GS][words]
  constexpr int ROUND = kUnionThreads * 16;
  __shared__ uint32_t scratch[40];
  __shared__ int s_ids[ROUND];              // the entries one round adds, in order, for coalesced stores
  __shared__ unsigned char s_masks[ROUND];
  const int gid = blockIdx.x, tid = threadIdx.x;
  const int b = gid / c.kv_heads, hkv = gid % c.kv_heads;
  const int bh0 = b * q_heads + hkv * GS;
  const int S = c.seq_lens[b], P = c.page_size;
  const int n_pages = min((S + P - 1) / P, c.page_capacity);
  const int words = (c.page_capacity + 31) / 32;
  for (int i = tid; i < GS * words; i += kUnionThreads) s_bits[i] = 0u;
  __syncthreads();
  for (int j = 0; j < GS; ++j) {
    const int n = num_selected[bh0 + j];
    const int* row = page_indices + (size_t)(bh0 + j) * pi_stride;
    for (int i = tid; i < n; i += kUnionThreads) {
      const int pg = row[i];
      if ((unsigned)pg < (unsigned)n_pages) atomicOr(&s_bits[j * words + (pg >> 5)], 1u << (pg & 31));
    }
  }
  __syncthreads();
  int count = 0;
  bool has_last = false;
  for (int r0 = 0; r0 < n_pages; r0 += ROUND) {
    const int id0 = r0 + tid * 16;
    uint32_t m16[GS];
    uint32_t any = 0u;
#pragma unroll
    for (int j = 0; j < GS; ++j) m16[j] = 0u;
    if (id0 < n_pages) {
      const int w = id0 >> 5, sh = id0 & 16;
#pragma unroll
      for (int j = 0; j < GS; ++j) {
        m16[j] = (s_bits[j * words + w] >> sh) & 0xffffu;
        any |= m16[j];
      }
    }
    uint32_t total;
    int pos = (int)block_scan_excl((uint32_t)__popc(any), scratch, &total);
#pragma unroll 4
    for (int k = 0; k < 16; ++k)
      if ((any >> k) & 1u) {
        const int id = id0 + k;
        s_ids[pos] = id;
        uint32_t mk = 0u;
#pragma unroll
        for (int j = 0; j < GS; ++j) mk |= ((m16[j] >> k) & 1u) << j;
        s_masks[pos] = (unsigned char)mk;
        if (id == n_pages - 1) has_last = true;
        ++pos;
      }
    __syncthreads();
    for (int i = tid; i < (int)total; i += kUnionThreads) {
      const int id = s_ids[i];
#pragma unroll
      for (int j = 0; j < GS; ++j) u_pages[(size_t)(bh0 + j) * u_stride + count + i] = id;
      member[(size_t)gid * m_stride + count + i] = s_masks[i];
    }
    count += (int)total;
    __syncthreads();
  }
  // the in-progress last page is the largest id: if present it is the final entry and holds fewer rows
  __shared__ int s_last;
  if (tid == 0) s_last = 0;
  __syncthreads();
  if (has_last) s_last = 1;
  __syncthreads();
  const int last_tokens = S - (n_pages - 1) * P;
  const int T = min(count * P - (s_last ? P - last_tokens : 0), max_tokens);
  if (tid < GS) u_tok_heads[bh0 + tid] = T;
  for (int ch = tid; ch < cph; ch += kUnionThreads)
    g_items[(size_t)gid * cph + ch] =
        ch * kChunkTokens < T ? make_item(bh0, ch, T) : 0ull;
  // the per-head list over the union (tau kernel and V pass): fixed slots (head, chunk)
  if (h_items)
    for (int i = tid; i < GS * cph; i += kUnionThreads)
      h_items[(size_t)bh0 * cph + i] = make_item(bh0 + i / cph, i % cph, T);
}

// First index i in [0, n) with row[i] >= key (n if none) of an ascending row: the 32 lanes of a warp probe 32
// evenly spaced positions per round, so a table of tens of thousands of entries takes three or four dependent
// loads instead of fifteen.  Warp-collective; every lane returns the answer.
__device__ __forceinline__ int warp_lower_bound(const int* __restrict__ row, int n, int key) {
  const int lane = threadIdx.x & 31;
  int lo = 0, hi = n;
  while (hi > lo) {
    const long long span = hi - lo;
    const int p = lo + (int)(((long long)(lane + 1) * span) / 33);      // non-decreasing in the lane, < hi
    const uint32_t below = __ballot_sync(0xffffffffu, __ldg(row + p) < key);   // a prefix of ones
    const int cnt = __popc(below);
    const int p_last = __shfl_sync(0xffffffffu, p, max(cnt - 1, 0));
    const int p_next = __shfl_sync(0xffffffffu, p, min(cnt, 31));
    if (cnt > 0) lo = p_last + 1;
    if (cnt < 32) hi = p_next;
  }
  return lo;
}

// The same union for FEW groups (a long request: B*H_kv blocks would leave the GPU idle and one block would
// walk tens of thousands of pages alone): a thread-block cluster of CL blocks per group.  Block r of the
// cluster owns the page ids [r*seg, (r+1)*seg): it finds its slice of every head's ascending table by
// warp_lower_bound, builds the bitmaps of its slice only, counts its union entries, trades the counts with
// the other blocks over distributed shared memory (plain remote stores + a cluster barrier) and writes its
// entries at the prefix of the lower blocks' counts.  Same outputs as group_union_kernel, bit for bit.
template <int GS, int CL>
__global__ void __launch_bounds__(kUnionThreads)
group_union_cluster_kernel(ekv_cache_desc c, int q_heads, const int* __restrict__ page_indices, int64_t pi_stride,
                           const int* __restrict__ num_selected, int max_tokens, int* __restrict__ u_pages,
                           int64_t u_stride, unsigned char* __restrict__ member, int64_t m_stride,
                           int* __restrict__ u_tok_heads, unsigned long long* __restrict__ g_items, int cph,
                           unsigned long long* __restrict__ h_items) {
  namespace cg = cooperative_groups;
  extern __shared__ uint32_t s_bits[];      // [GS][seg_words]
  constexpr int ROUND = kUnionThreads * 16;
  __shared__ uint32_t scratch[40];
  __shared__ int s_ids[ROUND];
  __shared__ unsigned char s_masks[ROUND];
  __shared__ int s_lo[GS], s_hi[GS];
  __shared__ uint32_t s_cnt[CL];            // every block's {has_last : count}, written by its owner over DSMEM
  cg::cluster_group cluster = cg::this_cluster();
  const int r = (int)cluster.block_rank();
  const int gid = blockIdx.x / CL, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = gid / c.kv_heads, hkv = gid % c.kv_heads;
  const int bh0 = b * q_heads + hkv * GS;
  const int S = c.seq_lens[b], P = c.page_size;
  const int n_pages = min((S + P - 1) / P, c.page_capacity);
  const int seg = ((n_pages + CL - 1) / CL + 31) / 32 * 32;      // whole bitmap words per block
  const int seg_words = seg / 32;
  const int id_lo = r * seg, id_hi = min(id_lo + seg, n_pages);   // this block's page ids
  cluster.sync();                            // every block of the cluster is running: remote stores may begin
  for (int i = tid; i < GS * seg_words; i += kUnionThreads) s_bits[i] = 0u;
  // slice [s_lo[j], s_hi[j]) of head j's table that falls into this block's ids: warp 2j finds the start,
  // warp 2j + 1 the end
  if (warp < 2 * GS) {
    const int j = warp >> 1;
    const int n = num_selected[bh0 + j];
    const int* row = page_indices + (size_t)(bh0 + j) * pi_stride;
    const int pos = warp_lower_bound(row, n, (warp & 1) ? id_hi : id_lo);
    if (lane == 0) ((warp & 1) ? s_hi : s_lo)[j] = pos;
  }
  __syncthreads();
  for (int j = 0; j < GS; ++j) {
    const int* row = page_indices + (size_t)(bh0 + j) * pi_stride;
    for (int i = s_lo[j] + tid; i < s_hi[j]; i += kUnionThreads) {
      const int pg = row[i] - id_lo;
      if ((unsigned)pg < (unsigned)seg) atomicOr(&s_bits[j * seg_words + (pg >> 5)], 1u << (pg & 31));
    }
  }
  __syncthreads();
  // this block's union entries, and whether the sequence's last page is among them
  uint32_t mine = 0;
  for (int w = tid; w < seg_words; w += kUnionThreads) {
    uint32_t any = 0u;
#pragma unroll
    for (int j = 0; j < GS; ++j) any |= s_bits[j * seg_words + w];
    mine += (uint32_t)__popc(any);
  }
  uint32_t my_count;
  block_scan_excl(mine, scratch, &my_count);
  bool last_here = false;
  if (n_pages >= 1 && n_pages - 1 >= id_lo && n_pages - 1 < id_hi) {
    const int pg = n_pages - 1 - id_lo;
#pragma unroll
    for (int j = 0; j < GS; ++j) last_here |= (s_bits[j * seg_words + (pg >> 5)] >> (pg & 31)) & 1u;
  }
  if (tid < CL) cluster.map_shared_rank(s_cnt, tid)[r] = my_count | (last_here ? 0x80000000u : 0u);
  cluster.sync();
  int count = 0, total = 0;
  bool has_last = false;
#pragma unroll
  for (int q = 0; q < CL; ++q) {
    const uint32_t v = s_cnt[q];
    if (q < r) count += (int)(v & 0x7fffffffu);
    total += (int)(v & 0x7fffffffu);
    has_last |= (v >> 31) != 0u;
  }
  for (int r0 = 0; r0 < seg; r0 += ROUND) {
    const int l0 = r0 + tid * 16;                 // local id of this thread's first page
    uint32_t m16[GS];
    uint32_t any = 0u;
#pragma unroll
    for (int j = 0; j < GS; ++j) m16[j] = 0u;
    if (l0 < seg && id_lo + l0 < n_pages) {
      const int w = l0 >> 5, sh = l0 & 16;
#pragma unroll
      for (int j = 0; j < GS; ++j) {
        m16[j] = (s_bits[j * seg_words + w] >> sh) & 0xffffu;
        any |= m16[j];
      }
    }
    uint32_t round_total;
    int pos = (int)block_scan_excl((uint32_t)__popc(any), scratch, &round_total);
#pragma unroll 4
    for (int k = 0; k < 16; ++k)
      if ((any >> k) & 1u) {
        s_ids[pos] = id_lo + l0 + k;
        uint32_t mk = 0u;
#pragma unroll
        for (int j = 0; j < GS; ++j) mk |= ((m16[j] >> k) & 1u) << j;
        s_masks[pos] = (unsigned char)mk;
        ++pos;
      }
    __syncthreads();
    for (int i = tid; i < (int)round_total; i += kUnionThreads) {
      const int id = s_ids[i];
#pragma unroll
      for (int j = 0; j < GS; ++j) u_pages[(size_t)(bh0 + j) * u_stride + count + i] = id;
      member[(size_t)gid * m_stride + count + i] = s_masks[i];
    }
    count += (int)round_total;
    __syncthreads();
  }
  const int last_tokens = S - (n_pages - 1) * P;
  const int T = min(total * P - (has_last ? P - last_tokens : 0), max_tokens);
  if (r == 0 && tid < GS) u_tok_heads[bh0 + tid] = T;
  for (int ch = r * kUnionThreads + tid; ch < cph; ch += CL * kUnionThreads)
    g_items[(size_t)gid * cph + ch] = ch * kChunkTokens < T ? make_item(bh0, ch, T) : 0ull;
  if (h_items)
    for (int i = r * kUnionThreads + tid; i < GS * cph; i += CL * kUnionThreads)
      h_items[(size_t)bh0 * cph + i] = make_item(bh0 + i / cph, i % cph, T);
}

// ---- group-shared K pass (GQA groups of four or eight) -----------------------------------
//
// The query heads of a GQA group read the same K rows.  When the heads keep a large part of
// the pages (Gaussian-aware selection: ~44 % each at 128k), scoring them one head at a time
// fetches most rows several times.  Here the group shares ONE page table - the ascending
// union of its heads' selections, with a membership bit per head and entry - and an item is a
// 256-token chunk of that table: every page is fetched once and each of its rows is scored
// against the group's queries at once.
// Head j's score of a row is written to head j's score row at the union position; rows of
// pages head j did not select get -inf, which no later stage can take into a support, so
// tau and the output are those of the per-head lists.  Statistics are kept per head.

// Warp maximum in one instruction: floats map monotonically to signed integers
// (negative values: all bits below the sign flipped), and redux.sync takes the integer maximum.
__device__ __forceinline__ float warp_max_redux(float v) {
  int k = __float_as_int(v);
  k ^= (k >> 31) & 0x7fffffff;
  k = __reduce_max_sync(0xffffffffu, k);
  k ^= (k >> 31) & 0x7fffffff;
  return __int_as_float(k);
}

// Tensor-core pieces of the group-shared K pass.  A score block is a 16x8 tile: 16 K rows by
// the group's queries (groups of four: columns 4..7 are zero padding), contracted 16 elements at a time.
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma_rows_by_queries(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (sizeof(T) == 2 && !std::is_same<T, __half>::value) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Shared-memory placement of page slot s of a stage: slots are skewed by 16 bytes modulo 128,
// so the same in-page row of eight consecutive slots falls into eight different bank groups
// and an 8x8 fragment whose rows come from eight slots loads without bank conflicts (rows of
// one page are 256 bytes apart and would all collide).  Every eight slots the skew starts
// over, 128 bytes further, so that slot 8k does not overlap the skewed end of slot 8k-1.
constexpr size_t kGroupStageBytes = (size_t)kChunkTokens * 128 * 2 + 128 * (kChunkTokens / 4 / 8);
__device__ __forceinline__ uint32_t group_slot_offset(int slot, int page_bytes) {
  return (uint32_t)(slot * page_bytes + (slot & 7) * 16 + (slot >> 3) * 128);
}

// Fold of the run statistics: thread tid holds the partials of the heads tid / 128 + 4 p, p < GS / 4.
template <int GS>
__device__ __forceinline__ void group_run_store(const DecodeArgs& a, float (*red)[16][4], float (&s0)[GS / 4],
                                                float (&s1)[GS / 4], float (&s2)[GS / 4], float (&mx)[GS / 4],
                                                int bh0, int chunk) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int p = 0; p < GS / 4; ++p) {
    float v0 = s0[p], v1 = s1[p], v2 = s2[p], v3 = mx[p];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      v0 += __shfl_xor_sync(0xffffffffu, v0, o);
      v1 += __shfl_xor_sync(0xffffffffu, v1, o);
      v2 += __shfl_xor_sync(0xffffffffu, v2, o);
      v3 = fmaxf(v3, __shfl_xor_sync(0xffffffffu, v3, o));
    }
    if (lane == 0) {
      red[p][warp][0] = v0;
      red[p][warp][1] = v1;
      red[p][warp][2] = v2;
      red[p][warp][3] = v3;
    }
  }
  __syncthreads();
  if (tid < 4 * GS) {
    const int j = tid >> 2, l = tid & 3;      // head j of the group: set j / 4, warps 4 (j % 4) .. + 3
    const int p = j >> 2, w0 = 4 * (j & 3);
    float v = red[p][w0][l];
#pragma unroll
    for (int w = 1; w < 4; ++w) v = l == 3 ? fmaxf(v, red[p][w0 + w][l]) : v + red[p][w0 + w][l];
    a.ws.part[((size_t)(bh0 + j) * a.ws.nchunks + chunk) * 4 + l] = v;
  }
}
template <int GS>
__device__ __forceinline__ void group_neutral_store(const DecodeArgs& a, int bh0, int chunk) {
  const int tid = threadIdx.x;
  if (tid < 4 * GS)
    a.ws.part[((size_t)(bh0 + (tid >> 2)) * a.ws.nchunks + chunk) * 4 + (tid & 3)] = (tid & 3) == 3 ? -1.0e6f : 0.f;
}

// A block owns an equal share of the NON-EMPTY items of the group list: group g has
// ceil(tok_counts[GS g] / 256) of them (chunks 0, 1, ... of its shared table), and the pass
// enumerates them arithmetically instead of walking the fixed-slot list, whose empty slots past
// every group's end would cost a barrier each (three quarters of the slots when the selection
// is sparse).  Block-collective.  Returns the block's first item as (group, chunk) and its count.
__device__ __forceinline__ void group_item_range(const DecodeArgs& a, int gs, int& first_group, int& first_chunk,
                                                 int& n_mine) {
  __shared__ uint32_t scan[33];
  __shared__ int s_group, s_chunk;
  const int tid = threadIdx.x;
  const int n_groups = a.c.batch * a.c.kv_heads;
  auto chunks_of = [&](int g) -> uint32_t {
    return g < n_groups ? (uint32_t)((min(a.tok_counts[g * gs], a.max_tokens) + kChunkTokens - 1) / kChunkTokens) : 0u;
  };
  uint32_t mine = 0, total;
  for (int g = tid; g < n_groups; g += blockDim.x) mine += chunks_of(g);
  block_scan_excl(mine, scan, &total);
  const long long lo = (long long)total * blockIdx.x / gridDim.x;
  const long long hi = (long long)total * (blockIdx.x + 1) / gridDim.x;
  if (tid == 0) s_group = s_chunk = 0;
  __syncthreads();
  uint32_t running = 0;
  for (int g0 = 0; g0 < n_groups; g0 += blockDim.x) {
    const int g = g0 + tid;
    const uint32_t cnt = chunks_of(g);
    uint32_t round_total;
    const long long ex = (long long)running + block_scan_excl(cnt, scan, &round_total);
    if (hi > lo && cnt > 0 && lo >= ex && lo < ex + cnt) {
      s_group = g;
      s_chunk = (int)(lo - ex);
    }
    running += round_total;
  }
  __syncthreads();
  first_group = s_group;
  first_chunk = s_chunk;
  n_mine = (int)(hi - lo);
}

// The head field of a group item is the group's FIRST query head (b*H_q + h_kv*GS); the
// heads of the group are that and the next GS - 1.  Its page table row is the shared table.
//
// Per item (a 256-token chunk of the shared table, staged by the bulk-copy pipeline):
//   1. warp u computes the 16xGS score block of 16 rows of the chunk - one row of each of up
//      to 16 page slots - with eight m16n8k16 tensor-core steps over head_dim 128 (A = K rows
//      read from the skewed stage with ldmatrix, B = the group's queries, fp32 accumulators) and
//      parks it in shared memory,
//   2. after one block barrier, thread t takes head t / 128 (groups of eight: and head t / 128 + 4)
//      and two tokens (a warp takes a 64-token quarter of the chunk): applies the
//      membership mask (-inf for pages the head did not select), stores the scores and
//      accumulates the head's statistics.
// The arithmetic per row is a few tensor-core instructions, so the pass is bound by the bytes
// of the shared table, not by the number of heads.
template <typename T, int NS, int GS>
__global__ void __launch_bounds__(kDecThreads, 1) decode_scores_group_kernel(const DecodeArgs a) {
  constexpr int D = 128;
  constexpr int HP = GS / 4;          // heads per thread in step 2
  static_assert(GS == 4 || GS == 8, "groups of four or eight");
  static_assert(sizeof(T) == 2 && kDecThreads == 512 && kChunkTokens == 256, "16 warps, one per row set");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t full[NS];
  __shared__ float red[HP][16][4];
  // score blocks of two items in flight; token t of a head sits at t + t/16 and heads are 276
  // floats apart, so the fragment stores of step 1 (eight tokens 16 apart, two heads per lane: 16 banks for
  // groups of four, all 32 for groups of eight) do not collide
  constexpr int kZHead = kChunkTokens + 20;
  __shared__ float s_z[2][GS][kZHead];
  __shared__ unsigned char s_mem[4][kChunkTokens / 4];    // membership masks of four items in flight

  const int kind = alpha_kind_of(a.alpha);
  const float beta = 1.f / (a.alpha - 1.f);
  const float qscale = (a.alpha - 1.f) * 0.08838834764831845f;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int P = a.pd.P, shift = a.pd.shift;
  const int page_bytes = P * D * (int)sizeof(T);
  const int ppw = 32 >> shift;
  const int my_slot = (warp < kIssueWarps && lane < ppw) ? warp * ppw + lane : -1;

  // fragment geometry of this lane: rows of the score block <-> (page slot, row in page)
  const int npg = min(kChunkTokens >> shift, 16);
  auto slot_of = [&](int i) { return (i % npg) + 16 * (warp >> shift); };
  auto row_of = [&](int i) { return (warp & (P - 1)) + 16 * (i / npg); };
  const int frag_i = (lane & 7) + 8 * ((lane >> 3) & 1);          // ldmatrix: the row this lane addresses
  const uint32_t frag_off = group_slot_offset(slot_of(frag_i), page_bytes) + (uint32_t)row_of(frag_i) * (D * 2) +
                            (uint32_t)(lane >> 4) * 16;
  const int g = lane >> 2, t4 = lane & 3;
  const int tok_lo = slot_of(g) * P + row_of(g), tok_hi = slot_of(g + 8) * P + row_of(g + 8);
  const int my_head = tid >> 7, my_tok = ((warp & 3) << 6) + lane;  // step 2: head, first token of the warp's quarter

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) mbar_init(&full[s], kIssueWarps);
    mbar_fence_init();
  }
  __syncthreads();

  int gen_group, gen_chunk, n_mine;
  group_item_range(a, GS, gen_group, gen_chunk, n_mine);
  // Items come in list order from a generator (every call returns the next one): group g's first
  // query head is GS g, its items are the chunks of its shared table.
  const int n_groups = a.c.batch * a.c.kv_heads;
  int gen_left = n_mine;
  int gen_tok = n_mine > 0 ? min(a.tok_counts[gen_group * GS], a.max_tokens) : 0;
  auto next_desc = [&]() -> unsigned long long {
    if (gen_left <= 0) return 0ull;
    --gen_left;
    while (gen_chunk * kChunkTokens >= gen_tok && gen_group + 1 < n_groups) {   // block-uniform, rare
      ++gen_group;
      gen_chunk = 0;
      gen_tok = min(a.tok_counts[gen_group * GS], a.max_tokens);
    }
    if (gen_chunk * kChunkTokens >= gen_tok) return 0ull;
    return make_item(gen_group * GS, gen_chunk++, gen_tok);
  };
  // Page id and membership mask of this lane's slot (-1: no page).  The two loads are consumed one
  // item later, in issue(); nothing here touches their results, so an in-order warp does not wait
  // for them at the top of the iteration.
  struct SlotPage { int page, mask; };
  auto load_page = [&](unsigned long long d) -> SlotPage {
    SlotPage r;
    r.page = -1;
    r.mask = 0;
    if (my_slot >= 0 && my_slot * P < item_ntok(d)) {
      const int rank = ((item_chunk(d) * kChunkTokens) >> shift) + my_slot;
      const int gid = item_head(d) / GS;       // first query head of the group: GS * gid
      r.page = a.page_indices[(size_t)item_head(d) * a.pi_stride + rank];
      r.mask = a.member[(size_t)gid * a.member_stride + rank];
    }
    return r;
  };
  auto issue = [&](unsigned long long d, SlotPage sp, int st, int mslot) {
    const int ntok = item_ntok(d);
    if (ntok == 0 || warp >= kIssueWarps) return;
    int b, hq;
    a.div_heads.divmod(item_head(d), b, hq);
    const int hkv = a.div_group.div(hq);
    int rows = 0;
    if (my_slot >= 0 && my_slot * P < ntok) rows = min(P, ntok - my_slot * P);
    int page = sp.page;
    if (rows > 0) s_mem[mslot][my_slot] = (unsigned char)(sp.mask & ((1 << GS) - 1));
    if (rows > 0 && (unsigned)page >= (unsigned)a.page_limit) {
      atomicOr(a.ws.status, EKV_STATUS_PAGE_RANGE);
      page = 0;
    }
    const uint32_t bytes = (uint32_t)(rows * D * sizeof(T));
    uint32_t wbytes = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wbytes += __shfl_xor_sync(0xffffffffu, wbytes, o);
    if (lane == 0) mbar_expect_tx(&full[st], wbytes);
    __syncwarp();
    if (rows > 0) {
      const T* src = static_cast<const T*>(a.c.k) + b * a.kv_sb + hkv * a.c.kv_stride_h +
                     (size_t)page * a.kv_ps;
      bulk_load(smem_raw + (size_t)st * kGroupStageBytes + group_slot_offset(my_slot, page_bytes), src, bytes,
                &full[st]);
    }
  };

  // NS items are in flight; the stage of item k is refilled with item k + NS as soon as step 1
  // of item k is over (step 2 works from the parked scores), so the copy engine never waits
  // for the stores and the statistics.
  unsigned long long dq[NS + 1];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    dq[j] = next_desc();
    issue(dq[j], load_page(dq[j]), j, j & 3);
  }
  dq[NS] = next_desc();
  SlotPage pg_next = load_page(dq[NS]);
  unsigned long long dB = next_desc();   // descriptors run one item ahead of their page look-ups
  uint32_t phase_bits = 0;
  uint32_t bq[8][2];                  // B fragments: query g (< GS) of the loaded group, all of head_dim
  int loaded_head = -1;
  float tau0[HP], s0[HP], s1[HP], s2[HP], mx[HP];     // of the heads my_head + 4 p: incoming tau, run statistics
#pragma unroll
  for (int p = 0; p < HP; ++p) {
    tau0[p] = s0[p] = s1[p] = s2[p] = 0.f;
    mx[p] = -1.0e6f;
  }

  for (int k = 0; k < n_mine; ++k) {
    const SlotPage pgB = load_page(dB);
    const unsigned long long dC = next_desc();
    const unsigned long long dn = dq[1];   // item k+1

    const int st = k % NS;
    const unsigned long long dk = dq[0];
    const int ntok = item_ntok(dk);
    if (ntok > 0) {
      const int bh0 = item_head(dk), chunk = item_chunk(dk);
      if (bh0 != loaded_head) {          // block-uniform: a new group starts
        loaded_head = bh0;
        int b, hq;
        a.div_heads.divmod(bh0, b, hq);
        const T* qrow = static_cast<const T*>(a.q) + b * a.qsb + (hq + (g & (GS - 1))) * a.qsh;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t4);
          bq[ks][0] = g < GS ? w0 : 0u;
          bq[ks][1] = g < GS ? w1 : 0u;
        }
#pragma unroll
        for (int p = 0; p < HP; ++p) tau0[p] = a.tau_mode == EKV_TAU_EXACT ? 0.f : a.tau[bh0 + my_head + 4 * p];
      }
      mbar_wait_or_flag(&full[st], (phase_bits >> st) & 1u, a.ws.status);
      phase_bits ^= 1u << st;
      // step 1: the 16xGS score block of this warp's rows
      const uint32_t a_addr = smem_addr(smem_raw + (size_t)st * kGroupStageBytes) + frag_off;
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t af[4];
        ldmatrix_x4(a_addr + ks * 32, af);
        mma_rows_by_queries<T>(d4, af, bq[ks][0], bq[ks][1]);
      }
      float (*zb)[kZHead] = s_z[k & 1];
      if (2 * t4 < GS) {
        zb[2 * t4][tok_lo + (tok_lo >> 4)] = d4[0] * qscale;
        zb[2 * t4 + 1][tok_lo + (tok_lo >> 4)] = d4[1] * qscale;
        zb[2 * t4][tok_hi + (tok_hi >> 4)] = d4[2] * qscale;
        zb[2 * t4 + 1][tok_hi + (tok_hi >> 4)] = d4[3] * qscale;
      }
      __syncthreads();   // the block's scores are parked; nobody reads the stage any more
      issue(dq[NS], pg_next, st, (k + NS) & 3);
      // step 2: mask, store, statistics
      const unsigned char* mem = s_mem[k & 3];
#pragma unroll
      for (int p = 0; p < HP; ++p) {
        const int head = my_head + 4 * p;
        float* zrow = a.ws.z + (size_t)(bh0 + head) * a.ws.zstride + chunk * kChunkTokens;
        float wmax = -INFINITY;      // over this warp's 64-token quarter of the chunk: lets the tau kernel skip it
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int i = my_tok + 32 * h;
          if (i < ntok) {
            const bool mine = (mem[i >> shift] >> head) & 1;
            const float zv = zb[head][i + (i >> 4)];
            zrow[i] = mine ? zv : -INFINITY;
            if (mine) {
              wmax = fmaxf(wmax, zv);
              mx[p] = fmaxf(mx[p], zv);
              if (a.tau_mode != EKV_TAU_EXACT) halley_accumulate(zv, tau0[p], kind, beta, s0[p], s1[p], s2[p]);
            }
          }
        }
        wmax = warp_max_redux(wmax);
        if (lane == 0) a.ws.cmax[((size_t)(bh0 + head) * a.ws.nchunks + chunk) * 4 + (warp & 3)] = wmax;
      }
      if (same_run(dk, dn)) {
        group_neutral_store<GS>(a, bh0, chunk);
      } else {
        group_run_store<GS>(a, red, s0, s1, s2, mx, bh0, chunk);
#pragma unroll
        for (int p = 0; p < HP; ++p) {
          s0[p] = s1[p] = s2[p] = 0.f;
          mx[p] = -1.0e6f;
        }
      }
    } else {
      __syncthreads();   // one barrier per item: the mask slot written next was read in the previous item
      issue(dq[NS], pg_next, st, (k + NS) & 3);
    }
#pragma unroll
    for (int j = 0; j < NS; ++j) dq[j] = dq[j + 1];
    dq[NS] = dB;
    pg_next = pgB;
    dB = dC;
  }
}

}  // namespace ekv
