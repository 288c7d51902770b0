// Paged entmax decode for GQA groups of four: the shared (union) page table with membership masks and the
// group-shared K pass that fetches every row once and scores it against the four queries with tensor-core tiles.
#pragma once

#include "ekv_decode_args.cuh"

namespace ekv {

// ---- shared page table of a GQA group of four ------------------------------------------------

constexpr int kUnionThreads = 512;

// grid: B*H_kv blocks.  Merges the ascending page tables of the group's four query heads into
// one ascending table (written to the rows of all four heads, so every later stage can keep
// indexing by query head), with a 4-bit membership mask per entry, the token count of the
// union, and the K pass's work list over groups: fixed slots (group, chunk), empty past the end.
__global__ void __launch_bounds__(kUnionThreads)
group_union_kernel(ekv_cache_desc c, int q_heads, const int* __restrict__ page_indices, int64_t pi_stride,
                   const int* __restrict__ num_selected, int max_tokens, int* __restrict__ u_pages,
                   int64_t u_stride, unsigned char* __restrict__ member, int64_t m_stride,
                   int* __restrict__ u_tok_heads, unsigned long long* __restrict__ g_items, int cph) {
  extern __shared__ uint32_t s_bits[];      // [4][words]
  constexpr int ROUND = kUnionThreads * 16;
  __shared__ uint32_t scratch[40];
  __shared__ int s_ids[ROUND];              // the entries one round adds, in order, for coalesced stores
  __shared__ unsigned char s_masks[ROUND];
  const int gid = blockIdx.x, tid = threadIdx.x;
  const int b = gid / c.kv_heads, hkv = gid % c.kv_heads;
  const int bh0 = b * q_heads + hkv * 4;
  const int S = c.seq_lens[b], P = c.page_size;
  const int n_pages = min((S + P - 1) / P, c.page_capacity);
  const int words = (c.page_capacity + 31) / 32;
  for (int i = tid; i < 4 * words; i += kUnionThreads) s_bits[i] = 0u;
  __syncthreads();
  for (int j = 0; j < 4; ++j) {
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
    uint32_t m16[4] = {0u, 0u, 0u, 0u};
    if (id0 < n_pages) {
      const int w = id0 >> 5, sh = id0 & 16;
#pragma unroll
      for (int j = 0; j < 4; ++j) m16[j] = (s_bits[j * words + w] >> sh) & 0xffffu;
    }
    const uint32_t any = m16[0] | m16[1] | m16[2] | m16[3];
    uint32_t total;
    int pos = (int)block_scan_excl((uint32_t)__popc(any), scratch, &total);
#pragma unroll 4
    for (int k = 0; k < 16; ++k)
      if ((any >> k) & 1u) {
        const int id = id0 + k;
        s_ids[pos] = id;
        s_masks[pos] = (unsigned char)(((m16[0] >> k) & 1u) | (((m16[1] >> k) & 1u) << 1) |
                                       (((m16[2] >> k) & 1u) << 2) | (((m16[3] >> k) & 1u) << 3));
        if (id == n_pages - 1) has_last = true;
        ++pos;
      }
    __syncthreads();
    for (int i = tid; i < (int)total; i += kUnionThreads) {
      const int id = s_ids[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) u_pages[(size_t)(bh0 + j) * u_stride + count + i] = id;
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
  if (tid < 4) u_tok_heads[bh0 + tid] = T;
  for (int ch = tid; ch < cph; ch += kUnionThreads)
    g_items[(size_t)gid * cph + ch] =
        ch * kChunkTokens < T ? make_item(bh0, ch, T) : 0ull;
}

// ---- group-shared K pass (GQA groups of four) ------------------------------------------
//
// The query heads of a GQA group read the same K rows.  When the heads keep a large part of
// the pages (Gaussian-aware selection: ~44 % each at 128k), scoring them one head at a time
// fetches most rows several times.  Here the group shares ONE page table - the ascending
// union of its heads' selections, with a 4-bit membership mask per entry - and an item is a
// 256-token chunk of that table: every page is fetched once and each of its rows is scored
// against the four queries at once (the quad reduction runs over heads instead of rows).
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
// the group's four queries (columns 4..7 are zero padding), contracted 16 elements at a time.
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

// Fold of the run statistics: thread tid holds the partial of head tid / 128.
__device__ __forceinline__ void group_run_store(const DecodeArgs& a, float (*red)[4], float s0, float s1, float s2,
                                                float mx, int bh0, int chunk) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s0 += __shfl_xor_sync(0xffffffffu, s0, o);
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0) {
    red[warp][0] = s0;
    red[warp][1] = s1;
    red[warp][2] = s2;
    red[warp][3] = mx;
  }
  __syncthreads();
  if (tid < 16) {
    const int j = tid >> 2, l = tid & 3;      // head j of the group: warps 4j .. 4j+3
    float v = red[4 * j][l];
#pragma unroll
    for (int w = 1; w < 4; ++w) v = l == 3 ? fmaxf(v, red[4 * j + w][l]) : v + red[4 * j + w][l];
    a.ws.part[((size_t)(bh0 + j) * a.ws.nchunks + chunk) * 4 + l] = v;
  }
}
__device__ __forceinline__ void group_neutral_store(const DecodeArgs& a, int bh0, int chunk) {
  const int tid = threadIdx.x;
  if (tid < 16)
    a.ws.part[((size_t)(bh0 + (tid >> 2)) * a.ws.nchunks + chunk) * 4 + (tid & 3)] = (tid & 3) == 3 ? -1.0e6f : 0.f;
}

// A block owns an equal share of the NON-EMPTY items of the group list: group g has
// ceil(tok_counts[4g] / 256) of them (chunks 0, 1, ... of its shared table), and the pass
// enumerates them arithmetically instead of walking the fixed-slot list, whose empty slots past
// every group's end would cost a barrier each (three quarters of the slots when the selection
// is sparse).  Block-collective.  Returns the block's first item as (group, chunk) and its count.
__device__ __forceinline__ void group_item_range(const DecodeArgs& a, int& first_group, int& first_chunk,
                                                 int& n_mine) {
  __shared__ uint32_t scan[33];
  __shared__ int s_group, s_chunk;
  const int tid = threadIdx.x;
  const int n_groups = a.c.batch * a.c.kv_heads;
  auto chunks_of = [&](int g) -> uint32_t {
    return g < n_groups ? (uint32_t)((min(a.tok_counts[g * 4], a.max_tokens) + kChunkTokens - 1) / kChunkTokens) : 0u;
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

// The head field of a group item is the group's FIRST query head (b*H_q + h_kv*4); the four
// heads of the group are that and the next three.  Its page table row is the shared table.
//
// Per item (a 256-token chunk of the shared table, staged by the bulk-copy pipeline):
//   1. warp u computes the 16x4 score block of 16 rows of the chunk - one row of each of up
//      to 16 page slots - with eight m16n8k16 tensor-core steps over head_dim 128 (A = K rows
//      read from the skewed stage with ldmatrix, B = the four queries, fp32 accumulators) and
//      parks it in shared memory,
//   2. after one block barrier, thread t takes head t / 128 and two tokens (a warp takes a
//      64-token quarter of the chunk): applies the
//      membership mask (-inf for pages the head did not select), stores the scores and
//      accumulates the head's statistics.
// The arithmetic per row is a few tensor-core instructions, so the pass is bound by the bytes
// of the shared table, not by the number of heads.
template <typename T, int NS>
__global__ void __launch_bounds__(kDecThreads, 1) decode_scores_group_kernel(const DecodeArgs a) {
  constexpr int D = 128;
  static_assert(sizeof(T) == 2 && kDecThreads == 512 && kChunkTokens == 256, "16 warps, one per row set");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t full[NS];
  __shared__ float red[16][4];
  // score blocks of two items in flight; token t of a head sits at t + t/16 and heads are 276
  // floats apart, so the fragment stores of step 1 (eight tokens 16 apart, two heads) hit 16 banks
  constexpr int kZHead = kChunkTokens + 20;
  __shared__ float s_z[2][4][kZHead];
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
  group_item_range(a, gen_group, gen_chunk, n_mine);
  // Items come in list order from a generator (every call returns the next one): group g's first
  // query head is 4g, its items are the chunks of its shared table.
  const int n_groups = a.c.batch * a.c.kv_heads;
  int gen_left = n_mine;
  int gen_tok = n_mine > 0 ? min(a.tok_counts[gen_group * 4], a.max_tokens) : 0;
  auto next_desc = [&]() -> unsigned long long {
    if (gen_left <= 0) return 0ull;
    --gen_left;
    while (gen_chunk * kChunkTokens >= gen_tok && gen_group + 1 < n_groups) {   // block-uniform, rare
      ++gen_group;
      gen_chunk = 0;
      gen_tok = min(a.tok_counts[gen_group * 4], a.max_tokens);
    }
    if (gen_chunk * kChunkTokens >= gen_tok) return 0ull;
    return make_item(gen_group * 4, gen_chunk++, gen_tok);
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
      const int gid = item_head(d) >> 2;       // groups of four: first query head 4 * gid
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
    if (rows > 0) s_mem[mslot][my_slot] = (unsigned char)(sp.mask & 0xf);
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
  uint32_t bq[8][2];                  // B fragments: query g (< 4) of the loaded group, all of head_dim
  int loaded_head = -1;
  float tau0 = 0.f;                   // of head `my_head` of the loaded group
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, mx = -1.0e6f;   // of head `my_head`, over the current run

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
        const T* qrow = static_cast<const T*>(a.q) + b * a.qsb + (hq + (g & 3)) * a.qsh;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t4);
          bq[ks][0] = g < 4 ? w0 : 0u;
          bq[ks][1] = g < 4 ? w1 : 0u;
        }
        tau0 = a.tau_mode == EKV_TAU_EXACT ? 0.f : a.tau[bh0 + my_head];
      }
      mbar_wait_or_flag(&full[st], (phase_bits >> st) & 1u, a.ws.status);
      phase_bits ^= 1u << st;
      // step 1: the 16x4 score block of this warp's rows
      const uint32_t a_addr = smem_addr(smem_raw + (size_t)st * kGroupStageBytes) + frag_off;
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t af[4];
        ldmatrix_x4(a_addr + ks * 32, af);
        mma_rows_by_queries<T>(d4, af, bq[ks][0], bq[ks][1]);
      }
      float (*zb)[kZHead] = s_z[k & 1];
      if (t4 < 2) {
        zb[2 * t4][tok_lo + (tok_lo >> 4)] = d4[0] * qscale;
        zb[2 * t4 + 1][tok_lo + (tok_lo >> 4)] = d4[1] * qscale;
        zb[2 * t4][tok_hi + (tok_hi >> 4)] = d4[2] * qscale;
        zb[2 * t4 + 1][tok_hi + (tok_hi >> 4)] = d4[3] * qscale;
      }
      __syncthreads();   // the block's scores are parked; nobody reads the stage any more
      issue(dq[NS], pg_next, st, (k + NS) & 3);
      // step 2: mask, store, statistics
      float* zrow = a.ws.z + (size_t)(bh0 + my_head) * a.ws.zstride + chunk * kChunkTokens;
      const unsigned char* mem = s_mem[k & 3];
      float wmax = -INFINITY;      // over this warp's 64-token quarter of the chunk: lets the tau kernel skip it
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = my_tok + 32 * h;
        if (i < ntok) {
          const bool mine = (mem[i >> shift] >> my_head) & 1;
          const float zv = zb[my_head][i + (i >> 4)];
          zrow[i] = mine ? zv : -INFINITY;
          if (mine) {
            wmax = fmaxf(wmax, zv);
            mx = fmaxf(mx, zv);
            if (a.tau_mode != EKV_TAU_EXACT) halley_accumulate(zv, tau0, kind, beta, s0, s1, s2);
          }
        }
      }
      wmax = warp_max_redux(wmax);
      if (lane == 0) a.ws.cmax[((size_t)(bh0 + my_head) * a.ws.nchunks + chunk) * 4 + (warp & 3)] = wmax;
      if (same_run(dk, dn)) {
        group_neutral_store(a, bh0, chunk);
      } else {
        group_run_store(a, red, s0, s1, s2, mx, bh0, chunk);
        s0 = s1 = s2 = 0.f;
        mx = -1.0e6f;
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
