// Top-k decode step for MANY heads with the latency chains hidden inside the K pass.
//
// The general path runs selection (one block per head, a chain of ~12 barriers), the K pass, the tau kernel
// (another chain per head), the V pass and the output reduction as separate launches; at a thousand heads the
// two chains cost 90 us in which no key or value byte moves.  The K pass itself leaves most issue slots of an SM
// idle: it waits for bulk copies.  This kernel gives every SM one persistent block of two warp groups:
//
//   stream group (warps 0-7):  for the block's current head, gathers the selected pages of K through a ring of
//                              bulk-copy stages, scores them with tensor-core tiles and leaves the scores z in
//                              an L2-resident buffer;
//   helper group (warps 8-15): meanwhile solves tau for the PREVIOUS head from its kept scores (held in
//                              registers), gathers the value rows of its support and stores its output row, then
//                              runs the radix selection of the head two ahead (page scores come from the score
//                              sweep; they are requested before the tau and used after it).
//
// The groups meet at one block barrier per head; inside a group the barriers are named barriers of 256 threads.
// Heads are dealt out round-robin over the blocks (a shared counter would put a round trip on the helper's
// path and, claimed ahead as the pipeline needs, leave blocks without work when heads are few).  The page table of
// the next head is ready before the current head is finished, so the copy ring runs across head boundaries.
// With the helper at ~16 us per head against ~25 us of copies the kernel is bound by the stream group.
// First-time instruction fetches matter here: code that is first executed while every SM streams at full rate
// waits behind the copies (a first tau cost 45 us instead of 8).  Selection and tau are therefore inlined at one
// place each, and both are walked through once in the prologue, before any K page is requested.
// Selection, scores and tau follow the arithmetic of topk_select_kernel / the K pass / solve_head_tau: page tables
// are bit-identical, tau and the output equal to rounding (the block reductions combine in another order).
// The reference has no counterpart (it launches 7 + 2*niter kernels per step, entmaxkv/attention_topk.py:39-76,
// entmaxkv/kernels/adadecode_paged.py:567-762).
#include <type_traits>

#include "ekv_common.cuh"
#include "ekv_score_key.cuh"
#include "ekv_tau_math.cuh"

namespace ekv {

constexpr int kStThreads = 512;
constexpr int kStGroup = 256;             // threads of a warp group
constexpr int kStGroupWarps = kStGroup / 32;
constexpr int kStMaxTokens = 4352;        // kept scores of a head (17 chunks of 256 tokens)
constexpr int kStMaxSel = 1088;           // selected pages of a head without the last page (page size 4)
constexpr int kStRing = 4;                // heads in flight: previous (tau), current (K), next (prefetch), next + 1 (selection)
constexpr int kStList = 1024;             // support entries gathered per round

struct StreamArgs {
  ekv_cache_desc c;
  const void* q;
  int64_t qsb, qsh;
  int q_heads, token_budget, niter, max_scored, k_max;
  float alpha;
  const void* scores;
  int64_t score_stride;
  int* page_indices;
  int64_t pi_stride;
  int* num_selected;
  int* tok_counts;
  float* tau;
  void* out;
  int64_t osb, osh;
  int* support;      // may be null: tokens with a non-zero weight per head
  float* zbuf;       // [blocks][2][kStMaxTokens]: kept scores of a block's current and previous head (L2)
  int table_stride;
  int reg_keys;      // score rows are 64-byte aligned and padded to whole groups of 32: keys may live in registers
  int* status;
};

// ---- warp-group primitives (named barrier ID, 256 threads) ------------------------------------------------

template <int ID>
__device__ __forceinline__ void gsync() {
  asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(kStGroup) : "memory");
}
// sums with a fixed order: butterfly inside a warp, then the group's warps in index order
template <int ID>
__device__ __forceinline__ void gsum3(float& v0, float& v1, float& v2, float* scratch /* 3 * 8 */) {
  const int lane = threadIdx.x & 31, w = (threadIdx.x >> 5) & (kStGroupWarps - 1);
  v0 = warp_sum(v0);
  v1 = warp_sum(v1);
  v2 = warp_sum(v2);
  gsync<ID>();
  if (lane == 0) {
    scratch[w] = v0;
    scratch[kStGroupWarps + w] = v1;
    scratch[2 * kStGroupWarps + w] = v2;
  }
  gsync<ID>();
  float t0 = 0.f, t1 = 0.f, t2 = 0.f;
#pragma unroll
  for (int i = 0; i < kStGroupWarps; ++i) {
    t0 += scratch[i];
    t1 += scratch[kStGroupWarps + i];
    t2 += scratch[2 * kStGroupWarps + i];
  }
  v0 = t0;
  v1 = t1;
  v2 = t2;
}
template <int ID>
__device__ __forceinline__ float gmax(float v, float* scratch /* 8 */) {
  const int lane = threadIdx.x & 31, w = (threadIdx.x >> 5) & (kStGroupWarps - 1);
  v = warp_max(v);
  gsync<ID>();
  if (lane == 0) scratch[w] = v;
  gsync<ID>();
  float t = scratch[0];
#pragma unroll
  for (int i = 1; i < kStGroupWarps; ++i) t = fmaxf(t, scratch[i]);
  return t;
}
// exclusive scan of a packed pair of 16-bit counters over the group's threads; *total: the group's total
template <int ID>
__device__ __forceinline__ uint32_t gscan_excl(uint32_t v, uint32_t* scratch /* 8 */, uint32_t* total) {
  const int lane = threadIdx.x & 31, w = (threadIdx.x >> 5) & (kStGroupWarps - 1);
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  gsync<ID>();
  if (lane == 31) scratch[w] = inc;
  gsync<ID>();
  uint32_t base = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < kStGroupWarps; ++i) {
    const uint32_t s = scratch[i];
    if (i < w) base += s;
    tot += s;
  }
  *total = tot;
  return base + inc - v;
}

// The same reductions with ONE barrier: the caller hands consecutive reductions of a group different buffers
// (two, alternating).  A thread can only write a buffer again after it has passed the barrier of the reduction in
// between, which every thread reaches after it has read the buffer's previous contents.
// (barrier id at run time: the tau code below is run by both groups)
__device__ __forceinline__ void gsync_r(int id) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kStGroup) : "memory");
}
__device__ __forceinline__ float gmax1(int id, float v, float* buf /* 8 */) {
  const int lane = threadIdx.x & 31, w = (threadIdx.x >> 5) & (kStGroupWarps - 1);
  v = warp_max(v);
  if (lane == 0) buf[w] = v;
  gsync_r(id);
  float t = buf[0];
#pragma unroll
  for (int i = 1; i < kStGroupWarps; ++i) t = fmaxf(t, buf[i]);
  return t;
}
__device__ __forceinline__ void gsum3_1(int id, float& v0, float& v1, float& v2, float* buf /* 3 * 8 */) {
  const int lane = threadIdx.x & 31, w = (threadIdx.x >> 5) & (kStGroupWarps - 1);
  v0 = warp_sum(v0);
  v1 = warp_sum(v1);
  v2 = warp_sum(v2);
  if (lane == 0) {
    buf[w] = v0;
    buf[kStGroupWarps + w] = v1;
    buf[2 * kStGroupWarps + w] = v2;
  }
  gsync_r(id);
  float t0 = 0.f, t1 = 0.f, t2 = 0.f;
#pragma unroll
  for (int i = 0; i < kStGroupWarps; ++i) {
    t0 += buf[i];
    t1 += buf[kStGroupWarps + i];
    t2 += buf[2 * kStGroupWarps + i];
  }
  v0 = t0;
  v1 = t1;
  v2 = t2;
}
__device__ __forceinline__ uint32_t gscan_excl1(int id, uint32_t v, uint32_t* buf /* 8 */, uint32_t* total) {
  const int lane = threadIdx.x & 31, w = (threadIdx.x >> 5) & (kStGroupWarps - 1);
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  if (lane == 31) buf[w] = inc;
  gsync_r(id);
  uint32_t base = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < kStGroupWarps; ++i) {
    const uint32_t s = buf[i];
    if (i < w) base += s;
    tot += s;
  }
  *total = tot;
  return base + inc - v;
}

// Per-head descriptors of the ring (shared memory).
struct StreamHead {
  int bh;        // flat query head, -1: none
  int cnt;       // selected pages including the last page
  int T;         // kept tokens
  int last_tokens;
};

struct SelectScratch {
  int whist[kStGroupWarps][256];
  int hist[256];
  uint32_t scan[kStGroupWarps];
  uint32_t prefix;
  int krem;
  // register-key variant: a histogram set per radix pass, both cleared up front, and a result slot per pass
  int whist2[kStGroupWarps][256];
  uint32_t scan2[2][kStGroupWarps];
  uint32_t res_prefix[2];
  int res_krem[2];
};

// Scores of one head fetched ahead of its selection (issued before the previous head's tau, used after it):
// thread t's 32 consecutive scores of the first 8192 pages, the score of page 8192 + t, the row's length.
struct StreamKeys {
  uint4 raw[4];
  uint32_t tail;
  int S;
};
template <typename T>
__device__ __forceinline__ void stream_prefetch_keys(const StreamArgs& a, int bh, StreamKeys& pk) {
  const int gtid = threadIdx.x & (kStGroup - 1);
#pragma unroll
  for (int qd = 0; qd < 4; ++qd) pk.raw[qd] = make_uint4(0u, 0u, 0u, 0u);
  pk.tail = 0u;
  pk.S = 0;
  if (bh < 0) return;
  pk.S = a.c.seq_lens[bh / a.q_heads];
  if (!a.reg_keys) return;
  const T* sc = static_cast<const T*>(a.scores) + (size_t)bh * a.score_stride;
  if (gtid * 32 + 32 <= a.score_stride) {        // rows are padded to whole groups of 32; what lies past the
    const uint4* p = reinterpret_cast<const uint4*>(sc + gtid * 32);     // scored pages is masked by the counts
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) pk.raw[qd] = __ldcg(p + qd);
  }
  if (8192 + gtid < a.score_stride) pk.tail = __ldcg(reinterpret_cast<const unsigned short*>(sc) + 8192 + gtid);
}

// The same selection for 16-bit scores with the keys in registers: thread t holds the 32 consecutive scores
// [32 t, 32 t + 32) and the score of page 8192 + t, fetched ahead of time (stream_prefetch_keys); pages from 8448 on
// are read from memory in every pass.  Both radix passes and the packing run from registers.  In the first pass a
// thread adds the keys that share the top byte of its first key with ONE atomic (the top byte holds the sign and
// seven exponent bits, which most scores of a head share).  Each pass has its own histogram set (both cleared up
// front) and result slot, and the reductions take one barrier each: eight barriers per head.  Same results as
// stream_select_mem, bit for bit; needs 64-byte aligned score rows padded to whole groups of 32.
constexpr int kStRegPages = 8192 + kStGroup;     // pages whose keys live in registers
template <typename T, int ID>
__device__ __forceinline__ void stream_select_regs(const StreamArgs& a, int bh, const StreamKeys& pk,
                                                   int* __restrict__ table, StreamHead* hd, SelectScratch* ss) {
  using SK = ScoreKey<T>;
  static_assert(SK::BITS == 16, "16-bit scores");
  const int gtid = threadIdx.x & (kStGroup - 1), wg = gtid >> 5, lane = gtid & 31;
  const int P = a.c.page_size;
  const int S = pk.S;
  const int n_pages = (S + P - 1) / P;
  const int n = max(min(min(n_pages - 1, a.c.page_capacity), a.max_scored), 0);
  const int k_sel = min(min(a.token_budget / P, n), a.k_max);
  const T* sc = static_cast<const T*>(a.scores) + (size_t)bh * a.score_stride;
  int* out = a.page_indices + (size_t)bh * a.pi_stride;
  const int i0 = gtid * 32;
  const int nv = max(min(min(n, 8192) - i0, 32), 0);
  const bool has_tail = 8192 + gtid < n;
  uint32_t kw[16];        // keys 2j (low half) and 2j + 1 (high half) of this thread, order-preserving
  {
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
      const uint32_t wds[4] = {pk.raw[qd].x, pk.raw[qd].y, pk.raw[qd].z, pk.raw[qd].w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        kw[qd * 4 + e] = SK::of_bits(wds[e] & 0xffffu) | (SK::of_bits(wds[e] >> 16) << 16);
    }
  }
  const uint32_t tkey = SK::of_bits(pk.tail & 0xffffu);
  // the bin holding the krem-th largest key of a histogram set: thread = bin; suffix sums over the bins above
  auto find_bin = [&](int (*wh)[256], int pass, uint32_t prefix, int krem) {
    gsync<ID>();                                   // the pass's atomics are done
    int c = 0;
#pragma unroll
    for (int w = 0; w < kStGroupWarps; ++w) c += wh[w][gtid];
    int suf = c;                                   // inclusive suffix sum over the warp's bins
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_down_sync(0xffffffffu, suf, o);
      if (lane + o < 32) suf += v;
    }
    if (lane == 0) ss->scan2[pass][wg] = (uint32_t)suf;
    gsync<ID>();
    int above = suf - c;
#pragma unroll
    for (int w = 0; w < kStGroupWarps; ++w)
      if (w > wg) above += (int)ss->scan2[pass][w];
    if (above < krem && above + c >= krem) {       // exactly one bin
      ss->res_prefix[pass] = (prefix << 8) | (uint32_t)gtid;
      ss->res_krem[pass] = krem - above;
    }
    gsync<ID>();
  };
  uint32_t kth = 0;
  int r = 0;
  if (k_sel > 0 && k_sel < n) {
    for (int i = gtid; i < kStGroupWarps * 256; i += kStGroup) {
      (&ss->whist[0][0])[i] = 0;
      (&ss->whist2[0][0])[i] = 0;
    }
    gsync<ID>();
    if (nv > 0) {
      const uint32_t d0 = (kw[0] & 0xffffu) >> 8;
      int c0 = 0;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < nv) {
          const uint32_t d = ((kw[j >> 1] >> ((j & 1) * 16)) & 0xffffu) >> 8;
          if (d == d0) ++c0;
          else atomicAdd(&ss->whist[wg][d], 1);
        }
      atomicAdd(&ss->whist[wg][d0], c0);
    }
    if (has_tail) atomicAdd(&ss->whist[wg][tkey >> 8], 1);
    for (int i = kStRegPages + gtid; i < n; i += kStGroup) atomicAdd(&ss->whist[wg][SK::of(sc, i) >> 8], 1);
    find_bin(ss->whist, 0, 0u, k_sel);
    const uint32_t bin1 = ss->res_prefix[0];
    const int krem1 = ss->res_krem[0];
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < nv) {
        const uint32_t key = (kw[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
        if ((key >> 8) == bin1) atomicAdd(&ss->whist2[wg][key & 255u], 1);
      }
    if (has_tail && (tkey >> 8) == bin1) atomicAdd(&ss->whist2[wg][tkey & 255u], 1);
    for (int i = kStRegPages + gtid; i < n; i += kStGroup) {
      const uint32_t key = SK::of(sc, i);
      if ((key >> 8) == bin1) atomicAdd(&ss->whist2[wg][key & 255u], 1);
    }
    find_bin(ss->whist2, 1, bin1, krem1);
    kth = ss->res_prefix[1];
    r = ss->res_krem[1];
  }
  if (k_sel > 0) {
    const bool all = k_sel >= n;
    uint32_t gt_bits = 0, eq_bits = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < nv) {
        const uint32_t key = (kw[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
        gt_bits |= (uint32_t)(all || key > kth) << j;
        eq_bits |= (uint32_t)(!all && key == kth) << j;
      }
    uint32_t total;
    const uint32_t ex = gscan_excl1(ID, (uint32_t)__popc(gt_bits) | ((uint32_t)__popc(eq_bits) << 16), ss->scan2[0], &total);
    int gt_before = (int)(ex & 0xffffu), eq_before = (int)(ex >> 16);
    for (uint32_t left = gt_bits | eq_bits; left; left &= left - 1) {     // the thread's kept or tied pages, ascending
      const int j = __ffs(left) - 1;
      if ((gt_bits >> j) & 1u) {
        const int pos = gt_before + min(eq_before, r);
        table[pos] = i0 + j;
        out[pos] = i0 + j;
        ++gt_before;
      } else {
        if (eq_before < r) {
          const int pos = gt_before + eq_before;
          table[pos] = i0 + j;
          out[pos] = i0 + j;
        }
        ++eq_before;
      }
    }
    int gt_base = (int)(total & 0xffffu), eq_base = (int)(total >> 16);
    if (n > 8192) {                 // pages 8192 + t, one per thread, after all of the first 8192
      const bool g = has_tail && (all || tkey > kth), e = has_tail && !all && tkey == kth;
      uint32_t tot2;
      const uint32_t ex2 = gscan_excl1(ID, (uint32_t)g | ((uint32_t)e << 16), ss->scan2[1], &tot2);
      const int gtb = gt_base + (int)(ex2 & 0xffffu), eqb = eq_base + (int)(ex2 >> 16);
      if (g || (e && eqb < r)) {
        const int pos = gtb + min(eqb, r);
        table[pos] = 8192 + gtid;
        out[pos] = 8192 + gtid;
      }
      gt_base += (int)(tot2 & 0xffffu);
      eq_base += (int)(tot2 >> 16);
    }
    // pages from kStRegPages on, a round of 8192 at a time from memory (as stream_select_mem does)
    for (int f_base = kStRegPages; f_base < n; f_base += 8192) {
      gsync<ID>();
      const int f0 = f_base + gtid * 32;
      uint32_t gb = 0, eb = 0;
#pragma unroll 4
      for (int j = 0; j < 32; ++j) {
        const int i = f0 + j;
        if (i < n) {
          const uint32_t key = SK::of(sc, i);
          gb |= (uint32_t)(all || key > kth) << j;
          eb |= (uint32_t)(!all && key == kth) << j;
        }
      }
      uint32_t tot2;
      const uint32_t ex2 = gscan_excl<ID>((uint32_t)__popc(gb) | ((uint32_t)__popc(eb) << 16), ss->scan, &tot2);
      int gtb = gt_base + (int)(ex2 & 0xffffu), eqb = eq_base + (int)(ex2 >> 16);
#pragma unroll 4
      for (int j = 0; j < 32; ++j) {
        const bool g = (gb >> j) & 1u, e = (eb >> j) & 1u;
        if (g || (e && eqb < r)) {
          const int pos = gtb + min(eqb, r);
          table[pos] = f0 + j;
          out[pos] = f0 + j;
        }
        gtb += g;
        eqb += e;
      }
      gt_base += (int)(tot2 & 0xffffu);
      eq_base += (int)(tot2 >> 16);
    }
  }
  if (gtid == 0) {
    const int last_tokens = S - (n_pages - 1) * P;
    table[k_sel] = n_pages - 1;
    out[k_sel] = n_pages - 1;
    a.num_selected[bh] = k_sel + 1;
    a.tok_counts[bh] = k_sel * P + last_tokens;
    hd->bh = bh;
    hd->cnt = k_sel + 1;
    hd->T = k_sel * P + last_tokens;
    hd->last_tokens = last_tokens;
  }
  gsync<ID>();
}

// Radix selection + ordered packing of one head by one warp group: the arithmetic of topk_select_kernel (8 bits
// at a time, ties to the lower page id, ascending page ids, then the last page).  The table goes to shared
// memory (for the K pass of this block) and to global memory (the caller's page table); `hd` gets the counts.
template <typename T, int ID>
__device__ void stream_select_mem(const StreamArgs& a, int bh, int* __restrict__ table, StreamHead* hd,
                                  SelectScratch* ss) {
  using SK = ScoreKey<T>;
  constexpr int KPT = 32;                       // keys per thread and round: one bit each in a word
  constexpr int ROUND = kStGroup * KPT;         // 8192
  const int gtid = threadIdx.x & (kStGroup - 1), wg = gtid >> 5;
  const int b = bh / a.q_heads;
  const int S = a.c.seq_lens[b];
  const int P = a.c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n = max(min(min(n_pages - 1, a.c.page_capacity), a.max_scored), 0);
  const int k_sel = min(min(a.token_budget / P, n), a.k_max);
  const T* sc = static_cast<const T*>(a.scores) + (size_t)bh * a.score_stride;
  int* out = a.page_indices + (size_t)bh * a.pi_stride;
  const int n_rounds = (n + ROUND - 1) / ROUND;
  uint32_t kth = 0;
  int r = 0;
  if (k_sel > 0 && k_sel < n) {
    if (gtid == 0) {
      ss->prefix = 0;
      ss->krem = k_sel;
    }
    for (int shift = SK::BITS - 8; shift >= 0; shift -= 8) {
      for (int i = gtid; i < kStGroupWarps * 256; i += kStGroup) (&ss->whist[0][0])[i] = 0;
      gsync<ID>();
      const uint32_t prefix = ss->prefix;
      const int hi_shift = shift + 8;
      for (int rd = 0; rd < n_rounds; ++rd) {
        const int i0 = rd * ROUND + gtid * KPT;
#pragma unroll 4
        for (int j = 0; j < KPT; ++j) {
          const int i = i0 + j;
          if (i < n) {
            const uint32_t key = SK::of(sc, i);
            if (hi_shift >= SK::BITS || (key >> hi_shift) == prefix) atomicAdd(&ss->whist[wg][(key >> shift) & 255u], 1);
          }
        }
      }
      gsync<ID>();
      {
        int t = 0;
#pragma unroll
        for (int w = 0; w < kStGroupWarps; ++w) t += ss->whist[w][gtid];
        ss->hist[gtid] = t;
      }
      gsync<ID>();
      if (gtid < 32) {
        int cnt[8], lane_total = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          cnt[j] = ss->hist[gtid * 8 + j];
          lane_total += cnt[j];
        }
        int tot_above = 0;
        for (int l = 31; l >= 0; --l) {
          const int t = __shfl_sync(0xffffffffu, lane_total, l);
          if (l > gtid) tot_above += t;
        }
        const int krem = ss->krem;
        int run = tot_above, found_bin = -1, found_above = 0;
#pragma unroll
        for (int j = 7; j >= 0; --j) {
          if (found_bin < 0 && run < krem && run + cnt[j] >= krem) {
            found_bin = gtid * 8 + j;
            found_above = run;
          }
          run += cnt[j];
        }
        __syncwarp();
        if (found_bin >= 0) {
          ss->prefix = (prefix << 8) | (uint32_t)found_bin;
          ss->krem = krem - found_above;
        }
      }
      gsync<ID>();
    }
    kth = ss->prefix;
    r = ss->krem;
  }
  if (k_sel > 0) {
    const bool all = k_sel >= n;
    int gt_base = 0, eq_base = 0;
    for (int rd = 0; rd < n_rounds; ++rd) {
      const int i0 = rd * ROUND + gtid * KPT;
      uint32_t gt_bits = 0, eq_bits = 0;
#pragma unroll 4
      for (int j = 0; j < KPT; ++j) {
        const int i = i0 + j;
        if (i < n) {
          if (all) {
            gt_bits |= 1u << j;
          } else {
            const uint32_t key = SK::of(sc, i);
            gt_bits |= (uint32_t)(key > kth) << j;
            eq_bits |= (uint32_t)(key == kth) << j;
          }
        }
      }
      uint32_t total;
      const uint32_t ex = gscan_excl<ID>((uint32_t)__popc(gt_bits) | ((uint32_t)__popc(eq_bits) << 16), ss->scan, &total);
      int gt_before = gt_base + (int)(ex & 0xffffu);
      int eq_before = eq_base + (int)(ex >> 16);
#pragma unroll 4
      for (int j = 0; j < KPT; ++j) {
        const bool g = (gt_bits >> j) & 1u, e = (eq_bits >> j) & 1u;
        if (g || (e && eq_before < r)) {
          const int pos = gt_before + min(eq_before, r);
          table[pos] = i0 + j;
          out[pos] = i0 + j;
        }
        gt_before += g;
        eq_before += e;
      }
      gt_base += (int)(total & 0xffffu);
      eq_base += (int)(total >> 16);
      gsync<ID>();
    }
  }
  if (gtid == 0) {
    const int last_tokens = S - (n_pages - 1) * P;
    table[k_sel] = n_pages - 1;
    out[k_sel] = n_pages - 1;
    a.num_selected[bh] = k_sel + 1;
    a.tok_counts[bh] = k_sel * P + last_tokens;
    hd->bh = bh;
    hd->cnt = k_sel + 1;
    hd->T = k_sel * P + last_tokens;
    hd->last_tokens = last_tokens;
  }
  gsync<ID>();
}

template <typename T, int ID>
__device__ __forceinline__ void stream_select(const StreamArgs& a, int bh, const StreamKeys& pk, int* __restrict__ table,
                                              StreamHead* hd, SelectScratch* ss) {
  if constexpr (ScoreKey<T>::BITS == 16) {
    if (a.reg_keys) {
      stream_select_regs<T, ID>(a, bh, pk, table, hd, ss);
      return;
    }
  }
  stream_select_mem<T, ID>(a, bh, table, hd, ss);
}

// Halley sums / entmax weights over a thread's scores with the kind of alpha fixed at compile time: the unrolled
// bodies hold one variant each, so the code that runs is straight-line (and short to fetch the first time).
template <int KIND, int N>
__device__ __forceinline__ void halley_sums(const float (&z)[N], float t, float beta, float& s0, float& s1, float& s2) {
#pragma unroll
  for (int k = 0; k < N; ++k) halley_accumulate(z[k], t, KIND, beta, s0, s1, s2);
}
template <int KIND, int N>
__device__ __forceinline__ void support_lists(const float (&z)[N], uint32_t bits, int pos, float t, float beta,
                                              int* list_idx, float* list_w, int gtid) {
#pragma unroll
  for (int k = 0; k < N; ++k)
    if ((bits >> k) & 1u) {
      if (pos >= 0 && pos < kStList) {
        list_idx[pos] = gtid + k * kStGroup;
        list_w[pos] = entmax_weight(z[k], t, KIND, beta);
      }
      ++pos;
    }
}

struct TauScratch {
  float red[2][3 * kStGroupWarps];   // consecutive reductions alternate between the two
  int hist[kBins];
  uint32_t scan[kStGroupWarps];
  int list_idx[kStList];
  float list_w[kStList];
  float vred[kStGroup * 8];          // [lane groups][D]: 256 / (D / 8) groups of D floats
};

// Exact-mode tau of one head from its kept scores (maximum, 16-bin histogram, bracket, `niter` bracketed Halley
// steps: adadecode.py:12-112,381-426), then the value rows of its support and the output row.  One warp group;
// a thread keeps its 17 scores (tokens t, t + 256, ...) in registers from the one read of the score buffer on, and
// every thread ends up with the same tau.  The support (a handful of tokens for the usual head) is compacted
// once and gathered in rounds of kStList.  Eight barriers per head for niter = 2.
// `dry`: run the same instructions on a made-up head of one token (score 0, value row of page 0) and store
// nothing.  The kernel does that once before the first K page is requested: a first pass through this code
// while every SM streams at full rate costs ~30 us in instruction fetches that queue behind the copies.
template <typename T, int D>
__device__ __forceinline__ void stream_tau_out(const StreamArgs& a, const StreamHead& hd, const float* __restrict__ zp,
                                               const int* __restrict__ table, TauScratch* ts, const int ID,
                                               const bool dry) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kStGroup / LPR;
  constexpr int ZR = kStMaxTokens / kStGroup;
  const int gtid = threadIdx.x & (kStGroup - 1);
  const int lane_in_row = gtid % LPR, gi = gtid / LPR;
  const int bh = dry ? 0 : hd.bh, T_tok = dry ? 0 : hd.T;
  const int b = bh / a.q_heads, hq = bh % a.q_heads;
  const int hkv = hq / (a.q_heads / a.c.kv_heads);
  const int P = a.c.page_size;
  const int kind = alpha_kind_of(a.alpha);
  const float beta = 1.f / (a.alpha - 1.f);

  float z[ZR];
#pragma unroll
  for (int k = 0; k < ZR; ++k) {
    const int i = gtid + k * kStGroup;
    z[k] = i < T_tok ? __ldcg(zp + i) : -INFINITY;       // -inf: below every threshold, in no bin
  }
  if (dry && gtid == 0) z[0] = 0.f;
  if (gtid < kBins) ts->hist[gtid] = 0;
  float m = -1.0e6f;
#pragma unroll
  for (int k = 0; k < ZR; ++k) m = fmaxf(m, z[k]);
  m = gmax1(ID, m, ts->red[0]);
  {
    const float t0 = m - 1.f;
#pragma unroll
    for (int k = 0; k < ZR; ++k) {
      const int bin = min((int)((z[k] - t0) * (float)kBins), kBins - 1);   // conversion truncates toward zero
      if (bin >= 0) atomicAdd(&ts->hist[bin], 1);
    }
  }
  gsync_r(ID);
  int hist_all[kBins];
#pragma unroll
  for (int k = 0; k < kBins; ++k) hist_all[k] = ts->hist[k];
  float t_lo, t_hi;
  bracket_from_hist(hist_all, m, a.alpha, kind, t_lo, t_hi);
  float t = 0.5f * (t_lo + t_hi);
  for (int it = 0; it < a.niter; ++it) {
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
    if (kind == 1) halley_sums<1>(z, t, beta, s0, s1, s2);
    else if (kind == 0) halley_sums<0>(z, t, beta, s0, s1, s2);
    else halley_sums<2>(z, t, beta, s0, s1, s2);
    gsum3_1(ID, s0, s1, s2, ts->red[(it + 1) & 1]);
    halley_bracketed(t, t_lo, t_hi, s0, s1, s2, beta);
  }

  // value rows of the support
  float acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
  uint32_t bits = 0;
#pragma unroll
  for (int k = 0; k < ZR; ++k)
    if (z[k] > t) bits |= 1u << k;
  uint32_t total;
  const int pos0 = (int)gscan_excl1(ID, (uint32_t)__popc(bits), ts->scan, &total);
  const int support = (int)total;
  for (int base = 0; base < support; base += kStList) {
    if (base > 0) gsync_r(ID);       // the previous round's lists have been read
    if (bits) {        // (most threads hold no token of the support)
      if (kind == 1) support_lists<1>(z, bits, pos0 - base, t, beta, ts->list_idx, ts->list_w, gtid);
      else if (kind == 0) support_lists<0>(z, bits, pos0 - base, t, beta, ts->list_idx, ts->list_w, gtid);
      else support_lists<2>(z, bits, pos0 - base, t, beta, ts->list_idx, ts->list_w, gtid);
    }
    gsync_r(ID);
    const int n_act = min(support - base, kStList);
    constexpr int UV = 4;
    for (int e0 = gi; e0 < n_act; e0 += GROUPS * UV) {
      uint4 raw[UV];
      float pw[UV];
#pragma unroll
      for (int u = 0; u < UV; ++u) {
        const int e = e0 + u * GROUPS;
        pw[u] = 0.f;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (e < n_act) {
          const int i = ts->list_idx[e];
          const int pg = i / P, rr = i - pg * P;
          const int page = dry ? 0 : table[pg];
          size_t off;
          if ((unsigned)page < (unsigned)a.c.page_capacity && kv_page_offset(a.c, b, hkv, page, off)) {
            raw[u] = ld_stream(static_cast<const T*>(a.c.v) + off + (size_t)rr * D + lane_in_row * EPL);
            pw[u] = ts->list_w[e];
          } else if (!dry) {
            atomicOr(a.status, EKV_STATUS_PAGE_RANGE);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UV; ++u) {
        float vf[EPL];
        unpack<T>(raw[u], vf);
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc[j] = fmaf(pw[u], vf[j], acc[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < EPL; ++j) ts->vred[gi * D + lane_in_row * EPL + j] = acc[j];
  gsync_r(ID);
  if (gtid < D && !dry) {
    float sum = 0.f;
#pragma unroll 4
    for (int g = 0; g < GROUPS; ++g) sum += ts->vred[g * D + gtid];
    static_cast<T*>(a.out)[(size_t)b * a.osb + (size_t)hq * a.osh + gtid] = from_float<T>(sum);
  }
  if (gtid == 0 && !dry) {
    a.tau[bh] = t;
    if (a.support) a.support[bh] = support;
  }
  gsync_r(ID);      // the scratch is free for the selection that follows
}

// Tensor-core pieces of the stream group (as in the group-shared K pass): a score block is 16 K rows by the query
// (column 0 of the B fragment; the other seven columns are zero), contracted 16 elements at a time.
__device__ __forceinline__ void st_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void st_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
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

// A stage holds one chunk: 16 page slots of 16 rows of 256 bytes.  Slots are skewed by 16 bytes modulo 128, so
// the same in-page row of eight consecutive slots falls into eight different bank groups and an 8x8 fragment
// whose rows come from eight slots loads without bank conflicts (rows of one page are 256 bytes apart and would
// all collide); every eight slots the skew starts over, 128 bytes further.
constexpr int kStChunk = 256;                                    // tokens of a chunk
constexpr int kStPage = 16;                                      // rows of a page
constexpr int kStPageBytes = kStPage * 128 * 2;
constexpr int kStStageBytes = kStChunk * 128 * 2 + 128 * 2 + 768;  // 16 slots + skew, rounded to 1 KiB
constexpr int kStStages = 3;
__device__ __forceinline__ uint32_t st_slot_offset(int slot) {
  return (uint32_t)(slot * kStPageBytes + (slot & 7) * 16 + (slot >> 3) * 128);
}

union StreamScratch {      // the helper group selects and solves tau one after the other
  SelectScratch sel;
  TauScratch tau;
};

// dynamic shared memory: [3 stages] [4 page tables of table_stride ints] [StreamScratch]
inline size_t stream_smem_bytes(int table_stride) {
  return (size_t)kStStages * kStStageBytes + ((size_t)kStRing * table_stride * 4 + 15) / 16 * 16 +
         (sizeof(StreamScratch) + 15) / 16 * 16;
}

#ifdef EKV_STREAM_TIMING   // development aid: per-block phase times (never built into the product)
__device__ unsigned long long g_st_marks[160][8];
__device__ unsigned long long g_st_line[64];   // block 0: [it][0..2] stream thread, [it][3..5] helper thread
__device__ __forceinline__ unsigned long long st_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
  return t;
}
#define ST_T(var) const unsigned long long var = st_now()
#define ST_ADD(acc, from) acc += st_now() - (from)
#else
#define ST_T(var)
#define ST_ADD(acc, from)
#endif

// 16-bit caches, head_dim 128, page size 16.
template <typename T>
__global__ void __launch_bounds__(kStThreads, 1) topk_decode_stream_kernel(const StreamArgs a) {
  constexpr int D = 128;
  constexpr int NS = kStStages;
  constexpr int CT = kStChunk;
  static_assert(sizeof(T) == 2, "16-bit caches");
  const int TS = a.table_stride;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* after = smem + (size_t)NS * kStStageBytes;
  int* tables = reinterpret_cast<int*>(after);
  after += ((size_t)kStRing * TS * 4 + 15) / 16 * 16;
  StreamScratch* scratch = reinterpret_cast<StreamScratch*>(after);
  float* z_all = a.zbuf + (size_t)blockIdx.x * 2 * kStMaxTokens;   // written by the stream group (L2)
  __shared__ uint64_t full[NS];
  __shared__ StreamHead heads[kStRing];
  // query rows of the current and the next head (head_dim 128, 16-bit): the helper group fetches the next head's
  // row with asynchronous 16-byte copies during its own iteration, so that the stream group's first tile of a
  // head does not wait for a global load (its row was last touched by the score sweep, a gigabyte ago)
  __shared__ __align__(16) unsigned char s_q[2][D * 2];

  const int tid = threadIdx.x, gtid = tid & (kStGroup - 1), lane = tid & 31;
  const bool helper = tid >= kStGroup;
  const int n_heads = a.c.batch * a.q_heads;
  const int G = a.q_heads / a.c.kv_heads;

#ifdef EKV_STREAM_TIMING
  unsigned long long tm_stream = 0, tm_tau = 0, tm_sel = 0, tm_heads = 0, tm_wait = 0, tm_sync = 0;
  if (tid == 0) g_st_marks[blockIdx.x][0] = st_now();
#endif
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < NS; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
#pragma unroll
    for (int i = 0; i < kStRing; ++i) heads[i].bh = -1;
  }
  __syncthreads();
  // heads are dealt out round-robin: block i takes heads i, i + grid, i + 2 grid, ... (neighbouring heads - the
  // query heads of one KV head, which share some of their pages - are in flight on different SMs at the same time)
  auto head_of = [&](int j) -> int {
    const long long h = (long long)blockIdx.x + (long long)j * gridDim.x;
    return h < n_heads ? (int)h : -1;
  };
#ifdef EKV_STREAM_TIMING
  unsigned long long tm_pro = 0;
#endif
  // stream group: the issue cursor (head iteration, chunk) runs up to NS chunks ahead of the chunk being scored
  int iss_it = 0, iss_chunk = 0, iss_seq = 0, cmp_seq = 0;
  // fragment geometry of a stream warp w (0..7): it scores the in-page rows w and w + 8 of the chunk's 16 page
  // slots; ldmatrix row i of a tile = slot i
  const int w = (tid >> 5) & (kStGroupWarps - 1);
  const int frag_i = (lane & 7) + 8 * ((lane >> 3) & 1);
  const uint32_t frag_off = st_slot_offset(frag_i) + (uint32_t)(lane >> 4) * 16;
  const int g = lane >> 2, t4 = lane & 3;

  // Iteration -1 is the prologue (the first head is selected while the stream group walks through the tau code
  // once, see stream_tau_out); iteration it >= 0: K pass of head it | tau of head it - 1, selection of head it + 2
  // (iteration 0: of heads 1 and 2).  Selection and tau are inlined at ONE place each, so their instructions
  // are fetched once, before the copies saturate the memory system.
#pragma unroll 1
  for (int it = -1;; ++it) {
    const StreamHead cur = heads[it & (kStRing - 1)];
    const bool cur_valid = it >= 0 && cur.bh >= 0;
    const bool prev_valid = it > 0 && heads[(it - 1) & (kStRing - 1)].bh >= 0;
    if (it >= 0 && !cur_valid && !prev_valid) break;
    int h_sel = -1;
    StreamKeys pk;
    if (helper && gtid < D * 2 / 16) {
      const int hn = head_of(it + 1);
      if (hn >= 0) {
        const T* qn = static_cast<const T*>(a.q) + (hn / a.q_heads) * a.qsb + (hn % a.q_heads) * a.qsh + gtid * 8;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s_q[(it + 1) & 1][gtid * 16])), "l"(qn)
                     : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (helper && it > 0) {
      // page scores and row length of the head selected in this iteration are requested now and used after the
      // tau of the previous head
      h_sel = head_of(it + 2);
      stream_prefetch_keys<T>(a, h_sel, pk);
    }
    ST_T(t_b);
    if (helper ? prev_valid : it < 0) {
      const int ps = (it - 1) & (kStRing - 1);
      const StreamHead hp = heads[ps];
      stream_tau_out<T, D>(a, hp, z_all + (size_t)((it - 1) & 1) * kStMaxTokens, tables + ps * TS,
                           helper ? &scratch->tau : reinterpret_cast<TauScratch*>(smem), helper ? 2 : 1, !helper);
    }
    if (helper) ST_ADD(tm_tau, t_b);
    if (!helper) {
      if (cur_valid) {
        ST_T(t_a);
        // B fragments: the query in column 0 (lanes g == 0), zero elsewhere
        uint32_t bq[8][2];
        {
          const T* qrow = reinterpret_cast<const T*>(s_q[it & 1]);      // put there by the helper group an iteration ago
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t4);
            bq[ks][0] = g == 0 ? w0 : 0u;
            bq[ks][1] = g == 0 ? w1 : 0u;
          }
        }
        const float qscale = (a.alpha - 1.f) * 0.08838834764831845f;
        float* zb = z_all + (size_t)(it & 1) * kStMaxTokens;
        const bool next_ready = it >= 1 && heads[(it + 1) & (kStRing - 1)].bh >= 0;   // selected an iteration ago
        auto issue_next = [&]() {
          const int slot_h = iss_it & (kStRing - 1);
          const StreamHead h = heads[slot_h];
          const int* tab = tables + slot_h * TS;
          const int tok0 = iss_chunk * CT;
          const int ntok = min(CT, h.T - tok0);
          const int st = iss_seq % NS;
          if (gtid < 32) {
            const int hb = h.bh / a.q_heads, hkv = (h.bh % a.q_heads) / G;
            if (gtid == 0) mbar_expect_tx(&full[st], (uint32_t)(ntok * D * 2));
            __syncwarp();
            if (gtid < 16 && gtid * kStPage < ntok) {
              const int rows = min(kStPage, ntok - gtid * kStPage);
              const int page = tab[(tok0 >> 4) + gtid];
              size_t off;
              if ((unsigned)page >= (unsigned)a.c.page_capacity || !kv_page_offset(a.c, hb, hkv, page, off)) {
                atomicOr(a.status, EKV_STATUS_PAGE_RANGE);
                kv_page_offset(a.c, hb, hkv, 0, off);      // keep the byte count; the status bit marks the result invalid
              }
              bulk_load(smem + (size_t)st * kStStageBytes + st_slot_offset(gtid), static_cast<const T*>(a.c.k) + off,
                        (uint32_t)(rows * D * 2), &full[st]);
            }
          }
          ++iss_seq;
          if (++iss_chunk == (h.T + CT - 1) / CT) {
            ++iss_it;
            iss_chunk = 0;
          }
        };
        auto top_up = [&]() {
          while (iss_seq < cmp_seq + NS && (iss_it == it || (iss_it == it + 1 && next_ready))) issue_next();
        };
        top_up();
        const int nch = (cur.T + CT - 1) / CT;
        for (int c = 0; c < nch; ++c) {
          const int st = cmp_seq % NS;
          const int ntok = min(CT, cur.T - c * CT);
          ST_T(t_w);
          mbar_wait_or_flag(&full[st], (uint32_t)(cmp_seq / NS) & 1u, a.status);
          ST_ADD(tm_wait, t_w);
          const uint32_t a_base = smem_addr(smem + (size_t)st * kStStageBytes) + frag_off;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int row = w + 8 * half;                   // in-page row of this warp's tile
            float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              uint32_t af[4];
              st_ldmatrix_x4(a_base + (uint32_t)row * (D * 2) + ks * 32, af);
              st_mma<T>(d4, af, bq[ks][0], bq[ks][1]);
            }
            if (t4 == 0) {                                  // column 0: rows g (slot g) and g + 8 (slot g + 8)
              const int tok_lo = g * kStPage + row, tok_hi = (g + 8) * kStPage + row;
              if (tok_lo < ntok) zb[c * CT + tok_lo] = d4[0] * qscale;
              if (tok_hi < ntok) zb[c * CT + tok_hi] = d4[2] * qscale;
            }
          }
          ++cmp_seq;
          gsync<1>();      // the stage is free
          top_up();
        }
        ST_ADD(tm_stream, t_a);
#ifdef EKV_STREAM_TIMING
        ++tm_heads;
#endif
      }
    } else {
      ST_T(t_c);
      const int n_sel = it == 0 ? 2 : 1;
#pragma unroll 1
      for (int rsel = 0; rsel < n_sel; ++rsel) {
        int slot_h = (it + 2) & (kStRing - 1);
        if (it <= 0) {
          slot_h = it < 0 ? 0 : rsel + 1;
          h_sel = head_of(slot_h);
          stream_prefetch_keys<T>(a, h_sel, pk);
        }
        if (h_sel >= 0) {
          stream_select<T, 2>(a, h_sel, pk, tables + slot_h * TS, &heads[slot_h], &scratch->sel);
        } else if (gtid == 0) {
          heads[slot_h].bh = -1;
        }
      }
      ST_ADD(tm_sel, t_c);
    }
    if (helper && gtid < D * 2 / 16) asm volatile("cp.async.wait_group 0;" ::: "memory");   // the next head's query row has landed
#ifdef EKV_STREAM_TIMING
    const unsigned long long t_s = st_now();
    asm volatile("bar.sync 0;" ::: "memory");
    tm_sync += st_now() - t_s;
    if (it < 0 && tid == 0) tm_pro = st_now();
    if (blockIdx.x == 0 && it < 9 && (tid == 0 || tid == kStGroup)) {
      const int o = (it < 0 ? 9 : it) * 6 + (tid == 0 ? 0 : 3);
      g_st_line[o] = t_s - g_st_marks[0][0];
      g_st_line[o + 1] = st_now() - g_st_marks[0][0];
    }
#else
    __syncthreads();
#endif
  }
#ifdef EKV_STREAM_TIMING
  if (tid == 0) {
    g_st_marks[blockIdx.x][1] = st_now();
    g_st_marks[blockIdx.x][2] = tm_stream;
    g_st_marks[blockIdx.x][5] = tm_heads;
    g_st_marks[blockIdx.x][7] = tm_wait;
  }
  if (tid == kStGroup) {
    g_st_marks[blockIdx.x][3] = tm_tau;
    g_st_marks[blockIdx.x][4] = tm_sel;
  }
  if (tid == 0) g_st_marks[blockIdx.x][6] = ((tm_pro - g_st_marks[blockIdx.x][0]) & 0xffffffffull) | (tm_sync << 32);
#endif
}

}  // namespace ekv

static bool stream_topk_fits(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget, int32_t max_seq_len,
                             int32_t niter) {
  using namespace ekv;
  if (!c || check_desc(c) != EKV_OK || q_heads <= 0 || q_heads % c->kv_heads || max_seq_len <= 0) return false;
  const int P = c->page_size;
  if (P != kStPage || c->head_dim != 128 || c->dtype == EKV_F32) return false;     // the stream group's tensor-core tiles
  const int max_scored = (max_seq_len + P - 1) / P - 1;
  const int k_max = token_budget / P < max_scored ? token_budget / P : (max_scored > 0 ? max_scored : 0);
  if (k_max > kStMaxSel || (k_max + 1) * P > kStMaxTokens) return false;
  if (stream_smem_bytes((k_max + 1 + 3) / 4 * 4) > 227 * 1024 - 1024) return false;
  return niter >= 0 && niter <= 64;
}

extern "C" int ekv_topk_decode_stream_supported(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget,
                                                int32_t max_seq_len, int32_t niter) {
  if (!stream_topk_fits(c, q_heads, token_budget, max_seq_len, niter)) return 0;
  // One head per block already beats the separate kernels (81 against 85 us at 64 heads of 128k tokens, 94
  // against 107 us at 128); with fewer heads than a third of the SMs the general K pass, which splits a head's
  // pages over several SMs, is as fast or faster.
  return 3LL * c->batch * q_heads >= ekv::sm_count() ? 1 : 2;
}

extern "C" size_t ekv_topk_decode_stream_scratch_bytes(void) {
  return (size_t)ekv::sm_count() * 2 * ekv::kStMaxTokens * sizeof(float);
}

extern "C" int ekv_topk_decode_stream(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                      int32_t q_heads, int32_t token_budget, int32_t max_seq_len, float alpha,
                                      int32_t niter, const void* scores, int64_t score_stride,
                                      int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                                      int32_t* tok_counts, float* tau, void* out, int64_t out_stride_b,
                                      int64_t out_stride_h, int32_t* support, float* zbuf,
                                      size_t zbuf_bytes, int32_t* status, void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!q || !scores || !page_indices || !num_selected || !tok_counts || !tau || !out || !status || !zbuf)
    return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  if (!stream_topk_fits(c, q_heads, token_budget, max_seq_len, niter)) return EKV_ERR_ARG;
  const int P = c->page_size;
  const int max_scored = (max_seq_len + P - 1) / P - 1;
  const int k_max = token_budget / P < max_scored ? token_budget / P : (max_scored > 0 ? max_scored : 0);
  if (score_stride < max_scored || pi_stride < k_max + 1) return EKV_ERR_ARG;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((q_stride_b * esz) % 16 || (q_stride_h * esz) % 16 || (reinterpret_cast<uintptr_t>(q) & 15)) return EKV_ERR_ARG;
  StreamArgs a{};
  a.c = *c;
  a.q = q;
  a.qsb = q_stride_b;
  a.qsh = q_stride_h;
  a.q_heads = q_heads;
  a.token_budget = token_budget;
  a.niter = niter;
  a.max_scored = max_scored;
  a.k_max = k_max;
  a.alpha = alpha;
  a.scores = scores;
  a.score_stride = score_stride;
  a.page_indices = page_indices;
  a.pi_stride = pi_stride;
  a.num_selected = num_selected;
  a.tok_counts = tok_counts;
  a.tau = tau;
  a.out = out;
  a.osb = out_stride_b;
  a.osh = out_stride_h;
  a.support = support;
  a.status = status;
  const long long n_heads = (long long)c->batch * q_heads;
  const int blocks = (int)(n_heads < sm_count() ? n_heads : sm_count());
  if (zbuf_bytes < (size_t)blocks * 2 * kStMaxTokens * sizeof(float)) return EKV_ERR_ARG;
  a.zbuf = zbuf;
  a.table_stride = (k_max + 1 + 3) / 4 * 4;
  a.reg_keys = (score_stride % 32 == 0) && (reinterpret_cast<uintptr_t>(scores) % 64 == 0) && c->dtype != EKV_F32;
  constexpr size_t kSmemLimit = 227 * 1024 - 1024;       // dynamic shared memory of a block, less the static part
  const size_t smem = stream_smem_bytes(a.table_stride);
  if (smem > kSmemLimit) return EKV_ERR_ARG;
  if (c->dtype == EKV_BF16) {
    static bool once = cudaFuncSetAttribute(topk_decode_stream_kernel<__nv_bfloat16>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit) == cudaSuccess;
    (void)once;
    topk_decode_stream_kernel<__nv_bfloat16><<<blocks, kStThreads, smem, as_stream(stream)>>>(a);
  } else {
    static bool once = cudaFuncSetAttribute(topk_decode_stream_kernel<__half>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit) == cudaSuccess;
    (void)once;
    topk_decode_stream_kernel<__half><<<blocks, kStThreads, smem, as_stream(stream)>>>(a);
  }
  return launch_status();
}

#ifdef EKV_STREAM_TIMING
extern "C" int ekv_stream_timing_read(unsigned long long* host) {
  return cudaMemcpyFromSymbol(host, ekv::g_st_marks, sizeof(ekv::g_st_marks)) == cudaSuccess ? 0 : -1;
}
extern "C" int ekv_stream_timing_line(unsigned long long* host) {
  return cudaMemcpyFromSymbol(host, ekv::g_st_line, sizeof(ekv::g_st_line)) == cudaSuccess ? 0 : -1;
}
#endif

namespace ekv {
unsigned int copy_timeouts_stream_topk() { return copy_timeouts_here(); }
}  // namespace ekv
