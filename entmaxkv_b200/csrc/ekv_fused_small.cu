// The whole top-k decode step of a SMALL problem in one launch: a few dozen query heads (one long
// request) leave most of the GPU idle in every one of the general path's seven dependent launches,
// and the step's time is their launch and cold-start latency, not its bytes.  Here every query head
// gets a thread-block CLUSTER of four blocks (one block per SM) that runs the step from the page
// statistics to the output row without leaving the chip:
//
//   A  each block sweeps a quarter of the head's k_min / k_max pages through a deep bulk-copy ring
//      and keeps the page scores' order-preserving keys in shared memory (same arithmetic, bit for
//      bit, as the score sweep of the general path); the four blocks then read each other's keys
//      over distributed shared memory, so every block holds all of them;
//   B  every block runs the radix selection and the ordered packing on the full key set - redundantly,
//      which is cheaper than one more exchange - and so knows the head's page table;
//   C  each block gathers a quarter of the selected pages of K (one bulk copy per page, all in flight
//      together) and keeps its tokens' scores in shared memory;
//   D  the exact-mode tau procedure (maximum, 16-bin histogram, bracket, `niter` bracketed Halley steps)
//      with one cluster-wide exchange of a few floats per reduction: every block writes its partial
//      into the others' shared memory, a cluster barrier, and all of them add the four partials in rank
//      order, so all four hold the same tau;
//   E  each block gathers the value rows of its tokens with a non-zero weight, the partial output rows
//      meet in block 0's shared memory and it stores the head's output.
//
// Distributed shared memory is accessed with ordinary loads and stores on mapped addresses; no
// multicast copy of any kind is involved.  The reference has no counterpart (its step is 7 + 2*niter
// Triton launches, entmaxkv/kernels/adadecode_paged.py:567-762 after entmaxkv/attention_topk.py:39-76).
#include <cooperative_groups.h>

#include "ekv_common.cuh"
#include "ekv_score_key.cuh"
#include "ekv_tau_math.cuh"

namespace cg = cooperative_groups;

namespace ekv {

constexpr int kFsThreads = 256;
constexpr int kFsCluster = 4;
constexpr int kFsMaxScored = 8192;   // page keys held in every block's shared memory
constexpr int kFsMaxSelected = 2047; // selected pages per head (without the last page)
constexpr int kFsMaxTokens = 4096;   // kept scores per block
constexpr int kFsTilePages = 64;
constexpr int kFsSlotFloats = 16;    // floats one block contributes to a cluster-wide reduction
constexpr int kFsPhases = 2;         // reduction slots: consecutive reductions alternate between two
constexpr int kFsMaxIter = 64;
constexpr size_t kFsBufBytes = 160 * 1024;   // copy ring of phase A, page buffer of phase C

struct FusedArgs {
  ekv_cache_desc c;
  const void* q;
  int64_t qsb, qsh;
  int q_heads, token_budget, niter, max_scored;
  float alpha;
  void* scores;
  int64_t score_stride;
  int* page_indices;
  int64_t pi_stride;
  int* num_selected;
  int* tok_counts;
  float* tau;
  void* out;
  int64_t osb, osh;
  int* status;
};

struct FusedSmem {
  static constexpr size_t kKeys = kFsBufBytes;                                     // uint32 [kFsMaxScored]
  static constexpr size_t kSel = kKeys + (size_t)kFsMaxScored * 4;                 // int [kFsMaxSelected + 1]
  static constexpr size_t kZ = kSel + (size_t)(kFsMaxSelected + 1) * 4;            // float [kFsMaxTokens]
  static constexpr size_t kSlots = kZ + (size_t)kFsMaxTokens * 4;                  // float [phases][cluster][16]
  static constexpr size_t kParts = kSlots + (size_t)kFsPhases * kFsCluster * kFsSlotFloats * 4;   // float [cluster][128]
  static constexpr size_t kTotal = kParts + (size_t)kFsCluster * 128 * 4;
};

// Three block-wide sums with one barrier pair (warp butterflies, then warps in index order).
__device__ __forceinline__ void block_sum3(float& v0, float& v1, float& v2, float* scratch) {
  constexpr int W = kFsThreads / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v0 = warp_sum(v0);
  v1 = warp_sum(v1);
  v2 = warp_sum(v2);
  __syncthreads();
  if (lane == 0) {
    scratch[warp] = v0;
    scratch[W + warp] = v1;
    scratch[2 * W + warp] = v2;
  }
  __syncthreads();
  float t0 = 0.f, t1 = 0.f, t2 = 0.f;
#pragma unroll
  for (int w = 0; w < W; ++w) {
    t0 += scratch[w];
    t1 += scratch[W + w];
    t2 += scratch[2 * W + w];
  }
  v0 = t0;
  v1 = t1;
  v2 = t2;
}

#ifdef EKV_FUSED_TIMING   // development aid: phase time stamps of the first blocks (never built into the product)
__device__ unsigned long long g_fs_marks[64][8];
__device__ __forceinline__ unsigned long long fs_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define FS_MARK(i) do { if (threadIdx.x == 0 && blockIdx.x < 64) g_fs_marks[blockIdx.x][i] = fs_now(); } while (0)
#else
#define FS_MARK(i) do { } while (0)
#endif

template <typename T, int D>
__global__ void __launch_bounds__(kFsThreads, 1) fused_topk_small_kernel(const FusedArgs a) {
  using SK = ScoreKey<T>;
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kFsThreads / LPR;
  constexpr int C = kFsCluster;
  constexpr int kTileBytes = kFsTilePages * D * (int)sizeof(T);          // one statistic of a tile
  constexpr int NSA = (int)(kFsBufBytes / (2 * kTileBytes)) < 8 ? (int)(kFsBufBytes / (2 * kTileBytes)) : 8;
  static_assert(NSA >= 2, "the copy ring needs two stages");
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* buf = smem;
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem + FusedSmem::kKeys);
  int* sel = reinterpret_cast<int*>(smem + FusedSmem::kSel);
  float* s_z = reinterpret_cast<float*>(smem + FusedSmem::kZ);
  float* slots = reinterpret_cast<float*>(smem + FusedSmem::kSlots);
  float* parts = reinterpret_cast<float*>(smem + FusedSmem::kParts);
  __shared__ uint64_t bar[8];
  __shared__ uint64_t kbar;
  __shared__ int hist[256];
  __shared__ uint32_t scan_scratch[40];
  __shared__ float fscratch[32];
  __shared__ float fscratch3[3 * (kFsThreads / 32)];
  __shared__ uint32_t s_prefix;
  __shared__ int s_krem;

  cg::cluster_group cluster = cg::this_cluster();
  const int r = (int)cluster.block_rank();
  const int bh = blockIdx.x / C;
  const int tid = threadIdx.x, lane = tid & 31;
  const int b = bh / a.q_heads, hq = bh % a.q_heads;
  const int G = a.q_heads / a.c.kv_heads, hkv = hq / G;
  const int S = a.c.seq_lens[b];
  const int P = a.c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n = max(min(min(n_pages - 1, a.c.page_capacity), a.max_scored), 0);
  const int k_sel = min(min(a.token_budget / P, n), kFsMaxSelected);
  const int lane_in_row = tid % LPR, gi = tid / LPR;
  const T* qrow = static_cast<const T*>(a.q) + b * a.qsb + hq * a.qsh;

  FS_MARK(0);
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) mbar_init(&bar[i], 1);
    mbar_init(&kbar, 1);
    mbar_fence_init();
  }
  __syncthreads();

  // ---- A: page scores of this block's quarter of the pages
  {
    const int tiles = (n + kFsTilePages - 1) / kFsTilePages;
    const int per = (tiles + C - 1) / C;
    const int t_begin = r * per;
    const int my_tiles = max(min(tiles, t_begin + per) - t_begin, 0);
    const size_t head_off = b * a.c.meta_stride_b + hkv * a.c.meta_stride_h;
    auto issue = [&](int t) {   // thread 0
      const int page0 = (t_begin + t) * kFsTilePages;
      const int npg = min(kFsTilePages, n - page0);
      const uint32_t bytes = (uint32_t)(npg * D * sizeof(T));
      const int st = t % NSA;
      unsigned char* dst = buf + (size_t)st * 2 * kTileBytes;
      mbar_expect_tx(&bar[st], 2 * bytes);
      bulk_load(dst, static_cast<const T*>(a.c.k_min) + head_off + (size_t)page0 * D, bytes, &bar[st]);
      bulk_load(dst + kTileBytes, static_cast<const T*>(a.c.k_max) + head_off + (size_t)page0 * D, bytes, &bar[st]);
    };
    if (tid == 0)
      for (int t = 0; t < min(NSA, my_tiles); ++t) issue(t);
    float qp[EPL], qn[EPL];
    {
      float qf[EPL];
      unpack<T>(*reinterpret_cast<const uint4*>(qrow + lane_in_row * EPL), qf);
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        qp[j] = fmaxf(qf[j], 0.f);
        qn[j] = fminf(qf[j], 0.f);
      }
    }
    T* out_row = static_cast<T*>(a.scores) + (size_t)bh * a.score_stride;
    for (int t = 0; t < my_tiles; ++t) {
      const int page0 = (t_begin + t) * kFsTilePages;
      const int npg = min(kFsTilePages, n - page0);
      const int st = t % NSA;
      const T* s_lo = reinterpret_cast<const T*>(buf + (size_t)st * 2 * kTileBytes);
      const T* s_hi = reinterpret_cast<const T*>(buf + (size_t)st * 2 * kTileBytes + kTileBytes);
      mbar_wait_or_flag(&bar[st], (uint32_t)(t / NSA) & 1u, a.status);
      for (int pb = 0; pb < npg; pb += GROUPS) {        // uniform trip count: shuffles need whole warps
        const int p = min(pb + gi, npg - 1);
        float lo[EPL], hi[EPL];
        unpack<T>(lds128(s_lo + p * D + lane_in_row * EPL), lo);
        unpack<T>(lds128(s_hi + p * D + lane_in_row * EPL), hi);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {                 // the order of the general sweep: scores are bit-identical
          acc = __fmaf_rn(qp[j], hi[j], acc);
          acc = __fmaf_rn(qn[j], lo[j], acc);
        }
        const float rsum = row_sum<LPR>(acc);
        if (lane_in_row == 0 && pb + gi < npg) {
          const T sc = from_float<T>(rsum);
          out_row[page0 + p] = sc;
          keys[page0 + p] = SK::of_value(sc);
        }
      }
      __syncthreads();   // everyone is done with this stage
      if (tid == 0 && t + NSA < my_tiles) issue(t + NSA);
    }
    FS_MARK(1);
    cluster.sync();      // every block's keys are in its shared memory
    for (int qk = 1; qk < C; ++qk) {
      const int src = (r + qk) % C;
      const int lo_p = min(src * per * kFsTilePages, n), hi_p = min((src + 1) * per * kFsTilePages, n);
      const uint32_t* remote = cluster.map_shared_rank(keys, src);
      for (int i = lo_p + tid; i < hi_p; i += kFsThreads) keys[i] = remote[i];
    }
    __syncthreads();
  }

  FS_MARK(2);
  // ---- B: the k_sel best pages (ties: lower page id), ascending, then the last page - in every block
  const int KPT = (n + kFsThreads - 1) / kFsThreads;      // <= 32 consecutive keys per thread
  uint32_t kth = 0;
  int rq = 0;
  if (k_sel > 0 && k_sel < n) {
    if (tid == 0) {
      s_prefix = 0;
      s_krem = k_sel;
    }
    for (int shift = SK::BITS - 8; shift >= 0; shift -= 8) {
      hist[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const int hi_shift = shift + 8;
      for (int i = tid; i < n; i += kFsThreads) {
        const uint32_t key = keys[i];
        if (hi_shift >= SK::BITS || (key >> hi_shift) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (tid < 32) {
        // lane l owns bins 8l..8l+7; suffix counts from the top bin down
        int cnt[8], lane_total = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          cnt[j] = hist[tid * 8 + j];
          lane_total += cnt[j];
        }
        int tot_above = 0;
        for (int l = 31; l >= 0; --l) {
          const int tl = __shfl_sync(0xffffffffu, lane_total, l);
          if (l > tid) tot_above += tl;
        }
        const int krem = s_krem;
        int run = tot_above, found_bin = -1, found_above = 0;
#pragma unroll
        for (int j = 7; j >= 0; --j) {
          if (found_bin < 0 && run < krem && run + cnt[j] >= krem) {
            found_bin = tid * 8 + j;
            found_above = run;
          }
          run += cnt[j];
        }
        __syncwarp();
        if (found_bin >= 0) {   // exactly one lane finds it
          s_prefix = (prefix << 8) | (uint32_t)found_bin;
          s_krem = krem - found_above;
        }
      }
      __syncthreads();
    }
    kth = s_prefix;
    rq = s_krem;
  }
  if (k_sel > 0) {
    const bool all = k_sel >= n;
    const int i0 = tid * KPT;
    uint32_t gt_bits = 0, eq_bits = 0;
    for (int j = 0; j < KPT; ++j) {
      const int i = i0 + j;
      if (i < n) {
        const uint32_t key = keys[i];
        gt_bits |= (uint32_t)(all || key > kth) << j;
        eq_bits |= (uint32_t)(!all && key == kth) << j;
      }
    }
    uint32_t total;
    const uint32_t ex = block_scan_excl((uint32_t)__popc(gt_bits) | ((uint32_t)__popc(eq_bits) << 16), scan_scratch, &total);
    int gt_before = (int)(ex & 0xffffu), eq_before = (int)(ex >> 16);
    for (int j = 0; j < KPT; ++j) {
      const bool gg = (gt_bits >> j) & 1u, ee = (eq_bits >> j) & 1u;
      if (gg || (ee && eq_before < rq)) sel[gt_before + min(eq_before, rq)] = i0 + j;
      gt_before += gg;
      eq_before += ee;
    }
  }
  if (tid == 0) sel[k_sel] = n_pages - 1;
  __syncthreads();
  const int cnt_sel = k_sel + 1;
  const int last_tokens = S - (n_pages - 1) * P;
  if (r == 0) {
    int* pi = a.page_indices + (size_t)bh * a.pi_stride;
    for (int i = tid; i < cnt_sel; i += kFsThreads) pi[i] = sel[i];
    if (tid == 0) {
      a.num_selected[bh] = cnt_sel;
      a.tok_counts[bh] = k_sel * P + last_tokens;
    }
  }

  FS_MARK(3);
  // ---- C: scores of this block's quarter of the selected tokens
  const int per_pg = (cnt_sel + C - 1) / C;
  const int g0 = min(r * per_pg, cnt_sel), g1 = min(g0 + per_pg, cnt_sel);
  const int my_pages = g1 - g0;
  const int my_tok = min(my_pages * P - ((my_pages > 0 && g1 == cnt_sel) ? P - last_tokens : 0), kFsMaxTokens);
  const int page_bytes = P * D * (int)sizeof(T);
  const int ppr = (int)(kFsBufBytes / page_bytes);          // pages per round of the page buffer
  const float beta = 1.f / (a.alpha - 1.f);
  const int kind = alpha_kind_of(a.alpha);
  auto page_src = [&](const void* base, int g, size_t& off) -> bool {
    const int page = sel[g];
    if ((unsigned)page >= (unsigned)a.c.page_capacity || !kv_page_offset(a.c, b, hkv, page, off)) {
      atomicOr(a.status, EKV_STATUS_PAGE_RANGE);
      kv_page_offset(a.c, b, hkv, 0, off);
      return false;
    }
    return true;
  };
  {
    float qs[EPL];
    unpack<T>(*reinterpret_cast<const uint4*>(qrow + lane_in_row * EPL), qs);
    const float qscale = (a.alpha - 1.f) * (D == 64 ? 0.125f : 0.08838834764831845f);
#pragma unroll
    for (int j = 0; j < EPL; ++j) qs[j] *= qscale;
    uint32_t kphase = 0;
    for (int rd0 = 0; rd0 < my_pages; rd0 += ppr) {
      const int npg = min(ppr, my_pages - rd0);
      const int tok0 = rd0 * P;
      const int ntok = min(npg * P, my_tok - tok0);
      if (tid == 0) mbar_expect_tx(&kbar, (uint32_t)ntok * D * (uint32_t)sizeof(T));
      __syncthreads();
      for (int i = tid; i < npg; i += kFsThreads) {
        const int rows = min(P, ntok - i * P);
        size_t off;
        page_src(a.c.k, g0 + rd0 + i, off);
        if (rows > 0) bulk_load(buf + (size_t)i * page_bytes, static_cast<const T*>(a.c.k) + off, (uint32_t)(rows * D * sizeof(T)), &kbar);
      }
      mbar_wait_or_flag(&kbar, kphase, a.status);
      kphase ^= 1u;
      const T* tile = reinterpret_cast<const T*>(buf);
      for (int i0 = 0; i0 < ntok; i0 += GROUPS) {       // uniform trip count
        const int i = min(i0 + gi, ntok - 1);
        float kf[EPL];
        unpack<T>(lds128(tile + (size_t)i * D + lane_in_row * EPL), kf);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc = fmaf(qs[j], kf[j], acc);
        const float zv = row_sum<LPR>(acc);
        if (lane_in_row == 0 && i0 + gi < ntok) s_z[tok0 + i0 + gi] = zv;
      }
      __syncthreads();   // the page buffer is free for the next round
    }
  }

  FS_MARK(4);
  // ---- D: exact-mode tau, reductions over the cluster
  // reduction `ph`: this block's `nv` floats go to slot [ph % 2][r] of every block; after the barrier all
  // blocks read the four slots (in rank order: every block computes the same numbers).  Two slots are
  // enough: a block writes reduction ph + 2 only after the barrier of ph + 1, which every block reaches
  // after it has read reduction ph.
  auto exchange = [&](int ph, const float (&vals)[kFsSlotFloats], int nv) {
    if (tid < C) {
      float* remote = cluster.map_shared_rank(slots, tid) + ((size_t)(ph & 1) * C + r) * kFsSlotFloats;
      for (int k = 0; k < nv; ++k) remote[k] = vals[k];
    }
    cluster.sync();
  };
  float vals[kFsSlotFloats];
  float m_loc = -1.0e6f;
  for (int i = tid; i < my_tok; i += kFsThreads) m_loc = fmaxf(m_loc, s_z[i]);
  m_loc = block_max(m_loc, fscratch);
  vals[0] = m_loc;
  exchange(0, vals, 1);
  float zmax = slots[0];
#pragma unroll
  for (int qk = 1; qk < C; ++qk) zmax = fmaxf(zmax, slots[(size_t)qk * kFsSlotFloats]);
  if (tid < kBins) hist[tid] = 0;
  __syncthreads();
  {
    const float t0 = zmax - 1.f;
    for (int i = tid; i < my_tok; i += kFsThreads) {
      const int bin = min((int)((s_z[i] - t0) * (float)kBins), kBins - 1);   // conversion truncates toward zero
      if (bin >= 0) atomicAdd(&hist[bin], 1);
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kBins; ++k) vals[k] = (float)hist[k];
  exchange(1, vals, kBins);
  int hist_all[kBins];
#pragma unroll
  for (int k = 0; k < kBins; ++k) {
    float s = 0.f;
#pragma unroll
    for (int qk = 0; qk < C; ++qk) s += slots[((size_t)1 * C + qk) * kFsSlotFloats + k];
    hist_all[k] = (int)s;
  }
  float t_lo, t_hi;
  bracket_from_hist(hist_all, zmax, a.alpha, kind, t_lo, t_hi);     // every thread: the same bracket
  float t = 0.5f * (t_lo + t_hi);
  for (int it = 0; it < a.niter; ++it) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;
    for (int i = tid; i < my_tok; i += kFsThreads) halley_accumulate(s_z[i], t, kind, beta, a0, a1, a2);
    block_sum3(a0, a1, a2, fscratch3);
    vals[0] = a0;
    vals[1] = a1;
    vals[2] = a2;
    exchange(2 + it, vals, 3);
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int qk = 0; qk < C; ++qk) {
      const float* sl = slots + ((size_t)(it & 1) * C + qk) * kFsSlotFloats;
      s0 += sl[0];
      s1 += sl[1];
      s2 += sl[2];
    }
    halley_bracketed(t, t_lo, t_hi, s0, s1, s2, beta);
  }

  FS_MARK(5);
  // ---- E: value rows of the support, partial outputs to block 0
  // ordered compaction of this block's tokens with a non-zero weight (the key array is free by now:
  // every block has passed its copy of the keys before the first exchange above)
  int* s_list = reinterpret_cast<int*>(keys);
  float* s_w = reinterpret_cast<float*>(keys) + kFsMaxTokens;
  {
    const int K = (my_tok + kFsThreads - 1) / kFsThreads;      // <= 16 consecutive tokens per thread
    uint32_t bits = 0;
    for (int j = 0; j < K; ++j) {
      const int i = tid * K + j;
      if (i < my_tok && s_z[i] > t) bits |= 1u << j;
    }
    uint32_t total;
    int pos = (int)block_scan_excl((uint32_t)__popc(bits), scan_scratch, &total);
    for (int j = 0; j < K; ++j)
      if ((bits >> j) & 1u) {
        const int i = tid * K + j;
        s_list[pos] = i;
        s_w[pos] = entmax_weight(s_z[i], t, kind, beta);
        ++pos;
      }
    __syncthreads();
    const int n_act = (int)total;
    float acc[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
    constexpr int UV = 4;                                    // value rows in flight per lane group
    for (int e0 = gi; e0 < n_act; e0 += GROUPS * UV) {
      uint4 raw[UV];
      float pw[UV];
#pragma unroll
      for (int u = 0; u < UV; ++u) {
        const int e = e0 + u * GROUPS;
        pw[u] = 0.f;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (e < n_act) {
          const int i = s_list[e];
          const int pg = i / P, rr = i - pg * P;
          size_t off;
          if (page_src(a.c.v, g0 + pg, off)) {
            raw[u] = ld_stream(static_cast<const T*>(a.c.v) + off + (size_t)rr * D + lane_in_row * EPL);
            pw[u] = s_w[e];
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
    __syncthreads();       // s_z is free: it becomes the lane groups' reduction buffer
    float (*red)[D] = reinterpret_cast<float (*)[D]>(s_z);
    static_assert(GROUPS * D <= kFsMaxTokens, "the reduction buffer fits the score array");
#pragma unroll
    for (int j = 0; j < EPL; ++j) red[gi][lane_in_row * EPL + j] = acc[j];
    __syncthreads();
    if (tid < D) {
      float s = 0.f;
#pragma unroll 4
      for (int g = 0; g < GROUPS; ++g) s += red[g][tid];
      cluster.map_shared_rank(parts, 0)[r * 128 + tid] = s;
    }
  }
  FS_MARK(6);
  cluster.sync();
  FS_MARK(7);
  if (r == 0) {
    if (tid < D) {
      float s = parts[tid];
#pragma unroll
      for (int qk = 1; qk < C; ++qk) s += parts[qk * 128 + tid];
      static_cast<T*>(a.out)[(size_t)b * a.osb + (size_t)hq * a.osh + tid] = from_float<T>(s);
    }
    if (tid == 0) a.tau[bh] = t;
  }
  (void)lane;
}

}  // namespace ekv

static bool fused_small_supported(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget, int32_t max_seq_len,
                                  int32_t niter) {
  using namespace ekv;
  if (!c || check_desc(c) != EKV_OK || q_heads <= 0 || q_heads % c->kv_heads || max_seq_len <= 0) return false;
  if ((long long)c->batch * q_heads * kFsCluster > sm_count()) return false;     // one block per SM, one wave
  const int P = c->page_size;
  const int max_scored = (max_seq_len + P - 1) / P - 1;
  if (max_scored > kFsMaxScored) return false;
  const int esz = c->dtype == EKV_F32 ? 4 : 2;
  const int page_bytes = P * c->head_dim * esz;
  if (page_bytes % 16 || (size_t)page_bytes > kFsBufBytes) return false;
  const int k_max = token_budget / P < max_scored ? token_budget / P : (max_scored > 0 ? max_scored : 0);
  if (k_max > kFsMaxSelected) return false;
  if (((k_max + 1 + kFsCluster - 1) / kFsCluster) * P > kFsMaxTokens) return false;
  if (niter < 0 || niter > kFsMaxIter) return false;
  if (2 * kFsTilePages * c->head_dim * esz * 2 > (int)kFsBufBytes) return false;
  return true;
}

#ifdef EKV_FUSED_TIMING
extern "C" int ekv_fused_timing_read(unsigned long long* host) {
  return (int)cudaMemcpyFromSymbol(host, ekv::g_fs_marks, sizeof(unsigned long long) * 64 * 8);
}
#endif

extern "C" int ekv_topk_decode_fused_supported(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget,
                                               int32_t max_seq_len, int32_t niter) {
  return fused_small_supported(c, q_heads, token_budget, max_seq_len, niter) ? 1 : 0;
}

extern "C" int ekv_topk_decode_fused(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                     int32_t q_heads, int32_t token_budget, int32_t max_seq_len, float alpha,
                                     int32_t niter, void* scores, int64_t score_stride, int32_t* page_indices,
                                     int64_t pi_stride, int32_t* num_selected, int32_t* tok_counts, float* tau,
                                     void* out, int64_t out_stride_b, int64_t out_stride_h, int32_t* status,
                                     void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!q || !scores || !page_indices || !num_selected || !tok_counts || !tau || !out || !status) return EKV_ERR_ARG;
  if (!c->k_min || !c->k_max) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  if (!fused_small_supported(c, q_heads, token_budget, max_seq_len, niter)) return EKV_ERR_ARG;
  const int P = c->page_size;
  const int max_scored = (max_seq_len + P - 1) / P - 1;
  const int k_max = token_budget / P < max_scored ? token_budget / P : (max_scored > 0 ? max_scored : 0);
  if (score_stride < max_scored || pi_stride < k_max + 1) return EKV_ERR_ARG;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((q_stride_b * esz) % 16 || (q_stride_h * esz) % 16 || (reinterpret_cast<uintptr_t>(q) & 15)) return EKV_ERR_ARG;
  FusedArgs a{};
  a.c = *c;
  a.q = q;
  a.qsb = q_stride_b;
  a.qsh = q_stride_h;
  a.q_heads = q_heads;
  a.token_budget = token_budget;
  a.niter = niter;
  a.max_scored = max_scored;
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
  a.status = status;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(c->batch * q_heads * kFsCluster));
  cfg.blockDim = dim3(kFsThreads);
  cfg.dynamicSmemBytes = FusedSmem::kTotal;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kFsCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    auto kernel = fused_topk_small_kernel<T, D>;
    static bool once = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)FusedSmem::kTotal) == cudaSuccess;
    (void)once;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a);
    if (e != cudaSuccess) return (int)e;
  });
  return launch_status();
}

namespace ekv {
unsigned int copy_timeouts_fused_small() { return copy_timeouts_here(); }
}  // namespace ekv
