// Top-k page selection: key-range upper-bound scores swept from the page
// min/max statistics, then an exact radix selection with a deterministic tie
// rule (equal scores: lower page id wins) and ordered index packing.
//
// HBM-bound: the sweep reads k_min and k_max of every scored page once
// (2*D*sizeof(T) bytes per page and KV head, shared by the query heads of a GQA
// group); everything after it works on 2 or 4 bytes per page and query head.
#include <algorithm>

#include "ekv_common.cuh"
#include "ekv_work.cuh"

namespace ekv {

constexpr int kScorePagesPerBlock = 64;    // pages per tile
constexpr int kScoreTilesPerBlock = 4;   // tiles per chunk of a persistent block (fewer on small sweeps)
constexpr int kScoreThreads = 256;
constexpr int kSelectThreads = 512;

// score = sum_d max(q_d*lo_d, q_d*hi_d) = sum_d (max(q_d,0)*hi_d + min(q_d,0)*lo_d):
// one of the two products is an exact zero, so the two-FMA form rounds exactly
// like the select-then-multiply form.
//
// grid: persistent, three 256-thread blocks per SM (fewer when there is less work).  A block owns
// chunks of consecutive 64-page tiles of one KV head (TileWalk).  The k_min rows and the k_max rows of
// a tile are two contiguous 64*D*sizeof(T)-byte blocks, fetched with two bulk asynchronous copies
// into one of two shared-memory stages while the previous tile is being scored (these copies are the
// only global reads of the kernel besides q).  A page is scored by ceil(G/HPL) groups of LPR lanes,
// each group owning HPL query heads of the GQA group.
template <typename T, int D, int HPL, bool ALIBI>
__global__ void __launch_bounds__(kScoreThreads, 3)
page_score_kernel(ekv_cache_desc c, const T* __restrict__ q, int64_t qsb, int64_t qsh, int q_heads,
                  T* __restrict__ scores, int64_t score_stride, const float* __restrict__ alibi_slopes,
                  const int* __restrict__ q_positions, int tpc, int chunks_per_head, int n_chunks) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kScoreThreads / LPR;
  constexpr int kTileElems = kScorePagesPerBlock * D;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* s_tiles = reinterpret_cast<T*>(smem_raw);   // [stage][lo|hi][64*D]
  __shared__ uint64_t bar[2];

  const int G = q_heads / c.kv_heads;
  const int P = c.page_size;
  const int tid = threadIdx.x;
  auto n_scored_of = [&](int b) {
    const int S = c.seq_lens[b];
    return min((S + P - 1) / P - 1, c.page_capacity);
  };

  // thread 0 runs the copies two tiles ahead of the block; its walker lives in shared memory so that it
  // costs the other threads no registers
  __shared__ TileWalk wi;
  __shared__ int issued;
  auto issue_next = [&]() {   // thread 0 only
    if (!wi.advance(n_chunks, chunks_per_head, tpc, c.kv_heads, kScorePagesPerBlock, n_scored_of)) return;
    const int page0 = wi.page;
    const int npg = min(kScorePagesPerBlock, wi.n_swept - page0);
    const uint32_t bytes = (uint32_t)(npg * D * sizeof(T));
    const int wb = wi.bh / c.kv_heads;
    const size_t head_off = wb * c.meta_stride_b + (wi.bh - wb * c.kv_heads) * c.meta_stride_h;
    T* dst = s_tiles + (size_t)(issued & 1) * 2 * kTileElems;
    mbar_expect_tx(&bar[issued & 1], 2 * bytes);
    bulk_load(dst, static_cast<const T*>(c.k_min) + head_off + (size_t)page0 * D, bytes, &bar[issued & 1]);
    bulk_load(dst + kTileElems, static_cast<const T*>(c.k_max) + head_off + (size_t)page0 * D, bytes, &bar[issued & 1]);
    ++issued;
  };
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    mbar_fence_init();
    wi.start();
    issued = 0;
    issue_next();
    issue_next();
  }
  __syncthreads();   // the barriers are initialised before anyone waits on them

  const int lane_in_row = tid % LPR;
  const int gi = tid / LPR;
  const int GPP = (G + HPL - 1) / HPL;         // lane groups per page
  const int PPI = max(GROUPS / GPP, 1);        // pages per iteration
  const int slot = gi / GPP, sub = gi % GPP;
  const int h0 = sub * HPL;                    // first head (within the GQA group) of this lane group
  const bool group_live = slot < PPI;
  // which head's total this lane holds after the row reduction
  const int my_g = HPL == 4 ? (lane_in_row % (LPR / 4) == 0 ? lane_in_row / (LPR / 4) : -1)
                   : HPL == 2 ? (lane_in_row == 0 ? 0 : (lane_in_row == LPR / 2 ? 1 : -1))
                              : (lane_in_row == 0 ? 0 : -1);
  const bool writer = group_live && my_g >= 0 && h0 + my_g < G;

  float qp[HPL][EPL], qn[HPL][EPL];
  T* out_row = scores;
  // ALiBi bonus of a page: slope * (position of its last token - position of the query), added in
  // fp32 to the unscaled bound (entmaxkv/kernels/page_criticality.py:99-101,158-165)
  float slope = 0.f;
  int q_pos = 0, S_cur = 0;
  int loaded_bh = -1;

  TileWalk wc;
  wc.start();
  for (int s = 0; wc.advance(n_chunks, chunks_per_head, tpc, c.kv_heads, kScorePagesPerBlock, n_scored_of); ++s) {
    if (wc.bh != loaded_bh) {     // block-uniform: a new KV head starts
      loaded_bh = wc.bh;
      const int cb = wc.bh / c.kv_heads, chkv = wc.bh - cb * c.kv_heads;
#pragma unroll
      for (int g = 0; g < HPL; ++g) {
        const int hq = chkv * G + min(h0 + g, G - 1);
        float qf[EPL];
        unpack<T>(*reinterpret_cast<const uint4*>(q + cb * qsb + hq * qsh + lane_in_row * EPL), qf);
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          qp[g][j] = fmaxf(qf[j], 0.f);
          qn[g][j] = fminf(qf[j], 0.f);
        }
      }
      out_row = scores + ((size_t)cb * q_heads + chkv * G + h0 + max(my_g, 0)) * score_stride;
      if constexpr (ALIBI) {
        S_cur = c.seq_lens[cb];
        slope = writer ? alibi_slopes[chkv * G + h0 + my_g] : 0.f;
        q_pos = q_positions ? q_positions[cb] : S_cur - 1;
      }
    }
    const int page0 = wc.page;
    const int npg = min(kScorePagesPerBlock, wc.n_swept - page0);
    const T* s_lo = s_tiles + (size_t)(s & 1) * 2 * kTileElems;
    const T* s_hi = s_lo + kTileElems;
    // a copy that never lands leaves the scores undefined but cannot hang the GPU
    mbar_wait(&bar[s & 1], (uint32_t)(s >> 1) & 1u);
    for (int pb = 0; pb < npg; pb += PPI) {        // uniform trip count: shuffles need whole warps
      const int p = min(pb + slot, npg - 1);
      const bool live = writer && pb + slot < npg;
      float lo[EPL], hi[EPL];
      unpack<T>(lds128(s_lo + p * D + lane_in_row * EPL), lo);
      unpack<T>(lds128(s_hi + p * D + lane_in_row * EPL), hi);
      float acc[HPL];
#pragma unroll
      for (int g = 0; g < HPL; ++g) {
        acc[g] = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          acc[g] = __fmaf_rn(qp[g][j], hi[j], acc[g]);
          acc[g] = __fmaf_rn(qn[g][j], lo[j], acc[g]);
        }
      }
      float r;
      if constexpr (HPL == 4) r = row_sum_quad<LPR>(acc, lane_in_row);
      else if constexpr (HPL == 2) r = row_sum_pair<LPR>(acc[0], acc[1], lane_in_row);
      else r = row_sum<LPR>(acc[0]);
      if (live) {
        if constexpr (ALIBI) {
          const int last_pos = min((page0 + p + 1) * P - 1, S_cur - 1);
          r = __fadd_rn(r, __fmul_rn(slope, (float)(last_pos - q_pos)));
        }
        out_row[page0 + p] = from_float<T>(r);
      }
    }
    __syncthreads();   // everyone is done with this stage
    if (tid == 0) issue_next();
  }
}

// Monotone unsigned key of a stored score: larger score <=> larger key.
template <typename T> struct ScoreKey;
template <> struct ScoreKey<__half> {
  using Key = uint32_t;
  static constexpr int BITS = 16;
  static __device__ __forceinline__ Key of(const __half* p, int i) {
    const uint32_t u = reinterpret_cast<const unsigned short*>(p)[i];
    return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
  }
};
template <> struct ScoreKey<__nv_bfloat16> {
  using Key = uint32_t;
  static constexpr int BITS = 16;
  static __device__ __forceinline__ Key of(const __nv_bfloat16* p, int i) {
    const uint32_t u = reinterpret_cast<const unsigned short*>(p)[i];
    return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
  }
};
template <> struct ScoreKey<float> {
  using Key = uint32_t;
  static constexpr int BITS = 32;
  static __device__ __forceinline__ Key of(const float* p, int i) {
    const uint32_t u = __float_as_uint(p[i]);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  }
};

// grid: B*H_q blocks of 512 threads.  Radix-select the k-th largest key 8 bits at a time
// (warp-private histograms, so hot bins do not serialise the whole block), then ONE
// ordered pass packs the page ids:
//   selected(p) = key_p > K  ||  (key_p == K  &&  #{p' < p : key_p' == K} < r)
// with K the k-th largest key and r the number of slots left for keys equal to K.
// Thread t owns the 16 consecutive pages [16t, 16t+16) of every round of 8192 pages, so
// the packing needs a single block-wide scan per round.
template <typename T>
__global__ void __launch_bounds__(kSelectThreads)
topk_select_kernel(ekv_cache_desc c, int q_heads, int token_budget, const T* __restrict__ scores,
                   int64_t score_stride, int* __restrict__ page_indices, int64_t pi_stride,
                   int* __restrict__ num_selected, int* __restrict__ tok_counts,
                   const int* __restrict__ user_seqlens, int64_t usb, int64_t ush,
                   unsigned long long* __restrict__ work_items, int chunks_per_head) {
  using SK = ScoreKey<T>;
  constexpr int KPT = 16;                          // keys per thread and round
  constexpr int ROUND = kSelectThreads * KPT;      // 8192
  constexpr int WARPS = kSelectThreads / 32;
  __shared__ int whist[WARPS][256];
  __shared__ int hist[256];
  __shared__ uint32_t scan_scratch[40];
  __shared__ uint32_t s_prefix;
  __shared__ int s_krem;
  __shared__ int s_tokens;

  const int bh = blockIdx.x;
  const int b = bh / q_heads, hq = bh % q_heads;
  const int S = c.seq_lens[b];
  const int P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n = max(min(n_pages - 1, c.page_capacity), 0);
  const int k_sel = min(token_budget / P, n);
  const T* sc = scores + (size_t)bh * score_stride;
  int* out = page_indices + (size_t)bh * pi_stride;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_rounds = (n + ROUND - 1) / ROUND;

  uint32_t kth = 0;
  int r = 0;
  if (k_sel > 0 && k_sel < n) {
    if (tid == 0) {
      s_prefix = 0;
      s_krem = k_sel;
    }
    for (int shift = SK::BITS - 8; shift >= 0; shift -= 8) {
      for (int i = tid; i < WARPS * 256; i += kSelectThreads) (&whist[0][0])[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const int hi_shift = shift + 8;
      for (int rd = 0; rd < n_rounds; ++rd) {
        const int i0 = rd * ROUND + tid * KPT;
#pragma unroll 4
        for (int j = 0; j < KPT; ++j) {
          const int i = i0 + j;
          if (i < n) {
            const uint32_t key = SK::of(sc, i);
            if (hi_shift >= SK::BITS || (key >> hi_shift) == prefix)
              atomicAdd(&whist[warp][(key >> shift) & 255u], 1);
          }
        }
      }
      __syncthreads();
      if (tid < 256) {
        int t = 0;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) t += whist[w][tid];
        hist[tid] = t;
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
        // keys held by the lanes above this one
        int tot_above = 0;
        for (int l = 31; l >= 0; --l) {
          const int t = __shfl_sync(0xffffffffu, lane_total, l);
          if (l > tid) tot_above += t;
        }
        const int krem = s_krem;
        int run = tot_above;
        int found_bin = -1, found_above = 0;
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
    r = s_krem;
  }

  // ordered packing: one block scan per round of 8192 pages
  if (k_sel > 0) {
    const bool all = k_sel >= n;
    int gt_base = 0, eq_base = 0;
    for (int rd = 0; rd < n_rounds; ++rd) {
      const int i0 = rd * ROUND + tid * KPT;
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
      const uint32_t ex = block_scan_excl((uint32_t)__popc(gt_bits) | ((uint32_t)__popc(eq_bits) << 16),
                                          scan_scratch, &total);
      int gt_before = gt_base + (int)(ex & 0xffffu);
      int eq_before = eq_base + (int)(ex >> 16);
#pragma unroll 4
      for (int j = 0; j < KPT; ++j) {
        const bool g = (gt_bits >> j) & 1u, e = (eq_bits >> j) & 1u;
        if (g || (e && eq_before < r)) out[gt_before + min(eq_before, r)] = i0 + j;
        gt_before += g;
        eq_before += e;
      }
      gt_base += (int)(total & 0xffffu);
      eq_base += (int)(total >> 16);
      __syncthreads();
    }
  }
  if (tid == 0) {
    int count = k_sel;
    if (n_pages >= 1) {
      out[k_sel] = n_pages - 1;
      count = k_sel + 1;
    }
    num_selected[bh] = count;
    int T_tok = k_sel * P + (n_pages >= 1 ? S - (n_pages - 1) * P : 0);
    if (user_seqlens) {
      const int hkv = hq / (q_heads / c.kv_heads);
      T_tok = min(user_seqlens[b * usb + hkv * ush], count * P);
    }
    tok_counts[bh] = max(T_tok, 0);
    s_tokens = max(T_tok, 0);
  }
  if (work_items) {   // fixed slots: (head, chunk), empty beyond the head's tokens
    __syncthreads();
    const int T_tok = min(s_tokens, chunks_per_head * kChunkTokens);
    for (int ch = tid; ch < chunks_per_head; ch += kSelectThreads)
      work_items[(size_t)bh * chunks_per_head + ch] = make_item(bh, ch, T_tok);
  }
}

}  // namespace ekv

namespace ekv {

template <typename T, int D, int HPL, bool ALIBI>
static void launch_score_variant(const ekv_cache_desc* c, const T* q, int64_t qsb, int64_t qsh, int q_heads, T* scores,
                                 int64_t score_stride, const float* alibi_slopes, const int32_t* q_positions,
                                 int max_scored, cudaStream_t st) {
  const size_t smem = 4 * (size_t)kScorePagesPerBlock * D * sizeof(T);   // 2 stages x (k_min, k_max)
  static bool once = cudaFuncSetAttribute(page_score_kernel<T, D, HPL, ALIBI>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
  (void)once;
  // chunks of four tiles: long enough that a block rarely changes KV head, short enough that the
  // round-robin deal leaves every block the same work to within a few tiles; shorter chunks when
  // the sweep is too small to give every resident block one
  const int tiles = (max_scored + kScorePagesPerBlock - 1) / kScorePagesPerBlock;
  int tpc = kScoreTilesPerBlock;
  while (tpc > 1 && (long long)((tiles + tpc - 1) / tpc) * c->batch * c->kv_heads < 3LL * sm_count()) tpc /= 2;
  const int chunks_per_head = (tiles + tpc - 1) / tpc;
  const long long n_chunks = (long long)chunks_per_head * c->batch * c->kv_heads;
  const int blocks = (int)std::min<long long>(n_chunks, 3LL * sm_count());
  page_score_kernel<T, D, HPL, ALIBI><<<blocks, kScoreThreads, smem, st>>>(
      *c, q, qsb, qsh, q_heads, scores, score_stride, alibi_slopes, q_positions, tpc, chunks_per_head, (int)n_chunks);
}

static int launch_page_scores(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                              int32_t q_heads, int32_t max_seq_len, void* scores, int64_t score_stride,
                              const float* alibi_slopes, const int32_t* q_positions, cudaStream_t st) {
  if (int e = check_desc(c)) return e;
  if (!q || !scores || !c->k_min || !c->k_max) return EKV_ERR_ARG;
  if (q_heads <= 0 || q_heads % c->kv_heads || max_seq_len <= 0) return EKV_ERR_ARG;
  const int P = c->page_size;
  const int max_scored = (max_seq_len + P - 1) / P - 1;
  if (score_stride < max_scored) return EKV_ERR_ARG;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((q_stride_b * esz) % 16 || (q_stride_h * esz) % 16 || (reinterpret_cast<uintptr_t>(q) & 15))
    return EKV_ERR_ARG;
  if (max_scored <= 0) return EKV_OK;
  const int G = q_heads / c->kv_heads;
  if ((long long)((max_scored + kScorePagesPerBlock - 1) / kScorePagesPerBlock) * c->batch * c->kv_heads >= (1LL << 31))
    return EKV_ERR_ARG;
#define EKV_SCORE(HPL_, AL_) \
    launch_score_variant<T, D, HPL_, AL_>(c, qq, q_stride_b, q_stride_h, q_heads, ss, score_stride, alibi_slopes, \
                                          q_positions, max_scored, st)
  EKV_DISPATCH(c->dtype, c->head_dim, {
    // one page is scored by ceil(G/HPL) lane groups of a 256-thread block
    const int hpl = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
    if ((G + hpl - 1) / hpl > kScoreThreads / (D / ElemTraits<T>::EPL)) return EKV_ERR_ARG;
    const T* qq = static_cast<const T*>(q);
    T* ss = static_cast<T*>(scores);
    if (hpl == 4) { if (alibi_slopes) EKV_SCORE(4, true); else EKV_SCORE(4, false); }
    else if (hpl == 2) { if (alibi_slopes) EKV_SCORE(2, true); else EKV_SCORE(2, false); }
    else { if (alibi_slopes) EKV_SCORE(1, true); else EKV_SCORE(1, false); }
  });
#undef EKV_SCORE
  return launch_status();
}

static int launch_topk_pack(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget, int32_t max_seq_len,
                            const void* scores, int64_t score_stride, int32_t* page_indices, int64_t pi_stride,
                            int32_t* num_selected, int32_t* tok_counts, const int32_t* user_seqlens,
                            int64_t us_stride_b, int64_t us_stride_h, uint64_t* work_items, cudaStream_t st) {
  if (int e = check_desc(c)) return e;
  if (!scores || !page_indices || !num_selected || !tok_counts) return EKV_ERR_ARG;
  if (q_heads <= 0 || q_heads % c->kv_heads || token_budget < 0 || max_seq_len <= 0) return EKV_ERR_ARG;
  const int P = c->page_size;
  const int max_scored = (max_seq_len + P - 1) / P - 1;
  const int k_max = token_budget / P < max_scored ? token_budget / P : max_scored;
  if (score_stride < max_scored || pi_stride < k_max + 1) return EKV_ERR_ARG;
  const int chunks_per_head = ((k_max + 1) * P + kChunkTokens - 1) / kChunkTokens;
  if (work_items && (chunks_per_head > kItemMaxChunks || (int64_t)c->batch * q_heads >= kItemMaxHeads))
    return EKV_ERR_ARG;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    (void)D;
    topk_select_kernel<T><<<c->batch * q_heads, kSelectThreads, 0, st>>>(
        *c, q_heads, token_budget, static_cast<const T*>(scores), score_stride, page_indices,
        pi_stride, num_selected, tok_counts, user_seqlens, us_stride_b, us_stride_h,
        reinterpret_cast<unsigned long long*>(work_items), chunks_per_head);
  });
  return launch_status();
}

}  // namespace ekv

extern "C" int ekv_page_scores(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                               int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len, void* scores,
                               int64_t score_stride, void* stream) {
  return ekv::launch_page_scores(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, scores, score_stride,
                                 nullptr, nullptr, ekv::as_stream(stream));
}

extern "C" int ekv_page_scores_alibi(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                     int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len, void* scores,
                                     int64_t score_stride, const float* alibi_slopes,
                                     const int32_t* q_positions, void* stream) {
  if (!alibi_slopes) return EKV_ERR_ARG;
  return ekv::launch_page_scores(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, scores, score_stride,
                                 alibi_slopes, q_positions, ekv::as_stream(stream));
}

extern "C" int ekv_topk_pack(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget,
                             int32_t max_seq_len, const void* scores, int64_t score_stride,
                             int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                             int32_t* tok_counts, const int32_t* user_seqlens, int64_t us_stride_b,
                             int64_t us_stride_h, uint64_t* work_items, void* stream) {
  return ekv::launch_topk_pack(c, q_heads, token_budget, max_seq_len, scores, score_stride, page_indices,
                               pi_stride, num_selected, tok_counts, user_seqlens, us_stride_b, us_stride_h,
                               work_items, ekv::as_stream(stream));
}

extern "C" int ekv_topk_select(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                               int64_t q_stride_h, int32_t q_heads, int32_t token_budget,
                               int32_t max_seq_len, void* scores, int64_t score_stride,
                               int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                               int32_t* tok_counts, const int32_t* user_seqlens,
                               int64_t us_stride_b, int64_t us_stride_h, uint64_t* work_items,
                               void* stream) {
  if (int e = ekv::launch_page_scores(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, scores,
                                      score_stride, nullptr, nullptr, ekv::as_stream(stream)))
    return e;
  return ekv::launch_topk_pack(c, q_heads, token_budget, max_seq_len, scores, score_stride, page_indices,
                               pi_stride, num_selected, tok_counts, user_seqlens, us_stride_b, us_stride_h,
                               work_items, ekv::as_stream(stream));
}
