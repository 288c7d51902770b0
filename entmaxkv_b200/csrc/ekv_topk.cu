// Top-k page selection: key-range upper-bound scores swept from the page
// min/max statistics, then an exact radix selection with a deterministic tie
// rule (equal scores: lower page id wins) and ordered index packing.
//
// HBM-bound: the sweep reads k_min and k_max of every scored page once
// (2*D*sizeof(T) bytes per page and KV head, shared by the query heads of a GQA
// group); everything after it works on 2 or 4 bytes per page and query head.
#include <algorithm>
#include <cstdlib>

#include "ekv_common.cuh"
#include "ekv_score_key.cuh"
#include "ekv_work.cuh"

namespace ekv {

constexpr int kScoreTilePages = 64;       // pages per tile of the copy ring
constexpr int kScorePagesPerBlock = 256;  // pages a block sweeps (512 on grids of two waves or more)
constexpr int kScoreThreads = 256;
constexpr int kSelectThreads = 512;

// score = sum_d max(q_d*lo_d, q_d*hi_d) = sum_d (max(q_d,0)*hi_d + min(q_d,0)*lo_d):
// one of the two products is an exact zero, so the two-FMA form rounds exactly
// like the select-then-multiply form.
//
// grid: (ceil(max_scored / pages per block), B*H_kv), 256 threads, three blocks per SM.  A block owns
// `tiles_per_block` consecutive tiles of TILE pages of one KV head.  The k_min rows and the k_max rows
// of a tile are two contiguous TILE*D*sizeof(T)-byte blocks, fetched with two bulk asynchronous copies
// into one stage of an NS-stage shared-memory ring: while one tile is being scored the copies of the
// next NS-1 are in flight (these copies are the only global reads of the kernel besides q).
// A page is scored by ceil(G/HPL) groups of LPR lanes, each group owning HPL query heads of the GQA group.
template <typename T, int D, int HPL, bool ALIBI, int NS, int TILE, int BPS>
__global__ void __launch_bounds__(kScoreThreads, BPS)
page_score_kernel(ekv_cache_desc c, const T* __restrict__ q, int64_t qsb, int64_t qsh, int q_heads,
                  T* __restrict__ scores, int64_t score_stride, const float* __restrict__ alibi_slopes,
                  const int* __restrict__ q_positions, int tiles_per_block) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kScoreThreads / LPR;
  constexpr int kTileElems = TILE * D;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* s_tiles = reinterpret_cast<T*>(smem_raw);   // [stage][lo|hi][TILE*D]
  __shared__ uint64_t bar[NS];

  const int bh = blockIdx.y;
  const int b = bh / c.kv_heads, hkv = bh % c.kv_heads;
  const int G = q_heads / c.kv_heads;
  const int S = c.seq_lens[b];
  const int P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n_scored = min(n_pages - 1, c.page_capacity);
  const int first_page = blockIdx.x * TILE * tiles_per_block;
  if (first_page >= n_scored) return;
  const int n_tiles = min(tiles_per_block, (n_scored - first_page + TILE - 1) / TILE);
  const int tid = threadIdx.x;
  const size_t head_off = b * c.meta_stride_b + hkv * c.meta_stride_h;

  auto issue = [&](int t) {   // thread 0 only
    const int page0 = first_page + t * TILE;
    const int npg = min(TILE, n_scored - page0);
    const uint32_t bytes = (uint32_t)(npg * D * sizeof(T));
    const int st = t % NS;
    T* dst = s_tiles + (size_t)st * 2 * kTileElems;
    mbar_expect_tx(&bar[st], 2 * bytes);
    bulk_load(dst, static_cast<const T*>(c.k_min) + head_off + (size_t)page0 * D, bytes, &bar[st]);
    bulk_load(dst + kTileElems, static_cast<const T*>(c.k_max) + head_off + (size_t)page0 * D, bytes, &bar[st]);
  };
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < NS; ++i) mbar_init(&bar[i], 1);
    mbar_fence_init();
    for (int t = 0; t < min(NS, n_tiles); ++t) issue(t);
  }
  __syncthreads();   // the barriers are initialised before anyone waits on them

  const int lane_in_row = tid % LPR;
  const int gi = tid / LPR;
  const int GPP = (G + HPL - 1) / HPL;         // lane groups per page
  const int PPI = max(GROUPS / GPP, 1);        // pages per iteration
  const int slot = gi / GPP, sub = gi % GPP;
  const int h0 = sub * HPL;                    // first head (within the GQA group) of this lane group
  const bool group_live = slot < PPI;

  // Heads are handled two at a time with packed fp32 multiply-adds (fma.rn.f32x2: two independent IEEE
  // fused multiply-adds per instruction, so every head's sum is formed exactly as by scalar
  // instructions, in the same order): qp2[p][j] = {max(q,0) of head 2p, of head 2p+1} at element j.
  constexpr int HP = (HPL + 1) / 2;
  float2 qp2[HP][EPL], qn2[HP][EPL];
#pragma unroll
  for (int g = 0; g < 2 * HP; ++g) {
    const int hq = hkv * G + min(h0 + min(g, HPL - 1), G - 1);
    float qf[EPL];
    unpack<T>(*reinterpret_cast<const uint4*>(q + b * qsb + hq * qsh + lane_in_row * EPL), qf);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      if (g & 1) {
        qp2[g >> 1][j].y = fmaxf(qf[j], 0.f);
        qn2[g >> 1][j].y = fminf(qf[j], 0.f);
      } else {
        qp2[g >> 1][j].x = fmaxf(qf[j], 0.f);
        qn2[g >> 1][j].x = fminf(qf[j], 0.f);
      }
    }
  }
  // which head's total this lane holds after the row reduction
  const int my_g = HPL == 4 ? (lane_in_row % (LPR / 4) == 0 ? lane_in_row / (LPR / 4) : -1)
                   : HPL == 2 ? (lane_in_row == 0 ? 0 : (lane_in_row == LPR / 2 ? 1 : -1))
                              : (lane_in_row == 0 ? 0 : -1);
  const bool writer = group_live && my_g >= 0 && h0 + my_g < G;
  T* out_row = scores + ((size_t)b * q_heads + hkv * G + h0 + max(my_g, 0)) * score_stride;
  // ALiBi bonus of a page: slope * (position of its last token - position of the query), added in
  // fp32 to the unscaled bound (entmaxkv/kernels/page_criticality.py:99-101,158-165)
  float slope = 0.f;
  int q_pos = 0;
  if constexpr (ALIBI) {
    slope = writer ? alibi_slopes[hkv * G + h0 + my_g] : 0.f;
    q_pos = q_positions ? q_positions[b] : S - 1;
  }

  for (int t = 0; t < n_tiles; ++t) {
    const int page0 = first_page + t * TILE;
    const int npg = min(TILE, n_scored - page0);
    const int st = t % NS;
    const T* s_lo = s_tiles + (size_t)st * 2 * kTileElems;
    const T* s_hi = s_lo + kTileElems;
    // a copy that never lands leaves the scores undefined but cannot hang the GPU
    // plain bounded wait: recording a timeout here (a flag, a counter, a call - all were tried) pushes this
    // issue-bound kernel past its 80 registers and costs 15 % of its time; its waits are the one place where a
    // timed-out copy goes uncounted
    mbar_wait(&bar[st], (uint32_t)(t / NS) & 1u);
    for (int pb = 0; pb < npg; pb += PPI) {        // uniform trip count: shuffles need whole warps
      const int p = min(pb + slot, npg - 1);
      const bool live = writer && pb + slot < npg;
      float lo[EPL], hi[EPL];
      unpack<T>(lds128(s_lo + p * D + lane_in_row * EPL), lo);
      unpack<T>(lds128(s_hi + p * D + lane_in_row * EPL), hi);
      float2 acc2[HP];
#pragma unroll
      for (int p2 = 0; p2 < HP; ++p2) acc2[p2] = make_float2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const float2 hi2 = make_float2(hi[j], hi[j]), lo2 = make_float2(lo[j], lo[j]);
#pragma unroll
        for (int p2 = 0; p2 < HP; ++p2) {
          acc2[p2] = __ffma2_rn(qp2[p2][j], hi2, acc2[p2]);
          acc2[p2] = __ffma2_rn(qn2[p2][j], lo2, acc2[p2]);
        }
      }
      float acc[2 * HP];
#pragma unroll
      for (int p2 = 0; p2 < HP; ++p2) {
        acc[2 * p2] = acc2[p2].x;
        acc[2 * p2 + 1] = acc2[p2].y;
      }
      float r;
      if constexpr (HPL == 4) {
        const float a4[4] = {acc[0], acc[1], acc[2], acc[3]};
        r = row_sum_quad<LPR>(a4, lane_in_row);
      } else if constexpr (HPL == 2) {
        r = row_sum_pair<LPR>(acc[0], acc[1], lane_in_row);
      } else {
        r = row_sum<LPR>(acc[0]);
      }
      if (live) {
        if constexpr (ALIBI) {
          const int last_pos = min((page0 + p + 1) * P - 1, S - 1);
          r = __fadd_rn(r, __fmul_rn(slope, (float)(last_pos - q_pos)));
        }
        out_row[page0 + p] = from_float<T>(r);
      }
    }
    __syncthreads();   // everyone is done with this stage
    if (tid == 0 && t + NS < n_tiles) issue(t + NS);
  }
}

// grid: B*H_q blocks of 512 threads.  Radix-select the k-th largest key 8 bits at a time
// (warp-private histograms, so hot bins do not serialise the whole block), then ONE
// ordered pass packs the page ids:
//   selected(p) = key_p > K  ||  (key_p == K  &&  #{p' < p : key_p' == K} < r)
// with K the k-th largest key and r the number of slots left for keys equal to K.
// Thread t owns the 16 consecutive pages [16t, 16t+16) of every round of 8192 pages, so
// the packing needs a single block-wide scan per round.
template <typename T>
__global__ void __launch_bounds__(kSelectThreads, 4)
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
  // two stages of 64-page tiles, three blocks per SM (deeper rings of smaller tiles measured slower: the
  // sweep is bound by instruction issue, and every tile costs a block-wide barrier)
  constexpr int TILE = kScoreTilePages;
  // 512 pages per block halve the number of block start-ups (barrier set-up, first copies, query
  // load); worth it from two waves of the 3 blocks an SM holds (measured at 128k context: batch 8, 1024 such
  // blocks, 57.4 against 58.4 us; batch 16, 102.4 against 105.5 us; batch 4, one wave, 36.9 against 34.8 us)
  int tpb = 2 * kScorePagesPerBlock / TILE;
  {
    const long long blocks = (long long)((max_scored + TILE * tpb - 1) / (TILE * tpb)) * c->batch * c->kv_heads;
    if (blocks < 2LL * 3 * sm_count()) tpb = kScorePagesPerBlock / TILE;
  }
  dim3 grid((unsigned)((max_scored + TILE * tpb - 1) / (TILE * tpb)), (unsigned)(c->batch * c->kv_heads));
  // two stages, three blocks per SM: a third stage at two blocks per SM measured slower (190 -> 199 us at 128k)
  constexpr int NS = 2, BPS = 3;
  const size_t smem = (size_t)NS * 2 * TILE * D * sizeof(T);
  auto kernel = page_score_kernel<T, D, HPL, ALIBI, NS, TILE, BPS>;
  static bool once = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
  (void)once;
  kernel<<<grid, kScoreThreads, smem, st>>>(*c, q, qsb, qsh, q_heads, scores, score_stride, alibi_slopes,
                                            q_positions, tpb);
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

namespace ekv {
unsigned int copy_timeouts_topk() { return copy_timeouts_here(); }
}  // namespace ekv
