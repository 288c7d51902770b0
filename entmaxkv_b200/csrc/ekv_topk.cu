// Top-k page selection: key-range upper-bound scores swept from the page
// min/max statistics, then an exact radix selection with a deterministic tie
// rule (equal scores: lower page id wins) and ordered index packing.
//
// HBM-bound: the sweep reads k_min and k_max of every scored page once
// (2*D*sizeof(T) bytes per page and KV head, shared by the query heads of a GQA
// group); everything after it works on 2 or 4 bytes per page and query head.
#include "ekv_common.cuh"

namespace ekv {

constexpr int kScorePagesPerBlock = 64;
constexpr int kScoreThreads = 256;
constexpr int kSelectThreads = 512;

// score = sum_d max(q_d*lo_d, q_d*hi_d) = sum_d (max(q_d,0)*hi_d + min(q_d,0)*lo_d):
// one of the two products is an exact zero, so the two-FMA form rounds exactly
// like the select-then-multiply form.
//
// grid: (ceil(max_scored/64), B*H_kv), 256 threads; each group of LPR lanes owns a
// page at a time, the G query heads of the KV head are looped in tiles of GT.
template <typename T, int D, int GT>
__global__ void __launch_bounds__(kScoreThreads)
page_score_kernel(ekv_cache_desc c, const T* __restrict__ q, int64_t qsb, int64_t qsh, int q_heads,
                  T* __restrict__ scores, int64_t score_stride) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kScoreThreads / LPR;
  const int bh = blockIdx.y;
  const int b = bh / c.kv_heads, hkv = bh % c.kv_heads;
  const int G = q_heads / c.kv_heads;
  const int S = c.seq_lens[b];
  const int P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n_scored = min(n_pages - 1, c.page_capacity);
  const int page0 = blockIdx.x * kScorePagesPerBlock;
  if (page0 >= n_scored) return;
  const int page_end = min(page0 + kScorePagesPerBlock, n_scored);
  const int lane_in_row = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;

  const size_t mbase = b * c.meta_stride_b + hkv * c.meta_stride_h + lane_in_row * EPL;
  const T* lo_base = static_cast<const T*>(c.k_min) + mbase;
  const T* hi_base = static_cast<const T*>(c.k_max) + mbase;

  for (int g0 = 0; g0 < G; g0 += GT) {
    float qp[GT][EPL], qn[GT][EPL];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const int hq = hkv * G + min(g0 + g, G - 1);
      float qf[EPL];
      unpack<T>(*reinterpret_cast<const uint4*>(q + b * qsb + hq * qsh + lane_in_row * EPL), qf);
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        qp[g][j] = fmaxf(qf[j], 0.f);
        qn[g][j] = fminf(qf[j], 0.f);
      }
    }
    // uniform trip count: the row_sum shuffles need every lane of a warp
    for (int pb = page0; pb < page_end; pb += GROUPS) {
      const int p = min(pb + group, page_end - 1);
      const bool live = pb + group < page_end;
      float lo[EPL], hi[EPL];
      // later head tiles re-read the same 32 KB of statistics; keep them cacheable then
      if (G > GT) {
        unpack<T>(__ldg(reinterpret_cast<const uint4*>(lo_base + (size_t)p * D)), lo);
        unpack<T>(__ldg(reinterpret_cast<const uint4*>(hi_base + (size_t)p * D)), hi);
      } else {
        unpack<T>(ld_stream(lo_base + (size_t)p * D), lo);
        unpack<T>(ld_stream(hi_base + (size_t)p * D), hi);
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          acc = __fmaf_rn(qp[g][j], hi[j], acc);
          acc = __fmaf_rn(qn[g][j], lo[j], acc);
        }
        acc = row_sum<LPR>(acc);
        if (live && lane_in_row == 0 && g0 + g < G) {
          const int hq = hkv * G + g0 + g;
          scores[((size_t)b * q_heads + hq) * score_stride + p] = from_float<T>(acc);
        }
      }
    }
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

// grid: B*H_q blocks of 512 threads.  Radix-select the k-th largest key 8 bits at
// a time, then one ordered pass packs the page ids:
//   selected(p) = key_p > K  ||  (key_p == K  &&  #{p' < p : key_p' == K} < r)
// with K the k-th largest key and r the number of slots left for keys equal to K.
template <typename T>
__global__ void __launch_bounds__(kSelectThreads)
topk_select_kernel(ekv_cache_desc c, int q_heads, int token_budget, const T* __restrict__ scores,
                   int64_t score_stride, int* __restrict__ page_indices, int64_t pi_stride,
                   int* __restrict__ num_selected, int* __restrict__ tok_counts,
                   const int* __restrict__ user_seqlens, int64_t usb, int64_t ush) {
  using SK = ScoreKey<T>;
  __shared__ int hist[256];
  __shared__ uint32_t scan_scratch[40];
  __shared__ uint32_t s_prefix;
  __shared__ int s_krem;

  const int bh = blockIdx.x;
  const int b = bh / q_heads, hq = bh % q_heads;
  const int S = c.seq_lens[b];
  const int P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n = max(min(n_pages - 1, c.page_capacity), 0);
  const int k_sel = min(token_budget / P, n);
  const T* sc = scores + (size_t)bh * score_stride;
  int* out = page_indices + (size_t)bh * pi_stride;
  const int tid = threadIdx.x;

  uint32_t kth = 0;
  int r = 0;
  if (k_sel > 0 && k_sel < n) {
    if (tid == 0) {
      s_prefix = 0;
      s_krem = k_sel;
    }
    for (int shift = SK::BITS - 8; shift >= 0; shift -= 8) {
      for (int i = tid; i < 256; i += kSelectThreads) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const int hi_shift = shift + 8;
      for (int i = tid; i < n; i += kSelectThreads) {
        const uint32_t key = SK::of(sc, i);
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

  // ordered packing
  int gt_base = 0, eq_base = 0;
  if (k_sel > 0) {
    const bool all = k_sel >= n;
    for (int i0 = 0; i0 < n; i0 += kSelectThreads) {
      const int i = i0 + tid;
      uint32_t gt = 0, eq = 0;
      if (i < n) {
        if (all) {
          gt = 1;
        } else {
          const uint32_t key = SK::of(sc, i);
          gt = key > kth;
          eq = key == kth;
        }
      }
      uint32_t total;
      const uint32_t ex = block_scan_excl(gt | (eq << 16), scan_scratch, &total);
      const int gt_before = gt_base + (int)(ex & 0xffffu);
      const int eq_before = eq_base + (int)(ex >> 16);
      if (gt || (eq && eq_before < r)) out[gt_before + min(eq_before, r)] = i;
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
  }
}

}  // namespace ekv

namespace ekv {

static int launch_page_scores(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                              int32_t q_heads, int32_t max_seq_len, void* scores, int64_t score_stride,
                              cudaStream_t st) {
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
  EKV_DISPATCH(c->dtype, c->head_dim, {
    dim3 grid((unsigned)((max_scored + kScorePagesPerBlock - 1) / kScorePagesPerBlock),
              (unsigned)(c->batch * c->kv_heads));
    const T* qq = static_cast<const T*>(q);
    T* ss = static_cast<T*>(scores);
    if (G >= 4)
      page_score_kernel<T, D, 4><<<grid, kScoreThreads, 0, st>>>(*c, qq, q_stride_b, q_stride_h, q_heads, ss, score_stride);
    else if (G >= 2)
      page_score_kernel<T, D, 2><<<grid, kScoreThreads, 0, st>>>(*c, qq, q_stride_b, q_stride_h, q_heads, ss, score_stride);
    else
      page_score_kernel<T, D, 1><<<grid, kScoreThreads, 0, st>>>(*c, qq, q_stride_b, q_stride_h, q_heads, ss, score_stride);
  });
  return launch_status();
}

static int launch_topk_pack(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget, int32_t max_seq_len,
                            const void* scores, int64_t score_stride, int32_t* page_indices, int64_t pi_stride,
                            int32_t* num_selected, int32_t* tok_counts, const int32_t* user_seqlens,
                            int64_t us_stride_b, int64_t us_stride_h, cudaStream_t st) {
  if (int e = check_desc(c)) return e;
  if (!scores || !page_indices || !num_selected || !tok_counts) return EKV_ERR_ARG;
  if (q_heads <= 0 || q_heads % c->kv_heads || token_budget < 0 || max_seq_len <= 0) return EKV_ERR_ARG;
  const int P = c->page_size;
  const int max_scored = (max_seq_len + P - 1) / P - 1;
  const int k_max = token_budget / P < max_scored ? token_budget / P : max_scored;
  if (score_stride < max_scored || pi_stride < k_max + 1) return EKV_ERR_ARG;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    (void)D;
    topk_select_kernel<T><<<c->batch * q_heads, kSelectThreads, 0, st>>>(
        *c, q_heads, token_budget, static_cast<const T*>(scores), score_stride, page_indices,
        pi_stride, num_selected, tok_counts, user_seqlens, us_stride_b, us_stride_h);
  });
  return launch_status();
}

}  // namespace ekv

extern "C" int ekv_page_scores(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                               int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len, void* scores,
                               int64_t score_stride, void* stream) {
  return ekv::launch_page_scores(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, scores, score_stride,
                                 ekv::as_stream(stream));
}

extern "C" int ekv_topk_pack(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget,
                             int32_t max_seq_len, const void* scores, int64_t score_stride,
                             int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                             int32_t* tok_counts, const int32_t* user_seqlens, int64_t us_stride_b,
                             int64_t us_stride_h, void* stream) {
  return ekv::launch_topk_pack(c, q_heads, token_budget, max_seq_len, scores, score_stride, page_indices,
                               pi_stride, num_selected, tok_counts, user_seqlens, us_stride_b, us_stride_h,
                               ekv::as_stream(stream));
}

extern "C" int ekv_topk_select(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                               int64_t q_stride_h, int32_t q_heads, int32_t token_budget,
                               int32_t max_seq_len, void* scores, int64_t score_stride,
                               int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                               int32_t* tok_counts, const int32_t* user_seqlens,
                               int64_t us_stride_b, int64_t us_stride_h, void* stream) {
  if (int e = ekv::launch_page_scores(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, scores,
                                      score_stride, ekv::as_stream(stream)))
    return e;
  return ekv::launch_topk_pack(c, q_heads, token_budget, max_seq_len, scores, score_stride, page_indices,
                               pi_stride, num_selected, tok_counts, user_seqlens, us_stride_b, us_stride_h,
                               ekv::as_stream(stream));
}
