// Gaussian-aware page selection: per-page score moments swept from the page
// mean/std statistics, the single-Gaussian tau estimate, threshold selection with
// ordered index packing, and the tau clamp.
//
// HBM-bound: the sweep reads k_mean and k_std of every statistical page once
// (2*D*sizeof(T) bytes per page and KV head, shared by the query heads of a GQA
// group); everything after it works on 8 bytes per page and query head.
#include <algorithm>
#include <cstdlib>

#include "ekv_common.cuh"
#include "ekv_work.cuh"
#include "ekv_exchange.cuh"

namespace ekv {

constexpr int kMomPagesPerBlock = 64;     // pages per tile
constexpr int kMomTilesPerBlock = 4;        // at most; fewer when the grid would not fill the GPU
constexpr int kMomThreads = 256;
constexpr int kGSelThreads = 512;
constexpr int kWorkTile = 1024;       // heads per tile of the work-list prefix
// consecutive pages per thread and round of the selection kernel: 16 (rounds of 8192 pages, 68 KiB of
// shared memory, two blocks per SM) when the grid has few blocks, 8 (rounds of 4096, 34 KiB, four
// blocks per SM) when it has several waves of them
template <int KPT> struct GSel {
  static constexpr int kRound = kGSelThreads * KPT;               // pages per round
  static constexpr int kTile = kRound + kRound / KPT;             // one padding word per thread's run
  static constexpr size_t kSmem = 2 * (size_t)kTile * sizeof(float);
};

struct GaussianWs {
  int* counters;     // [B*H_kv] last-block tickets of the moments sweep
  float* partial;    // [B*H_q, tiles, 4]
  int tiles;         // partial-sum slots per head = thread blocks per KV head at one tile per block
  int tpb;           // tiles per block of this launch (1, 2, 4 or 8)
};

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline size_t gaussian_ws_layout(int batch, int q_heads, int max_pages, void* base, GaussianWs* ws) {
  const int tiles = (max_pages + kMomPagesPerBlock - 1) / kMomPagesPerBlock;
  size_t off = 0;
  char* p = static_cast<char*>(base);
  const size_t cnt_bytes = align_up((size_t)batch * q_heads * sizeof(int), 256);
  const size_t part_bytes = align_up((size_t)batch * q_heads * tiles * 4 * sizeof(float), 256);
  if (ws) {
    ws->counters = reinterpret_cast<int*>(p + off);
    ws->partial = reinterpret_cast<float*>(p + off + cnt_bytes);
    ws->tiles = tiles;
    ws->tpb = kMomTilesPerBlock;
  }
  off += cnt_bytes + part_bytes;
  return off;
}

// ---- tau_hat: root of n*E[(a*S - tau)_+^beta] = 1, S ~ N(mu_g, sigma_g^2) -------

// Phi(x) through the complementary error function: the roots sit far in the upper tail of the score
// distribution (x = -4.5 for a million tokens), where 0.5 * (1 + erf(x / sqrt 2)) has lost all but two
// digits of Phi to cancellation in fp32.
__device__ __forceinline__ float normal_cdf(float x) { return 0.5f * erfcf(-x * 0.70710678118654752f); }
__device__ __forceinline__ float normal_pdf(float x) { return expf(-0.5f * x * x) * 0.39894228040143268f; }

// alpha_kind 0: alpha = 2 (beta 1); 1: alpha = 1.5 (beta 2)
__device__ __forceinline__ void gaussian_constraint(float tau, float a, float mu_g, float sigma_g, float n,
                                                    int alpha_kind, float& f, float& fp, float& fpp) {
  const float sy = fmaxf(a * sigma_g, 1e-10f);
  const float my = a * mu_g - tau;
  const float t = my / sy;
  const float ph = normal_pdf(t), Ph = normal_cdf(t);
  const float m0 = Ph;
  const float m1 = my * Ph + sy * ph;
  if (alpha_kind == 0) {
    f = n * m1 - 1.f;
    fp = -n * m0;
    fpp = n * ph / sy;
  } else {
    const float m2 = (my * my + sy * sy) * Ph + my * sy * ph;
    f = n * m2 - 1.f;
    fp = -2.f * n * m1;
    fpp = 2.f * n * m0;
  }
}

// alpha = 4/3 (beta = 3): n * E[Y_+^3] - 1 with E[Y_+^3] = (my^3 + 3 my sy^2) Phi(t) + (sy^3 + 2 my^2 sy) phi(t),
// Y ~ N(my, sy^2), t = my / sy (entmaxkv/tau_solver.py:73-78).  In the upper tail the two terms cancel to
// one part in t^6 / 6, beyond what fp32 holds, so this constraint is evaluated in fp64 (a few dozen
// evaluations per head and step).
__host__ __device__ __forceinline__ bool alpha_is_four_thirds(float alpha) { return fabsf(alpha - 1.3333334f) < 1e-6f; }
__device__ __forceinline__ void gaussian_third_moments(double my, double sy, double& m2, double& m3) {
  const double t = my / sy;
  const double ph = exp(-0.5 * t * t) * 0.3989422804014327, Ph = 0.5 * erfc(-t * 0.7071067811865476);
  m2 = (my * my + sy * sy) * Ph + my * sy * ph;
  m3 = (my * my * my + 3.0 * my * sy * sy) * Ph + (sy * sy * sy + 2.0 * my * my * sy) * ph;
}

// tau_hat by a whole warp.  The reference brackets the root in [a*mu -+ a*sigma*(sqrt(2 ln(n+1)) + 8)]
// and runs a fixed number of safeguarded Halley steps with bisection fallback
// (entmaxkv/kernels/tau_solver_gpu.py:79-125; general alpha: tau_solver.py:276-344): dozens of
// dependent erf/exp evaluations for one root.  Here every lane evaluates the constraint at one
// of 32 points that split the same bracket into 33 parts, a ballot finds the sign change (the
// constraint decreases in tau), and the bracket shrinks 33-fold per round - fp32 resolution
// after about six rounds - followed by one bracketed Halley step from the midpoint.
// All 32 lanes must call it with the same arguments; all return the same value.  It lands on the same fp32 root up to the rounding
// noise of the constraint itself (~1e-6 relative).
__device__ float tau_hat_single_gaussian_warp(float mu_g, float sigma_g, float n, float alpha) {
  const float a = alpha - 1.f;
  const int kind = alpha_kind_of(alpha);
  const int lane = threadIdx.x & 31;
  const float logf_n = sqrtf(2.f * logf(n + 1.f));
  float lo, hi;
  const float beta = 1.f / a;
  const float sy = fmaxf(a * fmaxf(sigma_g, kind == 2 ? 0.f : 1e-6f), 1e-10f);
  const bool third = alpha_is_four_thirds(alpha);   // closed form; bracketed like the general case
  auto constraint = [&](float tau) {
    if (third) {
      double m2, m3;
      gaussian_third_moments((double)a * (double)mu_g - (double)tau, (double)sy, m2, m3);
      return (float)((double)n * m3 - 1.0);
    }
    if (kind == 2) {
      const float t = fmaxf((a * mu_g - tau) / sy, 0.f);
      return t > 0.f ? n * pow_pos(sy, beta) * pow_pos(t, beta) - 1.f : -1.f;
    }
    float f, d1, d2;
    gaussian_constraint(tau, a, mu_g, fmaxf(sigma_g, 1e-6f), n, kind, f, d1, d2);
    return f;
  };
  if (kind == 2) {
    lo = a * mu_g - 5.f * a * sigma_g;
    hi = a * mu_g + a * sigma_g * (logf_n + 5.f);
    for (int i = 0; i < 64 && constraint(lo) < 0.f; ++i) lo -= 2.f * sigma_g;
    for (int i = 0; i < 64 && constraint(hi) > 0.f; ++i) hi += 2.f * sigma_g;
  } else {
    const float radius = a * fmaxf(sigma_g, 1e-6f) * (logf_n + 8.f);
    lo = a * mu_g - radius;
    hi = a * mu_g + radius;
  }
  for (int round = 0; round < 12; ++round) {
    const float w = (hi - lo) * (1.f / 33.f);
    const float t = lo + (float)(lane + 1) * w;
    const unsigned above = __ballot_sync(0xffffffffu, constraint(t) > 0.f);   // root lies above t
    const int k = above == 0xffffffffu ? 32 : __ffs(~above) - 1;              // first lane at or past the root
    const float nlo = k == 0 ? lo : lo + (float)k * w;
    const float nhi = k == 32 ? hi : lo + (float)(k + 1) * w;
    if (!(nhi - nlo < hi - lo) || !(nhi > nlo)) break;                        // fp32 cannot split the bracket further
    lo = nlo;
    hi = nhi;
    if (hi - lo <= 2e-7f * fmaxf(fmaxf(fabsf(lo), fabsf(hi)), 1e-30f)) break;
  }
  float tau = 0.5f * (lo + hi);
  if (kind != 2) {
    float f, fp, fpp;
    gaussian_constraint(tau, a, mu_g, fmaxf(sigma_g, 1e-6f), n, kind, f, fp, fpp);
    const float den = 2.f * fp * fp - f * fpp;
    const float step = fabsf(den) > 1e-18f ? 2.f * f * fp / den : f / fminf(fp, -1e-12f);
    const float cand = tau - step;
    if (cand == cand && cand > lo && cand < hi) tau = cand;
  }
  return tau;
}

// head_stats = { mu_global, sigma_global, tau_hat, mean(mu_p + 1.5 sigma_p) }, computed by a whole
// warp (same arguments in every lane); lane 0 stores.  Not inlined: every kernel that finishes
// head statistics runs the same machine code, so the fused-exchange path and the plain path
// agree to the bit.
__device__ __noinline__ void finalize_head_warp(const float* sums, float n_pages, float n_tokens, float alpha,
                                                float* stats, bool solve_tau = true) {
  float mean = sums[0] / n_pages;
  const float mean_var = sums[2] / n_pages;
  const float var_means = fmaxf(sums[1] / n_pages - mean * mean, 0.f);
  float sg = sqrtf(mean_var + var_means);
  if (!(mean == mean) || isinf(mean)) mean = 0.f;
  if (!(sg == sg)) sg = 1e-6f;
  if (isinf(sg)) sg = sg > 0.f ? 1e6f : 1e-6f;
  sg = fmaxf(sg, 1e-6f);
  const float tau = solve_tau ? tau_hat_single_gaussian_warp(mean, sg, n_tokens, alpha) : 0.f;
  if ((threadIdx.x & 31) == 0) {
    stats[0] = mean;
    stats[1] = sg;
    stats[2] = tau;
    stats[3] = sums[3] / n_pages;
  }
}

// ---- moments sweep -----------------------------------------------------------

// grid: (blocks, B*H_kv), 256 threads.  A block owns up to four consecutive tiles of 64
// statistical pages of one KV head; the k_mean rows and k_std rows of a tile are two
// contiguous blocks fetched with two bulk asynchronous copies into one of two shared
// memory stages while the previous tile is processed.  A page is handled by ceil(G/HPL)
// groups of LPR lanes, each group owning HPL query heads.  The last block to finish a KV
// head folds the per-block partial sums of its query heads in block order.
template <typename T, int D, int HPL, bool ALIBI>
__global__ void __launch_bounds__(kMomThreads, 3)
gaussian_moments_kernel(ekv_cache_desc c, const T* __restrict__ q, int64_t qsb, int64_t qsh, int q_heads,
                        int exclude_last, float alpha, int finalize, float* __restrict__ mu_pages,
                        float* __restrict__ sigma_pages, int64_t pstride, float* __restrict__ head_sums,
                        float* __restrict__ head_stats, GaussianWs ws, const float* __restrict__ alibi_slopes,
                        const int* __restrict__ q_positions) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kMomThreads / LPR;
  constexpr int kTileElems = kMomPagesPerBlock * D;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* s_tiles = reinterpret_cast<T*>(smem_raw);   // [stage][mean|std][64*D]
  __shared__ uint64_t bar[2];
  __shared__ float red[GROUPS][HPL][4];
  __shared__ int s_ticket;

  const int bh = blockIdx.y;
  const int b = bh / c.kv_heads, hkv = bh % c.kv_heads;
  const int G = q_heads / c.kv_heads;
  const int S = c.seq_lens[b];
  const int P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n_stats = min((exclude_last && n_pages > 1) ? n_pages - 1 : n_pages, c.page_capacity);
  const int kPagesPerBlock = kMomPagesPerBlock * ws.tpb;
  const int my_blocks = (n_stats + kPagesPerBlock - 1) / kPagesPerBlock;
  if ((int)blockIdx.x >= my_blocks) return;
  const int first_page = blockIdx.x * kPagesPerBlock;
  const int n_tiles = min(ws.tpb, (n_stats - first_page + kMomPagesPerBlock - 1) / kMomPagesPerBlock);
  const int tid = threadIdx.x;
  const size_t head_off = b * c.meta_stride_b + hkv * c.meta_stride_h;

  auto issue = [&](int t) {   // thread 0 only
    const int page0 = first_page + t * kMomPagesPerBlock;
    const int npg = min(kMomPagesPerBlock, n_stats - page0);
    const uint32_t bytes = (uint32_t)(npg * D * sizeof(T));
    T* dst = s_tiles + (size_t)(t & 1) * 2 * kTileElems;
    mbar_expect_tx(&bar[t & 1], 2 * bytes);
    bulk_load(dst, static_cast<const T*>(c.k_mean) + head_off + (size_t)page0 * D, bytes, &bar[t & 1]);
    bulk_load(dst + kTileElems, static_cast<const T*>(c.k_std) + head_off + (size_t)page0 * D, bytes, &bar[t & 1]);
  };
  __shared__ int s_timeout;      // a bounded wait on a copy ran out (reported once, after the tile loop)
  if (tid == 0) {
    s_timeout = 0;
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    mbar_fence_init();
    issue(0);
    if (n_tiles > 1) issue(1);
  }
  __syncthreads();

  const int lane_in_row = tid % LPR;
  const int gi = tid / LPR;
  const int GPP = (G + HPL - 1) / HPL;
  const int PPI = max(GROUPS / GPP, 1);
  const int slot = gi / GPP, sub = gi % GPP;
  const int h0 = sub * HPL;
  const bool group_live = slot < PPI;
  static_assert(D == 64 || D == 128, "1/sqrt(D) constants below cover D = 64 and 128");
  const float scale = D == 64 ? 0.125f : 0.08838834764831845f;   // fp32(1/sqrt(D))

  float qs[HPL][EPL], qv[HPL][EPL];
#pragma unroll
  for (int g = 0; g < HPL; ++g) {
    const int hq = hkv * G + min(h0 + g, G - 1);
    float qf[EPL];
    unpack<T>(*reinterpret_cast<const uint4*>(q + b * qsb + hq * qsh + lane_in_row * EPL), qf);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      qs[g][j] = qf[j] * scale;
      qv[g][j] = qs[g][j] * qs[g][j];
    }
  }
  // which head's totals this lane ends up holding after the row reduction
  const int my_g = HPL == 4 ? (lane_in_row % (LPR / 4) == 0 ? lane_in_row / (LPR / 4) : -1)
                   : HPL == 2 ? (lane_in_row == 0 ? 0 : (lane_in_row == LPR / 2 ? 1 : -1))
                              : (lane_in_row == 0 ? 0 : -1);
  const bool writer = group_live && my_g >= 0 && h0 + my_g < G;
  const size_t out_off = ((size_t)b * q_heads + hkv * G + h0 + max(my_g, 0)) * pstride;
  float sums[4] = {0.f, 0.f, 0.f, 0.f};
  // ALiBi: a page's mean score gets slope * (mean position of the page - query position); the
  // global moments (sums 0..2) stay those of the unbiased means (gaussian_utils.py:136-153)
  float slope = 0.f, q_posf = 0.f, last_stat_pos = 0.f;
  if constexpr (ALIBI) {
    slope = writer ? alibi_slopes[hkv * G + h0 + my_g] : 0.f;
    q_posf = (float)(q_positions ? q_positions[b] : S - 1);
    last_stat_pos = (float)(((exclude_last && n_pages > 1) ? (n_pages - 1) * P : S) - 1);
  }

  for (int t = 0; t < n_tiles; ++t) {
    const int page0 = first_page + t * kMomPagesPerBlock;
    const int npg = min(kMomPagesPerBlock, n_stats - page0);
    const T* s_mean = s_tiles + (size_t)(t & 1) * 2 * kTileElems;
    const T* s_std = s_mean + kTileElems;
    mbar_wait_or_mark(&bar[t & 1], (uint32_t)(t >> 1) & 1u, &s_timeout);
    for (int pb = 0; pb < npg; pb += PPI) {          // uniform trip count: shuffles need whole warps
      const int p = min(pb + slot, npg - 1);
      const bool live = writer && pb + slot < npg;
      float km[EPL], ks[EPL];
      unpack<T>(lds128(s_mean + p * D + lane_in_row * EPL), km);
      unpack<T>(lds128(s_std + p * D + lane_in_row * EPL), ks);
#pragma unroll
      for (int j = 0; j < EPL; ++j) ks[j] = ks[j] * ks[j];
      float mu[HPL], var[HPL];
#pragma unroll
      for (int g = 0; g < HPL; ++g) {
        mu[g] = 0.f;
        var[g] = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          mu[g] = fmaf(km[j], qs[g][j], mu[g]);
          var[g] = fmaf(ks[j], qv[g][j], var[g]);
        }
      }
      float m, v;
      if constexpr (HPL == 4) {
        m = row_sum_quad<LPR>(mu, lane_in_row);
        v = row_sum_quad<LPR>(var, lane_in_row);
      } else if constexpr (HPL == 2) {
        m = row_sum_pair<LPR>(mu[0], mu[1], lane_in_row);
        v = row_sum_pair<LPR>(var[0], var[1], lane_in_row);
      } else {
        m = row_sum<LPR>(mu[0]);
        v = row_sum<LPR>(var[0]);
      }
      if (live) {
        const float sg = sqrtf(v);
        float mb = m;
        if constexpr (ALIBI) {
          const float mean_pos = fminf((float)((page0 + p) * P) + 0.5f * (float)(P - 1), last_stat_pos);
          mb = __fadd_rn(m, __fmul_rn(slope, mean_pos - q_posf));
        }
        mu_pages[out_off + page0 + p] = mb;
        sigma_pages[out_off + page0 + p] = sg;
        sums[0] += m;
        sums[1] += m * m;
        sums[2] += v;
        sums[3] += mb + 1.5f * sg;
      }
    }
    __syncthreads();   // everyone is done with this stage
    if (tid == 0 && t + 2 < n_tiles) issue(t + 2);
  }
  if (tid == 0 && s_timeout) note_copy_timeout(nullptr);
  if (my_g >= 0) {
#pragma unroll
    for (int k = 0; k < 4; ++k) red[gi][my_g][k] = sums[k];
  }
  __syncthreads();
  // thread (g_abs, k) folds the lane groups that own head g_abs, in page-slot order
  if (tid < G * 4) {
    const int g_abs = tid / 4, k = tid % 4;
    const int sub_g = g_abs / HPL, gg = g_abs % HPL;
    float tsum = 0.f;
    for (int sl = 0; sl < PPI; ++sl) tsum += red[sl * GPP + sub_g][gg][k];
    ws.partial[(((size_t)b * q_heads + hkv * G + g_abs) * ws.tiles + blockIdx.x) * 4 + k] = tsum;
  }

  // last block of this KV head folds the blocks' partial sums
  __threadfence();
  __syncthreads();
  if (tid == 0) s_ticket = atomicAdd(&ws.counters[bh], 1);
  __syncthreads();
  if (s_ticket != my_blocks - 1) return;
  __threadfence();
  const int warp = tid >> 5, lane = tid & 31;
  for (int g = warp; g < G; g += kMomThreads / 32) {
    const int hq = hkv * G + g;
    const float* part = ws.partial + ((size_t)b * q_heads + hq) * ws.tiles * 4;
    float tt[4] = {0.f, 0.f, 0.f, 0.f};
    for (int blk = lane; blk < my_blocks; blk += 32)
#pragma unroll
      for (int k = 0; k < 4; ++k) tt[k] += ld_cg(part + blk * 4 + k);
#pragma unroll
    for (int k = 0; k < 4; ++k) tt[k] = warp_sum(tt[k]);
    if (lane == 0) {
      float* hs = head_sums + ((size_t)b * q_heads + hq) * 4;
#pragma unroll
      for (int k = 0; k < 4; ++k) hs[k] = tt[k];
    }
    if (finalize) {   // the whole warp solves this head's tau_hat (finalize == 2: tau_hat comes later)
      const float n_tok = (exclude_last && n_pages > 1) ? (float)(n_pages - 1) * (float)P : (float)S;
      finalize_head_warp(tt, (float)n_stats, n_tok, alpha, head_stats + ((size_t)b * q_heads + hq) * 4,
                         finalize != 2);
    }
  }
  if (tid == 0) ws.counters[bh] = 0;
}

}  // namespace ekv

#include "ekv_moments_mma.cuh"

namespace ekv {

__global__ void gaussian_finalize_kernel(const float* __restrict__ head_sums, const int* __restrict__ n_pages,
                                         const int* __restrict__ n_tokens, int batch, int q_heads, float alpha,
                                         float* __restrict__ head_stats) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;   // a warp per head
  if (i >= batch * q_heads) return;
  const int b = i / q_heads;
  float s[4];
  for (int k = 0; k < 4; ++k) s[k] = head_sums[(size_t)i * 4 + k];
  finalize_head_warp(s, (float)n_pages[b], (float)n_tokens[b], alpha, head_stats + (size_t)i * 4);
}

// Same, with the page / token counts derived from global sequence lengths on the device
// (pages 0..Np-2 carry statistics; a single page counts itself).
__global__ void gaussian_finalize_lens_kernel(const float* __restrict__ head_sums, const int* __restrict__ total_lens,
                                              int page_size, int batch, int q_heads, float alpha,
                                              float* __restrict__ head_stats) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;   // a warp per head
  if (i >= batch * q_heads) return;
  const int S = total_lens[i / q_heads];
  const int n_pages = (S + page_size - 1) / page_size;
  const int n_stat = n_pages > 1 ? n_pages - 1 : n_pages;
  const int n_tok = n_pages > 1 ? (n_pages - 1) * page_size : S;
  float s[4];
  for (int k = 0; k < 4; ++k) s[k] = head_sums[(size_t)i * 4 + k];
  finalize_head_warp(s, (float)n_stat, (float)n_tok, alpha, head_stats + (size_t)i * 4);
}

// ---- page-mixture tau_hat (ALiBi) ---------------------------------------------------

constexpr int kMixThreads = 512;

// grid: B*H_q blocks.  Root of  sum_p P * E[(a*S_p - tau)_+^beta] = 1  with S_p ~ N(mu_p, sigma_p^2)
// over the statistical pages of one head, beta = 1 (alpha 2), 2 (alpha 1.5) or 3 (alpha 4/3): with ALiBi the page
// means drift with position, so the scores are modelled as a mixture of one Gaussian per page
// instead of a single one (entmaxkv/kernels/tau_solver_page_mixture.py:67-185,
// entmaxkv/kernels/tau_mixture_solver_triton.py:81-165).  The constraint is convex and
// decreasing in tau: safeguarded Newton inside the bracket of the page extremes, every
// evaluation one fixed-order block reduction over the pages.  Writes head_stats[bh][2].
__global__ void __launch_bounds__(kMixThreads)
gaussian_mixture_tau_kernel(ekv_cache_desc c, int q_heads, int exclude_last, float alpha,
                            const float* __restrict__ mu_pages, const float* __restrict__ sigma_pages,
                            int64_t pstride, float* __restrict__ head_stats) {
  __shared__ float scratch[32];
  const int bh = blockIdx.x, tid = threadIdx.x;
  const int b = bh / q_heads;
  const int S = c.seq_lens[b], P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n_stats = min((exclude_last && n_pages > 1) ? n_pages - 1 : n_pages, c.page_capacity);
  const float a = alpha - 1.f;
  const int kind = alpha_kind_of(alpha);
  const bool third = alpha_is_four_thirds(alpha);
  const float* mu = mu_pages + (size_t)bh * pstride;
  const float* sg = sigma_pages + (size_t)bh * pstride;
  float lo_t = INFINITY, hi_t = -INFINITY;
  for (int i = tid; i < n_stats; i += kMixThreads) {
    const float my = a * mu[i], sy = fmaxf(a * sg[i], 1e-10f);
    lo_t = fminf(lo_t, my - 12.f * sy);
    hi_t = fmaxf(hi_t, my + 12.f * sy);
  }
  float lo = -block_max(-lo_t, scratch) - 1.f;
  float hi = block_max(hi_t, scratch);
  float tau = 0.5f * (lo + hi);
  const float cnt = (float)P;
  for (int it = 0; it < 48; ++it) {
    float f = 0.f, fp = 0.f;
    for (int i = tid; i < n_stats; i += kMixThreads) {
      const float sy = fmaxf(a * sg[i], 1e-10f);
      const float my = a * mu[i] - tau;
      if (third) {
        double m2, m3;
        gaussian_third_moments((double)a * (double)mu[i] - (double)tau, (double)sy, m2, m3);
        f += (float)m3;
        fp -= (float)(3.0 * m2);
        continue;
      }
      const float t = my / sy;
      const float ph = normal_pdf(t), Ph = normal_cdf(t);
      const float m1 = my * Ph + sy * ph;
      if (kind == 0) {
        f += m1;
        fp -= Ph;
      } else {
        f += (my * my + sy * sy) * Ph + my * sy * ph;
        fp -= 2.f * m1;
      }
    }
    __syncthreads();
    f = cnt * block_sum(f, scratch) - 1.f;
    fp = cnt * block_sum(fp, scratch);
    if (fabsf(f) <= 1e-6f) break;                       // every thread holds the same f
    if (f > 0.f) lo = tau; else hi = tau;
    float cand = tau - f / fminf(fp, -1e-20f);
    if (!(cand > lo) || !(cand < hi)) cand = 0.5f * (lo + hi);
    if (!(hi - lo > 0.f) || fabsf(cand - tau) <= 1e-7f * fmaxf(fabsf(tau), 1e-3f)) {
      tau = cand;
      break;
    }
    tau = cand;
  }
  if (tid == 0) head_stats[(size_t)bh * 4 + 2] = tau;
}

// ---- threshold selection + packing + clamp ------------------------------------

// Sequence-sharded step: the selection also trades the clamp cap with the other ranks (exchange slot 1)
// and clamps tau with the world's maximum, instead of leaving that to a launch of its own.
struct SelectXch {
  XchDev xch;
  int use;
  int* status;
};

// grid: B*H_q blocks of 512 threads.
template <int KPT>
__global__ void __launch_bounds__(kGSelThreads)
gaussian_select_kernel(ekv_cache_desc c, int q_heads, int exclude_last, int append_last, float alpha,
                       float frac, float z_low, float z_high, float z_clamp, int apply_clamp,
                       const float* __restrict__ sigma_mean, const float* __restrict__ mu_pages,
                       const float* __restrict__ sigma_pages, int64_t pstride,
                       const float* __restrict__ head_stats, int* __restrict__ page_indices,
                       int64_t pi_stride, int* __restrict__ num_selected, int* __restrict__ tok_counts,
                       float* __restrict__ tau_floor_out, float* __restrict__ cap_out,
                       float* __restrict__ tau_out, unsigned long long* __restrict__ work_list, int* work_total,
                       int max_tokens, const SelectXch sx) {
  __shared__ float fscratch[32];
  __shared__ uint32_t uscratch[40];
  __shared__ float s_floor, s_z;

  Xch xe;
  if (sx.use) xe = xch_begin(sx.xch, 1, sx.status);
  const int bh = blockIdx.x;
  const int b = bh / q_heads;
  const int tid = threadIdx.x;
  const int n_heads_total = c.batch * q_heads;
  const int S = c.seq_lens[b];
  const int P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n_stats = min((exclude_last && n_pages > 1) ? n_pages - 1 : n_pages, c.page_capacity);
  const float a = alpha - 1.f;

  // batch-wide mean of sigma_global (fixed summation order)
  float sbar;
  if (sigma_mean) {
    sbar = *sigma_mean;
  } else {
    float part = 0.f;
    for (int i = tid; i < n_heads_total; i += kGSelThreads) part += head_stats[(size_t)i * 4 + 1];
    sbar = block_sum(part, fscratch) / (float)n_heads_total;
  }
  const float* hs = head_stats + (size_t)bh * 4;
  const float sigma_g = hs[1], tau_hat = hs[2], upper = hs[3];
  if (tid == 0) {
    const bool low = sbar < 1.5f;
    const float margin = (float)((low ? 0.01 : 0.05) * (double)sbar);
    const float thr = tau_hat / a;
    const float sigma_delta = margin * sigma_g;
    const float tau_delta = frac * fmaxf(thr - upper, 0.f);
    s_floor = tau_hat - fmaxf(sigma_delta, tau_delta) * a;
    s_z = low ? z_low : z_high;
  }
  __syncthreads();
  const float tau_floor = s_floor, z_page = s_z;

  const float* mu = mu_pages + (size_t)bh * pstride;
  const float* sg = sigma_pages + (size_t)bh * pstride;
  int* out = page_indices + (size_t)bh * pi_stride;
  int count = 0;
  float cap = -INFINITY;
  // thread t owns the KPT consecutive pages [KPT*t, KPT*t + KPT) of every round of 512*KPT pages, so
  // the ordered packing needs one block-wide scan per round
  constexpr int ROUND = GSel<KPT>::kRound;
  constexpr int kGSelTile = GSel<KPT>::kTile;
  // A round's statistics are first brought into shared memory with coalesced loads (consecutive
  // threads read consecutive pages, all 32 loads of a thread in flight), then each thread scans
  // its own KPT consecutive pages from the tile; one padding word per KPT keeps those reads
  // free of bank conflicts.  Loading the thread-contiguous pages straight from global memory
  // makes every warp-level load touch 32 different sectors, which the L1 cannot keep in flight.
  extern __shared__ float s_tile[];
  float* s_mu = s_tile;
  float* s_sg = s_tile + kGSelTile;
  for (int r0 = 0; r0 < n_stats; r0 += ROUND) {
    const int i0 = r0 + tid * KPT;
    {
      float lm[KPT], ls[KPT];
#pragma unroll
      for (int k = 0; k < KPT; ++k) {
        const int i = r0 + k * kGSelThreads + tid;
        const bool in = i < n_stats;
        lm[k] = in ? mu[i] : -INFINITY;     // pages past the end fail the threshold
        ls[k] = in ? sg[i] : 0.f;
      }
#pragma unroll
      for (int k = 0; k < KPT; ++k) {
        const int e = k * kGSelThreads + tid;
        s_mu[e + e / KPT] = lm[k];
        s_sg[e + e / KPT] = ls[k];
      }
    }
    __syncthreads();
    uint32_t bits = 0;
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
      const float m = s_mu[tid * (KPT + 1) + j], s = s_sg[tid * (KPT + 1) + j];
      if (a * (m + z_page * s) > tau_floor) {
        bits |= 1u << j;
        cap = fmaxf(cap, m + z_clamp * s * 0.3333333333333333f);
      }
    }
    uint32_t total;
    const uint32_t ex = block_scan_excl((uint32_t)__popc(bits), uscratch, &total);
    int pos = count + (int)ex;
#pragma unroll 4
    for (int j = 0; j < KPT; ++j)
      if ((bits >> j) & 1u) out[pos++] = i0 + j;
    count += (int)total;
    __syncthreads();
  }
  cap = block_max(cap, fscratch);
  if (tid == 0) {
    int n_sel = count;
    const bool has_last = append_last && n_pages > n_stats;
    if (has_last) {
      out[count] = n_pages - 1;
      n_sel = count + 1;
    } else if (append_last && n_pages == 1 && count == 0) {
      // single-page sequence whose only page failed the threshold: the reference
      // leaves the slot uninitialised; attend the page that exists
      out[0] = 0;
      n_sel = 1;
    }
    num_selected[bh] = n_sel;
    int T_tok;
    if (append_last) {
      const int last_size = S > P ? S - (n_pages - 1) * P : S;
      T_tok = max(n_sel - 1, 0) * P + last_size;
    } else {
      T_tok = n_sel * P;
    }
    tok_counts[bh] = T_tok;
    tau_floor_out[bh] = tau_floor;
    cap_out[bh] = cap;
    if (sx.use) {          // the world's cap: every rank clamps with the same number
      xe.send(bh, cap);
      cap = xe.max(bh, cap);
    }
    float t = tau_hat;
    if (apply_clamp && cap > -3.0e38f) t = fminf(t, fmaxf(a * cap - 1.0e-4f, tau_floor));
    tau_out[bh] = t;
    // chunk count of this head into the total of its tile of kWorkTile heads: integer adds commute,
    // so the totals - and the work-list layout derived from them - do not depend on block timing
    if (work_total) {
      const int nch = (min(T_tok, max_tokens) + kChunkTokens - 1) / kChunkTokens;
      if (nch > 0) atomicAdd(work_total + 1 + bh / kWorkTile, nch);
    }
  }
}

// grid: B*H_q blocks of 128 threads.  The work list of the decode: head h's chunks occupy the
// slots [sum_{h' < h} chunks(h'), ...) - offsets by head index, not by block timing, so the list,
// the way the K pass splits it between its persistent blocks and therefore every floating-point
// association downstream are the same from run to run.  The last head stores the total.
__global__ void __launch_bounds__(128)
gaussian_work_list_kernel(const int* __restrict__ tok_counts, int n_heads, int max_tokens,
                          unsigned long long* __restrict__ work_list, int* __restrict__ work_total) {
  __shared__ int s_part[4];
  const int bh = blockIdx.x, tid = threadIdx.x;
  // earlier tiles from their totals (work_total[1 + tile], filled by the selection kernel), earlier
  // heads of this tile from their own counts: O(heads / tile + tile) reads per head
  const int tile0 = bh / kWorkTile * kWorkTile;
  int before = 0;
  for (int t = tid; t < bh / kWorkTile; t += 128) before += work_total[1 + t];
  for (int i = tile0 + tid; i < bh; i += 128)
    before += (min(max(tok_counts[i], 0), max_tokens) + kChunkTokens - 1) / kChunkTokens;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
  if ((tid & 31) == 0) s_part[tid >> 5] = before;
  __syncthreads();
  const int base = s_part[0] + s_part[1] + s_part[2] + s_part[3];
  const int T_tok = min(max(tok_counts[bh], 0), max_tokens);
  const int nch = (T_tok + kChunkTokens - 1) / kChunkTokens;
  for (int i = tid; i < nch; i += 128) work_list[base + i] = make_item(bh, i, T_tok);
  if (bh == n_heads - 1 && tid == 0) *work_total = base + nch;
}

__global__ void tau_clamp_kernel(const float* __restrict__ tau_hat, int64_t stride,
                                 const float* __restrict__ cap, const float* __restrict__ tau_floor, int n,
                                 float a, float eps, float* __restrict__ tau) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float t = tau_hat[(size_t)i * stride];
  if (cap[i] > -3.0e38f) t = fminf(t, fmaxf(a * cap[i] - eps, tau_floor[i]));
  tau[i] = t;
}

// ---- sharded step: exchange + epilogue in one launch ---------------------------

// Slot 0: sum of every rank's per-head moment sums, then the per-head statistics and tau_hat
// (a warp per head; any grid).
__global__ void __launch_bounds__(kXchThreads)
xch_finalize_kernel(const XchDev x, const float* __restrict__ head_sums_local, const int* __restrict__ total_lens,
                    int page_size, int batch, int q_heads, float alpha, float* __restrict__ head_stats,
                    int* status) {
  const int n_heads = batch * q_heads;
  Xch e = xch_begin(x, 0, status);
  const int first = blockIdx.x * blockDim.x + threadIdx.x, stride = gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  // a warp sends the four sums of the heads it will finalize (lanes 0..3)
  for (int i = first >> 5; i < n_heads; i += stride >> 5)
    if (lane < 4) e.send(i * 4 + lane, head_sums_local[i * 4 + lane]);
  for (int i = first >> 5; i < n_heads; i += stride >> 5) {
    const int S = total_lens[i / q_heads];
    const int n_pages = (S + page_size - 1) / page_size;
    const int n_stat = n_pages > 1 ? n_pages - 1 : n_pages;
    const int n_tok = n_pages > 1 ? (n_pages - 1) * page_size : S;
    float mine = 0.f;
    if (lane < 4) mine = e.sum(i * 4 + lane, head_sums_local[i * 4 + lane]);
    float s[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) s[k] = __shfl_sync(0xffffffffu, mine, k);
    finalize_head_warp(s, (float)n_stat, (float)n_tok, alpha, head_stats + (size_t)i * 4);
  }
}

// Slot 1: max of every rank's clamp cap, then the clamp of tau (in place).
__global__ void __launch_bounds__(kXchThreads)
xch_tau_clamp_kernel(const XchDev x, float* __restrict__ tau, const float* __restrict__ cap_local,
                     const float* __restrict__ tau_floor, int n, float a, float eps, int* status) {
  Xch e = xch_begin(x, 1, status);
  for (int i = threadIdx.x; i < n; i += blockDim.x) e.send(i, cap_local[i]);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float cap = e.max(i, cap_local[i]);
    float t = tau[i];
    if (cap > -3.0e38f) t = fminf(t, fmaxf(a * cap - eps, tau_floor[i]));
    tau[i] = t;
  }
}

}  // namespace ekv

extern "C" int ekv_exchange_gaussian_finalize(ekv_exchange* x, const float* head_sums_local,
                                              const int32_t* total_lens, int32_t page_size, int32_t batch,
                                              int32_t q_heads, float alpha, float* head_stats,
                                              int32_t* status, void* stream) {
  using namespace ekv;
  XchDev d;
  if (!xch_device_view(x, &d) || !head_sums_local || !total_lens || !head_stats || !status || batch <= 0 ||
      q_heads <= 0 || page_size <= 0 || (int64_t)batch * q_heads * 4 > d.max_floats)
    return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  const int blocks = (batch * q_heads + 31) / 32;       // 32 warps per block, a warp per head
  xch_finalize_kernel<<<blocks, kXchThreads, 0, as_stream(stream)>>>(d, head_sums_local, total_lens, page_size, batch,
                                                               q_heads, alpha, head_stats, status);
  return launch_status();
}

extern "C" int ekv_exchange_tau_clamp(ekv_exchange* x, float* tau, const float* cap_local,
                                      const float* tau_floor, int32_t n, float alpha, float eps,
                                      int32_t* status, void* stream) {
  using namespace ekv;
  XchDev d;
  if (!xch_device_view(x, &d) || !tau || !cap_local || !tau_floor || !status || n <= 0 || n > d.max_floats)
    return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  xch_tau_clamp_kernel<<<1, kXchThreads, 0, as_stream(stream)>>>(d, tau, cap_local, tau_floor, n, alpha - 1.f, eps,
                                                                status);
  return launch_status();
}

extern "C" size_t ekv_gaussian_workspace_bytes(int32_t batch, int32_t q_heads, int32_t max_pages) {
  if (batch <= 0 || q_heads <= 0 || max_pages <= 0) return 0;
  return ekv::gaussian_ws_layout(batch, q_heads, max_pages, nullptr, nullptr);
}

static int gaussian_moments_launch(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                   int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len,
                                   int32_t exclude_last_page, float alpha, int32_t finalize,
                                   float* mu_pages, float* sigma_pages, int64_t page_stat_stride,
                                   float* head_sums, float* head_stats, void* workspace,
                                   size_t workspace_bytes, const float* alibi_slopes,
                                   const int32_t* q_positions, void* stream,
                                   const ekv::MomentsXch* mx = nullptr);
static bool moments_fuses_exchange(const ekv_cache_desc* c, int32_t q_heads);

extern "C" int ekv_gaussian_moments(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                    int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len,
                                    int32_t exclude_last_page, float alpha, int32_t finalize,
                                    float* mu_pages, float* sigma_pages, int64_t page_stat_stride,
                                    float* head_sums, float* head_stats, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  if (finalize != 0 && finalize != 1) return EKV_ERR_ARG;
  return gaussian_moments_launch(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, exclude_last_page, alpha,
                                 finalize, mu_pages, sigma_pages, page_stat_stride, head_sums, head_stats,
                                 workspace, workspace_bytes, nullptr, nullptr, stream);
}

extern "C" int ekv_exchange_gaussian_moments(ekv_exchange* x, const ekv_cache_desc* c, const void* q,
                                             int64_t q_stride_b, int64_t q_stride_h, int32_t q_heads,
                                             int32_t max_seq_len, int32_t exclude_last_page, float alpha,
                                             const int32_t* total_lens, float* mu_pages, float* sigma_pages,
                                             int64_t page_stat_stride, float* head_sums, float* head_stats,
                                             void* workspace, size_t workspace_bytes, int32_t* status,
                                             void* stream) {
  using namespace ekv;
  MomentsXch mx{};
  if (!c || !xch_device_view(x, &mx.xch) || !total_lens || !head_stats || !status ||
      (int64_t)c->batch * q_heads * 4 > mx.xch.max_floats)
    return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  if (c->kv_heads > 0 && q_heads > 0 && moments_fuses_exchange(c, q_heads)) {
    mx.use = 1;
    mx.status = status;
    mx.total_lens = total_lens;
    return gaussian_moments_launch(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, exclude_last_page, alpha, 0,
                                   mu_pages, sigma_pages, page_stat_stride, head_sums, head_stats, workspace,
                                   workspace_bytes, nullptr, nullptr, stream, &mx);
  }
  if (int e = gaussian_moments_launch(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, exclude_last_page, alpha, 0,
                                      mu_pages, sigma_pages, page_stat_stride, head_sums, head_stats, workspace,
                                      workspace_bytes, nullptr, nullptr, stream))
    return e;
  return ekv_exchange_gaussian_finalize(x, head_sums, total_lens, c->page_size, c->batch, q_heads, alpha, head_stats,
                                        status, stream);
}

extern "C" int ekv_gaussian_moments_alibi(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                          int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len,
                                          int32_t exclude_last_page, float alpha, float* mu_pages,
                                          float* sigma_pages, int64_t page_stat_stride, float* head_sums,
                                          float* head_stats, void* workspace, size_t workspace_bytes,
                                          const float* alibi_slopes, const int32_t* q_positions,
                                          void* stream) {
  using namespace ekv;
  if (!alibi_slopes || !head_stats) return EKV_ERR_ARG;
  // the page-mixture solver has closed forms for alpha 2, 1.5 and 4/3 only
  if (alpha_kind_of(alpha) == 2 && !alpha_is_four_thirds(alpha)) return EKV_ERR_ALPHA;
  // statistics without tau_hat, then the page-mixture root over the biased page means
  if (int e = gaussian_moments_launch(c, q, q_stride_b, q_stride_h, q_heads, max_seq_len, exclude_last_page,
                                      alpha, 2, mu_pages, sigma_pages, page_stat_stride, head_sums, head_stats,
                                      workspace, workspace_bytes, alibi_slopes, q_positions, stream))
    return e;
  gaussian_mixture_tau_kernel<<<c->batch * q_heads, kMixThreads, 0, as_stream(stream)>>>(
      *c, q_heads, exclude_last_page, alpha, mu_pages, sigma_pages, page_stat_stride, head_stats);
  return launch_status();
}

// EKV_MOMENTS_MMA=0 in the environment keeps the CUDA-core sweep for bfloat caches too (comparison runs).
static bool moments_mma_enabled() {
  static const bool on = [] {
    const char* e = getenv("EKV_MOMENTS_MMA");
    return !(e && e[0] == '0');
  }();
  return on;
}

// The tensor-core sweep (bfloat caches, groups of up to eight heads) can carry the sharded step's first
// exchange in its last blocks; other caches trade the sums in a launch of their own.
static bool moments_fuses_exchange(const ekv_cache_desc* c, int32_t q_heads) {
  return c->dtype == EKV_BF16 && q_heads / c->kv_heads <= 8 && moments_mma_enabled();
}

static int gaussian_moments_launch(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                   int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len,
                                   int32_t exclude_last_page, float alpha, int32_t finalize,
                                   float* mu_pages, float* sigma_pages, int64_t page_stat_stride,
                                   float* head_sums, float* head_stats, void* workspace,
                                   size_t workspace_bytes, const float* alibi_slopes,
                                   const int32_t* q_positions, void* stream, const ekv::MomentsXch* mx) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!q || !mu_pages || !sigma_pages || !head_sums || !workspace) return EKV_ERR_ARG;
  if (finalize && !head_stats) return EKV_ERR_ARG;
  if (!c->k_mean || !c->k_std) return EKV_ERR_ARG;
  if (q_heads <= 0 || q_heads % c->kv_heads || max_seq_len <= 0) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  const int max_pages = (max_seq_len + c->page_size - 1) / c->page_size;
  if (page_stat_stride < max_pages - (exclude_last_page && max_pages > 1 ? 1 : 0)) return EKV_ERR_ARG;
  GaussianWs ws;
  if (gaussian_ws_layout(c->batch, q_heads, max_pages, workspace, &ws) > workspace_bytes)
    return EKV_ERR_WORKSPACE;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((q_stride_b * esz) % 16 || (q_stride_h * esz) % 16 || (reinterpret_cast<uintptr_t>(q) & 15))
    return EKV_ERR_ARG;
  const int G = q_heads / c->kv_heads;
  cudaStream_t st = as_stream(stream);
  MomentsXch no_xch{};
  const MomentsXch& mxa = mx ? *mx : no_xch;
  if (mx && !moments_fuses_exchange(c, q_heads)) return EKV_ERR_ARG;   // the caller checks before it asks
  if (c->dtype == EKV_BF16 && G <= 8 && moments_mma_enabled()) {
    // tensor-core sweep: 128-thread blocks (four warps, 64-page tiles, two-stage ring), three per SM; a deeper
    // ring of smaller tiles measured slower (every tile costs a block-wide barrier)
    constexpr int kW = 4;      // (a third stage at two blocks per SM measured slower: 205 -> 250 us at 128k)
    const int bhk = c->batch * c->kv_heads;
    const int blocks4 = (ws.tiles + 3) / 4 * bhk, wave = 3 * sm_count();
    const long long blocks8 = (long long)((ws.tiles + 7) / 8) * bhk;
    ws.tpb = blocks8 >= 8LL * wave ? 8 : (blocks4 >= 4 * wave ? 4 : (blocks4 >= wave ? 2 : 1));
    dim3 grid((unsigned)((ws.tiles + ws.tpb - 1) / ws.tpb), (unsigned)bhk);
    const __nv_bfloat16* qq = static_cast<const __nv_bfloat16*>(q);
#define EKV_LAUNCH_MMA2(DD, AL, kNS, kBPS)                                                                      \
    do {                                                                                                          \
      using ML = MomMma<DD, kW, kNS>;                                                                             \
      auto kernel = gaussian_moments_mma_kernel<DD, AL, kW, kNS, kBPS>;                                           \
      static bool once = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,                \
                                              (int)ML::kSmem) == cudaSuccess;                                     \
      (void)once;                                                                                                 \
      kernel<<<grid, ML::kThreads, ML::kSmem, st>>>(                                                              \
          *c, qq, q_stride_b, q_stride_h, q_heads, exclude_last_page, alpha, finalize, mu_pages, sigma_pages,     \
          page_stat_stride, head_sums, head_stats, ws, alibi_slopes, q_positions, mxa);                           \
    } while (0)
#define EKV_LAUNCH_MMA(DD, AL) EKV_LAUNCH_MMA2(DD, AL, 2, 3)
    if (c->head_dim == 128) {
      if (alibi_slopes) EKV_LAUNCH_MMA(128, true); else EKV_LAUNCH_MMA(128, false);
    } else {
      if (alibi_slopes) EKV_LAUNCH_MMA(64, true); else EKV_LAUNCH_MMA(64, false);
    }
#undef EKV_LAUNCH_MMA
#undef EKV_LAUNCH_MMA2
    return launch_status();
  }
  EKV_DISPATCH(c->dtype, c->head_dim, {
    // one page is handled by ceil(G/HPL) lane groups of a 256-thread block
    const int hpl = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
    if ((G + hpl - 1) / hpl > kMomThreads / (D / ElemTraits<T>::EPL) || G * 4 > kMomThreads) return EKV_ERR_ARG;
    // four tiles per block amortise a block's start-up; with few pages (one shard of a
    // sequence-sharded request) fewer tiles per block keep every SM busy
    const int bhk = c->batch * c->kv_heads;
    const int blocks4 = (ws.tiles + 3) / 4 * bhk, wave = 3 * sm_count();
    const long long blocks8 = (long long)((ws.tiles + 7) / 8) * bhk;
    ws.tpb = blocks8 >= 8LL * wave ? 8 : (blocks4 >= 4 * wave ? 4 : (blocks4 >= wave ? 2 : 1));
    dim3 grid((unsigned)((ws.tiles + ws.tpb - 1) / ws.tpb), (unsigned)bhk);
    const T* qq = static_cast<const T*>(q);
    const size_t smem = 4 * (size_t)kMomPagesPerBlock * D * sizeof(T);   // 2 stages x (mean, std)
    if (hpl == 4) {
      if (alibi_slopes) {
        static bool once = cudaFuncSetAttribute(gaussian_moments_kernel<T, D, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        (void)once;
        gaussian_moments_kernel<T, D, 4, true><<<grid, kMomThreads, smem, st>>>(
            *c, qq, q_stride_b, q_stride_h, q_heads, exclude_last_page, alpha, finalize, mu_pages,
            sigma_pages, page_stat_stride, head_sums, head_stats, ws, alibi_slopes, q_positions);
      } else {
        static bool once = cudaFuncSetAttribute(gaussian_moments_kernel<T, D, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        (void)once;
        gaussian_moments_kernel<T, D, 4, false><<<grid, kMomThreads, smem, st>>>(
            *c, qq, q_stride_b, q_stride_h, q_heads, exclude_last_page, alpha, finalize, mu_pages,
            sigma_pages, page_stat_stride, head_sums, head_stats, ws, nullptr, nullptr);
      }
    } else if (hpl == 2) {
      if (alibi_slopes) {
        static bool once = cudaFuncSetAttribute(gaussian_moments_kernel<T, D, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        (void)once;
        gaussian_moments_kernel<T, D, 2, true><<<grid, kMomThreads, smem, st>>>(
            *c, qq, q_stride_b, q_stride_h, q_heads, exclude_last_page, alpha, finalize, mu_pages,
            sigma_pages, page_stat_stride, head_sums, head_stats, ws, alibi_slopes, q_positions);
      } else {
        static bool once = cudaFuncSetAttribute(gaussian_moments_kernel<T, D, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        (void)once;
        gaussian_moments_kernel<T, D, 2, false><<<grid, kMomThreads, smem, st>>>(
            *c, qq, q_stride_b, q_stride_h, q_heads, exclude_last_page, alpha, finalize, mu_pages,
            sigma_pages, page_stat_stride, head_sums, head_stats, ws, nullptr, nullptr);
      }
    } else {
      if (alibi_slopes) {
        static bool once = cudaFuncSetAttribute(gaussian_moments_kernel<T, D, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        (void)once;
        gaussian_moments_kernel<T, D, 1, true><<<grid, kMomThreads, smem, st>>>(
            *c, qq, q_stride_b, q_stride_h, q_heads, exclude_last_page, alpha, finalize, mu_pages,
            sigma_pages, page_stat_stride, head_sums, head_stats, ws, alibi_slopes, q_positions);
      } else {
        static bool once = cudaFuncSetAttribute(gaussian_moments_kernel<T, D, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        (void)once;
        gaussian_moments_kernel<T, D, 1, false><<<grid, kMomThreads, smem, st>>>(
            *c, qq, q_stride_b, q_stride_h, q_heads, exclude_last_page, alpha, finalize, mu_pages,
            sigma_pages, page_stat_stride, head_sums, head_stats, ws, nullptr, nullptr);
      }
    }
  });
  return launch_status();
}

extern "C" int ekv_gaussian_finalize(const float* head_sums, const int32_t* n_pages,
                                     const int32_t* n_tokens, int32_t batch, int32_t q_heads,
                                     float alpha, float* head_stats, void* stream) {
  using namespace ekv;
  if (!head_sums || !n_pages || !n_tokens || !head_stats || batch <= 0 || q_heads <= 0) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  const int n = batch * q_heads;
  gaussian_finalize_kernel<<<(n + 3) / 4, 128, 0, as_stream(stream)>>>(head_sums, n_pages, n_tokens,
                                                                          batch, q_heads, alpha, head_stats);
  return launch_status();
}

extern "C" int ekv_gaussian_finalize_from_lengths(const float* head_sums, const int32_t* total_lens,
                                                  int32_t page_size, int32_t batch, int32_t q_heads,
                                                  float alpha, float* head_stats, void* stream) {
  using namespace ekv;
  if (!head_sums || !total_lens || !head_stats || batch <= 0 || q_heads <= 0 || page_size <= 0) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  const int n = batch * q_heads;
  gaussian_finalize_lens_kernel<<<(n + 3) / 4, 128, 0, as_stream(stream)>>>(head_sums, total_lens, page_size,
                                                                               batch, q_heads, alpha, head_stats);
  return launch_status();
}

static int gaussian_select_launch(const ekv_cache_desc* c, int32_t q_heads, int32_t max_seq_len,
                                  int32_t exclude_last_page, int32_t append_last_page, float alpha,
                                  float excess_margin_fraction, float z_page_low, float z_page_high,
                                  float z_clamp, int32_t apply_clamp, const float* sigma_mean,
                                  const float* mu_pages, const float* sigma_pages,
                                  int64_t page_stat_stride, const float* head_stats,
                                  int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                                  int32_t* tok_counts, float* tau_floor, float* cap_max, float* tau,
                                  uint64_t* work_items, int32_t* work_total, const ekv::SelectXch& sx,
                                  void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!mu_pages || !sigma_pages || !head_stats || !page_indices || !num_selected || !tok_counts ||
      !tau_floor || !cap_max || !tau)
    return EKV_ERR_ARG;
  if (q_heads <= 0 || q_heads % c->kv_heads || max_seq_len <= 0) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  if ((work_items == nullptr) != (work_total == nullptr)) return EKV_ERR_ARG;
  const int max_pages = (max_seq_len + c->page_size - 1) / c->page_size;
  if (pi_stride < max_pages) return EKV_ERR_ARG;
  if ((int64_t)c->batch * q_heads >= kItemMaxHeads) return EKV_ERR_ARG;
  cudaStream_t st = as_stream(stream);
  const int n_blocks = c->batch * q_heads;
  if (work_total) {
    const size_t n_tiles = ((size_t)c->batch * q_heads + kWorkTile - 1) / kWorkTile;
    cudaError_t e = cudaMemsetAsync(work_total, 0, (1 + n_tiles) * sizeof(int32_t), st);
    if (e != cudaSuccess) return (int)e;
  }
  static bool once = cudaFuncSetAttribute(gaussian_select_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)GSel<16>::kSmem) == cudaSuccess &&
                     cudaFuncSetAttribute(gaussian_select_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)GSel<8>::kSmem) == cudaSuccess;
  (void)once;
  if (n_blocks >= 4 * sm_count())      // two waves of the large-round variant: smaller rounds overlap better
    gaussian_select_kernel<8><<<n_blocks, kGSelThreads, GSel<8>::kSmem, st>>>(
        *c, q_heads, exclude_last_page, append_last_page, alpha, excess_margin_fraction, z_page_low,
        z_page_high, z_clamp, apply_clamp, sigma_mean, mu_pages, sigma_pages, page_stat_stride,
        head_stats, page_indices, pi_stride, num_selected, tok_counts, tau_floor, cap_max, tau,
        reinterpret_cast<unsigned long long*>(work_items), work_total, max_seq_len, sx);
  else
    gaussian_select_kernel<16><<<n_blocks, kGSelThreads, GSel<16>::kSmem, st>>>(
        *c, q_heads, exclude_last_page, append_last_page, alpha, excess_margin_fraction, z_page_low,
        z_page_high, z_clamp, apply_clamp, sigma_mean, mu_pages, sigma_pages, page_stat_stride,
        head_stats, page_indices, pi_stride, num_selected, tok_counts, tau_floor, cap_max, tau,
        reinterpret_cast<unsigned long long*>(work_items), work_total, max_seq_len, sx);
  if (work_items)
    gaussian_work_list_kernel<<<c->batch * q_heads, 128, 0, st>>>(
        tok_counts, c->batch * q_heads, max_seq_len, reinterpret_cast<unsigned long long*>(work_items),
        work_total);
  return launch_status();
}

extern "C" int ekv_gaussian_select(const ekv_cache_desc* c, int32_t q_heads, int32_t max_seq_len,
                                   int32_t exclude_last_page, int32_t append_last_page, float alpha,
                                   float excess_margin_fraction, float z_page_low, float z_page_high,
                                   float z_clamp, int32_t apply_clamp, const float* sigma_mean,
                                   const float* mu_pages, const float* sigma_pages,
                                   int64_t page_stat_stride, const float* head_stats,
                                   int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                                   int32_t* tok_counts, float* tau_floor, float* cap_max, float* tau,
                                   uint64_t* work_items, int32_t* work_total, void* stream) {
  return gaussian_select_launch(c, q_heads, max_seq_len, exclude_last_page, append_last_page, alpha,
                                excess_margin_fraction, z_page_low, z_page_high, z_clamp, apply_clamp, sigma_mean,
                                mu_pages, sigma_pages, page_stat_stride, head_stats, page_indices, pi_stride,
                                num_selected, tok_counts, tau_floor, cap_max, tau, work_items, work_total,
                                ekv::SelectXch{}, stream);
}

extern "C" int ekv_exchange_gaussian_select(ekv_exchange* x, const ekv_cache_desc* c, int32_t q_heads,
                                            int32_t max_seq_len, int32_t exclude_last_page,
                                            int32_t append_last_page, float alpha, float excess_margin_fraction,
                                            float z_page_low, float z_page_high, float z_clamp,
                                            int32_t apply_clamp, const float* sigma_mean, const float* mu_pages,
                                            const float* sigma_pages, int64_t page_stat_stride,
                                            const float* head_stats, int32_t* page_indices, int64_t pi_stride,
                                            int32_t* num_selected, int32_t* tok_counts, float* tau_floor,
                                            float* cap_max, float* tau, uint64_t* work_items,
                                            int32_t* work_total, int32_t* status, void* stream) {
  ekv::SelectXch sx{};
  if (!c || !ekv::xch_device_view(x, &sx.xch) || !status || (int64_t)c->batch * q_heads > sx.xch.max_floats)
    return EKV_ERR_ARG;
  sx.use = 1;
  sx.status = status;
  return gaussian_select_launch(c, q_heads, max_seq_len, exclude_last_page, append_last_page, alpha,
                                excess_margin_fraction, z_page_low, z_page_high, z_clamp, apply_clamp, sigma_mean,
                                mu_pages, sigma_pages, page_stat_stride, head_stats, page_indices, pi_stride,
                                num_selected, tok_counts, tau_floor, cap_max, tau, work_items, work_total, sx,
                                stream);
}

extern "C" int ekv_tau_clamp(const float* tau_hat, int64_t tau_hat_stride, const float* cap_max,
                             const float* tau_floor, int32_t n, float alpha, float eps, float* tau,
                             void* stream) {
  using namespace ekv;
  if (!tau_hat || !cap_max || !tau_floor || !tau || n <= 0 || tau_hat_stride <= 0) return EKV_ERR_ARG;
  tau_clamp_kernel<<<(n + 127) / 128, 128, 0, as_stream(stream)>>>(tau_hat, tau_hat_stride, cap_max,
                                                                   tau_floor, n, alpha - 1.f, eps, tau);
  return launch_status();
}

namespace ekv {
unsigned int copy_timeouts_gaussian() { return copy_timeouts_here(); }
}  // namespace ekv
