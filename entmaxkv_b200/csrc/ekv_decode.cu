// Paged entmax decode over the selected pages, in two passes:
//
//   K pass  (decode_scores_kernel): every selected key row is read ONCE; its score
//           z = (alpha-1)/sqrt(D) * q.k is kept (4 bytes per token) in the workspace
//           together with per-chunk maxima / Halley sums.  The last thread block to
//           finish a head solves tau from the kept scores - so the histogram, the
//           bracket and all Halley iterations re-read 4-byte scores from L2, never K.
//   V pass  (decode_values_kernel): only rows whose weight (z-tau)_+^beta is non-zero
//           are read from V; partial outputs are summed per head in chunk order by
//           the last thread block to finish the head.
//
// Work is cut into chunks of 256 compacted tokens.  With a uniform token count the
// grid is (chunks, heads); with data-dependent counts (Gaussian selection) the
// blocks walk a device-built list of (head, chunk) items instead.
// Both passes are HBM-bound: 2*D*sizeof(T) bytes per selected token in total.
#include "ekv_common.cuh"

namespace ekv {

constexpr int kDecThreads = 256;
constexpr int kWorkChunkBits = 13;
constexpr int kStatusInts = 16;

struct DecodeWs {
  int* status;      // [16]; word 0 = status bits
  int* cnt_k;       // [BH]
  int* cnt_v;       // [BH]
  float* z;         // [BH, zstride]
  float* part;      // [BH, nchunks, 4] = {s0, s1, s2, max}
  int* nz;          // [BH, nchunks]
  float* pout;      // [BH, nchunks, D]
  int64_t zstride;
  int nchunks;
};

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

inline size_t decode_ws_layout(int batch, int q_heads, int head_dim, int max_tokens, void* base, DecodeWs* ws) {
  const size_t BH = (size_t)batch * q_heads;
  const int nchunks = (max_tokens + kChunkTokens - 1) / kChunkTokens;
  const size_t zstride = (size_t)nchunks * kChunkTokens;
  size_t off = 0;
  char* p = static_cast<char*>(base);
  auto take = [&](size_t bytes) {
    char* r = p + off;
    off += align256(bytes);
    return r;
  };
  char* st = take(kStatusInts * sizeof(int));
  char* ck = take(BH * sizeof(int));
  char* cv = take(BH * sizeof(int));
  char* z = take(BH * zstride * sizeof(float));
  char* part = take(BH * nchunks * 4 * sizeof(float));
  char* nz = take(BH * nchunks * sizeof(int));
  char* pout = take(BH * nchunks * head_dim * sizeof(float));
  if (ws) {
    ws->status = reinterpret_cast<int*>(st);
    ws->cnt_k = reinterpret_cast<int*>(ck);
    ws->cnt_v = reinterpret_cast<int*>(cv);
    ws->z = reinterpret_cast<float*>(z);
    ws->part = reinterpret_cast<float*>(part);
    ws->nz = reinterpret_cast<int*>(nz);
    ws->pout = reinterpret_cast<float*>(pout);
    ws->zstride = (int64_t)zstride;
    ws->nchunks = nchunks;
  }
  return off;
}

inline size_t decode_ws_header_bytes(int batch, int q_heads) {
  return align256(kStatusInts * sizeof(int)) + 2 * align256((size_t)batch * q_heads * sizeof(int));
}

struct PageDiv {   // c -> (c / P, c % P); shift/mask when P is a power of two
  int P, shift;
  __device__ __forceinline__ void split(int c, int& pg, int& off) const {
    if (shift >= 0) {
      pg = c >> shift;
      off = c & (P - 1);
    } else {
      pg = c / P;
      off = c - pg * P;
    }
  }
};

// ---- tau from kept scores (runs in the last block of a head) ------------------

// Bracket [t_lo, t_hi] from the 16-bin histogram of z on [max-1, max].
__device__ void bracket_from_hist(const int* hist, float zmax, float alpha, int kind, float& t_lo, float& t_hi) {
  if (kind != 2) {
    float sz = 1.f, sk = 1.f, sz2 = 1.f;
    for (int sj = kBins - 1; sj >= 0; --sj) {
      const float cnt = (float)hist[sj] - (sj == kBins - 1 ? 1.f : 0.f);
      const float ct = (float)sj / (float)kBins;
      const float nz = sz + cnt * ct, nk = sk + cnt, nz2 = sz2 + cnt * (ct * ct);
      const bool ok = kind == 0 ? (nz - nk * ct) < 1.f : (nk * ct * ct - 2.f * nz * ct + nz2) < 1.f;
      if (ok) {
        sz = nz;
        sk = nk;
        sz2 = nz2;
      }
    }
    float t_init;
    if (kind == 0) {
      t_init = zmax + (sz - 1.f) / sk - 1.f;
    } else {
      const float disc = sz * sz - sk * (sz2 - 1.f);
      t_init = zmax + (sz - sqrtf(disc)) / sk - 1.f;
    }
    t_lo = t_init;
    t_hi = t_init + 1.f / (float)kBins;
    return;
  }
  // general alpha: binary search for the bin whose edges bracket the root
  const float p = 1.f / (alpha - 1.f);
  int lo = 0, hi = kBins - 1, found = 0, b_idx = 0;
  for (int it = 0; it < 5; ++it) {
    const int mid = (int)((float)(lo + hi) * 0.5f);
    float fL = -1.f, fU = -1.f;
    for (int bin = 0; bin < kBins; ++bin) {
      const int off = bin - mid;
      if (off < 0) continue;
      const float cnt = (float)hist[bin] - (bin == kBins - 1 ? 1.f : 0.f);
      const float zL = (float)off / (float)kBins, zU = ((float)off + 1.f) / (float)kBins;
      if (zL > 0.f) fL += cnt * pow_pos(zL, p);
      fU += cnt * pow_pos(zU, p);
    }
    const bool go_right = fL > 0.f, go_left = fU < 0.f;
    if (!found) {
      if (!go_right && !go_left) {
        b_idx = mid;
        found = 1;
      }
      if (go_right) lo = mid + 1;
      if (go_left) hi = mid - 1;
    }
  }
  const int b_sel = found ? b_idx : min(lo, kBins - 1);
  const float t0 = zmax - 1.f;
  t_lo = t0 + (float)b_sel / (float)kBins;
  t_hi = t0 + (float)min(b_sel + 1, kBins) / (float)kBins;
}

__device__ __forceinline__ void halley_bracketed(float& t, float& t_lo, float& t_hi, float s0, float s1,
                                                 float s2, float beta) {
  const float ff = s0 - 1.f;
  const float df = -beta * s1;
  const float ddf = beta * (beta - 1.f) * s2;
  if (ff > 0.f) t_lo = t;
  if (ff < 0.f) t_hi = t;
  const float nt = t - (2.f * ff * df) / (2.f * df * df - ff * ddf);
  const bool good = (nt > t_lo - 1e-6f) && (nt < t_hi + 1e-6f);
  t = good ? nt : 0.5f * (t_lo + t_hi);
}

// Block-wide Halley sums over the kept scores of one head (fixed order).
__device__ void sums_over_scores(const float* z, int n, float tau, int kind, float beta, float* scratch,
                                 float& s0, float& s1, float& s2) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) halley_accumulate(ld_cg(z + i), tau, kind, beta, a0, a1, a2);
  s0 = block_sum(a0, scratch);
  s1 = block_sum(a1, scratch);
  s2 = block_sum(a2, scratch);
}

__device__ void solve_head_tau(const DecodeWs& ws, int bh, int T_tok, int nch, float alpha, int tau_mode,
                               int niter, float* tau, float* halley_sums) {
  __shared__ float scratch[32];
  __shared__ int hist[kBins];
  __shared__ float s_t;
  const int kind = alpha_kind_of(alpha);
  const float beta = 1.f / (alpha - 1.f);
  const float* z = ws.z + (size_t)bh * ws.zstride;
  const float* part = ws.part + (size_t)bh * ws.nchunks * 4;
  const int tid = threadIdx.x;

  if (tau_mode == EKV_TAU_EXACT) {
    float m = -1.0e6f;
    for (int i = tid; i < nch; i += blockDim.x) m = fmaxf(m, ld_cg(part + i * 4 + 3));
    m = block_max(m, scratch);
    if (tid < kBins) hist[tid] = 0;
    __syncthreads();
    const float t0 = m - 1.f;
    for (int i = tid; i < T_tok; i += blockDim.x) {
      const float proj = (ld_cg(z + i) - t0) * (float)kBins;
      const int bin = min((int)proj, kBins - 1);   // conversion truncates toward zero
      if (bin >= 0) atomicAdd(&hist[bin], 1);
    }
    __syncthreads();
    float t = 0.f, t_lo = 0.f, t_hi = 0.f;
    if (tid == 0) {
      bracket_from_hist(hist, m, alpha, kind, t_lo, t_hi);
      t = 0.5f * (t_lo + t_hi);
      s_t = t;
    }
    __syncthreads();
    for (int it = 0; it < niter; ++it) {
      float s0, s1, s2;
      sums_over_scores(z, T_tok, s_t, kind, beta, scratch, s0, s1, s2);
      __syncthreads();
      if (tid == 0) {
        halley_bracketed(t, t_lo, t_hi, s0, s1, s2, beta);
        s_t = t;
      }
      __syncthreads();
    }
    if (tid == 0) tau[bh] = s_t;
    return;
  }

  // sums at the incoming tau were accumulated by the K pass, one triple per chunk
  float a0 = 0.f, a1 = 0.f, a2 = 0.f;
  for (int i = tid; i < nch; i += blockDim.x) {
    a0 += ld_cg(part + i * 4 + 0);
    a1 += ld_cg(part + i * 4 + 1);
    a2 += ld_cg(part + i * 4 + 2);
  }
  float s0 = block_sum(a0, scratch), s1 = block_sum(a1, scratch), s2 = block_sum(a2, scratch);
  if (halley_sums && tid == 0) {
    halley_sums[(size_t)bh * 3 + 0] = s0;
    halley_sums[(size_t)bh * 3 + 1] = s1;
    halley_sums[(size_t)bh * 3 + 2] = s2;
  }
  if (tau_mode != EKV_TAU_CORRECTED || niter <= 0) return;
  float t = tau[bh];
  for (int it = 0; it < niter; ++it) {
    if (it > 0) {
      __syncthreads();
      sums_over_scores(z, T_tok, t, kind, beta, scratch, s0, s1, s2);
    }
    t = halley_unbounded(t, s0, s1, s2, beta);   // every thread computes the same value
  }
  if (tid == 0) tau[bh] = t;
}

// ---- K pass --------------------------------------------------------------------

template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads)
decode_scores_kernel(ekv_cache_desc c, const T* __restrict__ q, int64_t qsb, int64_t qsh, int q_heads,
                     const int* __restrict__ page_indices, int64_t pi_stride,
                     const int* __restrict__ tok_counts, int max_tokens, float alpha, int tau_mode,
                     int niter, float* tau, float* halley_sums, const uint32_t* __restrict__ work_list,
                     const int* __restrict__ work_total, DecodeWs ws, PageDiv pd) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kDecThreads / LPR;
  constexpr int U = 4;
  __shared__ float red[GROUPS][4];
  __shared__ int s_ticket;

  const int kind = alpha_kind_of(alpha);
  const float beta = 1.f / (alpha - 1.f);
  const float qscale = (alpha - 1.f) * (D == 64 ? 0.125f : 0.08838834764831845f);
  const int lane_in_row = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int G = q_heads / c.kv_heads;

  const int n_items = work_list ? *work_total : (int)(gridDim.x * gridDim.y);
  const int first = work_list ? (int)blockIdx.x : (int)(blockIdx.y * gridDim.x + blockIdx.x);
  const int step = work_list ? (int)gridDim.x : n_items;
  for (int w = first; w < n_items; w += step) {
    int bh, chunk;
    if (work_list) {
      const uint32_t item = work_list[w];
      bh = (int)(item >> kWorkChunkBits);
      chunk = (int)(item & ((1u << kWorkChunkBits) - 1));
    } else {
      bh = blockIdx.y;
      chunk = blockIdx.x;
    }
    int T_tok = tok_counts[bh];
    if (T_tok > max_tokens) {
      if (threadIdx.x == 0 && chunk == 0) atomicOr(ws.status, EKV_STATUS_TOKENS);
      T_tok = max_tokens;
    }
    const int c0 = chunk * kChunkTokens;
    if (c0 >= T_tok) continue;
    const int nch = (T_tok + kChunkTokens - 1) / kChunkTokens;
    const int ntok = min(kChunkTokens, T_tok - c0);
    const int b = bh / q_heads, hq = bh % q_heads, hkv = hq / G;

    float qs[EPL];
    unpack<T>(*reinterpret_cast<const uint4*>(q + b * qsb + hq * qsh + lane_in_row * EPL), qs);
#pragma unroll
    for (int j = 0; j < EPL; ++j) qs[j] *= qscale;
    const float tau0 = tau_mode == EKV_TAU_EXACT ? 0.f : tau[bh];
    const T* kbase = static_cast<const T*>(c.k) + b * c.kv_stride_b + hkv * c.kv_stride_h + lane_in_row * EPL;
    const int* pi = page_indices + (size_t)bh * pi_stride;
    float* zrow = ws.z + (size_t)bh * ws.zstride + c0;

    float s0 = 0.f, s1 = 0.f, s2 = 0.f, mx = -1.0e6f;
    // the loop bound is uniform over the block: the row_sum shuffles below need every
    // lane of a warp, also when only some of its lane groups still own a token
    for (int i0 = 0; i0 < ntok; i0 += GROUPS * U) {
      const int i = i0 + group;
      uint4 r[U];
      bool ok[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int ci = i + u * GROUPS;
        ok[u] = ci < ntok;
        r[u] = make_uint4(0, 0, 0, 0);
        if (ok[u]) {
          int pg, off;
          pd.split(c0 + ci, pg, off);
          const int page = pi[pg];
          if ((unsigned)page < (unsigned)c.page_capacity) {
            r[u] = ld_stream(kbase + ((size_t)page * pd.P + off) * D);
          } else if (lane_in_row == 0) {
            atomicOr(ws.status, EKV_STATUS_PAGE_RANGE);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float kf[EPL];
        unpack<T>(r[u], kf);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc = fmaf(qs[j], kf[j], acc);
        acc = row_sum<LPR>(acc);
        if (ok[u] && lane_in_row == 0) {
          zrow[i + u * GROUPS] = acc;
          mx = fmaxf(mx, acc);
          if (tau_mode != EKV_TAU_EXACT) halley_accumulate(acc, tau0, kind, beta, s0, s1, s2);
        }
      }
    }
    __syncthreads();   // red[] / s_ticket of the previous item are no longer read
    if (lane_in_row == 0) {
      red[group][0] = s0;
      red[group][1] = s1;
      red[group][2] = s2;
      red[group][3] = mx;
    }
    __syncthreads();
    if (threadIdx.x < 4) {
      float t = red[0][threadIdx.x];
      for (int g = 1; g < GROUPS; ++g) t = threadIdx.x == 3 ? fmaxf(t, red[g][3]) : t + red[g][threadIdx.x];
      ws.part[((size_t)bh * ws.nchunks + chunk) * 4 + threadIdx.x] = t;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(&ws.cnt_k[bh], 1);
    __syncthreads();
    if (s_ticket == nch - 1) {
      __threadfence();
      solve_head_tau(ws, bh, T_tok, nch, alpha, tau_mode, niter, tau, halley_sums);
      if (threadIdx.x == 0) ws.cnt_k[bh] = 0;
    }
  }
}

// Same pass with the chunk's pages staged in shared memory: every page of the chunk is
// one contiguous P*D*sizeof(T)-byte block of K, fetched by one bulk asynchronous copy
// (up to 256/P copies in flight per block, several blocks per SM), and scored from
// shared memory.  Needs a power-of-two page size that divides the 256-token chunk.
template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads)
decode_scores_bulk_kernel(ekv_cache_desc c, const T* __restrict__ q, int64_t qsb, int64_t qsh, int q_heads,
                          const int* __restrict__ page_indices, int64_t pi_stride,
                          const int* __restrict__ tok_counts, int max_tokens, float alpha, int tau_mode,
                          int niter, float* tau, float* halley_sums, const uint32_t* __restrict__ work_list,
                          const int* __restrict__ work_total, DecodeWs ws, PageDiv pd) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kDecThreads / LPR;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* s_k = reinterpret_cast<T*>(smem_raw);
  __shared__ uint64_t bar;
  __shared__ float red[GROUPS][4];
  __shared__ int s_ticket;

  const int kind = alpha_kind_of(alpha);
  const float beta = 1.f / (alpha - 1.f);
  const float qscale = (alpha - 1.f) * (D == 64 ? 0.125f : 0.08838834764831845f);
  const int tid = threadIdx.x;
  const int lane_in_row = tid % LPR;
  const int group = tid / LPR;
  const int G = q_heads / c.kv_heads;
  const int P = pd.P;

  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  uint32_t phase = 0;

  const int n_items = work_list ? *work_total : (int)(gridDim.x * gridDim.y);
  const int first = work_list ? (int)blockIdx.x : (int)(blockIdx.y * gridDim.x + blockIdx.x);
  const int step = work_list ? (int)gridDim.x : n_items;
  for (int w = first; w < n_items; w += step) {
    int bh, chunk;
    if (work_list) {
      const uint32_t item = work_list[w];
      bh = (int)(item >> kWorkChunkBits);
      chunk = (int)(item & ((1u << kWorkChunkBits) - 1));
    } else {
      bh = blockIdx.y;
      chunk = blockIdx.x;
    }
    int T_tok = tok_counts[bh];
    if (T_tok > max_tokens) {
      if (tid == 0 && chunk == 0) atomicOr(ws.status, EKV_STATUS_TOKENS);
      T_tok = max_tokens;
    }
    const int c0 = chunk * kChunkTokens;
    if (c0 >= T_tok) continue;
    const int nch = (T_tok + kChunkTokens - 1) / kChunkTokens;
    const int ntok = min(kChunkTokens, T_tok - c0);
    const int b = bh / q_heads, hq = bh % q_heads, hkv = hq / G;
    const T* khead = static_cast<const T*>(c.k) + b * c.kv_stride_b + hkv * c.kv_stride_h;

    // stage the chunk: one bulk copy per page, all on one barrier phase
    const int npg = (ntok + P - 1) >> pd.shift;
    if (tid == 0) mbar_expect_tx(&bar, (uint32_t)(ntok * D * sizeof(T)));
    if (tid < npg) {
      int page = page_indices[(size_t)bh * pi_stride + (c0 >> pd.shift) + tid];
      if ((unsigned)page >= (unsigned)c.page_capacity) {
        atomicOr(ws.status, EKV_STATUS_PAGE_RANGE);
        page = 0;   // keep the byte count the barrier expects; the status bit flags the result
      }
      const int rows = min(P, ntok - tid * P);
      bulk_load(s_k + (size_t)tid * P * D, khead + (size_t)page * P * D, (uint32_t)(rows * D * sizeof(T)), &bar);
    }
    float qs[EPL];
    unpack<T>(*reinterpret_cast<const uint4*>(q + b * qsb + hq * qsh + lane_in_row * EPL), qs);
#pragma unroll
    for (int j = 0; j < EPL; ++j) qs[j] *= qscale;
    const float tau0 = tau_mode == EKV_TAU_EXACT ? 0.f : tau[bh];
    float* zrow = ws.z + (size_t)bh * ws.zstride + c0;
    mbar_wait(&bar, phase);
    phase ^= 1u;

    float s0 = 0.f, s1 = 0.f, s2 = 0.f, mx = -1.0e6f;
#pragma unroll 4
    for (int i0 = 0; i0 < ntok; i0 += GROUPS) {     // uniform trip count (whole-warp shuffles)
      const int i = i0 + group;
      const bool ok = i < ntok;
      float kf[EPL];
      unpack<T>(lds128(s_k + (size_t)min(i, ntok - 1) * D + lane_in_row * EPL), kf);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) acc = fmaf(qs[j], kf[j], acc);
      acc = row_sum<LPR>(acc);
      if (ok && lane_in_row == 0) {
        zrow[i] = acc;
        mx = fmaxf(mx, acc);
        if (tau_mode != EKV_TAU_EXACT) halley_accumulate(acc, tau0, kind, beta, s0, s1, s2);
      }
    }
    __syncthreads();   // shared K tile, red[] and s_ticket of this block are free again
    if (lane_in_row == 0) {
      red[group][0] = s0;
      red[group][1] = s1;
      red[group][2] = s2;
      red[group][3] = mx;
    }
    __syncthreads();
    if (tid < 4) {
      float t = red[0][tid];
      for (int g = 1; g < GROUPS; ++g) t = tid == 3 ? fmaxf(t, red[g][3]) : t + red[g][tid];
      ws.part[((size_t)bh * ws.nchunks + chunk) * 4 + tid] = t;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(&ws.cnt_k[bh], 1);
    __syncthreads();
    if (s_ticket == nch - 1) {
      __threadfence();
      solve_head_tau(ws, bh, T_tok, nch, alpha, tau_mode, niter, tau, halley_sums);
      if (tid == 0) ws.cnt_k[bh] = 0;
    }
  }
}

// ---- V pass --------------------------------------------------------------------

template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads)
decode_values_kernel(ekv_cache_desc c, int q_heads, const int* __restrict__ page_indices, int64_t pi_stride,
                     const int* __restrict__ tok_counts, int max_tokens, float alpha,
                     const float* __restrict__ tau, void* __restrict__ out, int64_t osb, int64_t osh,
                     int out_is_f32, const uint32_t* __restrict__ work_list,
                     const int* __restrict__ work_total, DecodeWs ws, PageDiv pd) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kDecThreads / LPR;
  constexpr int SLICES = kDecThreads / D;
  __shared__ float red[GROUPS][D];
  __shared__ float s_p[kChunkTokens];
  __shared__ short s_idx[kChunkTokens];
  __shared__ int s_warp_cnt[kDecThreads / 32];
  __shared__ int s_page[kChunkTokens];   // page id of each page slot of the chunk
  __shared__ int s_ticket;

  const int kind = alpha_kind_of(alpha);
  const float beta = 1.f / (alpha - 1.f);
  const int lane_in_row = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int G = q_heads / c.kv_heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  const int n_items = work_list ? *work_total : (int)(gridDim.x * gridDim.y);
  const int first = work_list ? (int)blockIdx.x : (int)(blockIdx.y * gridDim.x + blockIdx.x);
  const int step = work_list ? (int)gridDim.x : n_items;
  for (int w = first; w < n_items; w += step) {
    int bh, chunk;
    if (work_list) {
      const uint32_t item = work_list[w];
      bh = (int)(item >> kWorkChunkBits);
      chunk = (int)(item & ((1u << kWorkChunkBits) - 1));
    } else {
      bh = blockIdx.y;
      chunk = blockIdx.x;
    }
    const int T_tok = min(tok_counts[bh], max_tokens);
    const int c0 = chunk * kChunkTokens;
    const int b = bh / q_heads, hq = bh % q_heads, hkv = hq / G;
    const bool empty_head = T_tok <= 0 && chunk == 0;   // still owes a zero output row
    if (c0 >= T_tok && !empty_head) continue;
    const int nch = max((T_tok + kChunkTokens - 1) / kChunkTokens, 1);
    const int ntok = max(min(kChunkTokens, T_tok - c0), 0);
    const float t = tau[bh];

    // ordered compaction of the tokens with non-zero weight
    float p = 0.f;
    if (tid < ntok) p = entmax_weight(ws.z[(size_t)bh * ws.zstride + c0 + tid], t, kind, beta);
    const unsigned ballot = __ballot_sync(0xffffffffu, p > 0.f);
    __syncthreads();   // shared arrays of the previous item are no longer read
    if (lane == 0) s_warp_cnt[warp] = __popc(ballot);
    // the chunk covers compact tokens c0 .. c0+ntok-1, i.e. page slots pg0 .. pg1 of the table
    int pg0, pg1, off_unused;
    pd.split(c0, pg0, off_unused);
    pd.split(c0 + max(ntok, 1) - 1, pg1, off_unused);
    if (ntok > 0 && tid <= pg1 - pg0) s_page[tid] = page_indices[(size_t)bh * pi_stride + pg0 + tid];
    __syncthreads();
    int base = 0, n_active = 0;
#pragma unroll
    for (int wv = 0; wv < kDecThreads / 32; ++wv) {
      const int cnt = s_warp_cnt[wv];
      if (wv < warp) base += cnt;
      n_active += cnt;
    }
    if (p > 0.f) {
      const int pos = base + __popc(ballot & ((1u << lane) - 1u));
      s_p[pos] = p;
      s_idx[pos] = (short)tid;
    }
    __syncthreads();

    if (n_active > 0) {
      const T* vbase = static_cast<const T*>(c.v) + b * c.kv_stride_b + hkv * c.kv_stride_h + lane_in_row * EPL;
      float acc[EPL];
#pragma unroll
      for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
      constexpr int UV = 4;   // rows in flight per lane group
      for (int a0 = group; a0 < n_active; a0 += GROUPS * UV) {
        uint4 r[UV];
        float pw[UV];
#pragma unroll
        for (int u = 0; u < UV; ++u) {
          const int a = a0 + u * GROUPS;
          r[u] = make_uint4(0, 0, 0, 0);
          pw[u] = 0.f;
          if (a < n_active) {
            int pg, off;
            pd.split(c0 + (int)s_idx[a], pg, off);
            const int page = s_page[pg - pg0];
            if ((unsigned)page < (unsigned)c.page_capacity) {
              r[u] = ld_stream(vbase + ((size_t)page * pd.P + off) * D);
              pw[u] = s_p[a];
            }
          }
        }
#pragma unroll
        for (int u = 0; u < UV; ++u) {
          float vf[EPL];
          unpack<T>(r[u], vf);
#pragma unroll
          for (int j = 0; j < EPL; ++j) acc[j] = fmaf(pw[u], vf[j], acc[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < EPL; ++j) red[group][lane_in_row * EPL + j] = acc[j];
      __syncthreads();
      if (tid < D) {
        float s = 0.f;
#pragma unroll 4
        for (int g = 0; g < GROUPS; ++g) s += red[g][tid];
        ws.pout[((size_t)bh * ws.nchunks + chunk) * D + tid] = s;
      }
    }
    if (tid == 0) ws.nz[(size_t)bh * ws.nchunks + chunk] = n_active > 0;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(&ws.cnt_v[bh], 1);
    __syncthreads();
    if (s_ticket == nch - 1) {
      // last block of this head: sum the partial outputs in chunk order
      __threadfence();
      const int d = tid % D, slice = tid / D;
      float s = 0.f;
      const int* nz = ws.nz + (size_t)bh * ws.nchunks;
      const float* po = ws.pout + (size_t)bh * ws.nchunks * D;
      for (int ch = slice; ch < nch; ch += SLICES)
        if (ld_cg(nz + ch)) s += ld_cg(po + (size_t)ch * D + d);
      red[slice][d] = s;   // SLICES <= GROUPS
      __syncthreads();
      if (tid < D) {
        float tot = red[0][tid];
#pragma unroll
        for (int sl = 1; sl < SLICES; ++sl) tot += red[sl][tid];
        const size_t o = (size_t)b * osb + (size_t)hq * osh + tid;
        if (out_is_f32) static_cast<float*>(out)[o] = tot;
        else static_cast<T*>(out)[o] = from_float<T>(tot);
      }
      if (tid == 0) ws.cnt_v[bh] = 0;
    }
  }
}

__global__ void halley_update_kernel(float* __restrict__ tau, const float* __restrict__ sums, int n, float beta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  tau[i] = halley_unbounded(tau[i], sums[(size_t)i * 3], sums[(size_t)i * 3 + 1], sums[(size_t)i * 3 + 2], beta);
}

inline PageDiv make_page_div(int P) {
  PageDiv pd;
  pd.P = P;
  pd.shift = -1;
  if ((P & (P - 1)) == 0) {
    int s = 0;
    while ((1 << s) < P) ++s;
    pd.shift = s;
  }
  return pd;
}

// Blocks of a work-list launch whose blocks each hold `smem` bytes of shared memory:
// as many as fit on the SMs at once (227 KB usable per SM), at most 8 per SM.
inline int persistent_blocks_for(size_t smem) {
  int dev = 0, sms = 148;
  static int cached_sms = 0;
  if (cached_sms == 0) {
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cached_sms = sms;
  }
  int per_sm = (int)((227 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  return cached_sms * per_sm;
}

inline int persistent_blocks() {
  static int blocks = 0;   // per process; all devices of a box are identical
  if (blocks == 0) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    blocks = sms * 8;
  }
  return blocks;
}

}  // namespace ekv

extern "C" size_t ekv_decode_workspace_bytes(int32_t batch, int32_t q_heads, int32_t head_dim,
                                             int32_t max_tokens) {
  if (batch <= 0 || q_heads <= 0 || head_dim <= 0 || max_tokens <= 0) return 0;
  return ekv::decode_ws_layout(batch, q_heads, head_dim, max_tokens, nullptr, nullptr);
}

extern "C" int ekv_decode_workspace_reset(void* workspace, int32_t batch, int32_t q_heads, void* stream) {
  if (!workspace || batch <= 0 || q_heads <= 0) return EKV_ERR_ARG;
  // the status word and the two per-head ticket arrays sit at the front of the layout
  cudaError_t e = cudaMemsetAsync(workspace, 0, ekv::decode_ws_header_bytes(batch, q_heads),
                                  ekv::as_stream(stream));
  return e == cudaSuccess ? EKV_OK : (int)e;
}

extern "C" int ekv_decode_scores(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                 int64_t q_stride_h, int32_t q_heads, const int32_t* page_indices,
                                 int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens,
                                 float alpha, int32_t tau_mode, int32_t niter, float* tau,
                                 float* halley_sums, const uint32_t* work_list,
                                 const int32_t* work_total, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!q || !page_indices || !tok_counts || !tau || !workspace) return EKV_ERR_ARG;
  if (q_heads <= 0 || q_heads % c->kv_heads || max_tokens <= 0 || niter < 0) return EKV_ERR_ARG;
  if (tau_mode < EKV_TAU_NONE || tau_mode > EKV_TAU_CORRECTED) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  if ((work_list == nullptr) != (work_total == nullptr)) return EKV_ERR_ARG;
  DecodeWs ws;
  if (decode_ws_layout(c->batch, q_heads, c->head_dim, max_tokens, workspace, &ws) > workspace_bytes)
    return EKV_ERR_WORKSPACE;
  if (ws.nchunks > (1 << kWorkChunkBits)) return EKV_ERR_ARG;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((q_stride_b * esz) % 16 || (q_stride_h * esz) % 16 || (reinterpret_cast<uintptr_t>(q) & 15))
    return EKV_ERR_ARG;
  const PageDiv pd = make_page_div(c->page_size);
  const int BH = c->batch * q_heads;
  dim3 grid = work_list ? dim3((unsigned)persistent_blocks()) : dim3((unsigned)ws.nchunks, (unsigned)BH);
  // pages that are power-of-two sized (>= 4 rows) are staged with bulk copies
  const bool bulk = pd.shift >= 2 && pd.P <= kChunkTokens;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    if (bulk) {
      const size_t smem = (size_t)kChunkTokens * D * sizeof(T);
      static bool attr_set = false;
      if (!attr_set) {
        cudaFuncSetAttribute(decode_scores_bulk_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
      }
      if (work_list) grid = dim3((unsigned)persistent_blocks_for(smem));
      decode_scores_bulk_kernel<T, D><<<grid, kDecThreads, smem, as_stream(stream)>>>(
          *c, static_cast<const T*>(q), q_stride_b, q_stride_h, q_heads, page_indices, pi_stride,
          tok_counts, max_tokens, alpha, tau_mode, niter, tau, halley_sums, work_list, work_total, ws, pd);
    } else {
      decode_scores_kernel<T, D><<<grid, kDecThreads, 0, as_stream(stream)>>>(
          *c, static_cast<const T*>(q), q_stride_b, q_stride_h, q_heads, page_indices, pi_stride,
          tok_counts, max_tokens, alpha, tau_mode, niter, tau, halley_sums, work_list, work_total, ws, pd);
    }
  });
  return launch_status();
}

extern "C" int ekv_halley_update(float* tau, const float* halley_sums, int32_t n, float alpha,
                                 void* stream) {
  using namespace ekv;
  if (!tau || !halley_sums || n <= 0) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  halley_update_kernel<<<(n + 127) / 128, 128, 0, as_stream(stream)>>>(tau, halley_sums, n, 1.f / (alpha - 1.f));
  return launch_status();
}

extern "C" int ekv_decode_values(const ekv_cache_desc* c, int32_t q_heads, const int32_t* page_indices,
                                 int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens,
                                 float alpha, const float* tau, void* out, int64_t out_stride_b,
                                 int64_t out_stride_h, int32_t out_is_f32, const uint32_t* work_list,
                                 const int32_t* work_total, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!page_indices || !tok_counts || !tau || !out || !workspace) return EKV_ERR_ARG;
  if (q_heads <= 0 || q_heads % c->kv_heads || max_tokens <= 0) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  if ((work_list == nullptr) != (work_total == nullptr)) return EKV_ERR_ARG;
  DecodeWs ws;
  if (decode_ws_layout(c->batch, q_heads, c->head_dim, max_tokens, workspace, &ws) > workspace_bytes)
    return EKV_ERR_WORKSPACE;
  const PageDiv pd = make_page_div(c->page_size);
  const int BH = c->batch * q_heads;
  dim3 grid = work_list ? dim3((unsigned)persistent_blocks()) : dim3((unsigned)ws.nchunks, (unsigned)BH);
  EKV_DISPATCH(c->dtype, c->head_dim, {
    decode_values_kernel<T, D><<<grid, kDecThreads, 0, as_stream(stream)>>>(
        *c, q_heads, page_indices, pi_stride, tok_counts, max_tokens, alpha, tau, out, out_stride_b,
        out_stride_h, out_is_f32, work_list, work_total, ws, pd);
  });
  return launch_status();
}

extern "C" int ekv_read_status(const void* workspace, int32_t* host_status, void* stream) {
  if (!workspace || !host_status) return EKV_ERR_ARG;
  cudaError_t e = cudaMemcpyAsync(host_status, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                  ekv::as_stream(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(ekv::as_stream(stream));
  return e == cudaSuccess ? EKV_OK : (int)e;
}
