// Paged entmax decode over the selected pages, in two passes:
//
//   K pass  (decode_scores_*): every selected key row is read ONCE; its score
//           z = (alpha-1)/sqrt(D) * q.k is kept (4 bytes per token) in the workspace
//           together with per-segment maxima / Halley sums.  A small per-head kernel
//           (tau_solve_kernel) then solves tau from the kept scores - the histogram, the
//           bracket and all Halley iterations re-read 4-byte scores from L2, never K.
//   V pass  (decode_values_*): only pages holding a token whose weight (z-tau)_+^beta
//           is non-zero are read from V; a small per-head kernel (out_reduce_kernel) sums
//           the partial outputs in chunk order.
//
// Work is cut into items of 256 compacted tokens of one query head, described by a
// 64-bit word (ekv_work.cuh) in a device-side list that the selection kernels emit.
// Persistent thread blocks each walk a contiguous range of the list (consecutive items
// mostly belong to one head, so statistics and partial outputs are carried in registers
// across them and stored once per run).  With power-of-two pages of 4..32 rows every
// page is a contiguous P*D*sizeof(T)-byte block of K (or V): it is fetched by ONE bulk
// asynchronous copy into a shared-memory stage, and the copies of the next items are
// issued (and the page ids of the item after those are prefetched into registers)
// while the current item is being computed - a software pipeline NS stages deep, so
// an SM always has tens of KB of reads in flight.  Other page sizes use a plain
// vectorised-load variant of the same two passes.
// Both passes are HBM-bound: 2*D*sizeof(T) bytes per selected token in total.
#include <algorithm>
#include <type_traits>

#include "ekv_common.cuh"
#include "ekv_work.cuh"
#include "ekv_exchange.cuh"
#include "ekv_tau_math.cuh"

namespace ekv {

constexpr int kDecThreads = 512;
constexpr int kStatusInts = 16;
constexpr int kIssueWarps = kChunkTokens / 32;   // warps whose lanes map 1:1 to the tokens of an item

struct DecodeWs {
  int* status;      // [16]; word 0 = status bits
  int* support;     // [BH]: tokens with non-zero weight, as counted by the tau kernel (-1: not counted)
  int* cnt_v;       // [BH]: 1 when the tau kernel already wrote the head's output (V pass skips it)
  float* z;         // [BH, zstride]
  float* part;      // [BH, nchunks, 4] = {s0, s1, s2, max}
  int* nz;          // [BH, nchunks]
  float* pout;      // [BH, nchunks, D]
  int64_t zstride;
  float* cmax;      // [BH, nchunks, 4] group-shared K pass: score maxima of the four token quarters of a chunk
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
  char* sup = take(BH * sizeof(int));
  char* cv = take(BH * sizeof(int));
  char* z = take(BH * zstride * sizeof(float));
  char* part = take(BH * nchunks * 4 * sizeof(float));
  char* nz = take(BH * nchunks * sizeof(int));
  char* pout = take(BH * nchunks * head_dim * sizeof(float));
  char* cmax = take(BH * nchunks * 4 * sizeof(float));
  if (ws) {
    ws->cmax = reinterpret_cast<float*>(cmax);
    ws->status = reinterpret_cast<int*>(st);
    ws->support = reinterpret_cast<int*>(sup);
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

// ---- tau from kept scores (one block per head, after the K pass) ---------------

// Kept scores are read either from a shared-memory copy or, written by other blocks of an
// earlier launch region, from L2.
__device__ __forceinline__ float rdz(const float* p, bool in_smem) { return in_smem ? *p : __ldcg(p); }

// Block-wide Halley sums over the kept scores of one head (fixed order).
__device__ void sums_over_scores(const float* z, bool z_smem, int n, float tau, int kind, float beta,
                                 float* scratch, float& s0, float& s1, float& s2) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) halley_accumulate(rdz(z + i, z_smem), tau, kind, beta, a0, a1, a2);
  s0 = block_sum(a0, scratch);
  s1 = block_sum(a1, scratch);
  s2 = block_sum(a2, scratch);
}

// Returns the head's final tau to every thread of the block.
// With an exchange (sequence-sharded step) the sums at the incoming tau are combined over the
// ranks before the first step, so every rank takes the same step; at most one step then.
__device__ float solve_head_tau(const DecodeWs& ws, const float* z, bool z_smem, int bh, int T_tok, int nch,
                                float alpha, int tau_mode, int niter, float* tau, float* halley_sums,
                                Xch* xch = nullptr) {
  __shared__ float scratch[32];
  __shared__ int hist[kBins];
  __shared__ float s_t;
  const int kind = alpha_kind_of(alpha);
  const float beta = 1.f / (alpha - 1.f);
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
      const float proj = (rdz(z + i, z_smem) - t0) * (float)kBins;
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
      sums_over_scores(z, z_smem, T_tok, s_t, kind, beta, scratch, s0, s1, s2);
      __syncthreads();
      if (tid == 0) {
        halley_bracketed(t, t_lo, t_hi, s0, s1, s2, beta);
        s_t = t;
      }
      __syncthreads();
    }
    if (tid == 0) tau[bh] = s_t;
    return s_t;
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
  float t = tau[bh];
  if (xch) {
    // one thread trades the head's three sums with the peers; the block takes the world's sums
    __syncthreads();                 // scratch is free again
    if (tid == 0) {
      xch->send(bh * 3 + 0, s0);
      xch->send(bh * 3 + 1, s1);
      xch->send(bh * 3 + 2, s2);
      scratch[0] = xch->sum(bh * 3 + 0, s0);
      scratch[1] = xch->sum(bh * 3 + 1, s1);
      scratch[2] = xch->sum(bh * 3 + 2, s2);
    }
    __syncthreads();
    s0 = scratch[0];
    s1 = scratch[1];
    s2 = scratch[2];
    __syncthreads();
  }
  if (tau_mode != EKV_TAU_CORRECTED || niter <= 0) return t;
  for (int it = 0; it < niter; ++it) {
    if (it > 0) {
      __syncthreads();
      sums_over_scores(z, z_smem, T_tok, t, kind, beta, scratch, s0, s1, s2);
    }
    t = halley_unbounded(t, s0, s1, s2, beta);   // every thread computes the same value
  }
  __syncthreads();   // every thread has read tau[bh] before it is overwritten
  if (tid == 0) tau[bh] = t;
  return t;
}

struct DecodeArgs {
  ekv_cache_desc c;
  const void* q;
  int64_t qsb, qsh;
  int q_heads;
  const int* page_indices;
  int64_t pi_stride;
  const int* tok_counts;
  int max_tokens;
  float alpha;
  int tau_mode, niter;
  float* tau;
  float* halley_sums;
  void* out;
  int64_t osb, osh;
  int out_is_f32;
  const unsigned long long* items;
  const int* work_total;
  int n_items;
  DecodeWs ws;
  PageDiv pd;
  FastDiv div_heads;   // by q_heads
  FastDiv div_group;   // by q_heads / kv_heads
  // ALiBi (null: none): per-query-head slopes and per-sequence query positions (null: last token)
  const float* alibi;
  const int* q_pos;
  // group-shared K pass (null: per-head K pass): one list over GQA groups, the membership mask of
  // every entry of the group's shared page table
  const unsigned long long* g_items;
  int g_n_items;
  const unsigned char* member;
  int64_t member_stride;
  int solve_cap;       // floats of dynamic shared memory the tau kernel has for a head's scores
  // where page `id` of (b, h_kv) starts: K/V base + b*kv_sb + h_kv*kv_stride_h + id*kv_ps.  Dense cache:
  // kv_sb = batch stride, kv_ps = P*D, ids are page numbers below page_limit = page_capacity.  Block-table
  // cache: kv_sb = 0, kv_ps = block stride, ids are physical block numbers below page_limit = num_blocks.
  int64_t kv_sb, kv_ps;
  int page_limit;
  // sequence-sharded step: the tau kernel trades its Halley sums with the other ranks (slot 2)
  int use_xch;
  int* xch_status;
  XchDev xch;
};

__device__ __forceinline__ int item_count(const DecodeArgs& a) {
  return a.work_total ? min(*a.work_total, a.n_items) : a.n_items;
}

// ---- per-run epilogues shared by the pipelined and the plain kernels --------------

// A block owns the items [first, first + n_mine) of the list.
__device__ __forceinline__ void my_item_range(const DecodeArgs& a, int& first, int& n_mine) {
  const int n_items = item_count(a);
  const long long lo = (long long)n_items * blockIdx.x / gridDim.x;
  const long long hi = (long long)n_items * (blockIdx.x + 1) / gridDim.x;
  first = (int)lo;
  n_mine = (int)(hi - lo);
}

// True when item `next` continues the run of item `cur` (same head, not an empty slot).
__device__ __forceinline__ bool same_run(unsigned long long cur, unsigned long long next) {
  return item_ntok(next) > 0 && item_head(next) == item_head(cur);
}

// K pass: per-chunk statistics slot {s0, s1, s2, max}.  Inside a run only the last item
// stores the run's folded statistics; the others store the neutral element.  Four lanes
// of every lane group carry statistics (one per row of a row quad): SLOTS = 4 * groups.
template <int SLOTS>
__device__ __forceinline__ void scores_run_store(const DecodeArgs& a, float (*red)[4], int slot, bool writer,
                                                 float s0, float s1, float s2, float mx, int bh, int chunk) {
  const int tid = threadIdx.x;
  if (writer) {
    red[slot][0] = s0;
    red[slot][1] = s1;
    red[slot][2] = s2;
    red[slot][3] = mx;
  }
  __syncthreads();
  if (tid < 32) {   // one warp folds the slots: lane l takes slots l, l+32, ..., then a butterfly (fixed order)
    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = -1.0e6f;
#pragma unroll
    for (int g = tid; g < SLOTS; g += 32) {
      v0 += red[g][0];
      v1 += red[g][1];
      v2 += red[g][2];
      v3 = fmaxf(v3, red[g][3]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      v0 += __shfl_xor_sync(0xffffffffu, v0, o);
      v1 += __shfl_xor_sync(0xffffffffu, v1, o);
      v2 += __shfl_xor_sync(0xffffffffu, v2, o);
      v3 = fmaxf(v3, __shfl_xor_sync(0xffffffffu, v3, o));
    }
    if (tid < 4) a.ws.part[((size_t)bh * a.ws.nchunks + chunk) * 4 + tid] = tid == 0 ? v0 : tid == 1 ? v1 : tid == 2 ? v2 : v3;
  }
}
__device__ __forceinline__ void scores_neutral_store(const DecodeArgs& a, int bh, int chunk) {
  if (threadIdx.x < 4)
    a.ws.part[((size_t)bh * a.ws.nchunks + chunk) * 4 + threadIdx.x] = threadIdx.x == 3 ? -1.0e6f : 0.f;
}

// V pass: fold the lane groups' partial outputs of a run into the slot of its last item.
template <int D, int GROUPS>
__device__ __forceinline__ void values_run_store(const DecodeArgs& a, float (*red)[D], bool any_active,
                                                 int bh, int chunk) {
  const int tid = threadIdx.x;
  if (any_active) {
    __syncthreads();   // red[] holds every group's partial sums
    if (tid < D) {
      float s = 0.f;
#pragma unroll 8
      for (int g = 0; g < GROUPS; ++g) s += red[g][tid];
      a.ws.pout[((size_t)bh * a.ws.nchunks + chunk) * D + tid] = s;
    }
  }
  if (tid == 0) a.ws.nz[(size_t)bh * a.ws.nchunks + chunk] = any_active ? 1 : 0;
}

constexpr int kInlineMax = 1024;     // heads with at most this many non-zero weights skip the V pass
constexpr int kSolveSmemScores = 8192;   // heads with at most this many tokens are solved from shared memory

// grid: B*H_q blocks of THREADS (256, or 1024 when there are few heads) threads.  tau of one head from its kept scores and per-chunk
// statistics.  When the output buffer is known (fused decode) and the head's support is
// small - the usual case for entmax - the few value rows are gathered right here, in
// token order, and the V pass skips the head (done[bh] = 1).
template <typename T, int D, int THREADS>
__global__ void __launch_bounds__(THREADS) tau_solve_kernel(const DecodeArgs a) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = THREADS / LPR;
  constexpr int WARPS = THREADS / 32;
  static_assert(GROUPS * D <= kSolveSmemScores, "the gather's reduction buffer re-uses the score copy");
  // score copy, later the gather's [GROUPS][D] buffer: a.solve_cap floats of dynamic shared memory
  // (the largest head this launch can meet, at most kSolveSmemScores), so that short heads - the
  // top-k budget is a few thousand tokens - leave room for every head of a batch to be resident at once
  extern __shared__ __align__(16) float s_z[];
  __shared__ int s_c[kInlineMax];
  __shared__ float s_w[kInlineMax];
  __shared__ int s_warp_cnt[WARPS];
  const int bh = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int* done = a.ws.cnt_v;
  const int T_tok = min(a.tok_counts[bh], a.max_tokens);
  Xch xe;
  if (a.use_xch) xe = xch_begin(a.xch, 2, a.xch_status);   // every block, before any early exit
  if (T_tok <= 0) {
    if (tid == 0) {
      a.ws.support[bh] = 0;
      done[bh] = 0;   // the output reduction writes the zero row
      if (a.use_xch) {
        // no local tokens: contribute zeros, and still take the world's step so tau stays the same everywhere
        for (int k = 0; k < 3; ++k) xe.send(bh * 3 + k, 0.f);
        const float s0 = xe.sum(bh * 3, 0.f), s1 = xe.sum(bh * 3 + 1, 0.f), s2 = xe.sum(bh * 3 + 2, 0.f);
        if (a.tau_mode == EKV_TAU_CORRECTED && a.niter > 0)
          a.tau[bh] = halley_unbounded(a.tau[bh], s0, s1, s2, 1.f / (a.alpha - 1.f));
      }
    }
    return;
  }
  const int nch = (T_tok + kChunkTokens - 1) / kChunkTokens;
  const float* zg = a.ws.z + (size_t)bh * a.ws.zstride;
  const bool z_smem = T_tok <= a.solve_cap;
  if (z_smem) {
    for (int i = tid; i < T_tok; i += THREADS) s_z[i] = ld_cg(zg + i);
    __syncthreads();
  }
  const float* z = z_smem ? s_z : zg;
  const float t = solve_head_tau(a.ws, z, z_smem, bh, T_tok, nch, a.alpha, a.tau_mode, a.niter, a.tau,
                                 a.halley_sums, a.use_xch ? &xe : nullptr);
  if (a.out == nullptr || a.tau_mode == EKV_TAU_NONE) {
    if (tid == 0) {
      a.ws.support[bh] = -1;
      done[bh] = 0;
    }
    return;
  }
  // Ordered compaction of the support.  Warp w owns the contiguous token segment w; its
  // lanes stride through it (coalesced), so ballots give positions in token order.
  const int kind = alpha_kind_of(a.alpha);
  const float beta = 1.f / (a.alpha - 1.f);
  // Scores of a long head come from L2: 16-byte loads, eight in flight per lane (a lane owns four
  // consecutive tokens of every 128-token group; rows are padded to whole chunks, so a load
  // past the head's end stays inside its row and is masked).  Short heads scan their shared copy.
  const bool wide = !z_smem;
  const int gran = wide ? 128 : 32;
  const int seg = ((T_tok + WARPS - 1) / WARPS + gran - 1) / gran * gran;
  const int w_lo = min(warp * seg, T_tok), w_hi = min(w_lo + seg, T_tok);
  constexpr int UZ = 8;   // score loads in flight per lane
  auto load4 = [&](int i) {   // tokens i..i+3 of this head, -inf past the warp's segment
    float4 v = __ldcg(reinterpret_cast<const float4*>(z + i));
    if (i + 0 >= w_hi) v.x = -INFINITY;
    if (i + 1 >= w_hi) v.y = -INFINITY;
    if (i + 2 >= w_hi) v.z = -INFINITY;
    if (i + 3 >= w_hi) v.w = -INFINITY;
    return v;
  };
  // After the group-shared K pass every 64-token quarter of a chunk carries its score maximum
  // (flat index token / 64).  A warp first lists the 128-token groups of its segment that have a
  // quarter above tau - 8 bytes per group, all loads independent - and both scans below walk
  // that list (kept in the score copy, which a long head does not use); without the maxima the
  // list is implicit: every group.
  const float* cm = a.g_items ? a.ws.cmax + (size_t)bh * a.ws.nchunks * 4 : nullptr;
  const int seg_groups = (w_hi - w_lo + 127) / 128;
  const int kListCap = a.solve_cap * 2 / WARPS;
  unsigned short* glist = reinterpret_cast<unsigned short*>(s_z) + warp * kListCap;
  const bool listed = wide && cm != nullptr && seg_groups <= kListCap && seg_groups <= 65535;
  int n_groups = wide ? seg_groups : 0;
  if (listed) {
    n_groups = 0;
    const unsigned below = (1u << lane) - 1u;
    for (int g0 = 0; g0 < seg_groups; g0 += 32 * UZ) {
      float2 m[UZ];
#pragma unroll
      for (int u = 0; u < UZ; ++u) {
        const int gi = g0 + u * 32 + lane;
        m[u] = gi < seg_groups ? __ldcg(reinterpret_cast<const float2*>(cm + (w_lo >> 6)) + gi)
                               : make_float2(-INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < UZ; ++u) {
        const bool above = m[u].x > t || m[u].y > t;
        const unsigned bal = __ballot_sync(0xffffffffu, above);
        if (above) glist[n_groups + __popc(bal & below)] = (unsigned short)(g0 + u * 32 + lane);
        n_groups += __popc(bal);
      }
    }
    __syncwarp();
  }
  // first token of this lane in the j-th group to scan (w_hi: nothing)
  auto lane_token = [&](int j) -> int {
    return j < n_groups ? w_lo + (listed ? (int)glist[j] : j) * 128 + lane * 4 : w_hi;
  };
  const float4 none4 = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
  int wcount = 0;
  if (wide) {
    for (int j0 = 0; j0 < n_groups; j0 += UZ) {
      float4 zv[UZ];
#pragma unroll
      for (int u = 0; u < UZ; ++u) {
        const int i = lane_token(j0 + u);
        zv[u] = i < w_hi ? load4(i) : none4;
      }
#pragma unroll
      for (int u = 0; u < UZ; ++u)
        wcount += __popc(__ballot_sync(0xffffffffu, zv[u].x > t)) + __popc(__ballot_sync(0xffffffffu, zv[u].y > t)) +
                  __popc(__ballot_sync(0xffffffffu, zv[u].z > t)) + __popc(__ballot_sync(0xffffffffu, zv[u].w > t));
    }
  } else {
    for (int i0 = w_lo; i0 < w_hi; i0 += 32 * UZ) {
      float zv[UZ];
#pragma unroll
      for (int u = 0; u < UZ; ++u) {
        const int i = i0 + u * 32 + lane;
        zv[u] = i < w_hi ? rdz(z + i, z_smem) : -INFINITY;
      }
#pragma unroll
      for (int u = 0; u < UZ; ++u) wcount += __popc(__ballot_sync(0xffffffffu, zv[u] > t));
    }
  }
  if (lane == 0) s_warp_cnt[warp] = wcount;
  __syncthreads();
  int base = 0, total = 0;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) {
    const int cw = s_warp_cnt[w];
    if (w < warp) base += cw;
    total += cw;
  }
  if (tid == 0) a.ws.support[bh] = total;
  if (total > kInlineMax) {
    if (tid == 0) done[bh] = 0;
    return;
  }
  if (wide) {
    const unsigned below = (1u << lane) - 1u;
    for (int j0 = 0; j0 < n_groups; j0 += UZ) {
      float4 zv[UZ];
      int tok[UZ];
#pragma unroll
      for (int u = 0; u < UZ; ++u) {
        tok[u] = lane_token(j0 + u);
        zv[u] = tok[u] < w_hi ? load4(tok[u]) : none4;
      }
#pragma unroll
      for (int u = 0; u < UZ; ++u) {
        // token order inside a group of 128: lane-major, then the lane's four tokens
        const float e[4] = {zv[u].x, zv[u].y, zv[u].z, zv[u].w};
        unsigned bal[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) bal[c] = __ballot_sync(0xffffffffu, e[c] > t);
        if ((bal[0] | bal[1] | bal[2] | bal[3]) == 0u) continue;   // uniform across the warp
        int pos = base + __popc(bal[0] & below) + __popc(bal[1] & below) + __popc(bal[2] & below) +
                  __popc(bal[3] & below);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (e[c] > t) {
            s_c[pos] = tok[u] + c;
            s_w[pos] = entmax_weight(e[c], t, kind, beta);
            ++pos;
          }
        base += __popc(bal[0]) + __popc(bal[1]) + __popc(bal[2]) + __popc(bal[3]);
      }
    }
  } else {
    for (int i0 = w_lo; i0 < w_hi; i0 += 32 * UZ) {
      float zv[UZ];
#pragma unroll
      for (int u = 0; u < UZ; ++u) {
        const int i = i0 + u * 32 + lane;
        zv[u] = i < w_hi ? rdz(z + i, z_smem) : -INFINITY;
      }
#pragma unroll
      for (int u = 0; u < UZ; ++u) {
        const bool act = zv[u] > t;
        const unsigned bal = __ballot_sync(0xffffffffu, act);
        if (act) {
          const int pos = base + __popc(bal & ((1u << lane) - 1u));
          s_c[pos] = i0 + u * 32 + lane;
          s_w[pos] = entmax_weight(zv[u], t, kind, beta);
        }
        base += __popc(bal);
      }
    }
  }
  __syncthreads();   // support list complete; the score copy is no longer read
  // gather the value rows: lane group g takes support entries g, g+GROUPS, ... (token order)
  float (*red)[D] = reinterpret_cast<float (*)[D]>(s_z);
  const int lane_in_row = tid % LPR, group = tid / LPR;
  const int G = a.q_heads / a.c.kv_heads;
  const int b = bh / a.q_heads, hq = bh % a.q_heads, hkv = hq / G;
  const T* vbase = static_cast<const T*>(a.c.v) + b * a.kv_sb + hkv * a.c.kv_stride_h + lane_in_row * EPL;
  const int* pi = a.page_indices + (size_t)bh * a.pi_stride;
  float acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
  constexpr int UV = 4;
  for (int e0 = group; e0 < total; e0 += GROUPS * UV) {
    uint4 r[UV];
    float pw[UV];
#pragma unroll
    for (int u = 0; u < UV; ++u) {
      const int e = e0 + u * GROUPS;
      r[u] = make_uint4(0, 0, 0, 0);
      pw[u] = 0.f;
      if (e < total) {
        int pg, off;
        a.pd.split(s_c[e], pg, off);
        const int page = pi[pg];
        if ((unsigned)page < (unsigned)a.page_limit) {
          r[u] = ld_stream(vbase + ((size_t)page * a.kv_ps + (size_t)off * D));
          pw[u] = s_w[e];
        } else if (lane_in_row == 0) {
          atomicOr(a.ws.status, EKV_STATUS_PAGE_RANGE);
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
    float sum = 0.f;
#pragma unroll 4
    for (int g = 0; g < GROUPS; ++g) sum += red[g][tid];
    const size_t o = (size_t)b * a.osb + (size_t)hq * a.osh + tid;
    if (a.out_is_f32) static_cast<float*>(a.out)[o] = sum;
    else static_cast<T*>(a.out)[o] = from_float<T>(sum);
  }
  if (tid == 0) done[bh] = 1;
}

// grid: B*H_q blocks of D threads.  out[b,h,:] = sum over the head's chunks, in chunk order,
// of the partial outputs the V pass stored (heads without tokens get zeros).
template <typename T, int D>
__global__ void __launch_bounds__(D) out_reduce_kernel(const DecodeArgs a) {
  const int bh = blockIdx.x, d = threadIdx.x;
  if (a.ws.cnt_v[bh] != 0) return;   // the tau solver already wrote this head's output
  const int T_tok = min(a.tok_counts[bh], a.max_tokens);
  const int nch = T_tok > 0 ? (T_tok + kChunkTokens - 1) / kChunkTokens : 0;
  const int* nz = a.ws.nz + (size_t)bh * a.ws.nchunks;
  const float* po = a.ws.pout + (size_t)bh * a.ws.nchunks * D;
  float s = 0.f;
  for (int ch = 0; ch < nch; ++ch)
    if (nz[ch]) s += po[(size_t)ch * D + d];
  const int b = bh / a.q_heads, hq = bh % a.q_heads;
  const size_t o = (size_t)b * a.osb + (size_t)hq * a.osh + d;
  if (a.out_is_f32) static_cast<float*>(a.out)[o] = s;
  else static_cast<T*>(a.out)[o] = from_float<T>(s);
}

// ---- pipelined K pass ---------------------------------------------------------------

// ALiBi term of one kept token: (alpha-1) * slope[h] * (its absolute position - the query's),
// entmaxkv/kernels/adadecode_paged.py:100-105,126-128.  `c` is the token's index in the head's
// compacted list; its absolute position comes from the page table.
struct AlibiRow {
  float slope_a;
  int q_idx;
  const int* pages;
  __device__ __forceinline__ void init(const DecodeArgs& a, int bh) {
    int b, hq;
    a.div_heads.divmod(bh, b, hq);
    slope_a = a.alibi[hq] * (a.alpha - 1.f);
    q_idx = a.q_pos ? a.q_pos[b] : a.c.seq_lens[b] - 1;
    pages = a.page_indices + (size_t)bh * a.pi_stride;
  }
  __device__ __forceinline__ float add(const DecodeArgs& a, float z, int c) const {
    int pg, off;
    a.pd.split(c, pg, off);
    const int row = pages[pg] * a.pd.P + off;
    return fmaf(slope_a, (float)(row - q_idx), z);
  }
};

template <typename T, int D, int NS, bool ALIBI>
__global__ void __launch_bounds__(kDecThreads, 1) decode_scores_pipe_kernel(const DecodeArgs a) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kDecThreads / LPR;
  constexpr int PD = NS - 1;   // items whose copies are in flight ahead of the one being computed
  constexpr size_t kStageElems = (size_t)kChunkTokens * D;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* s_k = reinterpret_cast<T*>(smem_raw);
  __shared__ uint64_t full[NS];
  __shared__ float red[GROUPS * 4][4];

  const int kind = alpha_kind_of(a.alpha);
  const float beta = 1.f / (a.alpha - 1.f);
  const float qscale = (a.alpha - 1.f) * (D == 64 ? 0.125f : 0.08838834764831845f);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lane_in_row = tid % LPR;
  const int group = tid / LPR;
  const int cluster = lane_in_row / (LPR / 4);          // which row of a quad this lane reports
  const bool writer = lane_in_row % (LPR / 4) == 0;
  const int P = a.pd.P, shift = a.pd.shift;
  const int ppw = 32 >> shift;                       // pages per issuing warp (P <= 32)
  const int my_slot = (warp < kIssueWarps && lane < ppw) ? warp * ppw + lane : -1;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) mbar_init(&full[s], kIssueWarps);
    mbar_fence_init();
  }
  __syncthreads();

  int first, n_mine;
  my_item_range(a, first, n_mine);
  auto load_desc = [&](int k) -> unsigned long long { return k < n_mine ? a.items[first + k] : 0ull; };
  auto load_page = [&](unsigned long long d) -> int {
    if (my_slot < 0 || my_slot * P >= item_ntok(d)) return -1;
    return a.page_indices[(size_t)item_head(d) * a.pi_stride + ((item_chunk(d) * kChunkTokens) >> shift) + my_slot];
  };
  auto load_q = [&](unsigned long long d) -> uint4 {
    if (item_ntok(d) == 0) return make_uint4(0, 0, 0, 0);
    int b, hq;
    a.div_heads.divmod(item_head(d), b, hq);
    return *reinterpret_cast<const uint4*>(static_cast<const T*>(a.q) + b * a.qsb + hq * a.qsh +
                                           lane_in_row * EPL);
  };
  auto load_tau = [&](unsigned long long d) -> float {
    return (a.tau_mode == EKV_TAU_EXACT || item_ntok(d) == 0) ? 0.f : a.tau[item_head(d)];
  };
  // Put one item's copies in flight into stage `st`: every issuing warp arms the barrier with
  // the bytes of its own pages, then its first lanes launch one bulk copy per page.
  auto issue = [&](unsigned long long d, int page, int st) {
    const int ntok = item_ntok(d);
    if (ntok == 0 || warp >= kIssueWarps) return;
    const int bh = item_head(d);
    int b, hq;
    a.div_heads.divmod(bh, b, hq);
    const int hkv = a.div_group.div(hq);
    int rows = 0;
    if (my_slot >= 0 && my_slot * P < ntok) rows = min(P, ntok - my_slot * P);
    if (rows > 0 && (unsigned)page >= (unsigned)a.page_limit) {
      atomicOr(a.ws.status, EKV_STATUS_PAGE_RANGE);
      page = 0;   // keep the byte count; the status bit marks the result as invalid
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
      bulk_load(s_k + st * kStageElems + (size_t)my_slot * P * D, src, bytes, &full[st]);
    }
  };

  // dq[j] = descriptor of item k+j; dq[PD] is the next one to issue, dB the one after it
  unsigned long long dq[NS];
#pragma unroll
  for (int j = 0; j < PD; ++j) {
    dq[j] = load_desc(j);
    issue(dq[j], load_page(dq[j]), j % NS);
  }
  dq[PD] = load_desc(PD);
  int pgA = load_page(dq[PD]);
  unsigned long long dB = load_desc(PD + 1);
  uint4 q_raw = load_q(dq[0]);
  float tau0 = load_tau(dq[0]);
  uint32_t phase_bits = 0;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, mx = -1.0e6f;   // statistics of the current run of items

  for (int k = 0; k < n_mine; ++k) {
    // copies of item k+PD go into the stage that item k-1 released at the end of its iteration
    issue(dq[PD], pgA, (k + PD) % NS);
    // everything the next iterations need from global memory is requested now and first
    // touched one iteration later
    const int pgB = load_page(dB);
    const unsigned long long dC = load_desc(k + PD + 2);
    const unsigned long long dn = PD >= 1 ? dq[PD >= 1 ? 1 : 0] : dB;   // item k+1
    const uint4 q_raw_n = load_q(dn);
    const float tau0_n = load_tau(dn);

    const int st = k % NS;
    const unsigned long long dk = dq[0];
    const int ntok = item_ntok(dk);
    if (ntok > 0) {
      const int bh = item_head(dk), chunk = item_chunk(dk);
      float qs[EPL];
      unpack<T>(q_raw, qs);
#pragma unroll
      for (int j = 0; j < EPL; ++j) qs[j] *= qscale;
      float* zrow = a.ws.z + (size_t)bh * a.ws.zstride + chunk * kChunkTokens;
      AlibiRow ali;
      if constexpr (ALIBI) ali.init(a, bh);
      mbar_wait(&full[st], (phase_bits >> st) & 1u);
      phase_bits ^= 1u << st;
      const T* tile = s_k + st * kStageElems;
      // a lane group scores four rows at a time; lane cluster r of the group ends up
      // holding the score of row r of the quad (uniform trip count: whole-warp shuffles)
#pragma unroll 2
      for (int i0 = 0; i0 < ntok; i0 += GROUPS * 4) {
        float acc4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int row = min(i0 + group + u * GROUPS, ntok - 1);
          float kf[EPL];
          unpack<T>(lds128(tile + (size_t)row * D + lane_in_row * EPL), kf);
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < EPL; ++j) acc = fmaf(qs[j], kf[j], acc);
          acc4[u] = acc;
        }
        float zv = row_sum_quad<LPR>(acc4, lane_in_row);
        const int i = i0 + group + cluster * GROUPS;
        if (writer && i < ntok) {
          if constexpr (ALIBI) zv = ali.add(a, zv, chunk * kChunkTokens + i);
          zrow[i] = zv;
          mx = fmaxf(mx, zv);
          if (a.tau_mode != EKV_TAU_EXACT) halley_accumulate(zv, tau0, kind, beta, s0, s1, s2);
        }
      }
      if (same_run(dk, dn)) {
        scores_neutral_store(a, bh, chunk);
      } else {
        scores_run_store<GROUPS * 4>(a, red, group * 4 + cluster, writer, s0, s1, s2, mx, bh, chunk);
        s0 = s1 = s2 = 0.f;
        mx = -1.0e6f;
      }
    }
    __syncthreads();   // the stage and red[] are free for re-use
#pragma unroll
    for (int j = 0; j < PD; ++j) dq[j] = dq[j + 1];
    dq[PD] = dB;
    pgA = pgB;
    dB = dC;
    q_raw = q_raw_n;
    tau0 = tau0_n;
  }
}

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
      mbar_wait(&full[st], (phase_bits >> st) & 1u);
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

// ---- pipelined V pass ---------------------------------------------------------------

template <typename T, int D, int NS>
__global__ void __launch_bounds__(kDecThreads, 1) decode_values_pipe_kernel(const DecodeArgs a) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kDecThreads / LPR;
  constexpr int PD = NS - 1;
  constexpr size_t kStageElems = (size_t)kChunkTokens * D;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* s_v = reinterpret_cast<T*>(smem_raw);
  float (*red)[D] = reinterpret_cast<float (*)[D]>(smem_raw + NS * kStageElems * sizeof(T));
  __shared__ uint64_t full[NS];
  __shared__ float s_p[NS][kChunkTokens];
  __shared__ int s_any[NS];

  const int kind = alpha_kind_of(a.alpha);
  const float beta = 1.f / (a.alpha - 1.f);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lane_in_row = tid % LPR;
  const int group = tid / LPR;
  const int P = a.pd.P, shift = a.pd.shift;
  const int ppw = 32 >> shift;
  const int my_slot = (warp < kIssueWarps && lane < ppw) ? warp * ppw + lane : -1;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], kIssueWarps);
      s_any[s] = 0;
    }
    mbar_fence_init();
  }
  __syncthreads();

  // Blocks own tiles of kValueTile consecutive items, dealt round-robin.  Usually the tau kernel
  // has produced nearly every head and the few heads left to this pass (support above the inline
  // limit) are long runs of consecutive items: dealt out in tiles they spread over all blocks
  // instead of keeping one block busy for the whole list of its head, while items of a tile still
  // fold into one partial output.  The partial of a run lands in the slot of its last chunk and
  // the output reduction adds the slots in chunk order, so the result does not depend on the deal.
  constexpr int kValueTile = 8;
  const int n_items = item_count(a);
  const int n_tiles = (n_items + kValueTile - 1) / kValueTile;
  const int tiles_mine = (int)blockIdx.x < n_tiles ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int n_mine = tiles_mine * kValueTile;
  auto item_at = [&](int k) -> unsigned long long {      // k-th item of this block (0 past the list)
    const int idx = ((int)blockIdx.x + (k / kValueTile) * (int)gridDim.x) * kValueTile + k % kValueTile;
    return idx < n_items ? a.items[idx] : 0ull;
  };
  {
    // the usual case - the tau kernel produced every head - shows in the per-head flags alone:
    // one pass over a few KB instead of a look-up per item
    const int n_heads = a.c.batch * a.q_heads;
    if (n_heads <= 16 * kDecThreads) {
      int open_heads = 0;
      for (int h = tid; h < n_heads; h += kDecThreads) open_heads |= a.ws.cnt_v[h] == 0 && a.tok_counts[h] > 0;
      if (__syncthreads_or(open_heads) == 0) return;
    }
  }
  {
    // nothing to stream when the tau kernel already produced every head of these tiles
    int pending = 0;
    for (int k = tid; k < n_mine; k += kDecThreads) {
      const unsigned long long d = item_at(k);
      pending |= item_ntok(d) > 0 && a.ws.cnt_v[item_head(d)] == 0;
    }
    if (__syncthreads_or(pending) == 0) return;
  }
  // items of heads whose output the tau solver already produced are treated as empty slots
  auto load_desc = [&](int k) -> unsigned long long {
    if (k >= n_mine) return 0ull;
    const unsigned long long d = item_at(k);
    return (item_ntok(d) > 0 && a.ws.cnt_v[item_head(d)] != 0) ? 0ull : d;
  };
  auto load_page = [&](unsigned long long d) -> int {
    if (my_slot < 0 || my_slot * P >= item_ntok(d)) return -1;
    return a.page_indices[(size_t)item_head(d) * a.pi_stride + ((item_chunk(d) * kChunkTokens) >> shift) + my_slot];
  };
  // score of this thread's token of item d (threads 0..255 map to the item's tokens) and the head's tau
  auto load_z = [&](unsigned long long d) -> float {
    if (tid >= item_ntok(d)) return -INFINITY;
    return a.ws.z[(size_t)item_head(d) * a.ws.zstride + item_chunk(d) * kChunkTokens + tid];
  };
  auto load_tau = [&](unsigned long long d) -> float { return item_ntok(d) == 0 ? 0.f : a.tau[item_head(d)]; };
  // Put in flight the pages of item d that hold at least one token with non-zero weight.
  auto issue = [&](unsigned long long d, int page, float z, float t, int st) {
    const int ntok = item_ntok(d);
    if (ntok == 0 || warp >= kIssueWarps) return;
    const float p = tid < ntok ? entmax_weight(z, t, kind, beta) : 0.f;
    s_p[st][tid] = p;
    const unsigned active = __ballot_sync(0xffffffffu, p > 0.f);
    const int bh = item_head(d);
    int b, hq;
    a.div_heads.divmod(bh, b, hq);
    const int hkv = a.div_group.div(hq);
    int rows = 0;
    if (my_slot >= 0 && my_slot * P < ntok) {
      const unsigned page_mask = (P == 32 ? 0xffffffffu : ((1u << P) - 1u)) << (lane * P);
      if (active & page_mask) rows = min(P, ntok - my_slot * P);
    }
    if (rows > 0 && (unsigned)page >= (unsigned)a.page_limit) {
      atomicOr(a.ws.status, EKV_STATUS_PAGE_RANGE);
      page = 0;
    }
    const uint32_t bytes = (uint32_t)(rows * D * sizeof(T));
    uint32_t wbytes = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wbytes += __shfl_xor_sync(0xffffffffu, wbytes, o);
    if (lane == 0) {
      mbar_expect_tx(&full[st], wbytes);
      if (active) s_any[st] = 1;   // several warps may store the same value
    }
    __syncwarp();
    if (rows > 0) {
      const T* src = static_cast<const T*>(a.c.v) + b * a.kv_sb + hkv * a.c.kv_stride_h +
                     (size_t)page * a.kv_ps;
      bulk_load(s_v + st * kStageElems + (size_t)my_slot * P * D, src, bytes, &full[st]);
    }
  };

  unsigned long long dq[NS];
#pragma unroll
  for (int j = 0; j < PD; ++j) {
    dq[j] = load_desc(j);
    issue(dq[j], load_page(dq[j]), load_z(dq[j]), load_tau(dq[j]), j % NS);
  }
  dq[PD] = load_desc(PD);
  int pgA = load_page(dq[PD]);
  float zA = load_z(dq[PD]), tA = load_tau(dq[PD]);
  unsigned long long dB = load_desc(PD + 1);
  uint32_t phase_bits = 0;
  float acc[EPL];   // partial output of the current run of items
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
  bool run_any = false;

  for (int k = 0; k < n_mine; ++k) {
    issue(dq[PD], pgA, zA, tA, (k + PD) % NS);
    const int pgB = load_page(dB);
    const float zB = load_z(dB), tB = load_tau(dB);
    const unsigned long long dC = load_desc(k + PD + 2);
    const unsigned long long dn = PD >= 1 ? dq[PD >= 1 ? 1 : 0] : dB;   // item k+1

    const int st = k % NS;
    const unsigned long long dk = dq[0];
    const int ntok = item_ntok(dk);
    if (ntok > 0) {
      const int bh = item_head(dk), chunk = item_chunk(dk);
      mbar_wait(&full[st], (phase_bits >> st) & 1u);
      phase_bits ^= 1u << st;
      __syncthreads();   // s_p / s_any of this stage, written by the issuing warps, are visible
      if (s_any[st] != 0) {
        run_any = true;
        const T* tile = s_v + st * kStageElems;
        for (int i = group; i < ntok; i += GROUPS) {
          const float pw = s_p[st][i];
          if (pw > 0.f) {
            float vf[EPL];
            unpack<T>(lds128(tile + (size_t)i * D + lane_in_row * EPL), vf);
#pragma unroll
            for (int j = 0; j < EPL; ++j) acc[j] = fmaf(pw, vf[j], acc[j]);
          }
        }
      }
      __syncthreads();   // every thread has read s_any before it is cleared
      if (tid == 0) s_any[st] = 0;
      if (same_run(dk, dn)) {
        if (tid == 0) a.ws.nz[(size_t)bh * a.ws.nchunks + chunk] = 0;
      } else {
        if (run_any) {
#pragma unroll
          for (int j = 0; j < EPL; ++j) red[group][lane_in_row * EPL + j] = acc[j];
        }
        values_run_store<D, GROUPS>(a, red, run_any, bh, chunk);
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
        run_any = false;
      }
    }
    __syncthreads();   // the stage, s_p and red[] are free for re-use
#pragma unroll
    for (int j = 0; j < PD; ++j) dq[j] = dq[j + 1];
    dq[PD] = dB;
    pgA = pgB;
    zA = zB;
    tA = tB;
    dB = dC;
  }
}

// ---- plain variants (any page size): vectorised global loads, no staging ------------------

template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads) decode_scores_plain_kernel(const DecodeArgs a) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kDecThreads / LPR;
  __shared__ float red[GROUPS * 4][4];
  const int kind = alpha_kind_of(a.alpha);
  const float beta = 1.f / (a.alpha - 1.f);
  const float qscale = (a.alpha - 1.f) * (D == 64 ? 0.125f : 0.08838834764831845f);
  const int lane_in_row = threadIdx.x % LPR;
  const int group = threadIdx.x / LPR;
  const int cluster = lane_in_row / (LPR / 4);
  const bool writer = lane_in_row % (LPR / 4) == 0;
  const int G = a.q_heads / a.c.kv_heads;
  int first, n_mine;
  my_item_range(a, first, n_mine);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, mx = -1.0e6f;
  for (int k = 0; k < n_mine; ++k) {
    const unsigned long long d = a.items[first + k];
    const unsigned long long dn = k + 1 < n_mine ? a.items[first + k + 1] : 0ull;
    const int ntok = item_ntok(d);
    if (ntok == 0) continue;
    const int bh = item_head(d), chunk = item_chunk(d);
    const int c0 = chunk * kChunkTokens;
    const int b = bh / a.q_heads, hq = bh % a.q_heads, hkv = hq / G;
    float qs[EPL];
    unpack<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(a.q) + b * a.qsb + hq * a.qsh +
                                              lane_in_row * EPL), qs);
#pragma unroll
    for (int j = 0; j < EPL; ++j) qs[j] *= qscale;
    const float tau0 = a.tau_mode == EKV_TAU_EXACT ? 0.f : a.tau[bh];
    const T* kbase = static_cast<const T*>(a.c.k) + b * a.kv_sb + hkv * a.c.kv_stride_h + lane_in_row * EPL;
    const int* pi = a.page_indices + (size_t)bh * a.pi_stride;
    float* zrow = a.ws.z + (size_t)bh * a.ws.zstride + c0;
    AlibiRow ali;
    if (a.alibi) ali.init(a, bh);
    // the loop bound is uniform over the block: the row-sum shuffles need every lane of a warp
    for (int i0 = 0; i0 < ntok; i0 += GROUPS * 4) {
      uint4 r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int ci = i0 + group + u * GROUPS;
        r[u] = make_uint4(0, 0, 0, 0);
        if (ci < ntok) {
          int pg, off;
          a.pd.split(c0 + ci, pg, off);
          const int page = pi[pg];
          if ((unsigned)page < (unsigned)a.page_limit) {
            r[u] = ld_stream(kbase + ((size_t)page * a.kv_ps + (size_t)off * D));
          } else if (lane_in_row == 0) {
            atomicOr(a.ws.status, EKV_STATUS_PAGE_RANGE);
          }
        }
      }
      float acc4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float kf[EPL];
        unpack<T>(r[u], kf);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc = fmaf(qs[j], kf[j], acc);
        acc4[u] = acc;
      }
      float zv = row_sum_quad<LPR>(acc4, lane_in_row);
      const int i = i0 + group + cluster * GROUPS;
      if (writer && i < ntok) {
        if (a.alibi) zv = ali.add(a, zv, c0 + i);
        zrow[i] = zv;
        mx = fmaxf(mx, zv);
        if (a.tau_mode != EKV_TAU_EXACT) halley_accumulate(zv, tau0, kind, beta, s0, s1, s2);
      }
    }
    if (same_run(d, dn)) {
      scores_neutral_store(a, bh, chunk);
    } else {
      scores_run_store<GROUPS * 4>(a, red, group * 4 + cluster, writer, s0, s1, s2, mx, bh, chunk);
      s0 = s1 = s2 = 0.f;
      mx = -1.0e6f;
      __syncthreads();   // red[] is free for the next run
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kDecThreads) decode_values_plain_kernel(const DecodeArgs a) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  constexpr int GROUPS = kDecThreads / LPR;
  __shared__ float red[GROUPS][D];
  __shared__ float s_p[kChunkTokens];
  __shared__ int s_any;
  const int kind = alpha_kind_of(a.alpha);
  const float beta = 1.f / (a.alpha - 1.f);
  const int tid = threadIdx.x;
  const int lane_in_row = tid % LPR;
  const int group = tid / LPR;
  const int G = a.q_heads / a.c.kv_heads;
  int first, n_mine;
  my_item_range(a, first, n_mine);
  if (tid == 0) s_any = 0;
  __syncthreads();
  float acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
  bool run_any = false;
  for (int k = 0; k < n_mine; ++k) {
    const unsigned long long d = a.items[first + k];
    const unsigned long long dn = k + 1 < n_mine ? a.items[first + k + 1] : 0ull;
    const int ntok = item_ntok(d);
    if (ntok == 0 || a.ws.cnt_v[item_head(d)] != 0) continue;   // empty slot, or solved inline
    const int bh = item_head(d), chunk = item_chunk(d);
    const int c0 = chunk * kChunkTokens;
    const int b = bh / a.q_heads, hq = bh % a.q_heads, hkv = hq / G;
    if (tid < kChunkTokens) {
      float p = 0.f;
      if (tid < ntok) p = entmax_weight(a.ws.z[(size_t)bh * a.ws.zstride + c0 + tid], a.tau[bh], kind, beta);
      s_p[tid] = p;
      if (p > 0.f) s_any = 1;
    }
    __syncthreads();
    if (s_any != 0) {
      run_any = true;
      const T* vbase = static_cast<const T*>(a.c.v) + b * a.kv_sb + hkv * a.c.kv_stride_h + lane_in_row * EPL;
      const int* pi = a.page_indices + (size_t)bh * a.pi_stride;
      for (int i = group; i < ntok; i += GROUPS) {
        const float pw = s_p[i];
        if (pw > 0.f) {
          int pg, off;
          a.pd.split(c0 + i, pg, off);
          const int page = pi[pg];
          if ((unsigned)page < (unsigned)a.page_limit) {
            float vf[EPL];
            unpack<T>(ld_stream(vbase + ((size_t)page * a.kv_ps + (size_t)off * D)), vf);
#pragma unroll
            for (int j = 0; j < EPL; ++j) acc[j] = fmaf(pw, vf[j], acc[j]);
          }
        }
      }
    }
    __syncthreads();
    if (tid == 0) s_any = 0;
    if (same_run(d, dn)) {
      if (tid == 0) a.ws.nz[(size_t)bh * a.ws.nchunks + chunk] = 0;
    } else {
      if (run_any) {
#pragma unroll
        for (int j = 0; j < EPL; ++j) red[group][lane_in_row * EPL + j] = acc[j];
      }
      values_run_store<D, GROUPS>(a, red, run_any, bh, chunk);
#pragma unroll
      for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
      run_any = false;
    }
    __syncthreads();
  }
}

__global__ void halley_update_kernel(float* __restrict__ tau, const float* __restrict__ sums, int n, float beta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  tau[i] = halley_unbounded(tau[i], sums[(size_t)i * 3], sums[(size_t)i * 3 + 1], sums[(size_t)i * 3 + 2], beta);
}

// Fixed-slot work list from per-head token counts: slot (head, chunk), empty when the head
// has fewer tokens.  For callers that bring their own page tables.
__global__ void build_work_items_kernel(const int* __restrict__ tok_counts, int n_heads, int max_tokens,
                                        int chunks_per_head, unsigned long long* __restrict__ items) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_heads * chunks_per_head) return;
  const int bh = i / chunks_per_head, chunk = i % chunks_per_head;
  items[i] = make_item(bh, chunk, min(tok_counts[bh], max_tokens));
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

constexpr size_t kSmemBudget = 216 * 1024;   // dynamic shared memory a pipelined block may take

template <typename K>
inline bool allow_smem(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess;
}

// Few heads (a single long request): give each head a 1024-thread block.
template <typename T, int D, int THREADS>
void launch_tau_solve_threads(DecodeArgs a, int heads, cudaStream_t st) {
  constexpr int kRed = THREADS / (D / ElemTraits<T>::EPL) * D;      // floats of the gather's reduction buffer
  const int chunked = (a.max_tokens + kChunkTokens - 1) / kChunkTokens * kChunkTokens;
  a.solve_cap = std::min(kSolveSmemScores, std::max(chunked, kRed));
  const size_t smem = (size_t)a.solve_cap * sizeof(float);
  static bool once = allow_smem(tau_solve_kernel<T, D, THREADS>, kSolveSmemScores * sizeof(float));
  (void)once;
  tau_solve_kernel<T, D, THREADS><<<heads, THREADS, smem, st>>>(a);
}
template <typename T, int D>
void launch_tau_solve(const DecodeArgs& a, int heads, cudaStream_t st) {
  // few heads: one big block each.  Many short heads (their scores fit the shared copy): 128-thread blocks,
  // eight to an SM, so that a thousand heads are resident at once (41 -> 34 us at 1024 heads of 4112 tokens;
  // 512 threads: 58 us).  Many long heads scan their scores from L2 and want the wider block.
  const int chunked = (a.max_tokens + kChunkTokens - 1) / kChunkTokens * kChunkTokens;
  if (heads <= 2 * sm_count()) launch_tau_solve_threads<T, D, 1024>(a, heads, st);
  else if (chunked <= kSolveSmemScores) launch_tau_solve_threads<T, D, 128>(a, heads, st);
  else launch_tau_solve_threads<T, D, 256>(a, heads, st);
}

template <typename T, int D, int NS, bool ALIBI>
void launch_scores_pipe(const DecodeArgs& a, int blocks, size_t smem, cudaStream_t st) {
  static bool once = allow_smem(decode_scores_pipe_kernel<T, D, NS, ALIBI>, smem);
  (void)once;
  decode_scores_pipe_kernel<T, D, NS, ALIBI><<<blocks, kDecThreads, smem, st>>>(a);
}

// Group-shared K pass: 16-bit caches with head_dim 128, groups of four.
template <typename T, int D>
int launch_scores_group(const DecodeArgs& a, cudaStream_t st) {
  if constexpr (sizeof(T) == 2 && D == 128) {
    const size_t smem = 3 * kGroupStageBytes;
    static bool once = allow_smem(decode_scores_group_kernel<T, 3>, smem);
    (void)once;
    decode_scores_group_kernel<T, 3><<<sm_count(), kDecThreads, smem, st>>>(a);
    return launch_status();
  } else {
    return EKV_ERR_DTYPE;
  }
}

// The ALiBi variant of the pipelined K pass is a separate instantiation, so the default kernel
// carries none of its registers.
template <typename T, int D>
int launch_scores(const DecodeArgs& a, cudaStream_t st) {
  if (a.g_items) return launch_scores_group<T, D>(a, st);
  const size_t stage = (size_t)kChunkTokens * D * sizeof(T);
  const bool pipe = a.pd.shift >= 2 && a.pd.P <= 32;
  // one persistent block per SM: a grid of 2-16x more, shorter blocks measured slower (200 -> 206-243 us at 128k)
  const int blocks = sm_count();
  const bool ali = a.alibi != nullptr;
  if (!pipe) {
    decode_scores_plain_kernel<T, D><<<blocks * 2, kDecThreads, 0, st>>>(a);
  } else if (3 * stage <= kSmemBudget) {
    if (ali) launch_scores_pipe<T, D, 3, true>(a, blocks, 3 * stage, st);
    else launch_scores_pipe<T, D, 3, false>(a, blocks, 3 * stage, st);
  } else if (2 * stage <= kSmemBudget) {
    if (ali) launch_scores_pipe<T, D, 2, true>(a, blocks, 2 * stage, st);
    else launch_scores_pipe<T, D, 2, false>(a, blocks, 2 * stage, st);
  } else {
    if (ali) launch_scores_pipe<T, D, 1, true>(a, blocks, stage, st);
    else launch_scores_pipe<T, D, 1, false>(a, blocks, stage, st);
  }
  return launch_status();
}

template <typename T, int D>
int launch_values(const DecodeArgs& a, cudaStream_t st) {
  const size_t stage = (size_t)kChunkTokens * D * sizeof(T);
  const size_t red = (size_t)(kDecThreads / (D / ElemTraits<T>::EPL)) * D * sizeof(float);
  const bool pipe = a.pd.shift >= 2 && a.pd.P <= 32;
  const int blocks = sm_count();
  if (!pipe) {
    decode_values_plain_kernel<T, D><<<blocks * 2, kDecThreads, 0, st>>>(a);
  } else if (3 * stage + red <= kSmemBudget) {
    static bool once = allow_smem(decode_values_pipe_kernel<T, D, 3>, 3 * stage + red);
    (void)once;
    decode_values_pipe_kernel<T, D, 3><<<blocks, kDecThreads, 3 * stage + red, st>>>(a);
  } else if (2 * stage + red <= kSmemBudget) {
    static bool once = allow_smem(decode_values_pipe_kernel<T, D, 2>, 2 * stage + red);
    (void)once;
    decode_values_pipe_kernel<T, D, 2><<<blocks, kDecThreads, 2 * stage + red, st>>>(a);
  } else {
    static bool once = allow_smem(decode_values_pipe_kernel<T, D, 1>, stage + red);
    (void)once;
    decode_values_pipe_kernel<T, D, 1><<<blocks, kDecThreads, stage + red, st>>>(a);
  }
  return launch_status();
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

extern "C" int32_t ekv_work_items_per_head(int32_t max_tokens) {
  return max_tokens <= 0 ? 0 : (max_tokens + ekv::kChunkTokens - 1) / ekv::kChunkTokens;
}

extern "C" int ekv_build_work_items(const int32_t* tok_counts, int32_t n_heads, int32_t max_tokens,
                                    uint64_t* work_items, void* stream) {
  using namespace ekv;
  if (!tok_counts || !work_items || n_heads <= 0 || max_tokens <= 0) return EKV_ERR_ARG;
  const int cph = (max_tokens + kChunkTokens - 1) / kChunkTokens;
  if (cph > kItemMaxChunks || n_heads >= kItemMaxHeads) return EKV_ERR_ARG;
  const int n = n_heads * cph;
  build_work_items_kernel<<<(n + 255) / 256, 256, 0, as_stream(stream)>>>(
      tok_counts, n_heads, max_tokens, cph, reinterpret_cast<unsigned long long*>(work_items));
  return launch_status();
}

static int fill_decode_args(ekv::DecodeArgs& a, const ekv_cache_desc* c, int32_t q_heads,
                            const int32_t* page_indices, int64_t pi_stride, const int32_t* tok_counts,
                            int32_t max_tokens, float alpha, const uint64_t* work_items, int32_t n_items,
                            const int32_t* work_total, void* workspace, size_t workspace_bytes) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!page_indices || !tok_counts || !workspace || !work_items) return EKV_ERR_ARG;
  if (q_heads <= 0 || q_heads % c->kv_heads || max_tokens <= 0 || n_items <= 0) return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  if (decode_ws_layout(c->batch, q_heads, c->head_dim, max_tokens, workspace, &a.ws) > workspace_bytes)
    return EKV_ERR_WORKSPACE;
  if (a.ws.nchunks > kItemMaxChunks || (int64_t)c->batch * q_heads >= kItemMaxHeads) return EKV_ERR_ARG;
  a.c = *c;
  a.q_heads = q_heads;
  a.page_indices = page_indices;
  a.pi_stride = pi_stride;
  a.tok_counts = tok_counts;
  a.max_tokens = max_tokens;
  a.alpha = alpha;
  a.items = reinterpret_cast<const unsigned long long*>(work_items);
  a.work_total = work_total;
  a.n_items = n_items;
  a.pd = make_page_div(c->page_size);
  a.kv_sb = c->block_table ? 0 : c->kv_stride_b;
  a.kv_ps = c->block_table ? c->kv_stride_block : (int64_t)c->page_size * c->head_dim;
  a.page_limit = c->block_table ? c->num_blocks : c->page_capacity;
  a.div_heads = make_fast_div(q_heads);
  a.div_group = make_fast_div(q_heads / c->kv_heads);
  return EKV_OK;
}

extern "C" int ekv_decode_scores(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                 int64_t q_stride_h, int32_t q_heads, const int32_t* page_indices,
                                 int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens,
                                 float alpha, int32_t tau_mode, int32_t niter, float* tau,
                                 float* halley_sums, const uint64_t* work_items, int32_t n_items,
                                 const int32_t* work_total, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  using namespace ekv;
  DecodeArgs a{};
  if (int e = fill_decode_args(a, c, q_heads, page_indices, pi_stride, tok_counts, max_tokens, alpha,
                               work_items, n_items, work_total, workspace, workspace_bytes))
    return e;
  if (!q || !tau || niter < 0) return EKV_ERR_ARG;
  if (tau_mode < EKV_TAU_NONE || tau_mode > EKV_TAU_CORRECTED) return EKV_ERR_ARG;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((q_stride_b * esz) % 16 || (q_stride_h * esz) % 16 || (reinterpret_cast<uintptr_t>(q) & 15))
    return EKV_ERR_ARG;
  a.q = q;
  a.qsb = q_stride_b;
  a.qsh = q_stride_h;
  a.tau_mode = tau_mode;
  a.niter = niter;
  a.tau = tau;
  a.halley_sums = halley_sums;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    if (int e = launch_scores<T, D>(a, as_stream(stream))) return e;
    launch_tau_solve<T, D>(a, c->batch * q_heads, as_stream(stream));
  });
  return launch_status();
}

static int decode_all(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                      int32_t q_heads, const int32_t* page_indices, int64_t pi_stride,
                      const int32_t* tok_counts, int32_t max_tokens, float alpha, int32_t tau_mode,
                      int32_t niter, float* tau, void* out, int64_t out_stride_b, int64_t out_stride_h,
                      const uint64_t* work_items, int32_t n_items, const int32_t* work_total,
                      void* workspace, size_t workspace_bytes, void** stage_events,
                      const float* alibi_slopes, const int32_t* q_positions, void* stream,
                      const uint64_t* group_items = nullptr, int32_t n_group_items = 0,
                      const uint8_t* member = nullptr, int64_t member_stride = 0) {
  using namespace ekv;
  DecodeArgs a{};
  a.alibi = alibi_slopes;
  a.q_pos = q_positions;
  a.g_items = reinterpret_cast<const unsigned long long*>(group_items);
  a.g_n_items = n_group_items;
  a.member = member;
  a.member_stride = member_stride;
  if (alibi_slopes && c && c->block_table) return EKV_ERR_ARG;   // token positions need page numbers
  if (group_items && (!member || n_group_items <= 0 || q_heads != 4 * c->kv_heads || alibi_slopes ||
                      c->page_size > 32 || (c->page_size & (c->page_size - 1)) || c->page_size < 4))
    return EKV_ERR_ARG;
  if (int e = fill_decode_args(a, c, q_heads, page_indices, pi_stride, tok_counts, max_tokens, alpha,
                               work_items, n_items, work_total, workspace, workspace_bytes))
    return e;
  if (!q || !tau || !out || niter < 0) return EKV_ERR_ARG;
  if (tau_mode != EKV_TAU_EXACT && tau_mode != EKV_TAU_CORRECTED) return EKV_ERR_ARG;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((q_stride_b * esz) % 16 || (q_stride_h * esz) % 16 || (reinterpret_cast<uintptr_t>(q) & 15))
    return EKV_ERR_ARG;
  a.q = q;
  a.qsb = q_stride_b;
  a.qsh = q_stride_h;
  a.tau_mode = tau_mode;
  a.niter = niter;
  a.tau = tau;
  a.out = out;
  a.osb = out_stride_b;
  a.osh = out_stride_h;
  a.out_is_f32 = 0;
  cudaStream_t st = as_stream(stream);
  auto mark = [&](int i) {
    if (stage_events && stage_events[i]) cudaEventRecord(static_cast<cudaEvent_t>(stage_events[i]), st);
  };
  EKV_DISPATCH(c->dtype, c->head_dim, {
    if (int e = launch_scores<T, D>(a, st)) return e;
    mark(0);
    launch_tau_solve<T, D>(a, c->batch * q_heads, st);
    mark(1);
    if (int e = launch_values<T, D>(a, st)) return e;
    mark(2);
    out_reduce_kernel<T, D><<<c->batch * q_heads, D, 0, st>>>(a);
  });
  return launch_status();
}

namespace ekv {

// Slot 2: sum of every rank's Halley sums, then the unbracketed step on tau (in place).
__global__ void __launch_bounds__(kXchThreads)
xch_halley_kernel(const XchDev x, float* __restrict__ tau, const float* __restrict__ sums_local, int n, float beta,
                  int* status) {
  Xch e = xch_begin(x, 2, status);
  for (int i = threadIdx.x; i < n * 3; i += blockDim.x) e.send(i, sums_local[i]);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float s0 = e.sum(i * 3, sums_local[i * 3]);
    const float s1 = e.sum(i * 3 + 1, sums_local[i * 3 + 1]);
    const float s2 = e.sum(i * 3 + 2, sums_local[i * 3 + 2]);
    tau[i] = halley_unbounded(tau[i], s0, s1, s2, beta);
  }
}

// Slot 3: sum of every rank's fp32 partial outputs, rounded once to the output dtype.
// Any grid: a thread exchanges the elements it stores.
template <typename T>
__global__ void __launch_bounds__(kXchThreads)
xch_output_kernel(const XchDev x, const float* __restrict__ partial_local, int n_heads, int head_dim,
                  T* __restrict__ out, int64_t out_stride_h, int* status) {
  const int n = n_heads * head_dim;
  Xch e = xch_begin(x, 3, status);
  const int first = blockIdx.x * blockDim.x + threadIdx.x, stride = gridDim.x * blockDim.x;
  for (int i = first; i < n; i += stride) e.send(i, partial_local[i]);
  for (int i = first; i < n; i += stride)
    out[(size_t)(i / head_dim) * out_stride_h + (i % head_dim)] = from_float<T>(e.sum(i, partial_local[i]));
}

}  // namespace ekv

namespace ekv {

// Slot 3 of the sharded step, with the chunk fold in front: a head's local partial output is
// either the row the tau kernel gathered (cnt_v != 0) or the sum of the V pass's chunk slots;
// the ranks' partials are then combined and rounded once.  One element per thread.
template <typename OutT>
__global__ void __launch_bounds__(kXchThreads)
xch_fold_output_kernel(const DecodeArgs a, const float* __restrict__ gathered, OutT* __restrict__ out,
                       int64_t osb, int64_t osh) {
  Xch e = xch_begin(a.xch, 3, a.xch_status);
  const int D = a.c.head_dim;
  const int n = a.c.batch * a.q_heads * D;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int bh = i / D, d = i % D;
  float v = 0.f;
  if (a.ws.cnt_v[bh] != 0) {
    v = gathered[i];
  } else {
    const int T_tok = min(a.tok_counts[bh], a.max_tokens);
    const int nch = T_tok > 0 ? (T_tok + kChunkTokens - 1) / kChunkTokens : 0;
    const int* nz = a.ws.nz + (size_t)bh * a.ws.nchunks;
    const float* po = a.ws.pout + (size_t)bh * a.ws.nchunks * D;
    for (int ch = 0; ch < nch; ++ch)
      if (nz[ch]) v += po[(size_t)ch * D + d];
  }
  e.send(i, v);
  const int b = bh / a.q_heads, hq = bh % a.q_heads;
  out[(size_t)b * osb + (size_t)hq * osh + d] = from_float<OutT>(e.sum(i, v));
}

}  // namespace ekv

extern "C" int ekv_exchange_decode(ekv_exchange* x, const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                   int64_t q_stride_h, int32_t q_heads, const int32_t* page_indices,
                                   int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens,
                                   float alpha, int32_t niter, float* tau, float* gathered, void* out,
                                   int64_t out_stride_b, int64_t out_stride_h, int32_t out_dtype,
                                   const uint64_t* work_items, int32_t n_items, const int32_t* work_total,
                                   void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  using namespace ekv;
  DecodeArgs a{};
  if (int e = fill_decode_args(a, c, q_heads, page_indices, pi_stride, tok_counts, max_tokens, alpha,
                               work_items, n_items, work_total, workspace, workspace_bytes))
    return e;
  if (!xch_device_view(x, &a.xch) || !q || !tau || !gathered || !out || !status || niter < 0 || niter > 1)
    return EKV_ERR_ARG;
  const int64_t n_out = (int64_t)c->batch * q_heads * c->head_dim;
  if (n_out > a.xch.max_floats || (int64_t)c->batch * q_heads > kXchMaxBlocks) return EKV_ERR_ARG;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((q_stride_b * esz) % 16 || (q_stride_h * esz) % 16 || (reinterpret_cast<uintptr_t>(q) & 15))
    return EKV_ERR_ARG;
  if (out_dtype != EKV_F32 && out_dtype != EKV_F16 && out_dtype != EKV_BF16) return EKV_ERR_DTYPE;
  a.q = q;
  a.qsb = q_stride_b;
  a.qsh = q_stride_h;
  a.tau_mode = EKV_TAU_CORRECTED;
  a.niter = niter;
  a.tau = tau;
  a.out = gathered;                      // rows gathered by the tau kernel: fp32 [B, H_q, D]
  a.osb = (int64_t)q_heads * c->head_dim;
  a.osh = c->head_dim;
  a.out_is_f32 = 1;
  a.use_xch = 1;
  a.xch_status = status;
  cudaStream_t st = as_stream(stream);
  const int blocks = (int)((n_out + kXchThreads - 1) / kXchThreads);
  EKV_DISPATCH(c->dtype, c->head_dim, {
    if (int e = launch_scores<T, D>(a, st)) return e;
    launch_tau_solve<T, D>(a, c->batch * q_heads, st);
    if (int e = launch_values<T, D>(a, st)) return e;
  });
  if (out_dtype == EKV_F32)
    xch_fold_output_kernel<float><<<blocks, kXchThreads, 0, st>>>(a, gathered, static_cast<float*>(out),
                                                                  out_stride_b, out_stride_h);
  else if (out_dtype == EKV_F16)
    xch_fold_output_kernel<__half><<<blocks, kXchThreads, 0, st>>>(a, gathered, static_cast<__half*>(out),
                                                                   out_stride_b, out_stride_h);
  else
    xch_fold_output_kernel<__nv_bfloat16><<<blocks, kXchThreads, 0, st>>>(
        a, gathered, static_cast<__nv_bfloat16*>(out), out_stride_b, out_stride_h);
  return launch_status();
}

extern "C" int ekv_exchange_halley_update(ekv_exchange* x, float* tau, const float* halley_sums_local,
                                          int32_t n, float alpha, int32_t* status, void* stream) {
  using namespace ekv;
  XchDev d;
  if (!xch_device_view(x, &d) || !tau || !halley_sums_local || !status || n <= 0 ||
      (int64_t)n * 3 > d.max_floats)
    return EKV_ERR_ARG;
  if (!(alpha > 1.f)) return EKV_ERR_ALPHA;
  xch_halley_kernel<<<1, kXchThreads, 0, as_stream(stream)>>>(d, tau, halley_sums_local, n, 1.f / (alpha - 1.f),
                                                             status);
  return launch_status();
}

extern "C" int ekv_exchange_output(ekv_exchange* x, const float* partial_local, int32_t n_heads,
                                   int32_t head_dim, void* out, int64_t out_stride_h, int32_t out_dtype,
                                   int32_t* status, void* stream) {
  using namespace ekv;
  XchDev d;
  if (!xch_device_view(x, &d) || !partial_local || !out || !status || n_heads <= 0 || head_dim <= 0 ||
      out_stride_h < head_dim || (int64_t)n_heads * head_dim > d.max_floats)
    return EKV_ERR_ARG;
  cudaStream_t st = as_stream(stream);
  const int blocks = (n_heads * head_dim + kXchThreads - 1) / kXchThreads;
  if (out_dtype == EKV_F32)
    xch_output_kernel<float><<<blocks, kXchThreads, 0, st>>>(d, partial_local, n_heads, head_dim,
                                                        static_cast<float*>(out), out_stride_h, status);
  else if (out_dtype == EKV_F16)
    xch_output_kernel<__half><<<blocks, kXchThreads, 0, st>>>(d, partial_local, n_heads, head_dim,
                                                         static_cast<__half*>(out), out_stride_h, status);
  else if (out_dtype == EKV_BF16)
    xch_output_kernel<__nv_bfloat16><<<blocks, kXchThreads, 0, st>>>(d, partial_local, n_heads, head_dim,
                                                                static_cast<__nv_bfloat16*>(out), out_stride_h,
                                                                status);
  else
    return EKV_ERR_DTYPE;
  return launch_status();
}

extern "C" int ekv_decode(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                          int32_t q_heads, const int32_t* page_indices, int64_t pi_stride,
                          const int32_t* tok_counts, int32_t max_tokens, float alpha, int32_t tau_mode,
                          int32_t niter, float* tau, void* out, int64_t out_stride_b, int64_t out_stride_h,
                          const uint64_t* work_items, int32_t n_items, const int32_t* work_total,
                          void* workspace, size_t workspace_bytes, void** stage_events, void* stream) {
  return decode_all(c, q, q_stride_b, q_stride_h, q_heads, page_indices, pi_stride, tok_counts, max_tokens, alpha,
                    tau_mode, niter, tau, out, out_stride_b, out_stride_h, work_items, n_items, work_total,
                    workspace, workspace_bytes, stage_events, nullptr, nullptr, stream);
}

extern "C" int ekv_group_union(const ekv_cache_desc* c, int32_t q_heads, const int32_t* page_indices,
                               int64_t pi_stride, const int32_t* num_selected, int32_t max_tokens,
                               int32_t* union_pages, int64_t union_stride, uint8_t* member,
                               int64_t member_stride, int32_t* union_tok_counts, uint64_t* group_items,
                               int32_t n_group_items, void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!page_indices || !num_selected || !union_pages || !member || !union_tok_counts || !group_items)
    return EKV_ERR_ARG;
  if (q_heads != 4 * c->kv_heads || max_tokens <= 0) return EKV_ERR_ARG;
  const int cph = (max_tokens + kChunkTokens - 1) / kChunkTokens;
  const int groups = c->batch * c->kv_heads;
  if (cph > kItemMaxChunks || (int64_t)c->batch * q_heads >= kItemMaxHeads) return EKV_ERR_ARG;
  if (n_group_items != groups * cph || union_stride < c->page_capacity || member_stride < c->page_capacity)
    return EKV_ERR_ARG;
  const size_t smem = 4 * (size_t)((c->page_capacity + 31) / 32) * sizeof(uint32_t);
  if (smem > 180 * 1024) return EKV_ERR_ARG;
  static bool once = cudaFuncSetAttribute(group_union_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          180 * 1024) == cudaSuccess;
  (void)once;
  group_union_kernel<<<groups, kUnionThreads, smem, as_stream(stream)>>>(
      *c, q_heads, page_indices, pi_stride, num_selected, max_tokens, union_pages, union_stride, member,
      member_stride, union_tok_counts, reinterpret_cast<unsigned long long*>(group_items), cph);
  return launch_status();
}

extern "C" int ekv_decode_grouped(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                  int32_t q_heads, const int32_t* union_pages, int64_t union_stride,
                                  const int32_t* union_tok_counts, int32_t max_tokens, float alpha,
                                  int32_t tau_mode, int32_t niter, float* tau, void* out, int64_t out_stride_b,
                                  int64_t out_stride_h, const uint64_t* head_items, int32_t n_head_items,
                                  const uint64_t* group_items, int32_t n_group_items, const uint8_t* member,
                                  int64_t member_stride, void* workspace, size_t workspace_bytes,
                                  void** stage_events, void* stream) {
  if (!group_items || !member) return EKV_ERR_ARG;
  return decode_all(c, q, q_stride_b, q_stride_h, q_heads, union_pages, union_stride, union_tok_counts, max_tokens,
                    alpha, tau_mode, niter, tau, out, out_stride_b, out_stride_h, head_items, n_head_items, nullptr,
                    workspace, workspace_bytes, stage_events, nullptr, nullptr, stream, group_items, n_group_items,
                    member, member_stride);
}

extern "C" int ekv_decode_alibi(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                int32_t q_heads, const int32_t* page_indices, int64_t pi_stride,
                                const int32_t* tok_counts, int32_t max_tokens, float alpha, int32_t tau_mode,
                                int32_t niter, float* tau, void* out, int64_t out_stride_b,
                                int64_t out_stride_h, const uint64_t* work_items, int32_t n_items,
                                const int32_t* work_total, void* workspace, size_t workspace_bytes,
                                void** stage_events, const float* alibi_slopes, const int32_t* q_positions,
                                void* stream) {
  if (!alibi_slopes) return EKV_ERR_ARG;
  return decode_all(c, q, q_stride_b, q_stride_h, q_heads, page_indices, pi_stride, tok_counts, max_tokens, alpha,
                    tau_mode, niter, tau, out, out_stride_b, out_stride_h, work_items, n_items, work_total,
                    workspace, workspace_bytes, stage_events, alibi_slopes, q_positions, stream);
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
                                 int64_t out_stride_h, int32_t out_is_f32, const uint64_t* work_items,
                                 int32_t n_items, const int32_t* work_total, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  using namespace ekv;
  DecodeArgs a{};
  if (int e = fill_decode_args(a, c, q_heads, page_indices, pi_stride, tok_counts, max_tokens, alpha,
                               work_items, n_items, work_total, workspace, workspace_bytes))
    return e;
  if (!tau || !out) return EKV_ERR_ARG;
  a.tau = const_cast<float*>(tau);
  a.out = out;
  a.osb = out_stride_b;
  a.osh = out_stride_h;
  a.out_is_f32 = out_is_f32;
  // tau is final here: heads whose support is small get their few value rows gathered by the
  // tau kernel (no iterations, tau left as it is); the streaming V pass then only sees the
  // heads with a large support, as in the fused ekv_decode.
  a.tau_mode = EKV_TAU_CORRECTED;
  a.niter = 0;
  a.halley_sums = nullptr;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    launch_tau_solve<T, D>(a, c->batch * q_heads, as_stream(stream));
    if (int e = launch_values<T, D>(a, as_stream(stream))) return e;
    out_reduce_kernel<T, D><<<c->batch * q_heads, D, 0, as_stream(stream)>>>(a);
  });
  return launch_status();
}

extern "C" int ekv_decode_support_counts(const void* workspace, size_t workspace_bytes, int32_t batch,
                                         int32_t q_heads, int32_t head_dim, int32_t max_tokens,
                                         int32_t* counts, void* stream) {
  using namespace ekv;
  if (!workspace || !counts || batch <= 0 || q_heads <= 0 || head_dim <= 0 || max_tokens <= 0) return EKV_ERR_ARG;
  DecodeWs ws;
  if (decode_ws_layout(batch, q_heads, head_dim, max_tokens, const_cast<void*>(workspace), &ws) > workspace_bytes)
    return EKV_ERR_WORKSPACE;
  cudaError_t e = cudaMemcpyAsync(counts, ws.support, (size_t)batch * q_heads * sizeof(int32_t),
                                  cudaMemcpyDeviceToDevice, as_stream(stream));
  return e == cudaSuccess ? EKV_OK : (int)e;
}

extern "C" int ekv_read_status(const void* workspace, int32_t* host_status, void* stream) {
  if (!workspace || !host_status) return EKV_ERR_ARG;
  cudaError_t e = cudaMemcpyAsync(host_status, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                  ekv::as_stream(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(ekv::as_stream(stream));
  return e == cudaSuccess ? EKV_OK : (int)e;
}
