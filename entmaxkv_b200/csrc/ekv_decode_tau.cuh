// Paged entmax decode: tau of one head from its kept scores (histogram bracket, Halley steps, optional
// exchange with the other ranks of a sequence-sharded step), the inline gather of small supports, and the
// output reduction over a head's chunks.
#pragma once

#include "ekv_decode_args.cuh"
#include "ekv_tau_math.cuh"

namespace ekv {

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

}  // namespace ekv
