// Paged entmax decode, K pass over per-head page tables: the pipelined kernel (one bulk copy per page into
// a shared-memory ring) and the plain variant for page sizes the ring does not serve.
#pragma once

#include "ekv_decode_args.cuh"

namespace ekv {

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
      mbar_wait_or_flag(&full[st], (phase_bits >> st) & 1u, a.ws.status);
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

// ---- plain variant (any page size): vectorised global loads, no staging ------------------

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

}  // namespace ekv
