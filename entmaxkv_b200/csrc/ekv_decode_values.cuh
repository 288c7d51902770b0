// Paged entmax decode, V pass: only pages that hold a token with a non-zero weight are fetched.
#pragma once

#include "ekv_decode_args.cuh"

namespace ekv {

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
      mbar_wait_or_flag(&full[st], (phase_bits >> st) & 1u, a.ws.status);
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

// ---- plain variant (any page size) ------------------

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

}  // namespace ekv
