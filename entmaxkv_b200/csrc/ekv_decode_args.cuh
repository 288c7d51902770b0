// Paged entmax decode: workspace layout, the argument block every decode kernel takes, and the per-run
// store epilogues shared by the pipelined and the plain kernels.
#pragma once

#include "ekv_common.cuh"
#include "ekv_work.cuh"
#include "ekv_exchange.cuh"

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

}  // namespace ekv
