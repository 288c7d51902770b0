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
//
// Kernels by family: ekv_decode_tau.cuh (tau solve, output reduction), ekv_decode_scores.cuh (K pass),
// ekv_decode_group.cuh (group-shared K pass), ekv_decode_values.cuh (V pass); this file holds the launchers,
// the C entry points and the exchange epilogues of the sequence-sharded step.
#include <algorithm>
#include <type_traits>

#include "ekv_decode_args.cuh"
#include "ekv_decode_tau.cuh"
#include "ekv_decode_scores.cuh"
#include "ekv_decode_group.cuh"
#include "ekv_decode_values.cuh"

namespace ekv {

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
  // as many heads as SMs or fewer: one big block each (a 1024-thread block fills an SM, so one head more than
  // that would start a second wave: 39 -> 28 us at 256 short heads).  Many short heads (their scores fit the shared copy): 128-thread blocks,
  // eight to an SM, so that a thousand heads are resident at once (41 -> 34 us at 1024 heads of 4112 tokens;
  // 512 threads: 58 us).  Many long heads scan their scores from L2 and want the wider block.
  const int chunked = (a.max_tokens + kChunkTokens - 1) / kChunkTokens * kChunkTokens;
  if (heads <= sm_count()) launch_tau_solve_threads<T, D, 1024>(a, heads, st);
  else if (chunked <= kSolveSmemScores) launch_tau_solve_threads<T, D, 128>(a, heads, st);
  else launch_tau_solve_threads<T, D, 256>(a, heads, st);
}

template <typename T, int D, int NS, bool ALIBI>
void launch_scores_pipe(const DecodeArgs& a, int blocks, size_t smem, cudaStream_t st) {
  static bool once = allow_smem(decode_scores_pipe_kernel<T, D, NS, ALIBI>, smem);
  (void)once;
  decode_scores_pipe_kernel<T, D, NS, ALIBI><<<blocks, kDecThreads, smem, st>>>(a);
}

// Group-shared K pass: 16-bit caches with head_dim 128, groups of four or eight.
template <typename T, int D>
int launch_scores_group(const DecodeArgs& a, cudaStream_t st) {
  if constexpr (sizeof(T) == 2 && D == 128) {
    const size_t smem = 3 * kGroupStageBytes;
    if (a.q_heads == 8 * a.c.kv_heads) {
      static bool once = allow_smem(decode_scores_group_kernel<T, 3, 8>, smem);
      (void)once;
      decode_scores_group_kernel<T, 3, 8><<<sm_count(), kDecThreads, smem, st>>>(a);
    } else {
      static bool once = allow_smem(decode_scores_group_kernel<T, 3, 4>, smem);
      (void)once;
      decode_scores_group_kernel<T, 3, 4><<<sm_count(), kDecThreads, smem, st>>>(a);
    }
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
  if (group_items && (!member || n_group_items <= 0 || (q_heads != 4 * c->kv_heads && q_heads != 8 * c->kv_heads) || alibi_slopes ||
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

static int exchange_decode_impl(ekv_exchange* x, const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                int64_t q_stride_h, int32_t q_heads, const int32_t* page_indices,
                                int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens,
                                float alpha, int32_t niter, float* tau, float* gathered, void* out,
                                int64_t out_stride_b, int64_t out_stride_h, int32_t out_dtype,
                                const uint64_t* work_items, int32_t n_items, const int32_t* work_total,
                                void* workspace, size_t workspace_bytes, int32_t* status, void* stream,
                                const uint64_t* group_items, int32_t n_group_items, const uint8_t* member,
                                int64_t member_stride) {
  using namespace ekv;
  DecodeArgs a{};
  if (group_items) {
    if (!c || !member || n_group_items <= 0 || (q_heads != 4 * c->kv_heads && q_heads != 8 * c->kv_heads) ||
        c->page_size > 32 || (c->page_size & (c->page_size - 1)) || c->page_size < 4 ||
        c->dtype == EKV_F32 || c->head_dim != 128)
      return EKV_ERR_ARG;
    a.g_items = reinterpret_cast<const unsigned long long*>(group_items);
    a.g_n_items = n_group_items;
    a.member = member;
    a.member_stride = member_stride;
  }
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

extern "C" int ekv_exchange_decode(ekv_exchange* x, const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                                   int64_t q_stride_h, int32_t q_heads, const int32_t* page_indices,
                                   int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens,
                                   float alpha, int32_t niter, float* tau, float* gathered, void* out,
                                   int64_t out_stride_b, int64_t out_stride_h, int32_t out_dtype,
                                   const uint64_t* work_items, int32_t n_items, const int32_t* work_total,
                                   void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  return exchange_decode_impl(x, c, q, q_stride_b, q_stride_h, q_heads, page_indices, pi_stride, tok_counts, max_tokens,
                              alpha, niter, tau, gathered, out, out_stride_b, out_stride_h, out_dtype, work_items,
                              n_items, work_total, workspace, workspace_bytes, status, stream, nullptr, 0, nullptr, 0);
}

extern "C" int ekv_exchange_decode_grouped(ekv_exchange* x, const ekv_cache_desc* c, const void* q,
                                           int64_t q_stride_b, int64_t q_stride_h, int32_t q_heads,
                                           const int32_t* union_pages, int64_t union_stride,
                                           const int32_t* union_tok_counts, int32_t max_tokens, float alpha,
                                           int32_t niter, float* tau, float* gathered, void* out,
                                           int64_t out_stride_b, int64_t out_stride_h, int32_t out_dtype,
                                           const uint64_t* head_items, int32_t n_head_items,
                                           const uint64_t* group_items, int32_t n_group_items,
                                           const uint8_t* member, int64_t member_stride, void* workspace,
                                           size_t workspace_bytes, int32_t* status, void* stream) {
  if (!group_items || !member) return EKV_ERR_ARG;
  return exchange_decode_impl(x, c, q, q_stride_b, q_stride_h, q_heads, union_pages, union_stride, union_tok_counts,
                              max_tokens, alpha, niter, tau, gathered, out, out_stride_b, out_stride_h, out_dtype,
                              head_items, n_head_items, nullptr, workspace, workspace_bytes, status, stream, group_items,
                              n_group_items, member, member_stride);
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
                               int32_t n_group_items, uint64_t* head_items, void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!page_indices || !num_selected || !union_pages || !member || !union_tok_counts || !group_items)
    return EKV_ERR_ARG;
  const int gs = q_heads / c->kv_heads;
  if ((gs != 4 && gs != 8) || q_heads != gs * c->kv_heads || max_tokens <= 0) return EKV_ERR_ARG;
  const int cph = (max_tokens + kChunkTokens - 1) / kChunkTokens;
  const int groups = c->batch * c->kv_heads;
  if (cph > kItemMaxChunks || (int64_t)c->batch * q_heads >= kItemMaxHeads) return EKV_ERR_ARG;
  if (n_group_items != groups * cph || union_stride < c->page_capacity || member_stride < c->page_capacity)
    return EKV_ERR_ARG;
  const size_t smem = gs * (size_t)((c->page_capacity + 31) / 32) * sizeof(uint32_t);
  if (smem > 180 * 1024) return EKV_ERR_ARG;
  // few groups (one long request): a cluster of eight blocks per group, each on an eighth of the page ids
  constexpr int CL = 8;
  if (groups * CL <= 2 * sm_count()) {
    const int seg = ((c->page_capacity + CL - 1) / CL + 31) / 32 * 32;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(groups * CL));
    cfg.blockDim = dim3(kUnionThreads);
    cfg.dynamicSmemBytes = (size_t)gs * (seg / 32) * sizeof(uint32_t);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    auto items = reinterpret_cast<unsigned long long*>(group_items);
    auto hitems = reinterpret_cast<unsigned long long*>(head_items);
    cudaError_t e;
    if (gs == 8) {
      static bool once = cudaFuncSetAttribute(group_union_cluster_kernel<8, CL>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 180 * 1024) == cudaSuccess;
      (void)once;
      e = cudaLaunchKernelEx(&cfg, group_union_cluster_kernel<8, CL>, *c, (int)q_heads, page_indices, pi_stride,
                             num_selected, (int)max_tokens, union_pages, union_stride, member, member_stride,
                             union_tok_counts, items, cph, hitems);
    } else {
      static bool once = cudaFuncSetAttribute(group_union_cluster_kernel<4, CL>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 180 * 1024) == cudaSuccess;
      (void)once;
      e = cudaLaunchKernelEx(&cfg, group_union_cluster_kernel<4, CL>, *c, (int)q_heads, page_indices, pi_stride,
                             num_selected, (int)max_tokens, union_pages, union_stride, member, member_stride,
                             union_tok_counts, items, cph, hitems);
    }
    if (e != cudaSuccess) return (int)e;
    return launch_status();
  }
  if (gs == 8) {
    static bool once = cudaFuncSetAttribute(group_union_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            180 * 1024) == cudaSuccess;
    (void)once;
    group_union_kernel<8><<<groups, kUnionThreads, smem, as_stream(stream)>>>(
        *c, q_heads, page_indices, pi_stride, num_selected, max_tokens, union_pages, union_stride, member,
        member_stride, union_tok_counts, reinterpret_cast<unsigned long long*>(group_items), cph,
        reinterpret_cast<unsigned long long*>(head_items));
  } else {
    static bool once = cudaFuncSetAttribute(group_union_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            180 * 1024) == cudaSuccess;
    (void)once;
    group_union_kernel<4><<<groups, kUnionThreads, smem, as_stream(stream)>>>(
        *c, q_heads, page_indices, pi_stride, num_selected, max_tokens, union_pages, union_stride, member,
        member_stride, union_tok_counts, reinterpret_cast<unsigned long long*>(group_items), cph,
        reinterpret_cast<unsigned long long*>(head_items));
  }
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

namespace ekv {
unsigned int copy_timeouts_decode() { return copy_timeouts_here(); }
}  // namespace ekv
