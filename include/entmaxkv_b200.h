/*
 * entmaxkv_b200 - C ABI of the B200 (sm_100a) sparse entmax decode step.
 *
 * Every entry point
 *   - takes raw device pointers, sizes and element strides (no framework types),
 *   - enqueues its kernels on the given CUDA stream and returns without
 *     synchronising,
 *   - allocates nothing: scratch comes from the caller (size queries below),
 *   - returns 0 on success, a negative EKV_ERR_* for an argument error found on
 *     the host, or the (positive) cudaError_t of a failed launch.
 * Device-side range checks never trap; they set bits in the int32 status word
 * at the start of the decode workspace (read it with ekv_read_status).
 *
 * Layouts (element strides, innermost dimension D contiguous):
 *   K, V              [B, H_kv, capacity,       D]   rows of a page are contiguous
 *                     or, with a block table, [num_blocks, H_kv, page_size, D] (see ekv_cache_desc)
 *   k_min ... k_std   [B, H_kv, page_capacity,  D]
 *   q, out            [B, H_q, 1, D]
 *   seq_lens          int32 [B] on the device: tokens currently in each sequence
 * Query head h reads KV head h / (H_q / H_kv); page tables and token counts are
 * kept per QUERY head.
 *
 * The reference project is pure Python + Triton; the citations name the
 * reference function each entry point stands in for.
 */
#ifndef ENTMAXKV_B200_H
#define ENTMAXKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { EKV_F16 = 0, EKV_BF16 = 1, EKV_F32 = 2 };

enum {
  EKV_OK = 0,
  EKV_ERR_DTYPE = -1,      /* unsupported dtype / head_dim combination */
  EKV_ERR_ARG = -2,        /* null pointer, non-positive size, bad stride */
  EKV_ERR_WORKSPACE = -3,  /* workspace too small */
  EKV_ERR_ALPHA = -4,      /* alpha <= 1 */
  EKV_ERR_STATIC_LIMIT = -5 /* more sequences than ekv_append_static has built-in counters for */
};

/* bits of the device status word */
enum {
  EKV_STATUS_PAGE_RANGE = 1,   /* a page id outside [0, page_capacity) was skipped */
  EKV_STATUS_CAPACITY = 2,     /* append past capacity was dropped */
  EKV_STATUS_TOKENS = 4,       /* a token count above the workspace bound was clipped */
  EKV_STATUS_PEER_TIMEOUT = 8, /* a peer exchange gave up waiting for another rank */
  EKV_STATUS_COPY_TIMEOUT = 16 /* a bulk copy did not land within its bounded wait: that launch's results are undefined */
};

/* tau procedures of the decode (ekv_decode_scores) */
enum {
  EKV_TAU_NONE = 0,      /* leave tau untouched; per-head Halley sums are written out */
  EKV_TAU_EXACT = 1,     /* max -> 16-bin histogram -> bracket -> niter bracketed Halley steps */
  EKV_TAU_CORRECTED = 2  /* start from tau[], take `niter` unbracketed Halley/Newton steps */
};

typedef struct ekv_cache_desc {
  void* k;                 /* [B, H_kv, capacity, D] */
  void* v;
  void* k_min;             /* [B, H_kv, page_capacity, D] */
  void* k_max;
  void* k_mean;
  void* k_std;
  int32_t* seq_lens;       /* [B] device */
  int64_t kv_stride_b, kv_stride_h;       /* elements */
  int64_t meta_stride_b, meta_stride_h;   /* elements */
  int32_t batch, kv_heads, head_dim, page_size;
  int32_t capacity;        /* rows allocated per (b, h) */
  int32_t page_capacity;   /* pages allocated per (b, h) */
  int32_t dtype;           /* EKV_F16 / EKV_BF16 / EKV_F32 */
  int32_t reserved;
  /* Block-table layout (optional; block_table == NULL: the dense layout above).  K and V are then pools
   * of physical blocks of page_size rows: page p of sequence b lives in block
   * block_table[b*bt_stride + p], and row r of that page of KV head h starts at element
   * block*kv_stride_block + h*kv_stride_h + r*D of k / v (kv_stride_b is not used).  The page
   * statistics stay dense per (b, h) and are indexed by the page number p. */
  const int32_t* block_table;   /* device int32 [B, bt_stride], entries in [0, num_blocks) */
  int64_t bt_stride;
  int64_t kv_stride_block;      /* elements between consecutive physical blocks */
  int32_t num_blocks;
  int32_t reserved2;
} ekv_cache_desc;

/* ---- cache ------------------------------------------------------------- */

/* min / max / mean / population-std (clamped at 1e-6) of every page of K.
 * Stands in for PagedKVCache.initialize, entmaxkv/kv_cache.py:47-70
 * (a Python loop over pages there; one launch here). */
int ekv_page_stats_init(const ekv_cache_desc* c, int32_t max_seq_len, void* stream);

/* Append one token per sequence in place and refresh the statistics of the page
 * it lands in; seq_lens[b] is incremented on the device.
 * Stands in for PagedKVCache.append, entmaxkv/kv_cache.py:72-116.
 * k_new / v_new: [B, H_kv, 1, D] with the given batch / head strides.
 * counters: int32 [B], zero before the first call, left zero by every call. */
int ekv_append(const ekv_cache_desc* c, const void* k_new, const void* v_new,
               int64_t new_stride_b, int64_t new_stride_h, int32_t* counters,
               int32_t* status, void* stream);

/* ekv_append for callers that cannot allocate device memory (a server whose memory
 * arena was sized at start-up, a step that runs where cudaMalloc is not allowed): the
 * per-sequence ticket counters that ekv_append takes from the caller live here in a fixed
 * array inside the library image, EKV_APPEND_STATIC_MAX_BATCH entries (16 KiB, resident on
 * every GPU that loads the library until the process exits).  The call allocates nothing;
 * batches larger than the limit are refused with EKV_ERR_STATIC_LIMIT.
 * The first call on a device looks up the array's device address; make that first call
 * before any stream capture begins.  All calls on a device share the array (each clears
 * the slots it uses), so calls that may overlap on the GPU must be ordered by the caller.
 * `stream` must belong to the device that is current at the call (the array of that device
 * is the one used).  If the host resets the device (cudaDeviceReset) between calls, the next
 * call notices the stale address and looks it up again.
 * It has no counterpart in the reference; results are identical to ekv_append. */
#define EKV_APPEND_STATIC_MAX_BATCH 4096
int ekv_append_static(const ekv_cache_desc* c, const void* k_new, const void* v_new,
                      int64_t new_stride_b, int64_t new_stride_h, int32_t* status, void* stream);

/* ---- top-k page selection ---------------------------------------------- */

/* score[b,h,p] = sum_d max(q_d*kmin[p,d], q_d*kmax[p,d]) for every page but the
 * last, rounded to the q dtype; then the min(token_budget / P, Np-1) best pages
 * per query head (ties: lower page id), written in ascending page order and
 * followed by the last page; tok_counts = k_sel*P + tokens in the last page,
 * or user_seqlens[b,h_kv] when that pointer is given.
 * Stands in for estimate_page_criticality + torch.topk + index packing,
 * entmaxkv/kernels/page_criticality.py:24-104, entmaxkv/attention_topk.py:39-76.
 * scores: q-dtype [B, H_q, score_stride]; page_indices: int32 [B, H_q, pi_stride];
 * num_selected, tok_counts: int32 [B, H_q].
 * max_seq_len is a host-side upper bound of seq_lens[] (it sizes the grid only; a
 * bound larger than the true lengths is harmless).
 * work_items (may be null): receives the decode work list in fixed slots, one per
 * (query head, 256-token chunk): B*H_q*ekv_work_items_per_head((k_max+1)*P) entries,
 * k_max = min(token_budget/P, pages(max_seq_len)-1). */
int ekv_topk_select(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                    int64_t q_stride_h, int32_t q_heads, int32_t token_budget,
                    int32_t max_seq_len, void* scores, int64_t score_stride,
                    int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                    int32_t* tok_counts, const int32_t* user_seqlens,
                    int64_t us_stride_b, int64_t us_stride_h, uint64_t* work_items, void* stream);

/* The two halves of ekv_topk_select as separate launches: the score sweep
 * (entmaxkv/kernels/page_criticality.py:24-104) and the selection + packing
 * (entmaxkv/attention_topk.py:54-76). */
int ekv_page_scores(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                    int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len, void* scores,
                    int64_t score_stride, void* stream);
/* ekv_page_scores with the ALiBi bonus of the reference's criticality kernel
 * (entmaxkv/kernels/page_criticality.py:99-101,158-165): score[b,h,p] +=
 * alibi_slopes[h] * (min((p+1)*page_size - 1, S - 1) - q_pos[b]), added in fp32 before the
 * score is rounded to the query dtype.  alibi_slopes: [H_q] fp32 (the reference indexes its
 * slopes by KV head here, which is the same thing for the one-KV-head-per-query-head caches
 * its wrappers support).  q_positions: [B] int32 or null = S - 1, the position of the token
 * just appended. */
int ekv_page_scores_alibi(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                          int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len, void* scores,
                          int64_t score_stride, const float* alibi_slopes,
                          const int32_t* q_positions, void* stream);
int ekv_topk_pack(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget,
                  int32_t max_seq_len, const void* scores, int64_t score_stride,
                  int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                  int32_t* tok_counts, const int32_t* user_seqlens, int64_t us_stride_b,
                  int64_t us_stride_h, uint64_t* work_items, void* stream);

/* ---- Gaussian-aware page selection -------------------------------------- */

/* Scratch of the Gaussian selection stage (per-tile partial sums, ticket counters).
 * Must be zero-filled once before its first use; every call leaves the counters zero. */
size_t ekv_gaussian_workspace_bytes(int32_t batch, int32_t q_heads, int32_t max_pages);

/* Per-page score moments mu_p = s*q.k_mean_p, sigma_p = s*sqrt(sum q^2 k_std_p^2),
 * s = 1/sqrt(D), and per-head sums
 *   head_sums[b,h] = { sum mu_p, sum mu_p^2, sum sigma_p^2, sum (mu_p + 1.5 sigma_p) }.
 * exclude_last_page != 0: the in-progress last page carries no statistics
 * (pages 0..Np-2 are swept, or the only page when Np == 1).
 * finalize != 0: also write mu_global, sigma_global and tau_hat (as
 * ekv_gaussian_finalize would) from this call's own sums.
 * Stands in for compute_page_gaussian_stats_triton,
 * entmaxkv/kernels/gaussian_page_stats.py:8-233. */
int ekv_gaussian_moments(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                         int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len,
                         int32_t exclude_last_page, float alpha, int32_t finalize,
                         float* mu_pages, float* sigma_pages, int64_t page_stat_stride,
                         float* head_sums, float* head_stats, void* workspace,
                         size_t workspace_bytes, void* stream);

/* ekv_gaussian_moments for ALiBi (two launches): every page mean gets alibi_slopes[h] *
 * (mean position of the page - q_pos[b]) while the head's global moments stay those of the
 * unbiased means (entmaxkv/gaussian_utils.py:136-153), and tau_hat is the root of the
 * page-mixture constraint  sum_p page_size * E[((alpha-1) S_p - tau)_+^beta] = 1,
 * S_p ~ N(mu_p, sigma_p^2)  (entmaxkv/kernels/tau_solver_page_mixture.py:67-185,
 * entmaxkv/kernels/tau_mixture_solver_triton.py:81-165) instead of the single-Gaussian one.
 * alpha 2, 1.5 and 4/3 only (EKV_ERR_ALPHA otherwise).  head_stats as ekv_gaussian_moments with
 * finalize = 1.  alibi_slopes: [H_q] fp32; q_positions: [B] int32 or null = S - 1. */
int ekv_gaussian_moments_alibi(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                               int64_t q_stride_h, int32_t q_heads, int32_t max_seq_len,
                               int32_t exclude_last_page, float alpha, float* mu_pages,
                               float* sigma_pages, int64_t page_stat_stride, float* head_sums,
                               float* head_stats, void* workspace, size_t workspace_bytes,
                               const float* alibi_slopes, const int32_t* q_positions, void* stream);

/* head_stats[b,h] = { mu_global, sigma_global, tau_hat, mean(mu_p + 1.5 sigma_p) }
 * from head_sums and the per-sequence page / token counts n_pages[b], n_tokens[b]
 * (device int32 [B]).  tau_hat is the bracketed-Halley root of the
 * single-Gaussian entmax constraint.  Stands in for
 * entmaxkv/gaussian_utils.py:155-181 + entmaxkv/kernels/tau_solver_gpu.py:79-125
 * (closed forms for alpha 2, 1.5 and 4/3 - the last bracketed and bisected as the reference does on
 * its CPU, entmaxkv/tau_solver.py:73-78,276-344; bisection on the reference's moment approximation,
 * entmaxkv/tau_solver.py:80-84, for any other alpha). */
int ekv_gaussian_finalize(const float* head_sums, const int32_t* n_pages,
                          const int32_t* n_tokens, int32_t batch, int32_t q_heads,
                          float alpha, float* head_stats, void* stream);

/* ekv_gaussian_finalize with the counts derived on the device from the global sequence
 * lengths total_lens[b] (device int32 [B]): statistical pages = ceil(len/P) - 1 (or 1 for a
 * single page), tokens = that many full pages (or len).  Lets a sharded step be replayed
 * as a CUDA graph while the sequence grows. */
int ekv_gaussian_finalize_from_lengths(const float* head_sums, const int32_t* total_lens,
                                       int32_t page_size, int32_t batch, int32_t q_heads,
                                       float alpha, float* head_stats, void* stream);

/* Threshold selection + ordered index packing + (optionally) tau clamp.
 *   margin / quantile: from mean_{b,h}(sigma_global) of THIS call's heads, or from
 *   *sigma_mean when that device pointer is given (a batch spread over several GPUs).
 *   selected <=> (alpha-1)*(mu_p + z_page*sigma_p) > tau_floor
 *   cap_max[b,h] = max over selected pages of mu_p + z_clamp*sigma_p/3 (-inf if none)
 *   apply_clamp != 0: tau[b,h] = min(tau_hat, max((alpha-1)*cap_max - 1e-4, tau_floor))
 *                     else tau[b,h] = tau_hat.
 *   append_last_page != 0: the in-progress last page is appended and counted.
 * Also emits tok_counts (compacted tokens per head) and, when work_items is given,
 * the decode work list: one entry per 256-token chunk of every head, densely packed in
 * head order (offsets come from a prefix sum of the heads' chunk counts, so the list is
 * the same from run to run), with their number in work_total[0] (both or neither).
 * work_total holds 1 + ceil(batch*q_heads/1024) ints: the entries after the first are
 * scratch of the prefix sum.
 * Stands in for select_gaussian_threshold_pack_triton
 * (entmaxkv/kernels/selection_pack.py:113-272), the tau clamp
 * (entmaxkv/kernels/tau_clamp.py:8-151) and cache_seqlens_from_page_counts_triton
 * (entmaxkv/kernels/selection_pack.py:7-43). */
int ekv_gaussian_select(const ekv_cache_desc* c, int32_t q_heads, int32_t max_seq_len,
                        int32_t exclude_last_page, int32_t append_last_page, float alpha,
                        float excess_margin_fraction, float z_page_low, float z_page_high,
                        float z_clamp, int32_t apply_clamp, const float* sigma_mean,
                        const float* mu_pages, const float* sigma_pages,
                        int64_t page_stat_stride, const float* head_stats,
                        int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                        int32_t* tok_counts, float* tau_floor, float* cap_max, float* tau,
                        uint64_t* work_items, int32_t* work_total, void* stream);

/* tau = min(tau_hat, max((alpha-1)*cap_max - eps, tau_floor)) where cap_max is finite.
 * For callers that reduce cap_max across GPUs between selection and clamp.
 * Stands in for entmaxkv/kernels/tau_clamp.py:60-73. */
int ekv_tau_clamp(const float* tau_hat, int64_t tau_hat_stride, const float* cap_max,
                  const float* tau_floor, int32_t n, float alpha, float eps, float* tau,
                  void* stream);

/* ---- paged entmax decode ------------------------------------------------ */

/* Scratch of the decode (scores of the gathered tokens, per-chunk partials). */
size_t ekv_decode_workspace_bytes(int32_t batch, int32_t q_heads, int32_t head_dim,
                                  int32_t max_tokens);

/* Zero the ticket counters and the status word at the front of a decode workspace
 * (once after allocation, or after a failed launch). */
int ekv_decode_workspace_reset(void* workspace, int32_t batch, int32_t q_heads, void* stream);

/* Decode work list.  The decode kernels walk a device-side list of 64-bit items, one
 * per 256-token chunk of one query head (the selection entry points emit it).  For a
 * caller-made page table, ekv_build_work_items fills the fixed-slot form from
 * tok_counts: n_heads * ekv_work_items_per_head(max_tokens) entries. */
int32_t ekv_work_items_per_head(int32_t max_tokens);
int ekv_build_work_items(const int32_t* tok_counts, int32_t n_heads, int32_t max_tokens,
                         uint64_t* work_items, void* stream);

/* Pass over K: z_i = (alpha-1)/sqrt(D) * q.k_i for the tok_counts[b,h] tokens the
 * page table enumerates (row = page_indices[c / P]*P + c % P), kept in the
 * workspace; then per head (a second, small launch) the tau procedure `tau_mode`
 * (see EKV_TAU_*).  halley_sums (fp32 [B*H_q*3], may be
 * null) receives sum (z-tau)_+^(beta-j), j=0..2, evaluated at the incoming tau.
 * work_items / n_items: the work list and its capacity; work_total (device, may be
 * null) holds the number of valid entries when the list is densely packed.
 * Stands in for stages 1-5 of entmaxkv/kernels/adadecode_paged.py:39-377 with
 * entmaxkv/kernels/adadecode.py:12-112,381-426,555-592, and for the correction
 * loop of entmaxkv/kernels/adadecode_paged_gaussian_tau.py:12-53,266-296. */
int ekv_decode_scores(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                      int64_t q_stride_h, int32_t q_heads, const int32_t* page_indices,
                      int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens,
                      float alpha, int32_t tau_mode, int32_t niter, float* tau,
                      float* halley_sums, const uint64_t* work_items, int32_t n_items,
                      const int32_t* work_total, void* workspace, size_t workspace_bytes,
                      void* stream);

/* One unbracketed Halley / Newton step per head from externally reduced sums.
 * Stands in for entmaxkv/kernels/adadecode_paged_gaussian_tau.py:23-53. */
int ekv_halley_update(float* tau, const float* halley_sums, int32_t n, float alpha,
                      void* stream);

/* Pass over V: out[b,h,:] = sum_i (z_i - tau)_+^(1/(alpha-1)) * v_i over the tokens
 * of the page table whose weight is non-zero (no normalisation, as in the
 * reference).  out_is_f32 != 0 writes fp32 partial outputs (for a sum-allreduce
 * across GPUs) instead of the cache dtype.  Heads without tokens get zeros.
 * Three launches: heads with at most 1024 non-zero weights have exactly those value
 * rows gathered (token order); the rest are streamed chunk by chunk; a final kernel
 * folds the chunks.  Stands in for stage 6 of entmaxkv/kernels/adadecode_paged.py:385-507 +
 * entmaxkv/kernels/adadecode.py:725-747 and
 * entmaxkv/kernels/adadecode_paged_gaussian_tau.py:57-175. */
int ekv_decode_values(const ekv_cache_desc* c, int32_t q_heads, const int32_t* page_indices,
                      int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens,
                      float alpha, const float* tau, void* out, int64_t out_stride_b,
                      int64_t out_stride_h, int32_t out_is_f32, const uint64_t* work_items,
                      int32_t n_items, const int32_t* work_total, void* workspace,
                      size_t workspace_bytes, void* stream);

/* K pass, tau, V pass and output in one call (four launches): what the two decode
 * wrappers of the reference do after page selection,
 * entmaxkv/kernels/adadecode_paged.py:567-762 (tau_mode EKV_TAU_EXACT) and
 * entmaxkv/kernels/adadecode_paged_gaussian_tau.py:192-331 (EKV_TAU_CORRECTED; niter = 0
 * is the "fixed" mode).  Heads whose support is small have their few value rows gathered
 * by the tau kernel itself, so the V pass only streams heads with a large support.
 * stage_events (may be null): three cudaEvent_t recorded after the K pass, after the
 * tau kernel and after the V pass, for per-kernel timing. */
int ekv_decode(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
               int32_t q_heads, const int32_t* page_indices, int64_t pi_stride,
               const int32_t* tok_counts, int32_t max_tokens, float alpha, int32_t tau_mode,
               int32_t niter, float* tau, void* out, int64_t out_stride_b, int64_t out_stride_h,
               const uint64_t* work_items, int32_t n_items, const int32_t* work_total,
               void* workspace, size_t workspace_bytes, void** stage_events, void* stream);

/* ---------------------------------------------------------------------------
 * Peer exchange for the sequence-page-sharded Gaussian step (one process per GPU).
 * No counterpart in the reference, which runs on a single GPU.  The sharded step needs
 * four tiny reductions per step (moment sums, clamp cap, Halley sums, partial outputs).
 * Here each of them is done by the kernel that consumes the result: every rank stores its
 * partials, one 64-bit word {epoch : value} each, into every peer's "inbox" over NVLink,
 * polls its own inbox - with an iteration budget - until the peers' words carry the
 * current epoch, combines them in rank order (bit-identical on all ranks) and finishes
 * the arithmetic in the same launch.  Peer stores and local loads only; no fences, no
 * multicast.
 *
 * Set-up: every rank calls ekv_exchange_create (allocates the inbox with cudaMalloc on the
 * current device), passes the 64-byte handle of ekv_exchange_handle to all other ranks by
 * any host channel, calls ekv_exchange_connect with the world's handles in rank order, and
 * synchronises with the other ranks on the host before the first exchange.  All ranks must
 * issue the same sequence of exchange calls.  A wait that runs out sets
 * EKV_STATUS_PEER_TIMEOUT in *status and the kernel returns; nothing hangs.
 * Before ekv_exchange_destroy every rank must have finished its last exchange (host barrier).
 * n is limited to max_floats (a multiple of 4, at most 4 Mi) per call.
 * ------------------------------------------------------------------------- */
typedef struct ekv_exchange ekv_exchange;
#define EKV_EXCHANGE_MAX_RANKS 8
#define EKV_EXCHANGE_HANDLE_BYTES 64
enum { EKV_XCH_SUM = 0, EKV_XCH_MAX = 1 };

int ekv_exchange_create(int32_t rank, int32_t world, int32_t max_floats, ekv_exchange** out);
int ekv_exchange_handle(const ekv_exchange* x, void* handle_out);
int ekv_exchange_connect(ekv_exchange* x, const void* all_handles);
/* Same-process alternative to handles: device pointers of every rank's inbox
 * (ekv_exchange_base), peer access between the devices already enabled by the caller. */
void* ekv_exchange_base(const ekv_exchange* x);
int ekv_exchange_connect_pointers(ekv_exchange* x, void* const* bases);
/* Polls a thread may spend per exchange (each: one load + a 32 ns sleep; default 2^21). */
int ekv_exchange_set_spin_limit(ekv_exchange* x, uint32_t iterations);
int ekv_exchange_destroy(ekv_exchange* x);

/* dst[i] = sum / max over ranks of src[i], i < n, on slot 0..3.  These four slots belong to this
 * call alone (the fused calls below use four others).  Exchanges on one slot are numbered per
 * launch - the k-th launch on a slot carries number k on every rank, whatever its grid - so the
 * launches that share a slot must be ordered on the device (one stream, or events): two of them in
 * flight at once is a race. */
int ekv_exchange_allreduce(ekv_exchange* x, int32_t slot, const float* src, float* dst, int32_t n,
                           int32_t op, int32_t* status, void* stream);
/* sum of the ranks' head_sums [B,H_q,4] + ekv_gaussian_finalize_from_lengths. */
int ekv_exchange_gaussian_finalize(ekv_exchange* x, const float* head_sums_local,
                                   const int32_t* total_lens, int32_t page_size, int32_t batch,
                                   int32_t q_heads, float alpha, float* head_stats,
                                   int32_t* status, void* stream);
/* ekv_gaussian_moments(finalize = 0) + ekv_exchange_gaussian_finalize in ONE launch where the sweep can
 * carry the exchange (bfloat caches, GQA groups of up to eight heads: the last block of every KV head
 * trades its heads' sums and finishes their statistics), otherwise in the two launches it replaces.
 * total_lens: device int32 [B], tokens of the whole request. */
int ekv_exchange_gaussian_moments(ekv_exchange* x, const ekv_cache_desc* c, const void* q,
                                  int64_t q_stride_b, int64_t q_stride_h, int32_t q_heads,
                                  int32_t max_seq_len, int32_t exclude_last_page, float alpha,
                                  const int32_t* total_lens, float* mu_pages, float* sigma_pages,
                                  int64_t page_stat_stride, float* head_sums, float* head_stats,
                                  void* workspace, size_t workspace_bytes, int32_t* status, void* stream);
/* ekv_gaussian_select whose clamp uses the maximum of the ranks' cap_max (traded by the selection
 * kernel itself): ekv_gaussian_select(apply_clamp = 0) + ekv_exchange_tau_clamp in one launch.
 * cap_max receives this rank's own value. */
int ekv_exchange_gaussian_select(ekv_exchange* x, const ekv_cache_desc* c, int32_t q_heads,
                                 int32_t max_seq_len, int32_t exclude_last_page,
                                 int32_t append_last_page, float alpha, float excess_margin_fraction,
                                 float z_page_low, float z_page_high, float z_clamp,
                                 int32_t apply_clamp, const float* sigma_mean, const float* mu_pages,
                                 const float* sigma_pages, int64_t page_stat_stride,
                                 const float* head_stats, int32_t* page_indices, int64_t pi_stride,
                                 int32_t* num_selected, int32_t* tok_counts, float* tau_floor,
                                 float* cap_max, float* tau, uint64_t* work_items,
                                 int32_t* work_total, int32_t* status, void* stream);
/* max of the ranks' cap [n] + ekv_tau_clamp in place on tau. */
int ekv_exchange_tau_clamp(ekv_exchange* x, float* tau, const float* cap_local,
                           const float* tau_floor, int32_t n, float alpha, float eps,
                           int32_t* status, void* stream);
/* sum of the ranks' Halley sums [n,3] + ekv_halley_update in place on tau. */
int ekv_exchange_halley_update(ekv_exchange* x, float* tau, const float* halley_sums_local,
                               int32_t n, float alpha, int32_t* status, void* stream);
/* sum of the ranks' fp32 partial outputs [n_heads, head_dim] stored to out (row stride
 * out_stride_h elements) in out_dtype (EKV_F16 / EKV_BF16 / EKV_F32). */
int ekv_exchange_output(ekv_exchange* x, const float* partial_local, int32_t n_heads,
                        int32_t head_dim, void* out, int64_t out_stride_h, int32_t out_dtype,
                        int32_t* status, void* stream);

/* The decode of a sequence-sharded step in four launches: K pass; tau kernel (local Halley sums
 * -> traded with the other ranks -> the `niter` (0 or 1) unbracketed step -> value rows of
 * small supports gathered into `gathered`, fp32 [B, H_q, head_dim]); V pass over the heads
 * with a large support; a last kernel that folds the local chunks, trades the partial outputs
 * and stores the sum in out_dtype.  tau holds the (clamped) estimate on entry and the final
 * threshold on return, identical on every rank.  Equivalent to ekv_decode_scores(EKV_TAU_NONE)
 * + ekv_exchange_halley_update + ekv_decode_values + ekv_exchange_output. */
int ekv_exchange_decode(ekv_exchange* x, const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                        int64_t q_stride_h, int32_t q_heads, const int32_t* page_indices,
                        int64_t pi_stride, const int32_t* tok_counts, int32_t max_tokens, float alpha,
                        int32_t niter, float* tau, float* gathered, void* out, int64_t out_stride_b,
                        int64_t out_stride_h, int32_t out_dtype, const uint64_t* work_items,
                        int32_t n_items, const int32_t* work_total, void* workspace,
                        size_t workspace_bytes, int32_t* status, void* stream);
/* ekv_exchange_decode over ONE page table per GQA group of four or eight (the shard's tables merged by
 * ekv_group_union; head_items from ekv_build_work_items over union_tok_counts): the sequence-sharded
 * counterpart of ekv_decode_grouped.  Same exchanges, same results as ekv_exchange_decode to rounding. */
int ekv_exchange_decode_grouped(ekv_exchange* x, const ekv_cache_desc* c, const void* q,
                                int64_t q_stride_b, int64_t q_stride_h, int32_t q_heads,
                                const int32_t* union_pages, int64_t union_stride,
                                const int32_t* union_tok_counts, int32_t max_tokens, float alpha,
                                int32_t niter, float* tau, float* gathered, void* out,
                                int64_t out_stride_b, int64_t out_stride_h, int32_t out_dtype,
                                const uint64_t* head_items, int32_t n_head_items,
                                const uint64_t* group_items, int32_t n_group_items,
                                const uint8_t* member, int64_t member_stride, void* workspace,
                                size_t workspace_bytes, int32_t* status, void* stream);

/* ekv_decode with ALiBi: every kept token's score gets (alpha-1) * alibi_slopes[h] *
 * (its absolute position - q_pos[b]) before tau is solved
 * (entmaxkv/kernels/adadecode_paged.py:100-105,126-128,
 * entmaxkv/kernels/adadecode_paged_gaussian_tau.py:124-126,152-153).  alibi_slopes: [H_q]
 * fp32; q_positions: [B] int32 or null = S - 1. */
int ekv_decode_alibi(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                     int32_t q_heads, const int32_t* page_indices, int64_t pi_stride,
                     const int32_t* tok_counts, int32_t max_tokens, float alpha, int32_t tau_mode,
                     int32_t niter, float* tau, void* out, int64_t out_stride_b, int64_t out_stride_h,
                     const uint64_t* work_items, int32_t n_items, const int32_t* work_total,
                     void* workspace, size_t workspace_bytes, void** stage_events,
                     const float* alibi_slopes, const int32_t* q_positions, void* stream);

/* ---------------------------------------------------------------------------
 * Group-shared K pass for GQA groups of four or eight query heads per KV head (G = q_heads / kv_heads;
 * 16-bit caches, head_dim 128, no ALiBi).
 * No counterpart in the reference, whose decode kernels fetch the K rows once per query
 * head.  When every head keeps a large share of the pages, the G heads of a KV head
 * read mostly the same rows; here they share one page table and each row is fetched once
 * and scored against the G queries.
 *
 * ekv_group_union merges the G ascending page tables of every group
 * (page_indices / num_selected, as written by a selection entry point) into
 *   union_pages      int32 [B*H_q, union_stride]: the ascending union, written to the rows
 *                    of all G heads of the group,
 *   member           uint8 [B*H_kv, member_stride]: bit j of entry i = head j of the group
 *                    selected union page i,
 *   union_tok_counts int32 [B*H_q]: tokens the union enumerates (the same for the G heads),
 *   group_items      B*H_kv * ekv_work_items_per_head(max_tokens) fixed-slot items whose head
 *                    field is the group's first query head (slot g*per_head + c = chunk c of
 *                    group g, empty past the group's end; the K pass derives the same items
 *                    from union_tok_counts and never visits the empty slots).
 *   head_items       (may be null) B*H_q * ekv_work_items_per_head(max_tokens) items: what
 *                    ekv_build_work_items makes of union_tok_counts, written here to save that launch.
 * union_stride and member_stride must be >= page_capacity; page_capacity <= 1474560 / G (the G page
 * bitmaps of a group sit in 180 KiB of shared memory).
 *
 * ekv_decode_grouped is ekv_decode over the shared table: the K pass walks group_items,
 * head j's score of a row of a page it did not select is -inf (outside every support, so
 * tau and the output are those of the head's own table); the tau kernel and the V pass
 * walk head_items, built by ekv_build_work_items from union_tok_counts. */
int ekv_group_union(const ekv_cache_desc* c, int32_t q_heads, const int32_t* page_indices,
                    int64_t pi_stride, const int32_t* num_selected, int32_t max_tokens,
                    int32_t* union_pages, int64_t union_stride, uint8_t* member,
                    int64_t member_stride, int32_t* union_tok_counts, uint64_t* group_items,
                    int32_t n_group_items, uint64_t* head_items, void* stream);
int ekv_decode_grouped(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                       int32_t q_heads, const int32_t* union_pages, int64_t union_stride,
                       const int32_t* union_tok_counts, int32_t max_tokens, float alpha,
                       int32_t tau_mode, int32_t niter, float* tau, void* out, int64_t out_stride_b,
                       int64_t out_stride_h, const uint64_t* head_items, int32_t n_head_items,
                       const uint64_t* group_items, int32_t n_group_items, const uint8_t* member,
                       int64_t member_stride, void* workspace, size_t workspace_bytes,
                       void** stage_events, void* stream);

/* counts[b*H_q + h] (device int32) = number of tokens of head h whose weight (z - tau)_+^beta was
 * non-zero in the last decode that used this workspace, i.e. the value rows that decode had to read;
 * -1 where the last call did not produce an output.  A measurement aid (bytes actually moved by the V
 * pass); no counterpart in the reference.  workspace_bytes and the four sizes are those of the decode. */
int ekv_decode_support_counts(const void* workspace, size_t workspace_bytes, int32_t batch,
                              int32_t q_heads, int32_t head_dim, int32_t max_tokens,
                              int32_t* counts, void* stream);

/* Every wait on an asynchronous bulk copy (the tile rings of the sweeps and of the K / V passes) is bounded,
 * so a copy that never lands cannot hang the GPU; the launch's results are then undefined.  Kernels with a
 * status word raise EKV_STATUS_COPY_TIMEOUT there; the moments sweeps have none, so every such event is
 * also counted: *count receives the number of timed-out waits since the library was loaded (0 in a
 * healthy run).  One kernel is left out: the page-score sweep runs at its register limit, and recording
 * the event there costs 15 % of its time; its waits are bounded like all others but not counted.
 * Synchronises the device.  No counterpart in the reference. */
int ekv_copy_timeouts(uint32_t* count);

/* Copies a step's three inputs (query, new key row, new value row; contiguous device buffers, 16-byte
 * aligned, sizes multiples of 16 bytes) into the fixed buffers a captured (CUDA graph) step reads, in one
 * launch.  The reference has no counterpart: it launches every kernel of a step from Python and needs no
 * fixed input buffers. */
int ekv_stage_inputs(void* q_dst, const void* q_src, size_t q_bytes, void* k_dst, const void* k_src,
                     size_t k_bytes, void* v_dst, const void* v_src, size_t v_bytes, void* stream);

/* The whole top-k decode step (page scores, selection, exact-mode tau, output) of a SMALL problem in one
 * launch: a cluster of four thread blocks per query head, scores and kept tokens in (distributed) shared
 * memory.  It replaces ekv_topk_select + ekv_decode (EKV_TAU_EXACT) - the Triton launches of
 * entmaxkv/attention_topk.py:39-76 followed by entmaxkv/kernels/adadecode_paged.py:567-762 - when the
 * general path's launches would each leave most of the GPU idle.  Page scores, page tables and counts
 * are bit-identical to ekv_topk_select's; tau and the output row agree with ekv_decode's to rounding
 * (the reductions combine in a different order).  No ALiBi, no caller-provided lengths.
 * ekv_topk_decode_fused_supported returns 1 when a problem fits: batch*q_heads*4 <= SM count, at most
 * 8192 scored pages per head, (k_max+1) pages of at most 4096 tokens per block of the cluster,
 * niter <= 64.  ekv_topk_decode_fused returns EKV_ERR_ARG for anything else.  The append still comes
 * first, as its own call.  status: one int32 the kernel ORs EKV_STATUS_* bits into (the cache's status
 * word of ekv_append serves). */
int ekv_topk_decode_fused_supported(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget,
                                    int32_t max_seq_len, int32_t niter);
int ekv_topk_decode_fused(const ekv_cache_desc* c, const void* q, int64_t q_stride_b,
                          int64_t q_stride_h, int32_t q_heads, int32_t token_budget,
                          int32_t max_seq_len, float alpha, int32_t niter, void* scores,
                          int64_t score_stride, int32_t* page_indices, int64_t pi_stride,
                          int32_t* num_selected, int32_t* tok_counts, float* tau, void* out,
                          int64_t out_stride_b, int64_t out_stride_h, int32_t* status, void* stream);

/* The top-k decode step after the score sweep (selection, K pass, exact-mode tau, value gather, output) for MANY
 * heads in one launch: one persistent block per SM, one warp group streaming the current head's selected K pages
 * while the other solves tau and gathers the value rows of the previous head and selects the pages of the head
 * after next - the latency chains of ekv_topk_pack and of the tau kernel run in issue slots the K pass leaves idle.
 * Replaces ekv_topk_pack + ekv_decode(EKV_TAU_EXACT) (entmaxkv/attention_topk.py:54-76 followed by
 * entmaxkv/kernels/adadecode_paged.py:567-762); scores come from ekv_page_scores.  Page tables and counts are
 * bit-identical to ekv_topk_pack's, tau and the output agree with ekv_decode's to rounding.  No ALiBi, no
 * caller-provided lengths; 16-bit caches, head_dim 128, page size 16, (k_max+1)*16 <= 4352 kept tokens per head,
 * score rows 64-byte aligned with a stride that is a multiple of 32 (otherwise a slower selection is used).
 * Heads are dealt out round-robin to one persistent block per SM.
 * ekv_topk_decode_stream_supported: 0 = does not fit, 1 = fits and pays off (3*batch*q_heads >= SM count),
 * 2 = fits.  support (may be null): int32 [B*H_q], tokens with a non-zero weight.  status: one int32 the kernel
 * ORs EKV_STATUS_* bits into. */
int ekv_topk_decode_stream_supported(const ekv_cache_desc* c, int32_t q_heads, int32_t token_budget,
                                     int32_t max_seq_len, int32_t niter);
int ekv_topk_decode_stream(const ekv_cache_desc* c, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                           int32_t q_heads, int32_t token_budget, int32_t max_seq_len, float alpha,
                           int32_t niter, const void* scores, int64_t score_stride,
                           int32_t* page_indices, int64_t pi_stride, int32_t* num_selected,
                           int32_t* tok_counts, float* tau, void* out, int64_t out_stride_b,
                           int64_t out_stride_h, int32_t* support, float* scratch,
                           size_t scratch_bytes, int32_t* status, void* stream);
/* Bytes of `scratch` (device memory; kept scores of every block's current and previous head). */
size_t ekv_topk_decode_stream_scratch_bytes(void);

/* Block-table caches: the decode entry points (ekv_decode*, ekv_decode_scores, ekv_decode_values,
 * ekv_exchange_decode) address K/V by PHYSICAL block id.  ekv_translate_pages turns the page tables the
 * selection entry points write (page numbers) into block ids: out[h, i] = block_table[b(h), in[h, i]]
 * for i < counts[h], h < batch*q_heads (rows beyond counts[h] are left alone).  in and out may be the same
 * buffer.  The reference has no counterpart (its cache is dense, entmaxkv/kv_cache.py:44-56); serving
 * engines that hand out KV blocks from a pool need the indirection.  ALiBi decodes need page numbers for
 * token positions and are not available on block-table caches (EKV_ERR_ARG). */
int ekv_translate_pages(const ekv_cache_desc* c, int32_t q_heads, const int32_t* page_indices,
                        int64_t pi_stride, const int32_t* counts, int32_t* block_ids, int64_t out_stride,
                        void* stream);

/* Copy the status word of a decode workspace to the host (synchronises the stream). */
int ekv_read_status(const void* workspace, int32_t* host_status, void* stream);

/* Library version (major*100 + minor). */
int ekv_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ENTMAXKV_B200_H */
