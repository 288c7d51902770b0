// Page statistics of the key cache: one-launch build over all pages, and the
// in-place single-token append that refreshes the statistics of one page.
//
// Arithmetic (identical in both kernels, mirrored by the CPU oracle): rows of a
// page in storage order; mean = (((x0+x1)+x2)+...)/n; var = ((d0*d0+d1*d1)+...)/n
// with d = x - mean and separately rounded products and sums;
// std = max(sqrt(var), 1e-6); one rounding to the storage dtype at the end.
#include <mutex>

#include "ekv_common.cuh"

namespace ekv {

template <typename T>
struct ColumnStats {
  static constexpr int EPL = ElemTraits<T>::EPL;
  float mn[EPL], mx[EPL], sum[EPL], mean[EPL], sq[EPL];
  __device__ __forceinline__ void begin() {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      mn[j] = INFINITY;
      mx[j] = -INFINITY;
      sum[j] = 0.f;
    }
  }
  __device__ __forceinline__ void first_pass(const uint4& raw) {
    float x[EPL];
    unpack<T>(raw, x);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      mn[j] = fminf(mn[j], x[j]);
      mx[j] = fmaxf(mx[j], x[j]);
      sum[j] = __fadd_rn(sum[j], x[j]);
    }
  }
  __device__ __forceinline__ void middle(float n) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      mean[j] = __fdiv_rn(sum[j], n);
      sq[j] = 0.f;
    }
  }
  __device__ __forceinline__ void second_pass(const uint4& raw) {
    float x[EPL];
    unpack<T>(raw, x);
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const float d = __fsub_rn(x[j], mean[j]);
      sq[j] = __fadd_rn(sq[j], __fmul_rn(d, d));
    }
  }
  __device__ __forceinline__ void finish(float n, T* o_min, T* o_max, T* o_mean, T* o_std) {
    float sd[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) sd[j] = fmaxf(__fsqrt_rn(__fdiv_rn(sq[j], n)), 1e-6f);
    *reinterpret_cast<uint4*>(o_min) = pack<T>(mn);
    *reinterpret_cast<uint4*>(o_max) = pack<T>(mx);
    *reinterpret_cast<uint4*>(o_mean) = pack<T>(mean);
    *reinterpret_cast<uint4*>(o_std) = pack<T>(sd);
  }
};

// Statistics of one 16-byte column of one page.  Pages of up to 16 rows (the usual page
// size) are read once, all rows in flight together, and both passes run from registers.
template <typename T>
__device__ __forceinline__ void page_column_stats(const T* page_base /* row 0, this lane's chunk */,
                                                  int row_stride, int n_rows, T* o_min, T* o_max,
                                                  T* o_mean, T* o_std) {
  ColumnStats<T> st;
  st.begin();
  const float n = (float)n_rows;
  if (n_rows <= 16) {
    uint4 r[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n_rows) r[i] = *reinterpret_cast<const uint4*>(page_base + (size_t)i * row_stride);
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n_rows) st.first_pass(r[i]);
    st.middle(n);
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n_rows) st.second_pass(r[i]);
  } else {
    for (int i = 0; i < n_rows; ++i)
      st.first_pass(*reinterpret_cast<const uint4*>(page_base + (size_t)i * row_stride));
    st.middle(n);
    for (int i = 0; i < n_rows; ++i)
      st.second_pass(*reinterpret_cast<const uint4*>(page_base + (size_t)i * row_stride));
  }
  st.finish(n, o_min, o_max, o_mean, o_std);
}

// grid: (ceil(max_pages * LPR / 256), B*H_kv); one lane per (page, 16-byte column).
template <typename T, int D>
__global__ void __launch_bounds__(256) page_stats_init_kernel(ekv_cache_desc c, int max_pages) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  const int bh = blockIdx.y;
  const int b = bh / c.kv_heads, h = bh % c.kv_heads;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int page = idx / LPR, col = idx % LPR;
  const int S = c.seq_lens[b];
  const int P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  if (page >= n_pages || page >= max_pages || page >= c.page_capacity) return;
  const int n_rows = min(P, S - page * P);
  size_t poff;
  if (!kv_page_offset(c, b, h, page, poff)) return;    // a block outside the pool: nothing to read
  const T* kb = static_cast<const T*>(c.k) + poff + col * EPL;
  const size_t mo = b * c.meta_stride_b + h * c.meta_stride_h + (size_t)page * D + col * EPL;
  page_column_stats<T>(kb, D, n_rows, static_cast<T*>(c.k_min) + mo, static_cast<T*>(c.k_max) + mo,
                       static_cast<T*>(c.k_mean) + mo, static_cast<T*>(c.k_std) + mo);
}

// grid: B*H_kv blocks of 32 threads; lanes < LPR own one 16-byte column each.
template <typename T, int D>
__global__ void __launch_bounds__(32) append_kernel(ekv_cache_desc c, const T* __restrict__ k_new,
                                                    const T* __restrict__ v_new, int64_t nsb,
                                                    int64_t nsh, int* counters, int* status) {
  constexpr int EPL = ElemTraits<T>::EPL;
  constexpr int LPR = D / EPL;
  const int bh = blockIdx.x;
  const int b = bh / c.kv_heads, h = bh % c.kv_heads;
  const int lane = threadIdx.x;
  const int pos = c.seq_lens[b];   // every block of this sequence reads it before the last one bumps it
  const int P = c.page_size;
  const int page = pos / P;
  const bool fits = pos < c.capacity && page < c.page_capacity;
  size_t poff = 0;
  const bool block_ok = fits && kv_page_offset(c, b, h, page, poff);
  if (block_ok && lane < LPR) {
    T* kb = static_cast<T*>(c.k) + poff;      // row 0 of the page the token lands in
    T* vb = static_cast<T*>(c.v) + poff;
    const int row = pos - page * P;
    const uint4 kn = *reinterpret_cast<const uint4*>(k_new + b * nsb + h * nsh + lane * EPL);
    const uint4 vn = *reinterpret_cast<const uint4*>(v_new + b * nsb + h * nsh + lane * EPL);
    *reinterpret_cast<uint4*>(kb + (size_t)row * D + lane * EPL) = kn;
    *reinterpret_cast<uint4*>(vb + (size_t)row * D + lane * EPL) = vn;
    // this lane re-reads only the column it just wrote, so no barrier is needed
    const size_t mo = b * c.meta_stride_b + h * c.meta_stride_h + (size_t)page * D + lane * EPL;
    page_column_stats<T>(kb + lane * EPL, D, row + 1,
                         static_cast<T*>(c.k_min) + mo, static_cast<T*>(c.k_max) + mo,
                         static_cast<T*>(c.k_mean) + mo, static_cast<T*>(c.k_std) + mo);
  }
  if (!fits && lane == 0) atomicOr(status, EKV_STATUS_CAPACITY);
  if (fits && !block_ok && lane == 0) atomicOr(status, EKV_STATUS_PAGE_RANGE);
  __syncwarp();
  if (lane == 0) {
    __threadfence();
    const int done = atomicAdd(&counters[b], 1);
    if (done == c.kv_heads - 1) {   // last head of this sequence: publish the new length
      counters[b] = 0;
      if (fits) c.seq_lens[b] = pos + 1;
    }
  }
}

}  // namespace ekv

extern "C" int ekv_page_stats_init(const ekv_cache_desc* c, int32_t max_seq_len, void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!c->k_min || !c->k_max || !c->k_mean || !c->k_std) return EKV_ERR_ARG;
  if (max_seq_len <= 0) return EKV_OK;
  const int max_pages = (max_seq_len + c->page_size - 1) / c->page_size;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    constexpr int LPR = D / ElemTraits<T>::EPL;
    dim3 grid((unsigned)(((int64_t)max_pages * LPR + 255) / 256), (unsigned)(c->batch * c->kv_heads));
    page_stats_init_kernel<T, D><<<grid, 256, 0, as_stream(stream)>>>(*c, max_pages);
  });
  return launch_status();
}

extern "C" int ekv_append(const ekv_cache_desc* c, const void* k_new, const void* v_new,
                          int64_t new_stride_b, int64_t new_stride_h, int32_t* counters,
                          int32_t* status, void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!k_new || !v_new || !counters || !status) return EKV_ERR_ARG;
  if (!c->k_min || !c->k_max || !c->k_mean || !c->k_std) return EKV_ERR_ARG;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((new_stride_b * esz) % 16 || (new_stride_h * esz) % 16) return EKV_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new)) & 15) return EKV_ERR_ARG;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    append_kernel<T, D><<<c->batch * c->kv_heads, 32, 0, as_stream(stream)>>>(
        *c, static_cast<const T*>(k_new), static_cast<const T*>(v_new), new_stride_b,
        new_stride_h, counters, status);
  });
  return launch_status();
}

// ---- append for callers that cannot hand over scratch memory ---------------------------
//
// Some hosts of this library cannot allocate device memory themselves: an inference server
// that gave its whole memory budget to one arena at start-up, or a step that runs where
// cudaMalloc is forbidden (inside a latency-critical loop, or after the process's memory
// limit has been reached).  ekv_append needs one ticket counter per sequence; here those
// counters live in a fixed array that is part of the loaded library image, so the caller
// passes only the cache, the new token and the status word.
//
// The array is shared by every call on a device and keeps whatever the previous call left
// in it, so each call clears the slots it uses first.  Two calls that overlap on the GPU
// (different streams, no ordering between them) would share tickets and are a data race.
// The array's address is looked up for the device that is CURRENT when the call is made, so
// `stream` must be a stream of that device.

constexpr int kAppendStaticMaxBatch = EKV_APPEND_STATIC_MAX_BATCH;
static __device__ __align__(256) int g_append_tickets[kAppendStaticMaxBatch];

namespace {
// Device address of g_append_tickets per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use: it is resolved once per device,
// with that device current.
constexpr int kMaxDevices = 64;
int* g_ticket_ptr[kMaxDevices] = {};
std::mutex g_ticket_mutex;

// `refresh`: look the address up again even if one is cached (the host application reset the
// device since the first call, which unloads and later reloads the library image on it).
int resolve_tickets(int** out, bool refresh = false) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return EKV_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_ticket_mutex);
  if (g_ticket_ptr[dev] == nullptr || refresh) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_append_tickets);
    if (e != cudaSuccess) return (int)e;
    g_ticket_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_ticket_ptr[dev];
  return EKV_OK;
}
}  // namespace

extern "C" int ekv_append_static(const ekv_cache_desc* c, const void* k_new, const void* v_new,
                                 int64_t new_stride_b, int64_t new_stride_h, int32_t* status,
                                 void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!k_new || !v_new || !status) return EKV_ERR_ARG;
  if (!c->k_min || !c->k_max || !c->k_mean || !c->k_std) return EKV_ERR_ARG;
  if (c->batch > kAppendStaticMaxBatch) return EKV_ERR_STATIC_LIMIT;   // more sequences than built-in counters
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  if ((new_stride_b * esz) % 16 || (new_stride_h * esz) % 16) return EKV_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new)) & 15) return EKV_ERR_ARG;
  int* tickets = nullptr;
  if (int e = resolve_tickets(&tickets)) return e;
  cudaStream_t st = as_stream(stream);
  // the previous call's leftovers (or those of a call that was cut short) must not count
  cudaError_t me = cudaMemsetAsync(tickets, 0, (size_t)c->batch * sizeof(int), st);
  if (me == cudaErrorInvalidValue) {
    // a cached address goes stale when the host calls cudaDeviceReset between two calls: resolve
    // the symbol again on the current device and retry once
    (void)cudaGetLastError();
    if (int e = resolve_tickets(&tickets, true)) return e;
    me = cudaMemsetAsync(tickets, 0, (size_t)c->batch * sizeof(int), st);
  }
  if (me != cudaSuccess) return (int)me;
  EKV_DISPATCH(c->dtype, c->head_dim, {
    append_kernel<T, D><<<c->batch * c->kv_heads, 32, 0, st>>>(
        *c, static_cast<const T*>(k_new), static_cast<const T*>(v_new), new_stride_b,
        new_stride_h, tickets, status);
  });
  return launch_status();
}

namespace ekv {
__global__ void translate_pages_kernel(ekv_cache_desc c, int q_heads, const int* __restrict__ in, int64_t in_stride,
                                       const int* __restrict__ counts, int* __restrict__ out, int64_t out_stride) {
  const int bh = blockIdx.y;
  const int n = counts[bh];
  const int b = bh / q_heads;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int page = in[(size_t)bh * in_stride + i];
    out[(size_t)bh * out_stride + i] =
        (unsigned)page < (unsigned)c.page_capacity ? c.block_table[(size_t)b * c.bt_stride + page] : -1;
  }
}
}  // namespace ekv

extern "C" int ekv_translate_pages(const ekv_cache_desc* c, int32_t q_heads, const int32_t* page_indices,
                                   int64_t pi_stride, const int32_t* counts, int32_t* block_ids,
                                   int64_t out_stride, void* stream) {
  using namespace ekv;
  if (int e = check_desc(c)) return e;
  if (!c->block_table || !page_indices || !counts || !block_ids || q_heads <= 0 || pi_stride <= 0 || out_stride <= 0)
    return EKV_ERR_ARG;
  const int64_t width = pi_stride < out_stride ? pi_stride : out_stride;
  dim3 grid((unsigned)((width + 255) / 256 < 64 ? (width + 255) / 256 : 64), (unsigned)(c->batch * q_heads));
  translate_pages_kernel<<<grid, 256, 0, as_stream(stream)>>>(*c, q_heads, page_indices, pi_stride, counts, block_ids,
                                                               out_stride);
  return launch_status();
}

namespace ekv {
// Copies the three inputs of a step (query, new key, new value) into the fixed buffers a captured step
// reads: one launch instead of three.  blockIdx.y picks the buffer; 16 bytes per thread.
struct StageCopy {
  const uint4* src[3];
  uint4* dst[3];
  int n16[3];
};
__global__ void __launch_bounds__(256) stage_inputs_kernel(const StageCopy s) {
  const int which = blockIdx.y;
  const int n = s.n16[which];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) s.dst[which][i] = s.src[which][i];
}
}  // namespace ekv

extern "C" int ekv_stage_inputs(void* q_dst, const void* q_src, size_t q_bytes, void* k_dst, const void* k_src,
                                size_t k_bytes, void* v_dst, const void* v_src, size_t v_bytes, void* stream) {
  using namespace ekv;
  const void* src[3] = {q_src, k_src, v_src};
  void* dst[3] = {q_dst, k_dst, v_dst};
  const size_t bytes[3] = {q_bytes, k_bytes, v_bytes};
  StageCopy s{};
  size_t most = 0;
  for (int i = 0; i < 3; ++i) {
    if (!src[i] || !dst[i] || bytes[i] % 16 || bytes[i] > ((size_t)1 << 34) ||
        ((reinterpret_cast<uintptr_t>(src[i]) | reinterpret_cast<uintptr_t>(dst[i])) & 15))
      return EKV_ERR_ARG;
    s.src[i] = static_cast<const uint4*>(src[i]);
    s.dst[i] = static_cast<uint4*>(dst[i]);
    s.n16[i] = (int)(bytes[i] / 16);
    most = bytes[i] > most ? bytes[i] : most;
  }
  if (most == 0) return EKV_OK;
  const size_t blocks = (most / 16 + 255) / 256;
  dim3 grid((unsigned)(blocks < 1024 ? blocks : 1024), 3);
  stage_inputs_kernel<<<grid, 256, 0, as_stream(stream)>>>(s);
  return launch_status();
}

extern "C" int ekv_copy_timeouts(uint32_t* count) {
  if (!count) return EKV_ERR_ARG;
  *count = ekv::copy_timeouts_topk() + ekv::copy_timeouts_gaussian() + ekv::copy_timeouts_decode() +
           ekv::copy_timeouts_fused_small() + ekv::copy_timeouts_stream_topk();
  return ekv::launch_status();
}

extern "C" int ekv_version(void) { return 103; }
