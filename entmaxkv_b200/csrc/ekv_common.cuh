// Shared device helpers of the sm_100a sparse entmax decode kernels.
//
// Element access is always in 16-byte chunks: a row of D elements is covered by
// LPR = D*sizeof(T)/16 consecutive lanes, each owning EPL = 16/sizeof(T) elements.
// Sums over D are formed in a fixed order - left to right inside a lane, then a
// halving butterfly across the LPR lanes - so results are reproducible and, for
// 16-bit inputs (whose pairwise products are exact in fp32), bit-identical to
// the CPU oracle's restatement of the same order.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/entmaxkv_b200.h"

namespace ekv {

constexpr int kChunkTokens = 256;   // tokens per decode work item
constexpr int kBins = 16;           // histogram bins of the exact tau bracket

template <typename T> struct ElemTraits;
template <> struct ElemTraits<__half> { static constexpr int EPL = 8; };
template <> struct ElemTraits<__nv_bfloat16> { static constexpr int EPL = 8; };
template <> struct ElemTraits<float> { static constexpr int EPL = 4; };

// ---- 16-byte loads ---------------------------------------------------------

// Streaming read-only load: data that is touched once per step (K, V, page
// statistics) should not displace the small reused state in L1.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// L2-coherent scalar loads for data another thread block wrote in this launch.
__device__ __forceinline__ float ld_cg(const float* p) { return __ldcg(p); }
__device__ __forceinline__ int ld_cg(const int* p) { return __ldcg(p); }

template <typename T>
__device__ __forceinline__ void unpack(const uint4& r, float (&f)[ElemTraits<T>::EPL]);

template <>
__device__ __forceinline__ void unpack<__half>(const uint4& r, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& r, float (&f)[8]) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack<float>(const uint4& r, float (&f)[4]) {
  f[0] = __uint_as_float(r.x);
  f[1] = __uint_as_float(r.y);
  f[2] = __uint_as_float(r.z);
  f[3] = __uint_as_float(r.w);
}

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }

template <typename T>
__device__ __forceinline__ uint4 pack(const float (&f)[ElemTraits<T>::EPL]);
template <>
__device__ __forceinline__ uint4 pack<__half>(const float (&f)[8]) {
  uint4 r;
  __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  return r;
}
template <>
__device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float (&f)[8]) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return r;
}
template <>
__device__ __forceinline__ uint4 pack<float>(const float (&f)[4]) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                    __float_as_uint(f[3]));
}

// ---- bulk asynchronous copies (TMA, 1-D) into shared memory --------------------
//
// One thread arms an mbarrier with the byte count it expects, any threads issue
// cp.async.bulk copies that complete on it, everybody waits on the phase parity.
// Source, destination and size must be multiples of 16 bytes.  No multicast.

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals));
}
// make the initialised barrier visible to the async proxy that completes the copies
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}
// Bounded wait: returns false if the phase did not complete within the limit, so a
// copy that never lands cannot hang the GPU (the caller's result is then undefined, not
// the machine).  Each attempt lets the hardware park the thread for up to ~0.1 ms instead
// of spinning, so waiting warps do not take issue slots from the warps that compute.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t a = smem_addr(bar);
  for (int it = 0; it < (1 << 15); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity), "r"(100000u)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// Bulk copies that did not land within the bounded wait, counted per translation unit (the library is built
// without relocatable device code, so every .cu file has its own counter; ekv_copy_timeouts adds them up).
static __device__ unsigned int g_copy_timeouts;
// The wait every kernel uses: on a timeout the launch's results are undefined, and the host can find out -
// the counter above, and EKV_STATUS_COPY_TIMEOUT in `status` where the kernel has a status word.
// (the bookkeeping is a call, not inline code: inlined into the issue-bound score sweep it cost registers on
// the path every tile takes and 8 % of that kernel's time)
static __device__ __noinline__ void note_copy_timeout(int* status) {
  atomicAdd(&g_copy_timeouts, 1u);
  if (status) atomicOr(status, EKV_STATUS_COPY_TIMEOUT);
}
__device__ __forceinline__ void mbar_wait_or_flag(uint64_t* bar, uint32_t parity, int* status) {
  if (!mbar_wait(bar, parity)) note_copy_timeout(status);
}
// The sweeps' form: a timed-out wait only raises a flag in shared memory (zeroed by the block before its first
// barrier); the block's last act, report_copy_timeout, turns it into the counter.
__device__ __forceinline__ void mbar_wait_or_mark(uint64_t* bar, uint32_t parity, int* s_flag) {
  if (!mbar_wait(bar, parity)) *s_flag = 1;
}
__device__ __forceinline__ void report_copy_timeout(const int* s_flag) {
  __syncthreads();
  if (threadIdx.x == 0 && *s_flag) note_copy_timeout(nullptr);
}
// host: this translation unit's counter (synchronises the device)
static inline unsigned int copy_timeouts_here() {
  unsigned int v = 0;
  return cudaMemcpyFromSymbol(&v, g_copy_timeouts, sizeof(v)) == cudaSuccess ? v : 0u;
}
// one accessor per source file that waits on bulk copies
unsigned int copy_timeouts_topk();
unsigned int copy_timeouts_gaussian();
unsigned int copy_timeouts_decode();
unsigned int copy_timeouts_fused_small();
unsigned int copy_timeouts_stream_topk();

// Division by a run-time constant as multiply-high + shift (n < 2^31).
struct FastDiv {
  uint32_t mul;
  int shift;
  int d;
  __device__ __forceinline__ int div(int n) const {
    return d == 1 ? n : (int)((__umulhi((uint32_t)n, mul) + (uint32_t)n) >> shift);
  }
  __device__ __forceinline__ void divmod(int n, int& q, int& r) const {
    q = div(n);
    r = n - q * d;
  }
};
inline FastDiv make_fast_div(int d) {
  FastDiv f;
  f.d = d;
  int l = 0;
  while ((1u << l) < (uint32_t)d) ++l;
  f.shift = l;
  f.mul = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << l) - (uint64_t)d)) / (uint64_t)d + 1);
  return f;
}

__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// ---- reductions ------------------------------------------------------------

// Butterfly sum over the LPR lanes that share a row (LPR is 8, 16 or 32 and the
// groups are aligned), highest offset first.  Every lane ends with the total.
template <int LPR>
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Two per-lane partial sums (one per head) over the LPR lanes of a row, for the price
// of one: after the first exchange the lower half of the lanes carries head 0 and the
// upper half head 1; lane 0 ends with the total of v0 and lane LPR/2 with the total of
// v1.  The additions pair the same operands, in the same order, as row_sum.
template <int LPR>
__device__ __forceinline__ float row_sum_pair(float v0, float v1, int lane_in_row) {
  const bool upper = (lane_in_row & (LPR / 2)) != 0;
  const float send = upper ? v0 : v1;
  float keep = upper ? v1 : v0;
  keep += __shfl_xor_sync(0xffffffffu, send, LPR / 2);
#pragma unroll
  for (int o = LPR / 4; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
  return keep;
}

// Four per-lane partial sums (four rows, or four heads) over the LPR lanes of a row in
// two exchange steps plus log2(LPR)-2 butterfly steps.  Returns the total of v[r] on the
// lanes whose index satisfies  lane_in_row / (LPR/4) == r  (all LPR/4 lanes of that
// cluster hold it).  The additions of one row pair the same operands, in the same order,
// as row_sum, so the result is bit-identical to row_sum(v[r]).
template <int LPR>
__device__ __forceinline__ float row_sum_quad(const float (&v)[4], int lane_in_row) {
  constexpr int H1 = LPR / 2, H2 = LPR / 4;
  const bool up1 = (lane_in_row & H1) != 0;
  const float a0 = (up1 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, up1 ? v[0] : v[2], H1);
  const float a1 = (up1 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, up1 ? v[1] : v[3], H1);
  const bool up2 = (lane_in_row & H2) != 0;
  float b = (up2 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, up2 ? a0 : a1, H2);
#pragma unroll
  for (int o = H2 / 2; o > 0; o >>= 1) b += __shfl_xor_sync(0xffffffffu, b, o);
  return b;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed combination order (warp butterfly, then warps in
// index order).  `scratch` holds at least 32 floats; all threads get the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nwarp; ++w) t += scratch[w];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = scratch[0];
  for (int w = 1; w < nwarp; ++w) t = fmaxf(t, scratch[w]);
  return t;
}

// Exclusive block scan of a packed pair of 16-bit counters (per-thread values 0/1
// in each half, block size <= 1024 so neither half overflows).  Returns the
// exclusive prefix; *total receives the block total.  scratch: >= 33 uint32.
__device__ __forceinline__ uint32_t block_scan_excl(uint32_t v, uint32_t* scratch, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  uint32_t base = 0, tot = 0;
  for (int w = 0; w < nwarp; ++w) {
    uint32_t s = scratch[w];
    if (w < warp) base += s;
    tot += s;
  }
  *total = tot;
  return base + inc - v;
}

// ---- entmax arithmetic ------------------------------------------------------

// (d)^e for d > 0.
__device__ __forceinline__ float pow_pos(float d, float e) { return exp2f(e * log2f(d)); }

// sum_j contributions of one score to the three Halley sums at threshold tau:
//   s0 += (z-tau)^beta, s1 += (z-tau)^(beta-1), s2 += (z-tau)^(beta-2)  for z > tau.
// alpha_kind: 0 -> alpha == 2, 1 -> alpha == 1.5, 2 -> general.
__device__ __forceinline__ void halley_accumulate(float z, float tau, int alpha_kind, float beta,
                                                  float& s0, float& s1, float& s2) {
  if (z > tau) {
    const float d = z - tau;
    if (alpha_kind == 0) {
      s0 += d;
      s1 += 1.f;
    } else if (alpha_kind == 1) {
      s0 += d * d;
      s1 += d;
      s2 += 1.f;
    } else {
      s0 += pow_pos(d, beta);
      s1 += pow_pos(d, beta - 1.f);
      s2 += pow_pos(d, beta - 2.f);
    }
  }
}

__device__ __forceinline__ float entmax_weight(float z, float tau, int alpha_kind, float beta) {
  const float d = z - tau;
  if (!(d > 0.f)) return 0.f;
  if (alpha_kind == 0) return d;
  if (alpha_kind == 1) return d * d;
  return pow_pos(d, beta);
}

__host__ __device__ inline int alpha_kind_of(float alpha) {
  return alpha == 2.0f ? 0 : (alpha == 1.5f ? 1 : 2);
}

// Unbracketed Halley step with Newton and keep-as-is fallbacks.
__device__ __forceinline__ float halley_unbounded(float t, float s0, float s1, float s2, float beta) {
  const float ff = s0 - 1.f;
  const float df = -beta * s1;
  const float ddf = beta * (beta - 1.f) * s2;
  const float hd = 2.f * df * df - ff * ddf;
  float tn = t;
  if (fabsf(hd) > 1e-12f) {
    tn = t - (2.f * ff * df) / hd;
  } else if (fabsf(df) > 1e-12f) {
    tn = t - ff / df;
  }
  if (!(tn == tn) || !(fabsf(tn) < 1.0e20f)) tn = t;
  return tn;
}

// ---- host-side dispatch helpers ---------------------------------------------

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline int sm_count() {
  static int sms = 0;   // per process; all devices of a box are identical
  if (sms == 0) {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    sms = n;
  }
  return sms;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? EKV_OK : static_cast<int>(e);
}

// Calls f.template operator()<T, D>() for the supported (dtype, head_dim) pairs.
#define EKV_DISPATCH(DTYPE, HDIM, ...)                                            \
  do {                                                                            \
    if ((DTYPE) == EKV_F16 && (HDIM) == 128) { using T = __half; constexpr int D = 128; __VA_ARGS__; }          \
    else if ((DTYPE) == EKV_F16 && (HDIM) == 64) { using T = __half; constexpr int D = 64; __VA_ARGS__; }      \
    else if ((DTYPE) == EKV_BF16 && (HDIM) == 128) { using T = __nv_bfloat16; constexpr int D = 128; __VA_ARGS__; } \
    else if ((DTYPE) == EKV_BF16 && (HDIM) == 64) { using T = __nv_bfloat16; constexpr int D = 64; __VA_ARGS__; }  \
    else if ((DTYPE) == EKV_F32 && (HDIM) == 128) { using T = float; constexpr int D = 128; __VA_ARGS__; }     \
    else if ((DTYPE) == EKV_F32 && (HDIM) == 64) { using T = float; constexpr int D = 64; __VA_ARGS__; }       \
    else return EKV_ERR_DTYPE;                                                    \
  } while (0)

// Element offset of row 0 of page `page` of (b, h_kv) in K / V: dense layout or block table.
// Returns false (and leaves `off` at a valid in-bounds value) when the table names a block outside the pool.
__device__ __forceinline__ bool kv_page_offset(const ekv_cache_desc& c, int b, int hkv, int page, size_t& off) {
  if (c.block_table) {
    const int blk = c.block_table[(size_t)b * c.bt_stride + page];
    const bool ok = (unsigned)blk < (unsigned)c.num_blocks;
    off = (size_t)(ok ? blk : 0) * c.kv_stride_block + (size_t)hkv * c.kv_stride_h;
    return ok;
  }
  off = (size_t)b * c.kv_stride_b + (size_t)hkv * c.kv_stride_h + (size_t)page * c.page_size * c.head_dim;
  return true;
}

inline int check_desc(const ekv_cache_desc* c) {
  if (!c || !c->k || !c->v || !c->seq_lens) return EKV_ERR_ARG;
  if (c->batch <= 0 || c->kv_heads <= 0 || c->page_size <= 0 || c->capacity <= 0 ||
      c->page_capacity <= 0)
    return EKV_ERR_ARG;
  if (c->dtype < EKV_F16 || c->dtype > EKV_F32) return EKV_ERR_DTYPE;
  if (c->head_dim != 64 && c->head_dim != 128) return EKV_ERR_DTYPE;
  const int64_t esz = c->dtype == EKV_F32 ? 4 : 2;
  // 16-byte accesses need 16-byte aligned row starts
  if ((c->kv_stride_b * esz) % 16 || (c->kv_stride_h * esz) % 16 ||
      (c->meta_stride_b * esz) % 16 || (c->meta_stride_h * esz) % 16)
    return EKV_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(c->k) | reinterpret_cast<uintptr_t>(c->v)) & 15) return EKV_ERR_ARG;
  if (c->block_table) {
    if (c->num_blocks <= 0 || c->bt_stride < c->page_capacity || (c->kv_stride_block * esz) % 16 ||
        c->kv_stride_block < (int64_t)c->page_size * c->head_dim)
      return EKV_ERR_ARG;
  }
  return EKV_OK;
}

}  // namespace ekv
