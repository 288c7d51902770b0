// Moments sweep on the tensor pipe (16-bit bfloat caches, GQA groups of up to eight query heads).
//
// mu_p = s * sum_d q_d k_mean[p,d] and var_p = s^2 * sum_d q_d^2 k_std[p,d]^2 for the G query heads of a
// KV head are two [pages x D] . [D x G] contractions.  On CUDA cores they cost 2*D*G fused
// multiply-adds per page and the sweep is bound by instruction issue, not by the 2*D*2 bytes it reads
// per page.  Here a warp takes 16 pages at a time and lets mma.sync.m16n8k16 (fp32 accumulators) do
// the contractions:
//   * mu: A = k_mean rows as stored, B = the queries as stored - both operands exact, the scale s is
//     applied to the fp32 sum;
//   * var: k_std^2 and q^2 do not fit 16-bit operands, but the square of a bfloat (8-bit significand)
//     has at most 16 significant bits and splits EXACTLY into two bfloats, hi = round(x*x) and
//     lo = fma(x, x, -hi), both formed by packed 16-bit arithmetic directly on the fragment registers
//     (one instruction per element pair each).  With q^2 split the same way, four tensor-core steps
//     (hi*hi, hi*lo, lo*hi, lo*lo) accumulate the exact products in fp32; s^2 = 1/D is applied at the end.
// Data movement: an NS-stage shared-memory ring of tiles filled by bulk asynchronous copies - while one
// tile is in the tensor pipe the copies of the next NS-1 are in flight.  A tile of 16*WARPS pages is
// copied as eight slots of 2*WARPS pages, every slot placed 16 bytes further (mod 128) than the previous
// one, so that the eight rows an ldmatrix instruction gathers - one page of each slot - fall into eight
// different bank groups (rows of consecutive pages are a multiple of 128 bytes apart and would all collide).
#pragma once

namespace ekv {

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// x*x of a bfloat pair as hi + lo, exactly
__device__ __forceinline__ void square_split(uint32_t x, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&x);
  const __nv_bfloat162 h = __hmul2(v, v);
  const __nv_bfloat162 l = __hfma2(v, v, __hneg2(h));
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

// Sequence-sharded step: the sweep's last block of a KV head also trades the head sums with the
// other ranks (exchange slot 0) and finishes the head statistics from the global sequence lengths.
struct MomentsXch {
  XchDev xch;
  int use;
  int* status;
  const int* total_lens;   // device int32 [B]: tokens of the whole request (all ranks)
};

template <int D, int WARPS, int NS>
struct MomMma {
  static constexpr int kThreads = 32 * WARPS;
  static constexpr int kTilePages = 16 * WARPS;               // one 16-page fragment row block per warp
  static constexpr int kSlotPages = 2 * WARPS;
  static constexpr int kRowBytes = D * 2;
  static constexpr int kSlotBytes = kSlotPages * kRowBytes + 16;   // the slot's pages + the skew
  static constexpr int kArrayBytes = 8 * kSlotBytes;          // one statistic of a tile
  static constexpr int kStageBytes = 2 * kArrayBytes;         // k_mean | k_std
  static constexpr int kOutStride = kTilePages + 4;           // staged results: [mu|sigma][8 heads][tile pages]
  static constexpr size_t kSmem = (size_t)NS * kStageBytes + 2 * 2 * 8 * kOutStride * sizeof(float);
};

// grid: (blocks, B*H_kv); a block owns 64 * ws.tpb consecutive pages of one KV head; same ticket / fold
// structure as gaussian_moments_kernel.
template <int D, bool ALIBI, int WARPS, int NS, int BPS>
__global__ void __launch_bounds__(32 * WARPS, BPS)
gaussian_moments_mma_kernel(ekv_cache_desc c, const __nv_bfloat16* __restrict__ q, int64_t qsb, int64_t qsh,
                            int q_heads, int exclude_last, float alpha, int finalize, float* __restrict__ mu_pages,
                            float* __restrict__ sigma_pages, int64_t pstride, float* __restrict__ head_sums,
                            float* __restrict__ head_stats, GaussianWs ws, const float* __restrict__ alibi_slopes,
                            const int* __restrict__ q_positions, const MomentsXch mx) {
  using L = MomMma<D, WARPS, NS>;
  constexpr int KS = D / 16;
  constexpr int TILE = L::kTilePages;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  float* s_out = reinterpret_cast<float*>(smem_raw + (size_t)NS * L::kStageBytes);   // [parity][mu|sigma][8][kOutStride]
  __shared__ uint64_t bar[NS];
  __shared__ float red[WARPS][8][4];      // [warp][head][sum]
  __shared__ int s_ticket;

  // sequence-sharded step: every block joins the exchange's launch count before it can leave
  Xch xe;
  if (mx.use) xe = xch_begin(mx.xch, 0, mx.status);
  const int bh = blockIdx.y;
  const int b = bh / c.kv_heads, hkv = bh % c.kv_heads;
  const int G = q_heads / c.kv_heads;
  const int S = c.seq_lens[b];
  const int P = c.page_size;
  const int n_pages = (S + P - 1) / P;
  const int n_stats = min((exclude_last && n_pages > 1) ? n_pages - 1 : n_pages, c.page_capacity);
  const int kPagesPerBlock = kMomPagesPerBlock * ws.tpb;
  const int my_blocks = (n_stats + kPagesPerBlock - 1) / kPagesPerBlock;
  if ((int)blockIdx.x >= my_blocks) return;
  const int first_page = blockIdx.x * kPagesPerBlock;
  const int n_tiles = (min(kPagesPerBlock, n_stats - first_page) + TILE - 1) / TILE;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t head_off = b * c.meta_stride_b + hkv * c.meta_stride_h;
  const __nv_bfloat16* g_mean = static_cast<const __nv_bfloat16*>(c.k_mean) + head_off;
  const __nv_bfloat16* g_std = static_cast<const __nv_bfloat16*>(c.k_std) + head_off;

  // Lanes 0..15 of warp 0 each launch one slot copy of a tile (eight slots per statistic).
  auto issue = [&](int t) {
    const int page0 = first_page + t * TILE;
    const int npg = min(TILE, n_stats - page0);
    const int st = t % NS;
    unsigned char* dst = smem_raw + (size_t)st * L::kStageBytes;
    if (lane == 0) mbar_expect_tx(&bar[st], 2u * (uint32_t)(npg * L::kRowBytes));
    __syncwarp();
    if (lane < 16) {
      const int s = lane & 7, arr = lane >> 3;
      const int rows = min(L::kSlotPages, npg - L::kSlotPages * s);
      if (rows > 0)
        bulk_load(dst + arr * L::kArrayBytes + s * L::kSlotBytes,
                  (arr ? g_std : g_mean) + (size_t)(page0 + L::kSlotPages * s) * D, (uint32_t)(rows * L::kRowBytes),
                  &bar[st]);
    }
  };
  __shared__ int s_timeout;      // a bounded wait on a copy ran out (reported once, after the tile loop)
  if (tid == 0) {
    s_timeout = 0;
#pragma unroll
    for (int i = 0; i < NS; ++i) mbar_init(&bar[i], 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 0)
    for (int t = 0; t < min(NS, n_tiles); ++t) issue(t);

  // B fragments: column n = head n of the group (zero beyond G), rows = head_dim
  const int g = lane >> 2, t4 = lane & 3;
  uint32_t bq[KS][2], bh2[KS][2], bl2[KS][2];
  {
    const __nv_bfloat16* qrow = q + b * qsb + (hkv * G + min(g, G - 1)) * qsh;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const uint32_t w0 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
      const uint32_t w1 = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t4);
      bq[ks][0] = g < G ? w0 : 0u;
      bq[ks][1] = g < G ? w1 : 0u;
      square_split(bq[ks][0], bh2[ks][0], bl2[ks][0]);
      square_split(bq[ks][1], bh2[ks][1], bl2[ks][1]);
    }
  }
  static_assert(D == 64 || D == 128, "1/sqrt(D) constants below cover D = 64 and 128");
  const float scale = D == 64 ? 0.125f : 0.08838834764831845f;   // fp32(1/sqrt(D))
  const float scale2 = 1.f / (float)D;
  // ldmatrix row of this lane: matrix m = lane / 8 (bit 0: rows 8..15, bit 1: upper k half), row r = lane % 8
  // = slot r of the tile, page (2 * warp + (m & 1)) of the slot
  const uint32_t frag_off = (uint32_t)((lane & 7) * L::kSlotBytes + (2 * warp + ((lane >> 3) & 1)) * L::kRowBytes +
                                       (lane >> 4) * 16);
  // accumulator rows of this lane: pages kSlotPages*g + 2*warp (+1) of the tile; columns: heads 2*t4, 2*t4+1
  const int pg_in_tile = L::kSlotPages * g + 2 * warp;
  const int h_a = 2 * t4, h_b = 2 * t4 + 1;
  float sums[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  float slope_a = 0.f, slope_b = 0.f, q_posf = 0.f, last_stat_pos = 0.f;
  if constexpr (ALIBI) {
    slope_a = h_a < G ? alibi_slopes[hkv * G + h_a] : 0.f;
    slope_b = h_b < G ? alibi_slopes[hkv * G + h_b] : 0.f;
    q_posf = (float)(q_positions ? q_positions[b] : S - 1);
    last_stat_pos = (float)(((exclude_last && n_pages > 1) ? (n_pages - 1) * P : S) - 1);
  }

  for (int t = 0; t < n_tiles; ++t) {
    const int page0 = first_page + t * TILE;
    const int npg = min(TILE, n_stats - page0);
    const int st = t % NS;
    const uint32_t a_mean = smem_addr(smem_raw + (size_t)st * L::kStageBytes) + frag_off;
    const uint32_t a_std = a_mean + L::kArrayBytes;
    mbar_wait_or_mark(&bar[st], (uint32_t)(t / NS) & 1u, &s_timeout);
    float dm[4] = {0.f, 0.f, 0.f, 0.f}, dv0[4] = {0.f, 0.f, 0.f, 0.f}, dv1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t am[4], as[4], ah[4], al[4];
      ldsm_x4(a_mean + ks * 32, am);
      ldsm_x4(a_std + ks * 32, as);
      mma_bf16_16816(dm, am, bq[ks][0], bq[ks][1]);
#pragma unroll
      for (int i = 0; i < 4; ++i) square_split(as[i], ah[i], al[i]);
      mma_bf16_16816(dv0, ah, bh2[ks][0], bh2[ks][1]);
      mma_bf16_16816(dv1, al, bh2[ks][0], bh2[ks][1]);
      mma_bf16_16816(dv0, ah, bl2[ks][0], bl2[ks][1]);
      mma_bf16_16816(dv1, al, bl2[ks][0], bl2[ks][1]);
    }
    // results of this lane: {page, page+1} x {head h_a, head h_b}
    float* o_mu = s_out + (size_t)(t & 1) * 2 * 8 * L::kOutStride;
    float* o_sg = o_mu + 8 * L::kOutStride;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int p = pg_in_tile + r;
      const bool live_p = p < npg;
#pragma unroll
      for (int cidx = 0; cidx < 2; ++cidx) {
        const int h = cidx ? h_b : h_a;
        const float m = dm[2 * r + cidx] * scale;
        const float v = (dv0[2 * r + cidx] + dv1[2 * r + cidx]) * scale2;
        const float sg = sqrtf(v);
        float mb = m;
        if constexpr (ALIBI) {
          const float mean_pos = fminf((float)((page0 + p) * P) + 0.5f * (float)(P - 1), last_stat_pos);
          mb = __fadd_rn(m, __fmul_rn(cidx ? slope_b : slope_a, mean_pos - q_posf));
        }
        o_mu[h * L::kOutStride + p] = mb;
        o_sg[h * L::kOutStride + p] = sg;
        if (live_p && h < G) {
          sums[cidx][0] += m;
          sums[cidx][1] += m * m;
          sums[cidx][2] += v;
          sums[cidx][3] += mb + 1.5f * sg;
        }
      }
    }
    __syncthreads();   // the stage is free, the staged results are complete
    if (warp == 0 && t + NS < n_tiles) issue(t + NS);
    // coalesced stores: consecutive threads write consecutive pages of one head
    for (int i = tid; i < G * TILE; i += L::kThreads) {
      const int h = i / TILE, p = i % TILE;
      if (p < npg) {
        const size_t o = ((size_t)b * q_heads + hkv * G + h) * pstride + page0 + p;
        mu_pages[o] = o_mu[h * L::kOutStride + p];
        sigma_pages[o] = o_sg[h * L::kOutStride + p];
      }
    }
  }
  // fold the lanes that share a head pair (same t4, the eight g), then the warps, in a fixed order
#pragma unroll
  for (int cidx = 0; cidx < 2; ++cidx)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float v = sums[cidx][k];
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      if (g == 0) red[warp][2 * t4 + cidx][k] = v;
    }
  __syncthreads();
  if (tid == 0 && s_timeout) note_copy_timeout(nullptr);
  if (tid < G * 4) {
    const int h = tid / 4, k = tid % 4;
    float tsum = red[0][h][k];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) tsum += red[w][h][k];
    ws.partial[(((size_t)b * q_heads + hkv * G + h) * ws.tiles + blockIdx.x) * 4 + k] = tsum;
  }

  // last block of this KV head folds the blocks' partial sums
  __threadfence();
  __syncthreads();
  if (tid == 0) s_ticket = atomicAdd(&ws.counters[bh], 1);
  __syncthreads();
  if (s_ticket != my_blocks - 1) return;
  __threadfence();
  for (int gh = warp; gh < G; gh += WARPS) {
    const int hq = hkv * G + gh;
    const float* part = ws.partial + ((size_t)b * q_heads + hq) * ws.tiles * 4;
    float tt[4] = {0.f, 0.f, 0.f, 0.f};
    for (int blk = lane; blk < my_blocks; blk += 32)
#pragma unroll
      for (int k = 0; k < 4; ++k) tt[k] += ld_cg(part + blk * 4 + k);
#pragma unroll
    for (int k = 0; k < 4; ++k) tt[k] = warp_sum(tt[k]);
    if (lane == 0) {
      float* hs = head_sums + ((size_t)b * q_heads + hq) * 4;
#pragma unroll
      for (int k = 0; k < 4; ++k) hs[k] = tt[k];
    }
    if (mx.use) {
      // sequence-sharded step: this rank's sums of the head go to the peers, theirs are added in rank
      // order, and the head's statistics and tau_hat follow from the request's GLOBAL length - what a
      // separate exchange kernel would do one launch later
      const int i = b * q_heads + hq;
      const float own = lane == 0 ? tt[0] : (lane == 1 ? tt[1] : (lane == 2 ? tt[2] : tt[3]));
      if (lane < 4) xe.send(i * 4 + lane, own);
      float mine = 0.f;
      if (lane < 4) mine = xe.sum(i * 4 + lane, own);
      float sw[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) sw[k] = __shfl_sync(0xffffffffu, mine, k);
      const int Sg = mx.total_lens[b];
      const int np = (Sg + P - 1) / P;
      finalize_head_warp(sw, (float)(np > 1 ? np - 1 : np), (float)(np > 1 ? (np - 1) * P : Sg), alpha,
                         head_stats + (size_t)i * 4);
    } else if (finalize) {   // the whole warp solves this head's tau_hat (finalize == 2: tau_hat comes later)
      const float n_tok = (exclude_last && n_pages > 1) ? (float)(n_pages - 1) * (float)P : (float)S;
      finalize_head_warp(tt, (float)n_stats, n_tok, alpha, head_stats + ((size_t)b * q_heads + hq) * 4,
                         finalize != 2);
    }
  }
  if (tid == 0) ws.counters[bh] = 0;
}

}  // namespace ekv
