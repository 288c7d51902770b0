// The exact-mode tau procedure's scalar pieces, shared by the per-head tau kernel of the paged decode
// and by the fused small-problem step: the bracket from the 16-bin histogram and the bracketed Halley
// step (entmaxkv/kernels/adadecode.py:12-112,381-426).
#pragma once

#include "ekv_common.cuh"

namespace ekv {

// Bracket [t_lo, t_hi] from the 16-bin histogram of z on [max-1, max].
__device__ inline void bracket_from_hist(const int* hist, float zmax, float alpha, int kind, float& t_lo, float& t_hi) {
  if (kind != 2) {
    float sz = 1.f, sk = 1.f, sz2 = 1.f;
    for (int sj = kBins - 1; sj >= 0; --sj) {
      const float cnt = (float)hist[sj] - (sj == kBins - 1 ? 1.f : 0.f);
      const float ct = (float)sj / (float)kBins;
      const float nz = sz + cnt * ct, nk = sk + cnt, nz2 = sz2 + cnt * (ct * ct);
      const bool ok = kind == 0 ? (nz - nk * ct) < 1.f : (nk * ct * ct - 2.f * nz * ct + nz2) < 1.f;
      if (ok) {
        sz = nz;
        sk = nk;
        sz2 = nz2;
      }
    }
    float t_init;
    if (kind == 0) {
      t_init = zmax + (sz - 1.f) / sk - 1.f;
    } else {
      const float disc = sz * sz - sk * (sz2 - 1.f);
      t_init = zmax + (sz - sqrtf(disc)) / sk - 1.f;
    }
    t_lo = t_init;
    t_hi = t_init + 1.f / (float)kBins;
    return;
  }
  // general alpha: binary search for the bin whose edges bracket the root
  const float p = 1.f / (alpha - 1.f);
  int lo = 0, hi = kBins - 1, found = 0, b_idx = 0;
  for (int it = 0; it < 5; ++it) {
    const int mid = (int)((float)(lo + hi) * 0.5f);
    float fL = -1.f, fU = -1.f;
    for (int bin = 0; bin < kBins; ++bin) {
      const int off = bin - mid;
      if (off < 0) continue;
      const float cnt = (float)hist[bin] - (bin == kBins - 1 ? 1.f : 0.f);
      const float zL = (float)off / (float)kBins, zU = ((float)off + 1.f) / (float)kBins;
      if (zL > 0.f) fL += cnt * pow_pos(zL, p);
      fU += cnt * pow_pos(zU, p);
    }
    const bool go_right = fL > 0.f, go_left = fU < 0.f;
    if (!found) {
      if (!go_right && !go_left) {
        b_idx = mid;
        found = 1;
      }
      if (go_right) lo = mid + 1;
      if (go_left) hi = mid - 1;
    }
  }
  const int b_sel = found ? b_idx : min(lo, kBins - 1);
  const float t0 = zmax - 1.f;
  t_lo = t0 + (float)b_sel / (float)kBins;
  t_hi = t0 + (float)min(b_sel + 1, kBins) / (float)kBins;
}

__device__ __forceinline__ void halley_bracketed(float& t, float& t_lo, float& t_hi, float s0, float s1,
                                                 float s2, float beta) {
  const float ff = s0 - 1.f;
  const float df = -beta * s1;
  const float ddf = beta * (beta - 1.f) * s2;
  if (ff > 0.f) t_lo = t;
  if (ff < 0.f) t_hi = t;
  const float nt = t - (2.f * ff * df) / (2.f * df * df - ff * ddf);
  const bool good = (nt > t_lo - 1e-6f) && (nt < t_hi + 1e-6f);
  t = good ? nt : 0.5f * (t_lo + t_hi);
}

}  // namespace ekv
