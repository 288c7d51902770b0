"""Oracle: per-page key statistics (test infrastructure, CPU only).

Follows ``PagedKVCache.initialize`` (entmaxkv/kv_cache.py:40-70) and
``PagedKVCache.append`` (entmaxkv/kv_cache.py:72-116): for every page of
``page_size`` consecutive keys the cache keeps min, max, mean and the
population standard deviation (clamped at 1e-6), all stored in the key dtype.

Arithmetic contract (what the CUDA kernels are compared against bit for bit):
values are widened to fp32; rows of a page are visited in storage order;
``mean = (((x0 + x1) + x2) + ...) / n``;
``var = ((d0*d0 + d1*d1) + ...) / n`` with ``d = x - mean``, products and sums
rounded separately (no fused multiply-add); ``std = max(sqrt(var), 1e-6)``;
each statistic is then rounded once to the storage dtype.  The reference
leaves the accumulation order to torch, so against the reference itself mean
and std are compared to within one unit in the last place of the storage
dtype, min and max exactly.
"""

from __future__ import annotations

import numpy as np
import torch


def page_stats(k: torch.Tensor, page_size: int, seq_len: int | None = None):
    """Statistics of every page of ``k[:, :, :seq_len]``.

    k: [B, H, S, D] (any float dtype).  Returns (k_min, k_max, k_mean, k_std),
    each [B, H, ceil(seq_len/page_size), D] in ``k.dtype``
    (entmaxkv/kv_cache.py:47-70).
    """
    B, H, S, D = k.shape
    if seq_len is None:
        seq_len = S
    P = page_size
    n_pages = (seq_len + P - 1) // P
    kf = k[:, :, :seq_len].to(torch.float32)
    pad = n_pages * P - seq_len
    if pad:
        kf = torch.cat([kf, torch.zeros(B, H, pad, D)], dim=2)
    kf = kf.view(B, H, n_pages, P, D)
    counts = torch.full((n_pages,), P, dtype=torch.int64)
    if pad:
        counts[-1] = P - pad

    vmin = torch.full((B, H, n_pages, D), float("inf"))
    vmax = torch.full((B, H, n_pages, D), float("-inf"))
    acc = torch.zeros(B, H, n_pages, D)
    for r in range(P):
        valid = (r < counts).view(1, 1, n_pages, 1)
        x = kf[:, :, :, r, :]
        vmin = torch.where(valid, torch.minimum(vmin, x), vmin)
        vmax = torch.where(valid, torch.maximum(vmax, x), vmax)
        acc = torch.where(valid, acc + x, acc)
    n = counts.to(torch.float32).view(1, 1, n_pages, 1)
    mean = acc / n
    acc2 = torch.zeros(B, H, n_pages, D)
    for r in range(P):
        valid = (r < counts).view(1, 1, n_pages, 1)
        d = kf[:, :, :, r, :] - mean
        acc2 = torch.where(valid, acc2 + d * d, acc2)
    # numpy's sqrt is correctly rounded; torch's vectorised CPU sqrt is not always
    std = torch.from_numpy(np.sqrt((acc2 / n).numpy())).clamp(min=1e-6)
    dt = k.dtype
    return vmin.to(dt), vmax.to(dt), mean.to(dt), std.to(dt)


class OracleCache:
    """Plain restatement of the reference cache object (kv_cache.py:16-116).

    Keeps dense K/V and the four statistics tensors; ``append`` concatenates a
    token and recomputes the statistics of the page that token falls in.
    """

    def __init__(self, page_size: int = 16):
        self.page_size = page_size
        self.k_cache = self.v_cache = None
        self.k_min = self.k_max = self.k_mean = self.k_std = None

    def initialize(self, k: torch.Tensor, v: torch.Tensor):
        self.k_cache = k.clone()
        self.v_cache = v.clone()
        self.k_min, self.k_max, self.k_mean, self.k_std = page_stats(k, self.page_size)

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor):
        self.k_cache = torch.cat([self.k_cache, k_new], dim=2)
        self.v_cache = torch.cat([self.v_cache, v_new], dim=2)
        S = self.k_cache.shape[2]
        P = self.page_size
        page = (S - 1) // P
        mn, mx, me, sd = page_stats(self.k_cache[:, :, page * P:S], P)
        if page >= self.k_min.shape[2]:
            self.k_min = torch.cat([self.k_min, mn], dim=2)
            self.k_max = torch.cat([self.k_max, mx], dim=2)
            self.k_mean = torch.cat([self.k_mean, me], dim=2)
            self.k_std = torch.cat([self.k_std, sd], dim=2)
        else:
            self.k_min[:, :, page] = mn[:, :, 0]
            self.k_max[:, :, page] = mx[:, :, 0]
            self.k_mean[:, :, page] = me[:, :, 0]
            self.k_std[:, :, page] = sd[:, :, 0]

    @property
    def seq_len(self) -> int:
        return self.k_cache.shape[2]
