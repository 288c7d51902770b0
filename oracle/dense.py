"""Oracle: dense entmax decode attention on the CPU (test infrastructure).

This is the reference test-suite's yardstick, ``reference_attention``
(tests/benchmark_utils.py:56-83): ``softmax``-like attention over the *whole*
cache with the alpha-entmax mapping in place of softmax.  The reference obtains
the mapping from a Triton-only kernel (entmaxkv/kernels/triton_entmax.py:686),
which cannot run without a GPU, so the mapping is restated from its
definition: ``p = ((alpha-1) x - tau)_+^(1/(alpha-1))`` with ``sum p = 1``.
For alpha in {1.5, 2} the threshold comes from the sort-based closed forms of
Peters, Niculae & Martins (2019) and Martins & Astudillo (2016); other alphas
use fp64 bisection on [max-1, max].  It is also the timed CPU baseline.
"""

from __future__ import annotations

import math

import torch


def entmax_threshold(x: torch.Tensor, alpha: float) -> torch.Tensor:
    """tau of alpha-entmax along the last axis, in z-space z=(alpha-1)*x.

    Returns tau with a trailing singleton axis, dtype of ``x``.
    """
    a = alpha - 1.0
    z = x * a
    zmax = z.amax(dim=-1, keepdim=True)
    zs = z - zmax                                   # <= 0
    n = z.shape[-1]
    if alpha == 2.0:
        srt = torch.sort(zs, dim=-1, descending=True).values
        cs = srt.cumsum(-1)
        k = torch.arange(1, n + 1, dtype=z.dtype)
        support = (1.0 + k * srt > cs).sum(-1, keepdim=True)
        tau = (cs.gather(-1, support - 1) - 1.0) / support.to(z.dtype)
        return tau + zmax
    if alpha == 1.5:
        srt = torch.sort(zs, dim=-1, descending=True).values
        k = torch.arange(1, n + 1, dtype=z.dtype)
        mean = srt.cumsum(-1) / k
        mean_sq = (srt * srt).cumsum(-1) / k
        ss = k * (mean_sq - mean * mean)
        delta = torch.clamp((1.0 - ss) / k, min=0.0)
        tau_k = mean - torch.sqrt(delta)
        support = (tau_k <= srt).sum(-1, keepdim=True)
        return tau_k.gather(-1, support - 1) + zmax
    beta = 1.0 / a
    lo = torch.full_like(zmax, -1.0)
    hi = torch.zeros_like(zmax)
    zs64 = zs.to(torch.float64)
    lo, hi = lo.to(torch.float64), hi.to(torch.float64)
    for _ in range(60):
        mid = 0.5 * (lo + hi)
        s = torch.clamp(zs64 - mid, min=0.0).pow(beta).sum(-1, keepdim=True)
        lo = torch.where(s > 1.0, mid, lo)
        hi = torch.where(s > 1.0, hi, mid)
    return (0.5 * (lo + hi)).to(z.dtype) + zmax


def entmax(x: torch.Tensor, alpha: float) -> torch.Tensor:
    """alpha-entmax probabilities along the last axis."""
    if alpha == 1.0:
        return torch.softmax(x, dim=-1)
    a = alpha - 1.0
    d = torch.clamp(x * a - entmax_threshold(x, alpha), min=0.0)
    if alpha == 2.0:
        return d
    if alpha == 1.5:
        return d * d
    return d.pow(1.0 / a)


def dense_entmax_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                        alpha: float = 1.5, compute_dtype=torch.float32) -> torch.Tensor:
    """q [B,H,1,D], k/v [B,Hkv,S,D] -> [B,H,1,D] (tests/benchmark_utils.py:64-83).

    K/V are repeat-expanded over a GQA group as the reference tests do
    (tests/test_topk.py:73-76).
    """
    G = q.shape[1] // k.shape[1]
    if G > 1:
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
    qf, kf, vf = q.to(compute_dtype), k.to(compute_dtype), v.to(compute_dtype)
    qk = torch.matmul(qf, kf.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    p = entmax(qk, alpha)
    return torch.matmul(p, vf)
