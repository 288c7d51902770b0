"""Seeded synthetic decode-step workloads (shapes and value distributions of the
benchmark configurations; no dataset is involved anywhere in this library).

Inputs are iid N(0,1) like the reference's own tests and benchmark script
(tests/test_topk.py:55-67, tests/run_benchmarks.py:56-66).  In a chosen fraction of
the full pages ("needle" pages, one Bernoulli mask shared by every batch row and
head) the keys are shifted by ``0.5*sqrt(D)*q_hat`` so that those pages dominate
the scores; for a GQA group ``q_hat`` is the unit query of the group's first head.

Generation order is fixed - k, v, q, k_new, v_new, needle mask - and everything is
drawn in fp32 and then cast, so the same seed gives the same bits on the CPU (for
the oracle) and on the GPU path (tensors are copied, not re-drawn).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class Workload:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    head_dim: int
    context: int                 # tokens in the cache before the step's append (max over batch)
    page_size: int = 16
    dtype: torch.dtype = torch.float16
    alpha: float = 1.5
    seed: int = 0
    needle_fraction: float = 0.01
    mode: str = "topk"           # "topk" | "gaussian"
    token_budget: int = 2048
    tau_mode: str = "corrected"
    context_range: Optional[tuple] = None    # (lo, hi): ragged contexts drawn uniformly
    extra: dict = field(default_factory=dict)


CONFIGS = {
    # the reference's CPU-runnable case
    "cpu_fp32_1k": Workload("cpu_fp32_1k", 1, 32, 32, 128, 1024, dtype=torch.float32, seed=0,
                            needle_fraction=0.0, token_budget=256),
    "topk_32k": Workload("topk_32k", 1, 32, 32, 128, 32768, dtype=torch.float16, seed=1,
                         token_budget=2048, mode="topk"),
    "gaussian_ragged": Workload("gaussian_ragged", 8, 32, 32, 128, 65536, dtype=torch.float16, seed=2,
                                mode="gaussian", context_range=(16384, 65536)),
    "gqa_128k_topk": Workload("gqa_128k_topk", 32, 32, 8, 128, 131072, dtype=torch.bfloat16, seed=3,
                              token_budget=4096, mode="topk"),
    "gqa_128k_gaussian": Workload("gqa_128k_gaussian", 32, 32, 8, 128, 131072, dtype=torch.bfloat16,
                                  seed=3, mode="gaussian"),
    "million_gaussian": Workload("million_gaussian", 1, 64, 8, 128, 1048576, dtype=torch.bfloat16,
                                 seed=4, needle_fraction=0.001, mode="gaussian"),
}


def make_inputs(w: Workload, device="cpu", batch_slice: Optional[slice] = None,
                kv_head_slice: Optional[slice] = None):
    """Draw the tensors of ``w`` on ``device``.

    Returns dict(k, v, q, k_new, v_new, seq_lens, needle_pages).  On a CUDA device the
    draws use that device's generator (large configurations cannot be staged through
    host memory); parity tests draw on the CPU and copy.
    ``batch_slice`` / ``kv_head_slice`` restrict the tensors to one shard of a
    batch x KV-head partition; each shard is drawn from its own seed stream
    (seed, first batch row, first KV head), so shards do not depend on world size
    only through their own coordinates.
    """
    B, Hq, Hkv, D, S, P = w.batch, w.q_heads, w.kv_heads, w.head_dim, w.context, w.page_size
    G = Hq // Hkv
    b0, b1 = (0, B) if batch_slice is None else (batch_slice.start, batch_slice.stop)
    h0, h1 = (0, Hkv) if kv_head_slice is None else (kv_head_slice.start, kv_head_slice.stop)
    nb, nh = b1 - b0, h1 - h0
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(w.seed * 1000003 + b0 * 1009 + h0)

    def randn(*shape):
        # drawn in the storage dtype's fp32 pre-image in pieces to bound peak memory
        out = torch.empty(shape, dtype=w.dtype, device=dev)
        flat = out.view(shape[0], -1)
        for i in range(shape[0]):
            flat[i] = torch.randn(flat.shape[1], generator=gen, device=dev, dtype=torch.float32).to(w.dtype)
        return out

    k = randn(nb, nh, S, D)
    v = randn(nb, nh, S, D)
    q = randn(nb, nh * G, 1, D)
    k_new = randn(nb, nh, 1, D)
    v_new = randn(nb, nh, 1, D)
    n_full_pages = S // P
    # masks and lengths depend on the seed only, so every shard sees the same ones
    mgen = torch.Generator(device="cpu")
    mgen.manual_seed(w.seed * 7919 + 17)
    needle = torch.rand(n_full_pages, generator=mgen) < w.needle_fraction
    if w.context_range is not None:
        lo, hi = w.context_range
        lens_all = torch.randint(lo, hi + 1, (B,), generator=mgen)
        seq_lens = lens_all[b0:b1].tolist()
    else:
        seq_lens = [S] * nb
    pages = torch.nonzero(needle).reshape(-1)
    if pages.numel():
        qh = q[:, ::G, 0, :].to(torch.float32)                       # first head of each group
        shift = (0.5 * math.sqrt(D)) * qh / qh.norm(dim=-1, keepdim=True)
        rows = (pages[:, None] * P + torch.arange(P)[None, :]).reshape(-1).to(dev)
        kk = k[:, :, rows, :].to(torch.float32) + shift[:, :, None, :]
        k[:, :, rows, :] = kk.to(w.dtype)
    return dict(k=k, v=v, q=q, k_new=k_new, v_new=v_new, seq_lens=seq_lens, needle_pages=pages)


def algorithmic_bytes(w: Workload, seq_lens, selected_tokens_total: int) -> dict:
    """Bytes one decode step must move (the roofline numerator).

    metadata: two statistics arrays (min+max for top-k, mean+std for Gaussian) of every
    scored page, once per KV head; kv: K and V rows of every selected token, per
    query head (no sharing inside a GQA group is assumed, which is what the kernels do).
    """
    e = torch.empty((), dtype=w.dtype).element_size()
    P, D = w.page_size, w.head_dim
    meta = 0
    for s in seq_lens:
        n_pages = (s + 1 + P - 1) // P
        meta += 2 * w.kv_heads * max(n_pages - 1, 0) * D * e
    kv = 2 * D * e * selected_tokens_total
    return {"metadata": meta, "kv": kv, "total": meta + kv}
