"""Seeded synthetic decode-step workloads (shapes and value distributions of the
benchmark configurations; no dataset is involved anywhere in this library).

Inputs are iid standard normal like the reference's own tests and benchmark script
(tests/test_topk.py:55-67, tests/run_benchmarks.py:56-66).  In a chosen fraction of
the full pages ("needle" pages, one Bernoulli mask shared by every batch row and
head) the keys are shifted by ``0.5*sqrt(D)*q_hat`` so that those pages dominate
the scores; for a GQA group ``q_hat`` is the unit query of the group's first head.

The draws are COUNTER BASED, so the same seed gives the same bits on every device:
element ``i`` of the (tensor, batch row, head) stream is the ``hash(stream key, i)``-th
entry of a table of 2**22 normal quantiles.  The hash is integer arithmetic (exact on
CPU and CUDA alike), the table is computed once on the host in fp64 and copied, and the
needle shift is computed on the host from the (small) query tensor and added with one
fp32 addition per element, so a tensor drawn on the GPU equals, bit for bit, the one
drawn on the CPU - and any (batch row, KV head) slice can be drawn alone, which is how
the CPU oracle is fed the benchmark's own inputs without staging 17 GB through the host.
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


_TABLE_BITS = 22
_M32 = 0xFFFFFFFF
_tables: dict = {}

# stream ids of the tensors of a workload
_T_K, _T_V, _T_Q, _T_KNEW, _T_VNEW, _T_POOL_K, _T_POOL_V = range(7)


def _normal_table(device) -> torch.Tensor:
    """2**22 standard-normal quantiles at the bucket midpoints, fp32 (largest |x| = 5.03)."""
    dev = torch.device(device)
    t = _tables.get("cpu")
    if t is None:
        n = 1 << _TABLE_BITS
        u = (torch.arange(n, dtype=torch.float64) + 0.5) / n
        t = torch.special.ndtri(u).to(torch.float32)
        _tables["cpu"] = t
    if dev.type == "cpu":
        return t
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    g = _tables.get(key)
    if g is None:
        g = t.to(dev)
        _tables[key] = g
    return g


def _mul32(x: torch.Tensor, c: int) -> torch.Tensor:
    """(x * c) mod 2**32 for int64 x in [0, 2**32) without leaving 63 bits."""
    lo, hi = c & 0xFFFF, c >> 16
    return (x * lo + (((x * hi) & 0xFFFF) << 16)) & _M32


def _mix32(x: torch.Tensor) -> torch.Tensor:
    """A 32-bit avalanche mix (xor-shift / odd multiply rounds) on int64 carriers."""
    x = x ^ (x >> 16)
    x = _mul32(x, 0x7FEB352D)
    x = x ^ (x >> 15)
    x = _mul32(x, 0x846CA68B)
    return x ^ (x >> 16)


def _mix32_int(x: int) -> int:
    x &= _M32
    x ^= x >> 16
    x = (x * 0x7FEB352D) & _M32
    x ^= x >> 15
    x = (x * 0x846CA68B) & _M32
    return x ^ (x >> 16)


def stream_key(seed: int, tensor_id: int, b: int, h: int) -> int:
    """32-bit key of the (tensor, batch row, head) stream of ``seed``."""
    k = _mix32_int(seed * 0x9E3779B1 + 0x85EBCA6B)
    k = _mix32_int(k ^ (tensor_id * 0xC2B2AE35 + 1))
    k = _mix32_int(k ^ (b * 0x27D4EB2F + 2))
    return _mix32_int(k ^ (h * 0x165667B1 + 3))


def normal_stream(key: int, n: int, device, dtype, start: int = 0) -> torch.Tensor:
    """Elements ``start .. start+n-1`` of stream ``key`` as a 1-D tensor of ``dtype`` on ``device``."""
    dev = torch.device(device)
    table = _normal_table(dev)
    out = torch.empty(n, dtype=dtype, device=dev)
    step = 1 << 24
    for i0 in range(0, n, step):
        i1 = min(n, i0 + step)
        idx = torch.arange(start + i0, start + i1, dtype=torch.int64, device=dev)
        x = _mix32((idx & _M32) ^ key)
        x = _mix32(x + (idx >> 32) * 0x9E3779B1 & _M32)
        out[i0:i1] = table[x >> (32 - _TABLE_BITS)].to(dtype)
    return out


def normal_tensor(seed: int, tensor_id: int, b_range, h_range, tail_shape, device, dtype,
                  first_row: int = 0) -> torch.Tensor:
    """[len(b_range), len(h_range), *tail_shape]: one stream per GLOBAL (batch row, head) pair.
    ``first_row``: the tensor holds rows first_row, first_row+1, ... of the stream's [rows, D] matrix."""
    n = 1
    for s in tail_shape:
        n *= s
    out = torch.empty((len(b_range), len(h_range)) + tuple(tail_shape), dtype=dtype, device=device)
    start = first_row * tail_shape[-1]
    for i, b in enumerate(b_range):
        for j, h in enumerate(h_range):
            out[i, j] = normal_stream(stream_key(seed, tensor_id, b, h), n, device, dtype, start).view(tail_shape)
    return out


def workload_lengths(w: Workload):
    """(needle page ids, per-row context lengths) of ``w``: functions of the seed only."""
    mgen = torch.Generator(device="cpu")
    mgen.manual_seed(w.seed * 7919 + 17)
    needle = torch.rand(w.context // w.page_size, generator=mgen) < w.needle_fraction
    if w.context_range is not None:
        lo, hi = w.context_range
        lens = torch.randint(lo, hi + 1, (w.batch,), generator=mgen).tolist()
    else:
        lens = [w.context] * w.batch
    return torch.nonzero(needle).reshape(-1), lens


def make_inputs(w: Workload, device="cpu", batch_slice: Optional[slice] = None,
                kv_head_slice: Optional[slice] = None, token_slice: Optional[slice] = None):
    """Draw the tensors of ``w`` (or of one batch x KV-head x token-range slice of it) on ``device``.

    Returns dict(k, v, q, k_new, v_new, seq_lens, needle_pages).  The bits depend on the
    seed and on each element's GLOBAL coordinates only: not on the device, and a slice
    equals the same rows, heads and tokens of the full draw.  ``token_slice`` (whole pages)
    restricts k and v to the context tokens [start, stop): one rank's share of a
    sequence-sharded request; seq_lens and needle_pages stay global.
    """
    B, Hq, Hkv, D, S, P = w.batch, w.q_heads, w.kv_heads, w.head_dim, w.context, w.page_size
    G = Hq // Hkv
    b0, b1 = (0, B) if batch_slice is None else (batch_slice.start, batch_slice.stop)
    h0, h1 = (0, Hkv) if kv_head_slice is None else (kv_head_slice.start, kv_head_slice.stop)
    rb, rh = range(b0, b1), range(h0, h1)
    rq = range(h0 * G, h1 * G)
    dev = torch.device(device)
    t0, t1 = (0, S) if token_slice is None else (token_slice.start, token_slice.stop)
    if t0 % P:
        raise ValueError("token_slice must start on a page boundary")
    k = normal_tensor(w.seed, _T_K, rb, rh, (t1 - t0, D), dev, w.dtype, first_row=t0)
    v = normal_tensor(w.seed, _T_V, rb, rh, (t1 - t0, D), dev, w.dtype, first_row=t0)
    # the small tensors are drawn on the host (the needle shift is host arithmetic) and copied
    q_host = normal_tensor(w.seed, _T_Q, rb, rq, (1, D), "cpu", w.dtype)
    k_new = normal_tensor(w.seed, _T_KNEW, rb, rh, (1, D), "cpu", w.dtype).to(dev)
    v_new = normal_tensor(w.seed, _T_VNEW, rb, rh, (1, D), "cpu", w.dtype).to(dev)
    pages, lens_all = workload_lengths(w)
    seq_lens = lens_all[b0:b1]
    if pages.numel():
        qh = q_host[:, ::G, 0, :].to(torch.float32)                  # first head of each group
        shift = ((0.5 * math.sqrt(D)) * qh / qh.norm(dim=-1, keepdim=True)).to(dev)
        mine = pages[(pages * P >= t0) & (pages * P + P <= t1)]
        rows = (mine[:, None] * P - t0 + torch.arange(P)[None, :]).reshape(-1).to(dev)
        kk = k[:, :, rows, :].to(torch.float32) + shift[:, :, None, :]
        k[:, :, rows, :] = kk.to(w.dtype)
    return dict(k=k, v=v, q=q_host.to(dev), k_new=k_new, v_new=v_new, seq_lens=seq_lens, needle_pages=pages)


def token_pool(w: Workload, n: int, device, batch_slice: Optional[slice] = None,
               kv_head_slice: Optional[slice] = None):
    """``n`` further (k_new, v_new) pairs, [n, B, H_kv, 1, D] each: the tokens a decode loop
    appends after the first one, from streams of their own (same device independence)."""
    b0, b1 = (0, w.batch) if batch_slice is None else (batch_slice.start, batch_slice.stop)
    h0, h1 = (0, w.kv_heads) if kv_head_slice is None else (kv_head_slice.start, kv_head_slice.stop)
    D = w.head_dim
    kp = normal_tensor(w.seed, _T_POOL_K, range(b0, b1), range(h0, h1), (n, 1, D), "cpu", w.dtype)
    vp = normal_tensor(w.seed, _T_POOL_V, range(b0, b1), range(h0, h1), (n, 1, D), "cpu", w.dtype)
    return kp.permute(2, 0, 1, 3, 4).contiguous().to(device), vp.permute(2, 0, 1, 3, 4).contiguous().to(device)


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
