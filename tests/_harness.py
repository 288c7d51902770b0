"""Shared helpers of the GPU parity tests: run one decode step through the public
API (CUDA path) and through the CPU oracle on identical inputs."""

from __future__ import annotations

import numpy as np
import torch

from oracle import cache as ocache, topk as otopk, gaussian as og, decode as od, dense as odense


def cpu_inputs(B, Hq, Hkv, D, S, dtype, seed, needle_pages=(), page_size=16):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, S, D, generator=g).to(dtype)
    q = torch.randn(B, Hq, 1, D, generator=g).to(dtype)
    k_new = torch.randn(B, Hkv, 1, D, generator=g).to(dtype)
    v_new = torch.randn(B, Hkv, 1, D, generator=g).to(dtype)
    G = Hq // Hkv
    for p in needle_pages:
        qh = q[:, ::G, 0, :].float()
        shift = 0.5 * (D ** 0.5) * qh / qh.norm(dim=-1, keepdim=True)
        rows = slice(p * page_size, (p + 1) * page_size)
        k[:, :, rows] = (k[:, :, rows].float() + shift[:, :, None, :]).to(dtype)
    return dict(k=k, v=v, q=q, k_new=k_new, v_new=v_new)


def to_cuda(d):
    return {n: (t.cuda() if torch.is_tensor(t) else t) for n, t in d.items()}


def oracle_cache_after_append(inp, P, seq_len=None):
    """Oracle cache state for one (uniform-length) batch after the step's append."""
    c = ocache.OracleCache(P)
    k, v = inp["k"], inp["v"]
    if seq_len is not None:
        k, v = k[:, :, :seq_len], v[:, :, :seq_len]
    c.initialize(k, v)
    c.append(inp["k_new"], inp["v_new"])
    return c


def oracle_topk_step(inp, P, token_budget, alpha, niter, seq_len=None, alibi_slopes=None, cache=None):
    """``cache``: an oracle cache already holding ``inp`` after the append (large cases build it once)."""
    c = oracle_cache_after_append(inp, P, seq_len) if cache is None else cache
    S = c.seq_len
    scores = otopk.criticality_scores(inp["q"], c.k_min, c.k_max, alibi_slopes=alibi_slopes, seq_len=S,
                                      page_size=P)
    pages, T = otopk.topk_select_and_pack(scores, token_budget, P, S)
    B, Hq = inp["q"].shape[:2]
    tables = [[pages[b, h].tolist() for h in range(Hq)] for b in range(B)]
    ntok = [[T] * Hq for _ in range(B)]
    ali = dict(alibi_slopes=alibi_slopes, q_pos=[S - 1] * B) if alibi_slopes is not None else {}
    out, taus, supp = od.decode(inp["q"], c.k_cache, c.v_cache, tables, ntok, P, alpha,
                                mode="exact", niter=niter, **ali)
    out_true, taus_true, _ = od.decode(inp["q"], c.k_cache, c.v_cache, tables, ntok, P, alpha, mode="true",
                                       **ali)
    return dict(cache=c, scores=scores, pages=pages, T=T, out=out, tau=taus, support=supp,
                out_true=out_true, tau_true=taus_true)


def oracle_gaussian_step(inp, P, alpha, tau_mode="corrected", iters=1, niter=2, seq_len=None,
                         sigma_mean=None, pages_override=None, tau0_override=None, alibi_slopes=None,
                         cache=None):
    c = oracle_cache_after_append(inp, P, seq_len) if cache is None else cache
    S = c.seq_len
    sel = og.gaussian_selection(inp["q"], c.k_mean, c.k_std, S, P, alpha,
                                sigma_mean_override=sigma_mean, alibi_slopes=alibi_slopes)
    B, Hq = inp["q"].shape[:2]
    pages = sel["pages"] if pages_override is None else pages_override
    tables = [[list(map(int, pages[b][h])) for h in range(Hq)] for b in range(B)]
    # a single-page sequence whose page fails the threshold: the reference leaves the
    # table slot uninitialised (selection_pack.py:190-198); the library attends page 0
    tables = [[t if t else [0] for t in row] for row in tables]
    last = og.last_page_size(S, P)
    ntok = [[max(len(tables[b][h]) - 1, 0) * P + last for h in range(Hq)] for b in range(B)]
    tau0 = sel["tau_clamped"].numpy() if tau0_override is None else tau0_override
    ali = dict(alibi_slopes=alibi_slopes, q_pos=[S - 1] * B) if alibi_slopes is not None else {}
    if tau_mode == "exact":
        out, taus, supp = od.decode(inp["q"], c.k_cache, c.v_cache, tables, ntok, P, alpha,
                                    mode="exact", niter=niter, **ali)
    else:
        out, taus, supp = od.decode(inp["q"], c.k_cache, c.v_cache, tables, ntok, P, alpha,
                                    mode="corrected", tau0=tau0, iters=iters, **ali)
    sel.update(cache=c, out=out, tau=taus, support=supp, ntok=ntok, tables=tables)
    return sel


def ulp_close(a, b, dt, ulps=1):
    a, b = a.float(), b.float()
    if dt == torch.float32:
        return torch.allclose(a, b, rtol=2e-6, atol=1e-7)
    eps = torch.finfo(dt).eps
    tiny = torch.finfo(dt).smallest_normal * eps
    spacing = torch.maximum(b.abs() * eps, torch.tensor(tiny))
    return bool(((a - b).abs() <= ulps * spacing * 1.0001).all())
