"""Generate ``ref_cpu.npz``: outputs of the reference's CPU-runnable code.

Run where the reference checkout is importable (it is NOT needed to run the
test-suite, only to regenerate the fixture):

    PYTHONPATH=<reference checkout> python tests/golden/make_golden_cpu.py

Every array is produced by the reference's own functions on seeded inputs;
nothing from this repository's oracle or kernels is involved.  16-bit tensors
are stored widened to fp32 (exact).
"""

import math
import os
import sys

import numpy as np
import torch

from entmaxkv.kv_cache import PagedKVCache
from entmaxkv.gaussian_utils import (
    compute_gaussian_aware_statistics,
    clamp_tau_to_selected_page_statistics,
)
from entmaxkv.tau_solver import solve_for_tau_hat_single_gaussian
from entmaxkv.kernels.tau_solver_page_mixture import solve_for_tau_hat_page_gaussian_mixture

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cpu.npz")
DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def f32(t):
    return t.detach().to(torch.float32).clone().numpy()


def main():
    g = {}

    # A. cache statistics: initialize + appends crossing a page boundary
    for name, dt in DT.items():
        torch.manual_seed(11)
        B, H, S0, D, P, n_app = 2, 3, 37, 64, 16, 14
        k = torch.randn(B, H, S0, D).to(dt)
        v = torch.randn(B, H, S0, D).to(dt)
        kn = torch.randn(n_app, B, H, 1, D).to(dt)
        vn = torch.randn(n_app, B, H, 1, D).to(dt)
        c = PagedKVCache(page_size=P)
        c.initialize(k, v)
        for nm in ("k_min", "k_max", "k_mean", "k_std"):
            g[f"cache_{name}_init_{nm}"] = f32(getattr(c, nm))
        for i in range(n_app):
            c.append(kn[i], vn[i])
        for nm in ("k_min", "k_max", "k_mean", "k_std", "k_cache", "v_cache"):
            g[f"cache_{name}_final_{nm}"] = f32(getattr(c, nm))
        g[f"cache_{name}_k"] = f32(k)
        g[f"cache_{name}_v"] = f32(v)
        g[f"cache_{name}_kn"] = f32(kn)
        g[f"cache_{name}_vn"] = f32(vn)

    # B. torch criticality (fp32) with the last page excluded
    torch.manual_seed(12)
    B, H, S, D, P = 2, 4, 150, 64, 16
    k = torch.randn(B, H, S, D)
    v = torch.randn(B, H, S, D)
    q = torch.randn(B, H, 1, D)
    c = PagedKVCache(page_size=P)
    c.initialize(k, v)
    g["crit_k"], g["crit_q"] = f32(k), f32(q)
    g["crit_scores"] = f32(c.estimate_page_criticality(q, use_triton=False, exclude_last_page=True))

    # B2. the same with ALiBi: page bonus slope * (last position of the page - q_pos)
    slopes = torch.exp2(-8.0 * torch.arange(1, H + 1) / H).float()
    g["alibi_slopes"] = f32(slopes)
    g["crit_alibi_scores"] = f32(c.estimate_page_criticality(q, use_triton=False, alibi_slopes=slopes,
                                                             q_pos=S - 1, exclude_last_page=True))
    # C2. Gaussian statistics with ALiBi: biased page means and the page-mixture tau_hat
    for alpha in (1.5, 2.0):
        st = compute_gaussian_aware_statistics(q=q, k_mean=c.k_mean, k_std=c.k_std, seq_len=S,
                                               page_size=P, alpha=alpha, alibi_slopes=slopes)
        tag = f"gauss_alibi_a{alpha}"
        for nm in ("mu_scores_per_page", "sigma_scores_per_page", "mu_global", "sigma_global",
                   "tau_hat"):
            g[f"{tag}_{nm}"] = f32(st[nm])
        g[f"{tag}_margin"] = np.float64(st["safety_margin_z"])
        g[f"{tag}_maxq"] = np.float64(st["max_quantile"])

    # C. Gaussian statistics + tau_hat through the torch fallback, alpha 1.5 and 2
    g["gauss_k"], g["gauss_q"] = g["crit_k"], g["crit_q"]
    for alpha in (1.5, 2.0):
        st = compute_gaussian_aware_statistics(q=q, k_mean=c.k_mean, k_std=c.k_std, seq_len=S,
                                               page_size=P, alpha=alpha)
        tag = f"gauss_a{alpha}"
        for nm in ("mu_scores_per_page", "sigma_scores_per_page", "mu_global", "sigma_global",
                   "tau_hat"):
            g[f"{tag}_{nm}"] = f32(st[nm])
        g[f"{tag}_margin"] = np.float64(st["safety_margin_z"])
        g[f"{tag}_maxq"] = np.float64(st["max_quantile"])
        g[f"{tag}_n"] = np.int64(st["seq_len_for_stats"])

        # E. CPU branch of the tau clamp on a hand-made page table
        torch.manual_seed(13)
        n_stats = st["pages_for_stats"]
        ids = torch.stack([torch.stack([torch.randperm(n_stats + 1)[:5].sort().values
                                        for _ in range(H)]) for _ in range(B)]).to(torch.int32)
        counts = torch.randint(0, 6, (B, H), dtype=torch.int32)
        st2 = dict(st)
        st2["tau_floor"] = st["tau_hat"] - 0.05
        out = clamp_tau_to_selected_page_statistics(st["tau_hat"] + 0.3, st2, ids, counts, P, alpha)
        g[f"{tag}_clamp_ids"] = ids.numpy()
        g[f"{tag}_clamp_counts"] = counts.numpy()
        g[f"{tag}_clamp_out"] = f32(out)

    # D. scalar tau solver on a grid (closed-form alphas and the bisection fallback)
    mus = torch.tensor([-0.8, -0.1, 0.0, 0.3, 1.2]).view(-1, 1, 1)
    sgs = torch.tensor([0.05, 0.4, 1.0, 2.5]).view(1, -1, 1)
    mu_g = mus.expand(5, 4, 1).contiguous()
    sg_g = sgs.expand(5, 4, 1).contiguous()
    g["tau_mu"], g["tau_sigma"] = f32(mu_g), f32(sg_g)
    for alpha in (1.5, 2.0, 1.7, 4 / 3):      # 4/3: closed-form third moment, bisected (tau_solver.py:73-78,276-344)
        for n in (64, 1008, 32768, 1048576):
            g[f"tau_a{alpha}_n{n}"] = f32(solve_for_tau_hat_single_gaussian(mu_g, sg_g, n, alpha))

    # F. page-mixture solver
    torch.manual_seed(14)
    mu_p = torch.randn(2, 3, 40) * 0.7
    sg_p = torch.rand(2, 3, 40) * 0.8 + 0.05
    g["mix_mu"], g["mix_sigma"] = f32(mu_p), f32(sg_p)
    for alpha in (1.5, 2.0, 4 / 3):
        cnt = torch.full(mu_p.shape, 16.0)
        g[f"mix_a{alpha}"] = f32(solve_for_tau_hat_page_gaussian_mixture(
            mu_p, sg_p, page_counts=cnt, alpha=alpha))

    # G. the CPU-runnable benchmark case: B=1,H=32,D=128,kv_len=1024,P=16, seed 0
    torch.manual_seed(0)
    B, H, S, D, P = 1, 32, 1024, 128, 16
    k = torch.randn(B, H, S, D)
    v = torch.randn(B, H, S, D)
    q = torch.randn(B, H, 1, D)
    c = PagedKVCache(page_size=P)
    c.initialize(k, v)
    sc = c.estimate_page_criticality(q, use_triton=False, exclude_last_page=True)
    top = torch.topk(sc, min(256 // P, sc.shape[-1]), dim=2).indices.sort(-1).values
    st = compute_gaussian_aware_statistics(q=q, k_mean=c.k_mean, k_std=c.k_std, seq_len=S,
                                           page_size=P, alpha=1.5)
    g["cfg1_topk"] = top.numpy().astype(np.int32)
    g["cfg1_tau_hat"] = f32(st["tau_hat"])
    g["cfg1_sigma_global"] = f32(st["sigma_global"])
    g["cfg1_checksum"] = np.array([k.double().sum().item(), v.double().sum().item(),
                                   q.double().sum().item()])

    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes;", len(g), "arrays; torch", torch.__version__,
          "python", sys.version.split()[0], "sqrt2", math.sqrt(2))


if __name__ == "__main__":
    main()
