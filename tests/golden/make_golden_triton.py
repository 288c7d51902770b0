"""Generate ``ref_triton.npz``: outputs of the reference's Triton path on a GPU.

The reference's page selection (threshold pack) and both paged decodes exist only as Triton
kernels, so they can be pinned only on a GPU.  Run on a CUDA machine with an UNMODIFIED copy
of the reference importable (installed with
``pip install --no-deps --target baseline/_ref <reference checkout>``):

    PYTHONPATH=baseline/_ref python tests/golden/make_golden_triton.py [output.npz]

Inputs are the seeded tensors of ``tests/_harness.cpu_inputs`` (only seeds and shapes are
stored); every stored array comes from the reference's own functions.
"""

import math
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from entmaxkv.kv_cache import PagedKVCache                                            # noqa: E402
from entmaxkv.attention_topk import sparse_attention_decode_paged                     # noqa: E402
from entmaxkv.attention_gaussian import sparse_attention_decode_gaussian_aware_entmax  # noqa: E402
from entmaxkv.gaussian_utils import (compute_gaussian_aware_statistics,               # noqa: E402
                                     clamp_tau_to_selected_page_statistics)
from entmaxkv.kernels.adadecode_paged import sparse_attention_decode_paged as paged_kernel  # noqa: E402
from entmaxkv.kernels.adadecode_paged_gaussian_tau import (                             # noqa: E402
    sparse_attention_decode_paged_gaussian_tau as gaussian_tau_kernel)
from entmaxkv.kernels.selection_pack import cache_seqlens_from_page_counts_triton      # noqa: E402
from tests._harness import cpu_inputs                                                  # noqa: E402

OUT = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_triton.npz")
DT = {"fp16": torch.float16, "fp32": torch.float32, "bf16": torch.bfloat16}

# name: (B, H, D, S before append, P, dtype, alpha, needle pages, seed)
TOPK_CASES = {
    "topk_fp16_a15": (2, 4, 64, 1024, 16, "fp16", 1.5, (3, 40), 301, 256),
    "topk_fp32_a20": (1, 4, 64, 777, 16, "fp32", 2.0, (9,), 302, 160),
    "topk_bf16_a15": (1, 8, 128, 2047, 16, "bf16", 1.5, (7,), 303, 512),
}
# the same with ALiBi slopes 2^(-8 i / H) (tests/run_benchmarks.py:76-78)
TOPK_ALIBI_CASES = {
    "topk_fp16_a15_alibi": (2, 4, 64, 1500, 16, "fp16", 1.5, (3, 60), 321, 256),
    "topk_fp32_a15_alibi": (1, 4, 64, 777, 16, "fp32", 1.5, (9,), 322, 160),
}
GAUSS_ALIBI_CASES = {
    "gauss_fp16_corrected_alibi": (2, 4, 64, 2048, 16, "fp16", 1.5, (3, 90), 331, "corrected"),
    "gauss_fp32_corrected_alibi": (1, 4, 64, 1500, 16, "fp32", 1.5, (5,), 332, "corrected"),
    "gauss_fp32_exact_alibi": (1, 4, 64, 1500, 16, "fp32", 1.5, (5,), 333, "exact"),
}
GAUSS_CASES = {
    "gauss_fp16_corrected": (2, 4, 64, 2048, 16, "fp16", 1.5, (3, 40), 311, "corrected"),
    "gauss_fp32_corrected": (1, 4, 64, 1500, 16, "fp32", 1.5, (5,), 312, "corrected"),
    "gauss_fp32_exact": (1, 4, 64, 1500, 16, "fp32", 1.5, (5,), 313, "exact"),
    "gauss_fp16_a20_fixed": (1, 4, 128, 3000, 16, "fp16", 2.0, (5, 99), 314, "fixed"),
}


def f32(t):
    return t.detach().float().cpu().clone().numpy()


def cuda_inputs(B, H, D, S, P, dtype, needles, seed):
    inp = cpu_inputs(B, H, H, D, S, DT[dtype], seed=seed, needle_pages=needles, page_size=P)
    return {k: v.cuda() for k, v in inp.items()}


def fresh_cache(inp, P):
    c = PagedKVCache(page_size=P)
    c.initialize(inp["k"], inp["v"])
    c.append(inp["k_new"], inp["v_new"])
    return c


def main():
    assert torch.cuda.is_available()
    g = {}
    for name, (B, H, D, S, P, dtype, alpha, needles, seed, budget) in {**TOPK_CASES, **TOPK_ALIBI_CASES}.items():
        inp = cuda_inputs(B, H, D, S, P, dtype, needles, seed)
        slopes = (torch.exp2(-8.0 * torch.arange(1, H + 1, device="cuda") / H).float()
                  if name in TOPK_ALIBI_CASES else None)
        c = fresh_cache(inp, P)
        S1 = S + 1
        total_pages = (S1 + P - 1) // P
        k_sel = min(budget // P, total_pages - 1)
        T = k_sel * P + (S1 - (total_pages - 1) * P)
        seqlens = torch.full((B,), T, device="cuda", dtype=torch.int32)
        qlens = torch.full((B,), S1, device="cuda", dtype=torch.int32)
        out = torch.zeros_like(inp["q"])
        sparse_attention_decode_paged(q=inp["q"], kv_cache=c, k_new=inp["k_new"], v_new=inp["v_new"], out=out,
                                      token_budget=budget, cache_seqlens=seqlens, q_seqlens=qlens, alpha=alpha,
                                      niter=2, append_cache=False, alibi_slopes=slopes)
        scores = c.estimate_page_criticality(inp["q"], use_triton=True, q_pos=S1 - 1, exclude_last_page=True,
                                             alibi_slopes=slopes)
        pages = c._page_indices_buf.clone()
        taus = torch.zeros(B, H, device="cuda", dtype=torch.float32)
        out2 = torch.zeros_like(out)
        paged_kernel(q=inp["q"], k_cache=c.k_cache, v_cache=c.v_cache, out=out2,
                     cache_seqlens=seqlens[:, None].expand(B, H), page_indices=pages, page_size=P, alpha=alpha,
                     niter=2, q_seqlens=qlens, taus_out=taus, alibi_slopes=slopes)
        torch.cuda.synchronize()
        g[f"{name}_scores"] = f32(scores)
        g[f"{name}_pages"] = pages.cpu().numpy()
        g[f"{name}_out"] = f32(out)
        g[f"{name}_tau"] = f32(taus)
        g[f"{name}_T"] = np.int64(T)

    for name, (B, H, D, S, P, dtype, alpha, needles, seed, mode) in {**GAUSS_CASES, **GAUSS_ALIBI_CASES}.items():
        inp = cuda_inputs(B, H, D, S, P, dtype, needles, seed)
        c = fresh_cache(inp, P)
        out = torch.zeros_like(inp["q"])
        slopes = (torch.exp2(-8.0 * torch.arange(1, H + 1, device="cuda") / H).float()
                  if name in GAUSS_ALIBI_CASES else None)
        qlens = torch.full((B,), S + 1, device="cuda", dtype=torch.int32)
        corr_iters = 0 if mode == "fixed" else (2 if slopes is not None else 1)
        # Twice: the reference's atomic-add output kernel is autotuned, and the tuner's trial
        # launches of the first call all accumulate into `out`; only later calls are meaningful.
        for _ in range(2):
            sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, inp["k_new"], inp["v_new"], out, alpha=alpha,
                                                          append_cache=False, tau_mode=mode, niter=2,
                                                          alibi_slopes=slopes, q_seqlens=qlens)
        # the same steps by hand, to capture the intermediates the wrapper keeps to itself
        S1 = S + 1
        st = compute_gaussian_aware_statistics(q=inp["q"], k_mean=c.k_mean, k_std=c.k_std, seq_len=S1,
                                               page_size=P, alpha=alpha, threshold_excess_margin_fraction=0.2,
                                               tau_clamp_page_max_quantile=0.5, alibi_slopes=slopes)
        raw, counts = c.select_gaussian_aware(inp["q"], alpha=alpha, gaussian_stats=st)
        pages = raw.to(torch.int32)
        tau = st["tau_hat"]
        if mode != "exact":
            tau = clamp_tau_to_selected_page_statistics(tau, st, pages, counts, P, alpha)
        last = S1 - (math.ceil(S1 / P) - 1) * P if S1 > P else S1
        seqlens = cache_seqlens_from_page_counts_triton(counts, P, last)
        out2 = torch.zeros_like(out)
        tau_final = torch.zeros(B, H, device="cuda", dtype=torch.float32)
        if mode == "exact":
            paged_kernel(q=inp["q"], k_cache=c.k_cache, v_cache=c.v_cache, out=out2, cache_seqlens=seqlens,
                         page_indices=pages, page_size=P, alpha=alpha, niter=2, taus_out=tau_final,
                         alibi_slopes=slopes, q_seqlens=qlens)
        else:
            for _ in range(2):
                tau_work = tau.clone().contiguous()
                gaussian_tau_kernel(q=inp["q"], k_cache=c.k_cache, v_cache=c.v_cache, out=out2,
                                    cache_seqlens=seqlens, page_indices=pages, page_size=P, tau=tau_work,
                                    alpha=alpha, tau_correction_iters=corr_iters, alibi_slopes=slopes,
                                    q_seqlens=qlens)
            tau_final = tau_work
        torch.cuda.synchronize()
        g[f"{name}_mu"] = f32(st["mu_scores_per_page"])
        g[f"{name}_sigma"] = f32(st["sigma_scores_per_page"])
        g[f"{name}_sigma_global"] = f32(st["sigma_global"])
        g[f"{name}_tau_hat"] = f32(st["tau_hat"])
        g[f"{name}_tau_floor"] = f32(st["tau_floor"])
        g[f"{name}_margin"] = np.float64(st["safety_margin_z"])
        g[f"{name}_maxq"] = np.float64(st["max_quantile"])
        g[f"{name}_counts"] = counts.cpu().numpy()
        pg = pages.cpu().numpy().copy()
        cn = counts.cpu().numpy()
        for b in range(B):                      # slots beyond the count are uninitialised memory
            for h in range(H):
                pg[b, h, cn[b, h]:] = -1
        g[f"{name}_pages"] = pg
        g[f"{name}_seqlens"] = seqlens.cpu().numpy()
        g[f"{name}_tau_clamped"] = f32(tau)
        g[f"{name}_tau_final"] = f32(tau_final)
        g[f"{name}_out"] = f32(out)
        g[f"{name}_out_by_hand"] = f32(out2)

    import triton
    g["versions"] = np.array([torch.__version__, triton.__version__, torch.cuda.get_device_name(0)])
    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
