"""CUDA path vs outputs of the reference's own Triton path recorded on a B200
(tests/golden/ref_triton.npz; tests/golden/make_golden_triton.py made it).

The fixture stores only seeds and shapes of the inputs, so both sides see the same
tensors.  Bars: page scores of 16-bit inputs bit-identical to the reference, page sets
identical (boundary ties aside), token counts identical, Gaussian statistics within 5e-5;
tau and outputs within what the reference's 16-bit dot products cost it
(adadecode_paged.py:97-98) - 1e-5 / 2e-5 for fp32 inputs, where it has no such rounding.
"""

import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import topk as otopk
from tests import _harness as H
from tests.test_oracle_triton_golden import (near_boundary_f16, ulp_distance_f16, DT, GAUSS_ALIBI_CASES, GAUSS_CASES, OUT_ATOL, TAU_ATOL, TAU_RTOL,
                                             TOPK_ALIBI_CASES, TOPK_CASES, alibi_slopes_for)


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_triton.npz"))


def _cache(E, ci, P):
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    c.append(ci["k_new"], ci["v_new"])
    return c


@pytest.mark.parametrize("name", list(TOPK_CASES) + list(TOPK_ALIBI_CASES))
def test_topk_step_against_triton_reference(golden, name):
    import entmaxkv_b200 as E
    g = golden
    B, Hh, D, S, P, dt, alpha, needles, seed, budget = {**TOPK_CASES, **TOPK_ALIBI_CASES}[name]
    slopes = alibi_slopes_for(name, Hh)
    slopes = None if slopes is None else slopes.cuda()
    inp = H.cpu_inputs(B, Hh, Hh, D, S, DT[dt], seed=seed, needle_pages=needles, page_size=P)
    ci = H.to_cuda(inp)
    c = _cache(E, ci, P)
    T = int(g[name + "_T"])
    seqlens = torch.full((B,), T, dtype=torch.int32, device="cuda")
    qlens = torch.full((B,), S + 1, dtype=torch.int32, device="cuda")
    out = torch.zeros_like(ci["q"])
    taus = torch.zeros(B, Hh, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_paged(q=ci["q"], kv_cache=c, k_new=ci["k_new"], v_new=ci["v_new"], out=out,
                                    token_budget=budget, cache_seqlens=seqlens, q_seqlens=qlens, alpha=alpha,
                                    niter=2, append_cache=False, taus_out=taus, alibi_slopes=slopes)
    torch.cuda.synchronize()
    want_scores = g[name + "_scores"]
    scores = c.last_topk_selection["scores"][:, :, :want_scores.shape[-1]].float().cpu()
    if dt == "fp32":
        np.testing.assert_allclose(scores.numpy(), want_scores, rtol=1e-5, atol=4e-5)
    else:
        assert np.array_equal(scores.numpy(), want_scores), "16-bit page scores must be bit-identical"
    want_pages = g[name + "_pages"]
    k = want_pages.shape[-1] - 1
    got = c.last_topk_selection["page_indices"][:, :, :k + 1].cpu().numpy()
    tied = otopk.boundary_tied_pages(scores, k).numpy()
    for b in range(B):
        for h in range(Hh):
            diff = set(want_pages[b, h, :k].tolist()) ^ set(got[b, h, :k].tolist())
            assert all(tied[b, h, p] for p in diff), (b, h, diff)
    assert (got[:, :, k] == want_pages[:, :, k]).all()
    assert c.last_topk_selection["tok_counts"].cpu().tolist() == [[T] * Hh] * B
    np.testing.assert_allclose(taus.cpu().numpy(), g[name + "_tau"], rtol=TAU_RTOL[dt], atol=TAU_ATOL[dt])
    assert np.abs(out.float().cpu().numpy() - g[name + "_out"]).max() <= OUT_ATOL[dt]


@pytest.mark.parametrize("name", list(GAUSS_CASES) + list(GAUSS_ALIBI_CASES))
def test_gaussian_step_against_triton_reference(golden, name):
    import entmaxkv_b200 as E
    g = golden
    B, Hh, D, S, P, dt, alpha, needles, seed, mode = {**GAUSS_CASES, **GAUSS_ALIBI_CASES}[name]
    slopes = alibi_slopes_for(name, Hh)
    ali = {} if slopes is None else dict(alibi_slopes=slopes.cuda())
    inp = H.cpu_inputs(B, Hh, Hh, D, S, DT[dt], seed=seed, needle_pages=needles, page_size=P)
    ci = H.to_cuda(inp)
    c = _cache(E, ci, P)
    out = torch.zeros_like(ci["q"])
    taus = torch.zeros(B, Hh, dtype=torch.float32, device="cuda")
    if mode != "exact":
        # "fixed" leaves the clamped estimate untouched: that is the reference's tau_clamped
        E.sparse_attention_decode_gaussian_aware_entmax(ci["q"], c, ci["k_new"], ci["v_new"], out, alpha=alpha,
                                                        append_cache=False, tau_mode="fixed", taus_out=taus, **ali)
        np.testing.assert_allclose(taus.cpu().numpy(), g[name + "_tau_clamped"], rtol=5e-5, atol=2e-5)
    E.sparse_attention_decode_gaussian_aware_entmax(ci["q"], c, ci["k_new"], ci["v_new"], out, alpha=alpha,
                                                    append_cache=False, tau_mode=mode, niter=2, taus_out=taus, **ali)
    torch.cuda.synchronize()
    sel = c.last_gaussian_selection
    n = g[name + "_mu"].shape[-1]
    np.testing.assert_allclose(sel["mu"][:, :, :n].cpu().numpy(), g[name + "_mu"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(sel["sigma"][:, :, :n].cpu().numpy(), g[name + "_sigma"], rtol=1e-4, atol=1e-5)
    hs = sel["head_stats"].cpu().numpy()
    np.testing.assert_allclose(hs[..., 1], g[name + "_sigma_global"].reshape(B, Hh), rtol=1e-4)
    np.testing.assert_allclose(hs[..., 2], g[name + "_tau_hat"], rtol=5e-5, atol=1e-6)
    np.testing.assert_allclose(sel["tau_floor"].cpu().numpy(), g[name + "_tau_floor"], rtol=5e-5, atol=2e-5)
    counts = sel["num_selected"].cpu().numpy()
    pages = sel["page_indices"].cpu().numpy()
    assert np.array_equal(counts, g[name + "_counts"])
    for b in range(B):
        for h in range(Hh):
            assert np.array_equal(pages[b, h, :counts[b, h]], g[name + "_pages"][b, h, :counts[b, h]]), (b, h)
    assert np.array_equal(sel["tok_counts"].cpu().numpy(), g[name + "_seqlens"])
    np.testing.assert_allclose(taus.cpu().numpy(), g[name + "_tau_final"], rtol=TAU_RTOL[dt], atol=TAU_ATOL[dt])
    want = g[name + "_out"]
    scale = max(1.0, float(np.abs(want).max()))
    assert np.abs(out.float().cpu().numpy() - want).max() <= OUT_ATOL[dt] * scale


def test_topk_32k_full_size_against_triton_reference(topk_path):
    """Benchmark configuration 2 at its own size against the reference's Triton path on the same inputs
    (tests/golden/ref_triton_topk_32k.npz): the CUDA path through the public wrapper, general kernels and the
    one-launch kernel."""
    import os
    import entmaxkv_b200 as E
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_triton_topk_32k.npz"))
    w = CONFIGS[str(g["workload"])]
    inp = make_inputs(w, "cuda")
    c = E.PagedKVCache(page_size=w.page_size)
    c.initialize(inp["k"], inp["v"], capacity=w.context + 64)
    out = torch.zeros_like(inp["q"])
    taus = torch.zeros(w.batch, w.q_heads, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, w.token_budget, alpha=w.alpha,
                                    niter=2, taus_out=taus)
    torch.cuda.synchronize()
    sel = c.last_topk_selection
    assert bool(sel.get("fused", False)) == (topk_path == "fused")
    k = g["pages"].shape[-1] - 1
    n_scored = (w.context + 1 + w.page_size - 1) // w.page_size - 1
    scores = sel["scores"][:, :, :n_scored].cpu()
    # the reference's Triton reduction and the fixed summation order used here round a handful of the 65 536
    # sums differently: one unit in the last place at most, and page sets may differ only at such scores
    ulps = ulp_distance_f16(scores.numpy(), g["scores_f16"][:, :, :n_scored])
    assert ulps.max() <= 1 and (ulps > 0).sum() <= 4 * w.q_heads, (int(ulps.max()), int((ulps > 0).sum()))
    got = sel["page_indices"][:, :, :k + 1].cpu().numpy()
    for h in range(w.q_heads):
        diff = set(g["pages"][0, h, :k].tolist()) ^ set(got[0, h, :k].tolist())
        near = near_boundary_f16(scores.numpy()[0, h], k)
        assert all(near[p] for p in diff), (h, diff)
    assert (got[:, :, k] == g["pages"][:, :, k]).all()
    assert sel["tok_counts"].cpu().tolist() == [[int(g["T"])] * w.q_heads]
    np.testing.assert_allclose(taus.cpu().numpy(), g["tau"], rtol=TAU_RTOL["fp16"], atol=TAU_ATOL["fp16"])
    assert np.abs(out.float().cpu().numpy() - g["out"]).max() <= OUT_ATOL["fp16"]
