"""The CPU oracle against outputs of the reference's Triton path recorded on a B200
(tests/golden/ref_triton.npz, made by tests/golden/make_golden_triton.py).

This pins the parts of the oracle the reference implements only in Triton: page scores in
the query dtype, the top-k page sets, the Gaussian threshold selection with packing and
token counts, the tau clamp, and both paged decodes.  Bars: everything that is exact in
the reference is compared exactly; quantities the reference computes with 16-bit dot
products (adadecode_paged.py:97-98,124) are compared with the tolerance that rounding
implies - the fp32 cases of the same code paths are tight.
"""

import numpy as np
import pytest
import torch

from oracle import topk as otopk
from tests import _harness as H

DT = {"fp16": torch.float16, "fp32": torch.float32, "bf16": torch.bfloat16}
TOPK_CASES = {
    "topk_fp16_a15": (2, 4, 64, 1024, 16, "fp16", 1.5, (3, 40), 301, 256),
    "topk_fp32_a20": (1, 4, 64, 777, 16, "fp32", 2.0, (9,), 302, 160),
    "topk_bf16_a15": (1, 8, 128, 2047, 16, "bf16", 1.5, (7,), 303, 512),
}
GAUSS_CASES = {
    "gauss_fp16_corrected": (2, 4, 64, 2048, 16, "fp16", 1.5, (3, 40), 311, "corrected"),
    "gauss_fp32_corrected": (1, 4, 64, 1500, 16, "fp32", 1.5, (5,), 312, "corrected"),
    "gauss_fp32_exact": (1, 4, 64, 1500, 16, "fp32", 1.5, (5,), 313, "exact"),
    "gauss_fp16_a20_fixed": (1, 4, 128, 3000, 16, "fp16", 2.0, (5, 99), 314, "fixed"),
}
# the same paths with ALiBi slopes 2^(-8 i / H)
TOPK_ALIBI_CASES = {
    "topk_fp16_a15_alibi": (2, 4, 64, 1500, 16, "fp16", 1.5, (3, 60), 321, 256),
    "topk_fp32_a15_alibi": (1, 4, 64, 777, 16, "fp32", 1.5, (9,), 322, 160),
}
GAUSS_ALIBI_CASES = {
    "gauss_fp16_corrected_alibi": (2, 4, 64, 2048, 16, "fp16", 1.5, (3, 90), 331, "corrected"),
    "gauss_fp32_corrected_alibi": (1, 4, 64, 1500, 16, "fp32", 1.5, (5,), 332, "corrected"),
    "gauss_fp32_exact_alibi": (1, 4, 64, 1500, 16, "fp32", 1.5, (5,), 333, "exact"),
}
TAU_ATOL = {"fp32": 1e-6, "fp16": 1e-3, "bf16": 1e-2}     # ALiBi can put tau near zero


def alibi_slopes_for(name, heads):
    return torch.exp2(-8.0 * torch.arange(1, heads + 1) / heads).float() if name.endswith("_alibi") else None


# what the reference's 16-bit q.k products cost it, relative to fp32 accumulation
TAU_RTOL = {"fp32": 1e-5, "fp16": 1e-3, "bf16": 1e-2}
# fp32: a tau within 1e-5 relative moves sum (z - tau)^2 v by a few 1e-5 of its magnitude
OUT_ATOL = {"fp32": 1e-4, "fp16": 2e-2, "bf16": 1e-1}


@pytest.fixture(scope="module")
def golden():
    import os
    return np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_triton.npz"))


@pytest.mark.parametrize("name", list(TOPK_CASES) + list(TOPK_ALIBI_CASES))
def test_topk_step_against_triton_reference(golden, name):
    g = golden
    B, Hh, D, S, P, dt, alpha, needles, seed, budget = {**TOPK_CASES, **TOPK_ALIBI_CASES}[name]
    inp = H.cpu_inputs(B, Hh, Hh, D, S, DT[dt], seed=seed, needle_pages=needles, page_size=P)
    ref = H.oracle_topk_step(inp, P, budget, alpha, 2, alibi_slopes=alibi_slopes_for(name, Hh))
    scores = ref["scores"].float().numpy()
    if dt == "fp32":
        np.testing.assert_allclose(scores, g[name + "_scores"], rtol=1e-5, atol=4e-5)
    else:
        assert np.array_equal(scores, g[name + "_scores"]), "16-bit page scores must be bit-identical"
    want = np.sort(g[name + "_pages"][:, :, :-1], axis=-1)       # torch.topk order is by score
    got = ref["pages"][:, :, :-1].numpy()
    tied = otopk.boundary_tied_pages(ref["scores"], got.shape[-1]).numpy()
    for b in range(B):
        for h in range(Hh):
            diff = set(want[b, h]) ^ set(got[b, h])
            assert all(tied[b, h, p] for p in diff), (b, h, diff)   # only boundary ties may differ
    assert (g[name + "_pages"][:, :, -1] == ref["pages"][:, :, -1].numpy()).all()
    assert int(g[name + "_T"]) == ref["T"]
    np.testing.assert_allclose(g[name + "_tau"], ref["tau"], rtol=TAU_RTOL[dt], atol=TAU_ATOL[dt])
    assert np.abs(g[name + "_out"][:, :, 0] - ref["out"]).max() <= OUT_ATOL[dt]


@pytest.mark.parametrize("name", list(GAUSS_CASES) + list(GAUSS_ALIBI_CASES))
def test_gaussian_step_against_triton_reference(golden, name):
    g = golden
    B, Hh, D, S, P, dt, alpha, needles, seed, mode = {**GAUSS_CASES, **GAUSS_ALIBI_CASES}[name]
    inp = H.cpu_inputs(B, Hh, Hh, D, S, DT[dt], seed=seed, needle_pages=needles, page_size=P)
    slopes = alibi_slopes_for(name, Hh)
    iters = {"corrected": 1 if slopes is None else 2, "fixed": 0}.get(mode, 1)
    ref = H.oracle_gaussian_step(inp, P, alpha, tau_mode="exact" if mode == "exact" else "corrected",
                                 iters=iters, niter=2, alibi_slopes=slopes)
    n = ref["mu"].shape[-1]
    np.testing.assert_allclose(g[name + "_mu"], ref["mu"].numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(g[name + "_sigma"], ref["sigma"].numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(g[name + "_tau_hat"], ref["tau_hat"].numpy(), rtol=5e-5, atol=1e-6)
    np.testing.assert_allclose(g[name + "_tau_floor"], ref["tau_floor"].numpy(), rtol=5e-5, atol=2e-5)
    assert float(g[name + "_maxq"]) == ref["max_quantile"]
    assert float(g[name + "_margin"]) == pytest.approx(ref["safety_margin_z"], rel=1e-5)
    counts, pages = g[name + "_counts"], g[name + "_pages"]
    for b in range(B):
        for h in range(Hh):
            got = pages[b, h, :counts[b, h]].tolist()
            want = [int(x) for x in ref["pages"][b][h]]
            diff = set(got) ^ set(want)
            assert all(p < n and abs(float(ref["margin"][b, h, p])) < 1e-5 for p in diff), (b, h, diff)
            if not diff:
                assert got == want                    # ascending, last page in the final slot
    if not any(set(pages[b, h, :counts[b, h]].tolist()) ^ set(int(x) for x in ref["pages"][b][h])
               for b in range(B) for h in range(Hh)):
        assert np.array_equal(counts, ref["counts"].numpy())
        assert np.array_equal(g[name + "_seqlens"], ref["cache_seqlens"].numpy())
    if mode != "exact":
        np.testing.assert_allclose(g[name + "_tau_clamped"], ref["tau_clamped"].numpy(), rtol=5e-5, atol=2e-5)
    np.testing.assert_allclose(g[name + "_tau_final"], ref["tau"], rtol=TAU_RTOL[dt], atol=TAU_ATOL[dt])
    scale = max(1.0, float(np.abs(ref["out"]).max()))
    assert np.abs(g[name + "_out"][:, :, 0] - ref["out"]).max() <= OUT_ATOL[dt] * scale
    # the reference's corrected decode accumulates with 16-bit atomics in arrival order
    assert np.abs(g[name + "_out"] - g[name + "_out_by_hand"]).max() <= OUT_ATOL[dt] * scale


def _keys_f16(x):
    """Order-preserving integers of fp16 values (adjacent representable values differ by one)."""
    u = np.ascontiguousarray(x, dtype=np.float16).view(np.uint16).astype(np.int32)
    return np.where(u & 0x8000, -(u & 0x7fff), u & 0x7fff)


def ulp_distance_f16(a, b):
    return np.abs(_keys_f16(a) - _keys_f16(b))


def near_boundary_f16(scores_row, k):
    """Pages whose fp16 score is within one unit in the last place of the k-th largest score."""
    keys = _keys_f16(scores_row)
    kth = np.sort(keys)[::-1][k - 1]
    return np.abs(keys - kth) <= 1


def test_topk_32k_full_size_against_triton_reference():
    """Benchmark configuration 2 at its own size (B=1, 32 heads, 32 769 tokens, fp16, budget 2048) against the
    reference's Triton path (tests/golden/ref_triton_topk_32k.npz, made by make_golden_triton_full.py on the
    benchmark's own inputs): the oracle, one head at a time."""
    import os
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    path = os.path.join(os.path.dirname(__file__), "golden", "ref_triton_topk_32k.npz")
    g = np.load(path)
    w = CONFIGS[str(g["workload"])]
    inp = make_inputs(w, "cpu")
    P, Hh = w.page_size, w.q_heads
    k_sel = g["pages"].shape[-1] - 1
    tied_most = off_by_one = 0
    for h in range(Hh):
        s = {n: inp[n][:, h:h + 1] for n in ("k", "v", "q", "k_new", "v_new")}
        ref = H.oracle_topk_step(s, P, w.token_budget, w.alpha, 2)
        n_scored = ref["scores"].shape[-1]
        ulps = ulp_distance_f16(ref["scores"].numpy(), g["scores_f16"][:, h:h + 1, :n_scored])
        assert ulps.max() <= 1, "16-bit page scores: at most one unit in the last place"
        off_by_one += int((ulps > 0).sum())
        want = set(g["pages"][0, h, :k_sel].tolist())
        got = set(ref["pages"][0, 0, :k_sel].tolist())
        near = near_boundary_f16(ref["scores"].numpy()[0, 0], k_sel)
        assert all(near[p] for p in want ^ got), (h, sorted(want ^ got))
        tied = otopk.boundary_tied_pages(ref["scores"], k_sel).numpy()[0, 0]
        tied_most = max(tied_most, int(tied.sum()))
        assert g["pages"][0, h, k_sel] == int(ref["pages"][0, 0, k_sel])
        assert int(g["T"]) == ref["T"]
        np.testing.assert_allclose(g["tau"][:, h:h + 1], ref["tau"], rtol=TAU_RTOL["fp16"], atol=TAU_ATOL["fp16"])
        assert np.abs(g["out"][:, h:h + 1, 0] - ref["out"]).max() <= OUT_ATOL["fp16"]
    # the reference's Triton reduction and the fixed order used here round a handful of sums differently
    assert off_by_one <= Hh * 4, off_by_one
    print("topk_32k: largest boundary-tied class", tied_most, "scores one ulp apart:", off_by_one, "of", Hh * n_scored)
