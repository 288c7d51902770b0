"""The CPU oracle against outputs of the reference's own CPU code (tests/golden/ref_cpu.npz)."""

import numpy as np
import pytest
import torch

from oracle import cache as ocache, topk as otopk, gaussian as og

DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def _ulp_close(a, b, dt, ulps=1):
    """|a-b| <= ulps units in the last place of dtype dt (inputs fp32 views of dt values)."""
    a = torch.from_numpy(np.asarray(a)).to(torch.float32)
    b = torch.from_numpy(np.asarray(b)).to(torch.float32)
    if dt == torch.float32:
        return torch.allclose(a, b, rtol=2e-6, atol=1e-7)
    eps = torch.finfo(dt).eps
    tiny = torch.finfo(dt).smallest_normal * eps          # subnormal step
    spacing = torch.maximum(torch.abs(b) * eps, torch.tensor(tiny))
    return bool(((a - b).abs() <= ulps * spacing * 1.0001).all())


@pytest.mark.parametrize("name", ["fp32", "fp16", "bf16"])
def test_cache_stats_match_reference(golden_cpu, name):
    g, dt = golden_cpu, DT[name]
    k = torch.from_numpy(g[f"cache_{name}_k"]).to(dt)
    v = torch.from_numpy(g[f"cache_{name}_v"]).to(dt)
    kn = torch.from_numpy(g[f"cache_{name}_kn"]).to(dt)
    vn = torch.from_numpy(g[f"cache_{name}_vn"]).to(dt)
    c = ocache.OracleCache(page_size=16)
    c.initialize(k, v)
    for nm in ("k_min", "k_max"):
        assert np.array_equal(getattr(c, nm).float().numpy(), g[f"cache_{name}_init_{nm}"])
    for nm in ("k_mean", "k_std"):
        assert _ulp_close(getattr(c, nm).float().numpy(), g[f"cache_{name}_init_{nm}"], dt)
    for i in range(kn.shape[0]):
        c.append(kn[i], vn[i])
    assert np.array_equal(c.k_cache.float().numpy(), g[f"cache_{name}_final_k_cache"])
    assert np.array_equal(c.v_cache.float().numpy(), g[f"cache_{name}_final_v_cache"])
    for nm in ("k_min", "k_max"):
        assert np.array_equal(getattr(c, nm).float().numpy(), g[f"cache_{name}_final_{nm}"])
    for nm in ("k_mean", "k_std"):
        assert _ulp_close(getattr(c, nm).float().numpy(), g[f"cache_{name}_final_{nm}"], dt)


def test_criticality_matches_reference_fp32(golden_cpu):
    g = golden_cpu
    k, q = torch.from_numpy(g["crit_k"]), torch.from_numpy(g["crit_q"])
    mn, mx, _, _ = ocache.page_stats(k, 16)
    s = otopk.criticality_scores(q, mn, mx)
    assert s.shape == g["crit_scores"].shape
    np.testing.assert_allclose(s.numpy(), g["crit_scores"], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("alpha", [1.5, 2.0])
def test_gaussian_statistics_with_alibi_match_reference(golden_cpu, alpha):
    """Reference: compute_gaussian_aware_statistics(..., alibi_slopes=...) on the CPU - biased page
    means, unbiased global moments, page-mixture tau_hat."""
    g = golden_cpu
    k, q = torch.from_numpy(g["gauss_k"]), torch.from_numpy(g["gauss_q"])
    _, _, mean, std = ocache.page_stats(k, 16)
    r = og.gaussian_selection(q, mean, std, k.shape[2], 16, alpha,
                              alibi_slopes=torch.from_numpy(g["alibi_slopes"]))
    tag = f"gauss_alibi_a{alpha}"
    np.testing.assert_allclose(r["mu"].numpy(), g[f"{tag}_mu_scores_per_page"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(r["sigma"].numpy(), g[f"{tag}_sigma_scores_per_page"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(r["mu_global"].numpy().reshape(-1), g[f"{tag}_mu_global"].reshape(-1),
                               rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(r["sigma_global"].numpy().reshape(-1), g[f"{tag}_sigma_global"].reshape(-1),
                               rtol=1e-5)
    np.testing.assert_allclose(r["tau_hat"].numpy().reshape(-1), g[f"{tag}_tau_hat"].reshape(-1), rtol=1e-4,
                               atol=1e-5)
    assert r["safety_margin_z"] == pytest.approx(float(g[f"{tag}_margin"]), rel=1e-5)


def test_criticality_with_alibi_matches_reference_fp32(golden_cpu):
    """Reference: PagedKVCache.estimate_page_criticality(use_triton=False, alibi_slopes=...)."""
    g = golden_cpu
    k, q = torch.from_numpy(g["crit_k"]), torch.from_numpy(g["crit_q"])
    mn, mx, _, _ = ocache.page_stats(k, 16)
    S = k.shape[2]
    s = otopk.criticality_scores(q, mn, mx, alibi_slopes=torch.from_numpy(g["alibi_slopes"]), seq_len=S,
                                 page_size=16, q_pos=S - 1)
    np.testing.assert_allclose(s.numpy(), g["crit_alibi_scores"], rtol=2e-5, atol=2e-5)
    assert np.abs(g["crit_alibi_scores"] - g["crit_scores"]).max() > 1.0     # the bonus is not a no-op


@pytest.mark.parametrize("alpha", [1.5, 2.0])
def test_gaussian_statistics_and_tau_match_reference(golden_cpu, alpha):
    g = golden_cpu
    k, q = torch.from_numpy(g["gauss_k"]), torch.from_numpy(g["gauss_q"])
    _, _, mean, std = ocache.page_stats(k, 16)
    r = og.gaussian_selection(q, mean, std, seq_len=k.shape[2], page_size=16, alpha=alpha)
    tag = f"gauss_a{alpha}"
    np.testing.assert_allclose(r["mu"].numpy(), g[f"{tag}_mu_scores_per_page"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(r["sigma"].numpy(), g[f"{tag}_sigma_scores_per_page"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(r["mu_global"].numpy(), g[f"{tag}_mu_global"][..., 0], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(r["sigma_global"].numpy(), g[f"{tag}_sigma_global"][..., 0], rtol=1e-5)
    np.testing.assert_allclose(r["tau_hat"].numpy(), g[f"{tag}_tau_hat"], rtol=1e-5, atol=1e-6)
    assert r["n_tokens"] == int(g[f"{tag}_n"])
    assert r["max_quantile"] == float(g[f"{tag}_maxq"])
    assert r["safety_margin_z"] == pytest.approx(float(g[f"{tag}_margin"]), rel=1e-6)


@pytest.mark.parametrize("alpha", [1.5, 2.0])
def test_tau_clamp_matches_reference_cpu_branch(golden_cpu, alpha):
    g = golden_cpu
    tag = f"gauss_a{alpha}"
    mu = torch.from_numpy(g[f"{tag}_mu_scores_per_page"])
    sigma = torch.from_numpy(g[f"{tag}_sigma_scores_per_page"])
    tau_hat = torch.from_numpy(g[f"{tag}_tau_hat"])
    ids = torch.from_numpy(g[f"{tag}_clamp_ids"])
    counts = g[f"{tag}_clamp_counts"]
    pages = [[ids[b, h, :counts[b, h]] for h in range(ids.shape[1])] for b in range(ids.shape[0])]
    out = og.clamp_tau(tau_hat + 0.3, mu, sigma, pages, tau_hat - 0.05, page_size=16, alpha=alpha)
    np.testing.assert_allclose(out.numpy(), g[f"{tag}_clamp_out"], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("alpha", [1.5, 2.0, 1.7, 4 / 3])
@pytest.mark.parametrize("n", [64, 1008, 32768, 1048576])
def test_tau_solver_matches_reference(golden_cpu, alpha, n):
    """Closed forms (alpha 2 and 1.5: Halley; alpha 4/3: bisection on the third-moment form) and the
    bisection on the reference's moment approximation (alpha 1.7)."""
    g = golden_cpu
    mu, sg = torch.from_numpy(g["tau_mu"])[..., 0], torch.from_numpy(g["tau_sigma"])[..., 0]
    got = og.tau_hat(mu, sg, n, alpha).numpy()
    want = g[f"tau_a{alpha}_n{n}"][..., 0]
    # the reference stops a whole batch when its worst element reaches |f| < 1e-6, this oracle stops
    # element by element: both sit within that tolerance of the root
    np.testing.assert_allclose(got, want, rtol=1e-6 if alpha != 4 / 3 else 2e-5, atol=1e-6)


@pytest.mark.parametrize("alpha", [1.5, 2.0, 4 / 3])
def test_page_mixture_tau_matches_reference(golden_cpu, alpha):
    g = golden_cpu
    got = og.tau_hat_page_mixture(torch.from_numpy(g["mix_mu"]), torch.from_numpy(g["mix_sigma"]),
                                  alpha=alpha, uniform_page_count=16.0).numpy()
    np.testing.assert_allclose(got, g[f"mix_a{alpha}"], rtol=2e-4, atol=2e-5)


def test_config1_topk_and_tau(golden_cpu):
    """B=1,H=32,D=128,kv_len=1024,P=16, seed 0: page sets at budget 256 and tau_hat."""
    g = golden_cpu
    torch.manual_seed(0)
    k = torch.randn(1, 32, 1024, 128)
    v = torch.randn(1, 32, 1024, 128)
    q = torch.randn(1, 32, 1, 128)
    chk = np.array([k.double().sum().item(), v.double().sum().item(), q.double().sum().item()])
    np.testing.assert_allclose(chk, g["cfg1_checksum"], rtol=0, atol=1e-9)
    mn, mx, mean, std = ocache.page_stats(k, 16)
    s = otopk.criticality_scores(q, mn, mx)
    ids = otopk.topk_page_sets(s, 256 // 16)
    assert np.array_equal(ids.numpy(), g["cfg1_topk"])
    r = og.gaussian_selection(q, mean, std, seq_len=1024, page_size=16, alpha=1.5)
    np.testing.assert_allclose(r["tau_hat"].numpy(), g["cfg1_tau_hat"], rtol=1e-5)
    np.testing.assert_allclose(r["sigma_global"].numpy(), g["cfg1_sigma_global"][..., 0], rtol=1e-5)
