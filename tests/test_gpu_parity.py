"""CUDA path vs CPU oracle on identical seeded inputs (run on a B200: ``-m gpu``).

Bars: cache statistics, page scores (16-bit dtypes) and top-k page sets are bit-exact;
Gaussian moments within 1e-5, tau within 1e-4 relative, Gaussian page sets exact
outside the pages whose selection margin is below 1e-5; outputs within max-abs 2e-3
of the oracle's decode over the same pages.
"""

import ctypes

import numpy as np
import pytest
import torch

from entmaxkv_b200 import _lib

pytestmark = pytest.mark.gpu

from tests import _harness as H

DT = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
OUT_TOL = 2e-3
TAU_RTOL = 1e-4


def _api():
    import entmaxkv_b200 as E
    return E


def assert_out_close(got, ref, dt, scale=1.0):
    """max-abs <= 2e-3 (times the output magnitude when it exceeds 1), plus the half-ulp
    that storing the result in the 16-bit output dtype costs (bf16: 3.9e-3 * |out|)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    half_ulp = 0.0 if dt == torch.float32 else 0.5 * float(torch.finfo(dt).eps)
    tol = OUT_TOL * scale + half_ulp * np.abs(ref) * 1.01
    bad = np.abs(got - ref) > tol
    assert not bad.any(), f"max-abs {np.abs(got - ref).max():.3e}, worst excess {(np.abs(got - ref) - tol).max():.3e}"


# --------------------------------------------------------------------------- cache

@pytest.mark.parametrize("name", ["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("D", [64, 128])
def test_cache_statistics_bit_exact(name, D):
    E = _api()
    dt = DT[name]
    B, Hkv, S0, P, n_app = 2, 3, 37, 16, 30
    inp = H.cpu_inputs(B, Hkv, Hkv, D, S0, dt, seed=21)
    g = torch.Generator().manual_seed(22)
    kn = torch.randn(n_app, B, Hkv, 1, D, generator=g).to(dt)
    vn = torch.randn(n_app, B, Hkv, 1, D, generator=g).to(dt)
    oc = H.ocache.OracleCache(P)
    oc.initialize(inp["k"], inp["v"])
    c = E.PagedKVCache(page_size=P)
    c.initialize(inp["k"].cuda(), inp["v"].cuda())
    for nm in ("k_min", "k_max", "k_mean", "k_std"):
        assert torch.equal(getattr(c, nm).cpu(), getattr(oc, nm)), nm
    for i in range(n_app):
        oc.append(kn[i], vn[i])
        c.append(kn[i].cuda(), vn[i].cuda())
    assert c.seq_len == S0 + n_app and c.seq_lens.tolist() == [S0 + n_app] * B
    assert torch.equal(c.k_cache.cpu(), oc.k_cache) and torch.equal(c.v_cache.cpu(), oc.v_cache)
    for nm in ("k_min", "k_max", "k_mean", "k_std"):
        assert getattr(c, nm).shape == getattr(oc, nm).shape
        assert torch.equal(getattr(c, nm).cpu(), getattr(oc, nm)), nm
    assert c.device_status() == 0


@pytest.mark.parametrize("name", ["fp32", "fp16", "bf16"])
def test_cache_statistics_against_reference_fixture(golden_cpu, name):
    """Same inputs as the fixture generated from the reference's own cache code."""
    E = _api()
    g, dt = golden_cpu, DT[name]
    k = torch.from_numpy(g[f"cache_{name}_k"]).to(dt).cuda()
    v = torch.from_numpy(g[f"cache_{name}_v"]).to(dt).cuda()
    kn = torch.from_numpy(g[f"cache_{name}_kn"]).to(dt).cuda()
    vn = torch.from_numpy(g[f"cache_{name}_vn"]).to(dt).cuda()
    c = E.PagedKVCache(page_size=16)
    c.initialize(k, v)
    for i in range(kn.shape[0]):
        c.append(kn[i], vn[i])
    for nm in ("k_min", "k_max", "k_cache", "v_cache"):
        assert np.array_equal(getattr(c, nm).float().cpu().numpy(), g[f"cache_{name}_final_{nm}"]), nm
    for nm in ("k_mean", "k_std"):
        assert H.ulp_close(getattr(c, nm).cpu(), torch.from_numpy(g[f"cache_{name}_final_{nm}"]), dt), nm


def test_cache_grows_past_capacity_and_handles_ragged_batches():
    E = _api()
    P, D = 16, 64
    inp = H.cpu_inputs(3, 2, 2, D, 40, torch.float16, seed=23)
    lens = [40, 17, 32]
    c = E.PagedKVCache(page_size=P, capacity=48)
    c.initialize(inp["k"].cuda(), inp["v"].cuda(), seq_lens=lens)
    g = torch.Generator().manual_seed(24)
    toks = [(torch.randn(3, 2, 1, D, generator=g).half(), torch.randn(3, 2, 1, D, generator=g).half())
            for _ in range(20)]
    for kn, vn in toks:
        c.append(kn.cuda(), vn.cuda())
    assert c.capacity >= 60 and c.seq_lens.tolist() == [60, 37, 52]
    for b, n0 in enumerate(lens):
        oc = H.ocache.OracleCache(P)
        oc.initialize(inp["k"][b:b + 1, :, :n0], inp["v"][b:b + 1, :, :n0])
        for kn, vn in toks:
            oc.append(kn[b:b + 1], vn[b:b + 1])
        n, npg = n0 + 20, (n0 + 20 + P - 1) // P
        assert torch.equal(c._k[b:b + 1, :, :n].cpu(), oc.k_cache)
        for i, nm in enumerate(("k_min", "k_max", "k_mean", "k_std")):
            assert torch.equal(c._meta[i][b:b + 1, :, :npg].cpu(), getattr(oc, nm)), (b, nm)


# --------------------------------------------------------------------------- top-k

TOPK_CASES = [
    # B, Hq, Hkv, D, S(before append), P, budget, dtype, alpha, needles
    (2, 4, 4, 64, 1024, 16, 256, "fp16", 1.5, (3, 40)),
    (1, 8, 2, 128, 2047, 16, 512, "bf16", 1.5, (7,)),       # GQA 4, append fills the page
    (2, 4, 2, 128, 2048, 16, 512, "fp16", 2.0, (5, 99)),    # append starts a new page
    (1, 2, 2, 64, 300, 16, 100000, "fp16", 1.5, ()),        # budget covers every page
    (1, 2, 2, 64, 300, 16, 8, "bf16", 2.0, ()),             # budget below one page: last page only
    (5, 32, 8, 128, 1100, 16, 256, "bf16", 1.5, (7,)),      # more heads than SMs: 128-thread tau blocks
    (1, 2, 2, 64, 9, 16, 64, "fp16", 1.5, ()),              # single page
    (2, 16, 2, 64, 700, 16, 128, "fp16", 1.5, (11,)),       # GQA 8
    (1, 4, 4, 128, 520, 8, 64, "bf16", 1.5, (2,)),          # page size 8
    (1, 2, 2, 64, 777, 16, 160, "fp32", 1.5, (9,)),
    (1, 4, 4, 64, 600, 16, 96, "fp16", 1.75, (4,)),         # general alpha
]


@pytest.mark.parametrize("case", TOPK_CASES, ids=[f"case{i}" for i in range(len(TOPK_CASES))])
def test_topk_step_matches_oracle(case, topk_path):
    E = _api()
    B, Hq, Hkv, D, S, P, budget, name, alpha, needles = case
    dt = DT[name]
    niter = 3
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, dt, seed=31 + S, needle_pages=needles, page_size=P)
    ref = H.oracle_topk_step(inp, P, budget, alpha, niter)
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    out = torch.zeros_like(ci["q"])
    taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_paged(ci["q"], c, ci["k_new"], ci["v_new"], out, budget, None, None,
                                    alpha=alpha, niter=niter, append_cache=True, taus_out=taus)
    torch.cuda.synchronize()
    n_scored = ref["scores"].shape[-1]
    scores = c.last_topk_selection["scores"][:, :, :n_scored].cpu()
    pages = c.last_topk_selection["page_indices"][:, :, :ref["pages"].shape[-1]].cpu()
    if dt != torch.float32:
        assert torch.equal(scores, ref["scores"]), "page scores must be bit-exact"
        assert torch.equal(pages, ref["pages"]), "page sets must be bit-exact"
    else:
        assert torch.allclose(scores, ref["scores"], rtol=1e-5, atol=1e-5)
        assert torch.equal(pages, ref["pages"])
    assert c.last_num_selected_per_head.cpu().tolist() == [[ref["pages"].shape[-1]] * Hq] * B
    assert c.last_topk_selection["tok_counts"].cpu().tolist() == [[ref["T"]] * Hq] * B
    if alpha in (1.5, 2.0):
        np.testing.assert_allclose(taus.cpu().numpy(), ref["tau_true"], rtol=TAU_RTOL, atol=1e-6)
    np.testing.assert_allclose(taus.cpu().numpy(), ref["tau"], rtol=TAU_RTOL, atol=1e-6)
    got = out[:, :, 0].float().cpu().numpy()
    assert_out_close(got, ref["out"], dt)
    if alpha in (1.5, 2.0):
        assert_out_close(got, ref["out_true"], dt)


@pytest.mark.parametrize("name,Hq,Hkv,alpha", [("bf16", 8, 2, 1.5), ("fp16", 16, 2, 2.0), ("fp16", 32, 8, 1.5)])
def test_dense_entmax_with_gqa_takes_the_group_shared_route(name, Hq, Hkv, alpha, monkeypatch):
    """A budget that covers the cache at any length on a GQA cache: every head of a group reads the same rows, the
    step fetches them once per group (groups of four and eight) and must still be exact alpha-entmax attention
    over all tokens; the per-head route gives the same to rounding."""
    E = _api()
    monkeypatch.setenv("EKV_FUSED_SMALL", "0")
    dt = DT[name]
    B, D, S, P = 2, 128, 6000, 16
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, dt, seed=311 + Hq, needle_pages=(3, 200), page_size=P)
    ci = H.to_cuda(inp)
    outs = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("EKV_GROUPED", flag)
        c = E.PagedKVCache(page_size=P, capacity=S + 64)
        c.initialize(ci["k"], ci["v"])
        out = torch.zeros_like(ci["q"])
        E.sparse_attention_decode_paged(ci["q"], c, ci["k_new"], ci["v_new"], out, token_budget=S + 64,
                                        alpha=alpha, niter=3)
        torch.cuda.synchronize()
        assert (getattr(c, "last_group_tables", None) is not None) == (flag == "1") and c.device_status() == 0
        assert c.last_topk_selection["tok_counts"].cpu().tolist() == [[S + 1] * Hq] * B
        outs[flag] = out[:, :, 0].float().cpu().numpy()
    k_all = torch.cat([inp["k"], inp["k_new"]], dim=2)
    v_all = torch.cat([inp["v"], inp["v_new"]], dim=2)
    want = H.odense.dense_entmax_decode(inp["q"], k_all, v_all, alpha, compute_dtype=torch.float64)[:, :, 0].numpy()
    assert_out_close(outs["1"], want, dt)
    assert_out_close(outs["0"], want, dt)
    assert np.abs(outs["1"] - outs["0"]).max() <= 1e-4 + float(torch.finfo(dt).eps)


@pytest.mark.parametrize("name,Hq,Hkv,alpha", [("fp16", 4, 4, 1.5), ("bf16", 8, 2, 1.5), ("fp16", 4, 4, 2.0),
                                                 ("fp32", 2, 2, 1.5)])
def test_topk_step_with_alibi_matches_oracle(name, Hq, Hkv, alpha):
    """ALiBi: page bonus in the scores (bit-exact for 16-bit dtypes) and the positional term in the
    decode logits; slopes 2^(-8 i / H) as in the reference's benchmark script."""
    E = _api()
    dt = DT[name]
    B, D, S, P, budget, niter = 2, 64, 1500, 16, 256, 3
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, dt, seed=77, needle_pages=(3, 60), page_size=P)
    slopes = torch.exp2(-8.0 * torch.arange(1, Hq + 1) / Hq).float()
    ref = H.oracle_topk_step(inp, P, budget, alpha, niter, alibi_slopes=slopes)
    plain = H.oracle_topk_step(inp, P, budget, alpha, niter)
    assert not torch.equal(ref["pages"], plain["pages"]), "the case must make ALiBi change the selection"
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    out = torch.zeros_like(ci["q"])
    taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
    q_seqlens = torch.full((B,), S + 1, dtype=torch.int32, device="cuda")
    E.sparse_attention_decode_paged(ci["q"], c, ci["k_new"], ci["v_new"], out, budget, None, q_seqlens,
                                    alibi_slopes=slopes.cuda(), alpha=alpha, niter=niter, append_cache=True,
                                    taus_out=taus)
    torch.cuda.synchronize()
    n_scored = ref["scores"].shape[-1]
    scores = c.last_topk_selection["scores"][:, :, :n_scored].cpu()
    pages = c.last_topk_selection["page_indices"][:, :, :ref["pages"].shape[-1]].cpu()
    if dt != torch.float32:
        assert torch.equal(scores, ref["scores"]), "page scores must be bit-exact"
    else:
        assert torch.allclose(scores, ref["scores"], rtol=1e-5, atol=1e-4)
    assert torch.equal(pages, ref["pages"])
    np.testing.assert_allclose(taus.cpu().numpy(), ref["tau"], rtol=TAU_RTOL, atol=1e-6)
    np.testing.assert_allclose(taus.cpu().numpy(), ref["tau_true"], rtol=TAU_RTOL, atol=1e-6)
    assert_out_close(out[:, :, 0].float().cpu().numpy(), ref["out"], dt)
    # default query position (no q_seqlens) is the appended token: same result
    out2 = torch.zeros_like(out)
    E.sparse_attention_decode_paged(ci["q"], c, ci["k_new"], ci["v_new"], out2, budget,
                                    alibi_slopes=slopes.cuda(), alpha=alpha, niter=niter, append_cache=False)
    assert torch.equal(out, out2)
    # the scoring helper of the cache
    sc = c.estimate_page_criticality(ci["q"], alibi_slopes=slopes.cuda(), q_pos=S, exclude_last_page=True)
    assert torch.equal(sc.cpu(), scores) or dt == torch.float32


@pytest.mark.parametrize("name,Hq,Hkv,D,S,alpha", [("fp16", 8, 2, 128, 3000, 1.5), ("bf16", 4, 4, 64, 1023, 2.0),
                                                   ("fp32", 2, 2, 64, 700, 1.5), ("fp16", 4, 4, 128, 2048, 2.0)])
def test_dense_entmax_attention_matches_dense_oracle(name, Hq, Hkv, D, S, alpha, topk_path):
    """A token budget that covers the whole cache makes the step dense entmax attention: every page goes
    through the same kernels and the output must be the reference tests' yardstick - exact alpha-entmax
    attention over ALL tokens (tests/benchmark_utils.py:56-83) - restated on the CPU.  (alpha 2 and 1.5: for
    other alphas the reference's histogram bracket is not guaranteed to hold the root, adadecode.py:74-112.)"""
    E = _api()
    dt = DT[name]
    B, P = 2, 16
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, dt, seed=300 + S, needle_pages=(3, 20), page_size=P)
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    out = torch.zeros_like(ci["q"])
    E.sparse_attention_decode_paged(ci["q"], c, ci["k_new"], ci["v_new"], out, token_budget=S + 4 * P,
                                    alpha=alpha, niter=3, append_cache=True)
    torch.cuda.synchronize()
    n_pages = (S + 1 + P - 1) // P
    assert c.last_num_selected_per_head.cpu().tolist() == [[n_pages] * Hq] * B        # every page
    assert c.last_topk_selection["tok_counts"].cpu().tolist() == [[S + 1] * Hq] * B   # every token
    k_all = torch.cat([inp["k"], inp["k_new"]], dim=2)
    v_all = torch.cat([inp["v"], inp["v_new"]], dim=2)
    want = H.odense.dense_entmax_decode(inp["q"], k_all, v_all, alpha, compute_dtype=torch.float64)
    assert_out_close(out[:, :, 0].float().cpu().numpy(), want[:, :, 0].numpy(), dt)


def test_topk_honours_user_cache_seqlens_and_append_false():
    E = _api()
    B, nh, D, S, P, budget = 2, 4, 64, 500, 16, 128
    inp = H.cpu_inputs(B, nh, nh, D, S, torch.float16, seed=41)
    ref = H.oracle_topk_step(inp, P, budget, 1.5, 2)
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    c.append(ci["k_new"], ci["v_new"])
    out = torch.zeros_like(ci["q"])
    seqlens = torch.full((B,), ref["T"], dtype=torch.int32, device="cuda")
    q_seqlens = torch.full((B,), S + 1, dtype=torch.int32, device="cuda")
    r = E.sparse_attention_decode_paged(q=ci["q"], kv_cache=c, k_new=ci["k_new"], v_new=ci["v_new"], out=out,
                                        token_budget=budget, cache_seqlens=seqlens, q_seqlens=q_seqlens,
                                        alpha=1.5, niter=2, append_cache=False)
    assert r is out and c.seq_len == S + 1
    assert_out_close(out[:, :, 0].float().cpu().numpy(), ref["out"], torch.float16)


def test_topk_ragged_batch_equals_per_sequence_runs():
    E = _api()
    B, nh, D, P, budget = 3, 4, 64, 16, 160
    lens = [400, 131, 257]
    inp = H.cpu_inputs(B, nh, nh, D, max(lens), torch.float16, seed=43)
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"], seq_lens=lens)
    out = torch.zeros_like(ci["q"])
    E.sparse_attention_decode_paged(ci["q"], c, ci["k_new"], ci["v_new"], out, budget, alpha=1.5, niter=2)
    for b, n in enumerate(lens):
        one = {k: v[b:b + 1] for k, v in inp.items()}
        ref = H.oracle_topk_step(one, P, budget, 1.5, 2, seq_len=n)
        assert_out_close(out[b:b + 1, :, 0].float().cpu().numpy(), ref["out"], torch.float16)


# --------------------------------------------------------------------------- Gaussian

GAUSS_CASES = [
    # B, Hq, Hkv, D, S, P, dtype, alpha, tau_mode, needles
    (2, 4, 4, 64, 2048, 16, "fp16", 1.5, "corrected", (3, 40)),
    (1, 8, 2, 128, 4095, 16, "bf16", 1.5, "corrected", (17,)),
    (2, 4, 4, 128, 3000, 16, "fp16", 2.0, "corrected", (5, 99)),
    (1, 4, 4, 64, 2048, 16, "fp16", 1.5, "fixed", (8,)),
    (1, 4, 4, 64, 2048, 16, "fp16", 1.5, "exact", (8,)),
    (1, 2, 2, 64, 9, 16, "fp16", 1.5, "corrected", ()),       # single page
    (1, 4, 2, 64, 1024, 16, "fp32", 1.5, "corrected", (6,)),
    (1, 16, 2, 128, 2048, 16, "bf16", 1.5, "corrected", (9,)),    # GQA 8: two lane groups per page
    (2, 8, 1, 64, 1024, 16, "fp16", 2.0, "corrected", (4,)),      # GQA 8, head_dim 64
    (1, 16, 1, 64, 777, 16, "fp32", 1.5, "corrected", (3,)),      # GQA 16, fp32
    (34, 32, 32, 64, 200, 16, "fp16", 1.5, "corrected", ()),      # 1088 heads: two tiles of the work-list prefix
    (2, 4, 4, 64, 2048, 16, "fp16", 4.0 / 3.0, "corrected", (3, 40)),   # alpha 4/3: closed-form third moment
    (1, 8, 2, 128, 3000, 16, "bf16", 4.0 / 3.0, "exact", (17,)),
    (2, 4, 4, 64, 2048, 16, "fp16", 1.75, "corrected", (3, 40)),        # general alpha: the reference's moment approximation
    (1, 8, 2, 128, 3000, 16, "bf16", 1.25, "fixed", (17,)),
    (5, 32, 32, 64, 9000, 16, "fp16", 1.5, "corrected", (3, 300)),      # more heads than SMs, rows too long for the
                                                                        # shared score copy: 256-thread tau blocks
]


@pytest.mark.parametrize("case", GAUSS_CASES, ids=[f"case{i}" for i in range(len(GAUSS_CASES))])
def test_gaussian_step_matches_oracle(case):
    E = _api()
    B, Hq, Hkv, D, S, P, name, alpha, tau_mode, needles = case
    dt = DT[name]
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, dt, seed=51 + S, needle_pages=needles, page_size=P)
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    out = torch.zeros_like(ci["q"])
    taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_gaussian_aware_entmax(ci["q"], c, ci["k_new"], ci["v_new"], out, alpha=alpha,
                                                    append_cache=True, tau_mode=tau_mode, niter=3,
                                                    taus_out=taus)
    torch.cuda.synchronize()
    sel = c.last_gaussian_selection
    ref = H.oracle_gaussian_step(inp, P, alpha, tau_mode="corrected", iters=0)
    n = ref["mu"].shape[-1]
    np.testing.assert_allclose(sel["mu"][:, :, :n].cpu().numpy(), ref["mu"].numpy(), rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(sel["sigma"][:, :, :n].cpu().numpy(), ref["sigma"].numpy(), rtol=1e-5, atol=2e-6)
    hs = sel["head_stats"].cpu().numpy()
    np.testing.assert_allclose(hs[..., 0], ref["mu_global"].numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(hs[..., 1], ref["sigma_global"].numpy(), rtol=1e-4)
    np.testing.assert_allclose(hs[..., 2], ref["tau_hat"].numpy(), rtol=TAU_RTOL, atol=1e-6)
    np.testing.assert_allclose(sel["tau_floor"].cpu().numpy(), ref["tau_floor"].numpy(), rtol=TAU_RTOL, atol=1e-6)
    # page sets: exact outside the boundary class |margin| < 1e-5
    counts = sel["num_selected"].cpu()
    pages = sel["page_indices"].cpu()
    margin = ref["margin"].numpy()
    got_tables = []
    for b in range(B):
        row = []
        for h in range(Hq):
            got = pages[b, h, :counts[b, h]].tolist()
            want = [int(x) for x in ref["pages"][b][h]]
            assert got == sorted(got), "page ids must be ascending with the last page at the end"
            diff = set(got) ^ set(want)
            assert all(p < n and abs(margin[b, h, p]) < 1e-5 for p in diff), (b, h, sorted(diff))
            row.append(got)
        got_tables.append(row)
    assert all(t[-1] == (S + 1 + P - 1) // P - 1 for row in got_tables for t in row)
    # decode over the kernel's own page sets and starting tau
    if tau_mode == "exact":
        ref2 = H.oracle_gaussian_step(inp, P, alpha, tau_mode="exact", niter=3, pages_override=got_tables)
    else:
        iters = 0 if tau_mode == "fixed" else 1
        # the clamp is part of the selection stage: check it, then start the oracle from it
        want_clamped = H.og.clamp_tau(ref["tau_hat"], ref["mu"], ref["sigma"],
                                      [[torch.tensor(t) for t in row] for row in got_tables],
                                      ref["tau_floor"], page_size=P, alpha=alpha).numpy()
        ref2 = H.oracle_gaussian_step(inp, P, alpha, tau_mode="corrected", iters=iters,
                                      pages_override=got_tables, tau0_override=want_clamped)
    # for 1/(alpha-1) < 2 the second-derivative sum of the correction step, sum (z-tau)^(beta-2), has a negative
    # exponent: tokens a hair above tau dominate it and fp32 noise in their scores moves the step
    tau_rtol = 1e-3 if (tau_mode == "corrected" and 1.0 / (alpha - 1.0) < 2.0) else TAU_RTOL
    np.testing.assert_allclose(taus.cpu().numpy(), ref2["tau"], rtol=tau_rtol, atol=1e-6)
    got = out[:, :, 0].float().cpu().numpy()
    scale = max(1.0, float(np.abs(ref2["out"]).max()))
    # unnormalised outputs can be O(10..100); the bar scales with that magnitude
    assert_out_close(got, ref2["out"], dt, scale=scale)


GROUP_CASES = [
    # B, Hq, Hkv, S or per-row lengths, P, dtype, alpha, tau_mode
    (2, 8, 2, 4095, 16, "bf16", 1.5, "corrected"),
    (1, 4, 1, 3000, 16, "fp16", 2.0, "corrected"),
    (2, 16, 4, 2048, 32, "fp16", 1.5, "exact"),
    (1, 8, 2, 9, 16, "fp16", 1.5, "corrected"),                  # single page
    (3, 8, 2, [5000, 777, 2049], 8, "bf16", 1.5, "fixed"),       # ragged batch, page size 8
    (1, 4, 1, 40000, 16, "bf16", 1.5, "corrected"),              # many chunks per group: runs cross blocks
    (2, 8, 2, [1500, 4000], 4, "fp16", 2.0, "corrected"),        # page size 4: 64 page slots per chunk
    (4, 32, 8, 300, 16, "fp16", 1.5, "exact"),                   # many short groups: two-chunk tables
    (10, 32, 8, 700, 16, "bf16", 1.5, "corrected"),              # 80 groups: one union block per group (fewer groups
                                                                 # than a quarter of the SMs take a cluster of eight each)
    (5, 64, 8, 1200, 16, "fp16", 1.5, "corrected"),              # the same for groups of eight
    # groups of eight (two heads per thread in the masking step, byte-wide membership masks)
    (2, 16, 2, 4095, 16, "bf16", 1.5, "corrected"),
    (1, 64, 8, 3000, 16, "bf16", 1.5, "corrected"),              # the million-token configuration's head layout
    (2, 8, 1, [9000, 1234], 16, "fp16", 2.0, "exact"),
    (1, 16, 2, 6000, 8, "fp16", 1.5, "fixed"),
    (1, 8, 1, 40000, 32, "bf16", 1.5, "corrected"),
    (2, 16, 2, [1500, 4000], 4, "fp16", 2.0, "corrected"),       # page size 4
    (1, 16, 2, 9, 16, "bf16", 1.5, "exact"),                     # single page
    (3, 8, 1, [70000, 33, 5000], 16, "bf16", 1.5, "corrected"),  # ragged: a cluster union over 4376 pages beside a 3-page row
]


@pytest.mark.parametrize("case", GROUP_CASES, ids=[f"case{i}" for i in range(len(GROUP_CASES))])
def test_group_shared_k_pass_equals_per_head_decode(case, monkeypatch):
    """GQA groups of four and eight, head_dim 128, 16-bit: the decode over one shared page table per group
    must reproduce the decode over the per-head tables (same selection, scores of the same rows),
    and the shared table must be the exact ascending union with the right membership bits."""
    E = _api()
    B, Hq, Hkv, S, P, name, alpha, tau_mode = case
    G = Hq // Hkv
    dt = DT[name]
    lens = S if isinstance(S, list) else [S] * B
    inp = H.cpu_inputs(B, Hq, Hkv, 128, max(lens), dt, seed=77 + max(lens), needle_pages=(2,), page_size=P)
    ci = H.to_cuda(inp)
    res = {}
    for flag in ("0", "1"):
        monkeypatch.setenv("EKV_GROUPED", flag)
        c = E.PagedKVCache(page_size=P)
        c.initialize(ci["k"], ci["v"], seq_lens=lens)
        out = torch.zeros_like(ci["q"])
        taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
        E.sparse_attention_decode_gaussian_aware_entmax(ci["q"], c, ci["k_new"], ci["v_new"], out, alpha=alpha,
                                                        append_cache=True, tau_mode=tau_mode, niter=3,
                                                        taus_out=taus)
        torch.cuda.synchronize()
        ws = next(v for k, v in c._scratch.items() if k[0] == "decode_ws")
        status = ctypes.c_int32(-1)
        _lib.check(_lib.load().ekv_read_status(ws.data_ptr(), ctypes.byref(status), _lib.stream_ptr()),
                   "ekv_read_status")
        assert status.value == 0 and c.device_status() == 0
        assert (getattr(c, "last_group_tables", None) is not None) == (flag == "1")
        res[flag] = (c, out.float().cpu().numpy(), taus.cpu().numpy())
    c0, out0, tau0 = res["0"]
    c1, out1, tau1 = res["1"]
    s0, s1 = c0.last_gaussian_selection, c1.last_gaussian_selection
    assert torch.equal(s0["num_selected"], s1["num_selected"])
    width = torch.arange(s0["page_indices"].shape[-1], device="cuda")
    valid = width[None, None, :] < s0["num_selected"][:, :, None]
    # the per-head tables stay what they were
    assert torch.equal(s0["page_indices"][valid], s1["page_indices"][valid])
    g = c1.last_group_tables
    counts, pages = s1["num_selected"].cpu().numpy(), s1["page_indices"].cpu().numpy()
    u_pages, member, u_tok = (g["union_pages"].cpu().numpy(), g["member"].cpu().numpy(),
                              g["union_tok_counts"].cpu().numpy())
    for b in range(B):
        n_tok = lens[b] + 1
        n_pages = (n_tok + P - 1) // P
        for hk in range(Hkv):
            sets = [set(pages[b, hk * G + j, :counts[b, hk * G + j]].tolist()) for j in range(G)]
            union = sorted(set().union(*sets))
            want_tok = len(union) * P - (P - (n_tok - (n_pages - 1) * P) if n_pages - 1 in union else 0)
            for j in range(G):
                assert u_pages[b, hk * G + j, :len(union)].tolist() == union
                assert u_tok[b, hk * G + j] == want_tok
            want_m = [sum(1 << j for j in range(G) if pg in sets[j]) for pg in union]
            assert member[b, hk, :len(union)].tolist() == want_m
    np.testing.assert_allclose(tau1, tau0, rtol=2e-5, atol=1e-6)
    scale = max(1.0, float(np.abs(out0).max()))
    np.testing.assert_allclose(out1, out0, rtol=0, atol=(2e-5 if tau_mode == "exact" else 1e-4) * scale
                               + float(torch.finfo(dt).eps) * scale)


@pytest.mark.parametrize("Hq,Hkv,name,alpha,tau_mode", [(16, 2, "bf16", 1.5, "corrected"), (64, 8, "fp16", 1.5, "corrected"),
                                                         (8, 1, "fp16", 2.0, "exact"), (8, 2, "bf16", 1.5, "corrected"),
                                                         (16, 4, "fp16", 1.5, "fixed")])
def test_group_shared_k_pass_matches_oracle(Hq, Hkv, name, alpha, tau_mode):
    """The grouped route (groups of eight and of four) against the oracle directly: tau and the output over
    the page sets the step selected, not only against the per-head route."""
    E = _api()
    dt = DT[name]
    B, S, P = 1, 5000, 16
    inp = H.cpu_inputs(B, Hq, Hkv, 128, S, dt, seed=900 + Hq, needle_pages=(3, 77), page_size=P)
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    out = torch.zeros_like(ci["q"])
    taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_gaussian_aware_entmax(ci["q"], c, ci["k_new"], ci["v_new"], out, alpha=alpha,
                                                    append_cache=True, tau_mode=tau_mode, niter=2, taus_out=taus)
    torch.cuda.synchronize()
    assert c.last_group_tables is not None and c.device_status() == 0
    sel = c.last_gaussian_selection
    counts = sel["num_selected"].cpu()
    tables = [[sel["page_indices"][b, h, :counts[b, h]].cpu().tolist() for h in range(Hq)] for b in range(B)]
    if tau_mode == "exact":
        ref = H.oracle_gaussian_step(inp, P, alpha, tau_mode="exact", niter=2, pages_override=tables)
    else:
        ref = H.oracle_gaussian_step(inp, P, alpha, tau_mode="corrected", iters=0 if tau_mode == "fixed" else 1,
                                     pages_override=tables)
    np.testing.assert_allclose(taus.cpu().numpy(), ref["tau"], rtol=TAU_RTOL, atol=1e-6)
    scale = max(1.0, float(np.abs(ref["out"]).max()))
    assert_out_close(out[:, :, 0].float().cpu().numpy(), ref["out"], dt, scale=scale)


@pytest.mark.parametrize("name,Hq,Hkv,alpha,tau_mode", [("fp16", 4, 4, 1.5, "corrected"), ("bf16", 8, 2, 1.5, "corrected"),
                                                          ("fp16", 4, 4, 2.0, "fixed"), ("fp32", 2, 2, 1.5, "exact"),
                                                          ("fp16", 4, 4, 4.0 / 3.0, "corrected")])
def test_gaussian_step_with_alibi_matches_oracle(name, Hq, Hkv, alpha, tau_mode):
    """ALiBi on the Gaussian path: biased page means, page-mixture tau_hat, positional logits and
    two correction steps by default."""
    E = _api()
    dt = DT[name]
    B, D, S, P = 2, 64, 2048, 16
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, dt, seed=83, needle_pages=(3, 90), page_size=P)
    slopes = torch.exp2(-8.0 * torch.arange(1, Hq + 1) / Hq).float()
    ref = H.oracle_gaussian_step(inp, P, alpha, tau_mode="corrected", iters=0, alibi_slopes=slopes)
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    out = torch.zeros_like(ci["q"])
    taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_gaussian_aware_entmax(ci["q"], c, ci["k_new"], ci["v_new"], out, alpha=alpha,
                                                    alibi_slopes=slopes.cuda(), append_cache=True,
                                                    tau_mode=tau_mode, niter=3, taus_out=taus)
    torch.cuda.synchronize()
    sel = c.last_gaussian_selection
    n = ref["mu"].shape[-1]
    np.testing.assert_allclose(sel["mu"][:, :, :n].cpu().numpy(), ref["mu"].numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(sel["sigma"][:, :, :n].cpu().numpy(), ref["sigma"].numpy(), rtol=1e-5, atol=2e-6)
    hs = sel["head_stats"].cpu().numpy()
    np.testing.assert_allclose(hs[..., 0], ref["mu_global"].numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(hs[..., 1], ref["sigma_global"].numpy(), rtol=1e-4)
    np.testing.assert_allclose(hs[..., 2], ref["tau_hat"].numpy(), rtol=TAU_RTOL, atol=1e-5)
    counts, pages, margin = sel["num_selected"].cpu(), sel["page_indices"].cpu(), ref["margin"].numpy()
    tables = []
    for b in range(B):
        row = []
        for h in range(Hq):
            got = pages[b, h, :counts[b, h]].tolist()
            diff = set(got) ^ set(int(x) for x in ref["pages"][b][h])
            assert all(p < n and abs(margin[b, h, p]) < 1e-4 for p in diff), (b, h, sorted(diff))
            row.append(got)
        tables.append(row)
    if tau_mode == "exact":
        ref2 = H.oracle_gaussian_step(inp, P, alpha, tau_mode="exact", niter=3, pages_override=tables,
                                      alibi_slopes=slopes)
    else:
        want_clamped = H.og.clamp_tau(ref["tau_hat"], ref["mu"], ref["sigma"],
                                      [[torch.tensor(t) for t in row] for row in tables],
                                      ref["tau_floor"], page_size=P, alpha=alpha).numpy()
        ref2 = H.oracle_gaussian_step(inp, P, alpha, tau_mode="corrected", iters=0 if tau_mode == "fixed" else 2,
                                      pages_override=tables, tau0_override=want_clamped, alibi_slopes=slopes)
    np.testing.assert_allclose(taus.cpu().numpy(), ref2["tau"], rtol=2 * TAU_RTOL, atol=1e-5)
    scale = max(1.0, float(np.abs(ref2["out"]).max()))
    assert_out_close(out[:, :, 0].float().cpu().numpy(), ref2["out"], dt, scale=scale)


def test_cache_helper_methods_of_the_reference_object():
    """select_gaussian_aware on its own (default excess-margin fraction 0.1 as in kv_cache.py:229),
    the page-table buffer and the workspace query."""
    E = _api()
    B, nh, D, S, P = 1, 4, 64, 2048, 16
    inp = H.cpu_inputs(B, nh, nh, D, S, torch.float16, seed=61, needle_pages=(8, 70))
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    c.append(ci["k_new"], ci["v_new"])
    pages, counts = c.select_gaussian_aware(ci["q"], alpha=1.5)
    oc = H.oracle_cache_after_append(inp, P)
    ref = H.og.gaussian_selection(inp["q"], oc.k_mean, oc.k_std, S + 1, P, 1.5, threshold_excess_margin_fraction=0.1)
    assert c.last_num_selected_per_head is counts
    margin = ref["margin"].numpy()
    for h in range(nh):
        got = pages[0, h, :int(counts[0, h])].tolist()
        diff = set(got) ^ set(int(x) for x in ref["pages"][0][h])
        assert all(abs(margin[0, h, p]) < 1e-5 for p in diff), (h, diff)
        assert got[-1] == (S + 1 + P - 1) // P - 1
    buf = c.get_page_indices_buf(B, nh, 5, 128)
    assert buf.shape == (B, nh, 6) and buf.dtype == torch.int32 and (buf[:, :, 5] == 128).all()
    assert c.get_paged_decode_workspace(B, nh, D)["workspace"].is_cuda


def test_gaussian_sigma_mean_override_reproduces_full_batch():
    """Half a batch + the full batch's mean of sigma_global == that half of the full batch."""
    E = _api()
    B, nh, D, S, P = 4, 4, 64, 1500, 16
    inp = H.cpu_inputs(B, nh, nh, D, S, torch.float16, seed=61, needle_pages=(5,))
    ci = H.to_cuda(inp)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    out = torch.zeros_like(ci["q"])
    E.sparse_attention_decode_gaussian_aware_entmax(ci["q"], c, ci["k_new"], ci["v_new"], out, append_cache=True)
    full_pages = c.last_gaussian_selection["page_indices"].clone()
    full_counts = c.last_gaussian_selection["num_selected"].clone()
    sigma_mean = c.last_gaussian_selection["head_stats"][..., 1].mean().reshape(1).clone()
    half = {k: v[:2].contiguous() for k, v in ci.items()}
    c2 = E.PagedKVCache(page_size=P)
    c2.initialize(half["k"], half["v"])
    out2 = torch.zeros_like(half["q"])
    E.sparse_attention_decode_gaussian_aware_entmax(half["q"], c2, half["k_new"], half["v_new"], out2,
                                                    append_cache=True, sigma_mean=sigma_mean)
    s2 = c2.last_gaussian_selection
    assert torch.equal(s2["num_selected"], full_counts[:2])
    for b in range(2):
        for h in range(nh):
            nsel = int(full_counts[b, h])
            assert torch.equal(s2["page_indices"][b, h, :nsel], full_pages[b, h, :nsel])
    assert torch.equal(out2, out[:2])


# --------------------------------------------------------------------------- properties at full size

def test_full_size_topk_properties():
    """B=1, H=32, D=128, 32k context, budget 2048, fp16: properties that need no oracle run."""
    E = _api()
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    w = CONFIGS["topk_32k"]
    inp = make_inputs(w, device="cuda")
    inp["v"].fill_(1.0)
    inp["v_new"].fill_(1.0)
    c = E.PagedKVCache(page_size=w.page_size)
    c.initialize(inp["k"], inp["v"])
    out = torch.zeros_like(inp["q"])
    taus = torch.zeros(1, 32, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, w.token_budget,
                                    alpha=w.alpha, niter=2, taus_out=taus)
    pages1 = c.last_topk_selection["page_indices"][:, :, :129].clone()
    out1 = out.clone()
    # with V == 1 every output element equals sum_i p_i, which entmax normalises to 1
    assert torch.allclose(out1.float(), torch.ones_like(out1, dtype=torch.float32), atol=2e-3)
    # every needle page must be selected by every head; sets are sorted, unique, end with the last page
    needles = set(inp["needle_pages"].tolist())
    for h in range(32):
        ids = pages1[0, h].tolist()
        assert ids == sorted(set(ids)) and ids[-1] == 2048 and needles <= set(ids)
    # determinism: a second call on the same state (no append) gives identical bits
    out.zero_()
    E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, w.token_budget,
                                    alpha=w.alpha, niter=2, append_cache=False)
    assert torch.equal(out, out1)
    assert torch.equal(c.last_topk_selection["page_indices"][:, :, :129], pages1)


def test_full_size_gaussian_properties():
    """B=8, H=32, D=128, ragged contexts in [16384, 65536], fp16 (the ragged Gaussian configuration):
    properties that need no oracle run - structure of the page tables, token counts, the exact-mode
    normalisation on a V of ones, and linearity of the output in V."""
    E = _api()
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    w = CONFIGS["gaussian_ragged"]
    inp = make_inputs(w, device="cuda")
    P, lens = w.page_size, inp["seq_lens"]
    c = E.PagedKVCache(page_size=P)
    c.initialize(inp["k"], inp["v"], seq_lens=lens)
    out = torch.zeros_like(inp["q"])
    E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, inp["k_new"], inp["v_new"], out, alpha=w.alpha,
                                                    append_cache=True, tau_mode="corrected")
    sel = c.last_gaussian_selection
    counts, pages, toks = sel["num_selected"].cpu(), sel["page_indices"].cpu(), sel["tok_counts"].cpu()
    needles = inp["needle_pages"].tolist()
    for b, n0 in enumerate(lens):
        S = n0 + 1
        n_pages = (S + P - 1) // P
        last_tokens = S - (n_pages - 1) * P
        for h in range(0, w.q_heads, 5):
            ids = pages[b, h, :counts[b, h]].tolist()
            assert ids == sorted(set(ids)) and ids[-1] == n_pages - 1 and ids[0] >= 0
            assert toks[b, h] == (len(ids) - 1) * P + last_tokens
            assert counts[b, h] < n_pages                      # the selection is a strict subset at these lengths
            assert all(p in ids for p in needles if p < n_pages - 1), (b, h)   # needle pages clear the threshold
    out1 = out.clone()
    assert torch.isfinite(out1.float()).all()
    # determinism and linearity in V: same state (no append), values doubled -> output doubled exactly
    # (a power-of-two factor commutes with every rounding on the way, and two executions are
    # bit-identical: the work list is laid out by head index)
    out1b = torch.zeros_like(out)
    E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, inp["k_new"], inp["v_new"], out1b, alpha=w.alpha,
                                                    append_cache=False, tau_mode="corrected")
    assert torch.equal(out1b, out1), "two executions on the same state must agree to the bit"
    c._v.mul_(2)
    out2 = torch.zeros_like(out)
    E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, inp["k_new"], inp["v_new"], out2, alpha=w.alpha,
                                                    append_cache=False, tau_mode="corrected")
    assert torch.equal(sel["page_indices"].cpu()[:, :, :8], c.last_gaussian_selection["page_indices"].cpu()[:, :, :8])
    normal = out1.float().abs() > 2.0 ** -13           # doubling is exact outside fp16's subnormal range
    assert torch.equal(out2.float()[normal], 2 * out1.float()[normal])
    assert torch.allclose(out2.float(), 2 * out1.float(), atol=2.0 ** -22)
    # exact mode on V == 1: every output element is sum_i p_i = 1
    c._v.fill_(1.0)
    out3 = torch.zeros_like(out)
    E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, inp["k_new"], inp["v_new"], out3, alpha=w.alpha,
                                                    append_cache=False, tau_mode="exact", niter=3)
    assert torch.allclose(out3.float(), torch.ones_like(out3, dtype=torch.float32), atol=2e-3)


@pytest.mark.parametrize("mode", ["topk", "gaussian"])
def test_graph_replay_equals_eager_steps(mode):
    """A captured step replayed token after token gives the bits of eager calls, across a
    page boundary, with the sequence lengths advancing on the device."""
    E = _api()
    from entmaxkv_b200.graph import DecodeStepGraph
    B, Hq, Hkv, D, S, P = 2, 8, 4, 128, 1000, 16
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.float16, seed=81, needle_pages=(9,)))
    g = torch.Generator(device="cuda").manual_seed(82)
    toks = [tuple(torch.randn(B, n, 1, D, generator=g, device="cuda").half() for n in (Hq, Hkv, Hkv))
            for _ in range(12)]
    ca, cb = E.PagedKVCache(P), E.PagedKVCache(P)
    ca.initialize(inp["k"], inp["v"])
    cb.initialize(inp["k"], inp["v"])
    graph = DecodeStepGraph(cb, Hq, mode, token_budget=256, alpha=1.5, niter=2)
    out = torch.zeros_like(inp["q"])
    for q, kn, vn in toks:
        if mode == "topk":
            E.sparse_attention_decode_paged(q, ca, kn, vn, out, 256, alpha=1.5, niter=2)
        else:
            E.sparse_attention_decode_gaussian_aware_entmax(q, ca, kn, vn, out, alpha=1.5, append_cache=True)
        got = graph.step(q, kn, vn)
        assert torch.equal(got, out)
    assert ca.seq_len == cb.seq_len == S + 12 and torch.equal(ca.seq_lens, cb.seq_lens)
    assert torch.equal(ca.k_cache, cb.k_cache) and torch.equal(ca.k_std, cb.k_std)


@pytest.mark.parametrize("mode", ["topk", "gaussian"])
def test_graph_step_with_pinned_host_buffers_equals_device_steps(mode):
    """``step_pinned``: inputs in the graph's page-locked buffers, the host-to-device copies and the step (whose
    last kernel stores the output rows into the page-locked output buffer) as ONE replayed graph; same bits as ``step`` on device tensors, also when the
    two kinds of step alternate on one cache and when the cache has to grow."""
    E = _api()
    from entmaxkv_b200.graph import DecodeStepGraph
    B, Hq, Hkv, D, S, P = 2, 8, 2, 128, 1000, 16
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=181, needle_pages=(9,)))
    g = torch.Generator(device="cuda").manual_seed(182)
    toks = [tuple(torch.randn(B, n, 1, D, generator=g, device="cuda").bfloat16() for n in (Hq, Hkv, Hkv))
            for _ in range(20)]
    ca, cb = E.PagedKVCache(P, capacity=S + 10), E.PagedKVCache(P, capacity=S + 10)    # both grow on the way
    ca.initialize(inp["k"], inp["v"])
    cb.initialize(inp["k"], inp["v"])
    ga = DecodeStepGraph(ca, Hq, mode, token_budget=256, alpha=1.5, niter=2)
    gb = DecodeStepGraph(cb, Hq, mode, token_budget=256, alpha=1.5, niter=2)
    io = gb.pinned_io()
    assert all(t.is_pinned() for t in io.values())
    for i, (q, kn, vn) in enumerate(toks):
        want = ga.step(q, kn, vn).clone()
        if i % 5 == 4:                          # now and then through the device-tensor entry of the same object
            got = gb.step(q, kn, vn).cpu()
        else:
            io["q"].copy_(q)
            io["k_new"].copy_(kn)
            io["v_new"].copy_(vn)
            got = gb.step_pinned()
            torch.cuda.current_stream().synchronize()
        assert torch.equal(got, want.cpu()), i
    assert ca.seq_len == cb.seq_len == S + 20 and ca.capacity == cb.capacity > S + 10


@pytest.mark.parametrize("world", [2, 4])
def test_sequence_sharded_step_on_one_device_equals_unsharded(world):
    """R shards driven in one process (local reduction instead of NCCL) through the stage entry
    points of the C ABI give the unsharded step's tau and output; page sets agree up to the offset."""
    E = _api()
    from entmaxkv_b200 import sharded
    B, Hq, Hkv, D, S, P = 1, 8, 2, 128, 64 * 16 + 7, 16
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=95, needle_pages=(5, 40)))
    c = E.PagedKVCache(P)
    c.initialize(inp["k"], inp["v"])
    out = torch.zeros_like(inp["q"])
    taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, inp["k_new"], inp["v_new"], out,
                                                    append_cache=True, taus_out=taus)
    full = c.last_gaussian_selection
    parts = sharded.split_pages(S, P, world)
    shards = []
    for r, (lo, hi) in enumerate(parts):
        sh = sharded.GpuSequenceShard(P, r, world)
        sh.initialize(inp["k"][:, :, lo:hi].contiguous(), inp["v"][:, :, lo:hi].contiguous())
        sh.set_global_lengths([S] * B)
        shards.append(sh)
    outs = sharded.sharded_gaussian_decode_step(
        shards, sharded.local_reduce, [inp["q"]] * world, [inp["k_new"]] * world, [inp["v_new"]] * world,
        alpha=1.5)
    torch.cuda.synchronize()
    np.testing.assert_allclose(shards[0].tau.cpu().numpy(), taus.cpu().numpy(), rtol=1e-5, atol=1e-6)
    for h in range(Hq):
        want = full["page_indices"][0, h, :int(full["num_selected"][0, h])].tolist()
        got = []
        for sh, (lo, _) in zip(shards, parts):
            n = int(sh.counts[0, h])
            got += [p + lo // P for p in sh.pages[0, h, :n].tolist()]
        assert got == want, h
    ref = out[:, :, 0].float().cpu().numpy()
    got = outs[0][:, :, 0].cpu().numpy()
    scale = max(1.0, float(np.abs(ref).max()))
    assert_out_close(ref, got, torch.bfloat16, scale=scale)


def test_library_reports_argument_errors():
    E = _api()
    inp = H.to_cuda(H.cpu_inputs(1, 2, 2, 64, 64, torch.float16, seed=71))
    c = E.PagedKVCache(16)
    c.initialize(inp["k"], inp["v"])
    out = torch.zeros_like(inp["q"])
    with pytest.raises(ValueError):
        E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, 64, alpha=1.0)
    with pytest.raises(ValueError):
        E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, inp["k_new"], inp["v_new"], out,
                                                        tau_mode="bogus")
    with pytest.raises(ValueError):
        E.sparse_attention_decode_paged(inp["q"].float(), c, inp["k_new"], inp["v_new"], out, 64)
    with pytest.raises(ValueError):
        c.append(inp["k_new"].cpu(), inp["v_new"].cpu())
