"""The benchmark configurations at their own sizes, CUDA path vs CPU oracle on the benchmark's
own bits (run on a B200: ``-m gpu``).

``entmaxkv_b200.workloads.make_inputs`` draws counter-based tensors that are identical on the
CPU and on the GPU, so the tensors the benchmark times are the tensors the oracle sees here:
they are drawn on the GPU (as the benchmark does), copied to the host one (batch row, KV head)
at a time, and the oracle runs on each slice.  A separate test draws slices on the CPU and
checks them against the GPU draw bit for bit.

Covered: the 32k top-k configuration whole; the shortest and the longest row of the ragged
Gaussian configuration; one full-context batch row (8 KV heads, 32 query heads, 131 073 tokens,
bf16) of the GQA configuration for top-k and for Gaussian-aware selection at alpha 1.5 and 2;
the million-token request whole (65 537 pages: the only configuration whose selection kernels
need more than one round of 8192 pages) unsharded and as eight sequence shards; and two small
synthetic cases built to cross the round boundaries of the top-k select and of the group union.

Bars (the same as the small cases): 16-bit page scores and top-k page sets bit-exact; Gaussian
moments 1e-5, tau_hat / tau_floor / tau 1e-4 relative; Gaussian page sets exact outside the
pages whose margin against the kernel's own tau_floor is below 1e-5; outputs within 2e-3 x
magnitude + the half-ulp of the 16-bit output.
"""

import dataclasses
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests import _harness as H
from tests.test_gpu_parity import OUT_TOL, TAU_RTOL, assert_out_close  # noqa: F401


def _api():
    import entmaxkv_b200 as E
    return E


def _slice_cpu(inp, b, hk, G, n):
    """CPU copies of one (batch row, KV head) of GPU inputs, trimmed to ``n`` context tokens."""
    return dict(k=inp["k"][b:b + 1, hk:hk + 1, :n].cpu(), v=inp["v"][b:b + 1, hk:hk + 1, :n].cpu(),
                q=inp["q"][b:b + 1, hk * G:(hk + 1) * G].cpu(),
                k_new=inp["k_new"][b:b + 1, hk:hk + 1].cpu(), v_new=inp["v_new"][b:b + 1, hk:hk + 1].cpu())


class OracleSide:
    """Per (batch row, KV head) oracle caches of a GPU-resident input set, built once."""

    def __init__(self, inp, lens, P, G):
        self.P, self.G, self.lens = P, G, lens
        B, Hkv = inp["k"].shape[:2]
        self.B, self.Hkv = B, Hkv
        self.slices, self.caches = {}, {}
        for b in range(B):
            for hk in range(Hkv):
                s = _slice_cpu(inp, b, hk, G, lens[b])
                self.slices[b, hk] = s
                self.caches[b, hk] = H.oracle_cache_after_append(s, P)

    def sigma_mean(self):
        """Batch-wide mean of sigma_global (the scalar that couples every head of a call)."""
        vals = []
        for (b, hk), c in self.caches.items():
            n_pages = c.k_mean.shape[2]
            n_stats = n_pages - 1 if n_pages > 1 else n_pages
            mu, var, _ = H.og.page_moments(self.slices[b, hk]["q"], c.k_mean, c.k_std, n_stats)
            _, mv, vm = H.og.head_moments(mu, var)
            vals.append(H.og.global_sigma(mv, vm).reshape(-1))
        return float(torch.cat(vals).to(torch.float32).mean().item())


def check_topk(E, c, inp, side, w, niter=2):
    """One top-k decode step on cache ``c`` against the oracle, every (row, KV head)."""
    P, G = side.P, side.G
    B, Hq = inp["q"].shape[:2]
    out = torch.zeros_like(inp["q"])
    taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, w.token_budget,
                                    alpha=w.alpha, niter=niter, append_cache=False, taus_out=taus)
    torch.cuda.synchronize()
    sel = c.last_topk_selection
    tied = []
    for (b, hk), oc in side.caches.items():
        ref = H.oracle_topk_step(side.slices[b, hk], P, w.token_budget, w.alpha, niter, cache=oc)
        hs = slice(hk * G, (hk + 1) * G)
        n_scored, width = ref["scores"].shape[-1], ref["pages"].shape[-1]
        assert torch.equal(sel["scores"][b:b + 1, hs, :n_scored].cpu(), ref["scores"]), (b, hk, "scores")
        assert torch.equal(sel["page_indices"][b:b + 1, hs, :width].cpu(), ref["pages"]), (b, hk, "page sets")
        assert sel["num_selected"][b, hs].tolist() == [width] * G
        assert sel["tok_counts"][b, hs].tolist() == [ref["T"]] * G
        tied.append(int(H.otopk.boundary_tied_pages(ref["scores"], width - 1).sum(-1).max()))
        np.testing.assert_allclose(taus[b:b + 1, hs].cpu().numpy(), ref["tau"], rtol=TAU_RTOL, atol=1e-6)
        np.testing.assert_allclose(taus[b:b + 1, hs].cpu().numpy(), ref["tau_true"], rtol=TAU_RTOL, atol=1e-6)
        got = out[b:b + 1, hs, 0].float().cpu().numpy()
        assert_out_close(got, ref["out"], w.dtype)
        assert_out_close(got, ref["out_true"], w.dtype)
    return {"largest_boundary_tied_class": max(tied)}


def check_gaussian(E, c, inp, side, w, alpha, tau_mode="corrected"):
    """One Gaussian-aware decode step on cache ``c`` against the oracle, every (row, KV head)."""
    P, G = side.P, side.G
    B, Hq = inp["q"].shape[:2]
    out = torch.zeros_like(inp["q"])
    taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
    E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, inp["k_new"], inp["v_new"], out, alpha=alpha,
                                                    append_cache=False, tau_mode=tau_mode, taus_out=taus)
    torch.cuda.synchronize()
    sel = c.last_gaussian_selection
    sigma_mean = side.sigma_mean()
    a = alpha - 1.0
    boundary = 0
    selected = 0
    for (b, hk), oc in side.caches.items():
        s = side.slices[b, hk]
        S = oc.seq_len
        ref = H.og.gaussian_selection(s["q"], oc.k_mean, oc.k_std, S, P, alpha, sigma_mean_override=sigma_mean)
        hs = slice(hk * G, (hk + 1) * G)
        n = ref["mu"].shape[-1]
        mu = sel["mu"][b, hs, :n].cpu()
        sigma = sel["sigma"][b, hs, :n].cpu()
        np.testing.assert_allclose(mu.numpy(), ref["mu"][0].numpy(), rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(sigma.numpy(), ref["sigma"][0].numpy(), rtol=1e-5, atol=2e-6)
        hst = sel["head_stats"][b, hs].cpu().numpy()
        np.testing.assert_allclose(hst[:, 0], ref["mu_global"][0].numpy(), rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(hst[:, 1], ref["sigma_global"][0].numpy(), rtol=1e-4)
        np.testing.assert_allclose(hst[:, 2], ref["tau_hat"][0].numpy(), rtol=TAU_RTOL, atol=1e-6)
        tfl = sel["tau_floor"][b, hs].cpu()
        np.testing.assert_allclose(tfl.numpy(), ref["tau_floor"][0].numpy(), rtol=TAU_RTOL, atol=1e-6)
        # page sets: the oracle's moments against the KERNEL's tau_floor (already held to 1e-4 above), so
        # that the only pages left open are those whose own margin is inside the moments' tolerance
        z_page = H.og.z_of_quantile(ref["max_quantile"], P)
        margin = (a * (ref["mu"][0] + float(z_page) * ref["sigma"][0]) - tfl[:, None]).numpy()
        counts = sel["num_selected"][b, hs].cpu()
        pages = sel["page_indices"][b, hs].cpu()
        n_pages = oc.k_mean.shape[2]
        tables = []
        for j in range(G):
            got = pages[j, :counts[j]].numpy()
            assert (np.diff(got) > 0).all() and got[-1] == n_pages - 1, "ascending, last page at the end"
            want = np.nonzero(margin[j] > 0)[0]
            diff = np.setxor1d(got[got < n], want)
            assert (np.abs(margin[j, diff]) < 1e-5).all(), (b, hk, j, diff[:8], margin[j, diff[:8]])
            boundary += diff.size
            selected += got.size
            tables.append(got.tolist())
        last = H.og.last_page_size(S, P)
        assert sel["tok_counts"][b, hs].tolist() == [(len(t) - 1) * P + last for t in tables]
        if tau_mode == "exact":
            ref2 = H.oracle_gaussian_step(s, P, alpha, tau_mode="exact", niter=2, pages_override=[tables], cache=oc)
        else:
            want_clamped = H.og.clamp_tau(ref["tau_hat"], ref["mu"], ref["sigma"], [[torch.tensor(t) for t in tables]],
                                          ref["tau_floor"], page_size=P, alpha=alpha).numpy()
            ref2 = H.oracle_gaussian_step(s, P, alpha, tau_mode="corrected", iters=0 if tau_mode == "fixed" else 1,
                                          pages_override=[tables], tau0_override=want_clamped, cache=oc)
        np.testing.assert_allclose(taus[b:b + 1, hs].cpu().numpy(), ref2["tau"], rtol=TAU_RTOL, atol=1e-6)
        scale = max(1.0, float(np.abs(ref2["out"]).max()))
        assert_out_close(out[b:b + 1, hs, 0].float().cpu().numpy(), ref2["out"], w.dtype, scale=scale)
    return {"boundary_pages": boundary, "selected_pages": selected, "out": out, "taus": taus}


def _build(E, w, inp, lens):
    c = E.PagedKVCache(page_size=w.page_size)
    c.initialize(inp["k"], inp["v"], seq_lens=lens, capacity=inp["k"].shape[2] + 64)
    c.append(inp["k_new"], inp["v_new"])
    return c


def _status_clean(c):
    import ctypes
    from entmaxkv_b200 import _lib
    assert c.device_status() == 0
    for key, ws in c._scratch.items():
        if key[0] == "decode_ws":
            st = ctypes.c_int32(-1)
            _lib.check(_lib.load().ekv_read_status(ws.data_ptr(), ctypes.byref(st), _lib.stream_ptr()), "status")
            assert st.value == 0


# --------------------------------------------------------------------------- the generator itself

@pytest.mark.parametrize("name,b,hk", [("topk_32k", 0, 5), ("gqa_128k_topk", 17, 3), ("gaussian_ragged", 6, 30)])
def test_workload_draws_are_device_independent(name, b, hk):
    """A (batch row, KV head) slice drawn on the CPU equals the same slice drawn on the GPU, and a slice
    equals the corresponding part of a larger draw: the oracle can be fed the benchmark's own bits."""
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    w = CONFIGS[name]
    on_cpu = make_inputs(w, "cpu", batch_slice=slice(b, b + 1), kv_head_slice=slice(hk, hk + 1))
    on_gpu = make_inputs(w, "cuda", batch_slice=slice(b, b + 1), kv_head_slice=slice(max(hk - 1, 0), hk + 1))
    j = 1 if hk else 0
    G = w.q_heads // w.kv_heads
    for nm in ("k", "v", "k_new", "v_new"):
        assert torch.equal(on_gpu[nm][:, j:j + 1].cpu(), on_cpu[nm]), nm
    assert torch.equal(on_gpu["q"][:, j * G:(j + 1) * G].cpu(), on_cpu["q"])
    assert on_gpu["seq_lens"] == on_cpu["seq_lens"] and torch.equal(on_gpu["needle_pages"], on_cpu["needle_pages"])
    x = on_cpu["v"].float()
    assert abs(float(x.mean())) < 1e-3 and abs(float(x.std()) - 1.0) < 2e-3


# --------------------------------------------------------------------------- the configurations

def test_topk_32k_whole_against_oracle(topk_path):
    """B=1, 32 heads (MHA), 32 769 tokens, fp16, budget 2048: every head."""
    E = _api()
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    w = CONFIGS["topk_32k"]
    inp = make_inputs(w, "cuda")
    lens = inp["seq_lens"]
    c = _build(E, w, inp, lens)
    side = OracleSide(inp, lens, w.page_size, 1)
    info = check_topk(E, c, inp, side, w)
    _status_clean(c)
    print("topk_32k", info)


def test_dense_entmax_32k_against_dense_oracle():
    """The 32k configuration with a budget that covers every page: dense entmax attention through the same
    kernels (the "Entmax dense" arm of the reference's figure), against exact alpha-entmax attention over all
    32 769 tokens on the CPU."""
    E = _api()
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    w = CONFIGS["topk_32k"]
    inp = make_inputs(w, "cuda")
    c = _build(E, w, inp, inp["seq_lens"])
    out = torch.zeros_like(inp["q"])
    E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, token_budget=w.context + 4096,
                                    alpha=w.alpha, niter=2, append_cache=False)
    torch.cuda.synchronize()
    assert c.last_topk_selection["tok_counts"].cpu().tolist() == [[w.context + 1] * w.q_heads]
    k_all = torch.cat([inp["k"], inp["k_new"]], dim=2).cpu()
    v_all = torch.cat([inp["v"], inp["v_new"]], dim=2).cpu()
    want = H.odense.dense_entmax_decode(inp["q"].cpu(), k_all, v_all, w.alpha, compute_dtype=torch.float64)
    assert_out_close(out[:, :, 0].float().cpu().numpy(), want[:, :, 0].numpy(), w.dtype)
    _status_clean(c)


def test_gaussian_ragged_shortest_and_longest_row_against_oracle():
    """Two rows of the ragged B=8 configuration (fp16, 32 heads), as a ragged batch of two."""
    E = _api()
    from entmaxkv_b200.workloads import CONFIGS, make_inputs, workload_lengths
    w = CONFIGS["gaussian_ragged"]
    _, lens_all = workload_lengths(w)
    rows = [int(np.argmin(lens_all)), int(np.argmax(lens_all))]
    parts = [make_inputs(w, "cuda", batch_slice=slice(r, r + 1)) for r in rows]
    inp = {nm: torch.cat([p[nm] for p in parts], dim=0) for nm in ("k", "v", "q", "k_new", "v_new")}
    lens = [lens_all[r] for r in rows]
    c = _build(E, w, inp, lens)
    side = OracleSide(inp, lens, w.page_size, 1)
    info = check_gaussian(E, c, inp, side, w, w.alpha)
    _status_clean(c)
    print("gaussian_ragged rows", rows, lens, {k: v for k, v in info.items() if k.endswith("pages")})


def test_gqa_128k_one_batch_row_against_oracle():
    """One full-context row of the B=32 GQA configuration: 8 KV heads, 32 query heads, 131 073 tokens,
    bf16 - top-k at budget 4096 (alpha 1.5 and 2) and Gaussian-aware selection (alpha 1.5 and 2; the
    alpha 1.5 step goes through the group-shared K pass) on the same cache."""
    E = _api()
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    w = CONFIGS["gqa_128k_topk"]
    row = 11
    inp = make_inputs(w, "cuda", batch_slice=slice(row, row + 1))
    lens = inp["seq_lens"]
    c = _build(E, w, inp, lens)
    side = OracleSide(inp, lens, w.page_size, w.q_heads // w.kv_heads)
    print("gqa_128k topk a=1.5", check_topk(E, c, inp, side, w))
    print("gqa_128k topk a=2", check_topk(E, c, inp, side, dataclasses.replace(w, alpha=2.0)))
    # the same two steps through the many-head kernel (the whole B=32 configuration takes it by default)
    os.environ["EKV_STREAM_TOPK"] = "1"
    try:
        print("gqa_128k topk a=1.5, stream", check_topk(E, c, inp, side, w))
        assert c.last_topk_selection.get("stream", False)
        print("gqa_128k topk a=2, stream", check_topk(E, c, inp, side, dataclasses.replace(w, alpha=2.0)))
    finally:
        os.environ.pop("EKV_STREAM_TOPK", None)
    for alpha in (1.5, 2.0):
        info = check_gaussian(E, c, inp, side, w, alpha)
        print("gqa_128k gaussian", alpha, {k: v for k, v in info.items() if k.endswith("pages")})
    _status_clean(c)


def test_million_token_request_against_oracle_unsharded_and_as_eight_shards():
    """B=1, 64 query heads / 8 KV heads, 1 048 577 tokens, bf16, 65 537 pages: the whole request against
    the oracle (Gaussian-aware, alpha 1.5), a top-k step over the same cache (nine rounds of the radix
    select), and the same request cut into eight sequence shards driven through the stage entry points."""
    E = _api()
    from entmaxkv_b200 import sharded
    from entmaxkv_b200.workloads import CONFIGS, make_inputs
    w = CONFIGS["million_gaussian"]
    inp = make_inputs(w, "cuda")
    lens = inp["seq_lens"]
    P, S = w.page_size, w.context
    c = _build(E, w, inp, lens)
    side = OracleSide(inp, lens, P, w.q_heads // w.kv_heads)
    info = check_gaussian(E, c, inp, side, w, w.alpha)
    print("million gaussian", {k: v for k, v in info.items() if k.endswith("pages")})
    wt = dataclasses.replace(w, mode="topk", token_budget=16 * 1024)
    print("million topk", check_topk(E, c, inp, side, wt))
    _status_clean(c)
    del side
    out_full, tau_full = info["out"], info["taus"]
    sel = c.last_gaussian_selection          # the top-k step above keeps its own record
    world = 8
    parts = sharded.split_pages(S, P, world)
    shards = []
    for r, (lo, hi) in enumerate(parts):
        sh = sharded.GpuSequenceShard(P, r, world)
        sh.initialize(inp["k"][:, :, lo:hi].contiguous(), inp["v"][:, :, lo:hi].contiguous())
        sh.set_global_lengths([S] * w.batch)
        shards.append(sh)
    outs = sharded.sharded_gaussian_decode_step(
        shards, sharded.local_reduce, [inp["q"]] * world, [inp["k_new"]] * world, [inp["v_new"]] * world,
        alpha=w.alpha)
    torch.cuda.synchronize()
    # page sets: the shards sum the moments in another order, so tau_floor moves in its last bits and pages
    # whose margin is within that noise may flip; everything else must be the unsharded selection
    a = w.alpha - 1.0
    sbar = float(sel["head_stats"][..., 1].mean().item())
    z_page = H.og.z_of_quantile(0.99 if sbar < 1.5 else 0.995, P)
    flipped = np.zeros(w.q_heads, dtype=np.int64)
    for h in range(w.q_heads):
        want = sel["page_indices"][0, h, :int(sel["num_selected"][0, h])].cpu().numpy()
        got = np.concatenate([sh.pages[0, h, :int(sh.counts[0, h])].cpu().numpy() + lo // P
                              for sh, (lo, _) in zip(shards, parts)])
        assert (np.diff(got) > 0).all() and got[-1] == want[-1]
        diff = np.setxor1d(got, want)
        if diff.size:
            idx = torch.from_numpy(diff).cuda()
            margin = a * (sel["mu"][0, h, idx] + z_page * sel["sigma"][0, h, idx]) - sel["tau_floor"][0, h]
            assert float(margin.abs().max()) < 1e-5, (h, diff[:8])
            flipped[h] = diff.size
    print("million sharded: pages flipped inside the margin class, per head:", flipped[flipped > 0], "heads", np.nonzero(flipped)[0])
    # tau: bit-level agreement is not expected (other summation order), 1e-5 where the page sets agree; a
    # head with a flipped page sums over a slightly different token list
    got_tau, want_tau = shards[0].tau.cpu().numpy()[0], tau_full.cpu().numpy()[0]
    same = flipped == 0
    np.testing.assert_allclose(got_tau[same], want_tau[same], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got_tau[~same], want_tau[~same], rtol=2e-3, atol=1e-6)
    ref = out_full[:, :, 0].float().cpu().numpy()
    got = outs[0][:, :, 0].cpu().numpy()
    assert_out_close(ref, got, torch.bfloat16, scale=max(1.0, float(np.abs(ref).max())))


# --------------------------------------------------------------------------- round boundaries, small

def test_topk_select_over_several_rounds_of_pages():
    """More than 8192 scored pages per head (three rounds of the radix select and of the ordered pack),
    D=64 so the case is 34 MB: page sets bit-exact, tau and outputs against the oracle."""
    E = _api()
    B, Hq, Hkv, D, P = 1, 4, 2, 64, 16
    S = 16 * 20000 + 5
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, torch.float16, seed=1234, needle_pages=(3, 9000, 17000, 19999), page_size=P)
    ci = H.to_cuda(inp)
    w = dataclasses.make_dataclass("W", ["token_budget", "alpha", "dtype"])(16 * 9000, 1.5, torch.float16)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    c.append(ci["k_new"], ci["v_new"])
    side = OracleSide(ci, [S], P, Hq // Hkv)
    print("topk multi-round, large k", check_topk(E, c, ci, side, w))
    w.token_budget = 16 * 300
    print("topk multi-round, small k", check_topk(E, c, ci, side, w))
    _status_clean(c)


@pytest.mark.parametrize("Hq,Hkv", [(4, 1), (8, 2)])
def test_group_union_over_several_rounds_against_oracle(Hq, Hkv):
    """GQA groups of four with more than 8192 pages per head: the grouped route (union table built in
    several rounds) directly against the oracle, not only against the per-head route."""
    E = _api()
    B, D, P = 1, 128, 16
    S = 16 * 9100 + 3
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=4321, needle_pages=(5, 4000, 9050), page_size=P)
    ci = H.to_cuda(inp)
    w = dataclasses.make_dataclass("W", ["alpha", "dtype"])(1.5, torch.bfloat16)
    c = E.PagedKVCache(page_size=P)
    c.initialize(ci["k"], ci["v"])
    c.append(ci["k_new"], ci["v_new"])
    side = OracleSide(ci, [S], P, Hq // Hkv)
    for tau_mode in ("corrected", "exact"):
        info = check_gaussian(E, c, ci, side, w, 1.5, tau_mode=tau_mode)
        print("grouped multi-round", tau_mode, {k: v for k, v in info.items() if k.endswith("pages")})
    assert getattr(c, "last_group_tables", None) is not None, "the case must take the group-shared route"
    _status_clean(c)
