"""The many-head top-k step with selection and tau hidden inside the K pass (one persistent kernel after the
score sweep) against the general kernels and the oracle: page scores, page tables and counts bit-identical, tau
and the output equal to rounding; problems that do not fit fall back."""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from tests import _harness as H

pytestmark = pytest.mark.gpu

DT = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def _step(E, inp, P, budget, alpha, niter, lens, stream, block_table=False, steps=1, toks=None):
    os.environ["EKV_STREAM_TOPK"] = "1" if stream else "0"
    os.environ["EKV_FUSED_SMALL"] = "0"
    try:
        c = E.PagedKVCache(P, block_table=True, block_order="random") if block_table else E.PagedKVCache(P)
        c.initialize(inp["k"], inp["v"], seq_lens=lens)
        B, Hq = inp["q"].shape[:2]
        outs = []
        for s in range(steps):
            out = torch.zeros_like(inp["q"])
            taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
            kn, vn = (inp["k_new"], inp["v_new"]) if toks is None else toks[s]
            E.sparse_attention_decode_paged(inp["q"], c, kn, vn, out, budget, alpha=alpha, niter=niter, taus_out=taus)
            torch.cuda.synchronize()
            assert c.device_status() == 0
            sel = c.last_topk_selection
            assert bool(sel.get("stream", False)) == stream
            outs.append((out, taus, {k: (v.clone() if torch.is_tensor(v) else v) for k, v in sel.items()}))
        return c, outs
    finally:
        os.environ.pop("EKV_STREAM_TOPK", None)
        os.environ.pop("EKV_FUSED_SMALL", None)


CASES = [
    # B, Hq, Hkv, lengths, budget, dtype, alpha, niter, block table        (head_dim 128, page size 16, 16-bit)
    (10, 32, 8, [2100] * 10, 512, "bf16", 1.5, 2, False),         # 320 heads on 148 blocks: two to three heads each
    (2, 8, 2, [3000, 1700], 256, "fp16", 1.5, 10, False),         # ragged rows, the wrapper's default niter
    (1, 4, 4, [1500], 128, "bf16", 2.0, 3, False),
    (1, 4, 4, [600], 96, "fp16", 1.75, 4, False),                 # general alpha
    (3, 4, 2, [9, 40, 17], 64, "fp16", 1.5, 2, False),            # one to three pages: little or nothing to score
    (1, 4, 2, [40], 4000, "bf16", 1.5, 2, False),                 # budget covers every page
    (1, 2, 2, [16 * 700], 8, "bf16", 1.5, 2, False),              # budget below one page: last page only
    (2, 8, 2, [2600, 2600], 256, "bf16", 1.5, 2, True),           # block-table cache
    (1, 160, 160, [300], 64, "fp16", 1.5, 2, False),              # more heads than blocks, one chunk each
    (1, 2, 1, [16 * 9000 + 3], 4096, "bf16", 1.5, 2, False),      # two selection rounds, 17 chunks per head
    (1, 2, 1, [16 * 8300 + 5], 2048, "fp16", 1.5, 2, False),      # pages 8192..8299: the one extra key per thread, no memory round
    (4, 8, 8, [5000, 4100, 4097, 4096], 4096, "fp16", 1.5, 2, False),   # chunk and page boundaries in the kept tokens
]


@pytest.mark.parametrize("case", CASES, ids=[f"case{i}" for i in range(len(CASES))])
def test_stream_step_equals_general_step(case):
    import entmaxkv_b200 as E
    B, Hq, Hkv, lens, budget, name, alpha, niter, bt = case
    D, P = 128, 16
    dt = DT[name]
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, max(lens), dt, seed=700 + max(lens), needle_pages=(1, 5), page_size=P))
    _, (r0,) = _step(E, inp, P, budget, alpha, niter, lens, stream=False, block_table=bt)
    _, (r1,) = _step(E, inp, P, budget, alpha, niter, lens, stream=True, block_table=bt)
    (out0, tau0, sel0), (out1, tau1, sel1) = r0, r1
    assert torch.equal(sel0["num_selected"], sel1["num_selected"])
    assert torch.equal(sel0["tok_counts"], sel1["tok_counts"])
    for b, n in enumerate(lens):
        n_scored = (n + 1 + P - 1) // P - 1
        assert torch.equal(sel0["scores"][b, :, :n_scored], sel1["scores"][b, :, :n_scored])
    width = torch.arange(sel0["page_indices"].shape[-1], device="cuda")[None, None, :] < sel0["num_selected"][:, :, None]
    assert torch.equal(sel0["page_indices"][width], sel1["page_indices"][width]), "page tables: bit-identical"
    np.testing.assert_allclose(tau1.cpu().numpy(), tau0.cpu().numpy(), rtol=2e-5, atol=1e-6)
    tol = {"fp16": 2e-3, "bf16": 1.6e-2}[name]
    assert (out1.float() - out0.float()).abs().max().item() <= tol
    assert (sel1["support"] > 0).all() and (sel1["support"] <= sel1["tok_counts"]).all()


def test_stream_step_with_a_support_wider_than_one_gather_round():
    """A nearly flat score row gives every kept token a non-zero weight: the support (2064 tokens here) is
    compacted once and its value rows are gathered in rounds of 1024."""
    import entmaxkv_b200 as E
    B, Hq, Hkv, D, S, P, budget = 2, 8, 2, 128, 4000, 16, 2048
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=99, page_size=P)
    inp["q"] = (inp["q"].float() * 1e-3).to(torch.bfloat16)
    inp = H.to_cuda(inp)
    _, ((out0, tau0, sel0),) = _step(E, inp, P, budget, 1.5, 3, [S] * B, stream=False)
    _, ((out1, tau1, sel1),) = _step(E, inp, P, budget, 1.5, 3, [S] * B, stream=True)
    assert torch.equal(sel0["page_indices"], sel1["page_indices"])
    assert (sel1["support"] == sel1["tok_counts"]).all() and int(sel1["tok_counts"].max()) > 2048
    np.testing.assert_allclose(tau1.cpu().numpy(), tau0.cpu().numpy(), rtol=2e-5, atol=1e-6)
    assert (out1.float() - out0.float()).abs().max().item() <= 1.6e-2


@pytest.mark.parametrize("flat", [False, True])
def test_selection_across_the_register_tail(flat):
    """8300 scored pages: pages 8192.. are the one extra key a thread holds.  With needle pages there, the best
    pages sit in the tail; with a zero query every score ties and the lower page ids must win."""
    import entmaxkv_b200 as E
    B, Hq, Hkv, D, P, S = 1, 4, 2, 128, 16, 16 * 8300 + 7
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=8300, needle_pages=(8195, 8250, 8299, 17), page_size=P)
    if flat:
        inp["q"] = torch.zeros_like(inp["q"])
    inp = H.to_cuda(inp)
    _, ((out0, tau0, sel0),) = _step(E, inp, P, 1024, 1.5, 2, [S], stream=False)
    _, ((out1, tau1, sel1),) = _step(E, inp, P, 1024, 1.5, 2, [S], stream=True)
    assert torch.equal(sel0["num_selected"], sel1["num_selected"])
    assert torch.equal(sel0["page_indices"], sel1["page_indices"])
    pages = sel1["page_indices"][0, 0, :int(sel1["num_selected"][0, 0])].tolist()
    if flat:
        assert pages == list(range(64)) + [8300]
    else:
        assert {8195, 8250, 8299, 17} <= set(pages)
    np.testing.assert_allclose(tau1.cpu().numpy(), tau0.cpu().numpy(), rtol=2e-5, atol=1e-6)
    assert (out1.float() - out0.float()).abs().max().item() <= 1.6e-2


def test_stream_step_matches_oracle_directly():
    import entmaxkv_b200 as E
    B, Hq, Hkv, D, S, P, budget, alpha, niter = 2, 16, 4, 128, 5000, 16, 512, 1.5, 3
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=4343, needle_pages=(7, 100, 250), page_size=P)
    ref = H.oracle_topk_step(inp, P, budget, alpha, niter)
    _, ((out, taus, sel),) = _step(E, H.to_cuda(inp), P, budget, alpha, niter, [S] * B, stream=True)
    n_scored, width = ref["scores"].shape[-1], ref["pages"].shape[-1]
    assert torch.equal(sel["scores"][:, :, :n_scored].cpu(), ref["scores"])
    assert torch.equal(sel["page_indices"][:, :, :width].cpu(), ref["pages"])
    assert sel["tok_counts"].cpu().tolist() == [[ref["T"]] * Hq] * B
    np.testing.assert_allclose(taus.cpu().numpy(), ref["tau"], rtol=2e-4, atol=1e-6)
    np.testing.assert_allclose(taus.cpu().numpy(), ref["tau_true"], rtol=2e-4, atol=1e-6)
    assert np.abs(out[:, :, 0].float().cpu().numpy() - ref["out"]).max() <= 1.6e-2


def test_stream_step_over_many_tokens_and_from_a_graph():
    """Twenty consecutive steps (pages complete on the way), eager and replayed from a graph: the counters the kernel
    hands heads out with are left at zero by every launch."""
    import entmaxkv_b200 as E
    from entmaxkv_b200.graph import DecodeStepGraph
    B, Hq, Hkv, D, S, P = 6, 32, 8, 128, 1000, 16
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=78, needle_pages=(4,)))
    g = torch.Generator().manual_seed(10)
    toks = [tuple(torch.randn(B, Hkv, 1, D, generator=g).to(torch.bfloat16).cuda() for _ in range(2)) for _ in range(20)]
    _, general = _step(E, inp, P, 256, 1.5, 2, [S] * B, stream=False, steps=20, toks=toks)
    c, streamed = _step(E, inp, P, 256, 1.5, 2, [S] * B, stream=True, steps=20, toks=toks)
    for s, ((o0, t0, s0), (o1, t1, s1)) in enumerate(zip(general, streamed)):
        assert torch.equal(s0["page_indices"], s1["page_indices"]) and torch.equal(s0["tok_counts"], s1["tok_counts"]), s
        np.testing.assert_allclose(t1.cpu().numpy(), t0.cpu().numpy(), rtol=2e-5, atol=1e-6)
        assert (o1.float() - o0.float()).abs().max().item() <= 1.6e-2
    os.environ["EKV_STREAM_TOPK"] = "1"
    os.environ["EKV_FUSED_SMALL"] = "0"
    try:
        eager, replay = E.PagedKVCache(P), E.PagedKVCache(P)
        eager.initialize(inp["k"], inp["v"])
        replay.initialize(inp["k"], inp["v"])
        graph = DecodeStepGraph(replay, Hq, "topk", token_budget=256, alpha=1.5, niter=2)
        out = torch.zeros_like(inp["q"])
        for kn, vn in toks[:8]:
            E.sparse_attention_decode_paged(inp["q"], eager, kn, vn, out, 256, alpha=1.5, niter=2)
            assert eager.last_topk_selection.get("stream", False)
            assert torch.equal(graph.step(inp["q"], kn, vn), out)        # bit-reproducible
    finally:
        os.environ.pop("EKV_STREAM_TOPK", None)
        os.environ.pop("EKV_FUSED_SMALL", None)


def test_host_to_host_step_through_the_many_head_kernel():
    """``step_pinned`` on a problem the many-head kernel takes: the inputs come through one copy node and the
    kernel stores its output rows straight into the page-locked buffer; same bits as the device-tensor step."""
    import entmaxkv_b200 as E
    from entmaxkv_b200.graph import DecodeStepGraph
    B, Hq, Hkv, D, S, P = 3, 32, 8, 128, 1200, 16           # 96 heads: the wrapper's default route
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=61, needle_pages=(3,)))
    g = torch.Generator().manual_seed(12)
    toks = [tuple(torch.randn(B, n, 1, D, generator=g).to(torch.bfloat16).cuda() for n in (Hq, Hkv, Hkv)) for _ in range(12)]
    ca, cb = E.PagedKVCache(P), E.PagedKVCache(P)
    ca.initialize(inp["k"], inp["v"])
    cb.initialize(inp["k"], inp["v"])
    ga = DecodeStepGraph(ca, Hq, "topk", token_budget=256, alpha=1.5, niter=2)
    gb = DecodeStepGraph(cb, Hq, "topk", token_budget=256, alpha=1.5, niter=2)
    io = gb.pinned_io()
    for i, (q, kn, vn) in enumerate(toks):
        want = ga.step(q, kn, vn).clone()
        assert ca.last_topk_selection.get("stream", False)
        io["q"].copy_(q)
        io["k_new"].copy_(kn)
        io["v_new"].copy_(vn)
        got = gb.step_pinned()
        torch.cuda.current_stream().synchronize()
        assert cb.last_topk_selection.get("stream", False)
        assert torch.equal(got, want.cpu()), i
    assert cb.device_status() == 0


def test_problems_that_do_not_fit_take_the_general_path():
    import entmaxkv_b200 as E
    from entmaxkv_b200 import _lib
    lib = _lib.load()
    inp = H.to_cuda(H.cpu_inputs(1, 4, 4, 128, 300, torch.float16, seed=5))
    c = E.PagedKVCache(16)
    c.initialize(inp["k"], inp["v"])
    d = c.desc()
    assert lib.ekv_topk_decode_stream_supported(C.byref(d), 4, 64, c.capacity, 2) == 2           # fits, too few heads to pay
    for bad in (dict(D=64), dict(P=8), dict(dt=torch.float32)):                                  # shapes its tiles do not cover
        x = H.to_cuda(H.cpu_inputs(1, 4, 4, bad.get("D", 128), 300, bad.get("dt", torch.float16), seed=5,
                                   page_size=bad.get("P", 16)))
        cx = E.PagedKVCache(bad.get("P", 16))
        cx.initialize(x["k"], x["v"])
        assert lib.ekv_topk_decode_stream_supported(C.byref(cx.desc()), 4, 64, cx.capacity, 2) == 0
    assert lib.ekv_topk_decode_stream_supported(C.byref(d), 4, 16 * 300, 16 * 4000, 2) == 0      # more kept tokens than score slots
    assert lib.ekv_topk_decode_stream_supported(C.byref(d), 3, 64, c.capacity, 2) == 0           # heads not a multiple of KV heads
    out = torch.zeros_like(inp["q"])
    E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, 64, alpha=1.5, niter=2)
    assert not c.last_topk_selection.get("stream", False)           # default: small problems stay on the other routes
