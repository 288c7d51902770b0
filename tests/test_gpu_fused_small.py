"""The one-launch top-k step of small problems against the general kernels and the oracle.

A problem that leaves most SMs idle (a few dozen query heads) runs scores, selection, tau and output in one
cluster kernel; page scores and page tables must be bit-identical to the general path's, tau and the output
equal to rounding, and a problem that does not fit must fall back without a trace.
"""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from tests import _harness as H

pytestmark = pytest.mark.gpu

DT = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def _step(E, inp, P, budget, alpha, niter, lens, fused, block_table=False, capacity=None):
    os.environ["EKV_FUSED_SMALL"] = "1" if fused else "0"
    try:
        c = (E.PagedKVCache(P, capacity, block_table=True, block_order="random") if block_table
             else E.PagedKVCache(P, capacity))
        c.initialize(inp["k"], inp["v"], seq_lens=lens)
        out = torch.zeros_like(inp["q"])
        B, Hq = inp["q"].shape[:2]
        taus = torch.zeros(B, Hq, dtype=torch.float32, device="cuda")
        E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, budget, alpha=alpha,
                                        niter=niter, taus_out=taus)
        torch.cuda.synchronize()
        assert c.device_status() == 0
        sel = c.last_topk_selection
        assert bool(sel.get("fused", False)) == fused
        return c, out, taus, sel
    finally:
        os.environ.pop("EKV_FUSED_SMALL", None)


CASES = [
    # B, Hq, Hkv, D, lengths, P, budget, dtype, alpha, niter, block table
    (1, 32, 8, 128, [4100], 16, 512, "bf16", 1.5, 2, False),          # the shape class of the 32k benchmark config
    (2, 8, 2, 128, [3000, 1700], 16, 256, "fp16", 1.5, 10, False),    # ragged rows, the wrapper's default niter
    (1, 4, 4, 64, [1500], 16, 128, "bf16", 2.0, 3, False),
    (1, 2, 2, 64, [777], 16, 160, "fp32", 1.5, 3, False),
    (1, 4, 4, 128, [520], 8, 64, "bf16", 1.5, 2, False),              # page size 8
    (1, 4, 4, 64, [600], 16, 96, "fp16", 1.75, 4, False),             # general alpha
    (1, 4, 2, 64, [9], 16, 64, "fp16", 1.5, 2, False),                # one page: nothing to score
    (1, 4, 2, 64, [40], 16, 100000, "bf16", 1.5, 2, False),           # budget covers every page
    (1, 2, 2, 128, [16 * 700], 16, 8, "bf16", 1.5, 2, False),         # budget below one page: last page only
    (2, 8, 2, 128, [2600, 2600], 16, 256, "bf16", 1.5, 2, True),      # block-table cache
    (1, 1, 1, 128, [16 * 8192 + 3], 16, 4096, "bf16", 1.5, 2, False),  # the most pages the kernel scores
]


@pytest.mark.parametrize("case", CASES, ids=[f"case{i}" for i in range(len(CASES))])
def test_fused_step_equals_general_step(case):
    import entmaxkv_b200 as E
    B, Hq, Hkv, D, lens, P, budget, name, alpha, niter, bt = case
    dt = DT[name]
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, max(lens), dt, seed=900 + max(lens), needle_pages=(1, 5), page_size=P))
    cap = P * 8193 if max(lens) > 100000 else None          # 8192 scored pages and the last one, exactly
    c0, out0, tau0, sel0 = _step(E, inp, P, budget, alpha, niter, lens, fused=False, block_table=bt, capacity=cap)
    c1, out1, tau1, sel1 = _step(E, inp, P, budget, alpha, niter, lens, fused=True, block_table=bt, capacity=cap)
    assert torch.equal(sel0["num_selected"], sel1["num_selected"])
    assert torch.equal(sel0["tok_counts"], sel1["tok_counts"])
    for b, n in enumerate(lens):
        n_scored = (n + 1 + P - 1) // P - 1
        assert torch.equal(sel0["scores"][b, :, :n_scored], sel1["scores"][b, :, :n_scored]), "page scores: bit-identical"
    width = torch.arange(sel0["page_indices"].shape[-1], device="cuda")[None, None, :] < sel0["num_selected"][:, :, None]
    assert torch.equal(sel0["page_indices"][width], sel1["page_indices"][width]), "page tables: bit-identical"
    np.testing.assert_allclose(tau1.cpu().numpy(), tau0.cpu().numpy(), rtol=2e-5, atol=1e-6)
    tol = {"fp16": 2e-3, "bf16": 1.6e-2, "fp32": 2e-5}[name]
    assert (out1.float() - out0.float()).abs().max().item() <= tol


def test_fused_step_matches_oracle_directly():
    import entmaxkv_b200 as E
    B, Hq, Hkv, D, S, P, budget, alpha, niter = 1, 16, 4, 128, 5000, 16, 512, 1.5, 3
    inp = H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=4242, needle_pages=(7, 100, 250), page_size=P)
    ref = H.oracle_topk_step(inp, P, budget, alpha, niter)
    _, out, taus, sel = _step(E, H.to_cuda(inp), P, budget, alpha, niter, [S], fused=True)
    n_scored, width = ref["scores"].shape[-1], ref["pages"].shape[-1]
    assert torch.equal(sel["scores"][:, :, :n_scored].cpu(), ref["scores"])
    assert torch.equal(sel["page_indices"][:, :, :width].cpu(), ref["pages"])
    assert sel["tok_counts"].cpu().tolist() == [[ref["T"]] * Hq]
    np.testing.assert_allclose(taus.cpu().numpy(), ref["tau"], rtol=2e-4, atol=1e-6)
    np.testing.assert_allclose(taus.cpu().numpy(), ref["tau_true"], rtol=2e-4, atol=1e-6)
    assert np.abs(out[:, :, 0].float().cpu().numpy() - ref["out"]).max() <= 1.6e-2


def test_problems_that_do_not_fit_take_the_general_path():
    import entmaxkv_b200 as E
    from entmaxkv_b200 import _lib
    lib = _lib.load()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    inp = H.to_cuda(H.cpu_inputs(1, 4, 4, 64, 300, torch.float16, seed=5))
    c = E.PagedKVCache(16)
    c.initialize(inp["k"], inp["v"])
    d = c.desc()
    heads_fit = sms // 4
    assert lib.ekv_topk_decode_fused_supported(C.byref(d), 4, 64, c.capacity, 2) == 1
    assert lib.ekv_topk_decode_fused_supported(C.byref(d), 4 * (heads_fit // 4 + 1), 64, c.capacity, 2) == 0      # more clusters than SMs / 4
    assert lib.ekv_topk_decode_fused_supported(C.byref(d), 4, 64, 16 * 8194, 2) == 0    # more pages than key slots
    assert lib.ekv_topk_decode_fused_supported(C.byref(d), 4, 16 * 2048, 16 * 4000, 2) == 0   # more selected pages than slots
    assert lib.ekv_topk_decode_fused_supported(C.byref(d), 4, 16 * 1100, 16 * 4000, 2) == 0   # more tokens per block than score slots
    assert lib.ekv_topk_decode_fused_supported(C.byref(d), 3, 64, c.capacity, 2) == 0   # heads not a multiple of KV heads
    # a batch too large for one wave of clusters: the wrapper takes the general kernels
    B = sms // 4 // 4 + 1
    big = H.to_cuda(H.cpu_inputs(B, 4, 4, 64, 300, torch.float16, seed=6))
    cb = E.PagedKVCache(16)
    cb.initialize(big["k"], big["v"])
    out = torch.zeros_like(big["q"])
    E.sparse_attention_decode_paged(big["q"], cb, big["k_new"], big["v_new"], out, 64, alpha=1.5, niter=2)
    assert not cb.last_topk_selection.get("fused", False)
    # caller-provided lengths and ALiBi are the general path's
    out = torch.zeros_like(inp["q"])
    E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, 64, alpha=1.5, niter=2,
                                    alibi_slopes=torch.ones(4, device="cuda"))
    assert not c.last_topk_selection.get("fused", False)
    E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, 64, alpha=1.5, niter=2)
    assert c.last_topk_selection.get("fused", False)


def test_fused_step_replays_from_a_graph_and_follows_the_cache_as_it_grows():
    import entmaxkv_b200 as E
    from entmaxkv_b200.graph import DecodeStepGraph
    B, Hq, Hkv, D, S, P = 1, 8, 2, 128, 1000, 16
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=77, needle_pages=(4,)))
    g = torch.Generator().manual_seed(9)
    toks = [tuple(torch.randn(B, n, 1, D, generator=g).to(torch.bfloat16).cuda() for n in (Hq, Hkv, Hkv)) for _ in range(40)]
    eager, replay = E.PagedKVCache(P), E.PagedKVCache(P)
    eager.initialize(inp["k"], inp["v"])
    replay.initialize(inp["k"], inp["v"])
    graph = DecodeStepGraph(replay, Hq, "topk", token_budget=256, alpha=1.5, niter=2)
    out = torch.zeros_like(inp["q"])
    for q, kn, vn in toks:                                 # 40 tokens: pages complete and join the scored set
        E.sparse_attention_decode_paged(q, eager, kn, vn, out, 256, alpha=1.5, niter=2)
        assert eager.last_topk_selection.get("fused", False)
        assert torch.equal(graph.step(q, kn, vn), out)
