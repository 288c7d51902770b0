"""Block-table (non-contiguous) KV layout against the dense layout (run on a B200: ``-m gpu``).

``PagedKVCache(page_size, block_table=True)`` keeps K and V as a pool of physical blocks behind a
per-sequence block table.  Everything a decode step computes must be the bits of the dense cache:
the cache statistics after ``initialize`` and ``append`` (the kernels read and write through the
table), the selected page sets (page numbers, not block ids) and the outputs of both decode steps,
across page boundaries, for ragged batches, for the group-shared route, after the cache has grown,
and replayed from a captured graph.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

from tests import _harness as H

DT = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}

CASES = [
    # mode, B, Hq, Hkv, D, S or lengths, P, dtype, order
    ("topk", 2, 4, 4, 64, 1000, 16, "fp16", "interleaved"),
    ("topk", 3, 8, 2, 128, [700, 333, 512], 16, "bf16", "random"),
    ("topk", 1, 2, 2, 64, 300, 8, "fp32", "random"),
    ("gaussian", 2, 8, 2, 128, 3000, 16, "bf16", "interleaved"),       # GQA 4: group-shared K pass
    ("gaussian", 3, 4, 4, 64, [2048, 1500, 900], 16, "fp16", "random"),
    ("gaussian", 1, 16, 2, 128, 2500, 16, "bf16", "random"),           # GQA 8: per-head K pass
]


@pytest.mark.parametrize("case", CASES, ids=[f"case{i}" for i in range(len(CASES))])
def test_block_table_cache_equals_dense_cache(case, topk_path):
    import entmaxkv_b200 as E
    mode, B, Hq, Hkv, D, S, P, name, order = case
    dt = DT[name]
    lens = S if isinstance(S, list) else [S] * B
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, max(lens), dt, seed=500 + max(lens), needle_pages=(3, 11), page_size=P))
    g = torch.Generator().manual_seed(7)
    toks = [(torch.randn(B, Hkv, 1, D, generator=g).to(dt).cuda(), torch.randn(B, Hkv, 1, D, generator=g).to(dt).cuda())
            for _ in range(P + 3)]                          # crosses a page boundary in every sequence
    caches = [E.PagedKVCache(P, capacity=max(lens) + 8),                       # too small: both grow on the way
              E.PagedKVCache(P, capacity=max(lens) + 8, block_table=True, block_order=order)]
    outs = []
    for c in caches:
        c.initialize(inp["k"], inp["v"], seq_lens=lens)
        res = []
        for kn, vn in toks:
            out = torch.zeros_like(inp["q"])
            if mode == "topk":
                E.sparse_attention_decode_paged(inp["q"], c, kn, vn, out, 16 * P, alpha=1.5, niter=2)
                sel = c.last_topk_selection
            else:
                E.sparse_attention_decode_gaussian_aware_entmax(inp["q"], c, kn, vn, out, alpha=1.5, append_cache=True)
                sel = c.last_gaussian_selection
            res.append((out.clone(), sel["num_selected"].clone(), sel["page_indices"].clone()))
        torch.cuda.synchronize()
        assert c.device_status() == 0
        outs.append(res)
    dense, blocks = caches
    assert blocks.block_mode and blocks.capacity == dense.capacity > max(lens) + 8
    table = blocks._table[:, :blocks.num_pages]
    assert table.unique().numel() == table.numel(), "every page has a block of its own"
    assert not torch.equal(table[0, 1:] - table[0, :-1], torch.ones_like(table[0, 1:])), "blocks are not contiguous"
    for nm in ("k_min", "k_max", "k_mean", "k_std"):
        assert torch.equal(getattr(dense, nm), getattr(blocks, nm)), nm
    for b, n in enumerate(dense.host_seq_lens):          # rows beyond a sequence's length are padding
        assert torch.equal(dense.k_cache[b, :, :n], blocks.k_cache[b, :, :n])
        assert torch.equal(dense.v_cache[b, :, :n], blocks.v_cache[b, :, :n])
    for step, ((o0, n0, p0), (o1, n1, p1)) in enumerate(zip(*outs)):
        assert torch.equal(n0, n1), step
        width = torch.arange(p0.shape[-1], device="cuda")[None, None, :] < n0[:, :, None]
        assert torch.equal(p0[width], p1[width]), step          # page numbers, not block ids
        assert torch.equal(o0, o1), f"step {step}: outputs differ"


def test_block_table_step_replays_from_a_graph():
    import entmaxkv_b200 as E
    from entmaxkv_b200.graph import DecodeStepGraph
    B, Hq, Hkv, D, S, P = 2, 8, 2, 128, 900, 16
    inp = H.to_cuda(H.cpu_inputs(B, Hq, Hkv, D, S, torch.bfloat16, seed=611, needle_pages=(4,)))
    g = torch.Generator().manual_seed(8)
    toks = [tuple(torch.randn(B, n, 1, D, generator=g).to(torch.bfloat16).cuda() for n in (Hq, Hkv, Hkv)) for _ in range(20)]
    for mode in ("topk", "gaussian"):
        eager = E.PagedKVCache(P, block_table=True, block_order="random")
        replay = E.PagedKVCache(P, block_table=True, block_order="random")
        eager.initialize(inp["k"], inp["v"])
        replay.initialize(inp["k"], inp["v"])
        graph = DecodeStepGraph(replay, Hq, mode, token_budget=256, alpha=1.5, niter=2)
        out = torch.zeros_like(inp["q"])
        for q, kn, vn in toks:
            if mode == "topk":
                E.sparse_attention_decode_paged(q, eager, kn, vn, out, 256, alpha=1.5, niter=2)
            else:
                E.sparse_attention_decode_gaussian_aware_entmax(q, eager, kn, vn, out, alpha=1.5, append_cache=True)
            assert torch.equal(graph.step(q, kn, vn), out)


def test_block_table_refuses_alibi():
    import entmaxkv_b200 as E
    inp = H.to_cuda(H.cpu_inputs(1, 2, 2, 64, 100, torch.float16, seed=612))
    c = E.PagedKVCache(16, block_table=True)
    c.initialize(inp["k"], inp["v"])
    out = torch.zeros_like(inp["q"])
    slopes = torch.tensor([0.5, 0.25], device="cuda")
    with pytest.raises(ValueError):
        E.sparse_attention_decode_paged(inp["q"], c, inp["k_new"], inp["v_new"], out, 64, alibi_slopes=slopes)
