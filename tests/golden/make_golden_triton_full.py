"""Generate ``ref_triton_topk_32k.npz``: the reference's Triton path on benchmark configuration 2 at FULL size.

B=1, 32 heads (MHA), head_dim 128, 32 768 tokens + the step's token, fp16, page size 16, budget 2048, alpha 1.5,
niter 2: the largest benchmark configuration the reference can address (its kernels index the cache with 32-bit
offsets).  Run on a CUDA machine with an UNMODIFIED copy of the reference importable:

    PYTHONPATH=baseline/_ref python tests/golden/make_golden_triton_full.py [output.npz]

Inputs are the benchmark's own tensors (``entmaxkv_b200.workloads.make_inputs``: a counter-based generator that
yields the same bits on CPU and CUDA; only the workload's name is stored).  Stored: page scores (fp16), page
tables, thresholds, outputs - every array comes from the reference's own functions.
"""

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from entmaxkv.kv_cache import PagedKVCache                                            # noqa: E402
from entmaxkv.attention_topk import sparse_attention_decode_paged                     # noqa: E402
from entmaxkv.kernels.adadecode_paged import sparse_attention_decode_paged as paged_kernel  # noqa: E402
from entmaxkv_b200.workloads import CONFIGS, make_inputs                               # noqa: E402

OUT = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                         "ref_triton_topk_32k.npz")


def main():
    assert torch.cuda.is_available()
    w = CONFIGS["topk_32k"]
    inp = make_inputs(w, "cuda")
    B, H, P = w.batch, w.q_heads, w.page_size
    c = PagedKVCache(page_size=P)
    c.initialize(inp["k"], inp["v"])
    c.append(inp["k_new"], inp["v_new"])
    S1 = w.context + 1
    total_pages = (S1 + P - 1) // P
    k_sel = min(w.token_budget // P, total_pages - 1)
    T = k_sel * P + (S1 - (total_pages - 1) * P)
    seqlens = torch.full((B,), T, device="cuda", dtype=torch.int32)
    qlens = torch.full((B,), S1, device="cuda", dtype=torch.int32)
    out = torch.zeros_like(inp["q"])
    sparse_attention_decode_paged(q=inp["q"], kv_cache=c, k_new=inp["k_new"], v_new=inp["v_new"], out=out,
                                  token_budget=w.token_budget, cache_seqlens=seqlens, q_seqlens=qlens,
                                  alpha=w.alpha, niter=2, append_cache=False)
    scores = c.estimate_page_criticality(inp["q"], use_triton=True, q_pos=S1 - 1, exclude_last_page=True)
    pages = c._page_indices_buf.clone()
    taus = torch.zeros(B, H, device="cuda", dtype=torch.float32)
    out2 = torch.zeros_like(out)
    paged_kernel(q=inp["q"], k_cache=c.k_cache, v_cache=c.v_cache, out=out2,
                 cache_seqlens=seqlens[:, None].expand(B, H), page_indices=pages, page_size=P, alpha=w.alpha,
                 niter=2, q_seqlens=qlens, taus_out=taus)
    torch.cuda.synchronize()
    assert torch.equal(out, out2), "the wrapper and the kernel called by hand disagree"
    import triton
    g = {
        "workload": np.array(w.name),
        "scores_f16": scores.detach().to(torch.float16).cpu().numpy(),
        "pages": pages[:, :, :k_sel + 1].cpu().numpy().astype(np.int32),
        "tau": taus.cpu().numpy(),
        "out": out.detach().float().cpu().numpy(),
        "T": np.int64(T),
        "versions": np.array([torch.__version__, triton.__version__, torch.cuda.get_device_name(0)]),
    }
    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
