"""Oracle: key-range page scores and top-k page selection (test infrastructure).

Score (entmaxkv/kernels/page_criticality.py:72-104, kv_cache.py:150-153):
``score[b,h,p] = sum_d max(q_d*kmin[p,d], q_d*kmax[p,d])`` over every page but
the in-progress last one, no 1/sqrt(D) factor, fp32 accumulation, result
rounded to the query dtype (page_criticality.py:168).  ``max(q*kmin, q*kmax)``
equals ``q*kmax`` for ``q >= 0`` and ``q*kmin`` otherwise
(page_criticality.py:92).

Selection (entmaxkv/attention_topk.py:42-71): the ``min(budget // P, Np-1)``
highest-scoring pages plus the last page.  ``torch.topk`` leaves the order of
tied scores open; this oracle fixes it: score descending, page index ascending.
Selected ids are reported in ascending page order (the set is the contract;
the order only changes floating-point summation order in the decode).

Summation order contract for 16-bit inputs (bit-exact against the CUDA
kernel, because a product of two fp16 or two bf16 numbers is exact in fp32):
the D products of a page are split into groups of ``16 bytes / element size``
consecutive elements; each group is summed left to right starting from 0;
the group sums are then combined by a halving tree (first half + second half,
repeatedly).
"""

from __future__ import annotations

import torch


def _lane_tree_sum(prod: torch.Tensor, elems_per_lane: int) -> torch.Tensor:
    """Sum the last axis in the fixed order described in the module docstring."""
    *lead, D = prod.shape
    lanes = D // elems_per_lane
    x = prod.reshape(*lead, lanes, elems_per_lane)
    acc = torch.zeros(*lead, lanes, dtype=torch.float32)
    for j in range(elems_per_lane):
        acc = acc + x[..., j]
    while acc.shape[-1] > 1:
        h = acc.shape[-1] // 2
        acc = acc[..., :h] + acc[..., h:]
    return acc[..., 0]


def criticality_scores(q: torch.Tensor, k_min: torch.Tensor, k_max: torch.Tensor,
                       n_scored: int | None = None, alibi_slopes: torch.Tensor | None = None,
                       seq_len: int | None = None, page_size: int = 16,
                       q_pos: int | None = None) -> torch.Tensor:
    """q [B,Hq,1,D]; k_min/k_max [B,Hkv,Np,D] -> scores [B,Hq,n_scored] in q.dtype.

    ``n_scored`` defaults to Np-1 (the last page is excluded, attention_topk.py:46-52).
    With ``alibi_slopes`` ([Hq] fp32) the page bonus ``slope * (min((p+1)*P-1, seq_len-1) -
    q_pos)`` is added in fp32 before rounding (kernels/page_criticality.py:99-101,158-165;
    kv_cache.py:155-163); ``q_pos`` defaults to ``seq_len - 1``.
    """
    B, Hq, _, D = q.shape
    Hkv, Np = k_min.shape[1], k_min.shape[2]
    G = Hq // Hkv
    if n_scored is None:
        n_scored = Np - 1
    qf = q[:, :, 0, :].to(torch.float32)                      # [B,Hq,D]
    lo = k_min[:, :, :n_scored].to(torch.float32).repeat_interleave(G, dim=1)
    hi = k_max[:, :, :n_scored].to(torch.float32).repeat_interleave(G, dim=1)
    bound = torch.where(qf[:, :, None, :] >= 0, hi, lo)       # [B,Hq,n,D]
    prod = qf[:, :, None, :] * bound
    epl = 16 // q.element_size()
    s = _lane_tree_sum(prod, epl)
    if alibi_slopes is not None:
        if q_pos is None:
            q_pos = seq_len - 1
        last_pos = torch.clamp((torch.arange(n_scored, dtype=torch.float32) + 1) * page_size - 1,
                               max=float(seq_len - 1))
        bonus = alibi_slopes.to(torch.float32).reshape(1, Hq, 1) * (last_pos - float(q_pos)).reshape(1, 1, -1)
        s = s + bonus
    return s.to(q.dtype)


def topk_page_sets(scores: torch.Tensor, k_sel: int):
    """Stable top-k per (b,h): returns int32 [B,H,k_sel] page ids, ascending.

    Ties at the boundary go to the lower page index.
    """
    s = scores.to(torch.float32)
    # stable descending sort == stable ascending sort of the negated values
    order = torch.sort(-s, dim=-1, stable=True).indices[..., :k_sel]
    return torch.sort(order, dim=-1).values.to(torch.int32)


def boundary_tied_pages(scores: torch.Tensor, k_sel: int):
    """Per (b,h): boolean mask of pages whose score equals the k-th largest score.

    Two correct selections may differ only inside this class.
    """
    s = scores.to(torch.float32)
    if k_sel <= 0 or k_sel > s.shape[-1]:
        return torch.zeros_like(s, dtype=torch.bool)
    kth = torch.sort(s, dim=-1, descending=True).values[..., k_sel - 1:k_sel]
    return s == kth


def topk_select_and_pack(scores: torch.Tensor, token_budget: int, page_size: int,
                         seq_len: int):
    """Page table and compacted token count of the top-k decode step.

    Returns (page_indices int32 [B,H,k_sel+1] with the last page in the final
    column, cache_seqlen int) following attention_topk.py:39-71 and the
    compacted-length convention ``k_sel*P + last_page_tokens``
    (tests/test_topk.py:84-89).
    """
    P = page_size
    total_pages = (seq_len + P - 1) // P
    k_sel = min(token_budget // P, total_pages - 1)
    ids = topk_page_sets(scores, k_sel)
    last = torch.full((*ids.shape[:-1], 1), total_pages - 1, dtype=torch.int32)
    last_tokens = seq_len - (total_pages - 1) * P
    return torch.cat([ids, last], dim=-1), k_sel * P + last_tokens
