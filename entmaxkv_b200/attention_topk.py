"""Decode step with top-k page selection (drop-in for entmaxkv/attention_topk.py:8-100).

append -> key-range page scores -> deterministic top-k + index packing -> paged
entmax decode; four kernel launches, no host synchronisation.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _lib
from .kv_cache import PagedKVCache


def _check_q_out(q, out, kv_cache):
    _lib.require_cuda(q, out)
    B, Hkv, _, D = kv_cache._k.shape
    if q.dim() != 4 or q.shape[0] != B or q.shape[2] != 1 or q.shape[3] != D:
        raise ValueError(f"q must be [{B}, H_q, 1, {D}]")
    if q.shape[1] % Hkv:
        raise ValueError("query heads must be a multiple of KV heads")
    if q.dtype != kv_cache._k.dtype:
        raise ValueError("q dtype differs from the cache dtype")
    if q.stride(-1) != 1:
        raise ValueError("q must be contiguous along head_dim")
    if out is not None:
        if out.shape != q.shape or out.dtype != q.dtype or out.stride(-1) != 1:
            raise ValueError("out must match q in shape and dtype and be contiguous along head_dim")


def _alibi_args(alibi_slopes, q_seqlens, B, Hq, device):
    """(slopes fp32 [H_q] contiguous, query positions int32 [B] or None) for the ALiBi entry points.
    The query position is ``q_seqlens - 1`` as in the reference's kernels; without ``q_seqlens``
    the kernels use the position of the token just appended."""
    _lib.require_cuda(alibi_slopes)
    slopes = alibi_slopes.to(device=device, dtype=torch.float32).reshape(-1).contiguous()
    if slopes.numel() != Hq:
        raise ValueError(f"alibi_slopes must hold one slope per query head ({Hq})")
    q_pos = None
    if q_seqlens is not None:
        _lib.require_cuda(q_seqlens)
        if q_seqlens.numel() != B:
            raise ValueError("q_seqlens must be [B]")
        q_pos = (q_seqlens.to(torch.int32).reshape(-1) - 1).contiguous()
    return slopes, q_pos


def _score_and_select(q, kv_cache: PagedKVCache, token_budget: int, cache_seqlens, alibi=None):
    """Launch scoring + top-k; returns (scores, page_indices, num_selected, tok_counts).
    ``alibi``: (slopes, q_pos) of ``_alibi_args`` or None."""
    lib = _lib.load()
    B, Hq = q.shape[0], q.shape[1]
    P = kv_cache.page_size
    # Grids and buffers are sized by the cache capacity, not by the current length: the
    # kernels read the true lengths from device memory, and launch parameters that do
    # not change from step to step let a whole step be replayed as one CUDA graph.
    S = kv_cache.capacity
    max_pages = kv_cache.page_capacity
    k_max = min(token_budget // P, max(max_pages - 1, 0))
    score_stride = max(kv_cache.page_capacity, 1)
    scores = kv_cache.scratch("topk_scores", (B, Hq, score_stride), q.dtype)
    page_indices = kv_cache.scratch("topk_pages", (B, Hq, k_max + 1), torch.int32)
    num_selected = kv_cache.scratch("topk_counts", (B, Hq), torch.int32)
    tok_counts = kv_cache.scratch("topk_tokens", (B, Hq), torch.int32)
    n_items = B * Hq * lib.ekv_work_items_per_head((k_max + 1) * P)
    work_items = kv_cache.scratch("topk_work", (n_items,), torch.int64)
    us_ptr, usb, ush = None, 0, 0
    if cache_seqlens is not None:
        _lib.require_cuda(cache_seqlens)
        if cache_seqlens.dtype != torch.int32:
            raise ValueError("cache_seqlens must be int32")
        if cache_seqlens.dim() == 1 and cache_seqlens.shape[0] == B:
            us_ptr, usb, ush = cache_seqlens.data_ptr(), cache_seqlens.stride(0), 0
        elif cache_seqlens.dim() == 2 and tuple(cache_seqlens.shape) == (B, kv_cache._k.shape[1]):
            us_ptr, usb, ush = cache_seqlens.data_ptr(), cache_seqlens.stride(0), cache_seqlens.stride(1)
        else:
            raise ValueError("cache_seqlens must be [B] or [B, H_kv]")
    if alibi is None:
        _lib.check(lib.ekv_topk_select(
            C.byref(kv_cache.desc()), q.data_ptr(), q.stride(0), q.stride(1), Hq, int(token_budget), S,
            scores.data_ptr(), score_stride, page_indices.data_ptr(), k_max + 1,
            num_selected.data_ptr(), tok_counts.data_ptr(), us_ptr, usb, ush, work_items.data_ptr(),
            _lib.stream_ptr()), "ekv_topk_select")
    else:
        slopes, q_pos = alibi
        _lib.check(lib.ekv_page_scores_alibi(
            C.byref(kv_cache.desc()), q.data_ptr(), q.stride(0), q.stride(1), Hq, S, scores.data_ptr(),
            score_stride, slopes.data_ptr(), _lib.ptr(q_pos), _lib.stream_ptr()), "ekv_page_scores_alibi")
        _lib.check(lib.ekv_topk_pack(
            C.byref(kv_cache.desc()), Hq, int(token_budget), S, scores.data_ptr(), score_stride,
            page_indices.data_ptr(), k_max + 1, num_selected.data_ptr(), tok_counts.data_ptr(),
            us_ptr, usb, ush, work_items.data_ptr(), _lib.stream_ptr()), "ekv_topk_pack")
    return scores, page_indices, num_selected, tok_counts, work_items


def _event_array(events):
    """ctypes array of the raw cudaEvent_t handles of torch events (created on first record)."""
    if not events:
        return None
    for e in events:
        if e.cuda_event == 0:          # lazily created: a record() on the current stream creates it
            e.record()
    return (C.c_void_p * len(events))(*[e.cuda_event for e in events])


def _decode_workspace(kv_cache: PagedKVCache, B, Hq, D, max_tokens):
    lib = _lib.load()
    nbytes = lib.ekv_decode_workspace_bytes(B, Hq, D, max_tokens)
    key = ("decode_ws", nbytes)
    ws = kv_cache._scratch.get(key)
    if ws is None:
        for old in [k for k in kv_cache._scratch if k[0] == "decode_ws"]:
            del kv_cache._scratch[old]
        ws = torch.empty(nbytes, dtype=torch.uint8, device=kv_cache._k.device)
        _lib.check(lib.ekv_decode_workspace_reset(ws.data_ptr(), B, Hq, _lib.stream_ptr()),
                   "ekv_decode_workspace_reset")
        kv_cache._scratch[key] = ws
    return ws


def _paged_decode(q, kv_cache, out, page_indices, tok_counts, max_tokens, alpha, tau_mode, niter,
                  tau, work_items, work_total=None, stage_events=None, alibi=None):
    """K pass, tau, V pass and output over the work list ``work_items`` (int64 device tensor).

    ``stage_events``: optional list of three ``torch.cuda.Event(enable_timing=True)`` recorded
    after the K pass, after the tau kernel and after the V pass."""
    lib = _lib.load()
    B, Hq, _, D = q.shape
    ws = _decode_workspace(kv_cache, B, Hq, D, max_tokens)
    desc = C.byref(kv_cache.desc())
    st = _lib.stream_ptr()
    wl, n_items, wt = work_items.data_ptr(), work_items.numel(), _lib.ptr(work_total)
    if alibi is None:
        _lib.check(lib.ekv_decode(
            desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, page_indices.data_ptr(),
            page_indices.stride(1), tok_counts.data_ptr(), max_tokens, float(alpha), tau_mode, int(niter),
            tau.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), wl, n_items, wt,
            ws.data_ptr(), ws.numel(), _event_array(stage_events), st), "ekv_decode")
    else:
        slopes, q_pos = alibi
        _lib.check(lib.ekv_decode_alibi(
            desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, page_indices.data_ptr(),
            page_indices.stride(1), tok_counts.data_ptr(), max_tokens, float(alpha), tau_mode, int(niter),
            tau.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), wl, n_items, wt,
            ws.data_ptr(), ws.numel(), _event_array(stage_events), slopes.data_ptr(), _lib.ptr(q_pos), st),
            "ekv_decode_alibi")
    return ws


def _fused_small_step(q, kv_cache: PagedKVCache, out, token_budget, alpha, niter, taus_out) -> bool:
    """Scores, selection, tau and output of a small problem in ONE launch (a cluster of thread blocks per
    query head); returns False, having done nothing, when the problem does not fit that kernel or
    ``EKV_FUSED_SMALL=0`` is set.  Results: page scores and page tables bit-identical to the general
    path's, tau and output equal to rounding."""
    if os.environ.get("EKV_FUSED_SMALL", "1") == "0":
        return False
    lib = _lib.load()
    B, Hq = q.shape[0], q.shape[1]
    P = kv_cache.page_size
    S = kv_cache.capacity
    desc = kv_cache.desc()
    if not lib.ekv_topk_decode_fused_supported(C.byref(desc), Hq, int(token_budget), S, int(niter)):
        return False
    k_max = min(token_budget // P, max(kv_cache.page_capacity - 1, 0))
    score_stride = max(kv_cache.page_capacity, 1)
    scores = kv_cache.scratch("topk_scores", (B, Hq, score_stride), q.dtype)
    page_indices = kv_cache.scratch("topk_pages", (B, Hq, k_max + 1), torch.int32)
    num_selected = kv_cache.scratch("topk_counts", (B, Hq), torch.int32)
    tok_counts = kv_cache.scratch("topk_tokens", (B, Hq), torch.int32)
    tau = taus_out if taus_out is not None else kv_cache.scratch("tau", (B, Hq), torch.float32)
    _lib.check(lib.ekv_topk_decode_fused(
        C.byref(desc), q.data_ptr(), q.stride(0), q.stride(1), Hq, int(token_budget), S, float(alpha),
        int(niter), scores.data_ptr(), score_stride, page_indices.data_ptr(), k_max + 1,
        num_selected.data_ptr(), tok_counts.data_ptr(), tau.data_ptr(), out.data_ptr(), out.stride(0),
        out.stride(1), kv_cache._ctl.data_ptr(), _lib.stream_ptr()), "ekv_topk_decode_fused")
    kv_cache.last_num_selected_per_head = num_selected
    kv_cache.last_topk_selection = dict(scores=scores, page_indices=page_indices,
                                        num_selected=num_selected, tok_counts=tok_counts, work_items=None,
                                        fused=True)
    return True


def _stream_step(q, kv_cache: PagedKVCache, out, token_budget, alpha, niter, taus_out, on_launch=None) -> bool:
    """The step for MANY heads: the score sweep, then ONE persistent kernel in which every SM streams the
    selected K pages of its current head while a second warp group solves tau and gathers the value rows of the
    previous head and selects the pages of the head after next (``ekv_topk_decode_stream``).  Returns False,
    having done nothing, when the problem does not fit or is too small to pay off; ``EKV_STREAM_TOPK=0`` turns
    the route off, ``=1`` takes it whenever the problem fits.  ``on_launch(name)`` is called after the score sweep
    has been launched (per-kernel timing)."""
    mode = os.environ.get("EKV_STREAM_TOPK", "")
    if mode == "0":
        return False
    lib = _lib.load()
    B, Hq = q.shape[0], q.shape[1]
    P = kv_cache.page_size
    S = kv_cache.capacity
    desc = kv_cache.desc()
    fit = lib.ekv_topk_decode_stream_supported(C.byref(desc), Hq, int(token_budget), S, int(niter))
    if fit == 0 or (fit == 2 and mode != "1"):
        return False
    k_max = min(token_budget // P, max(kv_cache.page_capacity - 1, 0))
    # score rows padded to whole groups of 32 pages (64-byte aligned 16-bit rows): the selection keeps a row's keys
    # in registers, 32 consecutive pages per thread
    score_stride = (max(kv_cache.page_capacity, 1) + 31) // 32 * 32
    scores = kv_cache.scratch("topk_scores_padded", (B, Hq, score_stride), q.dtype)
    page_indices = kv_cache.scratch("topk_pages", (B, Hq, k_max + 1), torch.int32)
    num_selected = kv_cache.scratch("topk_counts", (B, Hq), torch.int32)
    tok_counts = kv_cache.scratch("topk_tokens", (B, Hq), torch.int32)
    support = kv_cache.scratch("topk_support", (B, Hq), torch.int32)
    zbuf = kv_cache.scratch("stream_scores", (lib.ekv_topk_decode_stream_scratch_bytes(),), torch.uint8)
    tau = taus_out if taus_out is not None else kv_cache.scratch("tau", (B, Hq), torch.float32)
    st = _lib.stream_ptr()
    _lib.check(lib.ekv_page_scores(C.byref(desc), q.data_ptr(), q.stride(0), q.stride(1), Hq, S, scores.data_ptr(),
                                   score_stride, st), "ekv_page_scores")
    if on_launch:
        on_launch("page_score_kernel")
    _lib.check(lib.ekv_topk_decode_stream(
        C.byref(desc), q.data_ptr(), q.stride(0), q.stride(1), Hq, int(token_budget), S, float(alpha), int(niter),
        scores.data_ptr(), score_stride, page_indices.data_ptr(), k_max + 1, num_selected.data_ptr(),
        tok_counts.data_ptr(), tau.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), support.data_ptr(),
        zbuf.data_ptr(), zbuf.numel(), kv_cache._ctl.data_ptr(), st), "ekv_topk_decode_stream")
    kv_cache.last_num_selected_per_head = num_selected
    kv_cache.last_topk_selection = dict(scores=scores, page_indices=page_indices, num_selected=num_selected,
                                        tok_counts=tok_counts, work_items=None, stream=True, support=support)
    return True


def sparse_attention_decode_paged(
    q: torch.Tensor,
    kv_cache: PagedKVCache,
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    out: torch.Tensor,
    token_budget: int,
    cache_seqlens: Optional[torch.Tensor] = None,
    q_seqlens: Optional[torch.Tensor] = None,
    alibi_slopes: torch.Tensor = None,
    alpha: float = 1.5,
    splits: int = 32,
    niter: int = 10,
    append_cache: bool = True,
    use_triton_criticality: bool = True,
    workspace: dict = None,
    taus_out: Optional[torch.Tensor] = None,
):
    """Decode-phase entmax attention over the top-k pages (attention_topk.py:8-100).

    q [B,H_q,1,D]; ``out`` (same shape) is written in place and returned.  The
    ``token_budget // page_size`` highest-scoring pages (ties: lower page id) plus the
    in-progress last page are attended; ``cache_seqlens`` ([B] or [B,H_kv] int32, the
    compacted length ``k_sel*P + last_page_tokens``) is honoured when given and
    computed on the device when omitted.  ``splits``, ``use_triton_criticality`` and
    ``workspace`` are accepted for signature compatibility and have no effect.
    ``alibi_slopes`` ([H_q] fp32): each page's score gets ``slope * (last position of the page -
    query position)`` and each kept token's logit ``(alpha-1) * slope * (its position - query
    position)``; the query position is ``q_seqlens - 1`` (default: the token just appended).
    With GQA every query head selects its own pages over the shared KV head.  ``taus_out``
    ([B,H_q] fp32, optional) receives the thresholds.
    """
    if kv_cache._k is None:
        raise RuntimeError("kv_cache is not initialised")
    if not alpha > 1.0:
        raise ValueError("alpha must be > 1")
    _check_q_out(q, out, kv_cache)
    if append_cache:
        kv_cache.append(k_new, v_new)
    B, Hq, _, D = q.shape
    P = kv_cache.page_size
    alibi = None if alibi_slopes is None else _alibi_args(alibi_slopes, q_seqlens, B, Hq, q.device)
    if taus_out is not None:
        if tuple(taus_out.shape) != (B, Hq) or taus_out.dtype != torch.float32 or not taus_out.is_contiguous():
            raise ValueError("taus_out must be a contiguous fp32 [B, H_q] tensor")
    if alibi is None and cache_seqlens is None and _fused_small_step(q, kv_cache, out, token_budget, alpha,
                                                                    niter, taus_out):
        return out
    if alibi is None and cache_seqlens is None and _stream_step(q, kv_cache, out, token_budget, alpha, niter,
                                                                taus_out):
        return out
    scores, page_indices, num_selected, tok_counts, work_items = _score_and_select(
        q, kv_cache, token_budget, cache_seqlens, alibi)
    kv_cache.last_num_selected_per_head = num_selected
    kv_cache.last_topk_selection = dict(scores=scores, page_indices=page_indices,
                                        num_selected=num_selected, tok_counts=tok_counts,
                                        work_items=work_items)
    if kv_cache.block_mode:      # the decode addresses K/V by physical block id
        if alibi is not None:
            raise ValueError("ALiBi needs token positions and is not available on a block-table cache")
        page_indices = kv_cache.translate(page_indices, num_selected)
    k_max = page_indices.shape[2] - 1
    max_tokens = (k_max + 1) * P
    tau = taus_out if taus_out is not None else kv_cache.scratch("tau", (B, Hq), torch.float32)
    if k_max >= kv_cache.page_capacity - 1 and cache_seqlens is None and alibi is None:
        # the budget covers the cache whatever its length: dense entmax attention.  Every head of a GQA group
        # then reads the same rows, so where the group-shared K pass exists it fetches them once per group
        from .attention_gaussian import grouped_decode, grouped_enabled
        if grouped_enabled(q, kv_cache):
            sel = dict(page_indices=kv_cache.last_topk_selection["page_indices"], num_selected=num_selected, tau=tau)
            kv_cache.last_group_tables = grouped_decode(q, kv_cache, out, sel, alpha, _lib.TAU_EXACT, niter)
            return out
    _paged_decode(q, kv_cache, out, page_indices, tok_counts, max_tokens, alpha, _lib.TAU_EXACT,
                  niter, tau, work_items, alibi=alibi)
    return out
