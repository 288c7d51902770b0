"""Decode step with Gaussian-aware page selection
(drop-in for entmaxkv/attention_gaussian.py:20-144).

append -> per-page score moments + single-Gaussian tau estimate -> threshold
selection, index packing and tau clamp -> paged entmax decode (K pass, tau,
V pass, output reduction); no host synchronisation.  For GQA groups of four or eight
(16-bit cache, head_dim 128) the K pass walks one page table per group - the
union of its heads' selections - instead of one per query head.
"""

from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache
from statistics import NormalDist
from typing import Optional

import torch

from . import _lib
from .attention_topk import _alibi_args, _check_q_out, _decode_workspace, _event_array, _paged_decode
from .kv_cache import PagedKVCache

_CHUNK = 256


@lru_cache(maxsize=None)
def _z_of_quantile(quantile: float, page_size: int) -> float:
    """Normal quantile of ``quantile ** (1/page_size)`` (selection_pack.py:238-239)."""
    return NormalDist().inv_cdf(quantile ** (1.0 / page_size))


def gaussian_select(q, kv_cache: PagedKVCache, alpha: float, excess_margin_fraction: float,
                    clamp_quantile: float, apply_clamp: bool, sigma_mean=None,
                    alibi=None, build_work_list: bool = True):
    """Moments sweep + selection (two launches).  Returns a dict of device tensors:
    mu, sigma [B,H,pages]; head_stats [B,H,4] = (mu_g, sigma_g, tau_hat, mean upper);
    page_indices, num_selected, tok_counts, tau_floor, cap_max, tau, work_list, work_total.
    ``build_work_list=False`` skips the per-head decode work list (its launch and memset): the
    group-shared decode does not walk it; ``work_list`` / ``work_total`` are then None.
    """
    lib = _lib.load()
    B, Hq = q.shape[0], q.shape[1]
    P, S = kv_cache.page_size, kv_cache.capacity   # launch bounds; true lengths are on the device
    pcap = kv_cache.page_capacity
    st = _lib.stream_ptr()
    desc = C.byref(kv_cache.desc())
    mu = kv_cache.scratch("g_mu", (B, Hq, pcap), torch.float32)
    sigma = kv_cache.scratch("g_sigma", (B, Hq, pcap), torch.float32)
    head_sums = kv_cache.scratch("g_head_sums", (B, Hq, 4), torch.float32)
    head_stats = kv_cache.scratch("g_head_stats", (B, Hq, 4), torch.float32)
    ws_bytes = lib.ekv_gaussian_workspace_bytes(B, Hq, pcap)
    gws = kv_cache.scratch("g_ws", (ws_bytes,), torch.uint8, zero=True)
    if alibi is None:
        _lib.check(lib.ekv_gaussian_moments(
            desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, S, 1, float(alpha), 1, mu.data_ptr(),
            sigma.data_ptr(), pcap, head_sums.data_ptr(), head_stats.data_ptr(), gws.data_ptr(), ws_bytes,
            st), "ekv_gaussian_moments")
    else:
        slopes, q_pos = alibi      # biased page means + page-mixture tau_hat (two launches)
        _lib.check(lib.ekv_gaussian_moments_alibi(
            desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, S, 1, float(alpha), mu.data_ptr(),
            sigma.data_ptr(), pcap, head_sums.data_ptr(), head_stats.data_ptr(), gws.data_ptr(), ws_bytes,
            slopes.data_ptr(), _lib.ptr(q_pos), st), "ekv_gaussian_moments_alibi")

    if callable(sigma_mean):
        # a batch spread over several processes: the caller turns this process's sum of sigma_global
        # into the batch-wide mean (one scalar all-reduce) between the two launches
        sigma_mean = sigma_mean(head_stats[..., 1].sum().reshape(1), B * Hq)
    page_indices = kv_cache.scratch("g_pages", (B, Hq, pcap), torch.int32)
    num_selected = kv_cache.scratch("g_counts", (B, Hq), torch.int32)
    tok_counts = kv_cache.scratch("g_tokens", (B, Hq), torch.int32)
    tau_floor = kv_cache.scratch("g_tau_floor", (B, Hq), torch.float32)
    cap_max = kv_cache.scratch("g_cap", (B, Hq), torch.float32)
    tau = kv_cache.scratch("g_tau", (B, Hq), torch.float32)
    work_list = work_total = None
    if build_work_list:
        n_chunks = (kv_cache.capacity + _CHUNK - 1) // _CHUNK
        work_list = kv_cache.scratch("g_work", (B * Hq * n_chunks,), torch.int64)
        work_total = kv_cache.scratch("g_work_total", (2 + (B * Hq + 1023) // 1024,), torch.int32, zero=True)
    _lib.check(lib.ekv_gaussian_select(
        desc, Hq, S, 1, 1, float(alpha), float(excess_margin_fraction),
        _z_of_quantile(0.99, P), _z_of_quantile(0.995, P), _z_of_quantile(float(clamp_quantile), P),
        int(bool(apply_clamp)), _lib.ptr(sigma_mean), mu.data_ptr(), sigma.data_ptr(), pcap,
        head_stats.data_ptr(), page_indices.data_ptr(), pcap, num_selected.data_ptr(),
        tok_counts.data_ptr(), tau_floor.data_ptr(), cap_max.data_ptr(), tau.data_ptr(),
        _lib.ptr(work_list), _lib.ptr(work_total), st), "ekv_gaussian_select")
    return dict(mu=mu, sigma=sigma, head_stats=head_stats, head_sums=head_sums,
                page_indices=page_indices, num_selected=num_selected, tok_counts=tok_counts,
                tau_floor=tau_floor, cap_max=cap_max, tau=tau, work_list=work_list,
                work_total=work_total)


def grouped_enabled(q, kv_cache: PagedKVCache, alibi=None) -> bool:
    """Whether the decode after a Gaussian-aware selection shares K rows inside GQA groups.

    The group-shared K pass exists for groups of four or eight query heads per KV head, 16-bit caches with
    head_dim 128 and no ALiBi; ``EKV_GROUPED=0`` in the environment turns it off."""
    if os.environ.get("EKV_GROUPED", "1") == "0" or alibi is not None:
        return False
    _, Hq, _, D = q.shape
    P = kv_cache.page_size
    Hkv = kv_cache._k.shape[1]
    if Hq not in (4 * Hkv, 8 * Hkv):
        return False
    # the union kernel keeps one page bitmap per head of the group in shared memory (180 KiB in all)
    return (D == 128 and kv_cache._k.element_size() == 2 and 4 <= P <= 32 and P & (P - 1) == 0
            and kv_cache.page_capacity <= 368640 * 4 // (Hq // Hkv))


def grouped_decode(q, kv_cache: PagedKVCache, out, sel, alpha, tau_mode, niter, stage_events=None, on_launch=None):
    """Decode over the selection ``sel`` (of ``gaussian_select``) with one page table per GQA group.

    Two launches ahead of the tau kernel: the union of the group's page tables with membership masks
    (``ekv_group_union``, which also lays out the per-head work list of the union for the tau kernel and the
    V pass) and the K pass over groups.
    ``sel`` keeps the per-head tables; the shared tables are returned for inspection.
    ``stage_events`` as in ``_paged_decode``; ``on_launch(kernel_name)`` is called after the launch ahead of
    the K pass (per-kernel timing)."""
    lib = _lib.load()
    B, Hq, _, D = q.shape
    Hkv, pcap, max_tokens = kv_cache._k.shape[1], kv_cache.page_capacity, kv_cache.capacity
    cph = lib.ekv_work_items_per_head(max_tokens)
    u_pages = kv_cache.scratch("gu_pages", (B, Hq, pcap), torch.int32)
    member = kv_cache.scratch("gu_member", (B, Hkv, pcap), torch.uint8)
    u_tok = kv_cache.scratch("gu_tokens", (B, Hq), torch.int32)
    g_items = kv_cache.scratch("gu_group_items", (B * Hkv * cph,), torch.int64)
    h_items = kv_cache.scratch("gu_head_items", (B * Hq * cph,), torch.int64)
    ws = _decode_workspace(kv_cache, B, Hq, D, max_tokens)
    desc = C.byref(kv_cache.desc())
    st = _lib.stream_ptr()
    pages = sel["page_indices"]
    _lib.check(lib.ekv_group_union(
        desc, Hq, pages.data_ptr(), pages.stride(1), sel["num_selected"].data_ptr(), max_tokens,
        u_pages.data_ptr(), u_pages.stride(1), member.data_ptr(), member.stride(1), u_tok.data_ptr(),
        g_items.data_ptr(), g_items.numel(), h_items.data_ptr(), st), "ekv_group_union")
    if on_launch:
        on_launch("group_union_kernel")
    tau = sel["tau"]
    tables = dict(union_pages=u_pages, member=member, union_tok_counts=u_tok)
    if kv_cache.block_mode:      # the decode addresses K/V by physical block id
        P = kv_cache.page_size
        u_pages = kv_cache.translate(u_pages, torch.div(u_tok + (P - 1), P, rounding_mode="floor").to(torch.int32))
    _lib.check(lib.ekv_decode_grouped(
        desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, u_pages.data_ptr(), u_pages.stride(1),
        u_tok.data_ptr(), max_tokens, float(alpha), tau_mode, int(niter), tau.data_ptr(), out.data_ptr(),
        out.stride(0), out.stride(1), h_items.data_ptr(), h_items.numel(), g_items.data_ptr(), g_items.numel(),
        member.data_ptr(), member.stride(1), ws.data_ptr(), ws.numel(), _event_array(stage_events), st),
        "ekv_decode_grouped")
    return tables


def sparse_attention_decode_gaussian_aware_entmax(
    q: torch.Tensor,
    kv_cache: PagedKVCache,
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    out: torch.Tensor,
    alpha: float = 1.5,
    safety_margin_z: float = 0.0,
    max_quantile: float = 0.995,
    alibi_slopes: torch.Tensor = None,
    scale: Optional[float] = None,
    splits: int = 32,
    niter: int = 2,
    append_cache: bool = False,
    tau_mode: str = "corrected",
    tau_correction_iters: Optional[int] = None,
    clamp_tau: bool = True,
    threshold_excess_margin_fraction: Optional[float] = 0.2,
    tau_clamp_page_max_quantile: float = 0.50,
    q_seqlens: torch.Tensor = None,
    cache_seqlens: torch.Tensor = None,
    taus_out: Optional[torch.Tensor] = None,
    sigma_mean=None,
):
    """Gaussian-aware page selection feeding the paged entmax decode
    (attention_gaussian.py:20-144).

    tau_mode: "exact" solves tau on the selected tokens (histogram bracket + ``niter``
    Halley steps); "fixed" uses the clamped Gaussian estimate; "corrected" refines it
    with ``tau_correction_iters`` (default 1) unbracketed Halley steps.  The output is
    ``sum_i (z_i - tau)_+^(1/(alpha-1)) v_i`` without normalisation, as in the reference.

    As in the reference, ``safety_margin_z``, ``max_quantile`` and ``scale`` are accepted
    but have no effect: margin and quantile are derived from the batch-wide mean of
    sigma_global (gaussian_utils.py:163-169), the scale is 1/sqrt(head_dim).
    ``cache_seqlens`` is accepted and ignored (the reference README passes it).
    ``sigma_mean`` (optional) replaces that batch-wide mean when this process holds only part of
    a batch: a device fp32 scalar, or a callable ``f(local_sum, local_heads) -> device scalar`` that
    is handed this process's sum of sigma_global (fp32 [1], on the device) between the moments sweep
    and the selection and returns the mean over the whole batch (one scalar all-reduce).
    ``splits`` has no effect.
    ``alibi_slopes`` ([H_q] fp32; alpha 2, 1.5 or 4/3): page means get ``slope * (mean position of the
    page - query position)``, tau_hat comes from the page-mixture solver, kept tokens get the
    positional term in their logits and "corrected" takes two steps by default; the query position
    is ``q_seqlens - 1`` (default: the token just appended).
    """
    if kv_cache._k is None:
        raise RuntimeError("kv_cache is not initialised")
    if not alpha > 1.0:
        raise ValueError("alpha must be > 1")
    tau_mode = tau_mode.lower()
    if tau_mode not in ("exact", "fixed", "corrected"):
        raise ValueError(f"Unsupported tau_mode={tau_mode!r}; expected 'exact', 'fixed', or 'corrected'")
    _check_q_out(q, out, kv_cache)
    if append_cache:
        kv_cache.append(k_new, v_new)
    B, Hq, _, D = q.shape
    frac = 0.1 if threshold_excess_margin_fraction is None else threshold_excess_margin_fraction
    alibi = None
    if alibi_slopes is not None:
        if alpha not in (1.5, 2.0) and abs(alpha - 4.0 / 3.0) > 1e-6:
            raise ValueError("ALiBi with Gaussian-aware selection needs alpha 2, 1.5 or 4/3 (page-mixture tau solver)")
        alibi = _alibi_args(alibi_slopes, q_seqlens, B, Hq, q.device)
    grouped = grouped_enabled(q, kv_cache, alibi)
    sel = gaussian_select(q, kv_cache, alpha, frac, tau_clamp_page_max_quantile,
                          apply_clamp=(tau_mode != "exact" and clamp_tau), sigma_mean=sigma_mean, alibi=alibi,
                          build_work_list=not grouped)
    kv_cache.last_num_selected_per_head = sel["num_selected"]
    kv_cache.last_gaussian_selection = sel
    if tau_mode == "exact":
        mode, iters = _lib.TAU_EXACT, int(niter)
    else:
        if tau_correction_iters is None:     # attention_gaussian.py:123-127: two steps with ALiBi
            tau_correction_iters = 0 if tau_mode == "fixed" else (1 if alibi is None else 2)
        mode, iters = _lib.TAU_CORRECTED, int(tau_correction_iters)
    if kv_cache.block_mode and alibi is not None:
        raise ValueError("ALiBi needs token positions and is not available on a block-table cache")
    if grouped:
        kv_cache.last_group_tables = grouped_decode(q, kv_cache, out, sel, alpha, mode, iters)
    else:
        kv_cache.last_group_tables = None
        pages = sel["page_indices"]
        if kv_cache.block_mode:      # the decode addresses K/V by physical block id
            pages = kv_cache.translate(pages, sel["num_selected"])
        _paged_decode(q, kv_cache, out, pages, sel["tok_counts"], kv_cache.capacity, alpha,
                      mode, iters, sel["tau"], sel["work_list"], work_total=sel["work_total"], alibi=alibi)
    if taus_out is not None:
        taus_out.copy_(sel["tau"])
    return out
