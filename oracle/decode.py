"""Oracle: paged entmax decode over selected pages (test infrastructure, CPU).

All quantities live in z-space: ``z_i = (alpha-1)/sqrt(D) * q.k_i``,
``p_i = (z_i - tau)_+^(1/(alpha-1))``, ``out = sum_i p_i v_i`` (no division: the
reference never normalises, adadecode_paged.py:494-507,
adadecode_paged_gaussian_tau.py:160-175).

Two tau procedures are restated:
  * ``tau_exact_mode``  - the reference's "exact" decode: global max, 16-bin
    histogram on [max-1, max], bracket from the histogram, ``niter`` bracketed
    Halley steps (adadecode_paged.py:79-377; adadecode.py:12-112,381-426,555-592).
  * ``tau_corrected``   - the Gaussian decode: start from a given tau and take
    ``iters`` unbracketed Halley/Newton steps
    (adadecode_paged_gaussian_tau.py:23-53).
and, as the mathematical yardstick, ``tau_true`` (the exact entmax threshold).

Scores are accumulated in fp64 and rounded to fp32; the reference instead
rounds ``q*(alpha-1)/sqrt(D)`` to the input dtype and lets Triton carry the
products and the D-sum in that dtype (adadecode_paged.py:97-98,124), which is
an accuracy loss the CUDA path does not reproduce; ``round_q=True`` applies
the first of these two roundings for comparison runs.
"""

from __future__ import annotations

import math

import numpy as np
import torch

BINS = 16


# --------------------------------------------------------------------------- #
# token enumeration and scores
# --------------------------------------------------------------------------- #

def token_rows(page_ids, n_tokens: int, page_size: int) -> np.ndarray:
    """Cache rows of compact indices 0..n_tokens-1 (adadecode_paged.py:116-121)."""
    c = np.arange(n_tokens)
    pages = np.asarray(page_ids, dtype=np.int64)
    return pages[c // page_size] * page_size + c % page_size


def scores_z(q_vec: torch.Tensor, k_rows: torch.Tensor, alpha: float,
             round_q: bool = False, alibi_slope: float | None = None,
             rows: np.ndarray | None = None, q_pos: int = 0) -> np.ndarray:
    """z for one head: q_vec [D], k_rows [T,D] -> fp32 [T].

    With ``alibi_slope`` every token gets ``(alpha-1) * slope * (rows[i] - q_pos)``, its
    absolute position relative to the query's (kernels/adadecode_paged.py:100-105,126-128).
    """
    D = q_vec.shape[-1]
    scalar = (alpha - 1.0) / math.sqrt(D)
    if round_q:
        qs = (q_vec * scalar).to(q_vec.dtype).to(torch.float64)
    else:
        qs = q_vec.to(torch.float64) * scalar
    z = k_rows.to(torch.float64) @ qs
    if alibi_slope is not None:
        slope_a = float(np.float32(alibi_slope) * np.float32(alpha - 1.0))
        z = z + slope_a * torch.from_numpy((rows - q_pos).astype(np.float64))
    return z.to(torch.float32).numpy()


# --------------------------------------------------------------------------- #
# tau procedures
# --------------------------------------------------------------------------- #

def _power_sums(z: np.ndarray, tau: float, alpha: float):
    """acc_j = sum (z - tau)_+^(beta - j), j = 0,1,2 (adadecode_paged.py:359-372)."""
    beta = 1.0 / (alpha - 1.0)
    d = z.astype(np.float64) - tau
    d = d[d > 0]
    if alpha == 2.0:
        return d.sum(), float(d.size), 0.0
    if alpha == 1.5:
        return (d * d).sum(), d.sum(), float(d.size)
    return (d ** beta).sum(), (d ** (beta - 1.0)).sum(), (d ** (beta - 2.0)).sum()


def histogram16(z: np.ndarray, zmax: np.float32) -> np.ndarray:
    """16 equal bins on [max-1, max]; truncation toward zero; top bin closed.

    adadecode_paged.py:235-244: ``b = min(int((z - t0) * 16), 15)``, counted when
    ``b >= 0`` - so values in (t0 - 1/16, t0) land in bin 0 as well.
    """
    t0 = np.float32(zmax) - np.float32(1.0)
    proj = (z.astype(np.float32) - t0) * np.float32(BINS)
    b = np.minimum(np.trunc(proj).astype(np.int64), BINS - 1)
    b = b[b >= 0]
    return np.bincount(b, minlength=BINS).astype(np.int64)


def tau_bracket_from_hist(hist: np.ndarray, zmax: float, alpha: float):
    """(t_lo, t_hi) from the histogram (adadecode.py:38-112,399-421)."""
    if alpha in (2.0, 1.5):
        sz = sk = sz2 = 1.0
        for sj in range(BINS - 1, -1, -1):
            c = float(hist[sj]) - (1.0 if sj == BINS - 1 else 0.0)
            ct = sj / BINS
            nz, nk, nz2 = sz + c * ct, sk + c, sz2 + c * ct * ct
            if alpha == 2.0:
                ok = (nz - nk * ct) < 1.0
            else:
                ok = (nk * ct * ct - 2.0 * nz * ct + nz2) < 1.0
            if ok:
                sz, sk, sz2 = nz, nk, nz2
        if alpha == 2.0:
            t_init = zmax + (sz - 1.0) / sk - 1.0
        else:
            disc = sz * sz - sk * (sz2 - 1.0)
            t_init = zmax + (sz - math.sqrt(disc)) / sk - 1.0
        return t_init, t_init + 1.0 / BINS
    # generic alpha: binary search for the bin whose edges bracket the root
    counts = hist.astype(np.float64).copy()
    counts[BINS - 1] -= 1.0
    p = 1.0 / (alpha - 1.0)
    bins = np.arange(BINS)
    lo, hi, found, b_idx = 0, BINS - 1, False, 0
    for _ in range(5):
        mid = int((lo + hi) * 0.5)
        off = bins - mid
        mask = off >= 0
        zl = off / BINS
        zu = (off + 1.0) / BINS
        term_l = np.where(mask & (zl > 0), np.where(zl > 0, zl, 1.0) ** p, 0.0)
        term_u = np.where(mask, np.where(mask, zu, 1.0) ** p, 0.0)
        f_l = (counts * term_l).sum() - 1.0
        f_u = (counts * term_u).sum() - 1.0
        go_right, go_left = f_l > 0.0, f_u < 0.0
        if not found:
            if not go_right and not go_left:
                b_idx, found = mid, True
            if go_right:
                lo = mid + 1
            if go_left:
                hi = mid - 1
    b_sel = b_idx if found else min(lo, BINS - 1)
    t0 = zmax - 1.0
    return t0 + b_sel / BINS, t0 + min(b_sel + 1, BINS) / BINS


def halley_bracketed(t, t_lo, t_hi, acc, alpha):
    """One bracketed Halley step (adadecode.py:12-35)."""
    c0 = 1.0 / (alpha - 1.0)
    c1 = c0 - 1.0
    ff = acc[0] - 1.0
    df = -c0 * acc[1]
    ddf = c0 * c1 * acc[2]
    if ff > 0:
        t_lo = t
    if ff < 0:
        t_hi = t
    den = 2.0 * df * df - ff * ddf
    new_t = t - (2.0 * ff * df) / den if den != 0.0 else float("nan")
    good = (new_t > t_lo - 1e-6) and (new_t < t_hi + 1e-6)
    return (new_t if good else 0.5 * (t_lo + t_hi)), t_lo, t_hi


def tau_exact_mode(z: np.ndarray, alpha: float, niter: int) -> float:
    """Histogram-initialised, ``niter``-step tau of the exact decode."""
    zmax = np.float32(z.max()) if z.size else np.float32(-1.0e6)
    hist = histogram16(z, zmax)
    t_lo, t_hi = tau_bracket_from_hist(hist, float(zmax), alpha)
    t = 0.5 * (t_lo + t_hi)
    for _ in range(niter):
        t, t_lo, t_hi = halley_bracketed(t, t_lo, t_hi, _power_sums(z, t, alpha), alpha)
    return float(t)


def halley_unbounded(t, acc, alpha):
    """Unbracketed Halley step with Newton and keep-as-is fallbacks
    (adadecode_paged_gaussian_tau.py:40-53)."""
    c0 = 1.0 / (alpha - 1.0)
    c1 = c0 - 1.0
    ff = acc[0] - 1.0
    df = -c0 * acc[1]
    ddf = c0 * c1 * acc[2]
    den = 2.0 * df * df - ff * ddf
    if abs(den) > 1e-12:
        t_next = t - (2.0 * ff * df) / den
    elif abs(df) > 1e-12:
        t_next = t - ff / df
    else:
        t_next = t
    if not math.isfinite(t_next) or abs(t_next) >= 1.0e20:
        t_next = t
    return t_next


def tau_corrected(z: np.ndarray, tau0: float, alpha: float, iters: int) -> float:
    t = float(tau0)
    for _ in range(iters):
        t = halley_unbounded(t, _power_sums(z, t, alpha), alpha)
    return t


def tau_true(z: np.ndarray, alpha: float) -> float:
    """Exact entmax threshold: sum (z - tau)_+^beta = 1, by fp64 bisection on
    [max-1, max] (the root always lies there)."""
    zz = z.astype(np.float64)
    beta = 1.0 / (alpha - 1.0)
    hi = zz.max()
    lo = hi - 1.0
    for _ in range(100):
        mid = 0.5 * (lo + hi)
        s = (np.clip(zz - mid, 0.0, None) ** beta).sum()
        if s > 1.0:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


# --------------------------------------------------------------------------- #
# outputs
# --------------------------------------------------------------------------- #

def weights(z: np.ndarray, tau: float, alpha: float) -> np.ndarray:
    d = np.clip(z.astype(np.float64) - tau, 0.0, None)
    if alpha == 2.0:
        return d
    if alpha == 1.5:
        return d * d
    return np.where(d > 0, d ** (1.0 / (alpha - 1.0)), 0.0)


def _head_views(q, k_cache, v_cache, b, h):
    G = q.shape[1] // k_cache.shape[1]
    return q[b, h, 0], k_cache[b, h // G], v_cache[b, h // G]


def decode(q, k_cache, v_cache, page_tables, n_tokens, page_size: int, alpha: float,
           mode: str = "exact", niter: int = 2, tau0=None, iters: int = 1,
           round_q: bool = False, alibi_slopes=None, q_pos=None):
    """Decode every (b, h_q).

    page_tables[b][h] : sequence of page ids (last page in the final slot)
    n_tokens[b][h]    : compacted token count T of that head
    mode              : "exact" (histogram + niter Halley), "corrected"
                        (tau0[b][h] + iters unbounded steps; iters=0 is "fixed"),
                        or "true" (exact entmax threshold)
    alibi_slopes      : [Hq] slopes or None; q_pos[b] the query's absolute position
    Returns (out fp32 [B,Hq,D], tau fp64 [B,Hq], support sizes int [B,Hq]).
    """
    B, Hq, _, D = q.shape
    out = np.zeros((B, Hq, D), dtype=np.float32)
    taus = np.zeros((B, Hq), dtype=np.float64)
    supp = np.zeros((B, Hq), dtype=np.int64)
    for b in range(B):
        for h in range(Hq):
            qv, kc, vc = _head_views(q, k_cache, v_cache, b, h)
            T = int(n_tokens[b][h])
            rows = token_rows(np.asarray(page_tables[b][h]), T, page_size)
            rows_t = torch.from_numpy(rows)
            if alibi_slopes is None:
                z = scores_z(qv, kc[rows_t], alpha, round_q=round_q)
            else:
                z = scores_z(qv, kc[rows_t], alpha, round_q=round_q, alibi_slope=float(alibi_slopes[h]),
                             rows=rows, q_pos=int(q_pos[b]))
            if mode == "exact":
                tau = tau_exact_mode(z, alpha, niter)
            elif mode == "corrected":
                tau = tau_corrected(z, float(tau0[b][h]), alpha, iters)
            elif mode == "true":
                tau = tau_true(z, alpha)
            else:
                raise ValueError(mode)
            p = weights(z, tau, alpha)
            nz = np.nonzero(p)[0]
            vv = vc[rows_t[nz]].to(torch.float64).numpy()
            out[b, h] = (p[nz][:, None] * vv).sum(0).astype(np.float32)
            taus[b, h] = tau
            supp[b, h] = nz.size
    return out, taus, supp
