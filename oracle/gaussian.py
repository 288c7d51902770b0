"""Oracle: Gaussian-aware page selection and tau estimate (test infrastructure).

Follows, in this order,
  * per-page score moments        entmaxkv/kernels/gaussian_page_stats.py:50-73
  * per-head moments              entmaxkv/kernels/gaussian_page_stats.py:97-121
  * sigma_global, auto margin     entmaxkv/gaussian_utils.py:155-169
  * single-Gaussian tau solver    entmaxkv/tau_solver.py:210-273 (fp64 scalar),
                                  entmaxkv/kernels/tau_solver_gpu.py:79-125 (fp32)
  * threshold select + pack       entmaxkv/kernels/selection_pack.py:144-198
  * tau clamp                     entmaxkv/kernels/tau_clamp.py:42-73,
                                  entmaxkv/gaussian_utils.py:287-315
  * compacted token counts        entmaxkv/kernels/selection_pack.py:19
  * page-mixture tau              entmaxkv/kernels/tau_solver_page_mixture.py:67-185

fp32 sums here use torch's own reduction order; the CUDA kernels are compared
with a tolerance (1e-5 relative on moments, 1e-4 relative on tau), and page
sets are compared exactly outside a boundary class of pages whose selection
margin is below that tolerance.
"""

from __future__ import annotations

import math
from statistics import NormalDist

import torch

_SQRT2 = math.sqrt(2.0)
_SQRT2PI = math.sqrt(2.0 * math.pi)


# --------------------------------------------------------------------------- #
# moments
# --------------------------------------------------------------------------- #

def page_moments(q: torch.Tensor, k_mean: torch.Tensor, k_std: torch.Tensor,
                 pages_for_stats: int):
    """mu_p = scale*sum q*k_mean_p, var_p = scale^2*sum q^2*k_std_p^2 (fp32).

    q [B,Hq,1,D]; k_mean/k_std [B,Hkv,Np,D].  Returns (mu [B,Hq,n], var, sigma).
    (gaussian_page_stats.py:50-73; sigma = sqrt(var) as in :112-113)
    """
    B, Hq, _, D = q.shape
    G = Hq // k_mean.shape[1]
    scale = float(1.0 / math.sqrt(D))
    qs = q[:, :, 0, :].to(torch.float32) * scale              # [B,Hq,D]
    qv = qs * qs
    km = k_mean[:, :, :pages_for_stats].to(torch.float32).repeat_interleave(G, dim=1)
    ks = k_std[:, :, :pages_for_stats].to(torch.float32).repeat_interleave(G, dim=1)
    mu = (km * qs[:, :, None, :]).sum(dim=-1)
    var = (ks * ks * qv[:, :, None, :]).sum(dim=-1)
    return mu, var, torch.sqrt(var)


def head_moments(mu: torch.Tensor, var: torch.Tensor):
    """mean(mu), mean(var), max(E[mu^2]-mean^2, 0) per head -> each [B,H].

    (gaussian_page_stats.py:104-111)
    """
    n = float(mu.shape[-1])
    mean = mu.sum(-1) / n
    mean_var = var.sum(-1) / n
    var_means = torch.clamp((mu * mu).sum(-1) / n - mean * mean, min=0.0)
    return mean, mean_var, var_means


def global_sigma(mean_var: torch.Tensor, var_means: torch.Tensor) -> torch.Tensor:
    """sigma_global with the reference's NaN/inf scrubbing (gaussian_utils.py:156-161)."""
    return torch.nan_to_num(torch.sqrt(mean_var + var_means),
                            nan=1e-6, posinf=1e6, neginf=1e-6).clamp(min=1e-6)


def auto_margin(sigma_global: torch.Tensor):
    """(safety_margin_z, max_quantile) from the mean of sigma_global over all (b,h).

    gaussian_utils.py:163-169.  One scalar couples every head of the batch.
    """
    s = float(sigma_global.to(torch.float32).mean().item())
    low = s < 1.5
    return (0.01 if low else 0.05) * s, (0.99 if low else 0.995)


def z_of_quantile(quantile: float, page_size: int) -> float:
    """Normal quantile of ``quantile ** (1/page_size)`` (selection_pack.py:238-239)."""
    return NormalDist().inv_cdf(quantile ** (1.0 / page_size))


# --------------------------------------------------------------------------- #
# single-Gaussian tau
# --------------------------------------------------------------------------- #

def _phi(t):
    return math.exp(-0.5 * t * t) / _SQRT2PI


def _Phi(t):
    return 0.5 * math.erfc(-t / _SQRT2)


def _moments012(mu_y, sigma_y):
    t = mu_y / sigma_y
    ph, Ph = _phi(t), _Phi(t)
    m0 = Ph
    m1 = mu_y * Ph + sigma_y * ph
    m2 = (mu_y * mu_y + sigma_y * sigma_y) * Ph + mu_y * sigma_y * ph
    return m0, m1, m2, ph


def constraint(tau, mu_g, sigma_g, n, alpha):
    """f, f', f'' of  n*E[((alpha-1)S - tau)_+^(1/(alpha-1))] - 1,  S~N(mu_g, sigma_g^2).

    Closed forms for alpha in {2, 1.5} (tau_solver.py:176-207).
    """
    a = alpha - 1.0
    sigma_y = max(a * sigma_g, 1e-10)
    mu_y = a * mu_g - tau
    m0, m1, m2, ph = _moments012(mu_y, sigma_y)
    if alpha == 2.0:
        return n * m1 - 1.0, -n * m0, n * ph / sigma_y
    if alpha == 1.5:
        return n * m2 - 1.0, -2.0 * n * m1, 2.0 * n * m0
    raise ValueError("closed-form derivatives exist for alpha in {2, 1.5} only")


def tau_hat_scalar(mu_g: float, sigma_g: float, n: int, alpha: float,
                   iterations: int = 120, tol: float = 1e-6) -> float:
    """Bracketed Halley root of the single-Gaussian constraint, fp64 scalar.

    tau_solver.py:227-271: bracket a*mu +- a*sigma*(sqrt(2 ln(n+1)) + 8); per
    iteration a Halley step (Newton when the Halley denominator vanishes), the
    bracket midpoint when the step leaves the bracket, early exit at |f| <= tol.
    """
    a = alpha - 1.0
    sigma_g = max(sigma_g, 1e-6)
    radius = a * sigma_g * (math.sqrt(2.0 * math.log(n + 1.0)) + 8.0)
    lo, hi = a * mu_g - radius, a * mu_g + radius
    tau = 0.5 * (lo + hi)
    for _ in range(iterations):
        f, fp, fpp = constraint(tau, mu_g, sigma_g, n, alpha)
        if abs(f) <= tol:
            break
        mid = 0.5 * (lo + hi)
        den = 2.0 * fp * fp - f * fpp
        if abs(den) > 1e-18:
            step = 2.0 * f * fp / den
        else:
            step = f / fp if abs(fp) > 1e-18 else 0.0
        cand = tau - step
        if not math.isfinite(cand) or cand <= lo or cand >= hi:
            cand = mid
        fc = constraint(cand, mu_g, sigma_g, n, alpha)[0]
        if abs(fc) <= tol:
            tau = cand
            break
        if fc > 0.0:
            lo = cand
        else:
            hi = cand
        tau = 0.5 * (lo + hi)
    return tau


FOUR_THIRDS = 4.0 / 3.0


def is_four_thirds(alpha: float) -> bool:
    """alpha = 4/3 as the caller's double or after a trip through fp32."""
    return abs(alpha - FOUR_THIRDS) < 1e-6


def tau_hat_bisection(mu_g: float, sigma_g: float, n: int, alpha: float,
                      max_iter: int = 120, tol: float = 1e-6) -> float:
    """Bisection for every alpha but 2 and 1.5 (tau_solver.py:276-344).

    alpha = 4/3 has the closed form ``E[Y_+^3] = (mu^3 + 3 mu s^2) Phi(t) + (s^3 + 2 mu^2 s) phi(t)``
    (tau_solver.py:73-78); any other alpha uses the reference's crude approximation
    ``E[Y_+^beta] ~ sigma_Y^beta * max(t,0)^beta`` (:80-84).
    """
    third = is_four_thirds(alpha)
    a = FOUR_THIRDS - 1.0 if third else alpha - 1.0
    beta = 1.0 / a

    def f(tau):
        sigma_y = max(a * sigma_g, 1e-10)
        mu_y = a * mu_g - tau
        t = mu_y / sigma_y
        if third:
            return n * ((mu_y ** 3 + 3.0 * mu_y * sigma_y ** 2) * _Phi(t)
                        + (sigma_y ** 3 + 2.0 * mu_y * mu_y * sigma_y) * _phi(t)) - 1.0
        return n * (sigma_y ** beta) * (max(t, 0.0) ** beta) - 1.0

    logf = math.sqrt(2.0 * math.log(n + 1))
    lo = a * mu_g - 5.0 * a * sigma_g
    hi = a * mu_g + a * sigma_g * (logf + 5.0)
    while f(lo) < 0:
        lo -= 2.0 * sigma_g
    while f(hi) > 0:
        hi += 2.0 * sigma_g
    for _ in range(max_iter):
        mid = 0.5 * (lo + hi)
        fm = f(mid)
        if abs(fm) < tol:
            return mid
        if fm > 0:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


def tau_hat(mu_g: torch.Tensor, sigma_g: torch.Tensor, n: int, alpha: float) -> torch.Tensor:
    """Elementwise tau_hat for [B,H] inputs -> fp32 [B,H] (tau_solver.py:347-412)."""
    flat_mu = mu_g.reshape(-1).to(torch.float64).tolist()
    flat_sg = sigma_g.reshape(-1).to(torch.float64).tolist()
    solver = tau_hat_scalar if alpha in (2.0, 1.5) else tau_hat_bisection
    out = [solver(m, s, n, alpha) for m, s in zip(flat_mu, flat_sg)]
    return torch.tensor(out, dtype=torch.float64).reshape(mu_g.shape).to(torch.float32)


# --------------------------------------------------------------------------- #
# threshold selection, clamp, token counts
# --------------------------------------------------------------------------- #

def select_threshold_pack(mu: torch.Tensor, sigma: torch.Tensor, tau_hat_: torch.Tensor,
                          sigma_global: torch.Tensor, *, page_size: int, alpha: float,
                          safety_margin_z: float, max_quantile: float,
                          threshold_excess_margin_fraction: float, num_pages: int,
                          upper_mean: torch.Tensor | None = None):
    """Per (b,h): tau_floor, the ascending list of selected pages (+ last page), margins.

    selection_pack.py:161-198.  Returns
      pages   : list[B][H] of int32 tensors (selected statistical pages ascending,
                then ``num_pages-1`` when it carries no statistics)
      tau_floor [B,H] fp32
      margin  : [B,H,n] fp32 = a*(mu+z*sigma) - tau_floor  (selection iff > 0)
    """
    a = float(alpha - 1.0)
    n = mu.shape[-1]
    z_page = float(z_of_quantile(max_quantile, page_size))
    # mean of (mu + 1.5 sigma) over the statistical pages; supplied by the caller when this
    # call sees only a slice of the pages
    upper = (mu + float(1.5) * sigma).sum(-1) / float(n) if upper_mean is None else upper_mean
    thr = tau_hat_ / a
    sigma_delta = float(safety_margin_z) * sigma_global
    excess = torch.clamp(thr - upper, min=0.0)
    tau_delta = float(threshold_excess_margin_fraction) * excess
    delta = torch.maximum(sigma_delta, tau_delta)
    tau_floor = tau_hat_ - delta * a
    margin = a * (mu + z_page * sigma) - tau_floor[..., None]
    sel = margin > 0
    B, H = mu.shape[:2]
    pages = []
    for b in range(B):
        row = []
        for h in range(H):
            ids = torch.nonzero(sel[b, h]).reshape(-1).to(torch.int32)
            if num_pages > n:
                ids = torch.cat([ids, torch.tensor([num_pages - 1], dtype=torch.int32)])
            row.append(ids)
        pages.append(row)
    return pages, tau_floor, margin


def clamp_tau(tau: torch.Tensor, mu: torch.Tensor, sigma: torch.Tensor, pages,
              tau_floor: torch.Tensor, *, page_size: int, alpha: float,
              clamp_quantile: float = 0.5, eps: float = 1e-4) -> torch.Tensor:
    """tau <- min(tau, max(a*max_sel(mu + z_clamp*sigma/3) - eps, tau_floor)).

    Only statistical pages (id < n) count; heads without any keep tau
    (tau_clamp.py:48-73).
    """
    a = float(alpha - 1.0)
    n = mu.shape[-1]
    z_clamp = float(z_of_quantile(clamp_quantile, page_size))
    cap = mu + z_clamp * sigma * float(0.3333333333333333)
    out = tau.clone()
    B, H = tau.shape
    for b in range(B):
        for h in range(H):
            ids = pages[b][h].long()
            ids = ids[ids < n]
            if ids.numel() == 0:
                continue
            upper = a * cap[b, h, ids].max() - float(eps)
            upper = torch.maximum(upper, tau_floor[b, h])
            out[b, h] = torch.minimum(tau[b, h], upper)
    return out


def cache_seqlens_from_counts(counts: torch.Tensor, page_size: int, last_page_size: int):
    """max(count-1, 0)*P + last_page_size (selection_pack.py:19)."""
    return torch.clamp(counts.to(torch.int32) - 1, min=0) * page_size + last_page_size


def last_page_size(seq_len: int, page_size: int) -> int:
    """Tokens in the last page as the wrapper computes it (attention_gaussian.py:99)."""
    if seq_len > page_size:
        return seq_len - (math.ceil(seq_len / page_size) - 1) * page_size
    return seq_len


def gaussian_selection(q, k_mean, k_std, seq_len: int, page_size: int, alpha: float = 1.5,
                       threshold_excess_margin_fraction: float = 0.2,
                       clamp_quantile: float = 0.5, sigma_mean_override: float | None = None,
                       alibi_slopes: torch.Tensor | None = None):
    """The whole selection stage of the Gaussian-aware step for a uniform batch.

    With ``alibi_slopes`` ([Hq]) every page mean gets ``slope * (mean position of the page -
    (seq_len - 1))`` after the global moments were taken from the unbiased means, and tau_hat
    comes from the page-mixture solver with ``page_size`` tokens per page
    (gaussian_utils.py:142-153,171-177).

    Mirrors compute_gaussian_aware_statistics -> select_gaussian_aware ->
    clamp_tau_to_selected_page_statistics -> cache_seqlens
    (attention_gaussian.py:68-104).  ``sigma_mean_override`` supplies the
    batch-wide mean of sigma_global when this call sees only part of the batch.
    Returns a dict of every intermediate.
    """
    num_pages = k_mean.shape[2]
    n_stats = num_pages - 1 if num_pages > 1 else num_pages
    last_tokens = seq_len - (num_pages - 1) * page_size if num_pages > 1 else 0
    n_tokens = seq_len - last_tokens
    mu, var, sigma = page_moments(q, k_mean, k_std, n_stats)
    mean, mean_var, var_means = head_moments(mu, var)
    mu_g = torch.nan_to_num(mean, nan=0.0, posinf=0.0, neginf=0.0)
    sig_g = global_sigma(mean_var, var_means)
    if sigma_mean_override is None:
        margin_z, max_q = auto_margin(sig_g)
    else:
        low = sigma_mean_override < 1.5
        margin_z = (0.01 if low else 0.05) * sigma_mean_override
        max_q = 0.99 if low else 0.995
    if alibi_slopes is not None:
        mean_pos = torch.clamp(torch.arange(n_stats, dtype=torch.float32) * page_size + (page_size - 1) / 2.0,
                               max=float(n_tokens - 1))
        mu = mu + alibi_slopes.to(torch.float32).reshape(1, -1, 1) * (mean_pos - float(seq_len - 1))
        th = tau_hat_page_mixture(mu, sigma, alpha=alpha, uniform_page_count=float(page_size)).squeeze(-1)
    else:
        th = tau_hat(mu_g, sig_g, n_tokens, alpha)
    pages, tau_floor, margin = select_threshold_pack(
        mu, sigma, th, sig_g, page_size=page_size, alpha=alpha,
        safety_margin_z=margin_z, max_quantile=max_q,
        threshold_excess_margin_fraction=threshold_excess_margin_fraction,
        num_pages=num_pages)
    tau_c = clamp_tau(th, mu, sigma, pages, tau_floor, page_size=page_size, alpha=alpha,
                      clamp_quantile=clamp_quantile)
    counts = torch.tensor([[len(p) for p in row] for row in pages], dtype=torch.int32)
    seqlens = cache_seqlens_from_counts(counts, page_size, last_page_size(seq_len, page_size))
    return dict(mu=mu, sigma=sigma, mu_global=mu_g, sigma_global=sig_g, tau_hat=th,
                tau_floor=tau_floor, tau_clamped=tau_c, pages=pages, counts=counts,
                cache_seqlens=seqlens, margin=margin, safety_margin_z=margin_z,
                max_quantile=max_q, n_tokens=n_tokens)


# --------------------------------------------------------------------------- #
# page-mixture tau (ALiBi path of the reference)
# --------------------------------------------------------------------------- #

def tau_hat_page_mixture(mu_pages: torch.Tensor, sigma_pages: torch.Tensor,
                         page_counts: torch.Tensor | None = None, alpha: float = 1.5,
                         max_iter: int = 40, tol: float = 1e-6,
                         uniform_page_count: float = 1.0) -> torch.Tensor:
    """Root of sum_p count_p * E[((alpha-1)S_p - tau)_+^beta] = 1, S_p~N(mu_p,sigma_p^2).

    Bisection in fp64 on the monotone constraint; the reference
    (tau_solver_page_mixture.py:67-185) brackets with the page extremes and
    iterates Newton/bisection to the same root.  mu/sigma [B,H,n] -> tau [B,H,1].
    """
    a = alpha - 1.0
    beta = round(1.0 / a)
    mu = mu_pages.to(torch.float64) * a
    sg = (sigma_pages.to(torch.float64) * a).clamp(min=1e-10)
    cnt = (torch.full_like(mu, float(uniform_page_count)) if page_counts is None
           else page_counts.to(torch.float64))

    def f(tau):
        my = mu - tau
        t = my / sg
        ph = torch.exp(-0.5 * t * t) / _SQRT2PI
        Ph = 0.5 * (1.0 + torch.erf(t / _SQRT2))
        if beta == 1:
            m = my * Ph + sg * ph
        elif beta == 2:
            m = (my * my + sg * sg) * Ph + my * sg * ph
        else:
            m = (my ** 3 + 3 * my * sg * sg) * Ph + (sg ** 3 + 2 * my * my * sg) * ph
        return (cnt * m).sum(-1, keepdim=True) - 1.0

    lo = (mu - 12.0 * sg).amin(-1, keepdim=True) - 1.0
    hi = (mu + 12.0 * sg).amax(-1, keepdim=True)
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        fm = f(mid)
        lo = torch.where(fm > 0, mid, lo)
        hi = torch.where(fm <= 0, mid, hi)
    return (0.5 * (lo + hi)).to(torch.float32)
