"""Self-consistency of the decode oracle (CPU): the reference's tau procedures
must land on the true entmax threshold, and the paged decode over *all* pages
must reproduce dense entmax attention."""

import numpy as np
import pytest
import torch

from oracle import decode as od, dense as odense, topk as otopk, cache as ocache


@pytest.mark.parametrize("alpha", [1.5, 2.0, 1.75])
def test_exact_mode_tau_converges_to_true_tau(alpha):
    rng = np.random.default_rng(0)
    # For general alpha the reference's histogram bracket leaves out the maximum's own
    # term (adadecode.py:74-112), so on very short lists it can miss the root; the
    # restatement keeps that behaviour and is only required to converge on longer lists.
    for T in ((1, 7, 200, 3000) if alpha in (1.5, 2.0) else (1, 200, 3000)):
        z = (rng.standard_normal(T) * 0.4 * (alpha - 1.0)).astype(np.float32)
        t_true = od.tau_true(z, alpha)
        t2 = od.tau_exact_mode(z, alpha, niter=3)
        assert abs(t2 - t_true) <= 2e-5 * max(1.0, abs(t_true))
        p = od.weights(z, t_true, alpha)
        assert p.sum() == pytest.approx(1.0, abs=1e-9)


@pytest.mark.parametrize("alpha", [1.5, 2.0])
def test_corrected_tau_moves_toward_true_tau(alpha):
    rng = np.random.default_rng(1)
    z = (rng.standard_normal(500) * 0.5).astype(np.float32)
    t_true = od.tau_true(z, alpha)
    t0 = t_true - 0.3
    t1 = od.tau_corrected(z, t0, alpha, 1)
    t3 = od.tau_corrected(z, t0, alpha, 4)
    assert abs(t1 - t_true) < abs(t0 - t_true)
    assert abs(t3 - t_true) < 1e-6


@pytest.mark.parametrize("alpha", [1.5, 2.0, 1.75])
@pytest.mark.parametrize("S", [48, 53])
def test_paged_decode_over_all_pages_equals_dense(alpha, S):
    torch.manual_seed(3)
    B, Hq, Hkv, D, P = 2, 4, 2, 32, 16
    q = torch.randn(B, Hq, 1, D)
    k = torch.randn(B, Hkv, S, D)
    v = torch.randn(B, Hkv, S, D)
    n_pages = (S + P - 1) // P
    tables = [[list(range(n_pages)) for _ in range(Hq)] for _ in range(B)]
    ntok = [[S] * Hq for _ in range(B)]
    out, taus, _ = od.decode(q, k, v, tables, ntok, P, alpha, mode="true")
    dense = odense.dense_entmax_decode(q.double(), k.double(), v.double(), alpha,
                                       compute_dtype=torch.float64)[:, :, 0].numpy()
    np.testing.assert_allclose(out, dense, rtol=1e-4, atol=1e-5)
    if alpha in (1.5, 2.0):
        out2, taus2, _ = od.decode(q, k, v, tables, ntok, P, alpha, mode="exact", niter=3)
        np.testing.assert_allclose(out2, dense, rtol=1e-3, atol=1e-4)


def test_topk_tie_break_prefers_lower_page():
    s = torch.tensor([[[1.0, 3.0, 2.0, 3.0, 2.0, 0.5]]], dtype=torch.float16)
    ids = otopk.topk_page_sets(s, 3)
    assert ids.tolist() == [[[1, 2, 3]]]
    tied = otopk.boundary_tied_pages(s, 3)
    assert tied.tolist() == [[[False, False, True, False, True, False]]]
    pi, T = otopk.topk_select_and_pack(s, token_budget=3 * 16, page_size=16, seq_len=6 * 16 + 5)
    assert pi.tolist() == [[[1, 2, 3, 6]]] and T == 3 * 16 + 5


def test_criticality_is_an_upper_bound():
    torch.manual_seed(5)
    k = torch.randn(1, 2, 64, 32).half()
    q = torch.randn(1, 4, 1, 32).half()
    mn, mx, _, _ = ocache.page_stats(k, 16)
    s = otopk.criticality_scores(q, mn, mx, n_scored=4).float()
    true = torch.einsum("bhd,bhsd->bhs", q[:, :, 0].float(),
                        k.float().repeat_interleave(2, dim=1)).view(1, 4, 4, 16).amax(-1)
    assert (s + 2e-2 >= true).all()
