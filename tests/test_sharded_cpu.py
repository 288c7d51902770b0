"""Sequence-page sharding on CPU ranks (gloo, world size 2): the step function of
``entmaxkv_b200.sharded`` driven with oracle-backed shards must reproduce the unsharded oracle.
This covers the reduction algebra (what is summed, what is maxed, in which order) and the
host logic without touching a GPU."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import cache as ocache, gaussian as og, decode as od
from tests import _harness as H

P, ALPHA = 16, 1.5


class OracleShard:
    """CPU stand-in for GpuSequenceShard: same stage methods, oracle arithmetic."""

    def __init__(self, rank, world, page0):
        self.rank, self.world, self.is_last, self.page0 = rank, world, rank == world - 1, page0

    def initialize(self, k, v):
        self.c = ocache.OracleCache(P)
        self.c.initialize(k, v)

    def set_global_lengths(self, total):
        self.global_len = torch.tensor(list(total), dtype=torch.int32)

    def append(self, k_new, v_new):
        if self.is_last:
            self.c.append(k_new, v_new)
        self.global_len.add_(1)

    def _n_stats(self):
        n = self.c.k_mean.shape[2]
        return n - 1 if self.is_last else n

    def moments(self, q, alpha):
        self.q, self.alpha = q, alpha
        self.mu, var, self.sigma = og.page_moments(q, self.c.k_mean, self.c.k_std, self._n_stats())
        return torch.stack([self.mu.sum(-1), (self.mu * self.mu).sum(-1), var.sum(-1),
                            (self.mu + 1.5 * self.sigma).sum(-1)], dim=-1)

    def finalize(self, sums):
        lens = self.global_len.tolist()
        n_pages = [(x + P - 1) // P for x in lens]
        n_stat = [p - 1 if p > 1 else p for p in n_pages]
        n_tok = [(p - 1) * P if p > 1 else x for p, x in zip(n_pages, lens)]
        n = torch.tensor(n_stat, dtype=torch.float32).view(-1, 1)
        mean = sums[..., 0] / n
        var_means = torch.clamp(sums[..., 1] / n - mean * mean, min=0.0)
        sig = og.global_sigma(sums[..., 2] / n, var_means)
        tau_hat = torch.stack([og.tau_hat(mean[b], sig[b], int(n_tok[b]), self.alpha) for b in range(mean.shape[0])])
        self.stats = torch.stack([mean, sig, tau_hat, sums[..., 3] / n], dim=-1)
        return self.stats

    def select(self, frac, clamp_q):
        mean, sig, tau_hat, upper = self.stats.unbind(-1)
        margin_z, max_q = og.auto_margin(sig)
        n_local = self.mu.shape[-1]
        pages, self.tau_floor, _ = og.select_threshold_pack(
            self.mu, self.sigma, tau_hat, sig, page_size=P, alpha=self.alpha, safety_margin_z=margin_z,
            max_quantile=max_q, threshold_excess_margin_fraction=frac,
            num_pages=n_local + (1 if self.is_last else 0), upper_mean=upper)
        self.pages, self.tau = pages, tau_hat.clone()
        zc = og.z_of_quantile(clamp_q, P)
        cap = torch.full(tau_hat.shape, float("-inf"))
        for b, row in enumerate(pages):
            for h, ids in enumerate(row):
                ids = ids[ids < n_local].long()
                if ids.numel():
                    cap[b, h] = (self.mu[b, h, ids] + zc * self.sigma[b, h, ids] * 0.3333333333333333).max()
        return cap

    def clamp(self, cap):
        a = self.alpha - 1.0
        upper = torch.maximum(a * cap - 1e-4, self.tau_floor)
        self.tau = torch.where(torch.isfinite(cap), torch.minimum(self.tau, upper), self.tau)
        return self.tau

    def _scores(self):
        B, Hq = self.q.shape[:2]
        G = Hq // self.c.k_cache.shape[1]
        S = self.c.seq_len
        out = {}
        for b in range(B):
            for h in range(Hq):
                ids = [int(x) for x in self.pages[b][h]]
                T = len(ids) * P if not self.is_last else max(len(ids) - 1, 0) * P + og.last_page_size(S, P)
                rows = od.token_rows(np.asarray(ids), T, P) if ids else np.zeros(0, dtype=np.int64)
                rows_t = torch.from_numpy(rows)
                z = od.scores_z(self.q[b, h, 0], self.c.k_cache[b, h // G][rows_t], self.alpha)
                out[b, h] = (z, rows_t)
        return out

    def halley_sums(self):
        self.z = self._scores()
        B, Hq = self.q.shape[:2]
        s = torch.zeros(B, Hq, 3)
        for (b, h), (z, _) in self.z.items():
            s[b, h] = torch.tensor(od._power_sums(z, float(self.tau[b, h]), self.alpha))
        return s

    def halley_update(self, sums):
        for b in range(self.tau.shape[0]):
            for h in range(self.tau.shape[1]):
                self.tau[b, h] = od.halley_unbounded(float(self.tau[b, h]), sums[b, h].tolist(), self.alpha)
        return self.tau

    def partial_out(self):
        B, Hq, _, D = self.q.shape
        G = Hq // self.c.k_cache.shape[1]
        out = torch.zeros(B, Hq, 1, D)
        for (b, h), (z, rows) in self.z.items():
            p = od.weights(z, float(self.tau[b, h]), self.alpha)
            nz = np.nonzero(p)[0]
            v = self.c.v_cache[b, h // G][rows[nz]].double().numpy()
            out[b, h, 0] = torch.from_numpy((p[nz][:, None] * v).sum(0)).float()
        return out


def _inputs():
    return H.cpu_inputs(2, 4, 2, 32, 24 * P + 5, torch.float32, seed=7, needle_pages=(3, 17), page_size=P)


def _worker(rank, world, port, q):
    from entmaxkv_b200 import sharded
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        inp = _inputs()
        S = inp["k"].shape[2]
        lo, hi = sharded.split_pages(S, P, world)[rank]
        shard = OracleShard(rank, world, lo // P)
        shard.initialize(inp["k"][:, :, lo:hi], inp["v"][:, :, lo:hi])
        shard.set_global_lengths([S] * inp["q"].shape[0])
        outs = sharded.sharded_gaussian_decode_step(
            [shard], sharded.dist_reduce(), [inp["q"]], [inp["k_new"]], [inp["v_new"]], alpha=ALPHA)
        if rank == 0:
            q.put((outs[0].numpy(), shard.tau.numpy()))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.timeout(300)
def test_two_gloo_ranks_reproduce_the_unsharded_oracle():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out, tau = q.get(timeout=240)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    ref = H.oracle_gaussian_step(_inputs(), P, ALPHA, tau_mode="corrected", iters=1)
    np.testing.assert_allclose(tau, ref["tau"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(out[:, :, 0], ref["out"], rtol=1e-4, atol=1e-5)


def test_page_split_covers_the_sequence_with_whole_pages():
    from entmaxkv_b200.sharded import split_pages
    for total in (16, 100, 1000, 1048577):
        for world in (1, 2, 4, 8):
            if total // P < world:
                # a rank holding nothing but the in-progress page would give it statistics: refused
                with pytest.raises(ValueError):
                    split_pages(total, P, world)
                continue
            parts = split_pages(total, P, world)
            assert parts[0][0] == 0 and parts[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            assert all((hi - lo) % P == 0 for lo, hi in parts[:-1])


def test_local_reduce_matches_elementwise_definitions():
    from entmaxkv_b200.sharded import local_reduce
    a, b = torch.tensor([1.0, -float("inf")]), torch.tensor([2.0, 3.0])
    assert local_reduce([a, b], "sum")[0].tolist() == [3.0, -float("inf")]
    assert local_reduce([a, b], "max")[1].tolist() == [2.0, 3.0]


# ---- failures made on the host ------------------------------------------------------------

def _worker_with_absent_peer(rank, world, port, q):
    """Rank 1 joins the group and then leaves without contributing to the first reduction."""
    import datetime
    from entmaxkv_b200 import sharded
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        q.put(("left", 1))
        return                      # never reduces, never tears the group down
    inp = _inputs()
    S = inp["k"].shape[2]
    lo, hi = sharded.split_pages(S, P, world)[rank]
    shard = OracleShard(rank, world, lo // P)
    shard.initialize(inp["k"][:, :, lo:hi], inp["v"][:, :, lo:hi])
    shard.set_global_lengths([S] * inp["q"].shape[0])
    try:
        sharded.sharded_gaussian_decode_step([shard], sharded.dist_reduce(), [inp["q"]], [inp["k_new"]],
                                             [inp["v_new"]], alpha=ALPHA)
        q.put(("finished", 0))
    except Exception as e:          # the reduction must end with an error, not hang
        q.put(("error", type(e).__name__))


@pytest.mark.timeout(120)
def test_a_rank_that_never_contributes_ends_the_step_with_an_error():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_with_absent_peer, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    seen = dict(q.get(timeout=90) for _ in range(2))
    for p in procs:
        p.join(30)
    assert "left" in seen and "error" in seen and "finished" not in seen, seen


def test_inner_ranks_must_hold_whole_pages_and_worlds_are_bounded():
    from entmaxkv_b200 import sharded
    from entmaxkv_b200.exchange import PeerExchange
    sh = sharded.GpuSequenceShard(P, 0, 2)
    k = torch.zeros(1, 2, P + 3, 32)
    with pytest.raises(ValueError):
        sh.initialize(k, k)                       # rank 0 of 2 with a ragged tail: refused before any GPU work
    with pytest.raises(ValueError):
        PeerExchange(0, 9)                        # more ranks than an exchange supports
    with pytest.raises(ValueError):
        sharded.sharded_gaussian_decode_step([], None, [], [], [], tau_mode="exact")
