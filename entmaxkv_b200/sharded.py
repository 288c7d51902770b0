"""Sequence-page sharding of one long request across GPUs (Gaussian-aware decode).

Rank r of R owns a contiguous range of pages of every (batch row, KV head); the in-progress
last page lives on the last rank.  Because the entmax output ``sum_i p_i(tau) v_i`` is linear
in V once tau is fixed, a decode step needs only four tiny reductions:

    1. per-head moment sums            all-reduce SUM  [B, H_q, 4]
    2. clamp cap of the selected pages all-reduce MAX  [B, H_q]
    3. Halley sums at the clamped tau  all-reduce SUM  [B, H_q, 3]   (corrected mode)
    4. partial outputs                 all-reduce SUM  [B, H_q, D] fp32

Everything else (moments sweep, threshold selection, K pass, V pass) is local to a rank and
uses the same kernels as the single-GPU path, through the stage entry points of the C ABI.

The step is written once, over "shards" that implement the stage methods, and a ``reduce``
callable.  In a distributed run a process holds one ``GpuSequenceShard`` and ``reduce`` is an
NCCL (or gloo) all-reduce; the same function drives several shards inside one process with a
local reduction, which is how the logic is tested on one device and, with CPU shards built on
the test oracle, on CPU ranks.
"""

from __future__ import annotations

import ctypes as C
from typing import Callable, List, Sequence

import torch

from . import _lib
from .attention_gaussian import _z_of_quantile, grouped_enabled
from .attention_topk import _check_q_out, _decode_workspace
from .kv_cache import PagedKVCache

Reduce = Callable[[List[torch.Tensor], str], List[torch.Tensor]]


def local_reduce(tensors: List[torch.Tensor], op: str) -> List[torch.Tensor]:
    """Reduction over the shards held by this process (single-process emulation of R ranks)."""
    stacked = torch.stack([t.to(tensors[0].device) for t in tensors])
    red = stacked.sum(0) if op == "sum" else stacked.amax(0)
    return [red.to(t.device) for t in tensors]


def dist_reduce(group=None) -> Reduce:
    """All-reduce across processes; each process holds exactly one shard."""
    import torch.distributed as dist
    ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX}

    def reduce(tensors, op):
        assert len(tensors) == 1, "one shard per process in a distributed run"
        t = tensors[0].contiguous()
        dist.all_reduce(t, op=ops[op], group=group)
        return [t]
    return reduce


def split_pages(total_tokens: int, page_size: int, world: int) -> list[tuple[int, int]]:
    """Token ranges [start, stop) per rank: whole pages, as even as possible, remainder
    (and the in-progress last page) on the last rank."""
    full_pages = total_tokens // page_size
    if full_pages < world:
        # a rank left with the in-progress page alone would count it as a statistical page,
        # which the unsharded step does not
        raise ValueError(f"{total_tokens} tokens hold {full_pages} full pages: too few for {world} ranks")
    base, extra = divmod(full_pages, world)
    out, start = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * page_size
        stop = start + n if r < world - 1 else total_tokens
        out.append((start, stop))
        start = stop
    return out


class GpuSequenceShard:
    """One rank's slice of the cache plus the stage calls of the C ABI on it."""

    def __init__(self, page_size: int, rank: int, world: int):
        self.cache = PagedKVCache(page_size)
        self.rank, self.world = rank, world
        self.is_last = rank == world - 1

    def initialize(self, k_local: torch.Tensor, v_local: torch.Tensor, capacity=None):
        if not self.is_last and k_local.shape[2] % self.cache.page_size:
            raise ValueError("every rank but the last must hold whole pages")
        self.cache.initialize(k_local, v_local, capacity=capacity)

    # ---- stages -------------------------------------------------------------------

    def append(self, k_new, v_new):
        if self.is_last:
            self.cache.append(k_new, v_new)
        self.global_len.add_(1)

    def _common(self, q):
        c = self.cache
        B, Hq, _, D = q.shape
        return c, _lib.load(), C.byref(c.desc()), _lib.stream_ptr(), B, Hq, D

    def moments(self, q, alpha):
        c, lib, desc, st, B, Hq, D = self._common(q)
        self.q, self.alpha = q, float(alpha)
        pcap = c.page_capacity
        self.mu = c.scratch("g_mu", (B, Hq, pcap), torch.float32)
        self.sigma = c.scratch("g_sigma", (B, Hq, pcap), torch.float32)
        self.head_sums = c.scratch("g_head_sums", (B, Hq, 4), torch.float32)
        wsb = lib.ekv_gaussian_workspace_bytes(B, Hq, pcap)
        gws = c.scratch("g_ws", (wsb,), torch.uint8, zero=True)
        _lib.check(lib.ekv_gaussian_moments(
            desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, c.capacity, int(self.is_last), self.alpha, 0,
            self.mu.data_ptr(), self.sigma.data_ptr(), pcap, self.head_sums.data_ptr(), None,
            gws.data_ptr(), wsb, st), "ekv_gaussian_moments")
        return self.head_sums

    def set_global_lengths(self, total_tokens: Sequence[int]):
        """Global sequence lengths (all ranks' tokens), kept on the device and bumped by append()."""
        self.global_len = torch.tensor(list(total_tokens), dtype=torch.int32, device=self.cache._k.device)

    def finalize(self, head_sums):
        c, lib, desc, st, B, Hq, D = self._common(self.q)
        self.head_stats = c.scratch("g_head_stats", (B, Hq, 4), torch.float32)
        _lib.check(lib.ekv_gaussian_finalize_from_lengths(
            head_sums.data_ptr(), self.global_len.data_ptr(), c.page_size, B, Hq, self.alpha,
            self.head_stats.data_ptr(), st), "ekv_gaussian_finalize_from_lengths")
        return self.head_stats

    def select(self, excess_margin_fraction=0.2, clamp_quantile=0.5):
        c, lib, desc, st, B, Hq, D = self._common(self.q)
        P, pcap = c.page_size, c.page_capacity
        self.pages = c.scratch("g_pages", (B, Hq, pcap), torch.int32)
        self.counts = c.scratch("g_counts", (B, Hq), torch.int32)
        self.tokens = c.scratch("g_tokens", (B, Hq), torch.int32)
        self.tau_floor = c.scratch("g_tau_floor", (B, Hq), torch.float32)
        self.cap = c.scratch("g_cap", (B, Hq), torch.float32)
        self.tau = c.scratch("g_tau", (B, Hq), torch.float32)
        nch = (c.capacity + 255) // 256
        self.work = c.scratch("g_work", (B * Hq * nch,), torch.int64)
        self.work_total = c.scratch("g_work_total", (2 + (B * Hq + 1023) // 1024,), torch.int32, zero=True)
        _lib.check(lib.ekv_gaussian_select(
            desc, Hq, c.capacity, int(self.is_last), int(self.is_last), self.alpha, float(excess_margin_fraction),
            _z_of_quantile(0.99, P), _z_of_quantile(0.995, P), _z_of_quantile(float(clamp_quantile), P), 0, None,
            self.mu.data_ptr(), self.sigma.data_ptr(), pcap, self.head_stats.data_ptr(), self.pages.data_ptr(),
            pcap, self.counts.data_ptr(), self.tokens.data_ptr(), self.tau_floor.data_ptr(), self.cap.data_ptr(),
            self.tau.data_ptr(), self.work.data_ptr(), self.work_total.data_ptr(), st), "ekv_gaussian_select")
        return self.cap

    def clamp(self, cap_max):
        lib, st = _lib.load(), _lib.stream_ptr()
        n = self.tau.numel()
        # tau currently holds tau_hat (selection ran with apply_clamp = 0)
        _lib.check(lib.ekv_tau_clamp(self.tau.data_ptr(), 1, cap_max.data_ptr(), self.tau_floor.data_ptr(), n,
                                     self.alpha, 1.0e-4, self.tau.data_ptr(), st), "ekv_tau_clamp")
        return self.tau

    def halley_sums(self):
        c, lib, desc, st, B, Hq, D = self._common(self.q)
        q = self.q
        self.ws = _decode_workspace(c, B, Hq, D, c.capacity)
        self.sums = c.scratch("g_halley", (B, Hq, 3), torch.float32)
        self.sums.zero_()     # heads without local tokens contribute nothing
        _lib.check(lib.ekv_decode_scores(
            desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, self.pages.data_ptr(), self.pages.stride(1),
            self.tokens.data_ptr(), c.capacity, self.alpha, _lib.TAU_NONE, 0, self.tau.data_ptr(),
            self.sums.data_ptr(), self.work.data_ptr(), self.work.numel(), self.work_total.data_ptr(),
            self.ws.data_ptr(), self.ws.numel(), st), "ekv_decode_scores")
        return self.sums

    def halley_update(self, sums):
        lib, st = _lib.load(), _lib.stream_ptr()
        _lib.check(lib.ekv_halley_update(self.tau.data_ptr(), sums.data_ptr(), self.tau.numel(), self.alpha, st),
                   "ekv_halley_update")
        return self.tau

    def partial_out(self):
        c, lib, desc, st, B, Hq, D = self._common(self.q)
        self.partial = c.scratch("g_partial", (B, Hq, 1, D), torch.float32)
        _lib.check(lib.ekv_decode_values(
            desc, Hq, self.pages.data_ptr(), self.pages.stride(1), self.tokens.data_ptr(), c.capacity,
            self.alpha, self.tau.data_ptr(), self.partial.data_ptr(), self.partial.stride(0),
            self.partial.stride(1), 1, self.work.data_ptr(), self.work.numel(), self.work_total.data_ptr(),
            self.ws.data_ptr(), self.ws.numel(), st), "ekv_decode_values")
        return self.partial

    def local_seq_len(self) -> int:
        return self.cache.seq_len

    # ---- the same stages with the reduction done by the consuming kernel (peer exchange) ----

    def moments_x(self, q, alpha, x):
        """Moments sweep whose last blocks trade the head sums with the peers and finish the head
        statistics (tau_hat included): ``moments`` + ``finalize_x`` in one launch for bfloat caches
        with GQA groups of up to eight heads, in two launches otherwise."""
        c, lib, desc, st, B, Hq, D = self._common(q)
        self.q, self.alpha = q, float(alpha)
        pcap = c.page_capacity
        self.mu = c.scratch("g_mu", (B, Hq, pcap), torch.float32)
        self.sigma = c.scratch("g_sigma", (B, Hq, pcap), torch.float32)
        self.head_sums = c.scratch("g_head_sums", (B, Hq, 4), torch.float32)
        self.head_stats = c.scratch("g_head_stats", (B, Hq, 4), torch.float32)
        wsb = lib.ekv_gaussian_workspace_bytes(B, Hq, pcap)
        gws = c.scratch("g_ws", (wsb,), torch.uint8, zero=True)
        _lib.check(lib.ekv_exchange_gaussian_moments(
            x.handle, desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, c.capacity, int(self.is_last), self.alpha,
            self.global_len.data_ptr(), self.mu.data_ptr(), self.sigma.data_ptr(), pcap, self.head_sums.data_ptr(),
            self.head_stats.data_ptr(), gws.data_ptr(), wsb, x.status.data_ptr(), st), "ekv_exchange_gaussian_moments")

    def select_x(self, x, excess_margin_fraction=0.2, clamp_quantile=0.5, apply_clamp=True):
        """Threshold selection that also trades the clamp cap with the peers and clamps tau with the
        world's maximum: ``select`` + ``clamp_x`` in one launch."""
        c, lib, desc, st, B, Hq, D = self._common(self.q)
        P, pcap = c.page_size, c.page_capacity
        self.pages = c.scratch("g_pages", (B, Hq, pcap), torch.int32)
        self.counts = c.scratch("g_counts", (B, Hq), torch.int32)
        self.tokens = c.scratch("g_tokens", (B, Hq), torch.int32)
        self.tau_floor = c.scratch("g_tau_floor", (B, Hq), torch.float32)
        self.cap = c.scratch("g_cap", (B, Hq), torch.float32)
        self.tau = c.scratch("g_tau", (B, Hq), torch.float32)
        nch = (c.capacity + 255) // 256
        self.work = c.scratch("g_work", (B * Hq * nch,), torch.int64)
        self.work_total = c.scratch("g_work_total", (2 + (B * Hq + 1023) // 1024,), torch.int32, zero=True)
        grouped = grouped_enabled(self.q, c)       # decode_x then builds its lists from the groups' unions
        _lib.check(lib.ekv_exchange_gaussian_select(
            x.handle, desc, Hq, c.capacity, int(self.is_last), int(self.is_last), self.alpha,
            float(excess_margin_fraction), _z_of_quantile(0.99, P), _z_of_quantile(0.995, P),
            _z_of_quantile(float(clamp_quantile), P), int(bool(apply_clamp)), None, self.mu.data_ptr(),
            self.sigma.data_ptr(), pcap, self.head_stats.data_ptr(), self.pages.data_ptr(), pcap,
            self.counts.data_ptr(), self.tokens.data_ptr(), self.tau_floor.data_ptr(), self.cap.data_ptr(),
            self.tau.data_ptr(), None if grouped else self.work.data_ptr(),
            None if grouped else self.work_total.data_ptr(), x.status.data_ptr(), st),
            "ekv_exchange_gaussian_select")

    def finalize_x(self, x):
        c, lib, desc, st, B, Hq, D = self._common(self.q)
        self.head_stats = c.scratch("g_head_stats", (B, Hq, 4), torch.float32)
        _lib.check(lib.ekv_exchange_gaussian_finalize(
            x.handle, self.head_sums.data_ptr(), self.global_len.data_ptr(), c.page_size, B, Hq, self.alpha,
            self.head_stats.data_ptr(), x.status.data_ptr(), st), "ekv_exchange_gaussian_finalize")

    def clamp_x(self, x):
        lib, st = _lib.load(), _lib.stream_ptr()
        _lib.check(lib.ekv_exchange_tau_clamp(
            x.handle, self.tau.data_ptr(), self.cap.data_ptr(), self.tau_floor.data_ptr(), self.tau.numel(),
            self.alpha, 1.0e-4, x.status.data_ptr(), st), "ekv_exchange_tau_clamp")

    def halley_update_x(self, x):
        lib, st = _lib.load(), _lib.stream_ptr()
        _lib.check(lib.ekv_exchange_halley_update(
            x.handle, self.tau.data_ptr(), self.sums.data_ptr(), self.tau.numel(), self.alpha,
            x.status.data_ptr(), st), "ekv_exchange_halley_update")

    def decode_x(self, x, niter: int, out=None):
        """K pass, tau kernel (sums traded with the peers, Halley step, gather), V pass, and the
        fold + exchange of the partial outputs: four launches (``ekv_exchange_decode``)."""
        c, lib, desc, st, B, Hq, D = self._common(self.q)
        q = self.q
        self.ws = _decode_workspace(c, B, Hq, D, c.capacity)
        self.partial = c.scratch("g_partial", (B, Hq, 1, D), torch.float32)
        if out is None:
            out = c.scratch("g_out_full", (B, Hq, 1, D), torch.float32)
        if out.shape != (B, Hq, 1, D) or out.stride(3) != 1:
            raise ValueError("out must be [B, H_q, 1, D] with a contiguous last dimension")
        if grouped_enabled(q, c):
            # GQA groups of four or eight: the shard's page tables merged into one per group, every K row fetched
            # once (one small launch ahead of the K pass, as in the unsharded step)
            Hkv, pcap = c._k.shape[1], c.page_capacity
            cph = lib.ekv_work_items_per_head(c.capacity)
            u_pages = c.scratch("gu_pages", (B, Hq, pcap), torch.int32)
            member = c.scratch("gu_member", (B, Hkv, pcap), torch.uint8)
            u_tok = c.scratch("gu_tokens", (B, Hq), torch.int32)
            g_items = c.scratch("gu_group_items", (B * Hkv * cph,), torch.int64)
            h_items = c.scratch("gu_head_items", (B * Hq * cph,), torch.int64)
            _lib.check(lib.ekv_group_union(
                desc, Hq, self.pages.data_ptr(), self.pages.stride(1), self.counts.data_ptr(), c.capacity,
                u_pages.data_ptr(), u_pages.stride(1), member.data_ptr(), member.stride(1), u_tok.data_ptr(),
                g_items.data_ptr(), g_items.numel(), h_items.data_ptr(), st), "ekv_group_union")
            _lib.check(lib.ekv_exchange_decode_grouped(
                x.handle, desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, u_pages.data_ptr(), u_pages.stride(1),
                u_tok.data_ptr(), c.capacity, self.alpha, int(niter), self.tau.data_ptr(), self.partial.data_ptr(),
                out.data_ptr(), out.stride(0), out.stride(1), _lib._DTYPES[out.dtype], h_items.data_ptr(),
                h_items.numel(), g_items.data_ptr(), g_items.numel(), member.data_ptr(), member.stride(1),
                self.ws.data_ptr(), self.ws.numel(), x.status.data_ptr(), st), "ekv_exchange_decode_grouped")
            return out
        _lib.check(lib.ekv_exchange_decode(
            x.handle, desc, q.data_ptr(), q.stride(0), q.stride(1), Hq, self.pages.data_ptr(), self.pages.stride(1),
            self.tokens.data_ptr(), c.capacity, self.alpha, int(niter), self.tau.data_ptr(),
            self.partial.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1), _lib._DTYPES[out.dtype],
            self.work.data_ptr(), self.work.numel(), self.work_total.data_ptr(), self.ws.data_ptr(),
            self.ws.numel(), x.status.data_ptr(), st), "ekv_exchange_decode")
        return out

    def output_x(self, x, out=None):
        c, lib, desc, st, B, Hq, D = self._common(self.q)
        if out is None:
            out = c.scratch("g_out_full", (B, Hq, 1, D), torch.float32)
        if out.shape != (B, Hq, 1, D) or out.stride(3) != 1 or out.stride(0) != Hq * out.stride(1):
            raise ValueError("out must be [B, H_q, 1, D] with contiguous heads")
        _lib.check(lib.ekv_exchange_output(
            x.handle, self.partial.data_ptr(), B * Hq, D, out.data_ptr(), out.stride(1),
            _lib._DTYPES[out.dtype], x.status.data_ptr(), st), "ekv_exchange_output")
        return out


def sharded_gaussian_decode_step(shards: list, reduce: Reduce, q_per_shard: list, k_new, v_new,
                                 alpha: float = 1.5, tau_mode: str = "corrected", clamp_tau: bool = True,
                                 excess_margin_fraction: float = 0.2, clamp_quantile: float = 0.5,
                                 append_cache: bool = True, exchange=None, out=None):
    """One Gaussian-aware decode step over a sequence-sharded cache.

    shards: the shards this process drives (one in a distributed run), each initialised and told the
    global sequence lengths (``set_global_lengths``).  q_per_shard / k_new / v_new: the step's inputs on
    each shard's device.  Returns the list of full outputs (fp32 [B, H_q, 1, D]), one per local shard,
    identical everywhere.  With ``exchange`` (a ``PeerExchange``; distributed runs only) the four
    reductions run inside the consuming kernels over peer memory instead of through ``reduce``, and
    ``out`` may name the [B, H_q, 1, D] tensor (any supported dtype) that receives the result.  Mirrors entmaxkv/attention_gaussian.py:58-142 with the reductions listed in
    the module docstring.  Nothing here reads device memory from the host, so the whole step -
    collectives included - can be captured into a CUDA graph.
    """
    if tau_mode not in ("fixed", "corrected"):
        raise ValueError("sequence-sharded decode supports tau_mode 'fixed' and 'corrected'")
    if append_cache:
        for s, kn, vn in zip(shards, k_new, v_new):
            s.append(kn, vn)
    if exchange is not None:
        # one shard per process; every reduction is done by the kernel that needs its result
        (s,), (q,) = shards, q_per_shard
        s.moments_x(q, alpha, exchange)
        s.select_x(exchange, excess_margin_fraction, clamp_quantile, apply_clamp=clamp_tau)
        return [s.decode_x(exchange, 1 if tau_mode == "corrected" else 0, out)]
    sums = reduce([s.moments(q, alpha) for s, q in zip(shards, q_per_shard)], "sum")
    for s, t in zip(shards, sums):
        s.finalize(t)
    caps = reduce([s.select(excess_margin_fraction, clamp_quantile) for s in shards], "max")
    if clamp_tau:
        for s, cap in zip(shards, caps):
            s.clamp(cap)
    if tau_mode == "corrected":
        hs = reduce([s.halley_sums() for s in shards], "sum")
        for s, t in zip(shards, hs):
            s.halley_update(t)
    else:
        for s in shards:
            s.halley_sums()      # the K pass also produces the scores the V pass needs
    return reduce([s.partial_out() for s in shards], "sum")


class ShardedStepGraph:
    """The sharded step of one rank (kernels and NCCL all-reduces) captured as one CUDA graph.

    Drop the object (or call ``release()``) before destroying the process group: tearing a
    communicator down while a graph still holds its captured collectives blocks.
    """

    def __init__(self, shard: GpuSequenceShard, reduce: Reduce, q_heads: int, alpha: float = 1.5,
                 tau_mode: str = "corrected", exchange=None):
        self.shard, self.reduce, self.alpha, self.tau_mode = shard, reduce, alpha, tau_mode
        self.exchange = exchange
        k = shard.cache._k
        B, Hkv, _, D = k.shape
        # q | k_new | v_new are views of one buffer: the host-to-host step moves them with one copy node
        nq, nk = B * q_heads * D, B * Hkv * D
        self._in = torch.zeros(nq + 2 * nk, dtype=k.dtype, device=k.device)
        self._split = lambda flat: (flat[:nq].view(B, q_heads, 1, D), flat[nq:nq + nk].view(B, Hkv, 1, D),
                                    flat[nq + nk:].view(B, Hkv, 1, D))
        self.q, self.k_new, self.v_new = self._split(self._in)
        self.graph = None
        self.out = None
        self._pinned = None          # host-I/O variant: page-locked staging buffers and their graph
        self.graph_io = None
        self.out_io = None

    def release(self):
        self.graph = None
        self.graph_io = None

    def _run(self, append: bool):
        return sharded_gaussian_decode_step([self.shard], self.reduce, [self.q], [self.k_new], [self.v_new],
                                            alpha=self.alpha, tau_mode=self.tau_mode, append_cache=append,
                                            exchange=self.exchange)[0]

    def _capture(self, with_io: bool):
        cache = self.shard.cache
        # two eager passes without the append allocate every scratch buffer and warm NCCL up
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._run(append=False)
            self._run(append=False)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        lens = list(cache._host_lens)
        g = torch.cuda.CUDAGraph()
        # thread-local capture mode: the process group's watchdog thread keeps polling its
        # events while this thread captures
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            if with_io:
                self._in.copy_(self._pinned_in, non_blocking=True)
            out = self._run(append=True)
            if with_io:
                self._pinned["out"].copy_(out, non_blocking=True)
        cache._host_lens = lens      # the capture itself appended nothing
        if with_io:
            self.graph_io, self.out_io = g, out
        else:
            self.graph, self.out = g, out

    def _replay(self, g):
        cache = self.shard.cache
        if self.shard.is_last and cache.seq_len + 1 > cache.capacity:
            raise RuntimeError("the captured step cannot grow the cache; reserve capacity up front")
        g.replay()
        if self.shard.is_last:
            cache._host_lens = [n + 1 for n in cache._host_lens]

    def step(self, q, k_new, v_new):
        from .graph import stage_inputs
        stage_inputs(((self.q, q), (self.k_new, k_new), (self.v_new, v_new)))
        if self.graph is None:
            self._capture(with_io=False)
        self._replay(self.graph)
        return self.out

    def pinned_io(self) -> dict:
        """Page-locked host buffers ``q``, ``k_new``, ``v_new`` (the caller writes a step's inputs there) and
        ``out`` (fp32 [B, H_q, 1, D]: ``step_pinned`` leaves the result there)."""
        if self._pinned is None:
            B, Hq, _, D = self.q.shape
            self._pinned_in = torch.empty(self._in.shape, dtype=self._in.dtype).pin_memory()
            hq, hk, hv = self._split(self._pinned_in)
            self._pinned = {"q": hq, "k_new": hk, "v_new": hv,
                            "out": torch.empty(B, Hq, 1, D, dtype=torch.float32).pin_memory()}
        return self._pinned

    def step_pinned(self) -> torch.Tensor:
        """The step with its inputs in ``pinned_io()`` and its output copied back there, the copies being nodes
        of the replayed graph (one launch per step from the host).  The returned pinned tensor is valid once the
        current stream has been synchronised."""
        io = self.pinned_io()
        if self.graph_io is None:
            self.q.copy_(io["q"], non_blocking=True)      # the capture's eager passes run on the real query
            self.k_new.copy_(io["k_new"], non_blocking=True)
            self.v_new.copy_(io["v_new"], non_blocking=True)
            self._capture(with_io=True)
        self._replay(self.graph_io)
        return io["out"]
