"""Replay a whole decode step (append -> select -> decode) as one CUDA graph.

A decode step is five short kernels; launched one by one from Python the GPU waits
for the host between them.  Because sequence lengths live in device memory and all
launch parameters are sized by the cache capacity, the step's launch sequence is
identical from token to token and can be captured once and replayed.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .attention_gaussian import sparse_attention_decode_gaussian_aware_entmax
from .attention_topk import sparse_attention_decode_paged
from .kv_cache import PagedKVCache


def stage_inputs(pairs) -> None:
    """Copy a step's inputs into a captured step's fixed buffers: ``pairs`` = ((dst, src), ...) for q, k_new and
    v_new.  Contiguous device tensors of the right shape and dtype go in ONE launch (``ekv_stage_inputs``);
    anything else - host tensors (the copy engine moves pinned rows faster than a kernel pulling them over PCIe 16
    bytes at a time: 80 against 86 us end to end on the 32k step), strided views, other dtypes - in three copies."""
    if all(s.is_cuda and s.device == d.device and s.dtype == d.dtype and s.shape == d.shape and s.is_contiguous()
           and s.data_ptr() % 16 == 0 and d.numel() * d.element_size() % 16 == 0 for d, s in pairs):
        flat = [x for d, s in pairs for x in (d.data_ptr(), s.data_ptr(), d.numel() * d.element_size())]
        _lib.check(_lib.load().ekv_stage_inputs(*flat, _lib.stream_ptr()), "ekv_stage_inputs")
    else:
        for d, s in pairs:
            d.copy_(s, non_blocking=True)


class _HostAlias:
    """Lets ``torch.as_tensor`` wrap a page-locked host tensor as a CUDA tensor of the same address (unified
    addressing maps page-locked host memory into the device's address space at the same pointer)."""

    def __init__(self, t: torch.Tensor):
        self.keep = t
        self.__cuda_array_interface__ = {"shape": (t.numel() * t.element_size(),), "typestr": "|u1",
                                         "data": (t.data_ptr(), False), "version": 2}


def device_alias(t: torch.Tensor) -> torch.Tensor:
    """A CUDA tensor whose storage IS the page-locked host tensor ``t``: kernels that write it write host memory
    over the bus, with no separate device-to-host copy afterwards."""
    if not t.is_pinned() or not t.is_contiguous():
        raise ValueError("device_alias needs a contiguous page-locked host tensor")
    return torch.as_tensor(_HostAlias(t), device="cuda").view(t.dtype).view(t.shape)


class DecodeStepGraph:
    """Captured decode step over one ``PagedKVCache``.

    mode "topk" replays ``sparse_attention_decode_paged`` and mode "gaussian" replays
    ``sparse_attention_decode_gaussian_aware_entmax``, both with ``append_cache=True``.
    ``step(q, k_new, v_new)`` copies the three inputs (device or pinned host tensors)
    into fixed buffers, replays the graph and returns the fixed output buffer.
    The graph is re-captured automatically when the cache has to grow.
    """

    def __init__(self, kv_cache: PagedKVCache, q_heads: int, mode: str = "topk", *,
                 token_budget: Optional[int] = None, alpha: float = 1.5, niter: int = 2,
                 tau_mode: str = "corrected", **kwargs):
        if mode not in ("topk", "gaussian"):
            raise ValueError("mode must be 'topk' or 'gaussian'")
        if mode == "topk" and token_budget is None:
            raise ValueError("mode='topk' needs token_budget")
        if kv_cache._k is None:
            raise RuntimeError("kv_cache is not initialised")
        self.cache, self.mode = kv_cache, mode
        self.token_budget, self.alpha, self.niter, self.tau_mode = token_budget, alpha, niter, tau_mode
        self.kwargs = kwargs
        B, Hkv, _, D = kv_cache._k.shape
        dt, dev = kv_cache._k.dtype, kv_cache._k.device
        # the three inputs are views of ONE buffer (q | k_new | v_new), on the device and in page-locked host
        # memory alike: the host-to-host step moves them with one copy node instead of three
        self._in_shapes = ((B, q_heads, 1, D), (B, Hkv, 1, D), (B, Hkv, 1, D))
        self._in = torch.zeros(sum(b * h * D for b, h, _, _ in self._in_shapes), dtype=dt, device=dev)
        self.q, self.k_new, self.v_new = self._views(self._in)
        self.out = torch.zeros(B, q_heads, 1, D, dtype=dt, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._captured_capacity = -1
        # host-to-host variant (``step_pinned``): page-locked staging buffers and a graph that holds the three
        # host-to-device copies, the step and the device-to-host copy of the output as nodes
        self._pinned = None
        self._out_alias = None
        self.graph_io: Optional[torch.cuda.CUDAGraph] = None
        self._captured_capacity_io = -1

    def _views(self, flat: torch.Tensor):
        views, at = [], 0
        for shape in self._in_shapes:
            n = shape[0] * shape[1] * shape[3]
            views.append(flat[at:at + n].view(shape))
            at += n
        return views

    def _call(self, append: bool, out: Optional[torch.Tensor] = None):
        out = self.out if out is None else out
        if self.mode == "topk":
            sparse_attention_decode_paged(self.q, self.cache, self.k_new, self.v_new, out,
                                          self.token_budget, alpha=self.alpha, niter=self.niter,
                                          append_cache=append, **self.kwargs)
        else:
            sparse_attention_decode_gaussian_aware_entmax(self.q, self.cache, self.k_new, self.v_new,
                                                          out, alpha=self.alpha, niter=self.niter,
                                                          append_cache=append, tau_mode=self.tau_mode,
                                                          **self.kwargs)

    def _capture(self, with_io: bool = False):
        cache = self.cache
        # one eager pass without the append allocates every scratch buffer outside the capture
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._call(append=False)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        lens = list(cache._host_lens)
        g = torch.cuda.CUDAGraph()
        # a step that holds a collective (``sigma_mean`` given as a callable) is captured in
        # thread-local mode: the process group's watchdog thread keeps polling while this one captures
        mode = "thread_local" if callable(self.kwargs.get("sigma_mean")) else "global"
        with torch.cuda.graph(g, capture_error_mode=mode):
            if with_io:
                self._in.copy_(self._pinned_in, non_blocking=True)
            # host-to-host: the step's last kernel stores the output rows straight into the page-locked buffer
            # (256 KB trickle over the bus while the kernel runs, instead of a copy node after it)
            self._call(append=True, out=self._out_alias if with_io else None)
            if with_io and self._out_alias is None:        # no alias of the host buffer: copy the output back
                self._pinned["out"].copy_(self.out, non_blocking=True)
        cache._host_lens = lens          # the capture itself appended nothing
        if with_io:
            self.graph_io, self._captured_capacity_io = g, cache.capacity
        else:
            self.graph, self._captured_capacity = g, cache.capacity

    def pinned_io(self) -> dict:
        """Page-locked host buffers ``q``, ``k_new``, ``v_new`` (the caller writes a step's inputs there) and
        ``out`` (``step_pinned`` leaves the result there)."""
        if self._pinned is None:
            self._pinned_in = torch.empty(self._in.shape, dtype=self._in.dtype).pin_memory()
            hq, hk, hv = self._views(self._pinned_in)
            self._pinned = {"q": hq, "k_new": hk, "v_new": hv,
                            "out": torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()}
            try:
                self._out_alias = device_alias(self._pinned["out"])
            except (RuntimeError, TypeError, ValueError):      # this torch cannot wrap a host pointer: copy node instead
                self._out_alias = None
        return self._pinned

    def step_pinned(self) -> torch.Tensor:
        """One step whose inputs are in ``pinned_io()`` and whose output goes back there: the input copies are
        one node of the replayed graph and the output is stored by the kernels directly, so the host issues ONE
        launch per step.  Returns the pinned output tensor; it is
        valid once the current stream has been synchronised."""
        cache = self.cache
        io = self.pinned_io()
        if cache.seq_len + 1 > cache.capacity:
            cache.reserve(max(cache.capacity + 4096, cache.capacity * 5 // 4))
        if self.graph_io is None or self._captured_capacity_io != cache.capacity:
            self.q.copy_(io["q"], non_blocking=True)      # the capture's eager warm-up pass runs on the real query
            self._capture(with_io=True)
        self.graph_io.replay()
        cache._host_lens = [n + 1 for n in cache._host_lens]
        return io["out"]

    def step(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor) -> torch.Tensor:
        cache = self.cache
        if cache.seq_len + 1 > cache.capacity:
            cache.reserve(max(cache.capacity + 4096, cache.capacity * 5 // 4))
        # inputs first: the eager warm-up pass of a (re)capture then runs on this step's real query
        # (an all-zero query would make every page pass the Gaussian threshold)
        stage_inputs(((self.q, q), (self.k_new, k_new), (self.v_new, v_new)))
        if self.graph is None or self._captured_capacity != cache.capacity:
            self._capture()
        self.graph.replay()
        cache._host_lens = [n + 1 for n in cache._host_lens]
        return self.out
