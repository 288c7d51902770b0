"""Paged KV cache with per-page key statistics, resident in HBM and updated in place.

Drop-in for the reference ``PagedKVCache`` (entmaxkv/kv_cache.py:16-255):
same constructor, ``initialize`` / ``append``, and the attributes callers read
(``page_size``, ``k_cache``, ``v_cache``, ``k_min``, ``k_max``, ``k_mean``,
``k_std``, ``last_num_selected_per_head``).

Differences a user can observe:
  * K/V and the statistics live in capacity-sized buffers; ``append`` writes one
    row and refreshes one statistics row per (batch, head) instead of
    concatenating the whole cache (kv_cache.py:81-82).  The public attributes are
    views ``[:, :, :seq_len]`` of those buffers, hence non-contiguous across heads.
  * sequence lengths are kept on the device (``seq_lens``), one per batch row, so a
    batch may be ragged (``initialize(..., seq_lens=...)``) and a decode step needs
    no host synchronisation.
  * ``PagedKVCache(page_size, block_table=True)`` stores K and V as a POOL of physical blocks of
    ``page_size`` rows ([num_blocks, H_kv, page_size, D]) addressed through a per-sequence block
    table, the layout serving engines hand out (the reference cache is dense,
    kv_cache.py:44-56).  Pages of one sequence are then not contiguous in memory; the page
    statistics stay dense.  ``k_cache`` / ``v_cache`` are gathered copies in that mode.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib


class PagedKVCache:
    """KV cache with min/max/mean/std statistics per page of ``page_size`` keys."""

    #: rows of head-room added when a capacity is chosen automatically
    DEFAULT_HEADROOM = 1024

    def __init__(self, page_size: int = 16, capacity: Optional[int] = None, block_table: bool = False,
                 block_order: str = "interleaved"):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if block_order not in ("interleaved", "random"):
            raise ValueError("block_order must be 'interleaved' or 'random'")
        self.page_size = int(page_size)
        self._requested_capacity = capacity
        #: K/V live in a pool of physical blocks behind a block table (see the module docstring)
        self.block_mode = bool(block_table)
        self._block_order = block_order
        self._table = None                     # int32 [B, page_capacity]: page -> physical block
        self._pool_k = self._pool_v = None     # [num_blocks, H_kv, page_size, D]
        self._k = self._v = None
        self._meta = None                      # [4, B, H, page_capacity, D]: min, max, mean, std
        self.seq_lens: Optional[torch.Tensor] = None     # int32 [B] on the device
        self._host_lens: list[int] = []
        self._ctl = None                       # int32: [0]=status, [16:16+B] append tickets
        self.last_num_selected_per_head = None
        self._scratch: dict = {}
        self._desc = None

    # ------------------------------------------------------------------ state

    @property
    def seq_len(self) -> int:
        """Longest sequence of the batch (the reference's ``k_cache.shape[2]``)."""
        return max(self._host_lens) if self._host_lens else 0

    @property
    def host_seq_lens(self) -> list[int]:
        return list(self._host_lens)

    @property
    def is_ragged(self) -> bool:
        return len(set(self._host_lens)) > 1

    @property
    def capacity(self) -> int:
        return 0 if self._k is None else self._k.shape[2]

    @property
    def page_capacity(self) -> int:
        return 0 if self._meta is None else self._meta.shape[3]

    @property
    def num_pages(self) -> int:
        return (self.seq_len + self.page_size - 1) // self.page_size

    def _view_rows(self, t, pool=None):
        if t is None:
            return None
        if self.block_mode:      # gather the sequence's blocks back into [B, H, S, D] (a copy)
            B, H, _, D = t.shape
            n = self.num_pages
            blocks = pool[self._table[:, :n].reshape(-1).long()]                 # [B*n, H, P, D]
            dense = blocks.view(B, n, H, self.page_size, D).permute(0, 2, 1, 3, 4).reshape(B, H, n * self.page_size, D)
            return dense[:, :, :self.seq_len]
        return t[:, :, :self.seq_len]

    @property
    def k_cache(self):
        return self._view_rows(self._k, self._pool_k)

    @property
    def v_cache(self):
        return self._view_rows(self._v, self._pool_v)

    def _meta_view(self, i):
        return None if self._meta is None else self._meta[i][:, :, :self.num_pages]

    @property
    def k_min(self):
        return self._meta_view(0)

    @property
    def k_max(self):
        return self._meta_view(1)

    @property
    def k_mean(self):
        return self._meta_view(2)

    @property
    def k_std(self):
        return self._meta_view(3)

    # ------------------------------------------------------------------ build

    def _allocate(self, B, H, D, capacity, dtype, device):
        P = self.page_size
        capacity = (capacity + P - 1) // P * P
        self._k = torch.empty(B, H, capacity, D, dtype=dtype, device=device)
        self._v = torch.empty(B, H, capacity, D, dtype=dtype, device=device)
        self._meta = torch.zeros(4, B, H, capacity // P, D, dtype=dtype, device=device)
        self._desc = None
        if self.block_mode:
            # the same memory seen as a pool of B * page_capacity blocks; _k / _v keep their dense SHAPE
            # (the wrappers read sizes from it) but their rows are only meaningful through the table
            pcap = capacity // P
            self._pool_k = self._k.view(B * pcap, H, P, D)
            self._pool_v = self._v.view(B * pcap, H, P, D)
            old = self._table
            table = torch.empty(B, pcap, dtype=torch.int32, device=device)
            if self._block_order == "interleaved":     # consecutive pages of a sequence lie B blocks apart
                table.copy_((torch.arange(pcap, device=device)[None, :] * B +
                             torch.arange(B, device=device)[:, None]).to(torch.int32))
            else:
                n_old = 0 if old is None else old.numel()
                if old is not None:
                    table[:, :old.shape[1]] = old
                g = torch.Generator(device="cpu").manual_seed(1234 + n_old)
                fresh = (torch.randperm(B * pcap - n_old, generator=g) + n_old).to(torch.int32).to(device)
                pcap_old = 0 if old is None else old.shape[1]
                table[:, pcap_old:] = fresh.view(B, pcap - pcap_old)
            self._table = table

    def initialize(self, k: torch.Tensor, v: torch.Tensor,
                   seq_lens: Optional[Sequence[int]] = None, capacity: Optional[int] = None):
        """Copy prefill keys/values in and build every page's statistics in one launch.

        k, v: [B, H_kv, S, D] (kv_cache.py:40-70).  ``seq_lens`` (optional, length B)
        gives the valid length of each row of a padded, ragged batch.
        """
        _lib.require_cuda(k, v)
        if k.shape != v.shape or k.dim() != 4:
            raise ValueError("k and v must both be [batch, kv_heads, seq_len, head_dim]")
        _lib.dtype_code(k.dtype)
        B, H, S, D = k.shape
        lens = [S] * B if seq_lens is None else [int(x) for x in seq_lens]
        if len(lens) != B or min(lens) < 1 or max(lens) > S:
            raise ValueError("seq_lens must hold one length in [1, S] per batch row")
        cap = capacity or self._requested_capacity or (S + self.DEFAULT_HEADROOM)
        if cap < S:
            raise ValueError("capacity is smaller than the prefill length")
        self._table = None
        self._allocate(B, H, D, cap, k.dtype, k.device)
        if self.block_mode:
            self._scatter_pages(k, v)
        else:
            self._k[:, :, :S].copy_(k)
            self._v[:, :, :S].copy_(v)
        self._host_lens = lens
        self.seq_lens = torch.tensor(lens, dtype=torch.int32, device=k.device)
        self._ctl = torch.zeros(16 + B, dtype=torch.int32, device=k.device)
        self._scratch = {}
        lib = _lib.load()
        _lib.check(lib.ekv_page_stats_init(C.byref(self.desc()), max(lens), _lib.stream_ptr()),
                   "ekv_page_stats_init")

    def _scatter_pages(self, k, v):
        """Block mode: copy [B, H, S, D] tensors page by page into the blocks the table assigns."""
        B, H, S, D = k.shape
        P = self.page_size
        n = (S + P - 1) // P
        ids = self._table[:, :n].reshape(-1).long()
        for src, pool in ((k, self._pool_k), (v, self._pool_v)):
            if n * P != S:
                src = torch.cat([src, src.new_zeros(B, H, n * P - S, D)], dim=2)
            pool[ids] = src.view(B, H, n, P, D).permute(0, 2, 1, 3, 4).reshape(B * n, H, P, D)

    def translate(self, page_indices: torch.Tensor, counts: torch.Tensor, out: Optional[torch.Tensor] = None):
        """Block mode: page numbers -> physical block ids for the first ``counts[b, h]`` entries of every
        row of a page table ([B, H_q, width] int32); the decode kernels address K/V by block id."""
        if out is None:
            out = self.scratch("phys_" + str(page_indices.shape[2]), tuple(page_indices.shape), torch.int32)
        lib = _lib.load()
        _lib.check(lib.ekv_translate_pages(C.byref(self.desc()), page_indices.shape[1], page_indices.data_ptr(),
                                           page_indices.stride(1), counts.data_ptr(), out.data_ptr(),
                                           out.stride(1), _lib.stream_ptr()), "ekv_translate_pages")
        return out

    def reserve(self, capacity: int):
        """Grow the buffers so that ``capacity`` rows fit (copies the cache once)."""
        if self._k is None:
            self._requested_capacity = capacity
            return
        if capacity <= self.capacity:
            return
        B, H, _, D = self._k.shape
        old_k, old_v, old_meta, S = self._k, self._v, self._meta, self.seq_len
        old_pools = (self._pool_k, self._pool_v)
        self._allocate(B, H, D, capacity, old_k.dtype, old_k.device)
        if self.block_mode:
            if self._block_order == "interleaved":
                # block ids p*B + b do not depend on the capacity: the old blocks keep their numbers
                n_old = old_pools[0].shape[0]
                self._pool_k[:n_old].copy_(old_pools[0])
                self._pool_v[:n_old].copy_(old_pools[1])
            else:
                n_old = old_pools[0].shape[0]      # old table entries were kept, new pages got new blocks
                self._pool_k[:n_old].copy_(old_pools[0])
                self._pool_v[:n_old].copy_(old_pools[1])
        else:
            self._k[:, :, :S].copy_(old_k[:, :, :S])
            self._v[:, :, :S].copy_(old_v[:, :, :S])
        self._meta[:, :, :, :old_meta.shape[3]].copy_(old_meta)
        self._scratch = {}

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor):
        """Append one token per sequence (k_new, v_new: [B, H_kv, 1, D]); kv_cache.py:72-116."""
        if self._k is None:
            raise RuntimeError("initialize() the cache before append()")
        _lib.require_cuda(k_new, v_new)
        B, H, _, D = self._k.shape
        if tuple(k_new.shape) != (B, H, 1, D) or tuple(v_new.shape) != (B, H, 1, D):
            raise ValueError(f"k_new / v_new must be [{B}, {H}, 1, {D}]")
        if k_new.dtype != self._k.dtype or v_new.dtype != self._k.dtype:
            raise ValueError("k_new / v_new dtype differs from the cache dtype")
        if k_new.stride(-1) != 1 or v_new.stride(-1) != 1 or k_new.stride() != v_new.stride():
            k_new, v_new = k_new.contiguous(), v_new.contiguous()
        if self.seq_len + 1 > self.capacity:
            self.reserve(max(self.capacity + 4096, self.capacity * 5 // 4))
        lib = _lib.load()
        _lib.check(lib.ekv_append(C.byref(self.desc()), k_new.data_ptr(), v_new.data_ptr(),
                                  k_new.stride(0), k_new.stride(1),
                                  self._ctl[16:].data_ptr(), self._ctl.data_ptr(), _lib.stream_ptr()),
                   "ekv_append")
        self._host_lens = [n + 1 for n in self._host_lens]

    # ------------------------------------------------------------------ C ABI view

    def desc(self) -> _lib.CacheDesc:
        """The plain-C description of this cache that every entry point takes."""
        if self._desc is None:
            k, m = self._k, self._meta
            d = _lib.CacheDesc()
            d.k, d.v = k.data_ptr(), self._v.data_ptr()
            d.k_min, d.k_max, d.k_mean, d.k_std = (m[i].data_ptr() for i in range(4))
            d.kv_stride_b, d.kv_stride_h = k.stride(0), k.stride(1)
            d.meta_stride_b, d.meta_stride_h = m.stride(1), m.stride(2)
            d.batch, d.kv_heads, d.head_dim = k.shape[0], k.shape[1], k.shape[3]
            d.page_size, d.capacity, d.page_capacity = self.page_size, k.shape[2], m.shape[3]
            d.dtype = _lib.dtype_code(k.dtype)
            if self.block_mode:
                P, H, D = self.page_size, k.shape[1], k.shape[3]
                d.kv_stride_b, d.kv_stride_h = 0, P * D
                d.block_table, d.bt_stride = self._table.data_ptr(), self._table.stride(0)
                d.kv_stride_block, d.num_blocks = H * P * D, self._pool_k.shape[0]
            self._desc = d
        self._desc.seq_lens = self.seq_lens.data_ptr()
        return self._desc

    def scratch(self, name: str, shape, dtype, zero: bool = False) -> torch.Tensor:
        """Persistent per-cache scratch tensor, reallocated only when its shape changes."""
        key = (name, tuple(shape), dtype)
        t = self._scratch.get(key)
        if t is None:
            for old in [k for k in self._scratch if k[0] == name]:
                del self._scratch[old]
            make = torch.zeros if zero else torch.empty
            t = make(tuple(shape), dtype=dtype, device=self._k.device)
            self._scratch[key] = t
        return t

    def device_status(self) -> int:
        """Status bits raised by device-side range checks of cache updates, plus ``COPY_TIMEOUT`` (16) when
        any bulk copy of this process timed out in one of the library's kernels (synchronises)."""
        bits = int(self._ctl[0].item())
        n = C.c_uint32(0)
        _lib.check(_lib.load().ekv_copy_timeouts(C.byref(n)), "ekv_copy_timeouts")
        return bits | (16 if n.value else 0)

    # ------------------------------------------------------------------ scoring helper

    def estimate_page_criticality(self, q: torch.Tensor, use_triton: bool = True,
                                  alibi_slopes=None, q_pos: int = 0,
                                  exclude_last_page: bool = False) -> torch.Tensor:
        """Key-range upper-bound score of every page, [B, H_q, pages] in q.dtype.

        kv_cache.py:118-165.  Only the decode-step form (last page excluded) exists
        as a kernel.  With ``alibi_slopes`` ([H_q]) the page bonus ``slope * (last position of
        the page - q_pos)`` is added (``q_pos``: an int for all sequences).
        """
        if not exclude_last_page:
            raise NotImplementedError("only exclude_last_page=True is implemented")
        from .attention_topk import _alibi_args, _score_and_select
        alibi = None
        if alibi_slopes is not None:
            B, Hq = q.shape[0], q.shape[1]
            q_len = torch.full((B,), int(q_pos) + 1, dtype=torch.int32, device=q.device)
            alibi = _alibi_args(alibi_slopes, q_len, B, Hq, q.device)
        scores = _score_and_select(q, self, token_budget=0, cache_seqlens=None, alibi=alibi)[0]
        return scores[:, :, :max(self.num_pages - 1, 0)]

    # ------------------------------------------------------------------ helpers kept from the reference object

    def select_gaussian_aware(self, q: torch.Tensor, alpha: float = 1.5, safety_margin_z: float = 0.0,
                              max_quantile: float = 0.99, gaussian_stats: Optional[dict] = None):
        """Gaussian-aware page selection on its own (kv_cache.py:205-255).

        Returns ``(page_indices int32 [B, H_q, pages], num_selected int32 [B, H_q])``: per head the
        selected pages in ascending order with the in-progress last page in the final valid slot; only
        the first ``num_selected`` entries of a row are meaningful.  ``safety_margin_z`` and
        ``max_quantile`` are derived from the batch's mean sigma exactly as the decode wrapper does, so
        the arguments have no effect (as in the reference, where the statistics dictionary overrides
        them).  Of ``gaussian_stats`` only ``threshold_excess_margin_fraction`` and
        ``tau_clamp_page_max_quantile`` are read; the statistics themselves are recomputed on the
        device (one sweep) rather than taken from the dictionary.  The statistics and tau_floor of the
        call stay in ``last_gaussian_selection``.
        """
        from .attention_gaussian import gaussian_select
        stats = gaussian_stats or {}
        frac = stats.get("threshold_excess_margin_fraction", 0.1)
        frac = 0.1 if frac is None else frac
        sel = gaussian_select(q, self, alpha, frac, stats.get("tau_clamp_page_max_quantile", 0.5),
                              apply_clamp=False)
        self.last_num_selected_per_head = sel["num_selected"]
        self.last_gaussian_selection = sel
        return sel["page_indices"], sel["num_selected"]

    def get_page_indices_buf(self, batch: int, num_heads: int, num_pages_to_select: int,
                             last_page_idx: int) -> torch.Tensor:
        """Persistent int32 ``[B, H, n_selected + 1]`` page table whose last column holds
        ``last_page_idx`` (kv_cache.py:167-185).  The wrappers of this library fill their own table
        on the device; the method exists for callers that build page tables themselves."""
        buf = self.scratch("user_page_indices", (batch, num_heads, num_pages_to_select + 1), torch.int32)
        buf[:, :, num_pages_to_select].fill_(last_page_idx)
        return buf

    def get_paged_decode_workspace(self, batch: int, nheads: int, dim: int, max_splits: int = 32,
                                   bins: int = 16, dtype: torch.dtype = None, device=None) -> dict:
        """The decode workspace for one shape (kv_cache.py:187-203).  The reference returns a dictionary
        of Triton intermediates; here it is one byte buffer sized by ``ekv_decode_workspace_bytes``
        (``max_splits`` and ``bins`` do not apply: splits follow the 256-token work list and the
        histogram lives in shared memory)."""
        from .attention_topk import _decode_workspace
        return {"workspace": _decode_workspace(self, batch, nheads, dim, self.capacity)}
