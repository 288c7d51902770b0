"""Peer exchange object of the sequence-sharded step (host side of ``ekv_exchange_*``).

One ``PeerExchange`` per process (= per GPU).  Creation allocates this rank's inbox on the
current device, passes its 64-byte memory handle to the other ranks through the process
group and maps theirs; after that the four reductions of a sharded Gaussian step run as
four kernels that store to the peers' inboxes over NVLink and wait, with an iteration
limit, on their own - no collective library call is on the step's path.

The reference is single-GPU and has nothing comparable.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib


class PeerTimeout(RuntimeError):
    """A rank gave up waiting for another rank's contribution to an exchange."""


class PeerExchange:
    def __init__(self, rank: int, world: int, max_floats: int = 1 << 16, group=None,
                 device: Optional[torch.device] = None, connect: bool = True):
        if not 1 <= world <= _lib.EXCHANGE_MAX_RANKS:
            raise ValueError(f"world size must be 1..{_lib.EXCHANGE_MAX_RANKS}")
        self.rank, self.world, self.max_floats, self.group = rank, world, int(max_floats), group
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        lib = _lib.load()
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.ekv_exchange_create(rank, world, self.max_floats, C.byref(h)), "ekv_exchange_create")
        self._h = h
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        if world > 1 and connect:
            self._connect_through_group()

    # -- set-up ---------------------------------------------------------------------
    def _connect_through_group(self):
        import torch.distributed as dist
        lib = _lib.load()
        mine = (C.c_char * _lib.EXCHANGE_HANDLE_BYTES)()
        _lib.check(lib.ekv_exchange_handle(self._h, mine), "ekv_exchange_handle")
        local = torch.frombuffer(bytearray(mine.raw), dtype=torch.uint8).to(self.device)
        everyone = torch.empty(self.world * _lib.EXCHANGE_HANDLE_BYTES, dtype=torch.uint8, device=self.device)
        dist.all_gather_into_tensor(everyone, local, group=self.group)
        raw = bytes(everyone.cpu().numpy().tobytes())
        with torch.cuda.device(self.device):
            _lib.check(lib.ekv_exchange_connect(self._h, raw), "ekv_exchange_connect")
        dist.barrier(group=self.group)          # every inbox is zeroed and mapped before first use

    def base_pointer(self) -> int:
        return _lib.load().ekv_exchange_base(self._h)

    def connect_pointers(self, bases):
        """Same-process set-up: ``bases[r]`` is rank r's ``base_pointer()``."""
        arr = (C.c_void_p * self.world)(*bases)
        _lib.check(_lib.load().ekv_exchange_connect_pointers(self._h, arr), "ekv_exchange_connect_pointers")

    def set_spin_limit(self, iterations: int):
        _lib.check(_lib.load().ekv_exchange_set_spin_limit(self._h, int(iterations)), "ekv_exchange_set_spin_limit")

    # -- calls ------------------------------------------------------------------------
    @property
    def handle(self):
        if self._h is None:
            raise RuntimeError("exchange is closed")
        return self._h

    def all_reduce(self, src: torch.Tensor, op: str = "sum", slot: int = 0) -> torch.Tensor:
        assert src.dtype == torch.float32 and src.is_contiguous()
        dst = torch.empty_like(src)
        _lib.check(_lib.load().ekv_exchange_allreduce(
            self.handle, slot, src.data_ptr(), dst.data_ptr(), src.numel(),
            _lib.XCH_MAX if op == "max" else _lib.XCH_SUM, self.status.data_ptr(), _lib.stream_ptr()),
            "ekv_exchange_allreduce")
        return dst

    def check(self):
        """Raise if any exchange since the last check timed out (synchronises)."""
        st = int(self.status.item())
        if st & _lib.STATUS_PEER_TIMEOUT:
            self.status.zero_()
            raise PeerTimeout(f"rank {self.rank}: a peer did not contribute to an exchange in time")

    def close(self):
        """Free the inbox.  Every rank must be past its last exchange (barrier on the host first)."""
        if self._h is not None:
            torch.cuda.synchronize(self.device)
            with torch.cuda.device(self.device):
                _lib.load().ekv_exchange_destroy(self._h)
            self._h = None
