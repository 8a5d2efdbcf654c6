"""Symmetric receive buffers for the fused all-reduce: every rank owns the same layout and
holds a pointer to every peer's copy (NVLink peer memory, reached with plain loads/stores
from inside the kernels).

The plumbing uses ``torch.distributed`` only: the buffers come from
``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged over the process
group); if that is unavailable the legacy CUDA IPC handles of ``torch`` storages are
exchanged with ``all_gather_object``.  The kernels never see NCCL.

Layout per rank:  recv [2 sites][N ranks][8 rows][H] of {value bits, epoch} (8 bytes each).
The epoch rides in every element, so there are no separate flags.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops.decode import PushOut, ReduceIn

MAX_RANKS = 8
MAX_ROWS = 8


class SymmetricArena:
    def __init__(self, hidden: int, rank: int, world: int, device, group=None, local_only: bool = False,
                 peers: Optional[List["SymmetricArena"]] = None):
        if world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks per node")
        self.H, self.rank, self.world = hidden, rank, world
        self.device = torch.device(device)
        self.recv_bytes = 2 * world * MAX_ROWS * hidden * 8
        self.total = self.recv_bytes + 256
        self._keep = []
        if world == 1 or local_only:
            self.buf = torch.zeros(self.total, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.buf.data_ptr()] * world
            self.how = "local"
        else:
            self.buf, self.ptrs, self.how = self._exchange(group)
        # pass counter: the first kernel of every pass bumps it; epochs derive from it
        self.step = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sites_per_step = 2

    def adopt_peers(self, arenas: List["SymmetricArena"]) -> None:
        """Single-process emulation: point at other arenas on the same device (tests)."""
        self.ptrs = [a.buf.data_ptr() for a in arenas]

    def _exchange(self, group):
        group = group or dist.group.WORLD
        try:
            import torch.distributed._symmetric_memory as symm_mem
            buf = symm_mem.empty(self.total, dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(buf, group)
            buf.zero_()
            ptrs = [int(x) for x in hdl.buffer_ptrs]
            self._keep.append(hdl)
            torch.cuda.synchronize(self.device)
            dist.barrier(group)
            return buf, ptrs, "symmetric_memory"
        except Exception as exc:  # noqa: BLE001 - fall back to legacy IPC handles
            self._symm_error = repr(exc)
        buf = torch.zeros(self.total, dtype=torch.uint8, device=self.device)
        handle = buf.untyped_storage()._share_cuda_()
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handle, group=group)
        ptrs = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                ptrs.append(buf.data_ptr())
                continue
            st = torch.UntypedStorage._new_shared_cuda(*h)
            t = torch.empty(0, dtype=torch.uint8, device=st.device).set_(st)
            self._keep.append(t)
            ptrs.append(t.data_ptr())
        torch.cuda.synchronize(self.device)
        dist.barrier(group)
        return buf, ptrs, "cuda_ipc"

    # ---- descriptors -----------------------------------------------------------------
    def _recv(self, base: int, site: int, slot: int) -> int:
        return base + ((site * self.world + slot) * MAX_ROWS * self.H) * 8

    def push(self, site: int, site_index: int) -> PushOut:
        """Producer descriptor: ``site`` picks the buffer (0 attention, 1 MoE), ``site_index``
        numbers the reduction inside the pass (unique per pass)."""
        p = PushOut()
        for r in range(self.world):
            p.peer_recv[r] = self._recv(self.ptrs[r], site, self.rank)
        p.step = self.step.data_ptr()
        p.sites_per_step, p.site_index = self.sites_per_step, site_index
        p.n_ranks, p.my_rank = self.world, self.rank
        return p

    def reduce(self, site: int, site_index: int, x_out: torch.Tensor, fault: Optional[torch.Tensor], layer: int) -> ReduceIn:
        r = ReduceIn()
        r.recv = self._recv(self.ptrs[self.rank], site, 0)
        r.step = self.step.data_ptr()
        r.sites_per_step, r.site_index = self.sites_per_step, site_index
        r.x_out = x_out.data_ptr()
        r.x_out_stride = x_out.stride(0)
        r.n_ranks, r.H = self.world, self.H
        r.fault = fault.data_ptr() if fault is not None else 0
        r.layer = layer
        return r


class SymmetricBuffer:
    """A byte buffer that exists on every rank with the same layout; ``ptrs[r]`` is rank r's copy as seen from
    this process (peer memory for r != rank).  ``local_only`` gives an ordinary buffer whose peers are set
    later with :meth:`adopt_peers` (several emulated ranks in one process)."""

    def __init__(self, n_bytes: int, rank: int, world: int, device, group=None, local_only: bool = False):
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.total = (n_bytes + 255) // 256 * 256
        self._keep = []
        if world == 1 or local_only:
            self.buf = torch.zeros(self.total, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.buf.data_ptr()] * world
            self.how = "local"
        else:
            self.H = 0
            self.buf, self.ptrs, self.how = SymmetricArena._exchange(self, group)

    def adopt_peers(self, bufs: List["SymmetricBuffer"]) -> None:
        self.ptrs = [b.buf.data_ptr() for b in bufs]

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        nb = n * torch.empty(0, dtype=dtype).element_size()
        return self.buf[offset:offset + nb].view(dtype).view(*shape)

    def peers(self, offset: int) -> List[int]:
        return [p_ + offset for p_ in self.ptrs]
