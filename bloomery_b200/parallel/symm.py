"""Symmetric receive buffers for the fused all-reduce: every rank owns the same layout and
holds a pointer to every peer's copy (NVLink peer memory, reached with plain loads/stores
from inside the kernels).

The plumbing uses ``torch.distributed`` only: the buffers come from
``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged over the process
group); if that is unavailable the legacy CUDA IPC handles of ``torch`` storages are
exchanged with ``all_gather_object``.  The kernels never see NCCL.

Layout per rank (bytes):  recv  [2 sites][N ranks][8 rows][H] fp32
                          flags [2 sites][N ranks] u32          (128-byte aligned)
                          seq   [2] u32, ticket [2] u32          (local use only)
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
        self.recv_bytes = 2 * world * MAX_ROWS * hidden * 4
        self.flag_off = (self.recv_bytes + 127) // 128 * 128
        self.total = self.flag_off + 256
        self._keep = []
        if world == 1 or local_only:
            self.buf = torch.zeros(self.total, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.buf.data_ptr()] * world
            self.how = "local"
        else:
            self.buf, self.ptrs, self.how = self._exchange(group)
        # local bookkeeping words: seq[2], ticket[2]
        self.words = torch.zeros(8, dtype=torch.int32, device=self.device)

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
        return base + ((site * self.world + slot) * MAX_ROWS * self.H) * 4

    def local_slot(self, site: int) -> torch.Tensor:
        """This rank's own slot of its own receive buffer, as fp32 [8, H]."""
        off = ((site * self.world + self.rank) * MAX_ROWS * self.H) * 4
        return self.buf[off:off + MAX_ROWS * self.H * 4].view(torch.float32).view(MAX_ROWS, self.H)

    def push(self, site: int, rows: int) -> PushOut:
        p = PushOut()
        p.local = self._recv(self.ptrs[self.rank], site, self.rank)
        for r in range(self.world):
            p.peer_recv[r] = self._recv(self.ptrs[r], site, self.rank)
            p.peer_flag[r] = self.ptrs[r] + self.flag_off + (site * self.world + self.rank) * 4
        p.seq = self.words.data_ptr() + site * 4
        p.ticket = self.words.data_ptr() + (2 + site) * 4
        p.n_ranks, p.my_rank, p.n_floats = self.world, self.rank, rows * self.H
        return p

    def reduce(self, site: int, x_out: torch.Tensor, fault: Optional[torch.Tensor], layer: int) -> ReduceIn:
        r = ReduceIn()
        r.recv = self._recv(self.ptrs[self.rank], site, 0)
        r.flags = self.ptrs[self.rank] + self.flag_off + site * self.world * 4
        r.seq = self.words.data_ptr() + site * 4
        r.x_out = x_out.data_ptr()
        r.x_out_stride = x_out.stride(0)
        r.n_ranks, r.H = self.world, self.H
        r.fault = fault.data_ptr() if fault is not None else 0
        r.layer = layer
        return r
