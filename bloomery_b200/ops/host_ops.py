"""Python face of ``libbloomery_host.so`` (CPU quantised dots, pool, CPU expert leg)."""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from ..formats.resident import WT, resident_row_bytes
from ._lib import F, I, L, host, p


def act_q8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 [M, K] (CPU) -> (codes int8 [M, K], ds fp32 [M, K/32, 2]) with the device's rounding."""
    x = x.contiguous().float()
    m, k = x.shape
    codes = torch.empty(m, k, dtype=torch.int8)
    ds = torch.empty(m, k // 32, 2, dtype=torch.float32)
    host().blh_act_q8(p(x), I(m), I(k), p(codes), p(ds))
    return codes, ds


def gemv(w_res: torch.Tensor, qtype: str, k: int, codes: torch.Tensor, ds: torch.Tensor) -> torch.Tensor:
    """out[m, r] = W[r] . act[m] over resident rows on the CPU pool."""
    rows = w_res.shape[0]
    assert w_res.shape[1] == resident_row_bytes(qtype, k)
    m = codes.shape[0]
    out = torch.empty(m, rows, dtype=torch.float32)
    rc = host().blh_gemv(I(WT[qtype]), p(w_res), I(rows), I(k), p(codes), p(ds), I(m), p(out), L(rows))
    if rc != 0:
        raise ValueError(f"blh_gemv refused type {qtype} k={k}")
    return out


def decode_rows(w_res: torch.Tensor, qtype: str, k: int) -> torch.Tensor:
    rows = w_res.shape[0]
    out = torch.empty(rows, k, dtype=torch.float32)
    rc = host().blh_decode_rows(I(WT[qtype]), p(w_res), I(rows), I(k), p(out))
    if rc != 0:
        raise ValueError(f"blh_decode_rows refused type {qtype}")
    return out


def pool_size() -> int:
    return int(host().blh_pool_size())


def pool_configure(threads: int = 0, pin: bool = True, spin: int = 20000) -> int:
    """Apply the host-pool levers (size, CPU pinning, spins before a worker parks); returns the pool size."""
    h = host()
    h.blh_pool_set_spin(I(int(spin)))
    h.blh_pool_set_pin(I(1 if pin else 0))
    if threads > 0 and threads != int(h.blh_pool_size()):
        h.blh_pool_resize(I(int(threads)))
    return int(h.blh_pool_size())
