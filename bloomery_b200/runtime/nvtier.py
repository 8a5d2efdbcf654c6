"""Routed experts paged from a drive: side file writer and the arena handle.

The side file keeps every routed expert in its resident layout, one 4,096-aligned blob per
(layer, expert) = gate rows | up rows | down rows, so a miss is one contiguous direct read with nothing
to convert.  ``NvmeTier`` opens it, holds ``n_slots`` experts per layer in a RAM arena (least recently
used out, pins stay) and plugs into the host tier's service thread, which then answers the card's
hand-offs from the arena.  The C++ side is ``csrc/host/moe_cpu.cpp`` (``NvTier``).

The reference's NVMe expert tier: ``crates/gpu/src/host/nvtier.rs`` (RAM arena of expert slots filled by
O_DIRECT reads on reader threads, LRU / heat eviction, pins, a mirror side file in card layout).
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Dict, List, Optional

import numpy as np
import torch

from ..formats.resident import WT
from ..ops._lib import host

ALIGN = 4096


def _pad(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def write_sidecar(weights, path: str) -> Dict[str, object]:
    """Write the routed experts of ``weights`` (a :class:`Weights` on any device) to ``path`` (+ ``.json`` index)."""
    s = weights.spec
    layers = [il for il in range(s.n_layer + s.n_mtp) if f"blk.{il}.ffn_gate_exps.weight" in weights.q]
    if not layers:
        raise ValueError("this model has no routed experts")
    g0 = weights.q[f"blk.{layers[0]}.ffn_gate_exps.weight"]
    E, I_, K = g0.data.shape[0], g0.rows, g0.k
    gbytes = g0.data.shape[1] * g0.data.shape[2]
    gpart = _pad(gbytes)
    index = {"version": 1, "n_expert": E, "hidden": K, "inter": I_, "gate_type": g0.qtype, "gate_part": gpart, "layers": {}}
    with open(path, "wb") as f:
        off = 0
        for il in layers:
            g, u, d = (weights.q[f"blk.{il}.ffn_{p}_exps.weight"] for p in ("gate", "up", "down"))
            if (g.qtype, u.qtype) != (g0.qtype, g0.qtype):
                raise ValueError(f"layer {il}: gate / up types differ from layer {layers[0]}'s")
            dbytes = d.data.shape[1] * d.data.shape[2]
            blob = 2 * gpart + _pad(dbytes)
            index["layers"][str(il)] = {"offset": off, "down_type": d.qtype, "blob": blob}
            buf = np.zeros((E, blob), dtype=np.uint8)
            buf[:, :gbytes] = g.data.reshape(E, -1).cpu().numpy()
            buf[:, gpart:gpart + gbytes] = u.data.reshape(E, -1).cpu().numpy()
            buf[:, 2 * gpart:2 * gpart + dbytes] = d.data.reshape(E, -1).cpu().numpy()
            f.write(buf.tobytes())
            off += E * blob
    json.dump(index, open(path + ".json", "w"))
    return index


class NvmeTier:
    def __init__(self, path: str, n_slots: int, n_readers: int = 4):
        self.index = json.load(open(path + ".json"))
        ix = self.index
        self.layer_ids = sorted(int(k) for k in ix["layers"])
        self.n_layers = max(self.layer_ids) + 1
        L = ix["layers"]
        offs = (ctypes.c_long * self.n_layers)(*[int(L[str(l)]["offset"]) if str(l) in L else 0 for l in range(self.n_layers)])
        first = L[str(self.layer_ids[0])]
        dts = (ctypes.c_int * self.n_layers)(*[WT[(L.get(str(l)) or first)["down_type"]] for l in range(self.n_layers)])
        self.E, self.K, self.I = ix["n_expert"], ix["hidden"], ix["inter"]
        self.n_slots = min(n_slots, self.E)
        lib = host()
        lib.blh_nv_open.restype = ctypes.c_void_p
        self.h = lib.blh_nv_open(path.encode(), self.n_layers, offs, dts, self.E, self.n_slots, self.K, self.I,
                                 WT[ix["gate_type"]], n_readers)
        if not self.h:
            raise OSError(f"{path}: the side file could not be opened as an expert arena")
        self.lib = lib
        self.arena_bytes = sum(self.n_slots * L[str(l)]["blob"] for l in self.layer_ids)

    def moe(self, layer: int, ids: torch.Tensor, wts: torch.Tensor, xq: torch.Tensor, xds: torch.Tensor) -> torch.Tensor:
        """The expert leg of ``layer`` for M rows from the arena (loads what is missing first)."""
        M, k = ids.shape
        out = torch.zeros(M, self.K)
        ids, wts, xq, xds = ids.contiguous(), wts.contiguous(), xq.contiguous(), xds.contiguous()
        rc = self.lib.blh_nv_moe_experts(ctypes.c_void_p(self.h), layer, M, k, ctypes.c_void_p(ids.data_ptr()),
                                         ctypes.c_void_p(wts.data_ptr()), ctypes.c_void_p(xq.data_ptr()),
                                         ctypes.c_void_p(xds.data_ptr()), ctypes.c_void_p(out.data_ptr()))
        if rc != 0:
            raise OSError(f"expert arena: layer {layer} could not be served (code {rc})")
        return out

    def pin(self, layer: int, expert: int, on: bool = True) -> None:
        if self.lib.blh_nv_pin(ctypes.c_void_p(self.h), layer, expert, 1 if on else 0) != 0:
            raise OSError(f"expert arena: cannot pin expert {expert} of layer {layer}")

    def resident(self, layer: int) -> List[int]:
        buf = (ctypes.c_int * self.n_slots)()
        n = self.lib.blh_nv_resident(ctypes.c_void_p(self.h), layer, buf)
        return sorted(buf[i] for i in range(n))

    def stats(self) -> Dict[str, int]:
        v = (ctypes.c_uint64 * 7)()
        self.lib.blh_nv_stats(ctypes.c_void_p(self.h), v)
        return {"hits": v[0], "misses": v[1], "evictions": v[2], "bytes_read": v[3], "read_ns": v[4], "failed": v[5],
                "direct_io": bool(v[6])}

    def attach(self, host_tier) -> None:
        """Let the host tier's service thread answer the card from this arena."""
        self.lib.blh_host_tier_set_nv(host_tier.handle, ctypes.c_void_p(self.h))

    def close(self) -> None:
        if self.h:
            self.lib.blh_nv_close(ctypes.c_void_p(self.h))
            self.h = None
