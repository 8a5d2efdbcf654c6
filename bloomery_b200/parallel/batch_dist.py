"""Batched decode over the GPUs of one node: every rank runs the attention half on all the rows, the routed experts are
split by index, and the experts' partial rows meet in a deterministic all-reduce.

Why this shape.  A pass of 16 to 64 rows is bound by streaming the weights, and almost all of them are routed experts
(16.5 of 17 GB on the Qwen3-30B-A3B shape): splitting the experts divides the bytes every rank streams by the rank
count.  The attention half (0.4 GB) is cheaper to repeat than to split, and with the rows replicated the experts need
no dispatch at all -- every rank already holds every row, routes it identically, plans only the rows of ITS experts
(``localize_ids`` + ``moe_plan``), runs the quantised-weight GEMMs on them and produces partial rows.  A shared expert
and the dense layers of a DeepSeek-style model are split by width; their partial rows ride the same exchange.  The
combine is the only exchange of a layer:

    push_rows           my partial rows [M, H] fp32 into slot ``rank`` of every peer's gather buffer (plain peer stores)
    rank_barrier_step   bounded flag barrier whose epoch comes from a device-side pass counter (CUDA-graph replayable)
    sum_ranks           x += slot 0 + slot 1 + ... in rank order: the same bits on every rank

Two gather buffers alternate by layer, so a rank that runs ahead never writes the buffer a peer is still adding up.
The reference has no counterpart (its several-card split keeps one request per pass).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..ops import gemm as G
from ..runtime.batch_decode import BatchDecode
from .symm import SymmetricBuffer


class ShardedBatchDecode(BatchDecode):
    """``engine``: a :class:`DecodeEngine` whose weights hold the whole attention half and this rank's experts
    (``synth_tensors(shard=(rank, world), shard_attn=False)`` / ``shard_items(..., attn=False)``) under a spec that
    still names ALL the experts."""

    def __init__(self, engine, rank: int, world: int, group=None, max_rows: int = 64, local_only: bool = False):
        super().__init__(engine, max_rows)
        s = engine.spec
        if not s.is_moe or s.n_expert % world:
            raise ValueError(f"{world} ranks do not divide {s.n_expert} experts")
        self.rank, self.world = rank, world
        self.e_per = s.n_expert // world
        dev = engine.device
        R, H = self.R, s.hidden
        self.slot_floats = R * H
        self.buf_bytes = world * self.slot_floats * 4
        self.off_flags = 2 * self.buf_bytes
        self.sym = SymmetricBuffer(self.off_flags + 256, rank, world, dev, group, local_only=local_only)
        self.emulated = local_only
        self.pass_counter = torch.zeros(1, dtype=torch.int32, device=dev)  # passes so far: the barrier epochs' base
        self.partial = torch.zeros(R, H, dtype=torch.float32, device=dev)
        self.ids_loc = torch.zeros(R, s.n_used, dtype=torch.int32, device=dev)
        self.moe_tiles = G.TileTable(R * s.n_used, self.e_per, dev, self.moe_tiles.tile_rows)
        self.sites = s.n_layer

    def embed(self, M: int, x: torch.Tensor) -> None:
        from ..ops import decode as K
        e = self.e
        K.embed_rows(self.tokens, M, e.w.q["token_embd.weight"], e.spec.vocab, x, e.fault, self.pass_counter)   # bumps the pass counter

    def _exchange(self, il: int, M: int, x: torch.Tensor):
        """The layer's one exchange: x += the sum over ranks of ``partial``, in rank order."""
        H = self.e.spec.hidden
        half = (il & 1) * self.buf_bytes
        mine = half + self.rank * self.slot_floats * 4
        G.push_rows(self.partial, [p_ + mine for p_ in self.sym.ptrs], M * H * 4)
        yield 1
        n = 0
        yield None                                   # every rank has pushed before any rank adds
        if not (self.emulated or self.world == 1):
            G.rank_barrier_step(self.sym.peers(self.off_flags), self.sym.ptrs[self.rank] + self.off_flags, self.pass_counter,
                                self.sites, il, self.rank, self.status); n += 1
        gathered = self.sym.view(half, (self.world, self.slot_floats), torch.float32)
        G.sum_ranks(gathered, self.slot_floats, self.world, x, M * H); n += 1
        yield n

    def dense_ffn(self, il: int, M: int, x: torch.Tensor, xn: torch.Tensor, tiles):
        """This rank's slice of the dense width, then the exchange."""
        w = self.e.w
        b = f"blk.{il}."
        n = self._mm(xn, w.q[b + "ffn_gate.weight"], tiles, M, W2=w.q[b + "ffn_up.weight"], out_bf16=self.dact[:M])
        yield n + self._mm(self.dact[:M], w.q[b + "ffn_down.weight"], tiles, M, out_f32=self.partial[:M])
        yield from self._exchange(il, M, x)

    def experts(self, il: int, M: int, x: torch.Tensor, xn: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, tiles):
        e = self.e
        s, w = e.spec, e.w
        b = f"blk.{il}."
        k, El = s.n_used, self.e_per
        n = 0
        G.localize_ids(ids, self.rank * El, (self.rank + 1) * El, self.ids_loc[:M]); n += 1
        G.moe_plan(self.ids_loc[:M], wts, El, self.moe_tiles, self.pos_of, self.dst_row, self.row_scale); n += 1
        G.gather_rows_bf16(xn, self.dst_row, self.moe_tiles.offsets[El:El + 1], self.cap, k, self.Ap); n += 1
        qg, qu, qd = (w.q[b + f"ffn_{nm}_exps.weight"] for nm in ("gate", "up", "down"))
        n += self._mm(self.Ap, qg, self.moe_tiles, M, W2=qu, out_bf16=self.act)
        n += self._mm(self.act, qd, self.moe_tiles, M, out_f32=self.slot_out, dst_row=self.dst_row, row_scale=self.row_scale)
        G.moe_combine(self.slot_out, self.pos_of, M, k, None, self.partial[:M]); n += 1        # this rank's share, no residual
        if s.n_shared:
            # this rank's slice of the shared expert's width rides the same exchange
            n += self.shared_expert(il, M, xn, tiles, self.partial[:M], self.partial[:M])
        yield n
        yield from self._exchange(il, M, x)


def lockstep(ranks: List[ShardedBatchDecode], M: int, advance: bool = False) -> None:
    """Walk several emulated ranks of one process through a pass in lockstep (tests): every rank runs to the next
    meeting point before any rank goes on."""
    gens = [bd.enqueue_steps(M, advance) for bd in ranks]
    live = list(gens)
    while live:
        nxt = []
        for g in live:
            try:
                next(g)
                nxt.append(g)
            except StopIteration:
                pass
        live = nxt
