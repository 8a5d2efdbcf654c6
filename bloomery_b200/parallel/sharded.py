"""Tensor-parallel attention + expert-parallel MoE decode over the GPUs of one node.

Each rank holds ``n_q / N`` query heads with their KV head(s), the matching K-slice of
o_proj, ``E / N`` routed experts and a ``1 / N`` slice of the width of every dense FFN and
shared expert (rows of gate / up, columns of down); with latent attention the low-rank
projections and the latent cache are replicated and the per-head products (q_b, k_b, v_b)
follow the heads.  Embeddings, norms, router and the output head are replicated (the reference's TP ranks split heads / FFN width and replicate router, norms
and embedding the same way: ``crates/gpu-glm5next/src/tp/mod.rs:5-12``).

Every layer needs two reductions of the residual update (after o_proj, after the
experts).  They are not collectives of their own: the producing kernel pushes its partial
rows into every peer's HBM over NVLink in its last block, and the next kernel's prologue
waits for the N flags and adds the partials in rank order (``csrc/common.cuh``,
"Fused all-reduce").  All ranks therefore hold bit-identical residual rows and pick the same
token without exchanging it.  ``NcclBaseline`` below is the same engine with the two
reductions done by ``torch.distributed.all_reduce`` -- the baseline the fused path is
measured against.
"""
from __future__ import annotations

import dataclasses
import functools
import math
from typing import Iterator, List, Optional

import torch
import torch.distributed as dist

from ..formats.quant import QTYPES
from ..formats.resident import PLANE_TYPES
from ..models.spec import ModelSpec
from ..models.weights import TensorItem, Weights
from ..ops import decode as K
from ..runtime.engine import DecodeEngine
from .symm import SymmetricArena

SITE_ATTN, SITE_MOE = 0, 1


ATTN_NAMES = ("attn_q.weight", "attn_q_b.weight", "attn_k.weight", "attn_v.weight", "attn_k_b.weight", "attn_v_b.weight",
              "attn_output.weight")


def shard_items(items: Iterator[TensorItem], spec: ModelSpec, rank: int, world: int, attn: bool = True) -> Iterator[TensorItem]:
    """Slice a full tensor stream down to one rank's share (raw block bytes, no re-quantisation).  ``attn`` off keeps
    the attention matrices whole on every rank (the replicated-attention engine)."""
    if spec.n_q % world or (spec.is_moe and spec.n_expert % world):
        raise ValueError(f"{world} ranks do not divide {spec.n_q} heads / {spec.n_expert} experts")
    hd = spec.head_dim
    q_lo, q_hi = rank * spec.q_rows // world, (rank + 1) * spec.q_rows // world
    # columns of o_proj: the heads' value rows (head_dim wide, or v_dim with latent attention)
    o_w = spec.n_q * (spec.v_dim if spec.mla else hd)
    o_lo, o_hi = rank * o_w // world, (rank + 1) * o_w // world
    h_lo, h_hi = rank * spec.n_q // world, (rank + 1) * spec.n_q // world

    def k_slice(name, shape, qtype, raw, lo, hi):
        if qtype in PLANE_TYPES:
            # FP8 / NVFP4 items already carry resident rows (codes, then scales): cut both parts of every row
            from ..formats.planes import PlaneError, resident_k_slice
            try:
                return name, (shape[0], hi - lo), qtype, resident_k_slice(raw.reshape(shape[0], -1), qtype, shape[1], lo, hi)
            except PlaneError as exc:
                raise ValueError(f"{name}: {exc}") from None
        qt = QTYPES[qtype]
        bv, bb = qt.block_values, qt.block_bytes
        if lo % bv or hi % bv:
            raise ValueError(f"{name}: a K-slice of {hi - lo} columns does not align to {bv}-value blocks")
        blk = raw.reshape(shape[0], shape[1] // bv, bb)[:, lo // bv:hi // bv]
        return name, (shape[0], hi - lo), qtype, blk.reshape(shape[0], -1).contiguous()

    def row_slice(name, shape, qtype, raw):
        lo, hi = rank * shape[0] // world, (rank + 1) * shape[0] // world
        return name, (hi - lo, shape[1]), qtype, raw[lo:hi]

    if spec.n_kv >= world:
        kv_lo, kv_hi = rank * spec.kv_rows // world, (rank + 1) * spec.kv_rows // world
    else:
        kvh = rank // (world // spec.n_kv)
        kv_lo, kv_hi = kvh * hd, (kvh + 1) * hd
    for name, shape, qtype, raw in items:
        if not attn and name.endswith(ATTN_NAMES):
            yield name, shape, qtype, raw
        elif name.endswith("attn_q.weight") or name.endswith("attn_q_b.weight"):
            yield name, (q_hi - q_lo, shape[1]), qtype, raw[q_lo:q_hi]
        elif name.endswith("attn_k.weight") or name.endswith("attn_v.weight"):
            yield name, (kv_hi - kv_lo, shape[1]), qtype, raw[kv_lo:kv_hi]
        elif name.endswith("attn_k_b.weight") or name.endswith("attn_v_b.weight"):
            per = shape[1]                                    # [head][rows per head][latent] stored as rows
            yield name, (h_hi - h_lo, shape[1], shape[2]), qtype, raw.reshape(shape[0] * per, -1)[h_lo * per:h_hi * per]
        elif name.endswith("attn_output.weight"):
            yield k_slice(name, shape, qtype, raw, o_lo, o_hi)
        elif name.endswith(("ffn_gate.weight", "ffn_up.weight", "ffn_gate_shexp.weight", "ffn_up_shexp.weight")):
            yield row_slice(name, shape, qtype, raw)
        elif name.endswith(("ffn_down.weight", "ffn_down_shexp.weight")):
            yield k_slice(name, shape, qtype, raw, rank * shape[1] // world, (rank + 1) * shape[1] // world)
        elif "_exps.weight" in name:
            e_lo, e_hi = rank * shape[0] // world, (rank + 1) * shape[0] // world
            yield name, (e_hi - e_lo, shape[1], shape[2]), qtype, raw[e_lo * shape[1]:e_hi * shape[1]]
        else:
            yield name, shape, qtype, raw


def local_spec(spec: ModelSpec, world: int, attn: bool = True) -> ModelSpec:
    s = dataclasses.replace(spec)
    if attn:
        s.n_q = spec.n_q // world
        s.n_kv = max(1, spec.n_kv // world)
    if spec.dense_inter:
        s.dense_inter = spec.dense_inter // world
    if spec.n_shared:
        s.shared_inter = spec.shared_inter // world
    return s


class ShardedEngine(DecodeEngine):
    """One rank of the TP-attention + EP-experts decode engine."""

    def __init__(self, weights: Weights, full_spec: ModelSpec, rank: int, world: int, group=None, fused: bool = True,
                 arena: Optional[SymmetricArena] = None, attn_replicated: bool = False, **kw):
        """``attn_replicated``: every rank runs the whole attention half on whole attention weights and only the FFN
        half (experts by index, dense and shared width) is split, so a layer has ONE reduction instead of two.  For a
        few rows of decode the chain is bound by latency, not by the bytes of the attention weights, and the
        reduction it saves is worth more than the split: this is the form whose speed grows with the rank count."""
        self.full_spec = full_spec
        self.rank, self.world, self.group = rank, world, group
        self.fused = fused
        self.attn_replicated = attn_replicated
        super().__init__(weights, **kw)
        s, dev = self.spec, self.device
        self.arena = arena or SymmetricArena(s.hidden, rank, world, dev, group, local_only=not fused)
        self.xbuf = [self.x, torch.zeros_like(self.x)]
        if s.is_moe:
            e_per = s.n_expert // world
            sm = torch.full((s.n_expert,), -1, dtype=torch.int32)
            sm[rank * e_per:(rank + 1) * e_per] = torch.arange(e_per, dtype=torch.int32)
            self.slot_map = sm.to(dev)
        self.partial = torch.zeros(8, s.hidden, dtype=torch.float32, device=dev)
        self.arena.sites_per_step = 2 * s.n_layer

    def _new_gemm_prefill(self):
        from .prefill_dist import ShardedGemmPrefill
        return ShardedGemmPrefill(self, ubatch=self.ubatch, group=self.group, local_only=self.world == 1)

    def enqueue(self, M: int, head: bool = True, advance: bool = False) -> int:
        ops = self.build_ops(M, head, advance)
        for op in ops:
            op()
        return sum(getattr(op, "launches", 1) for op in ops)

    def build_ops(self, M: int, head: bool = True, advance: bool = False) -> List:
        """The pass as a list of launch thunks (one kernel launch each unless marked), so a
        test can interleave the launches of several emulated ranks on one GPU."""
        s, w, ar = self.spec, self.w, self.arena
        ops: List = []

        def add(fn, *a, launches: int = 1, **k):
            t = functools.partial(fn, *a, **k)
            if launches != 1:
                t = _Thunk(t, launches)
            ops.append(t)

        cur = 0
        xb = self.xbuf
        add(K.embed_rows, self.tokens, M, w.q["token_embd.weight"], s.vocab, xb[0], self.fault, self.arena.step)
        kvp = self.kv
        fused = self.fused

        def allreduce_into(xr: torch.Tensor, part: torch.Tensor):
            # baseline: NCCL sums the partial rows, an eager add applies them to the residual
            dist.all_reduce(part, group=self.group)
            xr.add_(part)

        pending = None     # (site, index) whose partials the next consumer has to add
        H = s.hidden
        rep = self.attn_replicated
        for il in range(s.n_layer):
            b = f"blk.{il}."
            red = None
            # with one reduction per layer the two receive buffers alternate by layer: a rank that runs ahead writes
            # layer l + 1 into the buffer its peers are not reading layer l from
            site_ffn = (il & 1) if rep else SITE_MOE
            if fused and pending is not None:
                red = ar.reduce(pending[0], pending[1], xb[cur ^ 1], self.fault, il)
            if s.mla:
                # latent attention: the low-rank products and the latent append are the same on every rank, the per-head
                # products run on this rank's heads
                first = w.q[b + "attn_q_a.weight"] if s.q_lora else w.q[b + "attn_q.weight"]
                add(K.gemv, [first, w.q[b + "attn_kv_a_mqa.weight"]], M, self.qkv, x=xb[cur],
                    gain=w.f[b + "attn_norm.weight"], eps=s.rms_eps, red=red, fault=self.fault, layer=il)
                if red is not None:
                    cur ^= 1
                add(K.mla_kv_append, self.qkv[:, self.qa_w:], w.f[b + "attn_kv_a_norm.weight"], self.inv_freq, s.rms_eps, M,
                    self.row_pos, self.row_seq, kvp.table, kvp.n_pages, kvp.k[il], self.fault, il)
                if s.q_lora:
                    add(K.gemv, [w.q[b + "attn_q_b.weight"]], M, self.q_full, x=self.qkv[:, :s.q_lora],
                        gain=w.f[b + "attn_q_a_norm.weight"], eps=s.rms_eps, fault=self.fault, layer=il)
                    q = self.q_full
                else:
                    q = self.qkv[:, :self.qa_w]
                add(K.mla_q_absorb, q, w.f[b + "attn_k_b.weight"], self.inv_freq, self.attn_scale, s.n_q, s.nope_dim, M,
                    self.row_pos, self.row_seq, self.q_out)
                add(K.mla_flash_decode, self.q_out, kvp.k[il], self.row_pos, self.row_seq, kvp.table, kvp.n_pages, s.n_q, M,
                    self.n_seg, self.slot_ctx, self.part_ml, self.part_acc, w.f[b + "attn_v_b.weight"], s.v_dim, None,
                    self.attn_q, self.attn_ds, self.fault, il, launches=2)
            else:
                add(K.gemv, [w.q[b + "attn_q.weight"], w.q[b + "attn_k.weight"], w.q[b + "attn_v.weight"]], M, self.qkv,
                    x=xb[cur], gain=w.f[b + "attn_norm.weight"], eps=s.rms_eps, red=red, fault=self.fault, layer=il)
                if red is not None:
                    cur ^= 1
            if s.mla:
                pass
            elif K.staged_part("attn"):
                add(K.attn_fused, self.qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"),
                    self.inv_freq, s.rms_eps, self.attn_scale, s.head_dim, s.n_q, s.n_kv, M, self.row_pos, self.row_seq,
                    kvp.table, kvp.n_pages, kvp.k[il], kvp.v[il], self.n_seg, self.slot_ctx, self.part_ml, self.part_acc,
                    self.tickets, None, self.attn_q, self.attn_ds, self.fault, il)
            else:
                add(K.qk_norm_rope_append, self.qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"),
                    self.inv_freq, s.rms_eps, self.attn_scale, s.head_dim, s.n_q, s.n_kv, M,
                    self.row_pos, self.row_seq, kvp.table, kvp.n_pages, kvp.k[il], kvp.v[il], self.q_out, self.fault, il)
                add(K.flash_decode, self.q_out, kvp.k[il], kvp.v[il], self.row_pos, self.row_seq, kvp.table, kvp.n_pages,
                    s.head_dim, s.n_q, s.n_kv, M, self.n_seg, self.slot_ctx, self.part_ml, self.part_acc, None,
                    self.attn_q, self.attn_ds, self.fault, il, launches=2)
            if rep:
                add(K.gemv, [w.q[b + "attn_output.weight"]], M, xb[cur], xq=self.attn_q, xds=self.attn_ds, resid=xb[cur],
                    fault=self.fault, layer=il)
                red = None
            elif fused:
                add(K.gemv, [w.q[b + "attn_output.weight"]], M, self.partial, xq=self.attn_q,
                    xds=self.attn_ds, push=ar.push(SITE_ATTN, 2 * il), fault=self.fault, layer=il)
                red = ar.reduce(SITE_ATTN, 2 * il, xb[cur ^ 1], self.fault, il)
            else:
                add(K.gemv, [w.q[b + "attn_output.weight"]], M, self.partial, xq=self.attn_q, xds=self.attn_ds,
                    fault=self.fault, layer=il)
                add(allreduce_into, xb[cur], self.partial, launches=2)
                red = None
            if not s.layer_is_moe(il):
                # dense FFN: this rank's slice of the width; the down product's partial rows are the layer's second
                # reduction
                add(K.gemv, [w.q[b + "ffn_gate.weight"], w.q[b + "ffn_up.weight"]], M, self.gu, x=xb[cur],
                    gain=w.f[b + "ffn_norm.weight"], eps=s.rms_eps, red=red, fault=self.fault, layer=il)
                if red is not None:
                    cur ^= 1
                add(K.swiglu_q8, self.gu, s.dense_inter, M, self.dactq, self.dactds)
                if fused:
                    add(K.gemv, [w.q[b + "ffn_down.weight"]], M, self.partial, xq=self.dactq, xds=self.dactds,
                        push=ar.push(site_ffn, 2 * il + 1), fault=self.fault, layer=il)
                    pending = (site_ffn, 2 * il + 1)
                else:
                    add(K.gemv, [w.q[b + "ffn_down.weight"]], M, self.partial, xq=self.dactq, xds=self.dactds,
                        fault=self.fault, layer=il)
                    add(allreduce_into, xb[cur], self.partial, launches=2)
                    pending = None
                continue
            ids, wts = self.r_ids_all[il], self.r_wts_all[il]
            gate, up, down = w.q[b + "ffn_gate_exps.weight"], w.q[b + "ffn_up_exps.weight"], w.q[b + "ffn_down_exps.weight"]
            staged = gate.qtype == up.qtype and K.moe_fits_stage(gate, down, s.n_used)
            add(K.router, xb[cur], w.f[b + "ffn_norm.weight"], s.rms_eps, w.q[b + "ffn_gate_inp.weight"], M,
                self.r_logits, self.xq, self.xds, None, self.fault, il, red=red)
            if red is not None:
                cur ^= 1
            if staged:
                add(K.gate_up_staged, self.xq, self.xds, ids, self.slot_map, gate, up, s.n_expert, s.n_used, M, self.actq,
                    self.actds, None, self.fault, il, down=down, route_logits=self.r_logits, rule=self._rule(il), wts=wts,
                    heat=self.heat[il])
            else:
                add(K.gate_up_sel, self.xq, self.xds, ids, self.slot_map, gate, up, s.n_expert, s.n_used, M, self.actq,
                    self.actds, None, self.fault, il, route_logits=self.r_logits, rule=self._rule(il), wts=wts,
                    heat=self.heat[il])
            extra = None
            if s.n_shared:
                # this rank's slice of the shared expert's width lands as an extra addend of the partial rows
                add(K.gemv, [w.q[b + "ffn_gate_shexp.weight"], w.q[b + "ffn_up_shexp.weight"]], M, self.sh_gu, xq=self.xq,
                    xds=self.xds, fault=self.fault, layer=il)
                add(K.swiglu_q8, self.sh_gu, s.shared_inter, M, self.sh_actq, self.sh_actds)
                add(K.gemv, [w.q[b + "ffn_down_shexp.weight"]], M, self.sh_out, xq=self.sh_actq, xds=self.sh_actds,
                    fault=self.fault, layer=il)
                extra = self.sh_out
            # the pushing launch takes the staged form: it stores each peer's rows as runs of consecutive columns
            down_fn = K.down_staged if (staged or (fused and K.moe_fits_stage(gate, down, s.n_used, force=True))) else K.down_combine
            if fused:
                add(down_fn, self.actq, self.actds, ids, wts, self.slot_map, down, s.n_expert, s.n_used, M, None, extra,
                    self.partial, self.fault, il, push=ar.push(site_ffn, 2 * il + 1))
                pending = (site_ffn, 2 * il + 1)
            else:
                add(down_fn, self.actq, self.actds, ids, wts, self.slot_map, down, s.n_expert, s.n_used, M, None, extra,
                    self.partial, self.fault, il)
                add(allreduce_into, xb[cur], self.partial, launches=2)
                pending = None
        if head:
            head_w = w.q.get("output.weight", w.q["token_embd.weight"])
            red = ar.reduce(pending[0], pending[1], xb[cur ^ 1], self.fault, s.n_layer) if (fused and pending is not None) else None
            add(K.gemv, [head_w], M, self.logits, x=xb[cur], gain=w.f["output_norm.weight"], eps=s.rms_eps, red=red,
                fault=self.fault, layer=s.n_layer)
            add(K.argmax_rows, self.logits, s.vocab, M, self.am_blocks, self.am_v, self.am_i, self.counters[1:2],
                self.tokens_out, None, self.fault)
            if advance:
                add(K.advance_rows, self.tokens, self.row_pos, self.row_seq, self.tokens_out, M, self.hist,
                    self.hist_cap, self.counters[2:3])
        elif fused and pending is not None:
            # no head on this pass: a small consumer folds the last reduction into the residual rows
            red = ar.reduce(pending[0], pending[1], xb[cur ^ 1], self.fault, s.n_layer)
            small = w.q["blk.0.attn_kv_a_mqa.weight"] if s.mla else w.q["blk.0.attn_k.weight"]
            add(K.gemv, [small], M, self.qkv, x=xb[cur], gain=w.f["output_norm.weight"],
                eps=s.rms_eps, red=red, fault=self.fault, layer=s.n_layer)
        return ops


class _Thunk:
    def __init__(self, fn, launches: int):
        self.fn, self.launches = fn, launches

    def __call__(self):
        return self.fn()
