"""Python face of the decode-chain CUDA kernels (``csrc/*_decode.cu``, ``decode_gemv.cu``).

Each wrapper only marshals pointers and shapes; the host-side launch contract lives in
the C launcher and comes back as a negative code that :func:`check` turns into an
exception naming the call.  All launches go to the current torch stream, so they are
capturable in a ``torch.cuda.CUDAGraph``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..formats.resident import WT
from ._lib import F, I, L, check, cuda, p, stream

_sm_count_cache = {}


def sm_count(device=None) -> int:
    dev = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if dev not in _sm_count_cache:
        _sm_count_cache[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_count_cache[dev]


@dataclass
class QWeight:
    """A weight matrix (or stack of expert matrices) in its resident layout."""

    data: torch.Tensor        # uint8, [rows, resident_row_bytes] or [experts, rows, resident_row_bytes]
    qtype: str
    k: int

    @property
    def wt(self) -> int:
        return WT[self.qtype]

    @property
    def rows(self) -> int:
        return self.data.shape[-2]

    @property
    def n_bytes(self) -> int:
        return self.data.numel()


class PushOut(ctypes.Structure):
    """Producer half of the fused all-reduce (mirrors ``bl::PushOut`` in csrc/common.cuh)."""

    _fields_ = [("peer_recv", ctypes.c_void_p * 8), ("step", ctypes.c_void_p), ("sites_per_step", ctypes.c_uint),
                ("site_index", ctypes.c_uint), ("n_ranks", ctypes.c_int), ("my_rank", ctypes.c_int)]


class ReduceIn(ctypes.Structure):
    """Consumer half of the fused all-reduce (mirrors ``bl::ReduceIn``)."""

    _fields_ = [("recv", ctypes.c_void_p), ("step", ctypes.c_void_p), ("sites_per_step", ctypes.c_uint),
                ("site_index", ctypes.c_uint), ("x_out", ctypes.c_void_p), ("x_out_stride", ctypes.c_long),
                ("n_ranks", ctypes.c_int), ("H", ctypes.c_int), ("fault", ctypes.c_void_p), ("layer", ctypes.c_int)]


def _ref(s):
    return ctypes.byref(s) if s is not None else ctypes.c_void_p(0)


def set_pdl(on: bool) -> None:
    cuda().bl_set_pdl(I(1 if on else 0))


def _family(qtype: str) -> int:
    """Kernel family of a weight type: 0 K-quants and Q8_0, 1 float rows, 2 planes and re-laid 32-value blocks."""
    if qtype in ("F32", "F16", "BF16"):
        return 1
    return 2 if qtype in ("NVFP4", "FP8_B128", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K") else 0


_STAGED = True
_STAGE_SLICE_MAX = 90 * 1024
# which launches take the staged form when it is on (BLOOMERY_STAGED_PARTS): gemv, attn, moe, prefetch (L2
# prefetch of the next layer's projections and of the chosen down matrices) and cluster (a one-row pass runs a
# layer's whole expert half as one thread-block-cluster launch; measured at top-6 on the Qwen3-30B-A3B layer shape:
# 23.3 us against 18.9 us for the three launches, and a B200 holds only seven 16-CTA clusters of its 212 KB at once,
# so top-8 models cannot use it: off by default).  Measured on the Qwen3-30B-A3B shape
# (ms per decode step): none 2.09, attn 2.05, gemv +0.04, moe +0.22 (bulk copies that can only start once the
# routing is known lose to per-thread loads), so the default keeps the fused attention launch and the prefetches.
_PARTS = {"attn", "prefetch"}


def set_staged_parts(parts) -> None:
    global _PARTS
    _PARTS = {x.strip() for x in (parts.split(",") if isinstance(parts, str) else parts) if x.strip()}


def staged_part(name: str) -> bool:
    return _STAGED and name in _PARTS


def set_staged(on: bool) -> None:
    """Use the shared-memory staged decode kernels (``csrc/decode_staged.cu``) where a launch's weight rows fit the
    stage; off = the register-streaming kernels everywhere."""
    global _STAGED
    _STAGED = bool(on)


def staged() -> bool:
    return _STAGED


def _gemv_fits_stage(segs: Sequence[QWeight], M: int) -> bool:
    total = sum(s.data.numel() for s in segs)
    K = segs[0].k
    mb = 1 if M <= 1 else 2 if M <= 2 else 4 if M <= 4 else 8
    act = mb * K * 5 // 4 + 4096
    return total / (2 * sm_count()) <= _STAGE_SLICE_MAX * 0.85 and total / (2 * sm_count()) + act <= 190 * 1024 and all(
        s.data.dim() == 2 for s in segs)


def gemv(segs: Sequence[QWeight], M: int, out: torch.Tensor, *, x: Optional[torch.Tensor] = None,
         gain: Optional[torch.Tensor] = None, eps: float = 1e-6, xq: Optional[torch.Tensor] = None,
         xds: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
         red: Optional[ReduceIn] = None, push: Optional[PushOut] = None,
         fault: Optional[torch.Tensor] = None, layer: int = 0, prefetch: Optional[Sequence[torch.Tensor]] = None) -> None:
    """``prefetch``: up to six tensors a later launch will stream (the next layer's projections); the launch asks L2
    for them before it waits for its predecessor."""
    fams = [_family(sg.qtype) for sg in segs]
    if len(set(fams) - {1}) > 1 or (2 in fams and 1 in fams):
        # segments of different kernel families (e.g. a Q5_0 fallback tensor beside K-quants): one call per run
        col, i = 0, 0
        while i < len(segs):
            j = i
            while j < len(segs) and fams[j] == fams[i]:
                j += 1
            width = sum(sg.rows for sg in segs[i:j])
            gemv(segs[i:j], M, out[:, col:col + width], x=x, gain=gain, eps=eps, xq=xq, xds=xds,
                 resid=resid[:, col:col + width] if resid is not None else None, red=red if i == 0 else None,
                 push=push, fault=fault, layer=layer, prefetch=prefetch if i == 0 else None)
            col += width
            i = j
        return
    n = len(segs)
    K = segs[0].k
    wp = (ctypes.c_void_p * n)(*[s.data.data_ptr() for s in segs])
    rows = (ctypes.c_int * n)(*[s.rows for s in segs])
    wts = (ctypes.c_int * n)(*[s.wt for s in segs])
    norm = x is not None
    # a launch that pushes its rows to the peers takes the staged kernel whenever it fits: its epilogue stores each
    # peer's rows as runs of consecutive columns (whole NVLink packets) instead of one 8-byte store per warp
    if (staged_part("gemv") or (push is not None and _STAGED)) and 1 not in fams and _gemv_fits_stage(segs, M):
        rc = cuda().bl_gemv_staged(I(n), wp, rows, wts, I(K), I(M), I(1 if norm else 0),
                                   p(x), L(x.stride(0) if norm else 0), p(gain), F(eps), p(xq), p(xds),
                                   p(out), L(out.stride(0)), p(resid), L(resid.stride(0) if resid is not None else 0),
                                   _ref(red), _ref(push), p(fault), I(layer), I(sm_count()), stream())
        if rc != -5:                         # -5: a block's rows would not fit the stage; the streaming kernel serves it
            check(rc, "bl_gemv_staged")
            return
    pf = list(prefetch or [])[:6] if "prefetch" in _PARTS else []
    pfp = (ctypes.c_void_p * max(1, len(pf)))(*[t.data_ptr() for t in pf])
    pfb = (ctypes.c_long * max(1, len(pf)))(*[t.numel() * t.element_size() for t in pf])
    rc = cuda().bl_gemv(I(n), wp, rows, wts, I(K), I(M), I(1 if norm else 0),
                        p(x), L(x.stride(0) if norm else 0), p(gain), F(eps), p(xq), p(xds),
                        p(out), L(out.stride(0)), p(resid), L(resid.stride(0) if resid is not None else 0),
                        _ref(red), _ref(push), p(fault), I(layer), I(sm_count()), I(len(pf)), pfp, pfb, stream())
    check(rc, "bl_gemv")


def set_flash_mma(on: bool) -> None:
    """Run the GQA decode segment pass on tensor-core tiles (f16 q and probabilities) instead of fp32 FMAs."""
    cuda().bl_set_flash_mma(I(1 if on else 0))


def qk_norm_rope_append(qkv: torch.Tensor, q_gain, k_gain, inv_freq: torch.Tensor, eps: float, q_scale: float,
                        head: int, n_q: int, n_kv: int, M: int, row_pos, row_seq, block_table, n_pages: int,
                        k_cache, v_cache, q_out, fault, layer: int, kv_q8: bool = False) -> None:
    """``kv_q8``: the caches are uint8 q8_0 rows (head / 32 f16 scales, then head int8 codes per position and KV head)."""
    fn = cuda().bl_qk_norm_rope_append_q8 if kv_q8 else cuda().bl_qk_norm_rope_append
    rc = fn(p(qkv), L(qkv.stride(0)), p(q_gain), p(k_gain), p(inv_freq), F(eps), F(q_scale),
                                       I(head), I(n_q), I(n_kv), I(M), p(row_pos), p(row_seq), p(block_table),
                                       I(block_table.shape[1]), I(n_pages), p(k_cache), p(v_cache), p(q_out), p(fault),
                                       I(layer), stream())
    check(rc, "bl_qk_norm_rope_append")


def flash_decode(q, k_cache, v_cache, row_pos, row_seq, block_table, n_pages: int, head: int, n_q: int, n_kv: int,
                 M: int, n_seg: int, ctx_limit: int, part_ml, part_acc, out, outq, outds, fault, layer: int,
                 kv_q8: bool = False) -> None:
    fn = cuda().bl_flash_decode_q8 if kv_q8 else cuda().bl_flash_decode
    rc = fn(p(q), p(k_cache), p(v_cache), p(row_pos), p(row_seq), p(block_table),
                                I(block_table.shape[1]), I(n_pages), I(head), I(n_q), I(n_kv), I(M), I(n_seg),
                                I(ctx_limit), p(part_ml), p(part_acc), p(out), p(outq), p(outds), p(fault), I(layer),
                                stream())
    check(rc, "bl_flash_decode")


def attn_fused(qkv, q_gain, k_gain, inv_freq, eps: float, q_scale: float, head: int, n_q: int, n_kv: int, M: int,
               row_pos, row_seq, block_table, n_pages: int, k_cache, v_cache, n_seg: int, ctx_limit: int, part_ml,
               part_acc, tickets, out, outq, outds, fault, layer: int) -> None:
    """Per-head RMSNorm + RoPE + KV append + split-K flash decode + merge + q8 rows for o_proj, one launch.
    ``tickets``: int32 [M * n_kv], zero on entry (left zero)."""
    rc = cuda().bl_attn_fused(p(qkv), L(qkv.stride(0)), p(q_gain), p(k_gain), p(inv_freq), F(eps), F(q_scale), I(head),
                              I(n_q), I(n_kv), I(M), p(row_pos), p(row_seq), p(block_table), I(block_table.shape[1]),
                              I(n_pages), p(k_cache), p(v_cache), I(n_seg), I(ctx_limit), p(part_ml), p(part_acc),
                              p(tickets), p(out), p(outq), p(outds), p(fault), I(layer), stream())
    check(rc, "bl_attn_fused")


def attn_cluster_size(n_kv: int, M: int) -> int:
    """CTAs per cluster of the cluster form of the attention launch for M rows of n_kv KV heads (0 = use the ticket
    form): 16 while a B200 can hold all n_kv * M clusters at once, else 8."""
    if "attn" not in _PARTS or not _STAGED:
        return 0
    if n_kv * M <= 12:
        return 16
    return 8 if n_kv * M <= 32 else 0


def attn_cluster(qkv, q_gain, k_gain, inv_freq, eps: float, q_scale: float, head: int, n_q: int, n_kv: int, M: int,
                 row_pos, row_seq, block_table, n_pages: int, k_cache, v_cache, cluster: int, ctx_limit: int, out, outq,
                 outds, fault, layer: int) -> None:
    """The fused attention launch with the key segments of each (row, KV head) spread over a thread-block cluster
    of ``cluster`` CTAs that merge through distributed shared memory (no scratch, no tickets)."""
    rc = cuda().bl_attn_cluster(p(qkv), L(qkv.stride(0)), p(q_gain), p(k_gain), p(inv_freq), F(eps), F(q_scale), I(head),
                                I(n_q), I(n_kv), I(M), p(row_pos), p(row_seq), p(block_table), I(block_table.shape[1]),
                                I(n_pages), p(k_cache), p(v_cache), I(cluster), I(ctx_limit), p(out), p(outq), p(outds),
                                p(fault), I(layer), stream())
    check(rc, "bl_attn_cluster")


def router(x, gain, eps: float, w: QWeight, M: int, logits, xq_out, xds_out, xn_out, fault, layer: int,
           red: Optional[ReduceIn] = None, *, rule: Optional["RouteRule"] = None, ids=None, wts=None, heat=None,
           ticket=None, predict=None, predict_slot_map=None) -> None:
    """Router logits of M rows (RMSNorm folded in) + the q8 form of the normed rows.  With ``ticket`` (int32, one
    zeroed word per 8 rows) and ``rule`` the launch also routes: its last block writes ``ids`` / ``wts`` / ``heat``.
    ``predict`` = (gate, up, down) stacks: the prediction form -- run on a layer's INPUT rows, the last block asks L2
    to prefetch the matrices of the ``rule.top_k`` best-scoring experts and publishes nothing."""
    r = rule
    pg, pu, pd = predict if predict is not None else (None, None, None)
    rc = cuda().bl_router(p(x), L(x.stride(0)), p(gain), F(eps), p(w.data), I(w.wt), I(w.k), I(w.rows), I(M),
                          p(logits), p(xq_out), p(xds_out), p(xn_out), _ref(red), p(fault), I(layer),
                          p(ticket if r is not None else None), p(r.bias if r is not None else None),
                          I(r.top_k if r is not None else 0), I(r.mode if r is not None else 0),
                          I(1 if (r is not None and r.renorm) else 0), F(r.scale if r is not None else 1.0),
                          I(r.n_group if r is not None else 1), I(r.topk_group if r is not None else 1),
                          p(ids), p(wts), p(heat),
                          p(pg.data if pg is not None else None), p(pu.data if pu is not None else None),
                          p(pd.data if pd is not None else None), L(pg.data.stride(0) if pg is not None else 0),
                          L(pd.data.stride(0) if pd is not None else 0), p(predict_slot_map), stream())
    check(rc, "bl_router")


@dataclass
class RouteRule:
    """How logits become (ids, weights): softmax or sigmoid scores, optional selection bias,
    renormalisation, scale, optional group-limited choice."""

    top_k: int
    mode: int = 0              # 0 softmax, 1 sigmoid
    renorm: bool = True
    scale: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    bias: Optional[torch.Tensor] = None


def route_rows(logits, rule: RouteRule, M: int, ids, wts, heat, fault, layer: int) -> None:
    rc = cuda().bl_route_rows(p(logits), p(rule.bias), I(logits.shape[-1]), I(M), I(rule.top_k), I(rule.mode),
                              I(1 if rule.renorm else 0), F(rule.scale), I(rule.n_group), I(rule.topk_group), p(ids),
                              p(wts), p(heat), p(fault), I(layer), stream())
    check(rc, "bl_route_rows")


def gate_up_sel(xq, xds, ids, slot_map, gate: QWeight, up: QWeight, n_expert: int, n_used: int, M: int, actq, actds,
                act_f32, fault, layer: int, *, route_logits=None, rule: Optional[RouteRule] = None, wts=None,
                heat=None, down: Optional[QWeight] = None) -> None:
    """gate·up·SwiGLU of the chosen experts.  With ``route_logits`` every block routes its own
    row (and ids / wts / heat are written for the launches that follow); else ``ids`` is read.  ``down``: the
    layer's down stack; the launch asks L2 to prefetch the chosen experts' matrices for the launch that follows."""
    r = rule or RouteRule(n_used)
    if "prefetch" not in _PARTS:
        down = None
    rc = cuda().bl_gate_up_sel(p(xq), p(xds), p(route_logits), p(r.bias), I(r.mode), I(1 if r.renorm else 0),
                               F(r.scale), I(r.n_group), I(r.topk_group), p(ids), p(wts), p(heat), p(slot_map),
                               p(gate.data), p(up.data), I(gate.wt), I(up.wt), I(gate.k), I(gate.rows), I(n_expert),
                               I(n_used), I(M), p(actq), p(actds), p(act_f32), p(fault), I(layer),
                               p(down.data if down is not None else None), L(down.data.stride(0) if down is not None else 0),
                               stream())
    check(rc, "bl_gate_up_sel")


def down_combine(actq, actds, ids, wts, slot_map, down: QWeight, n_expert: int, n_used: int, M: int, resid, extra,
                 out, fault, layer: int, push: Optional[PushOut] = None) -> None:
    rc = cuda().bl_down_combine(p(actq), p(actds), p(ids), p(wts), p(slot_map), p(down.data), I(down.wt), I(down.k),
                                I(down.rows), I(n_expert), I(n_used), I(M), p(resid),
                                L(resid.stride(0) if resid is not None else 0), p(extra),
                                L(extra.stride(0) if extra is not None else 0), p(out), L(out.stride(0)), _ref(push),
                                p(fault), I(layer), stream())
    check(rc, "bl_down_combine")


def prefetch_experts(ids, n: int, gate: QWeight, up: QWeight, down: Optional[QWeight], blocks: int) -> None:
    """Ask L2 to prefetch the gate / up (/ down) matrices of the ``n`` expert slots named in ``ids`` (negative = skip)."""
    rc = cuda().bl_prefetch_experts(p(ids), I(n), p(gate.data), p(up.data), p(down.data if down is not None else None),
                                    L(gate.data.stride(0)), L(down.data.stride(0) if down is not None else 0), I(blocks),
                                    stream())
    check(rc, "bl_prefetch_experts")


def gate_up_staged(xq, xds, ids, slot_map, gate: QWeight, up: QWeight, n_expert: int, n_used: int, M: int, actq, actds,
                   act_f32, fault, layer: int, down: Optional[QWeight] = None, *, route_logits=None,
                   rule: Optional["RouteRule"] = None, wts=None, heat=None) -> None:
    """gate.x, up.x, SwiGLU, q8 of the chosen experts (shared-memory staged).  With ``route_logits`` every block routes
    its own row (warp 0, beside the activation fetch) and ``ids`` / ``wts`` / ``heat`` are written for the launches that
    follow; else ``ids`` is read.  ``down``: the layer's down stack, whose chosen matrices the launch asks L2 to
    prefetch for the launch that follows."""
    r = rule or RouteRule(n_used)
    if not staged_part("prefetch"):
        down = None
    deb = down.data.stride(0) if down is not None else 0
    rc = cuda().bl_gate_up_staged(p(xq), p(xds), p(route_logits), p(r.bias), I(r.mode), I(1 if r.renorm else 0), F(r.scale),
                                  I(r.n_group), I(r.topk_group), p(ids), p(wts), p(heat), p(slot_map), p(gate.data),
                                  p(up.data), I(gate.wt), p(down.data if down is not None else None), L(deb), I(gate.k),
                                  I(gate.rows), I(n_expert), I(n_used), I(M), p(actq), p(actds), p(act_f32), p(fault),
                                  I(layer), stream())
    check(rc, "bl_gate_up_staged")


def moe_fits_stage(gate: QWeight, down: QWeight, n_used: int, force: bool = False) -> bool:
    """Whether the staged expert kernels serve these stacks (a block's rows fit the shared-memory stage)."""
    if not (staged_part("moe") or (force and _STAGED)) or gate.qtype in ("F32", "F16", "BF16") or down.qtype in ("F32", "F16", "BF16"):
        return False
    rb_g = gate.data.shape[-1]
    rb_d = down.data.shape[-1]
    return 64 * rb_g + gate.k * 5 // 4 <= 180 * 1024 and n_used * 8 * rb_d + n_used * down.k * 5 // 4 <= 180 * 1024 and \
        n_used * (down.k // 64) <= 512


def down_staged(actq, actds, ids, wts, slot_map, down: QWeight, n_expert: int, n_used: int, M: int, resid, extra,
                out, fault, layer: int, push: Optional[PushOut] = None) -> None:
    rc = cuda().bl_down_staged(p(actq), p(actds), p(ids), p(wts), p(slot_map), p(down.data), I(down.wt), I(down.k),
                               I(down.rows), I(n_expert), I(n_used), I(M), p(resid),
                               L(resid.stride(0) if resid is not None else 0), p(extra),
                               L(extra.stride(0) if extra is not None else 0), p(out), L(out.stride(0)), _ref(push),
                               p(fault), I(layer), I(sm_count()), stream())
    check(rc, "bl_down_staged")


_cluster_fit_cache = {}


def moe_cluster_fits(router: QWeight, gate: QWeight, up: QWeight, down: QWeight, n_used: int) -> bool:
    """Whether the one-launch cluster form of a layer's expert half (``csrc/moe_cluster.cu``) serves these stacks on
    the current device: shapes divide by the 16 CTAs of a cluster, a CTA's rows fit its shared memory, and one
    16-CTA cluster per chosen expert can be resident at once."""
    if "cluster" not in _PARTS:
        return False
    key = (torch.cuda.current_device(), router.qtype, gate.qtype, up.qtype, down.qtype, gate.k, gate.rows, router.rows, n_used)
    if key not in _cluster_fit_cache:
        rc = cuda().bl_moe_cluster_fits(I(gate.k), I(gate.rows), I(router.rows), I(n_used), I(router.wt), I(gate.wt),
                                        I(up.wt), I(down.wt))
        _cluster_fit_cache[key] = rc == 0
    return _cluster_fit_cache[key]


def moe_cluster(x, gain, eps: float, router: QWeight, rule: "RouteRule", slot_map, gate: QWeight, up: QWeight,
                down: QWeight, n_used: int, extra, parts, tickets, x_out, logits, ids, wts, heat, fault, layer: int) -> None:
    """Router + top-k + chosen experts + weighted sum + residual of ONE row in one thread-block-cluster launch.
    ``x_out`` (a different buffer than ``x``) receives the new residual row; ``parts`` fp32 [n_used, H] and
    ``tickets`` (16 zeroed int32 words, left zero) are scratch; logits / ids / wts / heat are published as the
    three-launch chain publishes them."""
    rc = cuda().bl_moe_cluster(p(x), p(gain), F(eps), p(router.data), I(router.wt), p(rule.bias), I(rule.mode),
                               I(1 if rule.renorm else 0), F(rule.scale), I(rule.n_group), I(rule.topk_group),
                               p(slot_map), p(gate.data), p(up.data), I(gate.wt), I(up.wt), p(down.data), I(down.wt),
                               I(gate.k), I(gate.rows), I(router.rows), I(n_used), p(extra), p(parts), p(tickets),
                               p(x_out), p(logits), p(ids), p(wts), p(heat), p(fault), I(layer), stream())
    check(rc, "bl_moe_cluster")


def embed_rows(tokens, M: int, table: QWeight, vocab: int, out, fault, step=None) -> None:
    rc = cuda().bl_embed_rows(p(tokens), I(M), p(table.data), I(table.wt), I(table.k), I(vocab), p(out),
                              L(out.stride(0)), p(fault), p(step), stream())
    check(rc, "bl_embed_rows")


def argmax_rows(logits, V: int, M: int, nblk: int, part_v, part_i, counter, tokens_out, best_val, fault) -> None:
    rc = cuda().bl_argmax_rows(p(logits), L(logits.stride(0)), I(V), I(M), I(nblk), p(part_v), p(part_i), p(counter),
                               p(tokens_out), p(best_val), p(fault), stream())
    check(rc, "bl_argmax_rows")


def fill_u32(t: torch.Tensor, value: int) -> None:
    check(cuda().bl_fill_u32(p(t), ctypes.c_uint(value), I(t.numel()), stream()), "bl_fill_u32")


def advance_rows(tokens, row_pos, row_seq, chosen, M: int, hist=None, hist_cap: int = 0, hist_count=None) -> None:
    check(cuda().bl_advance_rows(p(tokens), p(row_pos), p(row_seq), p(chosen), I(M), p(hist), I(hist_cap),
                                 p(hist_count), stream()), "bl_advance_rows")


def swiglu_q8(gu: torch.Tensor, I_: int, M: int, actq, actds, act_f32=None) -> None:
    check(cuda().bl_swiglu_q8(p(gu), L(gu.stride(0)), I(I_), I(M), p(actq), p(actds), p(act_f32), stream()),
          "bl_swiglu_q8")


def mtp_prep(e, h, src, enorm, hnorm, eps: float, M: int, xq, xds) -> None:
    """q8 rows [M, 2H] = [norm(e) | norm(h[src])] for the multi-token-prediction layer's input product."""
    check(cuda().bl_mtp_prep(p(e), L(e.stride(0)), p(h), L(h.stride(0)), p(src), p(enorm), p(hnorm), F(eps), I(e.shape[1]),
                             I(M), p(xq), p(xds), stream()), "bl_mtp_prep")


_SPLIT_SCRATCH: dict = {}
SAMPLER_SPLIT_ROWS = 8            # up to this many rows a row's vocabulary is split over 32 blocks (two launches)


def sample_rows(logits, V: int, M: int, params, seeds, draws, out_token, *, recent=None, n_recent=None, work=None,
                out_n_cand=None, fault=None, split: Optional[bool] = None, cap: int = 1024) -> None:
    """The sampling chain on the card (``csrc/sampler.cu``): one block per row, or for few rows (``split``, default
    M <= 8) 32 blocks per row that each select their slice's top-k followed by the same chain on the candidate lists
    -- the same picks, bit for bit.  ``cap``: the largest top_k of the rows (1024 when a row has top_k <= 0).
    ``params`` fp32 [M, 8] = temperature, top_k, top_p, min_p, repeat_penalty, frequency_penalty,
    presence_penalty, repeat_last_n; ``seeds``/``draws`` uint64-as-int64 [M]; ``recent`` int32 [M, W]."""
    if split is None:
        split = M <= SAMPLER_SPLIT_ROWS
    if split:
        cap = max(1, min(1024, cap))
        key = (str(logits.device), cap)
        sc = _SPLIT_SCRATCH.get(key)
        if sc is None or sc[0].shape[0] < M:
            rows = max(M, SAMPLER_SPLIT_ROWS)
            sc = (torch.zeros(rows, 32 * cap, dtype=torch.float32, device=logits.device),
                  torch.zeros(rows, 32 * cap, dtype=torch.int32, device=logits.device))
            _SPLIT_SCRATCH[key] = sc
        rc = cuda().bl_sample_rows_split(p(logits), L(logits.stride(0)), I(V), I(M), p(recent),
                                         I(recent.shape[1] if recent is not None else 0), p(n_recent), p(params), p(seeds),
                                         p(draws), p(sc[0]), p(sc[1]), I(cap), p(out_token), p(out_n_cand), p(fault), stream())
        check(rc, "bl_sample_rows_split")
        return
    rc = cuda().bl_sample_rows(p(logits), L(logits.stride(0)), I(V), I(M), p(recent),
                               I(recent.shape[1] if recent is not None else 0), p(n_recent), p(params), p(seeds), p(draws),
                               p(work), p(out_token), p(out_n_cand), p(fault), stream())
    check(rc, "bl_sample_rows")


# ---- multi-head latent attention (csrc/mla_decode.cu) ---------------------------------
def _fw(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 30
    raise TypeError(f"per-head MLA weights are f32 or bf16, got {t.dtype}")


def mla_kv_append(kv, gain, inv_freq, eps: float, M: int, row_pos, row_seq, block_table, n_pages: int, cache, fault,
                  layer: int, kv_lora: int = 512, rope_dim: int = 64) -> None:
    """``kv`` fp32 [M, >=576] (a view is fine): RMSNorm the latent, rotate the shared key part, append as f16."""
    rc = cuda().bl_mla_kv_append(p(kv), L(kv.stride(0)), p(gain), p(inv_freq), F(eps), I(kv_lora), I(rope_dim), I(M),
                                 p(row_pos), p(row_seq), p(block_table), I(block_table.shape[1]), I(n_pages), p(cache),
                                 p(fault), I(layer), stream())
    check(rc, "bl_mla_kv_append")


def mla_q_absorb(q, w_kb, inv_freq, scale: float, n_q: int, nope: int, M: int, row_pos, row_seq, q_lat,
                 kv_lora: int = 512, rope_dim: int = 64) -> None:
    """``q`` fp32 [M, n_q * (nope + 64)] -> ``q_lat`` fp32 [M, n_q, 576], pre-scaled; ``w_kb`` [n_q, nope, 512]."""
    rc = cuda().bl_mla_q_absorb(p(q), L(q.stride(0)), p(w_kb), I(_fw(w_kb)), p(inv_freq), F(scale), I(n_q), I(nope),
                                I(kv_lora), I(rope_dim), I(M), p(row_pos), p(row_seq), p(q_lat), stream())
    check(rc, "bl_mla_q_absorb")


def mla_flash_decode(q_lat, cache, row_pos, row_seq, block_table, n_pages: int, n_q: int, M: int, n_seg: int,
                     ctx_limit: int, part_ml, part_acc, w_vb, v_dim: int, out, outq, outds, fault, layer: int) -> None:
    """Latent flash decode (segments + merge) with the per-head value up-projection and the q8 form for o_proj."""
    rc = cuda().bl_mla_flash_decode(p(q_lat), p(cache), p(row_pos), p(row_seq), p(block_table), I(block_table.shape[1]),
                                    I(n_pages), I(n_q), I(M), I(n_seg), I(ctx_limit), p(part_ml), p(part_acc), p(w_vb),
                                    I(_fw(w_vb)), I(v_dim), p(out), p(outq), p(outds), p(fault), I(layer), stream())
    check(rc, "bl_mla_flash_decode")
