"""Prompt (prefill) path on the tcgen05 GEMM: whole micro-batches of prompt rows per layer
instead of 8-row passes.

Counterpart of the reference's GEMM ubatches (``crates/gpu/src/arch/qwen3moe/ubatch.rs:1-40``:
per layer norm -> QKV GEMM -> norm/RoPE/append -> prefill flash -> o GEMM -> router logits +
route -> grouped gate/up GEMM with SwiGLU -> grouped down GEMM -> combine).  Here:

  * block-quantised weights of the layer are expanded to bf16 scratch right before use
    (one expander kernel per matrix; the scratch is shared by all layers);
  * every matmul is the persistent TMA + tcgen05 kernel; gate and up run in one main loop
    with SwiGLU in the epilogue; the down GEMM's epilogue scatters router-weighted rows to
    their (token, slot) cell and a fixed-order combine adds slots in ascending order;
  * attention is three launches per query chunk: Q K^T (grouped over heads, KV head shared
    by its query heads), causal softmax, P V (epilogue writes token-major rows).

Token bits are not equal to the 8-row pass path (bf16 operands, different sum order); a
band test covers it, as the reference does (``ubatch.rs:19-30``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import os

import torch

from ..ops import decode as K
from ..ops import gemm as G
from .kv import PAGE


POISON = None          # None: follow the BLOOMERY_POISON lever; tests set True / False


def _poison() -> bool:
    if POISON is not None:
        return bool(POISON)
    from ..utils import levers
    return bool(levers.get("BLOOMERY_POISON"))


class GemmPrefill:
    def __init__(self, engine, ubatch: int = 2048, score_bytes: int = 1 << 30):
        self.e = engine
        self.ubatch = ubatch
        self.score_bytes = score_bytes
        self._buf = {}
        self._router_w = {}
        self.status = torch.zeros(1, dtype=torch.int32, device=engine.device)
        self.launches = 0
        # where a layer's expert stacks come from: the resident weights, or a streamer that brings them from the host
        self.expert_source = None
        self.expand_ahead = True                # bf16 expansion of layer l + 1's weights on a side stream during layer l
        self._side = None
        self.flash = True                       # head size 128: fused attention on tensor memory (csrc/flash_tcgen05.cu)
        # Resident bf16 copy of every layer's matrices, built by the first prompt that runs (58 GB for a 30 B-parameter
        # mixture beside its 17 GB of Q4_K_M blocks): later prompts skip the expansion launches altogether.  None = only
        # when the copy leaves a quarter of the card free; True / False force it.
        from ..utils import levers
        self.resident_bf16 = {"1": True, "0": False}.get(str(levers.get("BLOOMERY_PREFILL_BF16")), None)
        self._resident = {}
        self._resident_ok = None
        from .timing import PromptTiming
        self.timing = PromptTiming()            # arm() it to get per-unit milliseconds of the next micro-batch

    def _get(self, name: str, shape, dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        b = self._buf.get(name)
        if b is None or b.numel() < n or b.dtype != dtype:
            b = torch.empty(n, dtype=dtype, device=self.e.device)
            if _poison():                   # scratch starts as NaN / -1: a read of something never written shows at once
                b.fill_(float("nan") if dtype.is_floating_point else -1)
            self._buf[name] = b
        return b[:n].view(*shape)

    def run(self, slot: int, tokens: Sequence[int], start: int = 0) -> None:
        """Append ``tokens`` at positions start.. of ``slot``; leaves the last row's hidden
        state in ``engine.x[0]`` (the caller runs the head)."""
        e = self.e
        n = len(tokens)
        e.kv.ensure(slot, start + n)
        for p in range(start, start + n, PAGE):
            e.kv.own(slot, p)
        e.kv.sync_table()
        i = 0
        while i < n:
            chunk = tokens[i:i + self.ubatch]
            self._ubatch(slot, chunk, start + i)
            i += len(chunk)
        e.slot_len[slot] = max(e.slot_len[slot], start + n)

    def _ubatch(self, slot: int, tokens: Sequence[int], p0: int) -> None:
        e = self.e
        s, w, dev = e.spec, e.w, e.device
        T = len(tokens)
        H, V = s.hidden, s.vocab
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        tok = torch.tensor(list(tokens), dtype=i32, device=dev)
        row_pos = torch.arange(p0, p0 + T, dtype=i32, device=dev)
        row_seq = torch.full((T,), slot, dtype=i32, device=dev)
        x = self._get("x", (T, H), f32)
        xn = self._get("xn", (T, H), bf)
        K.embed_rows(tok, T, w.q["token_embd.weight"], V, x, e.fault)
        qkv_w = s.q_rows + 2 * s.kv_rows
        qkv = self._get("qkv", (T, qkv_w), f32)
        # Quantised weights are expanded to bf16 one layer AHEAD of their use, on a side stream: the expansion is bound
        # by HBM traffic, the products by the tensor cores, so the two overlap.  Two sets of bf16 buffers alternate.
        resident = self._use_resident()
        ahead = self.expert_source is None and self.expand_ahead and not resident
        nset = 2 if ahead else 1
        wqkv_s = [self._get(f"wqkv{i}", (qkv_w, H), bf) for i in range(nset)]
        wo_s = [self._get(f"wo{i}", (H, s.q_rows), bf) for i in range(nset)]
        q_bf = self._get("q_bf", (s.n_q, T, s.head_dim), bf)
        attn = self._get("attn", (T, s.q_rows), bf)
        dense_tiles = G.TileTable.dense(T, dev)
        n_keys = p0 + T
        T_pad = (n_keys + 127) // 128 * 128
        Kb = self._get("Kb", (s.n_kv, T_pad, s.head_dim), bf)
        Vt = self._get("Vt", (s.n_kv, s.head_dim, T_pad), bf)
        Tq_max = max(128, min(T, self.score_bytes // (s.n_q * T_pad * 4) // 128 * 128))
        Gq = s.n_q // s.n_kv
        if s.is_moe:
            E, I_, k = s.n_expert, s.moe_inter, s.n_used
            nslot = T * k
            cap = nslot + 128
            wg_s = [self._get(f"wg{i}", (E, I_, H), bf) for i in range(nset)]
            wu_s = [self._get(f"wu{i}", (E, I_, H), bf) for i in range(nset)]
            wd_s = [self._get(f"wd{i}", (E, H, I_), bf) for i in range(nset)]
            logits = self._get("rl", (T, E), f32)
            xn3 = self._get("xn3", (T, 3 * H), bf)
            ids = self._get("ids", (T, k), i32)
            wts = self._get("wts", (T, k), f32)
            counts = self._get("counts", (E,), i32)
            cursor = self._get("cursor", (E,), i32)
            pos_of = self._get("pos_of", (nslot,), i32)
            dst_row = self._get("dst_row", (cap,), i32)
            row_scale = self._get("row_scale", (cap,), f32)
            Ap = self._get("Ap", (cap, H), bf)
            act = self._get("act", (cap, I_), bf)
            slot_out = self._get("slot_out", (nslot, H), f32)
            moe_tiles = G.TileTable(nslot, E, dev)
        if s.dense_inter and (s.first_dense > 0 or not s.is_moe):
            Id = s.dense_inter
            dg_s = [self._get(f"dg{i}", (Id, H), bf) for i in range(nset)]
            du_s = [self._get(f"du{i}", (Id, H), bf) for i in range(nset)]
            dd_s = [self._get(f"dd{i}", (H, Id), bf) for i in range(nset)]
            dact = self._get("dact", (T, Id), bf)
        st = self.status

        def expand(il: int, which: str) -> None:
            """bf16 copies of layer il's weights into buffer set il % nset: 'attn', 'gate_up', 'down' or 'all'."""
            b = f"blk.{il}."
            i = il % nset
            if which in ("attn", "all"):
                G.dequant_bf16(w.q[b + "attn_q.weight"], wqkv_s[i][:s.q_rows])
                G.dequant_bf16(w.q[b + "attn_k.weight"], wqkv_s[i][s.q_rows:s.q_rows + s.kv_rows])
                G.dequant_bf16(w.q[b + "attn_v.weight"], wqkv_s[i][s.q_rows + s.kv_rows:])
                G.dequant_bf16(w.q[b + "attn_output.weight"], wo_s[i])
            if s.layer_is_moe(il):
                if self.expert_source is not None:
                    qg, qu, qd = self.expert_source(il)
                else:
                    qg, qu, qd = (w.q[b + f"ffn_{n}_exps.weight"] for n in ("gate", "up", "down"))
                if which in ("gate_up", "all"):
                    G.dequant_bf16(qg, wg_s[i])
                    G.dequant_bf16(qu, wu_s[i])
                if which in ("down", "all"):
                    G.dequant_bf16(qd, wd_s[i])
            else:
                if which in ("gate_up", "all"):
                    G.dequant_bf16(w.q[b + "ffn_gate.weight"], dg_s[i])
                    G.dequant_bf16(w.q[b + "ffn_up.weight"], du_s[i])
                if which in ("down", "all"):
                    G.dequant_bf16(w.q[b + "ffn_down.weight"], dd_s[i])

        main = torch.cuda.current_stream(dev)
        if ahead:
            if self._side is None:
                self._side = torch.cuda.Stream(device=dev)
            side = self._side
            ready = [torch.cuda.Event() for _ in range(s.n_layer)]
            freed = [torch.cuda.Event() for _ in range(s.n_layer)]
            side.wait_stream(main)
            with torch.cuda.stream(side):
                expand(0, "all")
                ready[0].record(side)
        for il in range(s.n_layer):
            b = f"blk.{il}."
            self.timing.mark(il, "ffn")
            i = il % nset
            wqkv, wo = wqkv_s[i], wo_s[i]
            if s.is_moe:
                wg, wu, wd = wg_s[i], wu_s[i], wd_s[i]
            if s.dense_inter and (s.first_dense > 0 or not s.is_moe):
                dg, du, dd = dg_s[i], du_s[i], dd_s[i]
            if resident:
                hit = self._resident.get(il)
                if hit is None:
                    # first use of this layer: expand into the shared scratch as always, then keep a copy
                    expand(il, "all")
                    hit = {"wqkv": wqkv.clone(), "wo": wo.clone()}
                    if s.layer_is_moe(il):
                        hit.update(wg=wg.clone(), wu=wu.clone(), wd=wd.clone())
                    else:
                        hit.update(dg=dg.clone(), du=du.clone(), dd=dd.clone())
                    self._resident[il] = hit
                wqkv, wo = hit["wqkv"], hit["wo"]
                if s.layer_is_moe(il):
                    wg, wu, wd = hit["wg"], hit["wu"], hit["wd"]
                else:
                    dg, du, dd = hit["dg"], hit["du"], hit["dd"]
            if ahead:
                if il + 1 < s.n_layer:
                    with torch.cuda.stream(side):
                        if il >= 1:
                            side.wait_event(freed[il - 1])          # the set's previous user (layer il - 1) is done with it
                        expand(il + 1, "all")
                        ready[il + 1].record(side)
                main.wait_event(ready[il])
            G.rmsnorm_bf16(x, w.f[b + "attn_norm.weight"], s.rms_eps, xn)
            if not ahead and not resident:
                expand(il, "attn")
            G.gemm_bf16(xn, wqkv, dense_tiles, out_f32=qkv, status=st)
            self.timing.mark(il, "qkv_gemm")
            G.qk_norm_rope_append_prefill(qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"),
                                          e.inv_freq, s.rms_eps, 1.0 / math.sqrt(s.head_dim), s.head_dim, s.n_q, s.n_kv,
                                          T, row_pos, row_seq, e.kv.table, e.kv.n_pages, e.kv.k[il], e.kv.v[il], q_bf,
                                          e.fault, il)
            self.timing.mark(il, "rope_append")
            G.kv_gather_bf16(e.kv.k[il], e.kv.v[il], e.kv.table[slot], e.kv.n_pages, s.n_kv, s.head_dim, n_keys, T_pad,
                             Kb, Vt)
            self.timing.mark(il, "qkv")
            if s.head_dim == 128 and self.flash:
                # scores, softmax and values in one tcgen05 launch: the score matrix stays in tensor memory
                G.flash_prefill(q_bf, Kb, Vt, attn, p0, st)
                self.timing.mark(il, "flash")
            for c0 in range(0, T if not (s.head_dim == 128 and self.flash) else 0, Tq_max):
                Tq = min(Tq_max, T - c0)
                rows = s.n_q * Tq
                S = self._get("S", (rows, T_pad), f32)
                P = self._get("P", (rows, T_pad), bf)
                qk_tiles, pv_tiles, map_s, map_o = self._attn_tables(T, Tq, c0, s.n_q, Gq, p0)
                G.gemm_bf16(q_bf.view(s.n_q * T, s.head_dim), Kb, qk_tiles, out_f32=S, dst_row=map_s, status=st)
                self.timing.mark(il, "scores")
                G.softmax_causal(S, rows, Tq, p0 + c0, T_pad, P)
                self.timing.mark(il, "softmax")
                G.gemm_bf16(P, Vt, pv_tiles, out_bf16=attn.view(T * s.n_q, s.head_dim), dst_row=map_o, status=st)
                self.timing.mark(il, "values")
            self.timing.mark(il, "attention")
            G.gemm_bf16(attn, wo, dense_tiles, out_f32=x, resid=x, status=st)
            self.timing.mark(il, "o_proj")
            if s.layer_is_moe(il):
                rw = w.q[b + "ffn_gate_inp.weight"]
                if rw.qtype == "F32" and T >= 128 and E % 32 == 0:
                    # split-precision tensor-core router: fp32-grade logits from one bf16 GEMM of depth 3K
                    wr = self._router_w.get(il)
                    if wr is None:
                        wr = G.hilo_weights(rw.data.view(torch.float32).view(E, H))
                        self._router_w[il] = wr
                    G.rmsnorm_hilo(x, w.f[b + "ffn_norm.weight"], s.rms_eps, xn3)
                    G.gemm_bf16(xn3, wr, dense_tiles, out_f32=logits, status=st)
                else:
                    K.router(x, w.f[b + "ffn_norm.weight"], s.rms_eps, rw, T, logits, None, None, None, e.fault, il)
                self.timing.mark(il, "router_logits")
                K.route_rows(logits, e._rule(il), T, ids, wts, e.heat[il], e.fault, il)
                self.timing.mark(il, "route")
                G.rmsnorm_bf16(x, w.f[b + "ffn_norm.weight"], s.rms_eps, xn)
                G.moe_plan(ids, wts, E, moe_tiles, pos_of, dst_row, row_scale)
                self.timing.mark(il, "count_scatter")
                G.gather_rows_bf16(xn, dst_row, moe_tiles.offsets[E:E + 1], cap, k, Ap)
                self.timing.mark(il, "dispatch")
                if not ahead and not resident:
                    expand(il, "gate_up")
                self.timing.mark(il, "expand_gate_up")
                G.gemm_bf16(Ap, wg, moe_tiles, out_bf16=act, B2=wu, status=st)
                self.timing.mark(il, "gemm_gate_up")
                if not ahead and not resident:
                    expand(il, "down")
                self.timing.mark(il, "expand_down")
                G.gemm_bf16(act, wd, moe_tiles, out_f32=slot_out, dst_row=dst_row, row_scale=row_scale, status=st)
                self.timing.mark(il, "gemm_down")
                G.moe_combine(slot_out, pos_of, T, k, x, x)
                self.timing.mark(il, "combine")
            else:
                G.rmsnorm_bf16(x, w.f[b + "ffn_norm.weight"], s.rms_eps, xn)
                if not ahead and not resident:
                    expand(il, "gate_up")
                G.gemm_bf16(xn, dg, dense_tiles, out_bf16=dact, B2=du, status=st)
                if not ahead and not resident:
                    expand(il, "down")
                G.gemm_bf16(dact, dd, dense_tiles, out_f32=x, resid=x, status=st)
            if ahead:
                freed[il].record(main)
        if ahead:
            main.wait_stream(side)
        e.x[0].copy_(x[T - 1])
        if int(st.item()) != 0:
            raise RuntimeError("a bounded wait inside the GEMM kernel ran out (status word set)")

    def _use_resident(self) -> bool:
        """Whether the layers' bf16 copies stay in HBM between prompts (decided once, before the first copy exists)."""
        if self.expert_source is not None or self.resident_bf16 is False:
            return False
        if any(q.qtype == "BF16" and q.data.dim() == 3 for q in self.e.w.q.values()):     # bf16 stacks: a copy would only double them
            return False
        if self._resident_ok is None:
            if self.resident_bf16:
                self._resident_ok = True
            else:
                s = self.e.spec
                per_layer = (s.q_rows + 2 * s.kv_rows) * s.hidden + s.hidden * s.q_rows
                per_layer += 3 * s.n_expert * s.moe_inter * s.hidden if s.is_moe else 3 * (s.dense_inter or 0) * s.hidden
                need = 2 * per_layer * s.n_layer
                free, total = torch.cuda.mem_get_info(self.e.device)
                self._resident_ok = free - need >= total // 4
        return self._resident_ok

    def _attn_tables(self, T: int, Tq: int, c0: int, n_q: int, Gq: int, pos0: int = 0):
        key = ("attn", T, Tq, c0, n_q, pos0)
        hit = self._buf.get(key)
        if hit is not None:
            return hit
        dev = self.e.device
        i32 = torch.int32
        rows = torch.full((n_q,), Tq, dtype=i32, device=dev)
        qk = G.TileTable(n_q * Tq, n_q, dev)
        qk.build(rows, group_div=Gq, group_stride=T, base=c0, causal_pos0=pos0 + c0, causal_kind=1)
        pv = G.TileTable(n_q * Tq, n_q, dev)
        pv.build(rows, group_div=Gq, causal_pos0=pos0 + c0, causal_kind=2)
        h = torch.arange(n_q, device=dev).view(n_q, 1)
        i = torch.arange(Tq, device=dev).view(1, Tq)
        map_s = torch.full((n_q * T,), -1, dtype=i32, device=dev)
        map_s.view(n_q, T)[:, c0:c0 + Tq] = (h * Tq + i).to(i32)
        map_o = ((c0 + i) * n_q + h).to(i32).reshape(-1).contiguous()   # index h*Tq + i -> token-major row
        out = (qk, pv, map_s, map_o)
        self._buf[key] = out
        return out
