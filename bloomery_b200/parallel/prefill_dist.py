"""Prompt path on several GPUs: tensor-parallel attention and expert-parallel experts on the tcgen05
GEMM, with the collectives inside the GEMM kernels.

Between layers the residual stream is ROW-SHARDED: rank r owns rows [r * Tr, (r + 1) * Tr) of the
micro-batch (fp32 residual ``x_sh`` and its bf16 normed copy ``xn_sh``, both in symmetric memory).

  all-gather -> QKV GEMM     the GEMM's A tiles are TMA loads straight from the owning rank's ``xn_sh``
                             (one tensor map per source rank, plain tile loads, no cluster multicast);
  o_proj GEMM -> reduce-     the epilogue adds every finished 128 x 256 tile into the owner's ``x_sh`` rows
  scatter                    (``red.global.add.v4.f32`` over NVLink) while the next tile's MMAs run;
  expert dispatch            rows routed to this rank's experts are pulled from their owners' ``xn_sh`` by a
                             gather kernel (plain 16-byte peer loads) into the expert-sorted A matrix;
  down GEMM -> combine       the epilogue scales each row by its router weight and adds it into the owner's
                             ``x_sh`` row of its token: the weighted sum over experts and ranks is the add.

Four flag barriers per layer separate "everyone has written" from "anyone reads" (bounded waits, a status
word on expiry).  NCCL is not on this path.  The floating-point adds into a row arrive in any order, so
prompt logits are reproducible to rounding, not to the bit (the 8-row pass path stays bit-exact).

The reference has no counterpart: its tensor-parallel ranks exchange partial sums through host-side links
(``crates/gpu/src/host/rank.rs``) and it has no expert-parallel all-to-all.
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import os

import torch

from ..ops import decode as K
from ..ops import gemm as G
from ..runtime.kv import PAGE
from .symm import SymmetricBuffer

Phase = List[Callable[[], None]]


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


POISON = None          # None: follow the BLOOMERY_POISON lever; tests set True / False


def _poison() -> bool:
    if POISON is not None:
        return bool(POISON)
    from ..utils import levers
    return bool(levers.get("BLOOMERY_POISON"))


class ShardedGemmPrefill:
    def __init__(self, engine, ubatch: int = 4096, score_bytes: int = 1 << 30, group=None, local_only: bool = False):
        """``engine``: this rank's :class:`ShardedEngine` (local heads and experts, local KV)."""
        self.e = engine
        self.rank, self.world = engine.rank, engine.world
        s = engine.spec
        self.full = engine.full_spec
        N = self.world
        self.tr_max = (ubatch + 128 * N - 1) // (128 * N) * 128
        self.ubatch = self.tr_max * N
        self.score_bytes = score_bytes
        H, k = s.hidden, max(1, s.n_used)
        self.off_x = 0
        self.off_xn = self.off_x + _align(self.tr_max * H * 4)
        self.off_ids = self.off_xn + _align(self.tr_max * H * 2)
        self.off_wts = self.off_ids + _align(self.tr_max * k * 4)
        self.off_flags = self.off_wts + _align(self.tr_max * k * 4)
        total = self.off_flags + 256
        self.sym = SymmetricBuffer(total, self.rank, N, engine.device, group, local_only=local_only)
        self.status = torch.zeros(1, dtype=torch.int32, device=engine.device)
        self.epoch = 0
        self._buf = {}
        self._router_w = {}
        self.emulated = local_only
        self.flash = True                       # head size 128: fused attention on tensor memory (csrc/flash_tcgen05.cu)
        # resident bf16 copies of this rank's matrices, built by the first prompt (see GemmPrefill.resident_bf16)
        from ..utils import levers
        self.resident_bf16 = {"1": True, "0": False}.get(str(levers.get("BLOOMERY_PREFILL_BF16")), None)
        self._resident = {}

    def _bf16(self, il: int, name: str, scratch: torch.Tensor, fill) -> torch.Tensor:
        """Layer il's matrix ``name`` in bf16: expanded into ``scratch`` by ``fill``, and kept as its own copy from then on
        when the card has room (a quarter of it stays free), so later prompts skip the expansion."""
        if self.resident_bf16 is False:
            fill()
            return scratch
        hit = self._resident.get((il, name))
        if hit is None:
            fill()
            if self.resident_bf16 is None:
                free, total = torch.cuda.mem_get_info(self.e.device)
                if free - scratch.numel() * 2 < total // 4:
                    self.resident_bf16 = False
                    return scratch
            hit = scratch.clone()
            self._resident[(il, name)] = hit
        return hit

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

    # ---------------------------------------------------------------------------------
    def barrier(self) -> None:
        self.epoch += 1
        if self.emulated or self.world == 1:
            return                      # emulated ranks share one stream: order is the barrier
        G.rank_barrier(self.sym.peers(self.off_flags), self.sym.ptrs[self.rank] + self.off_flags, self.epoch, self.rank,
                       self.status)

    def run(self, slot: int, tokens: Sequence[int], start: int = 0) -> None:
        """All ranks call this with the same arguments; leaves the last row's hidden state in ``engine.x[0]``."""
        i = 0
        n = len(tokens)
        self.e.kv.ensure(slot, start + n)
        for p in range(start, start + n, PAGE):
            self.e.kv.own(slot, p)
        self.e.kv.sync_table()
        while i < n:
            chunk = tokens[i:i + self.ubatch]
            for phase in self.phases(slot, chunk, start + i):
                for fn in phase:
                    fn()
                self.barrier()
            i += len(chunk)
        self.e.slot_len[slot] = max(self.e.slot_len[slot], start + n)
        if int(self.status.item()) != 0:
            raise RuntimeError("a bounded wait of the several-GPU prompt path ran out (status word set)")

    # ---------------------------------------------------------------------------------
    def phases(self, slot: int, tokens: Sequence[int], p0: int) -> List[Phase]:
        """The micro-batch as barrier-separated lists of launches."""
        e, N, r = self.e, self.world, self.rank
        s, w, dev, full = e.spec, e.w, e.device, self.full
        T = len(tokens)
        Tr = (T + 128 * N - 1) // (128 * N) * 128
        Tp = Tr * N
        H, V, hd = s.hidden, s.vocab, s.head_dim
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        sym = self.sym
        x_sh = sym.view(self.off_x, (Tr, H), f32)
        xn_sh = sym.view(self.off_xn, (Tr, H), bf)
        x_peers, xn_peers = sym.peers(self.off_x), sym.peers(self.off_xn)
        padded = list(tokens) + [0] * (Tp - T)
        tok_own = torch.tensor(padded[r * Tr:(r + 1) * Tr], dtype=i32, device=dev)
        row_pos = torch.arange(p0, p0 + Tp, dtype=i32, device=dev)
        row_seq = torch.full((Tp,), slot, dtype=i32, device=dev)
        row_seq[T:] = -1                                     # pad rows never reach the cache
        qkv_w = s.q_rows + 2 * s.kv_rows
        qkv = self._get("qkv", (Tp, qkv_w), f32)
        wqkv = self._get("wqkv", (qkv_w, H), bf)
        wo = self._get("wo", (H, s.q_rows), bf)
        q_bf = self._get("q_bf", (s.n_q, Tp, hd), bf)
        attn = self._get("attn", (Tp, s.q_rows), bf)
        if Tp > T:
            q_bf[:, T:].zero_()         # pad rows never pass the rope kernel (no sequence): their queries are zeros, not leftovers
        gather_tiles = G.TileTable.sharded(Tp, Tr, dev)
        dense_all = G.TileTable.dense(Tp, dev)
        dense_own = G.TileTable.dense(Tr, dev)
        n_keys = p0 + T
        T_pad = (p0 + Tp + 127) // 128 * 128
        Kb = self._get("Kb", (s.n_kv, T_pad, hd), bf)
        Vt = self._get("Vt", (s.n_kv, hd, T_pad), bf)
        Tq_max = max(128, min(Tp, self.score_bytes // (s.n_q * T_pad * 4) // 128 * 128))
        Gq = s.n_q // s.n_kv
        st = self.status
        moe = s.is_moe
        if moe:
            E, El, I_, k = full.n_expert, full.n_expert // N, s.moe_inter, s.n_used
            e_lo = r * El
            nslot = Tp * k
            cap = nslot + 128
            ids_sh = sym.view(self.off_ids, (Tr, k), i32)
            wts_sh = sym.view(self.off_wts, (Tr, k), f32)
            ids_peers, wts_peers = sym.peers(self.off_ids), sym.peers(self.off_wts)
            logits = self._get("rl", (Tr, E), f32)
            xn3 = self._get("xn3", (Tr, 3 * H), bf)
            ids_all = self._get("ids_all", (Tp, k), i32)
            wts_all = self._get("wts_all", (Tp, k), f32)
            ids_loc = self._get("ids_loc", (Tp, k), i32)
            counts = self._get("counts", (El,), i32)
            cursor = self._get("cursor", (El,), i32)
            pos_of = self._get("pos_of", (nslot,), i32)
            dst_row = self._get("dst_row", (cap,), i32)
            row_scale = self._get("row_scale", (cap,), f32)
            Ap = self._get("Ap", (cap, H), bf)
            act = self._get("act", (cap, I_), bf)
            wg = self._get("wg", (El, I_, H), bf)
            wu = self._get("wu", (El, I_, H), bf)
            wd = self._get("wd", (El, H, I_), bf)
            moe_tiles = G.TileTable(nslot, El, dev)
            heat_scratch = self._get("heat", (E,), i32)
        out: List[Phase] = []

        def first():
            K.embed_rows(tok_own, Tr, w.q["token_embd.weight"], V, x_sh, e.fault)
        cur: Phase = [first]
        for il in range(s.n_layer):
            b = f"blk.{il}."

            def norm1(b=b):
                G.rmsnorm_bf16(x_sh, w.f[b + "attn_norm.weight"], s.rms_eps, xn_sh)
            cur.append(norm1)
            out.append(cur)                                   # ---- barrier: every xn shard is written

            def attention(b=b, il=il):
                def fill_qkv():
                    G.dequant_bf16(w.q[b + "attn_q.weight"], wqkv[:s.q_rows])
                    G.dequant_bf16(w.q[b + "attn_k.weight"], wqkv[s.q_rows:s.q_rows + s.kv_rows])
                    G.dequant_bf16(w.q[b + "attn_v.weight"], wqkv[s.q_rows + s.kv_rows:])
                # all-gather fused: A tiles come from every rank's xn shard
                G.gemm_bf16_dist(xn_peers, Tr, H, self._bf16(il, "wqkv", wqkv, fill_qkv), gather_tiles, src_rows=Tr,
                                 out_f32=qkv, status=st)
                G.qk_norm_rope_append_prefill(qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"),
                                              e.inv_freq, s.rms_eps, e.attn_scale, hd, s.n_q, s.n_kv, Tp, row_pos,
                                              row_seq, e.kv.table, e.kv.n_pages, e.kv.k[il], e.kv.v[il], q_bf, e.fault, il)
                G.kv_gather_bf16(e.kv.k[il], e.kv.v[il], e.kv.table[slot], e.kv.n_pages, s.n_kv, hd, n_keys, T_pad, Kb, Vt)
                if hd == 128 and self.flash:
                    # this rank's heads over the whole chunk: scores, softmax and values in one tcgen05 launch
                    G.flash_prefill(q_bf, Kb, Vt, attn, p0, st)
                for c0 in range(0, Tp if not (hd == 128 and self.flash) else 0, Tq_max):
                    Tq = min(Tq_max, Tp - c0)
                    rows = s.n_q * Tq
                    S = self._get("S", (rows, T_pad), f32)
                    P = self._get("P", (rows, T_pad), bf)
                    qk_tiles, pv_tiles, map_s, map_o = self._attn_tables(Tp, Tq, c0, s.n_q, Gq, p0)
                    G.gemm_bf16(q_bf.view(s.n_q * Tp, hd), Kb, qk_tiles, out_f32=S, dst_row=map_s, status=st)
                    G.softmax_causal(S, rows, Tq, p0 + c0, T_pad, P)
                    G.gemm_bf16(P, Vt, pv_tiles, out_bf16=attn.view(Tp * s.n_q, hd), dst_row=map_o, status=st)
                wo_l = self._bf16(il, "wo", wo, lambda: G.dequant_bf16(w.q[b + "attn_output.weight"], wo))
                # reduce-scatter fused: partial rows are added into their owner's residual shard
                G.gemm_bf16_dist([attn.data_ptr()], Tp, s.q_rows, wo_l, dense_all, owners=x_peers, rows_per_owner=Tr,
                                 ldc=H, status=st)
            out.append([attention])                           # ---- barrier: every residual shard has all partials
            if s.layer_is_moe(il):
                def route(b=b, il=il):
                    rw = w.q[b + "ffn_gate_inp.weight"]
                    if rw.qtype == "F32" and E % 32 == 0:
                        wr = self._router_w.get(il)
                        if wr is None:
                            wr = G.hilo_weights(rw.data.view(torch.float32).view(E, H))
                            self._router_w[il] = wr
                        G.rmsnorm_hilo(x_sh, w.f[b + "ffn_norm.weight"], s.rms_eps, xn3)
                        G.gemm_bf16(xn3, wr, dense_own, out_f32=logits, status=st)
                    else:
                        K.router(x_sh, w.f[b + "ffn_norm.weight"], s.rms_eps, rw, Tr, logits, None, None, None, e.fault, il)
                    K.route_rows(logits, e._rule(il), Tr, ids_sh, wts_sh, heat_scratch, e.fault, il)
                    G.rmsnorm_bf16(x_sh, w.f[b + "ffn_norm.weight"], s.rms_eps, xn_sh)
                out.append([route])                           # ---- barrier: routes and normed rows of all ranks exist

                def experts(b=b, il=il):
                    for src in range(N):                      # routes of every token (a few KiB per rank)
                        G.copy_bytes(ids_peers[src], ids_all[src * Tr:].data_ptr(), Tr * k * 4)
                        G.copy_bytes(wts_peers[src], wts_all[src * Tr:].data_ptr(), Tr * k * 4)
                    G.localize_ids(ids_all, e_lo, e_lo + El, ids_loc)
                    G.moe_plan(ids_loc, wts_all, El, moe_tiles, pos_of, dst_row, row_scale)
                    # dispatch: pull the rows routed to this rank's experts from the ranks that own them
                    G.gather_rows_peer(xn_peers, H, Tr, dst_row, moe_tiles.offsets[El:El + 1], cap, k, H, Ap)
                    wg_l = self._bf16(il, "wg", wg, lambda: G.dequant_bf16(w.q[b + "ffn_gate_exps.weight"], wg))
                    wu_l = self._bf16(il, "wu", wu, lambda: G.dequant_bf16(w.q[b + "ffn_up_exps.weight"], wu))
                    G.gemm_bf16(Ap, wg_l, moe_tiles, out_bf16=act, B2=wu_l, status=st)
                    wd_l = self._bf16(il, "wd", wd, lambda: G.dequant_bf16(w.q[b + "ffn_down_exps.weight"], wd))
                    # combine fused: weighted rows are added into the token owner's residual shard
                    G.gemm_bf16_dist([act.data_ptr()], cap, I_, wd_l, moe_tiles, dst_row=dst_row, row_scale=row_scale,
                                     owners=x_peers, rows_per_owner=Tr, ldc=H, dst_div=k, status=st)
                out.append([experts])                         # ---- barrier: every expert's rows have landed
                cur = []
            else:
                raise NotImplementedError("dense FFN layers are not sharded on the several-GPU prompt path")

        def last():
            owner, lrow = (T - 1) // Tr, (T - 1) % Tr
            G.copy_bytes(x_peers[owner] + lrow * H * 4, e.x.data_ptr(), H * 4)
        out.append([last])
        return out

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
        map_o = ((c0 + i) * n_q + h).to(i32).reshape(-1).contiguous()
        out = (qk, pv, map_s, map_o)
        self._buf[key] = out
        return out
