"""GPU decode engine: static arenas, the per-layer kernel chain, one CUDA graph per
row bucket, a device fault word with a bounded readback.

Counterpart of the reference's ``GpuModel`` (``crates/gpu/src/model.rs``: ``step`` :1419,
``launch_token`` :1471 = refresh params -> replay -> keep rows; ``step_ahead`` :1505;
``MAX_PASS_ROWS = 8`` :369) and of its graph wrapper (``graph.rs``).  Everything that
changes from step to step (token ids, positions, slot of each row, block table, live key
counts, expert ids) lives in device buffers, so a captured graph is replayed unchanged.

Per layer the chain is 8 launches:
  norm+q8+QKV gemv | qk-norm+RoPE+append | flash segments | merge+q8 |
  o_proj+residual | norm+router+top-k | gate·up·SwiGLU+q8 (sel) | down+combine+residual
"""
from __future__ import annotations

import math
import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..models.spec import ModelSpec
from ..models.weights import Weights
from ..ops import decode as K
from .kv import PAGE, KvPool

MAX_ROWS = 8
FAULT_CLEAN = 0xFFFFFFFF

FAULT_SITES = {1: "token id out of range", 2: "non-finite activation", 3: "non-finite router logit",
               4: "expert id out of range", 5: "key count out of range", 6: "KV page missing",
               7: "device wait ran out", 8: "sampler"}


class EngineFault(RuntimeError):
    """The device fault word is set; the engine is poisoned until ``reset_fault``."""

    def __init__(self, word: int):
        self.word = word
        self.layer, self.site = word >> 8, word & 0xFF
        super().__init__(f"device fault at layer {self.layer}: {FAULT_SITES.get(self.site, self.site)}")


class EngineStalled(RuntimeError):
    """A bounded wait on the device ran out (the reference's ``GpuError::Stalled``)."""


def bucket_of(m: int) -> int:
    for b in (1, 2, 4, 8):
        if m <= b:
            return b
    raise ValueError(f"{m} rows exceed a pass of {MAX_ROWS}")


class DecodeEngine:
    def __init__(self, weights: Weights, n_slots: int = 1, slot_ctx: int = 4096, n_seg: Optional[int] = None,
                 use_graphs: bool = True, keep_logits: bool = True, engine_bound_s: float = 60.0,
                 layers: Optional[Tuple[int, int]] = None, stage_first: bool = True, stage_last: bool = True,
                 kv_pages: Optional[int] = None, kv_type: str = "f16"):
        """``kv_type`` "q8_0": keys and values are kept as q8_0 rows (one f16 scale per 32 values, 34 bytes instead of
        64), written by the append launch and expanded to f16 tiles inside the attention launch; GQA models only.
        Prompts of such an engine take the 8-row pass path."""
        self.w = weights
        self.spec: ModelSpec = weights.spec
        s = self.spec
        if kv_type not in ("f16", "q8_0"):
            raise ValueError(f"KV cache type {kv_type!r}: f16 or q8_0")
        self.kv_q8 = kv_type == "q8_0"
        if self.kv_q8 and s.mla:
            raise ValueError("the latent cache of MLA models is f16; q8_0 serves GQA caches")
        if s.mla and (s.kv_lora != 512 or s.rope_dim != 64 or s.nope_dim > 128 or s.v_dim > 128 or s.v_dim % 32):
            raise ValueError("the latent attention kernels serve latent 512 + rope 64, nope and v up to 128")
        self.device = weights.device
        dev = self.device
        self.n_slots, self.slot_ctx = n_slots, slot_ctx
        self.use_graphs = use_graphs
        self.bound_s = engine_bound_s
        max_pages = (slot_ctx + PAGE - 1) // PAGE
        # multi-token-prediction layers ride behind the trunk when the checkpoint carries them
        self.n_mtp = s.n_mtp if f"blk.{s.n_layer}.nextn.eh_proj.weight" in weights.q else 0
        # pipeline stage: this engine runs layers [lo, hi) only; the first stage embeds, the last one has the head
        self.lo, self.hi = layers if layers is not None else (0, s.n_layer)
        self.stage_first, self.stage_last = stage_first, stage_last
        n_kv_layers = (self.hi - self.lo) + (self.n_mtp if stage_last else 0)
        sm = K.sm_count(dev)
        if s.mla:
            self.kv = KvPool(n_kv_layers, 1, s.kv_lora + s.rope_dim, kv_pages or n_slots * max_pages, n_slots, max_pages, dev, v_dim=0)
            self.n_seg = n_seg or max(1, min((slot_ctx + 31) // 32, max(1, 2 * sm // ((s.n_q + 15) // 16))))
        else:
            # kv_pages below n_slots * max_pages overcommits the pool: idle slots spill to pinned host memory
            if self.kv_q8:      # rows of head / 32 f16 scales + head int8 codes; the pool only moves pages of bytes
                self.kv = KvPool(n_kv_layers, s.n_kv, s.head_dim // 32 * 34, kv_pages or n_slots * max_pages, n_slots,
                                 max_pages, dev, dtype=torch.uint8)
            else:
                self.kv = KvPool(n_kv_layers, s.n_kv, s.head_dim, kv_pages or n_slots * max_pages, n_slots, max_pages, dev)
            self.n_seg = n_seg or max(1, min((slot_ctx + 31) // 32, max(1, sm // s.n_kv)))
        H, V = s.hidden, s.vocab
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        R = MAX_ROWS
        # step parameters: tokens, positions, slot of each row (one H2D copy)
        self.params = torch.zeros(4, R, **i32)       # row 3: source row of a draft-layer row
        self.params[2].fill_(-1)
        # pinned staging ring: a slot is rewritten only after the copy that read it has run
        self._stage_n = 16
        self._stage = [torch.zeros(4, R, dtype=torch.int32, pin_memory=True) for _ in range(self._stage_n)]
        self._stage_np = [t.numpy() for t in self._stage]          # same memory: rows are written without tensor indexing
        self._stage_ev = [None] * self._stage_n
        self._stage_i = 0
        self.params_host = self._stage[0]
        self.tokens, self.row_pos, self.row_seq = self.params[0], self.params[1], self.params[2]
        self.x = torch.zeros(R, H, **f32)
        from ..models.rope import attn_scale, inv_freq_table
        self.attn_scale = attn_scale(s)
        if s.mla:
            qk = s.nope_dim + s.rope_dim
            self.o_in = s.n_q * s.v_dim
            # first projection: [q_a (or q) | latent + rope]; the q_b product follows when q is low-rank
            self.qa_w = s.q_lora if s.q_lora else s.n_q * qk
            self.qkv = torch.zeros(R, self.qa_w + s.kv_lora + s.rope_dim, **f32)
            self.q_full = torch.zeros(R, s.n_q * qk, **f32) if s.q_lora else None
            self.q_out = torch.zeros(R, s.n_q, s.kv_lora + s.rope_dim, **f32)
            self.part_ml = torch.zeros(R * s.n_q * self.n_seg * 2, **f32)
            self.part_acc = torch.zeros(R * s.n_q * self.n_seg * s.kv_lora, **f32)
            self.inv_freq = inv_freq_table(s, s.rope_dim).to(dev)
        else:
            self.o_in = s.q_rows
            qkv_w = s.q_rows + 2 * s.kv_rows
            self.qkv = torch.zeros(R, qkv_w, **f32)
            self.q_out = torch.zeros(R, s.n_q, s.head_dim, **f32)
            self.part_ml = torch.zeros(R * s.n_q * self.n_seg * 2, **f32)
            self.part_acc = torch.zeros(R * s.n_q * self.n_seg * s.head_dim, **f32)
            self.inv_freq = inv_freq_table(s, s.head_dim).to(dev)
        self.attn_q = torch.zeros(R, self.o_in, dtype=torch.int8, device=dev)
        self.attn_ds = torch.zeros(R, self.o_in // 32, 2, **f32)
        self.xq = torch.zeros(R, H, dtype=torch.int8, device=dev)
        self.xds = torch.zeros(R, H // 32, 2, **f32)
        # completion tickets of the fused attention launch (one per row and KV head) and of the routing launch (one
        # per group of 8 rows); the kernels leave them zero
        self.tickets = torch.zeros(R * max(1, s.n_kv) + R + 16 + 8, **i32)
        self.x_alt = torch.zeros(R, H, **f32)        # the cluster launch of a layer's expert half writes the residual here
        if s.is_moe:
            self.r_logits = torch.zeros(R, s.n_expert, **f32)
            # chosen experts and weights of every layer of the last pass (the route trace reads them)
            self.r_ids_all = torch.zeros(s.n_layer + self.n_mtp, R, s.n_used, **i32)
            self.r_wts_all = torch.zeros(s.n_layer + self.n_mtp, R, s.n_used, **f32)
            self.r_ids, self.r_wts = self.r_ids_all[0], self.r_wts_all[0]
            self.actq = torch.zeros(R, s.n_used, s.moe_inter, dtype=torch.int8, device=dev)
            self.actds = torch.zeros(R, s.n_used, s.moe_inter // 32, 2, **f32)
            self.heat = torch.zeros(s.n_layer + self.n_mtp, s.n_expert, **i32)
            self.moe_parts = torch.zeros(s.n_used, H, **f32)
            self.p_logits = torch.zeros(R, s.n_expert, **f32)      # scratch of the expert-prediction launches
            self.p_ids = torch.full((R, 16), -1, **i32)
            if s.n_shared:
                self.sh_gu = torch.zeros(R, 2 * s.shared_inter, **f32)
                self.sh_actq = torch.zeros(R, s.shared_inter, dtype=torch.int8, device=dev)
                self.sh_actds = torch.zeros(R, s.shared_inter // 32, 2, **f32)
                self.sh_out = torch.zeros(R, H, **f32)
        if s.dense_inter and (s.first_dense > 0 or not s.is_moe):
            self.gu = torch.zeros(R, 2 * s.dense_inter, **f32)
            self.dactq = torch.zeros(R, s.dense_inter, dtype=torch.int8, device=dev)
            self.dactds = torch.zeros(R, s.dense_inter // 32, 2, **f32)
        if self.n_mtp:
            self.mtp_e = torch.zeros(R, H, **f32)
            self.mtp_x = torch.zeros(R, H, **f32)
            self.mtp_xq = torch.zeros(R, 2 * H, dtype=torch.int8, device=dev)
            self.mtp_xds = torch.zeros(R, 2 * H // 32, 2, **f32)
            self.mtp_logits = torch.zeros(R, V, **f32)
        self.counters = torch.zeros(4, **i32)
        self.logits = torch.zeros(R, V, **f32)
        self.am_blocks = 64
        self.am_v = torch.zeros(R * self.am_blocks, **f32)
        self.am_i = torch.zeros(R * self.am_blocks, **i32)
        self.tokens_out = torch.zeros(R + 1, **i32)
        self.tokens_out_host = torch.zeros(R + 1, dtype=torch.int32, pin_memory=True)
        self._tokens_out_np = self.tokens_out_host.numpy()
        self.fault = torch.full((1,), -1, **i32)  # 0xFFFFFFFF
        self.hist_cap = 4096
        self.hist = torch.zeros(self.hist_cap * R, **i32)
        self.graphs: Dict[Tuple[int, bool, bool], torch.cuda.CUDAGraph] = {}
        self.poisoned: Optional[int] = None
        self.slot_len = [0] * n_slots
        self.launches_per_step = 0
        self.steps = 0
        # prompts at least this long use the GEMM path (0 = never; the GEMM path serves the GQA + routed-expert plan)
        self.gemm_threshold = 0 if (s.mla or s.n_shared or layers is not None or self.kv_q8) else 64
        self.ubatch = 4096
        self._gemm_prefill = None
        self._stream = torch.cuda.Stream(device=dev)
        self._done = torch.cuda.Event()
        self._lock = threading.Lock()
        from .watchdog import Waits, Watchdog
        self.waits = Waits()
        self.watchdog: Optional[Watchdog] = None      # attached by the server; names a wedged wait, never kills
        from ..utils import levers
        self.check_finite = bool(levers.get("BLOOMERY_CHECK_FINITE"))   # read the residual rows back after every pass
        self.step_stats = bool(levers.get("BLOOMERY_STEP_STATS"))       # one stderr record every 256 passes
        self.route_trace = None                       # a RouteTraceWriter when BLOOMERY_ROUTE_TRACE names a directory
        # Expert prediction: at the start of a layer a side-stream launch scores the router on the layer's INPUT rows
        # and asks L2 to prefetch the matrices of the best-scoring experts while the attention launches run; the
        # residual stream moves little across the attention half, so most of the experts the real routing picks
        # ~20 us later are on chip by then (measured on the Qwen3-30B-A3B shape with random weights: the 12 best of
        # the input rows hold 86 % of the 8 the real routing picks).  Only bytes move earlier: results do not change.
        # Measured effect on the decode step: none (2.00 ms off, 2.01 / 2.03 ms with 8 / 12 experts prefetched): the
        # expert launches are bound by their own instruction chains, not by where the bytes come from.  Off.
        self.predict_experts = 0
        self._side = None
        self._forked = False
        self.predict_down = True
        # key segments of a (row, KV head) over a thread-block cluster instead of blocks + completion ticket: about
        # equal at a few hundred keys (1.98 against 1.99 ms per step), behind at 4,096 (351 against 407 tok/s)
        self.attn_clusters = False
        self.mtp_on = False                           # run the draft layer beside every pass (``enable_mtp``)
        self.mtp_draft: Dict[int, Tuple[int, int]] = {}   # slot -> (number of ids the draft extends, drafted id)

    # ---------------------------------------------------------------------------------
    # the kernel chain
    # ---------------------------------------------------------------------------------
    def enqueue(self, M: int, head: bool = True, advance: bool = False) -> int:
        """Enqueue one pass of M rows on the current stream; returns the launch count."""
        s, w = self.spec, self.w
        n = 0
        x = self.x
        if self.stage_first:
            K.embed_rows(self.tokens, M, w.q["token_embd.weight"], s.vocab, x, self.fault); n += 1
        for il in range(self.lo, self.hi):
            x, nl = self._layer(il, M, x)
            n += nl
        if x is not self.x:
            self.x.copy_(x); n += 1            # the residual rows of a finished pass live in self.x
            x = self.x
        self._join_side()
        if head and self.stage_last:
            head_w = w.q.get("output.weight", w.q["token_embd.weight"])
            K.gemv([head_w], M, self.logits, x=x, gain=w.f["output_norm.weight"], eps=s.rms_eps,
                   fault=self.fault, layer=s.n_layer); n += 1
            K.argmax_rows(self.logits, s.vocab, M, self.am_blocks, self.am_v, self.am_i, self.counters[1:2],
                          self.tokens_out, None, self.fault); n += 1
            if advance:
                K.advance_rows(self.tokens, self.row_pos, self.row_seq, self.tokens_out, M, self.hist, self.hist_cap,
                               self.counters[2:3]); n += 1
        return n

    def _layer(self, il: int, M: int, x: torch.Tensor):
        """One transformer block on the residual rows ``x``; returns (the buffer that now holds the residual rows,
        the launch count)."""
        s, w = self.spec, self.w
        n = 0
        b = f"blk.{il}."
        if self.predict_experts and M <= 2 and s.layer_is_moe(il) and type(self)._moe is DecodeEngine._moe:
            n += self._predict(il, M, x)
        n += self._attn(il, M, x)
        K.gemv([w.q[b + "attn_output.weight"]], M, x, xq=self.attn_q, xds=self.attn_ds, resid=x,
               fault=self.fault, layer=il); n += 1
        if s.layer_is_moe(il):
            if M == 1 and type(self)._moe is DecodeEngine._moe and not s.n_shared and self._cluster_ok(il):
                # one row: router, routing, the chosen experts and the weighted sum as ONE cluster launch
                other = self.x_alt if x is not self.x_alt else self.x
                K.moe_cluster(x, w.f[b + "ffn_norm.weight"], s.rms_eps, w.q[b + "ffn_gate_inp.weight"], self._rule(il), None,
                              w.q[b + "ffn_gate_exps.weight"], w.q[b + "ffn_up_exps.weight"], w.q[b + "ffn_down_exps.weight"],
                              s.n_used, None, self.moe_parts, self.tickets[MAX_ROWS * max(1, s.n_kv) + MAX_ROWS:], other,
                              self.r_logits, self.r_ids_all[il], self.r_wts_all[il], self.heat[il], self.fault, il)
                return other, n + 1
            n += self._moe(il, M, x)
        else:
            K.gemv([w.q[b + "ffn_gate.weight"], w.q[b + "ffn_up.weight"]], M, self.gu, x=x,
                   gain=w.f[b + "ffn_norm.weight"], eps=s.rms_eps, fault=self.fault, layer=il); n += 1
            K.swiglu_q8(self.gu, s.dense_inter, M, self.dactq, self.dactds); n += 1
            K.gemv([w.q[b + "ffn_down.weight"]], M, x, xq=self.dactq, xds=self.dactds, resid=x,
                   fault=self.fault, layer=il); n += 1
        return x, n

    def _join_side(self) -> None:
        if self._forked:
            torch.cuda.current_stream(self.device).wait_stream(self._side)      # join the prediction branch
            self._forked = False

    def _predict(self, il: int, M: int, x: torch.Tensor) -> int:
        """Fork a side-stream launch that predicts this layer's experts from its input rows and prefetches them to L2.
        It reads ``x`` while the main chain later updates it in place; a late read only blurs the prediction."""
        s, w = self.spec, self.w
        b = f"blk.{il}."
        main = torch.cuda.current_stream(self.device)
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            r = self._rule(il)
            rule = K.RouteRule(self.predict_experts, r.mode, r.renorm, r.scale, 1, 1, r.bias)
            gate, up, down = w.q[b + "ffn_gate_exps.weight"], w.q[b + "ffn_up_exps.weight"], w.q[b + "ffn_down_exps.weight"]
            K.router(x, w.f[b + "ffn_norm.weight"], s.rms_eps, w.q[b + "ffn_gate_inp.weight"], M, self.p_logits, None, None,
                     None, None, il, rule=rule, ids=self.p_ids, ticket=self.tickets[MAX_ROWS * max(1, s.n_kv) + MAX_ROWS + 16:],
                     predict=(gate, up, down))
            K.prefetch_experts(self.p_ids, M * self.predict_experts, gate, up, down if self.predict_down else None,
                               K.sm_count(self.device))
        self._forked = True
        return 2

    def _cluster_ok(self, il: int) -> bool:
        w, b = self.w, f"blk.{il}."
        return K.moe_cluster_fits(w.q[b + "ffn_gate_inp.weight"], w.q[b + "ffn_gate_exps.weight"],
                                  w.q[b + "ffn_up_exps.weight"], w.q[b + "ffn_down_exps.weight"], self.spec.n_used)

    def enqueue_mtp(self, M: int) -> int:
        """The draft layer on M rows: params row 0 = the token that FOLLOWS each position, row 3 = the pass row whose
        final hidden state it pairs with (``self.x`` still holds the trunk's last pass).  Greedy draft ids land in
        ``tokens_out`` like a trunk pass's picks (the reference: ``crates/app/src/mtp.rs:1-33``)."""
        s, w = self.spec, self.w
        il = s.n_layer
        b = f"blk.{il}."
        n = 0
        K.embed_rows(self.tokens, M, w.q["token_embd.weight"], s.vocab, self.mtp_e, self.fault); n += 1
        K.mtp_prep(self.mtp_e, self.x, self.params[3], w.f[b + "nextn.enorm.weight"], w.f[b + "nextn.hnorm.weight"],
                   s.rms_eps, M, self.mtp_xq, self.mtp_xds); n += 1
        K.gemv([w.q[b + "nextn.eh_proj.weight"]], M, self.mtp_x, xq=self.mtp_xq, xds=self.mtp_xds, fault=self.fault,
               layer=il); n += 1
        xo, nl = self._layer(il, M, self.mtp_x)
        n += nl
        head_w = w.q.get("output.weight", w.q["token_embd.weight"])
        K.gemv([head_w], M, self.mtp_logits, x=xo, gain=w.f[b + "nextn.shared_head_norm.weight"], eps=s.rms_eps,
               fault=self.fault, layer=il); n += 1
        K.argmax_rows(self.mtp_logits, s.vocab, M, self.am_blocks, self.am_v, self.am_i, self.counters[1:2],
                      self.tokens_out, None, self.fault); n += 1
        self._join_side()
        return n

    def mtp_step(self, rows: Sequence[Tuple[int, int, int, int]]) -> List[int]:
        """rows = [(slot, next token, position, source row of the last trunk pass)]; returns the drafted id after
        each row's next token (the layer's KV rows at those positions are written on the way)."""
        if not self.n_mtp:
            raise RuntimeError("this checkpoint has no multi-token-prediction layer")
        with self._lock:
            M = self.set_rows([(sl, tok, pos) for sl, tok, pos, _ in rows], src=[r[3] for r in rows])
            if self.poisoned is not None:
                raise EngineFault(self.poisoned)
            if self.use_graphs:
                key = ("mtp", M)
                g = self.graphs.get(key)
                if g is None:
                    st = self._stream
                    st.wait_stream(torch.cuda.current_stream(self.device))
                    saved = self.params.clone()
                    with torch.cuda.stream(st):
                        self.params[2].fill_(-1)
                        self.enqueue_mtp(M)
                        st.synchronize()
                        self.params.copy_(saved)
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g, stream=st):
                            self.enqueue_mtp(M)
                    torch.cuda.current_stream(self.device).wait_stream(st)
                    self.graphs[key] = g
                g.replay()
            else:
                self.enqueue_mtp(M)
            out = self.read_tokens(len(rows))
            word = out[M] & 0xFFFFFFFF
            if word != FAULT_CLEAN:
                self.poisoned = word
                raise EngineFault(word)
            return out[:len(rows)]

    def enable_mtp(self, on: bool = True) -> bool:
        self.mtp_on = bool(on) and self.n_mtp > 0
        return self.mtp_on

    def draft_after(self, rows: Sequence[Tuple[int, int, int]], picks: Sequence[int], slots=None) -> None:
        """Run the draft layer for the rows of the pass that just ended (``self.x`` still holds their hidden states).
        A row counts when every earlier row of its slot in the pass was followed by the token the trunk picked
        (rows of rejected drafts are skipped); the last counted row of a slot leaves that slot's next draft."""
        by_slot: Dict[int, List[int]] = {}
        for i, (sl, _, _) in enumerate(rows):
            if slots is None or sl in slots:
                by_slot.setdefault(sl, []).append(i)
        mrows, last_of = [], {}
        for sl, idx in by_slot.items():
            for j, ri in enumerate(idx):
                if j > 0 and rows[ri][1] != picks[idx[j - 1]]:
                    break
                last_of[sl] = len(mrows)
                mrows.append((sl, int(picks[ri]), rows[ri][2], ri))
        for i in range(0, len(mrows), MAX_ROWS):
            part = mrows[i:i + MAX_ROWS]
            drafts = self.mtp_step(part)
            for sl, k in last_of.items():
                if i <= k < i + len(part):
                    self.mtp_draft[sl] = (part[k - i][2] + 2, drafts[k - i])

    def _attn(self, il: int, M: int, x: torch.Tensor) -> int:
        """Attention of one layer up to the q8 rows that feed o_proj; returns the launch count."""
        s, w, kvp = self.spec, self.w, self.kv
        b = f"blk.{il}."
        if s.mla:
            return self._attn_mla(il, M, x)
        K.gemv([w.q[b + "attn_q.weight"], w.q[b + "attn_k.weight"], w.q[b + "attn_v.weight"]], M, self.qkv,
               x=x, gain=w.f[b + "attn_norm.weight"], eps=s.rms_eps, fault=self.fault, layer=il,
               prefetch=self._static_next(il))
        cl = K.attn_cluster_size(s.n_kv, M) if (self.attn_clusters and not self.kv_q8) else 0
        if cl:
            K.attn_cluster(self.qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"), self.inv_freq,
                           s.rms_eps, self.attn_scale, s.head_dim, s.n_q, s.n_kv, M, self.row_pos, self.row_seq, kvp.table,
                           kvp.n_pages, kvp.k[il - self.lo], kvp.v[il - self.lo], cl, self.slot_ctx, None, self.attn_q,
                           self.attn_ds, self.fault, il)
            return 2
        if K.staged_part("attn") and not self.kv_q8:
            K.attn_fused(self.qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"), self.inv_freq,
                         s.rms_eps, self.attn_scale, s.head_dim, s.n_q, s.n_kv, M, self.row_pos, self.row_seq, kvp.table,
                         kvp.n_pages, kvp.k[il - self.lo], kvp.v[il - self.lo], self.n_seg, self.slot_ctx, self.part_ml,
                         self.part_acc, self.tickets, None, self.attn_q, self.attn_ds, self.fault, il)
            return 2
        K.qk_norm_rope_append(self.qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"),
                              self.inv_freq, s.rms_eps, self.attn_scale, s.head_dim, s.n_q, s.n_kv, M,
                              self.row_pos, self.row_seq, kvp.table, kvp.n_pages, kvp.k[il - self.lo], kvp.v[il - self.lo], self.q_out,
                              self.fault, il, kv_q8=self.kv_q8)
        K.flash_decode(self.q_out, kvp.k[il - self.lo], kvp.v[il - self.lo], self.row_pos, self.row_seq, kvp.table, kvp.n_pages,
                       s.head_dim, s.n_q, s.n_kv, M, self.n_seg, self.slot_ctx, self.part_ml, self.part_acc, None,
                       self.attn_q, self.attn_ds, self.fault, il, kv_q8=self.kv_q8)
        return 4

    def _static_next(self, il: int):
        """Weights of the NEXT layer that do not depend on routing (projections, router): the first launch of a layer
        asks L2 to fetch them, a whole layer ahead of their use."""
        nb = f"blk.{il + 1}."
        names = ("attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight", "ffn_gate_inp.weight")
        return [self.w.q[nb + n].data for n in names if nb + n in self.w.q] if il + 1 < self.hi else None

    def _attn_mla(self, il: int, M: int, x: torch.Tensor) -> int:
        """Latent attention: [q_a | kv_a] product, latent append, (q_b product), absorb, latent flash + value
        up-projection (the reference's MLA seat: ``crates/gpu/src/flash.rs``, deepseek2 chain)."""
        s, w, kvp = self.spec, self.w, self.kv
        b = f"blk.{il}."
        n = 0
        first = w.q[b + "attn_q_a.weight"] if s.q_lora else w.q[b + "attn_q.weight"]
        K.gemv([first, w.q[b + "attn_kv_a_mqa.weight"]], M, self.qkv, x=x, gain=w.f[b + "attn_norm.weight"],
               eps=s.rms_eps, fault=self.fault, layer=il); n += 1
        K.mla_kv_append(self.qkv[:, self.qa_w:], w.f[b + "attn_kv_a_norm.weight"], self.inv_freq, s.rms_eps, M,
                        self.row_pos, self.row_seq, kvp.table, kvp.n_pages, kvp.k[il - self.lo], self.fault, il); n += 1
        if s.q_lora:
            K.gemv([w.q[b + "attn_q_b.weight"]], M, self.q_full, x=self.qkv[:, :s.q_lora],
                   gain=w.f[b + "attn_q_a_norm.weight"], eps=s.rms_eps, fault=self.fault, layer=il); n += 1
            q = self.q_full
        else:
            q = self.qkv[:, :self.qa_w]
        K.mla_q_absorb(q, w.f[b + "attn_k_b.weight"], self.inv_freq, self.attn_scale, s.n_q, s.nope_dim, M,
                       self.row_pos, self.row_seq, self.q_out); n += 1
        K.mla_flash_decode(self.q_out, kvp.k[il - self.lo], self.row_pos, self.row_seq, kvp.table, kvp.n_pages, s.n_q, M,
                           self.n_seg, self.slot_ctx, self.part_ml, self.part_acc, w.f[b + "attn_v_b.weight"], s.v_dim,
                           None, self.attn_q, self.attn_ds, self.fault, il); n += 2
        return n

    def _moe(self, il: int, M: int, x: torch.Tensor) -> int:
        """Router + routed experts + combine of one layer (3 launches); returns the launch count."""
        s, w = self.spec, self.w
        b = f"blk.{il}."
        ids, wts = self.r_ids_all[il], self.r_wts_all[il]
        gate, up, down = w.q[b + "ffn_gate_exps.weight"], w.q[b + "ffn_up_exps.weight"], w.q[b + "ffn_down_exps.weight"]
        staged = gate.qtype == up.qtype and K.moe_fits_stage(gate, down, s.n_used)
        K.router(x, w.f[b + "ffn_norm.weight"], s.rms_eps, w.q[b + "ffn_gate_inp.weight"], M, self.r_logits,
                 self.xq, self.xds, None, self.fault, il)
        if staged:
            # warp 0 of every block routes its row from the logits while the other warps fetch the activations
            K.gate_up_staged(self.xq, self.xds, ids, None, gate, up, s.n_expert, s.n_used, M, self.actq, self.actds,
                             None, self.fault, il, down=down, route_logits=self.r_logits, rule=self._rule(il), wts=wts,
                             heat=self.heat[il])
        else:
            K.gate_up_sel(self.xq, self.xds, ids, None, gate, up, s.n_expert, s.n_used, M, self.actq, self.actds, None,
                          self.fault, il, route_logits=self.r_logits, rule=self._rule(il), wts=wts, heat=self.heat[il],
                          down=down)
        extra, n = None, 3
        if s.n_shared:
            # the shared expert reads the router's q8 rows and lands as an extra addend of the combine
            K.gemv([w.q[b + "ffn_gate_shexp.weight"], w.q[b + "ffn_up_shexp.weight"]], M, self.sh_gu, xq=self.xq,
                   xds=self.xds, fault=self.fault, layer=il)
            K.swiglu_q8(self.sh_gu, s.shared_inter, M, self.sh_actq, self.sh_actds)
            K.gemv([w.q[b + "ffn_down_shexp.weight"]], M, self.sh_out, xq=self.sh_actq, xds=self.sh_actds,
                   fault=self.fault, layer=il)
            extra, n = self.sh_out, 6
        (K.down_staged if staged else K.down_combine)(self.actq, self.actds, ids, wts, None, down, s.n_expert, s.n_used,
                                                      M, x, extra, x, self.fault, il)
        return n

    def _after_pass(self, n_rows: int) -> None:
        """Hook between passes (residency boundaries live here in the tiered engine)."""

    def _rule(self, il: int) -> "K.RouteRule":
        s = self.spec
        return K.RouteRule(s.n_used, 0 if s.router_mode == "softmax" else 1, s.router_renorm, s.router_scale,
                           s.n_group, s.topk_group, self.w.f.get(f"blk.{il}.exp_probs_b.bias"))

    def _graph(self, M: int, head: bool, advance: bool) -> torch.cuda.CUDAGraph:
        key = (M, head, advance)
        g = self.graphs.get(key)
        if g is None:
            # warm up eagerly once (sets function attributes, loads modules), then capture
            st = self._stream
            st.wait_stream(torch.cuda.current_stream(self.device))
            saved = self.params.clone()
            with torch.cuda.stream(st):
                self.params[2].fill_(-1)        # padding rows only: touches no KV
                self.enqueue(M, head, False)
                st.synchronize()
                self.params.copy_(saved)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    self.launches_per_step = self.enqueue(M, head, advance)
            torch.cuda.current_stream(self.device).wait_stream(st)
            self.graphs[key] = g
        return g

    # ---------------------------------------------------------------------------------
    # host protocol
    # ---------------------------------------------------------------------------------
    def set_rows(self, rows: Sequence[Tuple[int, int, int]], src: Optional[Sequence[int]] = None) -> int:
        """rows = [(slot, token, position)]; pads to the bucket; returns the bucket size."""
        m = len(rows)
        M = bucket_of(m)
        i = self._stage_i
        self._stage_i = (i + 1) % self._stage_n
        if self._stage_ev[i] is not None:
            self._stage_ev[i].synchronize()
        ph = self.params_host = self._stage[i]
        hp = self._stage_np[i]
        hp[2, :] = -1
        self.kv.protect = {r[0] for r in rows}          # slots of this pass never spill
        for r, (slot, tok, pos) in enumerate(rows):
            hp[0, r] = tok
            hp[1, r] = pos
            hp[2, r] = slot
            hp[3, r] = src[r] if src is not None else r
            self.kv.ensure(slot, pos + 1)
            self.kv.own(slot, pos)
        self.kv.sync_table()
        self.params.copy_(ph, non_blocking=True)
        ev = self._stage_ev[i]
        if ev is None:
            ev = self._stage_ev[i] = torch.cuda.Event()
        ev.record()
        return M

    def launch(self, M: int, head: bool = True, advance: bool = False) -> None:
        if self.poisoned is not None:
            raise EngineFault(self.poisoned)
        if self.use_graphs:
            self._graph(M, head, advance).replay()
        else:
            self.enqueue(M, head, advance)
        self.steps += 1

    def read_tokens(self, m: int) -> List[int]:
        """Bounded readback of the chosen tokens and the fault word."""
        self.tokens_out_host.copy_(self.tokens_out, non_blocking=True)
        self._done.record()
        t0 = time.monotonic()
        tok = self.watchdog.enter("step readback") if self.watchdog is not None else None
        try:
            while not self._done.query():
                if time.monotonic() - t0 > self.bound_s:
                    raise EngineStalled(f"no answer from the device within {self.bound_s:.0f} s")
                time.sleep(0)
        finally:
            if tok is not None:
                self.watchdog.leave(tok)
            self.waits.add("card", time.monotonic() - t0)
        # the kernel writes the fault copy at index M (the bucket size)
        return self._tokens_out_np.tolist()

    def _float_expert_pass(self):
        """bf16 expert stacks have no int8-dot kernel: every pass of such a model, however few rows, is the batched
        tensor-core pass (``runtime/batch_decode.py``), which multiplies bf16 rows in place."""
        if not hasattr(self, "_float_pass"):
            self._float_pass = None
            s = self.spec
            if s.is_moe and type(self) is DecodeEngine:
                moe0 = next(il for il in range(s.n_layer) if s.layer_is_moe(il))
                if self.w.q[f"blk.{moe0}.ffn_gate_exps.weight"].qtype == "BF16":
                    from .batch_decode import BatchDecode
                    self._float_pass = BatchDecode(self, max_rows=16)
        return self._float_pass

    def step(self, rows: Sequence[Tuple[int, int, int]], head: bool = True) -> List[int]:
        """One pass over ``rows``; returns the greedy token of every row."""
        bd = self._float_expert_pass()
        if bd is not None:
            with self._lock:
                out = bd.step(rows)
                self.logits[:len(rows)].copy_(bd.logits[:len(rows)])
                return out if head else []
        with self._lock:
            M = self.set_rows(rows)
            self.launch(M, head, False)
            self._after_pass(len(rows))
            for slot, _, pos in rows:
                self.slot_len[slot] = max(self.slot_len[slot], pos + 1)
            if self.route_trace is not None and self.spec.is_moe:
                # the picks of every layer of this pass are still on the card: one read per pass
                ids = self.r_ids_all[:, :len(rows)].cpu().tolist()
                wts = self.r_wts_all[:, :len(rows)].cpu().tolist()
                for il in range(self.spec.first_dense, self.spec.n_layer):
                    for r, (_, _, pos) in enumerate(rows):
                        self.route_trace.add(pos, il, ids[il][r], wts[il][r])
            if self.check_finite and not bool(torch.isfinite(self.x[:len(rows)]).all()):
                self.poisoned = (self.spec.n_layer << 8) | 2
                raise EngineFault(self.poisoned)
            if self.step_stats and self.steps % 256 == 0:
                from ..utils import records
                records.write("step_stats", steps=self.steps, card_wait_s=round(self.waits.ns.get("card", 0) / 1e9, 4),
                              kv_free_pages=self.kv.free_pages(), kv_spills=self.kv.n_spills,
                              free_bytes=int(torch.cuda.mem_get_info(self.device)[0]))
            if not head:
                return []
            out = self.read_tokens(len(rows))
            word = out[M] & 0xFFFFFFFF
            if word != FAULT_CLEAN:
                self.poisoned = word
                raise EngineFault(word)
            return out[:len(rows)]

    def _new_gemm_prefill(self):
        from .prefill import GemmPrefill
        return GemmPrefill(self, ubatch=self.ubatch)

    def prefill(self, slot: int, tokens: Sequence[int], start: int = 0, gemm: Optional[bool] = None) -> int:
        """Feed a prompt; returns the greedy token after it.  Prompts of at least
        ``gemm_threshold`` rows go through the tcgen05 GEMM path in micro-batches, shorter
        ones through passes of up to 8 rows of the decode chain."""
        n = len(tokens)
        use_gemm = gemm if gemm is not None else (self.gemm_threshold > 0 and n >= self.gemm_threshold)
        use_gemm = use_gemm and not self.mtp_on        # the draft layer's prompt rows run on the pass path
        if use_gemm and n > 1:
            if self._gemm_prefill is None:
                self._gemm_prefill = self._new_gemm_prefill()
            with self._lock:
                if self.poisoned is not None:
                    raise EngineFault(self.poisoned)
                self._gemm_prefill.run(slot, tokens, start)
                head_w = self.w.q.get("output.weight", self.w.q["token_embd.weight"])
                K.gemv([head_w], 1, self.logits, x=self.x, gain=self.w.f["output_norm.weight"], eps=self.spec.rms_eps,
                       fault=self.fault, layer=self.spec.n_layer)
                K.argmax_rows(self.logits, self.spec.vocab, 1, self.am_blocks, self.am_v, self.am_i,
                              self.counters[1:2], self.tokens_out, None, self.fault)
                out = self.read_tokens(1)
                word = out[1] & 0xFFFFFFFF
                if word != FAULT_CLEAN:
                    self.poisoned = word
                    raise EngineFault(word)
                return out[0]
        last = None
        n = len(tokens)
        i = 0
        while i < n:
            chunk = tokens[i:i + MAX_ROWS]
            is_last = i + len(chunk) >= n
            rows = [(slot, int(t), start + i + j) for j, t in enumerate(chunk)]
            out = self.step(rows, head=is_last)
            if self.mtp_on:
                # the draft layer keeps KV rows for the prompt too: row j pairs with the prompt token after it,
                # the last row with the greedy pick
                mrows = [(slot, int(tokens[i + j + 1]), start + i + j, j) for j in range(len(chunk)) if i + j + 1 < n]
                if is_last:
                    mrows.append((slot, int(out[len(chunk) - 1]), start + n - 1, len(chunk) - 1))
                drafts = self.mtp_step(mrows)
                if is_last:
                    self.mtp_draft[slot] = (start + n + 1, drafts[-1])
            if is_last:
                last = out[len(chunk) - 1]
            i += len(chunk)
        return last

    def score(self, slot: int, tokens: Sequence[int], start: int = 0) -> List[int]:
        """Greedy pick after every position of ``tokens`` (teacher forcing; the head runs on each pass)."""
        picks: List[int] = []
        for i in range(0, len(tokens), MAX_ROWS):
            chunk = tokens[i:i + MAX_ROWS]
            picks += self.step([(slot, int(t), start + i + j) for j, t in enumerate(chunk)], head=True)
        return picks

    def decode_chain(self, slot: int, first_token: int, start_pos: int, n_steps: int) -> List[int]:
        """Greedy decode of ``n_steps`` tokens with the next step's input kept on the card:
        the graph ends in a kernel that feeds the pick back and advances the position, so
        replays are launched back to back and read once (``step_ahead`` in the reference)."""
        self.kv.ensure(slot, start_pos + n_steps + 1)
        with self._lock:
            if n_steps > self.hist_cap:
                raise ValueError(f"a chain of {n_steps} steps exceeds the history ring of {self.hist_cap}")
            self.set_rows([(slot, first_token, start_pos)])
            self.counters[2:3].zero_()
            for i in range(n_steps):
                self.launch(1, True, True)
                self._after_pass(1)
            out = self.hist[:n_steps].cpu().tolist()
            self.slot_len[slot] = start_pos + n_steps
            self.check_fault()
            return out

    def check_fault(self) -> None:
        word = int(self.fault.cpu().item()) & 0xFFFFFFFF
        if word != FAULT_CLEAN:
            self.poisoned = word
            raise EngineFault(word)

    def reset_fault(self) -> None:
        self.fault.fill_(-1)
        self.counters.zero_()
        self.poisoned = None

    def plant_fault(self, layer: int, site: int) -> None:
        """Host-side injection used by tests (``GpuModel::plant_fault`` in the reference)."""
        self.fault.fill_(((layer << 8) | site) - (1 << 32))

    # slot management --------------------------------------------------------------------
    def cut(self, slot: int, n_positions: int) -> None:
        self.kv.truncate(slot, n_positions)
        self.slot_len[slot] = min(self.slot_len[slot], n_positions)

    def reset(self, slot: int) -> None:
        self.cut(slot, 0)

    def memory_report(self) -> Dict[str, int]:
        return {"weights": self.w.n_bytes, "kv": self.kv.bytes}
