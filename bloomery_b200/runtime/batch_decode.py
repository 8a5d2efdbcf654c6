"""Batched decode on the tensor cores: one pass of up to 64 rows (one token of 64 different sequences).

The 8-row decode chain reads every weight byte once per pass with int8 dot products; that is the right shape up to a
handful of rows.  Past that the matrix products move to tcgen05 with the weights still block-quantised in HBM
(``csrc/qgemm_tcgen05.cu``): the rows are the N side of the MMA in tiles of 32, every weight block is read and
expanded once per pass whatever the row count, and a pass over a routed-expert layer touches each chosen expert once
for all the rows routed to it.  Per layer:

  RMSNorm -> bf16 rows, Q / K / V products, per-head norm + RoPE + KV append, split-K flash decode over the paged
  cache (every row its own sequence and position), o product with the residual, router logits + top-k, expert-sorted
  plan (count / offsets / 32-row tiles / scatter in one launch), gather, gate+up with SwiGLU in the epilogue, down
  with the router weight in the epilogue, slot-ordered combine, the shared expert as one more dense SwiGLU pair.
  Latent-attention models run q_a / kv_a / q_b as products of the same kind around the latent append, the absorb and
  the latent flash decode of the 8-row chain, whose kernels take any row count.

The whole pass is one CUDA graph per row bucket (16 / 32 / 64).  The reference's counterpart is its batched decode
over sequences (``crates/gpu/src/arch/qwen3moe/decode.rs``: the int8 mma.sync grouped GEMMs take over from the GEMV
kernels above a row threshold).
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence, Tuple

import torch

from ..ops import decode as K
from ..ops import gemm as G

TILE = 32
BUCKETS = (16, 32, 64)


class BatchDecode:
    """Rows beyond the 8-row chain of a :class:`DecodeEngine`: grouped-query or latent attention, routed experts (with
    or without a shared expert) or dense FFN layers."""

    def __init__(self, engine, max_rows: int = 64):
        e = self.e = engine
        s = e.spec
        if e.lo != 0 or e.hi != s.n_layer:
            raise NotImplementedError("the batched tensor-core pass runs whole models, not a stage of layers")
        if max_rows > BUCKETS[-1]:
            raise ValueError(f"at most {BUCKETS[-1]} rows per pass")
        self.R = R = max_rows
        dev = e.device
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        H, V = s.hidden, s.vocab
        self.params = torch.zeros(3, R, **i32)
        self.params[2].fill_(-1)
        self.params_host = torch.zeros(3, R, dtype=torch.int32, pin_memory=True)
        self.tokens, self.row_pos, self.row_seq = self.params[0], self.params[1], self.params[2]
        self.x = torch.zeros(R, H, **f32)
        self.xn = torch.zeros(R, H, **bf)
        sm = K.sm_count(dev)
        if s.mla:
            # latent attention: [q_a | kv_a] rows, the full per-head queries, the absorbed queries [n_q, latent + rope]
            qk = s.nope_dim + s.rope_dim
            self.qa_w = s.q_lora if s.q_lora else s.n_q * qk
            self.qkv = torch.zeros(R, self.qa_w + s.kv_lora + s.rope_dim, **f32)
            self.qn = torch.zeros(R, s.q_lora, **bf) if s.q_lora else None
            self.q_full = torch.zeros(R, s.n_q * qk, **f32) if s.q_lora else None
            self.q_out = torch.zeros(R, s.n_q, s.kv_lora + s.rope_dim, **f32)
            self.n_seg = max(1, min(e.n_seg, (2 * sm) // (((s.n_q + 15) // 16) * BUCKETS[0]) + 1))
            self.part_ml = torch.zeros(R * s.n_q * self.n_seg * 2, **f32)
            self.part_acc = torch.zeros(R * s.n_q * self.n_seg * s.kv_lora, **f32)
            aw = s.n_q * s.v_dim
        else:
            self.qkv = torch.zeros(R, s.q_rows + 2 * s.kv_rows, **f32)
            self.q_out = torch.zeros(R, s.n_q, s.head_dim, **f32)
            # key segments: enough blocks to fill the card at the smallest bucket, no more
            self.n_seg = max(1, min(e.n_seg, (2 * sm) // (s.n_kv * BUCKETS[0]) + 1))
            self.part_ml = torch.zeros(R * s.n_q * self.n_seg * 2, **f32)
            self.part_acc = torch.zeros(R * s.n_q * self.n_seg * s.head_dim, **f32)
            aw = s.q_rows
        self.attn = torch.zeros(R, aw, **f32)
        self.attn_bf = torch.zeros(R, aw, **bf)
        self.attn_q = torch.zeros(R, aw, dtype=torch.int8, device=dev)
        self.attn_ds = torch.zeros(R, aw // 32, 2, **f32)
        if s.is_moe:
            E, k, I_ = s.n_expert, s.n_used, s.moe_inter
            n = R * k
            self.cap = n + 128
            self.logits_r = torch.zeros(R, E, **f32)
            self.ids = torch.zeros(R, k, **i32)
            self.wts = torch.zeros(R, k, **f32)
            self.pos_of = torch.zeros(n, **i32)
            self.dst_row = torch.zeros(self.cap, **i32)
            self.row_scale = torch.zeros(self.cap, **f32)
            self.Ap = torch.zeros(self.cap, H, **bf)
            self.act = torch.zeros(self.cap, I_, **bf)
            self.slot_out = torch.zeros(n, H, **f32)
            # bf16 expert stacks multiply as they are through the bf16 GEMM, whose token tiles are 128 rows
            moe0 = next(il for il in range(s.n_layer) if s.layer_is_moe(il))
            self.float_experts = e.w.q[f"blk.{moe0}.ffn_gate_exps.weight"].qtype == "BF16"
            self.moe_tiles = G.TileTable(n, E, dev, 128 if self.float_experts else TILE)
        # widths come from the weights: a rank of a several-GPU engine holds a slice of the dense and shared widths
        wq = e.w.q
        dense = [il for il in range(s.n_layer) if not s.layer_is_moe(il)]
        if dense:
            self.dact = torch.zeros(R, wq[f"blk.{dense[0]}.ffn_gate.weight"].rows, **bf)
        if s.n_shared:
            moe = [il for il in range(s.n_layer) if s.layer_is_moe(il)]
            self.sh_act = torch.zeros(R, wq[f"blk.{moe[0]}.ffn_gate_shexp.weight"].rows, **bf)
        self._check_types()
        self.logits = torch.zeros(R, V, **f32)
        self.am_blocks = 64
        self.am_v = torch.zeros(R * self.am_blocks, **f32)
        self.am_i = torch.zeros(R * self.am_blocks, **i32)
        self.counters = torch.zeros(4, **i32)
        self.tokens_out = torch.zeros(R + 1, **i32)
        self.tokens_out_host = torch.zeros(R + 1, dtype=torch.int32, pin_memory=True)
        self.hist_cap = 1024
        self.hist = torch.zeros(self.hist_cap * R, **i32)
        self.status = torch.zeros(1, **i32)
        # dense products take the whole bucket as one token tile where a tile size exists for it
        self.dense_tiles: Dict[int, G.TileTable] = {m: G.TileTable.dense(m, dev, 64 if m == 64 else TILE)
                                                    for m in BUCKETS if m <= R}
        self.graphs: Dict[Tuple[int, bool], torch.cuda.CUDAGraph] = {}
        self.launches_per_step = 0
        self._scratch_w: Dict[str, torch.Tensor] = {}
        from ..utils import levers
        self.fp8_native = bool(levers.get("BLOOMERY_FP8_NATIVE"))
        # the engine's own stream: its 8-row passes and prompts and these passes touch the same KV pages in order
        self._stream = getattr(engine, "_stream", None) or torch.cuda.Stream(device=dev)
        self._side = [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)]
        from .timing import PromptTiming
        self.timing = PromptTiming()            # arm() it and call enqueue() eagerly for per-unit milliseconds of a pass

    # ---- products ---------------------------------------------------------------------------------------------
    def _q8(self, X: torch.Tensor):
        """E4M3 codes and 1 x 128 scales of the bf16 rows X (one launch), in buffers of X's own."""
        key = ("q8", X.data_ptr(), X.shape[0], X.shape[1])
        buf = self._scratch_w.get(key)
        if buf is None:
            dev = self.e.device
            buf = self._scratch_w[key] = (torch.zeros(X.shape[0], X.shape[1], dtype=torch.uint8, device=dev),
                                          torch.zeros(X.shape[0], X.shape[1] // 128, dtype=torch.float32, device=dev))
        G.fp8_rows(X, buf[0], buf[1])
        return buf

    def _native_fp8(self, Wq) -> bool:
        return self.fp8_native and Wq.qtype == "FP8_B128" and Wq.k % 128 == 0

    def _mm(self, X, Wq, tiles, M, x8=None, W2=None, **kw):
        """X [rows, K] bf16 times a resident matrix (or, with W2, the SwiGLU pair): FP8 weights against E4M3 rows on the
        tensor cores, other quantised types expanded in flight, the rest through a bf16 expansion launch.  ``x8``: the
        rows' E4M3 form when the caller already made it (several products of one input).  Returns the launch count."""
        if self._native_fp8(Wq):
            n = 0
            if x8 is None:
                x8 = self._q8(X); n += 1
            if tiles.tile_rows != 32:                            # the dense table of a 64-row bucket
                tiles = self._dense32(M)
            G.fp8_gemm(x8[0], x8[1], Wq, tiles, W2=W2, status=self.status, **kw)
            return n + 1
        if G.qgemm_supports(Wq):
            G.qgemm(X, Wq, tiles, W2=W2, status=self.status, **kw)
            return 1
        if Wq.qtype == "BF16":
            # bf16 rows need no expansion: the bf16 GEMM reads them in place (token tiles of 128 rows)
            if tiles.tile_rows != 128:
                tiles = self._dense128(M)
            G.gemm_bf16(X, Wq.data.view(torch.bfloat16), tiles, B2=W2.data.view(torch.bfloat16) if W2 is not None else None,
                        status=self.status, **kw)
            return 1
        assert W2 is None, "the SwiGLU pair needs a type with a quantised-weight kernel"
        name = f"{Wq.rows}x{Wq.k}"
        wb = self._scratch_w.get(name)
        if wb is None:
            wb = self._scratch_w[name] = torch.empty(Wq.rows, Wq.k, dtype=torch.bfloat16, device=self.e.device)
        G.dequant_bf16(Wq, wb)
        G.gemm_bf16(X, wb, self._dense128(M), status=self.status, **kw)
        return 2

    def _dense128(self, M: int):
        t = self._scratch_w.get(("t", M))
        if t is None:
            t = self._scratch_w[("t", M)] = G.TileTable.dense(M, self.e.device)
        return t

    def _dense32(self, M: int):
        t = self._scratch_w.get(("t32", M))
        if t is None:
            t = self._scratch_w[("t32", M)] = G.TileTable.dense(M, self.e.device, TILE)
        return t

    def enqueue(self, M: int, advance: bool = False) -> int:
        """Enqueue one pass of the first M row cells on the current stream; returns the launch count."""
        n = 0
        for n in self.enqueue_steps(M, advance):
            pass
        return n

    def embed(self, M: int, x: torch.Tensor) -> None:
        e = self.e
        K.embed_rows(self.tokens, M, e.w.q["token_embd.weight"], e.spec.vocab, x, e.fault)

    def _check_types(self) -> None:
        """Refuse at construction what the pass has no kernel for (the caller then keeps the 8-row chain)."""
        s, w = self.e.spec, self.e.w
        for il in range(s.n_layer):
            b = f"blk.{il}."
            if s.layer_is_moe(il):
                pairs = [("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight")]
                if s.n_shared:
                    pairs.append(("ffn_gate_shexp.weight", "ffn_up_shexp.weight", None))
            else:
                pairs = [("ffn_gate.weight", "ffn_up.weight", None)]
            for g_, u_, d_ in pairs:
                qg, qu = w.q[b + g_], w.q[b + u_]
                ok = lambda q_: G.qgemm_supports(q_) or q_.qtype == "BF16"          # noqa: E731
                if d_ is not None and (w.q[b + d_].qtype == "BF16") != (qg.qtype == "BF16"):
                    raise NotImplementedError(f"{b}{d_}: expert stacks mix bf16 with block types")
                if not (ok(qg) and qg.qtype == qu.qtype and (d_ is None or ok(w.q[b + d_]))):
                    raise NotImplementedError(f"{b}{g_}: type {qg.qtype}/{qu.qtype} has no kernel in the batched pass")

    def shared_expert(self, il: int, M: int, xn: torch.Tensor, tiles, out: torch.Tensor, resid: torch.Tensor) -> int:
        """out = resid + the shared expert of layer il over the normed rows (a dense SwiGLU pair)."""
        w = self.e.w
        b = f"blk.{il}."
        qg, qu = w.q[b + "ffn_gate_shexp.weight"], w.q[b + "ffn_up_shexp.weight"]
        n = self._mm(xn, qg, tiles, M, W2=qu, out_bf16=self.sh_act[:M])
        return n + self._mm(self.sh_act[:M], w.q[b + "ffn_down_shexp.weight"], tiles, M, out_f32=out, resid=resid)

    def dense_ffn(self, il: int, M: int, x: torch.Tensor, xn: torch.Tensor, tiles):
        """Dense SwiGLU FFN of layer il; a generator like :meth:`experts`."""
        w = self.e.w
        b = f"blk.{il}."
        n = self._mm(xn, w.q[b + "ffn_gate.weight"], tiles, M, W2=w.q[b + "ffn_up.weight"], out_bf16=self.dact[:M])
        yield n + self._mm(self.dact[:M], w.q[b + "ffn_down.weight"], tiles, M, out_f32=x, resid=x)

    def experts(self, il: int, M: int, x: torch.Tensor, xn: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, tiles):
        """Routed experts (and the shared one) of layer il on the routed rows; a generator of launch counts (it yields
        where ranks of a several-GPU pass must meet; here it never does)."""
        e = self.e
        s, w = e.spec, e.w
        b = f"blk.{il}."
        E, k = s.n_expert, s.n_used
        mark = self.timing.mark
        n = 0
        G.moe_plan(ids, wts, E, self.moe_tiles, self.pos_of, self.dst_row, self.row_scale); n += 1
        G.gather_rows_bf16(xn, self.dst_row, self.moe_tiles.offsets[E:E + 1], self.cap, k, self.Ap); n += 1
        mark(il, "route_plan_gather")
        qg, qu, qd = (w.q[b + f"ffn_{nm}_exps.weight"] for nm in ("gate", "up", "down"))
        n += self._mm(self.Ap, qg, self.moe_tiles, M, W2=qu, out_bf16=self.act)
        mark(il, "gate_up")
        n += self._mm(self.act, qd, self.moe_tiles, M, out_f32=self.slot_out, dst_row=self.dst_row, row_scale=self.row_scale)
        mark(il, "down")
        G.moe_combine(self.slot_out, self.pos_of, M, k, x, x); n += 1
        if s.n_shared:
            n += self.shared_expert(il, M, xn, tiles, x, x)
            mark(il, "shared_expert")
        yield n

    def _attn_gqa(self, il: int, M: int, xn: torch.Tensor, tiles) -> int:
        """Grouped-query attention of layer il up to the attention rows (fp32, before the o product)."""
        e = self.e
        s, w = e.spec, e.w
        b = f"blk.{il}."
        q_scale = 1.0 / math.sqrt(s.head_dim)
        n = 0
        # the three projections are small grids (32 + 4 + 4 weight tiles on the 30 B shape): K and V run on side
        # streams beside Q (parallel branches of the captured graph)
        main = torch.cuda.current_stream(e.device)
        x8 = None
        if any(self._native_fp8(w.q[b + nm]) for nm in ("attn_q.weight", "attn_k.weight", "attn_v.weight")):
            x8 = self._q8(xn); n += 1                            # one E4M3 form of the rows for the three products
        fork = torch.cuda.Event()
        fork.record(main)
        joins = []
        for side, name, lo, hi in ((self._side[0], "attn_k.weight", s.q_rows, s.q_rows + s.kv_rows),
                                   (self._side[1], "attn_v.weight", s.q_rows + s.kv_rows, s.q_rows + 2 * s.kv_rows)):
            side.wait_event(fork)
            with torch.cuda.stream(side):
                n += self._mm(xn, w.q[b + name], tiles, M, x8=x8, out_f32=self.qkv[:M, lo:hi])
                ev = torch.cuda.Event()
                ev.record(side)
                joins.append(ev)
        n += self._mm(xn, w.q[b + "attn_q.weight"], tiles, M, x8=x8, out_f32=self.qkv[:M, :s.q_rows])
        for ev in joins:
            main.wait_event(ev)
        kvp = e.kv
        self.timing.mark(il, "qkv")
        K.qk_norm_rope_append(self.qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"), e.inv_freq,
                              s.rms_eps, q_scale, s.head_dim, s.n_q, s.n_kv, M, self.row_pos, self.row_seq, kvp.table,
                              kvp.n_pages, kvp.k[il], kvp.v[il], self.q_out, e.fault, il, kv_q8=e.kv_q8); n += 1
        K.flash_decode(self.q_out, kvp.k[il], kvp.v[il], self.row_pos, self.row_seq, kvp.table, kvp.n_pages, s.head_dim,
                       s.n_q, s.n_kv, M, self.n_seg, e.slot_ctx, self.part_ml, self.part_acc, self.attn, self.attn_q,
                       self.attn_ds, e.fault, il, kv_q8=e.kv_q8); n += 2
        return n

    def _attn_mla(self, il: int, M: int, xn: torch.Tensor, tiles) -> int:
        """Latent attention of layer il (the 8-row chain's steps, ``DecodeEngine._attn_mla``, with the products on the
        tensor cores): q_a and kv_a products side by side, latent append, q_b product, absorb, latent flash decode with
        the value up-projection."""
        e = self.e
        s, w, kvp = e.spec, e.w, e.kv
        b = f"blk.{il}."
        n = 0
        main = torch.cuda.current_stream(e.device)
        first = w.q[b + "attn_q_a.weight"] if s.q_lora else w.q[b + "attn_q.weight"]
        x8 = None
        if self._native_fp8(first) or self._native_fp8(w.q[b + "attn_kv_a_mqa.weight"]):
            x8 = self._q8(xn); n += 1                            # one E4M3 form of the rows for both products
        fork = torch.cuda.Event()
        fork.record(main)
        side = self._side[0]
        side.wait_event(fork)
        with torch.cuda.stream(side):
            n += self._mm(xn, w.q[b + "attn_kv_a_mqa.weight"], tiles, M, x8=x8, out_f32=self.qkv[:M, self.qa_w:])
            K.mla_kv_append(self.qkv[:, self.qa_w:], w.f[b + "attn_kv_a_norm.weight"], e.inv_freq, s.rms_eps, M, self.row_pos,
                            self.row_seq, kvp.table, kvp.n_pages, kvp.k[il], e.fault, il); n += 1
            join = torch.cuda.Event()
            join.record(side)
        n += self._mm(xn, first, tiles, M, x8=x8, out_f32=self.qkv[:M, :self.qa_w])
        if s.q_lora:
            G.rmsnorm_bf16(self.qkv[:M, :s.q_lora], w.f[b + "attn_q_a_norm.weight"], s.rms_eps, self.qn[:M]); n += 1
            n += self._mm(self.qn[:M], w.q[b + "attn_q_b.weight"], tiles, M, out_f32=self.q_full[:M])
            q = self.q_full
        else:
            q = self.qkv[:, :self.qa_w]
        K.mla_q_absorb(q, w.f[b + "attn_k_b.weight"], e.inv_freq, e.attn_scale, s.n_q, s.nope_dim, M, self.row_pos,
                       self.row_seq, self.q_out); n += 1
        main.wait_event(join)
        self.timing.mark(il, "qkv")
        K.mla_flash_decode(self.q_out, kvp.k[il], self.row_pos, self.row_seq, kvp.table, kvp.n_pages, s.n_q, M, self.n_seg,
                           e.slot_ctx, self.part_ml, self.part_acc, w.f[b + "attn_v_b.weight"], s.v_dim, self.attn,
                           self.attn_q, self.attn_ds, e.fault, il); n += 2
        return n

    def enqueue_steps(self, M: int, advance: bool = False):
        """The pass as a generator: it yields its running launch count wherever the ranks of a several-GPU pass have to
        meet (never, on one GPU), so a test can walk several emulated ranks in lockstep on one stream."""
        e = self.e
        s, w = e.spec, e.w
        tiles = self.dense_tiles[M]
        x, xn = self.x[:M], self.xn[:M]
        n = 0
        self.embed(M, x); n += 1
        for il in range(s.n_layer):
            b = f"blk.{il}."
            mark = self.timing.mark
            mark(il, "ffn_tail")
            G.rmsnorm_bf16(x, w.f[b + "attn_norm.weight"], s.rms_eps, xn); n += 1
            mark(il, "norm")
            if s.mla:
                n += self._attn_mla(il, M, xn, tiles)
            else:
                n += self._attn_gqa(il, M, xn, tiles)
            G.rmsnorm_bf16(self.attn[:M], None, s.rms_eps, self.attn_bf[:M]); n += 1
            mark(il, "attention")
            n += self._mm(self.attn_bf[:M], w.q[b + "attn_output.weight"], tiles, M, out_f32=x, resid=x)
            mark(il, "o_proj")
            if s.layer_is_moe(il):
                E, k = s.n_expert, s.n_used
                K.router(x, w.f[b + "ffn_norm.weight"], s.rms_eps, w.q[b + "ffn_gate_inp.weight"], M, self.logits_r, None,
                         None, None, e.fault, il); n += 1
                K.route_rows(self.logits_r, e._rule(il), M, self.ids, self.wts, e.heat[il], e.fault, il); n += 1
                G.rmsnorm_bf16(x, w.f[b + "ffn_norm.weight"], s.rms_eps, xn); n += 1
                steps = self.experts(il, M, x, xn, self.ids[:M], self.wts[:M], tiles)
            else:
                G.rmsnorm_bf16(x, w.f[b + "ffn_norm.weight"], s.rms_eps, xn); n += 1
                steps = self.dense_ffn(il, M, x, xn, tiles)
            for got in steps:
                if got is None:
                    yield n                          # the ranks meet here
                else:
                    n += got
        G.rmsnorm_bf16(x, w.f["output_norm.weight"], s.rms_eps, xn); n += 1
        head_w = w.q.get("output.weight", w.q["token_embd.weight"])
        n += self._mm(xn, head_w, tiles, M, out_f32=self.logits[:M])
        K.argmax_rows(self.logits, s.vocab, M, self.am_blocks, self.am_v, self.am_i, self.counters[1:2], self.tokens_out,
                      None, e.fault); n += 1
        if advance:
            K.advance_rows(self.tokens, self.row_pos, self.row_seq, self.tokens_out, M, self.hist, self.hist_cap,
                           self.counters[2:3]); n += 1
        yield n

    # ---- driving ----------------------------------------------------------------------------------------------
    @staticmethod
    def bucket(m: int) -> int:
        for b in BUCKETS:
            if m <= b:
                return b
        raise ValueError(f"{m} rows in one pass")

    def _graph(self, M: int, advance: bool) -> torch.cuda.CUDAGraph:
        g = self.graphs.get((M, advance))
        if g is None:
            with torch.cuda.stream(self._stream):
                self.enqueue(M, advance)                 # warm-up: attribute calls, scratch allocation
                self._stream.synchronize()
                if advance:                              # undo the warm-up's advance
                    self.params.copy_(self.params_host, non_blocking=True)
                    self.counters[2:3].zero_()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self._stream):
                    self.launches_per_step = self.enqueue(M, advance)
            self.graphs[(M, advance)] = g
        return g

    def set_rows(self, rows: Sequence[Tuple[int, int, int]]) -> int:
        """rows: (slot, token, position); pads the bucket with dead rows (slot -1).  Returns the bucket size."""
        m = len(rows)
        M = self.bucket(m)
        e = self.e
        h = self.params_host
        h[0].zero_(); h[1].zero_(); h[2].fill_(-1)
        for i, (slot, tok, pos) in enumerate(rows):
            e.kv.ensure(slot, pos + 1)
            e.kv.own(slot, pos)
            h[0, i], h[1, i], h[2, i] = tok, pos, slot
            e.slot_len[slot] = max(e.slot_len[slot], pos + 1)
        e.kv.sync_table()
        with torch.cuda.stream(self._stream):
            self.params.copy_(h, non_blocking=True)
        return M

    def launch(self, M: int, advance: bool = False) -> None:
        g = self._graph(M, advance)
        with torch.cuda.stream(self._stream):
            g.replay()

    def prefill(self, slot: int, tokens: Sequence[int], start: int = 0) -> int:
        """Feed a prompt through passes of up to ``max_rows`` consecutive positions of one sequence (every row attends
        to the rows before it in the same pass); returns the greedy token after the last one.  The several-GPU form of
        the pass has no other prompt path for models whose 8-row chain cannot run on a rank's share of the weights."""
        last = -1
        for i in range(0, len(tokens), self.R):
            chunk = tokens[i:i + self.R]
            last = self.step([(slot, int(t), start + i + j) for j, t in enumerate(chunk)])[len(chunk) - 1]
        return last

    def step(self, rows: Sequence[Tuple[int, int, int]]) -> List[int]:
        """One pass: the arg-max token of every row."""
        M = self.set_rows(rows)
        self.launch(M)
        with torch.cuda.stream(self._stream):
            self.tokens_out_host.copy_(self.tokens_out, non_blocking=True)
        self._stream.synchronize()
        if int(self.status.item()) != 0:
            raise RuntimeError("a bounded wait inside the GEMM kernel ran out (status word set)")
        self.e.check_fault()
        return self.tokens_out_host[:len(rows)].tolist()
