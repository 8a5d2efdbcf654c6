"""Batched decode on the tensor cores: one pass of up to 64 rows (one token of 64 different sequences).

The 8-row decode chain reads every weight byte once per pass with int8 dot products; that is the right shape up to a
handful of rows.  Past that the matrix products move to tcgen05 with the weights still block-quantised in HBM
(``csrc/qgemm_tcgen05.cu``): the rows are the N side of the MMA in tiles of 32, every weight block is read and
expanded once per pass whatever the row count, and a pass over a routed-expert layer touches each chosen expert once
for all the rows routed to it.  Per layer:

  RMSNorm -> bf16 rows, Q / K / V products, per-head norm + RoPE + KV append, split-K flash decode over the paged
  cache (every row its own sequence and position), o product with the residual, router logits + top-k, expert-sorted
  plan (count / offsets / 32-row tiles / scatter in one launch), gather, gate+up with SwiGLU in the epilogue, down
  with the router weight in the epilogue, slot-ordered combine.

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
    """Rows beyond the 8-row chain of a :class:`DecodeEngine` (GQA attention + routed experts or dense FFN)."""

    def __init__(self, engine, max_rows: int = 64):
        e = self.e = engine
        s = e.spec
        if s.mla or s.n_shared or e.lo != 0 or e.hi != s.n_layer:
            raise NotImplementedError("the batched tensor-core pass serves GQA attention with routed or dense FFN layers")
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
        self.qkv = torch.zeros(R, s.q_rows + 2 * s.kv_rows, **f32)
        self.q_out = torch.zeros(R, s.n_q, s.head_dim, **f32)
        sm = K.sm_count(dev)
        # key segments: enough blocks to fill the card at the smallest bucket, no more
        self.n_seg = max(1, min(e.n_seg, (2 * sm) // (s.n_kv * BUCKETS[0]) + 1))
        self.part_ml = torch.zeros(R * s.n_q * self.n_seg * 2, **f32)
        self.part_acc = torch.zeros(R * s.n_q * self.n_seg * s.head_dim, **f32)
        self.attn = torch.zeros(R, s.q_rows, **f32)
        self.attn_bf = torch.zeros(R, s.q_rows, **bf)
        self.attn_q = torch.zeros(R, s.q_rows, dtype=torch.int8, device=dev)
        self.attn_ds = torch.zeros(R, s.q_rows // 32, 2, **f32)
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
            self.moe_tiles = G.TileTable(n, E, dev, TILE)
        if s.dense_inter and (s.first_dense > 0 or not s.is_moe):
            self.dact = torch.zeros(R, s.dense_inter, **bf)
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
        # the engine's own stream: its 8-row passes and prompts and these passes touch the same KV pages in order
        self._stream = getattr(engine, "_stream", None) or torch.cuda.Stream(device=dev)
        self._side = [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)]
        from .timing import PromptTiming
        self.timing = PromptTiming()            # arm() it and call enqueue() eagerly for per-unit milliseconds of a pass

    # ---- products ---------------------------------------------------------------------------------------------
    def _mm(self, X, Wq, tiles, M, **kw):
        """X [M, K] bf16 times a resident matrix: quantised in flight when the type has a kernel, else through a bf16
        expansion (float and the rarer block types)."""
        if G.qgemm_supports(Wq):
            G.qgemm(X, Wq, tiles, status=self.status, **kw)
            return 1
        name = f"{Wq.rows}x{Wq.k}"
        wb = self._scratch_w.get(name)
        if wb is None:
            wb = self._scratch_w[name] = torch.empty(Wq.rows, Wq.k, dtype=torch.bfloat16, device=self.e.device)
        G.dequant_bf16(Wq, wb)
        dt = self._scratch_w.get(("t", M))
        if dt is None:
            dt = self._scratch_w[("t", M)] = G.TileTable.dense(M, self.e.device)
        G.gemm_bf16(X, wb, dt, status=self.status, **kw)
        return 2

    def enqueue(self, M: int, advance: bool = False) -> int:
        """Enqueue one pass of the first M row cells on the current stream; returns the launch count."""
        n = 0
        for n in self.enqueue_steps(M, advance):
            pass
        return n

    def embed(self, M: int, x: torch.Tensor) -> None:
        e = self.e
        K.embed_rows(self.tokens, M, e.w.q["token_embd.weight"], e.spec.vocab, x, e.fault)

    def experts(self, il: int, M: int, x: torch.Tensor, xn: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor):
        """Routed experts of layer il on the routed rows; a generator of launch counts (it yields where ranks of a
        several-GPU pass must meet; here it never does)."""
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
        if not (G.qgemm_supports(qg) and qg.qtype == qu.qtype and G.qgemm_supports(qd)):
            raise NotImplementedError(f"expert stacks of type {qg.qtype}/{qu.qtype}/{qd.qtype} in the batched pass")
        G.qgemm(self.Ap, qg, self.moe_tiles, out_bf16=self.act, W2=qu, status=self.status); n += 1
        mark(il, "gate_up")
        G.qgemm(self.act, qd, self.moe_tiles, out_f32=self.slot_out, dst_row=self.dst_row, row_scale=self.row_scale,
                status=self.status); n += 1
        mark(il, "down")
        G.moe_combine(self.slot_out, self.pos_of, M, k, x, x); n += 1
        yield n

    def enqueue_steps(self, M: int, advance: bool = False):
        """The pass as a generator: it yields its running launch count wherever the ranks of a several-GPU pass have to
        meet (never, on one GPU), so a test can walk several emulated ranks in lockstep on one stream."""
        e = self.e
        s, w = e.spec, e.w
        tiles = self.dense_tiles[M]
        x, xn = self.x[:M], self.xn[:M]
        n = 0
        self.embed(M, x); n += 1
        q_scale = 1.0 / math.sqrt(s.head_dim)
        for il in range(s.n_layer):
            b = f"blk.{il}."
            mark = self.timing.mark
            mark(il, "ffn_tail")
            G.rmsnorm_bf16(x, w.f[b + "attn_norm.weight"], s.rms_eps, xn); n += 1
            mark(il, "norm")
            # the three projections are small grids (32 + 4 + 4 weight tiles on the 30 B shape): K and V run on side
            # streams beside Q (parallel branches of the captured graph)
            main = torch.cuda.current_stream(e.device)
            fork = torch.cuda.Event()
            fork.record(main)
            joins = []
            for side, name, lo, hi in ((self._side[0], "attn_k.weight", s.q_rows, s.q_rows + s.kv_rows),
                                       (self._side[1], "attn_v.weight", s.q_rows + s.kv_rows, s.q_rows + 2 * s.kv_rows)):
                side.wait_event(fork)
                with torch.cuda.stream(side):
                    n += self._mm(xn, w.q[b + name], tiles, M, out_f32=self.qkv[:M, lo:hi])
                    ev = torch.cuda.Event()
                    ev.record(side)
                    joins.append(ev)
            n += self._mm(xn, w.q[b + "attn_q.weight"], tiles, M, out_f32=self.qkv[:M, :s.q_rows])
            for ev in joins:
                main.wait_event(ev)
            kvp = e.kv
            mark(il, "qkv")
            K.qk_norm_rope_append(self.qkv, w.f.get(b + "attn_q_norm.weight"), w.f.get(b + "attn_k_norm.weight"), e.inv_freq,
                                  s.rms_eps, q_scale, s.head_dim, s.n_q, s.n_kv, M, self.row_pos, self.row_seq, kvp.table,
                                  kvp.n_pages, kvp.k[il], kvp.v[il], self.q_out, e.fault, il, kv_q8=e.kv_q8); n += 1
            K.flash_decode(self.q_out, kvp.k[il], kvp.v[il], self.row_pos, self.row_seq, kvp.table, kvp.n_pages, s.head_dim,
                           s.n_q, s.n_kv, M, self.n_seg, e.slot_ctx, self.part_ml, self.part_acc, self.attn, self.attn_q,
                           self.attn_ds, e.fault, il, kv_q8=e.kv_q8); n += 2
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
                for got in self.experts(il, M, x, xn, self.ids[:M], self.wts[:M]):
                    if got is None:
                        yield n                      # the ranks meet here
                    else:
                        n += got
            else:
                G.rmsnorm_bf16(x, w.f[b + "ffn_norm.weight"], s.rms_eps, xn); n += 1
                qg, qu = w.q[b + "ffn_gate.weight"], w.q[b + "ffn_up.weight"]
                if not (G.qgemm_supports(qg) and qg.qtype == qu.qtype):
                    raise NotImplementedError(f"dense FFN of type {qg.qtype}/{qu.qtype} in the batched pass")
                G.qgemm(xn, qg, tiles, out_bf16=self.dact[:M], W2=qu, status=self.status); n += 1
                n += self._mm(self.dact[:M], w.q[b + "ffn_down.weight"], tiles, M, out_f32=x, resid=x)
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
