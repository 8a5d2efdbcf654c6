"""The native host decoder: a whole decode step of a grouped-query mixture-of-experts model in one C++ call
(``csrc/host/model_cpu.cpp``), over the resident quantised rows of a :class:`Weights` that lives in host memory.

``models/cpu_ref.py`` stays the oracle (plain PyTorch on dequantised weights); this class is what the CPU engine decodes
with where the model is one it covers: the same q8 activation sites, the same f16-rounded K/V, the same router rule, so
its logits follow the oracle's to the order of fp32 sums.  One decoder holds one sequence's cache.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops._lib import host
from ..ops.decode import QWeight

I, F, P = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


MAT = {n: i for i, n in enumerate(("q", "k", "v", "o", "q_a", "q_b", "kv_a", "gate", "up", "down", "sh_gate", "sh_up", "sh_down"))}
VEC = {n: i for i, n in enumerate(("attn_norm", "q_norm", "k_norm", "ffn_norm", "router", "router_bias", "q_a_norm", "kv_a_norm",
                                   "k_b", "v_b"))}


def covers(spec) -> bool:
    """Whether the native step serves this model: grouped-query or latent attention, routed layers (softmax, or sigmoid
    with bias and groups) with or without a shared expert, leading dense layers; widths the quantised row dots take."""
    if spec.hidden % 256 or getattr(spec, "n_mtp", 0) and False:
        return False
    if spec.is_moe and (spec.moe_inter % 256 or spec.n_expert % max(1, spec.n_group)):
        return False
    if spec.n_shared and spec.shared_inter % 32:
        return False
    if (spec.first_dense or not spec.is_moe) and (not spec.dense_inter or spec.dense_inter % 32):
        return False
    if spec.mla:
        return spec.kv_lora % 32 == 0 and spec.rope_dim % 2 == 0 and (spec.n_q * spec.v_dim) % 64 == 0 and (not spec.q_lora or spec.q_lora % 256 == 0)
    return spec.head_dim % 2 == 0 and (spec.n_q * spec.head_dim) % 64 == 0


class HostDecoder:
    def __init__(self, weights, ctx: int = 4096):
        s = self.spec = weights.spec
        if not covers(s):
            raise NotImplementedError(f"{s.arch}: the native host step does not cover this shape")
        if str(weights.device) != "cpu":
            raise ValueError("the host decoder reads weights in host memory")
        self.w = weights                          # keeps every tensor the C++ side points into alive
        self._keep: List[torch.Tensor] = []       # float copies made for it (latent attention's per-head matrices)
        self.ctx = ctx
        self.n_past = 0
        lib = self.lib = host()
        lib.blh_model_create.restype = ctypes.c_void_p
        from ..models.rope import attn_scale, inv_freq_table
        self._inv = inv_freq_table(s, s.rope_dim if s.mla else s.head_dim).float().contiguous()
        self.h = lib.blh_model_create(I(s.n_layer), I(s.hidden), I(s.n_q), I(max(1, s.n_kv)), I(s.head_dim), I(s.vocab),
                                      I(s.n_expert if s.is_moe else 0), I(s.n_used if s.is_moe else 0), I(s.moe_inter if s.is_moe else 0),
                                      I(ctx), F(s.rms_eps), I(1 if s.router_renorm else 0), F(s.router_scale),
                                      P(self._inv.data_ptr()), I(self._inv.numel()))
        if not self.h:
            raise ValueError("the host decoder refused this shape")
        rc = lib.blh_model_set_arch(P(self.h), I(1 if s.mla else 0), I(s.q_lora or 0), I(s.kv_lora or 0), I(s.rope_dim or 0),
                                    I(s.nope_dim or 0), I(s.v_dim or 0), F(attn_scale(s)), I(s.first_dense if s.is_moe else s.n_layer),
                                    I(s.dense_inter or 0), I(s.shared_inter if s.n_shared else 0),
                                    I(0 if s.router_mode == "softmax" else 1), I(max(1, s.n_group)), I(max(1, s.topk_group)))
        if rc != 0:
            self.close()
            raise NotImplementedError("the host decoder refused this layer plan")
        q, f = weights.q, weights.f
        embd = q["token_embd.weight"]
        out = q.get("output.weight", embd)
        lib.blh_model_set_io(P(self.h), self._p(embd), I(embd.wt), self._p(out), I(out.wt), P(f["output_norm.weight"].data_ptr()))

        def mat(il, slot, name):
            m = q[f"blk.{il}.{name}"]
            if lib.blh_model_set_mat(P(self.h), I(il), I(MAT[slot]), self._p(m), I(m.wt), I(m.rows), I(m.k)) != 0:
                raise NotImplementedError(f"blk.{il}.{name}: rows of type {m.qtype} and width {m.k} have no host dot")

        def vec(il, slot, t):
            if t is None:
                return
            if t.dtype != torch.float32 or not t.is_contiguous():
                t = t.float().contiguous()
                self._keep.append(t)
            lib.blh_model_set_vec(P(self.h), I(il), I(VEC[slot]), P(t.data_ptr()))
        for il in range(s.n_layer):
            b = f"blk.{il}."
            vec(il, "attn_norm", f[b + "attn_norm.weight"])
            vec(il, "ffn_norm", f[b + "ffn_norm.weight"])
            mat(il, "o", "attn_output.weight")
            if s.mla:
                if s.q_lora:
                    mat(il, "q_a", "attn_q_a.weight"); mat(il, "q_b", "attn_q_b.weight")
                    vec(il, "q_a_norm", f[b + "attn_q_a_norm.weight"])
                else:
                    mat(il, "q", "attn_q.weight")
                mat(il, "kv_a", "attn_kv_a_mqa.weight")
                vec(il, "kv_a_norm", f[b + "attn_kv_a_norm.weight"])
                vec(il, "k_b", f[b + "attn_k_b.weight"]); vec(il, "v_b", f[b + "attn_v_b.weight"])
            else:
                mat(il, "q", "attn_q.weight"); mat(il, "k", "attn_k.weight"); mat(il, "v", "attn_v.weight")
                vec(il, "q_norm", f.get(b + "attn_q_norm.weight")); vec(il, "k_norm", f.get(b + "attn_k_norm.weight"))
            if s.layer_is_moe(il):
                router = q[b + "ffn_gate_inp.weight"]
                if router.qtype != "F32":
                    raise NotImplementedError("the host router reads f32 rows")
                lib.blh_model_set_vec(P(self.h), I(il), I(VEC["router"]), self._p(router))
                vec(il, "router_bias", f.get(b + "exp_probs_b.bias"))
                g, u, d = q[b + "ffn_gate_exps.weight"], q[b + "ffn_up_exps.weight"], q[b + "ffn_down_exps.weight"]
                if g.qtype != u.qtype:
                    raise NotImplementedError("gate and up stacks of different types")
                lib.blh_model_set_experts(P(self.h), I(il), self._p(g), self._p(u), self._p(d), I(g.wt), I(d.wt))
                if s.n_shared:
                    mat(il, "sh_gate", "ffn_gate_shexp.weight"); mat(il, "sh_up", "ffn_up_shexp.weight")
                    mat(il, "sh_down", "ffn_down_shexp.weight")
            else:
                mat(il, "gate", "ffn_gate.weight"); mat(il, "up", "ffn_up.weight"); mat(il, "down", "ffn_down.weight")
        self._logits = torch.zeros(s.vocab, dtype=torch.float32)
        self._kw = (s.kv_lora + s.rope_dim) if s.mla else s.n_kv * s.head_dim
        self._vw = 0 if s.mla else self._kw

    @staticmethod
    def _p(w: QWeight) -> ctypes.c_void_p:
        assert w.data.is_contiguous()
        return P(w.data.data_ptr())

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.blh_model_destroy(P(self.h))
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:      # noqa: BLE001 - interpreter shutdown
            pass

    def reset(self) -> None:
        self.n_past = 0

    def cut(self, n: int) -> None:
        self.n_past = min(self.n_past, n)

    def kv(self, n: Optional[int] = None):
        """(k, v) of the first ``n`` positions (default: all kept), each [layer, n, n_kv * head] fp32."""
        s = self.spec
        n = self.n_past if n is None else min(n, self.n_past)
        k = torch.empty(s.n_layer, n, self._kw, dtype=torch.float32)
        v = torch.empty(s.n_layer, n, self._vw, dtype=torch.float32)
        if self.lib.blh_model_kv_get(P(self.h), I(n), P(k.data_ptr()), P(v.data_ptr())) != 0:
            raise RuntimeError("blh_model_kv_get refused the span")
        return k, v

    def load_kv(self, k: torch.Tensor, v: torch.Tensor, n: Optional[int] = None) -> int:
        """Take the first ``n`` positions of a saved (k, v) as this sequence's cache; returns the positions now kept."""
        n = k.shape[1] if n is None else min(n, k.shape[1])
        if n > self.ctx:
            raise ValueError(f"{n} positions do not fit the decoder's context of {self.ctx}")
        k, v = k[:, :n].contiguous().float(), v[:, :n].contiguous().float()
        if self.lib.blh_model_kv_set(P(self.h), I(n), P(k.data_ptr()), P(v.data_ptr())) != 0:
            raise RuntimeError("blh_model_kv_set refused the span")
        self.n_past = n
        return n

    def step(self, token: int, want_logits: bool = True) -> Optional[torch.Tensor]:
        """Evaluate ``token`` at the next position; the logits row after it (a view reused by the next call)."""
        if self.n_past >= self.ctx:
            raise ValueError(f"position {self.n_past} is beyond the decoder's context of {self.ctx}")
        rc = self.lib.blh_model_step(P(self.h), I(int(token)), I(self.n_past), P(self._logits.data_ptr() if want_logits else 0))
        if rc != 0:
            raise RuntimeError(f"blh_model_step failed with {rc}")
        self.n_past += 1
        return self._logits if want_logits else None

    def forward(self, tokens: Sequence[int]) -> torch.Tensor:
        """Logits of every position of ``tokens`` (the oracle's call shape)."""
        rows = [self.step(int(t)).clone() for t in tokens]
        return torch.stack(rows) if rows else torch.zeros(0, self.spec.vocab)

    def generate(self, prompt: Sequence[int], n_new: int) -> List[int]:
        from ..models.cpu_ref import greedy_pick
        for t in prompt[:-1]:
            self.step(int(t), want_logits=False)
        tok = greedy_pick(self.step(int(prompt[-1])))
        out = [tok]
        for _ in range(n_new - 1):
            tok = greedy_pick(self.step(tok))
            out.append(tok)
        return out
