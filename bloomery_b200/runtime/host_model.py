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


def covers(spec) -> bool:
    """Whether the native step serves this model: GQA attention, softmax routing without groups, every layer routed, no
    shared expert."""
    return (not spec.mla and spec.is_moe and spec.first_dense == 0 and not spec.n_shared and spec.router_mode == "softmax"
            and spec.n_group <= 1 and spec.hidden % 256 == 0 and spec.moe_inter % 256 == 0 and spec.head_dim % 2 == 0)


class HostDecoder:
    def __init__(self, weights, ctx: int = 4096):
        s = self.spec = weights.spec
        if not covers(s):
            raise NotImplementedError(f"{s.arch}: the native host step covers GQA models whose layers are all routed")
        if str(weights.device) != "cpu":
            raise ValueError("the host decoder reads weights in host memory")
        self.w = weights                          # keeps every tensor the C++ side points into alive
        self.ctx = ctx
        self.n_past = 0
        lib = self.lib = host()
        lib.blh_model_create.restype = ctypes.c_void_p
        from ..models.rope import inv_freq_table
        self._inv = inv_freq_table(s, s.head_dim).float().contiguous()
        self.h = lib.blh_model_create(I(s.n_layer), I(s.hidden), I(s.n_q), I(s.n_kv), I(s.head_dim), I(s.vocab), I(s.n_expert),
                                      I(s.n_used), I(s.moe_inter), I(ctx), F(s.rms_eps), I(1 if s.router_renorm else 0),
                                      F(s.router_scale), P(self._inv.data_ptr()))
        if not self.h:
            raise ValueError("the host decoder refused this shape")
        q, f = weights.q, weights.f
        embd = q["token_embd.weight"]
        out = q.get("output.weight", embd)
        lib.blh_model_set_io(P(self.h), self._p(embd), I(embd.wt), self._p(out), I(out.wt), P(f["output_norm.weight"].data_ptr()))
        for il in range(s.n_layer):
            b = f"blk.{il}."
            router = q[b + "ffn_gate_inp.weight"]
            if router.qtype != "F32":
                raise NotImplementedError("the host router reads f32 rows")
            g, u, d = q[b + "ffn_gate_exps.weight"], q[b + "ffn_up_exps.weight"], q[b + "ffn_down_exps.weight"]
            if g.qtype != u.qtype:
                raise NotImplementedError("gate and up stacks of different types")
            qn, kn = f.get(b + "attn_q_norm.weight"), f.get(b + "attn_k_norm.weight")
            mats = [q[b + n] for n in ("attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight")]
            args = []
            for m in mats:
                args += [self._p(m), I(m.wt)]
            lib.blh_model_set_layer(P(self.h), I(il), *args, P(f[b + "attn_norm.weight"].data_ptr()),
                                    P(qn.data_ptr() if qn is not None else 0), P(kn.data_ptr() if kn is not None else 0),
                                    P(f[b + "ffn_norm.weight"].data_ptr()), self._p(router), self._p(g), self._p(u), self._p(d),
                                    I(g.wt), I(d.wt))
        self._logits = torch.zeros(s.vocab, dtype=torch.float32)

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
        k = torch.empty(s.n_layer, n, s.n_kv * s.head_dim, dtype=torch.float32)
        v = torch.empty_like(k)
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
