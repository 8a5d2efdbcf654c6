"""Plain PyTorch fp32 restatement of the decode chain: the oracle of every GPU test and
the engine behind the CPU-only path.

The reference has no CPU Qwen3 trunk (its host seat runs ``deepseek2`` only:
``crates/gpu-gates/src/bin/bloomery_serve.rs:46``), so this follows the documented kernel
math of the card path instead: q8 activations at the integer-dot sites, RMSNorm with an
f64 sum, NEOX RoPE, f16 K/V, softmax router with ties to the smaller id, slots combined
in ascending order.  ``quantize_acts=False`` gives the exact fp32 model for band checks.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from ..formats.quant import dequantize_act_q8, quantize_act_q8
from .spec import ModelSpec
from .weights import Weights


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    ss = (x.double() ** 2).mean(-1, keepdim=True)
    scale = (1.0 / torch.sqrt(ss + eps)).float()
    return x * scale * gain


def rope_neox(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x [T, heads, D]; pairs (i, i + D/2)."""
    half = x.shape[-1] // 2
    ang = pos.float()[:, None] * inv_freq[None, :]          # [T, D/2] in fp32 like the card
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], -1)


def rope_pairs(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x [T, ..., D]; interleaved pairs (2i, 2i + 1), the DeepSeek convention."""
    ang = pos.float()[:, None] * inv_freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [x.shape[-1] // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], -1).reshape(x.shape)


def route(logits: torch.Tensor, spec: ModelSpec, bias: Optional[torch.Tensor] = None):
    """[T, E] -> (ids [T, k], weights [T, k]) with the device's tie rule (smaller id wins)."""
    if spec.router_mode == "softmax":
        probs = torch.softmax(logits.float(), -1)
        choice = probs
    else:
        probs = torch.sigmoid(logits.float())
        choice = probs + (bias if bias is not None else 0.0)
    T, E = logits.shape
    if spec.n_group > 1:
        g = choice.reshape(T, spec.n_group, E // spec.n_group)
        gs = g.topk(2, -1).values.sum(-1)
        keep = torch.zeros_like(gs, dtype=torch.bool)
        keep.scatter_(1, gs.topk(spec.topk_group, -1).indices, True)
        choice = torch.where(keep[:, :, None].expand_as(g), g, torch.full_like(g, -float("inf"))).reshape(T, E)
    # stable sort descending => ties resolved to the smaller id
    order = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :spec.n_used]
    w = torch.gather(probs, 1, order)
    if spec.router_renorm:
        w = w / w.double().sum(-1, keepdim=True).float()
    return order.to(torch.int32), w * spec.router_scale


class CpuModel:
    def __init__(self, weights: Weights, quantize_acts: bool = True, device="cpu"):
        self.spec = weights.spec
        self.device = torch.device(device)
        self.qa = quantize_acts
        self.w: Dict[str, torch.Tensor] = {}
        for n in list(weights.q) + list(weights.f):
            self.w[n] = weights.dequant(n).to(self.device)
        s = self.spec
        from .rope import attn_scale, inv_freq_table
        self.inv_freq = inv_freq_table(s, s.rope_dim if s.mla else s.head_dim).to(self.device)
        self.scale = attn_scale(s)
        self.reset()

    def reset(self):
        s = self.spec
        kd = (1, s.kv_lora + s.rope_dim) if s.mla else (s.n_kv, s.head_dim)
        self.k: List[torch.Tensor] = [torch.zeros(0, *kd, device=self.device) for _ in range(s.n_layer + s.n_mtp)]
        self.v: List[torch.Tensor] = [torch.zeros(0, *kd, device=self.device) for _ in range(s.n_layer + s.n_mtp)]
        self.hidden: Optional[torch.Tensor] = None      # the trunk's final hidden rows of the last forward
        self.n_past = 0

    def _q(self, x: torch.Tensor) -> torch.Tensor:
        if not self.qa:
            return x
        c, ds = quantize_act_q8(x)
        return dequantize_act_q8(c, ds)


    def _gqa(self, il: int, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        s, w = self.spec, self.w
        b = f"blk.{il}."
        T = h.shape[0]
        q = (h @ w[b + "attn_q.weight"].T).reshape(T, s.n_q, s.head_dim)
        k = (h @ w[b + "attn_k.weight"].T).reshape(T, s.n_kv, s.head_dim)
        v = (h @ w[b + "attn_v.weight"].T).reshape(T, s.n_kv, s.head_dim)
        if s.qk_norm:
            q = rms_norm(q, w[b + "attn_q_norm.weight"], s.rms_eps)
            k = rms_norm(k, w[b + "attn_k_norm.weight"], s.rms_eps)
        q = rope_neox(q, pos, self.inv_freq)
        k = rope_neox(k, pos, self.inv_freq)
        k = k.half().float()
        v = v.half().float()
        self.k[il] = torch.cat([self.k[il], k], 0)
        self.v[il] = torch.cat([self.v[il], v], 0)
        G = s.n_q // s.n_kv
        kk = self.k[il].repeat_interleave(G, 1)      # [S, n_q, D]
        vv = self.v[il].repeat_interleave(G, 1)
        S = kk.shape[0]
        sc = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(s.head_dim)
        mask = torch.arange(S, device=self.device)[None, :] > pos[:, None]
        sc = sc.masked_fill(mask[None], -float("inf"))
        pr = torch.softmax(sc, -1)
        att = torch.einsum("hts,shd->thd", pr, vv).reshape(T, s.q_rows)
        return att

    def _mla(self, il: int, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """Multi-head latent attention in its plain (un-absorbed) form: keys and values are rebuilt per head
        from the cached latent, scores add the shared rotary part."""
        s, w = self.spec, self.w
        b = f"blk.{il}."
        T = h.shape[0]
        qk = s.nope_dim + s.rope_dim
        if s.q_lora:
            qa = h @ w[b + "attn_q_a.weight"].T
            q = self._q(rms_norm(qa, w[b + "attn_q_a_norm.weight"], s.rms_eps)) @ w[b + "attn_q_b.weight"].T
        else:
            q = h @ w[b + "attn_q.weight"].T
        q = q.reshape(T, s.n_q, qk)
        q_nope, q_rope = q[..., :s.nope_dim], rope_pairs(q[..., s.nope_dim:], pos, self.inv_freq)
        kva = h @ w[b + "attn_kv_a_mqa.weight"].T
        c = rms_norm(kva[:, :s.kv_lora], w[b + "attn_kv_a_norm.weight"], s.rms_eps)
        kr = rope_pairs(kva[:, s.kv_lora:], pos, self.inv_freq)
        row = torch.cat([c, kr], -1).half().float()[:, None, :]
        self.k[il] = torch.cat([self.k[il], row], 0)
        lat, krope = self.k[il][:, 0, :s.kv_lora], self.k[il][:, 0, s.kv_lora:]
        S = lat.shape[0]
        k_nope = torch.einsum("hnc,sc->shn", w[b + "attn_k_b.weight"], lat)
        v = torch.einsum("hvc,sc->shv", w[b + "attn_v_b.weight"], lat)
        sc = (torch.einsum("thn,shn->hts", q_nope, k_nope) + torch.einsum("thr,sr->hts", q_rope, krope)) * self.scale
        mask = torch.arange(S, device=self.device)[None, :] > pos[:, None]
        pr = torch.softmax(sc.masked_fill(mask[None], -float("inf")), -1)
        return torch.einsum("hts,shv->thv", pr, v).reshape(T, s.n_q * s.v_dim)

    def _layer(self, il: int, x: torch.Tensor, pos: torch.Tensor, collect: Optional[dict] = None) -> torch.Tensor:
        s, w = self.spec, self.w
        T = x.shape[0]
        b = f"blk.{il}."
        h = self._q(rms_norm(x, w[b + "attn_norm.weight"], s.rms_eps))
        att = self._mla(il, h, pos) if s.mla else self._gqa(il, h, pos)
        x = x + self._q(att) @ w[b + "attn_output.weight"].T
        hn = rms_norm(x, w[b + "ffn_norm.weight"], s.rms_eps)
        if s.layer_is_moe(il):
            logits = hn @ w[b + "ffn_gate_inp.weight"].T
            ids, wts = route(logits, s, w.get(b + "exp_probs_b.bias"))
            if collect is not None:
                collect.setdefault("ids", []).append(ids)
                collect.setdefault("wts", []).append(wts)
            hq = self._q(hn)
            y = torch.zeros_like(x)
            for t in range(T):
                acc = torch.zeros(s.hidden, device=self.device)
                for j in range(s.n_used):
                    e = int(ids[t, j])
                    g = hq[t] @ w[b + "ffn_gate_exps.weight"][e].T
                    u = hq[t] @ w[b + "ffn_up_exps.weight"][e].T
                    a = self._q((torch.nn.functional.silu(g) * u)[None])[0]
                    acc = acc + wts[t, j] * (a @ w[b + "ffn_down_exps.weight"][e].T)
                y[t] = acc
            if s.n_shared:
                g = hq @ w[b + "ffn_gate_shexp.weight"].T
                u = hq @ w[b + "ffn_up_shexp.weight"].T
                y = y + self._q(torch.nn.functional.silu(g) * u) @ w[b + "ffn_down_shexp.weight"].T
            x = x + y
        else:
            hq = self._q(hn)
            g = hq @ w[b + "ffn_gate.weight"].T
            u = hq @ w[b + "ffn_up.weight"].T
            a = self._q(torch.nn.functional.silu(g) * u)
            x = x + a @ w[b + "ffn_down.weight"].T
        if collect is not None:
            collect.setdefault("x", []).append(x.clone())
        return x

    @torch.no_grad()
    def mtp_forward(self, next_tokens: torch.Tensor, hidden: torch.Tensor, pos: torch.Tensor, il: Optional[int] = None) -> torch.Tensor:
        """Logits of the multi-token-prediction layer: row i combines the trunk's hidden state at ``pos[i]`` with
        the embedding of the token that follows it and predicts the token after that; the layer keeps its own
        KV rows at those positions (DeepSeek-V3's MTP module; the reference: ``crates/runtime/src/mtp``)."""
        s, w = self.spec, self.w
        il = s.n_layer if il is None else il
        b = f"blk.{il}."
        e = rms_norm(w["token_embd.weight"][next_tokens.long()], w[b + "nextn.enorm.weight"], s.rms_eps)
        hh = rms_norm(hidden, w[b + "nextn.hnorm.weight"], s.rms_eps)
        z = torch.cat([self._q(e), self._q(hh)], -1)          # each half is quantised on its own
        x = z @ w[b + "nextn.eh_proj.weight"].T
        if self.k[il].shape[0] > int(pos[0]):
            self.k[il], self.v[il] = self.k[il][:int(pos[0])], self.v[il][:int(pos[0])]
        x = self._layer(il, x, pos)
        hn = self._q(rms_norm(x, w[b + "nextn.shared_head_norm.weight"], s.rms_eps))
        head = w.get("output.weight", w["token_embd.weight"])
        return hn @ head.T

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, collect: Optional[dict] = None) -> torch.Tensor:
        """tokens [T] appended to the sequence; returns logits [T, vocab]."""
        s, w = self.spec, self.w
        T = tokens.shape[0]
        pos = torch.arange(self.n_past, self.n_past + T, device=self.device)
        x = w["token_embd.weight"][tokens.long()]
        for il in range(s.n_layer):
            x = self._layer(il, x, pos, collect)
        self.hidden = x
        self.n_past += T
        h = self._q(rms_norm(x, w["output_norm.weight"], s.rms_eps))
        head = w.get("output.weight", w["token_embd.weight"])
        return h @ head.T

    @torch.no_grad()
    def generate(self, prompt: List[int], n_new: int) -> List[int]:
        """Greedy continuation with the engine's tie rule (lower id wins)."""
        logits = self.forward(torch.tensor(prompt, device=self.device))
        out = []
        tok = int(greedy_pick(logits[-1]))
        out.append(tok)
        for _ in range(n_new - 1):
            logits = self.forward(torch.tensor([tok], device=self.device))
            tok = int(greedy_pick(logits[-1]))
            out.append(tok)
        return out


def greedy_pick(row: torch.Tensor) -> int:
    """Strictly greater wins; equal wins at the lower id; NaN never wins; all-NaN row -> 0."""
    r = torch.where(torch.isnan(row), torch.full_like(row, -float("inf")), row)
    mx = r.max()
    if mx == -float("inf") and torch.isnan(row).all():
        return 0
    return int(torch.nonzero(r == mx)[0, 0])
