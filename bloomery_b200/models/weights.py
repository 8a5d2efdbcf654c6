"""Weight sets: synthetic fixtures, GGUF loading, GGUF writing.

* :func:`synth_tensors` yields seeded random tensors of a :class:`ModelSpec` already
  quantised with the llama.cpp ``Q4_K_M`` type mix (attention V and FFN down in Q6_K on
  the "more bits" layers, output head Q6_K, router and norms F32).  It runs on any
  device, so the 30 B-parameter benchmark model is generated and quantised on the card.
  This is the fixture tier of the reference (``crates/model/src/fixture/mod.rs:1-60``:
  tiny synthetic files that keep every per-layer shape and type).
* :func:`load_gguf` streams a GGUF file (or split) through a pinned staging ring into
  resident layouts, one final synchronise (the reference's upload ring,
  ``crates/gpu/src/upload.rs:1-8``).
* :func:`write_gguf` writes any tensor stream as a GGUF v3 file.
"""
from __future__ import annotations

import math
from typing import Dict, Iterator, Optional, Tuple

import torch

from ..formats import quant
from ..formats.gguf import Gguf, GgufWriter
from ..formats.resident import FLOAT_TYPES, INT_DOT_TYPES, UnsupportedType, to_resident
from ..ops.decode import QWeight
from .spec import ModelSpec

TensorItem = Tuple[str, Tuple[int, ...], str, torch.Tensor]  # name, shape (row-major), qtype, raw bytes [rows, row_bytes]


def use_more_bits(i: int, n: int) -> bool:
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


def q4_k_m_type(name: str, il: int, n_layer: int) -> str:
    """Type that llama.cpp's Q4_K_M recipe gives a tensor (norms and router stay F32)."""
    if name.endswith("_norm.weight") or name.endswith("ffn_gate_inp.weight") or name.endswith(".bias"):
        return "F32"
    if name == "output.weight":
        return "Q6_K"
    if name.endswith("attn_v.weight") or name.endswith("ffn_down_exps.weight") or name.endswith("ffn_down.weight"):
        return "Q6_K" if use_more_bits(il, n_layer) else "Q4_K"
    return "Q4_K"


def _rand(shape, std, gen, device):
    return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std


def synth_tensors(spec: ModelSpec, device="cpu", seed: int = 0, mix: str = "Q4_K_M", std: float = 0.02,
                  with_vocab: bool = False) -> Iterator[TensorItem]:
    """Seeded N(0, std) weights of ``spec``, quantised per ``mix`` ("Q4_K_M", "Q8_0", "F16", ...)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    H, L = spec.hidden, spec.n_layer

    def qt(name: str, il: int) -> str:
        if mix == "Q4_K_M":
            return q4_k_m_type(name, il, L)
        t = q4_k_m_type(name, il, L)
        return "F32" if t == "F32" else mix

    def emit(name: str, shape, il: int = 0, std_=std, ones: bool = False) -> TensorItem:
        t = qt(name, il)
        if ones:
            w = torch.ones(*shape, device=device) + _rand(shape, 0.02, gen, device)
        else:
            w = _rand(shape, std_, gen, device)
        raw = quant.quantize(w.reshape(-1, shape[-1]), t)
        return (name, tuple(shape), t, raw)

    yield emit("token_embd.weight", (spec.vocab, H))
    for il in range(L):
        b = f"blk.{il}."
        yield emit(b + "attn_norm.weight", (H,), il, ones=True)
        yield emit(b + "attn_q.weight", (spec.q_rows, H), il)
        yield emit(b + "attn_k.weight", (spec.kv_rows, H), il)
        yield emit(b + "attn_v.weight", (spec.kv_rows, H), il)
        if spec.qk_norm:
            yield emit(b + "attn_q_norm.weight", (spec.head_dim,), il, ones=True)
            yield emit(b + "attn_k_norm.weight", (spec.head_dim,), il, ones=True)
        yield emit(b + "attn_output.weight", (H, spec.q_rows), il)
        yield emit(b + "ffn_norm.weight", (H,), il, ones=True)
        if spec.layer_is_moe(il):
            yield emit(b + "ffn_gate_inp.weight", (spec.n_expert, H), il)
            yield emit(b + "ffn_gate_exps.weight", (spec.n_expert, spec.moe_inter, H), il)
            yield emit(b + "ffn_up_exps.weight", (spec.n_expert, spec.moe_inter, H), il)
            yield emit(b + "ffn_down_exps.weight", (spec.n_expert, H, spec.moe_inter), il)
        else:
            yield emit(b + "ffn_gate.weight", (spec.dense_inter, H), il)
            yield emit(b + "ffn_up.weight", (spec.dense_inter, H), il)
            yield emit(b + "ffn_down.weight", (H, spec.dense_inter), il)
    yield emit("output_norm.weight", (H,), 0, ones=True)
    yield emit("output.weight", (spec.vocab, H))


def spec_metadata(spec: ModelSpec) -> Dict[str, object]:
    a = spec.arch
    md: Dict[str, object] = {
        "general.name": spec.name or a,
        f"{a}.block_count": spec.n_layer,
        f"{a}.context_length": spec.ctx_train,
        f"{a}.embedding_length": spec.hidden,
        f"{a}.feed_forward_length": spec.dense_inter or spec.moe_inter,
        f"{a}.attention.head_count": spec.n_q,
        f"{a}.attention.head_count_kv": spec.n_kv,
        f"{a}.attention.key_length": spec.head_dim,
        f"{a}.attention.value_length": spec.head_dim,
        f"{a}.attention.layer_norm_rms_epsilon": float(spec.rms_eps),
        f"{a}.rope.freq_base": float(spec.rope_theta),
        f"{a}.vocab_size": spec.vocab,
    }
    if spec.is_moe:
        md[f"{a}.expert_count"] = spec.n_expert
        md[f"{a}.expert_used_count"] = spec.n_used
        md[f"{a}.expert_feed_forward_length"] = spec.moe_inter
    return md


def write_gguf(spec: ModelSpec, items: Iterator[TensorItem], path: str, extra_meta: Optional[Dict[str, object]] = None):
    w = GgufWriter(spec.arch)
    for k, v in spec_metadata(spec).items():
        w.set(k, v)
    for k, v in (extra_meta or {}).items():
        w.set(k, v)
    for name, shape, qtype, raw in items:
        w.add(name, shape, qtype, raw)
    w.write(path)


class Weights:
    """Resident tensors of one model on one device."""

    def __init__(self, spec: ModelSpec, device):
        self.spec = spec
        self.device = torch.device(device)
        self.q: Dict[str, QWeight] = {}
        self.f: Dict[str, torch.Tensor] = {}
        self.n_bytes = 0

    def add(self, name: str, shape: Tuple[int, ...], qtype: str, raw: torch.Tensor) -> None:
        k = shape[-1]
        raw = raw.to(self.device, non_blocking=True)
        if len(shape) == 1:
            if qtype != "F32":
                raise UnsupportedType(f"{name}: 1-D tensor of type {qtype}")
            t = raw.reshape(-1).view(torch.float32).clone()
            self.f[name] = t
            self.n_bytes += t.numel() * 4
            return
        if qtype not in INT_DOT_TYPES and qtype not in FLOAT_TYPES:
            raise UnsupportedType(f"{name}: block type {qtype} has no kernel in this build")
        res = to_resident(raw.reshape(-1, raw.shape[-1]), qtype, k)
        if len(shape) == 3:
            res = res.reshape(shape[0], shape[1], -1)
        self.q[name] = QWeight(res, qtype, k)
        self.n_bytes += res.numel()

    @classmethod
    def from_items(cls, spec: ModelSpec, items: Iterator[TensorItem], device) -> "Weights":
        w = cls(spec, device)
        for name, shape, qtype, raw in items:
            w.add(name, shape, qtype, raw)
        return w

    def dequant(self, name: str) -> torch.Tensor:
        """fp32 copy of a weight (oracle use)."""
        from ..formats.resident import from_resident
        if name in self.f:
            return self.f[name].float()
        qw = self.q[name]
        flat = qw.data.reshape(-1, qw.data.shape[-1])
        raw = from_resident(flat, qw.qtype, qw.k)
        out = quant.dequantize(raw, qw.qtype, qw.k)
        return out.reshape(*qw.data.shape[:-1], qw.k)


def load_gguf(path: str, device, ring_bytes: int = 256 << 20) -> Tuple[ModelSpec, Weights, Gguf]:
    """Open a GGUF model and upload it through a pinned two-slot ring with one final sync."""
    g = Gguf.open(path)
    spec = ModelSpec.from_gguf(g)
    w = Weights(spec, device)
    dev = torch.device(device)
    use_ring = dev.type == "cuda"
    ring = [torch.empty(ring_bytes, dtype=torch.uint8, pin_memory=True) for _ in range(2)] if use_ring else None
    events = [None, None]
    slot = 0
    for name, info in g.tensors.items():
        rows = g.tensor_rows(name)
        shape = info.shape
        if not use_ring:
            w.add(name, shape, info.qtype.name, rows.clone())
            continue
        n = rows.numel()
        if n > ring_bytes:
            # larger than a ring slot: stage in row chunks
            rb = rows.shape[1]
            per = max(1, ring_bytes // rb)
            parts = []
            for r0 in range(0, rows.shape[0], per):
                chunk = rows[r0:r0 + per]
                if events[slot] is not None:
                    events[slot].synchronize()
                stage = ring[slot][:chunk.numel()].view(chunk.shape)
                stage.copy_(chunk)
                parts.append(stage.to(dev, non_blocking=True))
                events[slot] = torch.cuda.Event()
                events[slot].record()
                slot ^= 1
            w.add(name, shape, info.qtype.name, torch.cat(parts, 0))
        else:
            if events[slot] is not None:
                events[slot].synchronize()
            stage = ring[slot][:n].view(rows.shape)
            stage.copy_(rows)
            dev_t = stage.to(dev, non_blocking=True)
            events[slot] = torch.cuda.Event()
            events[slot].record()
            slot ^= 1
            w.add(name, shape, info.qtype.name, dev_t)
    if use_ring:
        torch.cuda.synchronize(dev)
    return spec, w, g
