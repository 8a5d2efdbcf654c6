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
from ..formats.resident import (FLOAT_TYPES, INT_DOT_TYPES, PLANE_TYPES, UnsupportedType, quantize_resident, resident_type,
                                to_resident)
from ..ops.decode import QWeight
from .spec import ModelSpec

TensorItem = Tuple[str, Tuple[int, ...], str, torch.Tensor]  # name, shape (row-major), qtype, raw bytes [rows, row_bytes]


def use_more_bits(i: int, n: int) -> bool:
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


def q4_k_m_type(name: str, il: int, n_layer: int) -> str:
    """Type that llama.cpp's Q4_K_M recipe gives a tensor (norms and router stay F32)."""
    if name.endswith("_norm.weight") or name.endswith("ffn_gate_inp.weight") or name.endswith(".bias") \
            or name.endswith("nextn.enorm.weight") or name.endswith("nextn.hnorm.weight"):
        return "F32"
    if name == "output.weight":
        return "Q6_K"
    if name.endswith("attn_v.weight") or name.endswith("ffn_down_exps.weight") or name.endswith("ffn_down.weight") or name.endswith("ffn_down_shexp.weight"):
        return "Q6_K" if use_more_bits(il, n_layer) else "Q4_K"
    return "Q4_K"


def _rand(shape, std, gen, device):
    return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std


def shard_shape(name: str, shape, spec: ModelSpec, rank: int, world: int, attn: bool = True):
    """Shape of rank ``rank``'s share of a tensor under the head / expert / width split of the sharded engines
    (``parallel/sharded.py`` ``shard_items``), and whether the tensor is split at all.  ``attn`` off leaves the
    attention matrices whole (the replicated-attention engine)."""
    shape = tuple(shape)
    if not attn and name.endswith(("attn_q.weight", "attn_q_b.weight", "attn_k.weight", "attn_v.weight", "attn_k_b.weight",
                                   "attn_v_b.weight", "attn_output.weight")):
        return shape, False
    rows_split = ("attn_q.weight", "attn_q_b.weight", "ffn_gate.weight", "ffn_up.weight", "ffn_gate_shexp.weight",
                  "ffn_up_shexp.weight")
    cols_split = ("attn_output.weight", "ffn_down.weight", "ffn_down_shexp.weight")
    if name.endswith(rows_split):
        return (shape[0] // world,) + shape[1:], True
    if name.endswith(("attn_k.weight", "attn_v.weight")):
        return ((shape[0] // world if spec.n_kv >= world else spec.head_dim),) + shape[1:], True
    if name.endswith(("attn_k_b.weight", "attn_v_b.weight")) or "_exps.weight" in name:
        return (shape[0] // world,) + shape[1:], True
    if name.endswith(cols_split):
        return shape[:-1] + (shape[-1] // world,), True
    return shape, False


def synth_tensors(spec: ModelSpec, device="cpu", seed: int = 0, mix: str = "Q4_K_M", std: float = 0.02,
                  with_vocab: bool = False, shard: Optional[Tuple[int, int]] = None, shard_attn: bool = True) -> Iterator[TensorItem]:
    """Seeded N(0, std) weights of ``spec``, quantised per ``mix`` ("Q4_K_M", "Q8_0", "F16", ...).

    ``shard`` = (rank, world): only that rank's share of every split tensor is generated, in the local shape the
    sharded engines load (a model that fits no single card is never built whole); every tensor is then seeded by its
    name, so replicated tensors are equal on all ranks and split ones differ from rank to rank."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    H, L = spec.hidden, spec.n_layer
    if shard is not None:
        import zlib
        full_gen = gen

        class _PerTensor:
            def reseed(self, name: str, split: bool) -> None:
                full_gen.manual_seed((zlib.crc32(name.encode()) ^ (seed * 2654435761) ^ ((shard[0] + 1) * 7919 if split else 0)) & 0x7FFFFFFF)
        per_tensor = _PerTensor()

    def qt(name: str, il: int) -> str:
        if mix == "Q4_K_M":
            return q4_k_m_type(name, il, L)
        t = q4_k_m_type(name, il, L)
        return "F32" if t == "F32" else mix

    def emit(name: str, shape, il: int = 0, std_=std, ones: bool = False) -> TensorItem:
        t = qt(name, il)
        if shard is not None:
            shape, split = shard_shape(name, shape, spec, shard[0], shard[1], shard_attn)
            per_tensor.reseed(name, split)
        if ones:
            w = torch.ones(*shape, device=device) + _rand(shape, 0.02, gen, device)
        else:
            w = _rand(shape, std_, gen, device)
        if t in PLANE_TYPES:                      # block-scaled float types travel as resident rows
            return (name, tuple(shape), t, quantize_resident(w.reshape(-1, shape[-1]), t, values=False)[0])
        raw = quant.quantize(w.reshape(-1, shape[-1]), t)
        return (name, tuple(shape), t, raw)

    yield emit("token_embd.weight", (spec.vocab, H))
    for il in range(L + spec.n_mtp):
        b = f"blk.{il}."
        if il >= L:        # a multi-token-prediction layer: a trunk block behind its own input projection
            yield emit(b + "nextn.enorm.weight", (H,), il, ones=True)
            yield emit(b + "nextn.hnorm.weight", (H,), il, ones=True)
            yield emit(b + "nextn.eh_proj.weight", (H, 2 * H), il)
            yield emit(b + "nextn.shared_head_norm.weight", (H,), il, ones=True)
        yield emit(b + "attn_norm.weight", (H,), il, ones=True)
        if spec.mla:
            qk = spec.nope_dim + spec.rope_dim
            if spec.q_lora:
                yield emit(b + "attn_q_a.weight", (spec.q_lora, H), il)
                yield emit(b + "attn_q_a_norm.weight", (spec.q_lora,), il, ones=True)
                yield emit(b + "attn_q_b.weight", (spec.n_q * qk, spec.q_lora), il, std_=0.05)
            else:
                yield emit(b + "attn_q.weight", (spec.n_q * qk, H), il)
            yield emit(b + "attn_kv_a_mqa.weight", (spec.kv_lora + spec.rope_dim, H), il, std_=0.05)
            yield emit(b + "attn_kv_a_norm.weight", (spec.kv_lora,), il, ones=True)
            # the per-head products keep float weights: [head][nope][latent] and [head][v][latent]
            nh = spec.n_q
            if shard is not None:
                nh = spec.n_q // shard[1] if shard_attn else spec.n_q
                per_tensor.reseed(b + "attn_k_b.weight", shard_attn)
            yield (b + "attn_k_b.weight", (nh, spec.nope_dim, spec.kv_lora), "F32",
                   _rand((nh * spec.nope_dim, spec.kv_lora), 0.05, gen, device).view(torch.uint8))
            if shard is not None:
                per_tensor.reseed(b + "attn_v_b.weight", shard_attn)
            yield (b + "attn_v_b.weight", (nh, spec.v_dim, spec.kv_lora), "F32",
                   _rand((nh * spec.v_dim, spec.kv_lora), 0.05, gen, device).view(torch.uint8))
            yield emit(b + "attn_output.weight", (H, spec.n_q * spec.v_dim), il)
        else:
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
            if spec.router_mode == "sigmoid":
                if shard is not None:
                    per_tensor.reseed(b + "exp_probs_b.bias", False)
                yield (b + "exp_probs_b.bias", (spec.n_expert,), "F32",
                       _rand((1, spec.n_expert), 0.05, gen, device).view(torch.uint8))
            if spec.n_shared:
                yield emit(b + "ffn_gate_shexp.weight", (spec.shared_inter, H), il)
                yield emit(b + "ffn_up_shexp.weight", (spec.shared_inter, H), il)
                yield emit(b + "ffn_down_shexp.weight", (H, spec.shared_inter), il)
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
    if spec.mla:
        md.update({f"{a}.attention.q_lora_rank": spec.q_lora, f"{a}.attention.kv_lora_rank": spec.kv_lora,
                   f"{a}.rope.dimension_count": spec.rope_dim, f"{a}.attention.key_length": spec.nope_dim + spec.rope_dim,
                   f"{a}.attention.value_length": spec.v_dim, f"{a}.leading_dense_block_count": spec.first_dense,
                   f"{a}.feed_forward_length": spec.dense_inter, f"{a}.expert_shared_count": spec.n_shared,
                   f"{a}.expert_gating_func": 2 if spec.router_mode == "sigmoid" else 1,
                   f"{a}.expert_weights_norm": bool(spec.router_renorm), f"{a}.expert_weights_scale": float(spec.router_scale),
                   f"{a}.expert_group_count": spec.n_group, f"{a}.expert_group_used_count": spec.topk_group,
                   f"{a}.nextn_predict_layers": spec.n_mtp})
        if spec.rope_yarn_factor > 1.0:
            md.update({f"{a}.rope.scaling.type": "yarn", f"{a}.rope.scaling.factor": float(spec.rope_yarn_factor),
                       f"{a}.rope.scaling.original_context_length": spec.rope_yarn_orig_ctx,
                       f"{a}.rope.scaling.yarn_log_multiplier": float(spec.rope_mscale_all_dim) * 0.1})
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
        if name.endswith(("attn_k_b.weight", "attn_v_b.weight", "attn_kv_b.weight")):
            self._add_mla_heads(name, shape, qtype, raw)
            return
        if resident_type(qtype) not in INT_DOT_TYPES and qtype not in FLOAT_TYPES:
            raise UnsupportedType(f"{name}: block type {qtype} has no kernel in this build")
        flat = raw.reshape(-1, raw.shape[-1])
        res = flat.contiguous() if qtype in PLANE_TYPES else to_resident(flat, qtype, k)
        if len(shape) == 3:
            res = res.reshape(shape[0], shape[1], -1)
        self.q[name] = QWeight(res, resident_type(qtype), k)
        self.n_bytes += res.numel()

    def _add_mla_heads(self, name: str, shape, qtype: str, raw: torch.Tensor) -> None:
        """The per-head MLA products run on float weights laid out [head][nope][latent] / [head][v][latent]:
        bf16 stays bf16, anything else is decoded to f32 (exact).  Accepts the split GGUF tensors
        (``attn_k_b`` stored [head][latent][nope], ``attn_v_b`` [head][v][latent]) and the joint checkpoint
        matrix ``attn_kv_b`` [head * (nope + v), latent]."""
        s = self.spec
        k = shape[-1]
        flat = raw.reshape(-1, raw.shape[-1])
        if qtype == "BF16":
            w = flat.view(torch.bfloat16)
        elif qtype == "F32":
            w = flat.view(torch.float32)
        elif qtype == "F16":
            w = flat.view(torch.float16).float()
        elif qtype in PLANE_TYPES:
            from ..formats.planes import resident_dequantize
            w = resident_dequantize(flat, qtype, k)
        else:
            w = quant.dequantize(flat, qtype, k)
        stem = name[:-len(name.split(".")[-2]) - len(".weight")]
        if name.endswith("attn_kv_b.weight"):
            w = w.reshape(s.n_q, s.nope_dim + s.v_dim, s.kv_lora)
            parts = {"attn_k_b.weight": w[:, :s.nope_dim], "attn_v_b.weight": w[:, s.nope_dim:]}
        elif name.endswith("attn_k_b.weight"):
            if k == s.kv_lora:
                parts = {"attn_k_b.weight": w.reshape(s.n_q, s.nope_dim, s.kv_lora)}
            else:                       # the GGUF order [head][latent][nope]
                parts = {"attn_k_b.weight": w.reshape(s.n_q, s.kv_lora, s.nope_dim).transpose(1, 2)}
        else:
            parts = {"attn_v_b.weight": w.reshape(s.n_q, s.v_dim, s.kv_lora)}
        for leaf, t in parts.items():
            t = t.contiguous().clone()
            self.f[stem + leaf] = t
            self.n_bytes += t.numel() * t.element_size()

    @classmethod
    def from_items(cls, spec: ModelSpec, items: Iterator[TensorItem], device) -> "Weights":
        w = cls(spec, device)
        for name, shape, qtype, raw in items:
            w.add(name, shape, qtype, raw)
        return w

    def to(self, device) -> "Weights":
        """The same resident tensors on another device (plain copies: nothing is re-laid or re-quantised)."""
        w = Weights(self.spec, device)
        for name, qw in self.q.items():
            w.q[name] = QWeight(qw.data.to(w.device, non_blocking=True), qw.qtype, qw.k)
        for name, t in self.f.items():
            w.f[name] = t.to(w.device, non_blocking=True)
        w.n_bytes = self.n_bytes
        return w

    def dequant(self, name: str) -> torch.Tensor:
        """fp32 copy of a weight (oracle use)."""
        from ..formats.resident import from_resident
        if name in self.f:
            return self.f[name].float()
        qw = self.q[name]
        flat = qw.data.reshape(-1, qw.data.shape[-1])
        if qw.qtype in PLANE_TYPES:
            from ..formats.planes import resident_dequantize
            return resident_dequantize(flat, qw.qtype, qw.k).reshape(*qw.data.shape[:-1], qw.k)
        if qw.qtype == "Q8_F32":
            from ..formats.resident import decode_q8_f32
            return decode_q8_f32(flat, qw.k).reshape(*qw.data.shape[:-1], qw.k)
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
    # how warm the file is, then the kernel's read-ahead for a front-to-back pass over it (both best effort: a file
    # system or platform that refuses leaves the load as it was)
    from ..utils import osshim
    g.page_cache = None
    try:
        seen = [osshim.populated(sh.map) for sh in g.shards]
        g.page_cache = round(sum(p_.resident for p_ in seen) / max(1, sum(p_.pages for p_ in seen)), 4)
        for sh in g.shards:
            osshim.advise(sh.map, "sequential")
    except OSError:
        pass
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


# ------------------------------------------------------------------------------------
# Checkpoint folders (safetensors + config.json)
# ------------------------------------------------------------------------------------
_HF_LAYER = {
    "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
    "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
    "self_attn.o_proj": "attn_output", "self_attn.q_norm.weight": "attn_q_norm.weight",
    "self_attn.k_norm.weight": "attn_k_norm.weight",
    "self_attn.q_a_proj": "attn_q_a", "self_attn.q_a_layernorm.weight": "attn_q_a_norm.weight",
    "self_attn.q_b_proj": "attn_q_b", "self_attn.kv_a_proj_with_mqa": "attn_kv_a_mqa",
    "self_attn.kv_a_layernorm.weight": "attn_kv_a_norm.weight", "self_attn.kv_b_proj": "attn_kv_b",
    "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down",
    "mlp.shared_experts.gate_proj": "ffn_gate_shexp", "mlp.shared_experts.up_proj": "ffn_up_shexp",
    "mlp.shared_experts.down_proj": "ffn_down_shexp",
    "mlp.gate.weight": "ffn_gate_inp.weight", "mlp.gate.e_score_correction_bias": "exp_probs_b.bias",
}
_HF_TOP = {"model.embed_tokens": "token_embd", "model.norm.weight": "output_norm.weight", "lm_head": "output"}


def folder_items(folder, spec: ModelSpec) -> Iterator[TensorItem]:
    """Tensors of a checkpoint folder under the GGUF names, quantised layers as resident rows.

    Per-expert matrices are stacked into ``ffn_{gate,up,down}_exps``; norms, the router and its
    selection bias become F32 (the reference reads folders through the same part names:
    ``crates/gpu/src/folder.rs``, ``crates/hf/src/modelopt.rs``)."""
    from ..formats import planes
    scheme = planes.detect_scheme(folder.config)

    def f32_item(src: str, dst: str) -> TensorItem:
        t = folder.tensor(src).float().contiguous()
        shape = tuple(t.shape)
        return (dst, shape, "F32", t.reshape(-1, shape[-1]).view(torch.uint8))

    def linear(stem: str, dst: str) -> TensorItem:
        res, ty, k = planes.linear_resident(folder, stem, scheme)
        return (dst + ".weight", (res.shape[0], k), ty, res)

    yield linear("model.embed_tokens", "token_embd")
    for il in range(spec.n_layer + spec.n_mtp):
        hp, b = f"model.layers.{il}.", f"blk.{il}."
        for src, dst in _HF_LAYER.items():
            if src.endswith(".weight") or src.endswith("_bias"):
                if hp + src in folder:
                    yield f32_item(hp + src, b + dst)
            elif any((hp + src + sfx) in folder for sfx in (".weight", ".weight_packed")):
                yield linear(hp + src, b + dst)
        if (hp + "mlp.experts.0.gate_proj.weight") in folder or (hp + "mlp.experts.0.gate_proj.weight_packed") in folder:
            for proj, dst in (("gate_proj", "ffn_gate_exps"), ("up_proj", "ffn_up_exps"), ("down_proj", "ffn_down_exps")):
                parts, ty, k = [], None, 0
                for e in range(spec.n_expert):
                    res, t1, k = planes.linear_resident(folder, f"{hp}mlp.experts.{e}.{proj}", scheme)
                    if ty not in (None, t1):
                        raise UnsupportedType(f"{hp}{proj}: experts of mixed types {ty} / {t1}")
                    ty = t1
                    parts.append(res)
                stack = torch.stack(parts, 0)
                yield (b + dst + ".weight", (spec.n_expert, stack.shape[1], k), ty, stack.reshape(-1, stack.shape[-1]))
    yield f32_item("model.norm.weight", "output_norm.weight")
    if "lm_head.weight" in folder:
        yield linear("lm_head", "output")


def load_folder(path: str, device) -> Tuple[ModelSpec, "Weights", object]:
    from ..formats.safetensors import Folder
    folder = Folder(path)
    spec = ModelSpec.from_hf_config(folder.config)
    w = Weights.from_items(spec, folder_items(folder, spec), device)
    if torch.device(device).type == "cuda":
        torch.cuda.synchronize(device)
    return spec, w, folder


def open_model(path: str, device, **kw):
    """A path opens as a GGUF file (or first shard of a split) or as a checkpoint folder
    (the reference's ``model_file``: ``crates/model-hf/src/lib.rs:1-12``)."""
    import os
    if os.path.isdir(path):
        return load_folder(path, device)
    return load_gguf(path, device, **kw)


def write_folder(spec: ModelSpec, path: str, scheme: str = "fp8_b128", seed: int = 0, std: float = 0.02, shards: int = 2) -> None:
    """Seeded synthetic checkpoint folder in one of the stored quantisation schemes (fixtures)."""
    from ..formats import planes
    from ..formats import safetensors as S
    gen = torch.Generator().manual_seed(seed)
    tensors: Dict[str, torch.Tensor] = {}
    tags: Dict[str, str] = {}

    def lin(stem: str, rows: int, k: int, quant_it: bool = True):
        w = torch.randn(rows, k, generator=gen) * std
        if not quant_it or scheme == "plain":
            tensors[stem + ".weight"] = w.bfloat16()
        elif scheme == "fp8_b128":
            c, sc = planes.fp8_b128_quantize(w)
            tensors[stem + ".weight"], tensors[stem + ".weight_scale_inv"] = c, sc
            tags[stem + ".weight"] = "F8_E4M3"
        else:
            pk, sc, ts = planes.nvfp4_quantize(w)
            tags[stem + ".weight_scale"] = "F8_E4M3"
            tensors[stem + ".weight_scale"] = sc
            if scheme == "nvfp4_modelopt":
                tensors[stem + ".weight"], tensors[stem + ".weight_scale_2"] = pk, ts.reshape(())
                tensors[stem + ".input_scale"] = torch.tensor(1.0)          # stored by ModelOpt; read and ignored
            else:
                tensors[stem + ".weight_packed"], tensors[stem + ".weight_global_scale"] = pk, (1.0 / ts).reshape(1)

    def norm(name: str, n: int):
        tensors[name] = (torch.ones(n) + 0.02 * torch.randn(n, generator=gen)).bfloat16()

    H = spec.hidden
    lin("model.embed_tokens", spec.vocab, H, quant_it=False)
    for il in range(spec.n_layer):
        hp = f"model.layers.{il}."
        norm(hp + "input_layernorm.weight", H)
        norm(hp + "post_attention_layernorm.weight", H)
        lin(hp + "self_attn.q_proj", spec.q_rows, H)
        lin(hp + "self_attn.k_proj", spec.kv_rows, H)
        lin(hp + "self_attn.v_proj", spec.kv_rows, H)
        lin(hp + "self_attn.o_proj", H, spec.q_rows)
        if spec.qk_norm:
            norm(hp + "self_attn.q_norm.weight", spec.head_dim)
            norm(hp + "self_attn.k_norm.weight", spec.head_dim)
        if spec.layer_is_moe(il):
            tensors[hp + "mlp.gate.weight"] = (torch.randn(spec.n_expert, H, generator=gen) * std).bfloat16()
            for e in range(spec.n_expert):
                lin(f"{hp}mlp.experts.{e}.gate_proj", spec.moe_inter, H)
                lin(f"{hp}mlp.experts.{e}.up_proj", spec.moe_inter, H)
                lin(f"{hp}mlp.experts.{e}.down_proj", H, spec.moe_inter)
        else:
            lin(hp + "mlp.gate_proj", spec.dense_inter, H)
            lin(hp + "mlp.up_proj", spec.dense_inter, H)
            lin(hp + "mlp.down_proj", H, spec.dense_inter)
    norm("model.norm.weight", H)
    lin("lm_head", spec.vocab, H, quant_it=False)
    qc = {"fp8_b128": {"quant_method": "fp8", "weight_block_size": [128, 128]},
          "nvfp4_modelopt": {"quant_method": "modelopt", "quant_algo": "NVFP4"},
          "nvfp4_ct": {"quant_method": "compressed-tensors", "format": "nvfp4-pack-quantized"}}.get(scheme)
    cfg = spec.to_hf_config()
    if qc:
        cfg["quantization_config"] = qc
    S.write_folder(path, tensors, cfg, shards=shards, dtypes=tags)
