"""Model description read from a checkpoint header.

Counterpart of ``crates/models`` (``ModelSpec``: layers, mixers, FFN, residual scheme;
``lib.rs:1-17``) and of the per-arch ``hparams``/``names`` readers in
``crates/model/src/arch/*``.  One dataclass covers the in-scope families: the Qwen3
mixture-of-experts shape (GQA with per-head QK norm, softmax top-k router) and the
DeepSeek shape (MLA, sigmoid router with selection bias, shared expert, leading dense
layers, optional MTP layer); dense llama/qwen3 models are the ``n_expert == 0`` case.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional


@dataclasses.dataclass
class ModelSpec:
    arch: str = "qwen3moe"
    name: str = ""
    n_layer: int = 0
    hidden: int = 0
    n_q: int = 0
    n_kv: int = 0
    head_dim: int = 128
    vocab: int = 0
    ctx_train: int = 32768
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scale: float = 1.0
    rope_yarn_factor: float = 1.0     # > 1: YaRN-scaled frequencies
    rope_yarn_orig_ctx: int = 4096
    rope_yarn_beta_fast: float = 32.0
    rope_yarn_beta_slow: float = 1.0
    rope_mscale_all_dim: float = 0.0
    qk_norm: bool = True
    # FFN
    dense_inter: int = 0
    n_expert: int = 0
    n_used: int = 0
    moe_inter: int = 0
    n_shared: int = 0
    shared_inter: int = 0
    first_dense: int = 0
    # router
    router_mode: str = "softmax"      # softmax | sigmoid
    router_renorm: bool = True
    router_scale: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    # MLA
    mla: bool = False
    q_lora: int = 0
    kv_lora: int = 0
    rope_dim: int = 0
    nope_dim: int = 0
    v_dim: int = 0
    # multi-token prediction
    n_mtp: int = 0
    # tokenizer / chat surface (header copies)
    bos_id: int = -1
    eos_id: int = -1

    @property
    def is_moe(self) -> bool:
        return self.n_expert > 0

    @property
    def q_rows(self) -> int:
        return self.n_q * self.head_dim

    @property
    def kv_rows(self) -> int:
        return self.n_kv * self.head_dim

    def layer_is_moe(self, il: int) -> bool:
        return self.is_moe and il >= self.first_dense

    def kv_bytes_per_token(self) -> int:
        if self.mla:
            return self.n_layer * (self.kv_lora + self.rope_dim) * 2
        return self.n_layer * 2 * self.n_kv * self.head_dim * 2

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    # ---- readers -------------------------------------------------------------------
    @classmethod
    def from_gguf(cls, g) -> "ModelSpec":
        arch = g.arch
        a = g.arch_get
        if arch in ("llama", "qwen2", "qwen2moe"):
            # llama-arch files carry Q/K rows permuted for interleaved RoPE pairs, qwen2 files carry QKV biases and
            # qwen2moe a gated shared expert: the chains here apply none of the three, so such a file is refused
            # instead of being decoded to wrong logits
            raise ValueError(f"architecture {arch!r} has no seat in this build")
        if arch in ("qwen3moe", "qwen3"):
            if any(n.endswith((".attn_q.bias", ".attn_k.bias", ".attn_v.bias")) for n in g.tensors):
                raise ValueError(f"architecture {arch!r} with attention biases has no seat in this build")
            n_q = int(a("attention.head_count"))
            hidden = int(a("embedding_length"))
            head = int(a("attention.key_length", hidden // n_q))
            tok = g.tensors.get("token_embd.weight")
            vocab = int(a("vocab_size", tok.shape[0] if tok else 0))
            return cls(
                arch=arch, name=str(g.get("general.name", "")), n_layer=int(a("block_count")), hidden=hidden,
                n_q=n_q, n_kv=int(a("attention.head_count_kv", n_q)), head_dim=head, vocab=vocab,
                ctx_train=int(a("context_length", 32768)),
                rms_eps=float(a("attention.layer_norm_rms_epsilon", 1e-6)),
                rope_theta=float(a("rope.freq_base", 10000.0)),
                qk_norm=("blk.0.attn_q_norm.weight" in g.tensors),
                dense_inter=int(a("feed_forward_length", 0) or 0),
                n_expert=int(a("expert_count", 0) or 0), n_used=int(a("expert_used_count", 0) or 0),
                moe_inter=int(a("expert_feed_forward_length", 0) or 0),
                router_mode="softmax", router_renorm=True,
                bos_id=int(g.get("tokenizer.ggml.bos_token_id", -1)), eos_id=int(g.get("tokenizer.ggml.eos_token_id", -1)),
            )
        if arch in ("deepseek2", "deepseek3"):
            n_q = int(a("attention.head_count"))
            return cls(
                arch=arch, name=str(g.get("general.name", "")), n_layer=int(a("block_count")),
                hidden=int(a("embedding_length")), n_q=n_q, n_kv=n_q, head_dim=int(a("attention.key_length", 192)),
                vocab=int(a("vocab_size", 0)), ctx_train=int(a("context_length", 4096)),
                rms_eps=float(a("attention.layer_norm_rms_epsilon", 1e-6)), rope_theta=float(a("rope.freq_base", 1e4)),
                qk_norm=False, dense_inter=int(a("feed_forward_length", 0) or 0),
                n_expert=int(a("expert_count", 0) or 0), n_used=int(a("expert_used_count", 0) or 0),
                moe_inter=int(a("expert_feed_forward_length", 0) or 0), n_shared=int(a("expert_shared_count", 0) or 0),
                shared_inter=int(a("expert_feed_forward_length", 0) or 0) * int(a("expert_shared_count", 0) or 0),
                first_dense=int(a("leading_dense_block_count", 0) or 0),
                router_mode="sigmoid" if int(a("expert_gating_func", 1) or 1) == 2 else "softmax",
                router_renorm=bool(a("expert_weights_norm", False)), router_scale=float(a("expert_weights_scale", 1.0)),
                n_group=int(a("expert_group_count", 1) or 1), topk_group=int(a("expert_group_used_count", 1) or 1),
                mla=True, q_lora=int(a("attention.q_lora_rank", 0) or 0), kv_lora=int(a("attention.kv_lora_rank", 512)),
                rope_dim=int(a("rope.dimension_count", 64)),
                nope_dim=int(a("attention.key_length", 192)) - int(a("rope.dimension_count", 64)),
                v_dim=int(a("attention.value_length", 128)), n_mtp=int(a("nextn_predict_layers", 0) or 0),
                rope_yarn_factor=float(a("rope.scaling.factor", 1.0) or 1.0) if a("rope.scaling.type", "") == "yarn" else 1.0,
                rope_yarn_orig_ctx=int(a("rope.scaling.original_context_length", 4096) or 4096),
                rope_mscale_all_dim=float(a("rope.scaling.yarn_log_multiplier", 0.0) or 0.0) * 10.0,
            )
        raise ValueError(f"architecture {arch!r} has no seat in this build")

    @classmethod
    def from_hf_config(cls, c: Dict[str, Any]) -> "ModelSpec":
        """config.json of a checkpoint folder (the reference: ``crates/hf``, ``crates/model-hf``)."""
        archs = c.get("architectures") or [""]
        kind = str(c.get("model_type") or archs[0]).lower()
        n_q = int(c["num_attention_heads"])
        hidden = int(c["hidden_size"])
        common = dict(
            name=str(c.get("_name_or_path", "") or kind), n_layer=int(c["num_hidden_layers"]), hidden=hidden, n_q=n_q,
            vocab=int(c["vocab_size"]), ctx_train=int(c.get("max_position_embeddings", 32768)),
            rms_eps=float(c.get("rms_norm_eps", 1e-6)), rope_theta=float(c.get("rope_theta", 1e4)),
            bos_id=int(c.get("bos_token_id", -1) if c.get("bos_token_id") is not None else -1),
            eos_id=int(c["eos_token_id"][0] if isinstance(c.get("eos_token_id"), list) else (c.get("eos_token_id", -1) if c.get("eos_token_id") is not None else -1)),
        )
        if "deepseek" in kind or "kimi" in kind:
            rope, nope = int(c.get("qk_rope_head_dim", 64)), int(c.get("qk_nope_head_dim", 128))
            n_sh = int(c.get("n_shared_experts", 0) or 0)
            return cls(arch="deepseek2", n_kv=n_q, head_dim=rope + nope, qk_norm=False,
                       dense_inter=int(c.get("intermediate_size", 0)), n_expert=int(c.get("n_routed_experts", 0) or 0),
                       n_used=int(c.get("num_experts_per_tok", 0) or 0), moe_inter=int(c.get("moe_intermediate_size", 0) or 0),
                       n_shared=n_sh, shared_inter=n_sh * int(c.get("moe_intermediate_size", 0) or 0),
                       first_dense=int(c.get("first_k_dense_replace", 0) or 0),
                       router_mode="sigmoid" if c.get("scoring_func", "softmax") == "sigmoid" else "softmax",
                       router_renorm=bool(c.get("norm_topk_prob", False)), router_scale=float(c.get("routed_scaling_factor", 1.0)),
                       n_group=int(c.get("n_group", 1) or 1), topk_group=int(c.get("topk_group", 1) or 1), mla=True,
                       q_lora=int(c.get("q_lora_rank") or 0), kv_lora=int(c.get("kv_lora_rank", 512)), rope_dim=rope,
                       nope_dim=nope, v_dim=int(c.get("v_head_dim", 128)), n_mtp=int(c.get("num_nextn_predict_layers", 0) or 0),
                       **_yarn_fields(c.get("rope_scaling")), **common)
        if kind in ("qwen3_moe", "qwen3moe", "qwen3moeforcausallm", "qwen3", "llama", "qwen2", "mistral", "qwen3forcausallm"):
            n_exp = int(c.get("num_experts", 0) or 0)
            return cls(arch="qwen3moe" if n_exp else ("qwen3" if "qwen3" in kind else "llama"),
                       n_kv=int(c.get("num_key_value_heads", n_q)), head_dim=int(c.get("head_dim") or hidden // n_q),
                       qk_norm="qwen3" in kind, dense_inter=int(c.get("intermediate_size", 0) or 0), n_expert=n_exp,
                       n_used=int(c.get("num_experts_per_tok", 0) or 0), moe_inter=int(c.get("moe_intermediate_size", 0) or 0),
                       router_mode="softmax", router_renorm=bool(c.get("norm_topk_prob", True)), **common)
        raise ValueError(f"model type {kind!r} has no seat in this build")

    def to_hf_config(self) -> Dict[str, Any]:
        """The config.json this spec would be read back from (fixtures)."""
        if self.mla:
            return {"model_type": "deepseek_v3", "architectures": ["DeepseekV3ForCausalLM"], "num_hidden_layers": self.n_layer,
                    "hidden_size": self.hidden, "num_attention_heads": self.n_q, "vocab_size": self.vocab,
                    "max_position_embeddings": self.ctx_train, "rms_norm_eps": self.rms_eps, "rope_theta": self.rope_theta,
                    "qk_rope_head_dim": self.rope_dim, "qk_nope_head_dim": self.nope_dim, "v_head_dim": self.v_dim,
                    "q_lora_rank": self.q_lora or None, "kv_lora_rank": self.kv_lora, "intermediate_size": self.dense_inter,
                    "n_routed_experts": self.n_expert, "num_experts_per_tok": self.n_used,
                    "moe_intermediate_size": self.moe_inter, "n_shared_experts": self.n_shared,
                    "first_k_dense_replace": self.first_dense, "scoring_func": self.router_mode,
                    "norm_topk_prob": self.router_renorm, "routed_scaling_factor": self.router_scale,
                    "n_group": self.n_group, "topk_group": self.topk_group, "num_nextn_predict_layers": self.n_mtp,
                    "rope_scaling": None if self.rope_yarn_factor <= 1.0 else {
                        "type": "yarn", "factor": self.rope_yarn_factor,
                        "original_max_position_embeddings": self.rope_yarn_orig_ctx, "beta_fast": self.rope_yarn_beta_fast,
                        "beta_slow": self.rope_yarn_beta_slow, "mscale": self.rope_mscale_all_dim,
                        "mscale_all_dim": self.rope_mscale_all_dim}}
        return {"model_type": "qwen3_moe" if self.is_moe else ("qwen3" if self.qk_norm else "llama"),
                "architectures": ["Qwen3MoeForCausalLM" if self.is_moe else "Qwen3ForCausalLM"],
                "num_hidden_layers": self.n_layer, "hidden_size": self.hidden, "num_attention_heads": self.n_q,
                "num_key_value_heads": self.n_kv, "head_dim": self.head_dim, "vocab_size": self.vocab,
                "max_position_embeddings": self.ctx_train, "rms_norm_eps": self.rms_eps, "rope_theta": self.rope_theta,
                "intermediate_size": self.dense_inter, "num_experts": self.n_expert, "num_experts_per_tok": self.n_used,
                "moe_intermediate_size": self.moe_inter, "norm_topk_prob": self.router_renorm}


def _yarn_fields(rs) -> Dict[str, Any]:
    if not isinstance(rs, dict) or str(rs.get("type", rs.get("rope_type", ""))).lower() != "yarn":
        return {}
    return {"rope_yarn_factor": float(rs.get("factor", 1.0)),
            "rope_yarn_orig_ctx": int(rs.get("original_max_position_embeddings", 4096)),
            "rope_yarn_beta_fast": float(rs.get("beta_fast", 32.0)), "rope_yarn_beta_slow": float(rs.get("beta_slow", 1.0)),
            "rope_mscale_all_dim": float(rs.get("mscale_all_dim", 0.0))}


# The named benchmark / test shapes.
def tiny_qwen3moe() -> ModelSpec:
    return ModelSpec(arch="qwen3moe", name="tiny-qwen3moe", n_layer=4, hidden=512, n_q=8, n_kv=2, head_dim=64,
                     vocab=32000, ctx_train=4096, rms_eps=1e-6, rope_theta=1e6, qk_norm=True, n_expert=16, n_used=4,
                     moe_inter=256)


def tiny_deepseek() -> ModelSpec:
    """The DeepSeek-V3 layer plan at toy size: MLA (latent 512 + rope 64), a leading dense layer, sigmoid router
    with selection bias and groups, one shared expert."""
    return ModelSpec(arch="deepseek2", name="tiny-deepseek", n_layer=3, hidden=512, n_q=8, n_kv=8, head_dim=192,
                     vocab=8192, ctx_train=4096, rms_eps=1e-6, rope_theta=1e4, qk_norm=False, dense_inter=1024,
                     n_expert=16, n_used=4, moe_inter=256, n_shared=1, shared_inter=256, first_dense=1,
                     router_mode="sigmoid", router_renorm=True, router_scale=2.5, n_group=4, topk_group=2, mla=True,
                     q_lora=256, kv_lora=512, rope_dim=64, nope_dim=128, v_dim=128, rope_yarn_factor=4.0,
                     rope_yarn_orig_ctx=1024, rope_mscale_all_dim=1.0)


def deepseek_v3() -> ModelSpec:
    return ModelSpec(arch="deepseek2", name="deepseek-v3-shaped", n_layer=61, hidden=7168, n_q=128, n_kv=128,
                     head_dim=192, vocab=129280, ctx_train=163840, rms_eps=1e-6, rope_theta=1e4, qk_norm=False,
                     dense_inter=18432, n_expert=256, n_used=8, moe_inter=2048, n_shared=1, shared_inter=2048,
                     first_dense=3, router_mode="sigmoid", router_renorm=True, router_scale=2.5, n_group=8, topk_group=4,
                     mla=True, q_lora=1536, kv_lora=512, rope_dim=64, nope_dim=128, v_dim=128, n_mtp=1,
                     rope_yarn_factor=40.0, rope_yarn_orig_ctx=4096, rope_mscale_all_dim=1.0)


def qwen3_30b_a3b() -> ModelSpec:
    return ModelSpec(arch="qwen3moe", name="qwen3-30b-a3b-shaped", n_layer=48, hidden=2048, n_q=32, n_kv=4,
                     head_dim=128, vocab=151936, ctx_train=40960, rms_eps=1e-6, rope_theta=1e6, qk_norm=True,
                     n_expert=128, n_used=8, moe_inter=768)


def qwen3_235b_a22b() -> ModelSpec:
    return ModelSpec(arch="qwen3moe", name="qwen3-235b-a22b-shaped", n_layer=94, hidden=4096, n_q=64, n_kv=4,
                     head_dim=128, vocab=151936, ctx_train=40960, rms_eps=1e-6, rope_theta=1e6, qk_norm=True,
                     n_expert=128, n_used=8, moe_inter=1536)


def kimi_k2() -> ModelSpec:
    return ModelSpec(arch="deepseek2", name="kimi-k2-shaped", n_layer=61, hidden=7168, n_q=64, n_kv=64, head_dim=192,
                     vocab=163840, ctx_train=131072, rms_eps=1e-6, rope_theta=5e4, qk_norm=False, dense_inter=18432,
                     n_expert=384, n_used=8, moe_inter=2048, n_shared=1, shared_inter=2048, first_dense=1,
                     router_mode="sigmoid", router_renorm=True, router_scale=2.827, n_group=1, topk_group=1,
                     mla=True, q_lora=1536, kv_lora=512, rope_dim=64, nope_dim=128, v_dim=128)


NAMED = {
    "tiny-qwen3moe": tiny_qwen3moe,
    "qwen3-30b-a3b": qwen3_30b_a3b,
    "qwen3-235b-a22b": qwen3_235b_a22b,
    "deepseek-v3": deepseek_v3,
    "kimi-k2": kimi_k2,
}
