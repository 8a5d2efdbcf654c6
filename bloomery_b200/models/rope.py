"""Rotary tables: plain and YaRN-scaled inverse frequencies, and the softmax scale that goes with them.

DeepSeek-V3 / Kimi-K2 stretch the context with YaRN: frequencies below a correction range are
divided by the factor, those above are kept, a linear ramp blends between, and the softmax scale is
multiplied by ``mscale**2`` with ``mscale = 0.1 * mscale_all_dim * ln(factor) + 1`` (the reference
carries the same header fields: ``crates/model/src/arch`` deepseek2 hparams).
"""
from __future__ import annotations

import math

import torch

from .spec import ModelSpec


def _yarn_correction_dim(n_rot: float, dim: int, base: float, orig_ctx: int) -> float:
    return dim * math.log(orig_ctx / (n_rot * 2 * math.pi)) / (2 * math.log(base))


def inv_freq_table(spec: ModelSpec, dim: int) -> torch.Tensor:
    """fp32 [dim/2] inverse frequencies of a rotary block of ``dim`` values."""
    expo = torch.arange(0, dim, 2, dtype=torch.float64) / dim
    extra = 1.0 / (spec.rope_theta ** expo)
    if spec.rope_yarn_factor <= 1.0:
        return (extra / spec.rope_scale).float()
    inter = extra / spec.rope_yarn_factor
    low = max(math.floor(_yarn_correction_dim(spec.rope_yarn_beta_fast, dim, spec.rope_theta, spec.rope_yarn_orig_ctx)), 0)
    high = min(math.ceil(_yarn_correction_dim(spec.rope_yarn_beta_slow, dim, spec.rope_theta, spec.rope_yarn_orig_ctx)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
    mask = 1.0 - ramp
    return (inter * (1 - mask) + extra * mask).float()


def yarn_mscale(factor: float, mscale: float) -> float:
    return 1.0 if factor <= 1.0 else 0.1 * mscale * math.log(factor) + 1.0


def attn_scale(spec: ModelSpec) -> float:
    """Softmax scale of the attention scores (1/sqrt(d_qk), times the YaRN magnitude correction)."""
    d = (spec.nope_dim + spec.rope_dim) if spec.mla else spec.head_dim
    m = yarn_mscale(spec.rope_yarn_factor, spec.rope_mscale_all_dim) if spec.rope_yarn_factor > 1.0 else 1.0
    return m * m / math.sqrt(d)
