"""Prompt flash attention on tcgen05 / tensor memory against a plain fp32 PyTorch attention."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ref(q, k, v, pos0):
    """q [n_q, T, d] (pre-scaled), k / v [n_kv, n_keys, d]; causal: query t sees keys 0 .. pos0 + t."""
    n_q, T, d = q.shape
    n_kv, n_keys, _ = k.shape
    g = n_q // n_kv
    kk = k.repeat_interleave(g, 0).float()
    vv = v.repeat_interleave(g, 0).float()
    s = torch.einsum("htd,hkd->htk", q.float(), kk)
    t_idx = torch.arange(T, device=q.device)[:, None] + pos0
    k_idx = torch.arange(n_keys, device=q.device)[None, :]
    s = s.masked_fill((k_idx > t_idx)[None], float("-inf"))
    return torch.einsum("htk,hkd->htd", torch.softmax(s, -1), vv)          # [n_q, T, d]


@pytest.mark.parametrize("n_q,n_kv,T,pos0", [(8, 2, 300, 0), (4, 4, 257, 77), (32, 4, 1024, 0), (2, 1, 128, 4000), (8, 1, 64, 0)])
def test_flash_prefill_matches_fp32_attention(n_q, n_kv, T, pos0):
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(0)
    d = 128
    n_keys = pos0 + T
    t_pad = (n_keys + 127) // 128 * 128
    q = (torch.randn(n_q, T, d, device=DEV) / math.sqrt(d)).bfloat16()
    k = torch.randn(n_kv, n_keys, d, device=DEV).bfloat16()
    v = torch.randn(n_kv, n_keys, d, device=DEV).bfloat16()
    Kb = torch.zeros(n_kv, t_pad, d, device=DEV, dtype=torch.bfloat16)
    Vt = torch.zeros(n_kv, d, t_pad, device=DEV, dtype=torch.bfloat16)
    Kb[:, :n_keys] = k
    Vt[:, :, :n_keys] = v.transpose(1, 2)
    out = torch.full((T, n_q * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    G.flash_prefill(q, Kb, Vt, out, pos0, status)
    torch.cuda.synchronize()
    assert int(status) == 0
    ref = _ref(q, k, v, pos0).permute(1, 0, 2).reshape(T, n_q * d)
    err = (out.float() - ref).abs().max().item()
    assert torch.isfinite(out.float()).all()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err      # bf16 probabilities and outputs
    out2 = torch.zeros_like(out)
    G.flash_prefill(q, Kb, Vt, out2, pos0, status)
    assert torch.equal(out, out2)                                   # bit-identical rerun


def test_engine_prompt_through_flash_matches_the_three_launch_path():
    """A prompt through the GEMM path with and without the fused attention: same greedy token, logits in band."""
    from bloomery_b200.models.spec import ModelSpec
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = ModelSpec(arch="qwen3moe", name="flash-test", n_layer=2, hidden=512, n_q=8, n_kv=2, head_dim=128, vocab=4096,
                     ctx_train=4096, rms_eps=1e-6, rope_theta=1e6, qk_norm=True, n_expert=16, n_used=4, moe_inter=256)
    w = Weights.from_items(spec, synth_tensors(spec, "cpu", seed=3), "cpu").to(DEV)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, spec.vocab, (333,), generator=g).tolist()
    outs = []
    for flash in (True, False):
        eng = DecodeEngine(w, n_slots=1, slot_ctx=512)
        eng._gemm_prefill = eng._new_gemm_prefill()
        eng._gemm_prefill.flash = flash
        tok = eng.prefill(0, prompt, gemm=True)
        outs.append((tok, eng.logits[0].clone()))
    scale = outs[1][1].abs().max().item()
    assert (outs[0][1] - outs[1][1]).abs().max().item() < 3e-2 * scale
    assert outs[0][0] == outs[1][0]
