"""Latent-attention kernels against a plain PyTorch fp32 restatement, and the DeepSeek-shaped engine
(MLA, leading dense layer, sigmoid router with bias and groups, shared expert) against the CPU oracle."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rope_pairs(x, pos, inv_freq):
    ang = pos.float()[:, None] * inv_freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [x.shape[-1] // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], -1).reshape(x.shape)


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,ctx", [(8, 70), (20, 300)])
def test_mla_kernels_match_fp32(wdtype, n_q, ctx):
    from bloomery_b200.formats import quant as Q
    from bloomery_b200.models.cpu_ref import rms_norm
    from bloomery_b200.ops import decode as K
    torch.manual_seed(0)
    nope, v_dim, M, n_seg, max_pages, n_pages = 128, 128, 3, 5, 8, 24
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, 64, 2).double() / 64))).float()
    scale = 1.0 / math.sqrt(nope + 64)
    cache = torch.zeros(n_pages, 64, 576, dtype=torch.float16, device=DEV)
    table = torch.full((2, max_pages), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages)
    table[0, :5] = perm[:5].int(); table[1, :5] = perm[5:10].int()
    table = table.to(DEV)
    gain = (1 + 0.1 * torch.randn(512))
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    # fill two sequences position by position through the append kernel
    kv_all = torch.randn(2, ctx, 576)
    kv_all[0, 3, 17] = 25.0
    for p0 in range(0, ctx):
        rows = kv_all[:, p0].contiguous().to(DEV)
        pos = torch.tensor([p0, p0], dtype=torch.int32, device=DEV)
        seq = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
        K.mla_kv_append(rows, gain.to(DEV), inv_freq.to(DEV), 1e-6, 2, pos, seq, table, n_pages, cache, fault, 0)
    assert int(fault) == -1
    posv = torch.arange(ctx)
    want_rows = []
    for sq in range(2):
        c = rms_norm(kv_all[sq, :, :512], gain, 1e-6)
        kr = _rope_pairs(kv_all[sq, :, 512:], posv, inv_freq)
        want_rows.append(torch.cat([c, kr], -1).half())
        got = torch.stack([cache[int(table[sq, p0 // 64]), p0 % 64] for p0 in range(ctx)]).cpu()
        assert ((got.float() - want_rows[sq].float()).abs().max() / want_rows[sq].float().abs().max()).item() < 2e-3
    # rows of the pass: sequence 0 at its last position, a padding row, sequence 1 in the middle
    row_pos = torch.tensor([ctx - 1, 0, ctx // 2], dtype=torch.int32, device=DEV)
    row_seq = torch.tensor([0, -1, 1], dtype=torch.int32, device=DEV)
    q = torch.randn(M, n_q * (nope + 64))
    w_kb = (torch.randn(n_q, nope, 512) * 0.05).to(wdtype)
    w_vb = (torch.randn(n_q, v_dim, 512) * 0.05).to(wdtype)
    q_lat = torch.zeros(M, n_q, 576, device=DEV)
    K.mla_q_absorb(q.to(DEV), w_kb.to(DEV), inv_freq.to(DEV), scale, n_q, nope, M, row_pos, row_seq, q_lat)
    part_ml = torch.zeros(M * n_q * n_seg * 2, device=DEV)
    part_acc = torch.zeros(M * n_q * n_seg * 512, device=DEV)
    out = torch.zeros(M, n_q * v_dim, device=DEV)
    outq = torch.zeros(M, n_q * v_dim, dtype=torch.int8, device=DEV)
    outds = torch.zeros(M, n_q * v_dim // 32, 2, device=DEV)
    for _ in range(2):
        K.mla_flash_decode(q_lat, cache, row_pos, row_seq, table, n_pages, n_q, M, n_seg, 512, part_ml, part_acc,
                           w_vb.to(DEV), v_dim, out, outq, outds, fault, 0)
    assert int(fault) == -1
    for m, item in enumerate([(0, ctx - 1), None, (1, ctx // 2)]):
        if item is None:
            continue
        sq, p0 = item
        qm = q[m].reshape(n_q, nope + 64)
        q_rope = _rope_pairs(qm[None, :, nope:], torch.tensor([p0]), inv_freq)[0]
        rows = torch.stack([cache[int(table[sq, t // 64]), t % 64] for t in range(p0 + 1)]).cpu().float()
        lat, kr = rows[:, :512], rows[:, 512:]
        k_nope = torch.einsum("hnc,sc->shn", w_kb.float(), lat)
        v = torch.einsum("hvc,sc->shv", w_vb.float(), lat)
        sc = (torch.einsum("hn,shn->hs", qm[:, :nope], k_nope) + torch.einsum("hr,sr->hs", q_rope, kr)) * scale
        ref = torch.einsum("hs,shv->hv", torch.softmax(sc.double(), -1).float(), v).reshape(-1)
        err = ((out[m].cpu() - ref).abs().max() / ref.abs().max()).item()
        assert err < 5e-3, (m, err)      # q and the probabilities pass through f16 on their way to the tensor cores
        c, ds = Q.quantize_act_q8(out[m].cpu()[None])
        assert torch.equal(outq[m].cpu(), c[0]) and torch.allclose(outds[m].cpu(), ds[0], rtol=1e-6)
    # a key count beyond the context is a fault and NaN rows
    row_pos[0] = 600
    K.mla_flash_decode(q_lat, cache, row_pos, row_seq, table, n_pages, n_q, M, n_seg, 512, part_ml, part_acc,
                       w_vb.to(DEV), v_dim, out, outq, outds, fault, 3)
    assert (int(fault) & 0xFFFFFFFF) == (3 << 8 | 5) and torch.isnan(out[0]).all() and not torch.isnan(out[2]).any()


def _engine(graphs=True):
    from bloomery_b200.models.spec import tiny_deepseek
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_deepseek()
    items = list(synth_tensors(spec, "cpu", seed=5))
    wg = Weights.from_items(spec, iter(items), DEV)
    wc = Weights.from_items(spec, iter(items), "cpu")
    return spec, DecodeEngine(wg, n_slots=2, slot_ctx=512, use_graphs=graphs), wc


def test_deepseek_engine_matches_oracle():
    from bloomery_b200.models.cpu_ref import CpuModel
    spec, eng, wc = _engine()
    _, eng2, _ = _engine(graphs=False)
    cpu = CpuModel(wc)
    g = torch.Generator().manual_seed(21)
    prompt = torch.randint(0, spec.vocab, (75,), generator=g).tolist()
    ref = cpu.forward(torch.tensor(prompt))
    eng.prefill(0, prompt)
    eng2.prefill(0, prompt)
    n_last = len(prompt) % 8 or 8
    got, want = eng.logits[:n_last].cpu(), ref[-n_last:]
    err = ((got - want).abs().max() / want.abs().max()).item()
    rms = ((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()).item()
    assert err < 4e-2 and rms < 1.5e-2, (err, rms)
    assert torch.equal(eng.logits[:n_last], eng2.logits[:n_last])         # replay == eager, bit for bit
    # chained greedy decode equals stepping one token at a time
    first = int(torch.argmax(eng.logits[n_last - 1]))
    chain = eng.decode_chain(0, first, len(prompt), 8)
    eng.cut(0, len(prompt))
    tok, single = first, []
    for i in range(8):
        tok = eng.step([(0, tok, len(prompt) + i)])[0]
        single.append(tok)
    assert chain == single


def test_mtp_draft_layer_matches_oracle_and_never_changes_tokens():
    """The multi-token-prediction layer: its logits follow the oracle's, and verifying its drafts as extra rows
    yields exactly the tokens of plain greedy decoding (a draft changes which passes run, never a token)."""
    from bloomery_b200.models.cpu_ref import CpuModel, greedy_pick
    from bloomery_b200.models.spec import tiny_deepseek
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_deepseek()
    spec.n_mtp = 1
    items = list(synth_tensors(spec, "cpu", seed=6))
    eng = DecodeEngine(Weights.from_items(spec, iter(items), DEV), n_slots=1, slot_ctx=512, use_graphs=True)
    assert eng.n_mtp == 1 and eng.kv.k.shape[0] == spec.n_layer + 1
    cpu = CpuModel(Weights.from_items(spec, iter(items), "cpu"))
    g = torch.Generator().manual_seed(31)
    prompt = torch.randint(0, spec.vocab, (21,), generator=g).tolist()
    # plain greedy decoding first
    first = eng.prefill(0, prompt)
    plain, tok = [first], first
    for i in range(12):
        tok = eng.step([(0, tok, len(prompt) + i)])[0]
        plain.append(tok)
    # the same with the draft layer on
    eng.reset(0)
    assert eng.enable_mtp()
    first2 = eng.prefill(0, prompt)
    assert first2 == first and eng.mtp_draft[0][0] == len(prompt) + 1
    # oracle of the draft layer over the prompt rows
    ref_logits = cpu.forward(torch.tensor(prompt))
    nxt = torch.tensor(prompt[1:] + [first])
    ref_mtp = cpu.mtp_forward(nxt, cpu.hidden, torch.arange(len(prompt)))
    n_last = len(prompt) % 8 or 8
    got, want = eng.mtp_logits[n_last - 1].cpu(), ref_mtp[-1]
    rms = ((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()).item()
    assert rms < 2e-2, rms
    assert eng.mtp_draft[0][1] == int(torch.argmax(eng.mtp_logits[n_last - 1]))
    # speculative loop: feed the pending token plus the draft, keep the draft when the trunk agrees
    out, tok, pos, passes, kept_total = [first], first, len(prompt), 0, 0
    while len(out) < 13:
        d = eng.mtp_draft.get(0)
        rows = [(0, tok, pos)]
        if d is not None and d[0] == pos + 1:
            rows.append((0, d[1], pos + 1))
        picks = eng.step(rows)
        passes += 1
        kept = 1 if len(rows) == 2 and picks[0] == rows[1][1] else 0
        if len(rows) == 2 and not kept:
            eng.cut(0, pos + 1)
        eng.draft_after(rows, picks)
        out.extend(picks[:kept + 1])
        kept_total += kept
        tok, pos = picks[kept], pos + 1 + kept
    assert out[:13] == plain[:13], (out, plain)
    assert passes + kept_total >= 12
