"""Decode-chain CUDA kernels against a plain PyTorch fp32 reference of the same op,
and the whole engine against the CPU oracle, token for token."""
import math

import pytest
import torch

from bloomery_b200.formats import quant as Q
from bloomery_b200.formats.resident import to_resident

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _qw(w, t):
    from bloomery_b200.formats.resident import quantize_resident
    from bloomery_b200.ops.decode import QWeight
    res, wd = quantize_resident(w.reshape(-1, w.shape[-1]), t)
    res = res.to(DEV)
    if w.dim() == 3:
        res = res.reshape(w.shape[0], w.shape[1], -1)
    from bloomery_b200.formats.resident import resident_type
    return QWeight(res, resident_type(t), w.shape[-1]), wd.reshape(w.shape)


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "NVFP4", "FP8_B128", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K",
                               "IQ4_NL", "IQ4_XS", "MXFP4", "IQ2_XXS"])
@pytest.mark.parametrize("M", [1, 3, 8])
def test_gemv_norm_matches_fp32(t, M):
    from bloomery_b200.ops import decode as K
    torch.manual_seed(0)
    Kd, rows = 2048, 520
    qw, wd = _qw(torch.randn(rows, Kd) * 0.02, t)
    x = torch.randn(M, Kd)
    x[0, 7] = 30.0
    gain = 1 + 0.1 * torch.randn(Kd)
    out = torch.zeros(M, rows, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    K.gemv([qw], M, out, x=x.to(DEV), gain=gain.to(DEV), eps=1e-6, fault=fault)
    from bloomery_b200.models.cpu_ref import rms_norm
    xn = rms_norm(x, gain, 1e-6)
    c, ds = Q.quantize_act_q8(xn)
    ref = (Q.dequantize_act_q8(c, ds).double() @ wd.double().T).float()
    err = ((out.cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err < 2e-3, err       # band covers code flips at .5 boundaries of the q8 rounding
    out2 = torch.zeros_like(out)
    K.gemv([qw], M, out2, x=x.to(DEV), gain=gain.to(DEV), eps=1e-6, fault=fault)
    assert torch.equal(out, out2)  # bit-identical rerun
    # each row of an m-row call equals its own 1-row call
    o1 = torch.zeros(1, rows, device=DEV)
    K.gemv([qw], 1, o1, x=x[M - 1:M].to(DEV), gain=gain.to(DEV), eps=1e-6, fault=fault)
    assert torch.equal(o1[0], out[M - 1])


def test_gemv_q8in_resid_multiseg():
    from bloomery_b200.ops import decode as K
    torch.manual_seed(1)
    Kd = 4096
    a, ad = _qw(torch.randn(300, Kd) * 0.02, "Q4_K")
    b, bd = _qw(torch.randn(77, Kd) * 0.02, "Q6_K")
    x = torch.randn(2, Kd)
    c, ds = Q.quantize_act_q8(x)
    resid = torch.randn(2, 377)
    out = torch.zeros(2, 377, device=DEV)
    K.gemv([a, b], 2, out, xq=c.to(DEV), xds=ds.to(DEV), resid=resid.to(DEV))
    xa = Q.dequantize_act_q8(c, ds).double()
    ref = torch.cat([xa @ ad.double().T, xa @ bd.double().T], 1).float() + resid
    assert ((out.cpu() - ref).abs().max() / ref.abs().max()).item() < 1e-5


def test_router_softmax_topk():
    from bloomery_b200.models.cpu_ref import rms_norm, route
    from bloomery_b200.models.spec import ModelSpec
    from bloomery_b200.ops import decode as K
    from bloomery_b200.ops.decode import QWeight, RouteRule
    torch.manual_seed(2)
    H, E, k, M = 2048, 128, 8, 5
    w = torch.randn(E, H) * 0.05
    x = torch.randn(M, H)
    gain = 1 + 0.1 * torch.randn(H)
    qw = QWeight(w.contiguous().view(torch.uint8).reshape(E, -1).to(DEV), "F32", H)
    logits = torch.zeros(M, E, device=DEV)
    ids = torch.zeros(M, k, dtype=torch.int32, device=DEV)
    wts = torch.zeros(M, k, device=DEV)
    xq = torch.zeros(M, H, dtype=torch.int8, device=DEV)
    xds = torch.zeros(M, H // 32, 2, device=DEV)
    heat = torch.zeros(E, dtype=torch.int32, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    rule = RouteRule(k)
    for _ in range(2):
        K.router(x.to(DEV), gain.to(DEV), 1e-6, qw, M, logits, xq, xds, None, fault, 0)
        K.route_rows(logits, rule, M, ids, wts, heat, fault, 0)
    xn = rms_norm(x, gain, 1e-6)
    ref_logits = xn @ w.T
    assert torch.allclose(logits.cpu(), ref_logits, rtol=1e-4, atol=1e-4)
    spec = ModelSpec(n_expert=E, n_used=k)
    rid, rw = route(logits.cpu(), spec)
    assert torch.equal(ids.cpu(), rid)
    assert torch.allclose(wts.cpu(), rw, rtol=1e-5, atol=1e-6)
    c, ds = Q.quantize_act_q8(xn)
    assert (xq.cpu() != c).float().mean() < 1e-3
    assert torch.allclose(xds.cpu(), ds, rtol=1e-3, atol=1e-6)
    assert int(heat.sum()) == 2 * M * k and int(fault) == -1


def test_router_sigmoid_groups_and_fault():
    from bloomery_b200.models.cpu_ref import route
    from bloomery_b200.models.spec import ModelSpec
    from bloomery_b200.ops import decode as K
    from bloomery_b200.ops.decode import QWeight, RouteRule
    torch.manual_seed(3)
    H, E, k, M = 512, 256, 8, 3
    w = torch.randn(E, H) * 0.05
    bias = torch.randn(E) * 0.1
    x = torch.randn(M, H)
    qw = QWeight(w.contiguous().view(torch.uint8).reshape(E, -1).to(DEV), "F32", H)
    logits = torch.zeros(M, E, device=DEV)
    ids = torch.zeros(M, k, dtype=torch.int32, device=DEV)
    wts = torch.zeros(M, k, device=DEV)
    xq = torch.zeros(M, H, dtype=torch.int8, device=DEV)
    xds = torch.zeros(M, H // 32, 2, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    rule = RouteRule(k, 1, True, 2.5, 8, 4, bias.to(DEV))
    K.router(x.to(DEV), torch.ones(H, device=DEV), 1e-6, qw, M, logits, xq, xds, None, fault, 0)
    K.route_rows(logits, rule, M, ids, wts, None, fault, 0)
    spec = ModelSpec(n_expert=E, n_used=k, router_mode="sigmoid", router_renorm=True, router_scale=2.5, n_group=8,
                     topk_group=4)
    rid, rw = route(logits.cpu(), spec, bias)
    assert torch.equal(ids.cpu(), rid)
    assert torch.allclose(wts.cpu(), rw, rtol=1e-5, atol=1e-6)
    # a non-finite logit raises the router fault, writes NaN weights and never traps
    xb = x.clone()
    xb[1, 3] = float("nan")
    K.router(xb.to(DEV), torch.ones(H, device=DEV), 1e-6, qw, M, logits, xq, xds, None, fault, 5)
    K.route_rows(logits, rule, M, ids, wts, None, fault, 5)
    assert (int(fault) & 0xFFFFFFFF) == (5 << 8 | 3)
    assert torch.isnan(wts[1]).all() and not torch.isnan(wts[0]).any()


def test_gate_up_routes_like_route_rows():
    """The routing done inside gate_up (from logits) equals the standalone routing launch."""
    from bloomery_b200.ops import decode as K
    from bloomery_b200.ops.decode import RouteRule
    torch.manual_seed(8)
    H, I, E, k, M = 512, 256, 16, 4, 3
    gate, _ = _qw(torch.randn(E, I, H) * 0.03, "Q4_K")
    up, _ = _qw(torch.randn(E, I, H) * 0.03, "Q4_K")
    x = torch.randn(M, H)
    c, ds = Q.quantize_act_q8(x)
    logits = torch.randn(M, E, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    rule = RouteRule(k)
    ids0 = torch.zeros(M, k, dtype=torch.int32, device=DEV); w0 = torch.zeros(M, k, device=DEV)
    K.route_rows(logits, rule, M, ids0, w0, None, fault, 0)
    outs = []
    for routed in (False, True):
        ids = ids0.clone() if not routed else torch.zeros_like(ids0)
        wts = torch.zeros(M, k, device=DEV)
        heat = torch.zeros(E, dtype=torch.int32, device=DEV)
        actq = torch.zeros(M, k, I, dtype=torch.int8, device=DEV)
        actds = torch.zeros(M, k, I // 32, 2, device=DEV)
        K.gate_up_sel(c.to(DEV), ds.to(DEV), ids, None, gate, up, E, k, M, actq, actds, None, fault, 0,
                      route_logits=logits if routed else None, rule=rule, wts=wts, heat=heat)
        outs.append((actq.clone(), actds.clone()))
        if routed:
            assert torch.equal(ids, ids0) and torch.equal(wts, w0) and int(heat.sum()) == M * k
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("gt,dt", [("Q4_K", "Q4_K"), ("Q4_K", "Q6_K"), ("Q8_0", "Q8_0"), ("Q5_K", "Q5_K"), ("NVFP4", "NVFP4"),
                                   ("FP8_B128", "FP8_B128"), ("Q4_0", "Q5_0"), ("Q5_1", "Q4_1"), ("Q2_K", "Q3_K"),
                                   ("IQ4_XS", "IQ4_NL"), ("MXFP4", "MXFP4"), ("IQ2_XXS", "Q4_K")])
def test_moe_sel_chain(gt, dt):
    from bloomery_b200.ops import decode as K
    torch.manual_seed(4)
    H, I, E, k, M = 1024, 768, 16, 4, 3
    gate, gd = _qw(torch.randn(E, I, H) * 0.03, gt)
    up, ud = _qw(torch.randn(E, I, H) * 0.03, gt)
    down, dd = _qw(torch.randn(E, H, I) * 0.03, dt)
    x = torch.randn(M, H)
    c, ds = Q.quantize_act_q8(x)
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(M)]).to(torch.int32)
    ids[2, 1] = -1                                          # served elsewhere: skipped silently
    wts = torch.rand(M, k)
    resid = torch.randn(M, H)
    actq = torch.zeros(M, k, I, dtype=torch.int8, device=DEV)
    actds = torch.zeros(M, k, I // 32, 2, device=DEV)
    actf = torch.zeros(M, k, I, device=DEV)
    out = torch.zeros(M, H, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    K.gate_up_sel(c.to(DEV), ds.to(DEV), ids.to(DEV), None, gate, up, E, k, M, actq, actds, actf, fault, 0)
    K.down_combine(actq, actds, ids.to(DEV), wts.to(DEV), None, down, E, k, M, resid.to(DEV), None, out, fault, 0)
    xa = Q.dequantize_act_q8(c, ds).double()
    ref = resid.clone().double()
    for m in range(M):
        for j in range(k):
            e = int(ids[m, j])
            if e < 0:
                continue
            g = xa[m] @ gd[e].double().T
            u = xa[m] @ ud[e].double().T
            a = (torch.nn.functional.silu(g) * u).float()
            assert torch.allclose(actf[m, j].cpu(), a, rtol=1e-4, atol=1e-5)
            ac, ads = Q.quantize_act_q8(actf[m, j].cpu()[None])
            ref[m] += wts[m, j].double() * (Q.dequantize_act_q8(ac, ads)[0].double() @ dd[e].double().T)
    assert ((out.cpu().double() - ref).abs().max() / ref.abs().max()).item() < 1e-5
    assert int(fault) == -1
    ids[0, 0] = E + 3                                       # any other id >= n_expert is a fault + NaN
    K.gate_up_sel(c.to(DEV), ds.to(DEV), ids.to(DEV), None, gate, up, E, k, M, actq, actds, actf, fault, 2)
    K.down_combine(actq, actds, ids.to(DEV), wts.to(DEV), None, down, E, k, M, resid.to(DEV), None, out, fault, 2)
    assert (int(fault) & 0xFFFFFFFF) == (2 << 8 | 4)
    assert torch.isnan(out[0]).all() and not torch.isnan(out[1]).any()


@pytest.mark.parametrize("head,n_q,n_kv", [(128, 32, 4), (64, 8, 2), (128, 64, 4)])
def test_rope_append_flash_decode(head, n_q, n_kv):
    from bloomery_b200.models.cpu_ref import rms_norm, rope_neox
    from bloomery_b200.ops import decode as K
    torch.manual_seed(5)
    M, ctx, n_seg = 3, 700, 9
    n_pages, max_pages = 40, 12
    lens = [1, 333, 700]                                    # keys each row sees (position + 1)
    width = (n_q + 2 * n_kv) * head
    qkv = torch.randn(M, width)
    qg, kg = 1 + 0.1 * torch.randn(head), 1 + 0.1 * torch.randn(head)
    inv = (1.0 / (1e6 ** (torch.arange(0, head, 2, dtype=torch.float64) / head))).float()
    table = torch.full((M, max_pages), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages)
    for s in range(M):
        table[s, :] = perm[s * max_pages:(s + 1) * max_pages] if (s + 1) * max_pages <= n_pages else perm[:max_pages]
    table[2] = perm[24:36]
    kc = torch.zeros(n_pages, n_kv, 64, head, dtype=torch.float16)
    vc = torch.zeros(n_pages, n_kv, 64, head, dtype=torch.float16)
    hist_k = [torch.randn(L - 1, n_kv, head).half() for L in lens]
    hist_v = [torch.randn(L - 1, n_kv, head).half() for L in lens]
    for s, L in enumerate(lens):
        for t in range(L - 1):
            pg = int(table[s, t // 64])
            kc[pg, :, t % 64] = hist_k[s][t]
            vc[pg, :, t % 64] = hist_v[s][t]
    pos = torch.tensor([L - 1 for L in lens], dtype=torch.int32)
    seq = torch.arange(M, dtype=torch.int32)
    d = lambda t: t.to(DEV)
    kc_d, vc_d = d(kc), d(vc)
    q_out = torch.zeros(M, n_q, head, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    K.qk_norm_rope_append(d(qkv), d(qg), d(kg), d(inv), 1e-6, 1 / math.sqrt(head), head, n_q, n_kv, M, d(pos), d(seq),
                          d(table), n_pages, kc_d, vc_d, q_out, fault, 0)
    q = qkv[:, :n_q * head].reshape(M, n_q, head)
    k = qkv[:, n_q * head:(n_q + n_kv) * head].reshape(M, n_kv, head)
    v = qkv[:, (n_q + n_kv) * head:].reshape(M, n_kv, head)
    qr = rope_neox(rms_norm(q, qg, 1e-6), pos, inv) / math.sqrt(head)
    kr = rope_neox(rms_norm(k, kg, 1e-6), pos, inv)
    assert torch.allclose(q_out.cpu(), qr, rtol=1e-4, atol=1e-4)
    part_ml = torch.zeros(M * n_q * n_seg * 2, device=DEV)
    part_acc = torch.zeros(M * n_q * n_seg * head, device=DEV)
    out = torch.zeros(M, n_q * head, device=DEV)
    outq = torch.zeros(M, n_q * head, dtype=torch.int8, device=DEV)
    outds = torch.zeros(M, n_q * head // 32, 2, device=DEV)
    K.flash_decode(q_out, kc_d, vc_d, d(pos), d(seq), d(table), n_pages, head, n_q, n_kv, M, n_seg, ctx, part_ml,
                   part_acc, out, outq, outds, fault, 0)
    G = n_q // n_kv
    for s, L in enumerate(lens):
        pg, off = int(table[s, (L - 1) // 64]), (L - 1) % 64
        assert torch.allclose(kc_d[pg, :, off].cpu().float(), kr[s].half().float(), atol=2e-3, rtol=2e-3)
        keys = torch.cat([hist_k[s].float(), kr[s].half().float()[None]], 0)      # [L, n_kv, head]
        vals = torch.cat([hist_v[s].float(), v[s].half().float()[None]], 0)
        sc = torch.einsum("hd,shd->hs", qr[s], keys.repeat_interleave(G, 1))
        pr = torch.softmax(sc, -1)
        ref = torch.einsum("hs,shd->hd", pr, vals.repeat_interleave(G, 1)).reshape(-1)
        assert torch.allclose(out[s].cpu(), ref, rtol=2e-3, atol=2e-3), (s, (out[s].cpu() - ref).abs().max())
    c, ds = Q.quantize_act_q8(out.cpu())
    assert (outq.cpu() != c).float().mean() < 1e-3
    assert int(fault) == -1
    # the tensor-tile variant of the segment pass (f16 q and probabilities): same result within the f16 band
    out_mma = torch.zeros_like(out)
    K.set_flash_mma(True)
    try:
        for _ in range(2):
            K.flash_decode(q_out, kc_d, vc_d, d(pos), d(seq), d(table), n_pages, head, n_q, n_kv, M, n_seg, ctx, part_ml,
                           part_acc, out_mma, outq, outds, fault, 0)
    finally:
        K.set_flash_mma(False)
    scale = out.abs().max().item()
    assert ((out_mma - out).abs().max().item()) < 5e-3 * max(scale, 1.0), (out_mma - out).abs().max()
    assert int(fault) == -1
    K.flash_decode(q_out, kc_d, vc_d, d(pos), d(seq), d(table), n_pages, head, n_q, n_kv, M, n_seg, ctx, part_ml,
                   part_acc, out, outq, outds, fault, 0)
    # a key count beyond the context is a fault and NaN, not a trap
    bad = pos.clone(); bad[1] = ctx + 5
    K.flash_decode(q_out, kc_d, vc_d, d(bad), d(seq), d(table), n_pages, head, n_q, n_kv, M, n_seg, ctx, part_ml,
                   part_acc, out, outq, outds, fault, 3)
    assert (int(fault) & 0xFFFFFFFF) == (3 << 8 | 5)
    assert torch.isnan(out[1]).all() and not torch.isnan(out[0]).any()


@pytest.mark.parametrize("t", ["Q4_K", "Q6_K", "Q8_0", "F16", "NVFP4", "FP8_B128", "Q4_0", "Q5_1", "IQ4_XS", "IQ2_XXS"])
def test_embed_and_argmax(t):
    from bloomery_b200.ops import decode as K
    from bloomery_b200.ops.decode import QWeight
    torch.manual_seed(6)
    V, H, M = 1000, 512, 4
    w = torch.randn(V, H) * 0.02
    if t == "F16":
        qw, wd = QWeight(w.half().contiguous().view(torch.uint8).reshape(V, -1).to(DEV), "F16", H), w.half().float()
    else:
        qw, wd = _qw(w, t)
    toks = torch.tensor([0, 999, 17, 5000], dtype=torch.int32, device=DEV)
    out = torch.zeros(M, H, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    K.embed_rows(toks, M, qw, V, out, fault)
    assert torch.equal(out[:3].cpu(), wd[[0, 999, 17]])
    assert torch.isnan(out[3]).all() and (int(fault) & 0xFFFFFFFF) == 1
    # argmax tie rule: lower id wins; NaN never wins; all-NaN row gives 0
    Vb = 151936
    logits = torch.randn(M, Vb, device=DEV)
    logits[0, 77] = 9.0; logits[0, 140000] = 9.0
    logits[1, 5] = float("nan"); logits[1, 6] = 8.0
    logits[2, :] = float("nan")
    logits[3, Vb - 1] = 50.0
    pv = torch.zeros(M * 64, device=DEV); pi = torch.zeros(M * 64, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(1, dtype=torch.int32, device=DEV)
    tout = torch.zeros(M + 1, dtype=torch.int32, device=DEV)
    for _ in range(2):
        K.argmax_rows(logits, Vb, M, 64, pv, pi, cnt, tout, None, fault)
    assert tout[:4].tolist() == [77, 6, 0, Vb - 1]
    assert (int(tout[4]) & 0xFFFFFFFF) == 1                 # the fault word rides beside the tokens


def _tiny_engine(graphs=True, mix="Q4_K_M", n_slots=2):
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_qwen3moe()
    items = list(synth_tensors(spec, "cpu", seed=7, mix=mix))
    wg = Weights.from_items(spec, iter(items), DEV)
    wc = Weights.from_items(spec, iter(items), "cpu")
    return spec, DecodeEngine(wg, n_slots=n_slots, slot_ctx=512, use_graphs=graphs), wc


def test_engine_matches_cpu_oracle_tokens():
    from bloomery_b200.models.cpu_ref import CpuModel, greedy_pick
    spec, eng, wc = _tiny_engine()
    cpu = CpuModel(wc)
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, spec.vocab, (64,), generator=g).tolist()
    ref = cpu.forward(torch.tensor(prompt))
    want = [greedy_pick(r) for r in ref]
    got = eng.score(0, prompt)
    agree = sum(int(a == b) for a, b in zip(want, got))
    # random-init logits are nearly flat, so a q8 rounding flip may move an arg-max; most must agree
    assert agree >= 58, (agree, got, want)
    # greedy continuation: the chained decode equals stepping one token at a time
    first = got[-1]
    chain = eng.decode_chain(0, first, len(prompt), 12)
    eng.cut(0, len(prompt))
    tok, single = first, []
    for i in range(12):
        tok = eng.step([(0, tok, len(prompt) + i)])[0]
        single.append(tok)
    assert chain == single


@pytest.mark.parametrize("mix", ["IQ4_XS", "MXFP4", "IQ2_XXS"])
def test_engine_on_codebook_types_matches_cpu_oracle(mix):
    """A model whose matrices are all of a code-book block type (loaded as int8 codes + f32 scales): logits against
    the CPU oracle over the same decoded weights."""
    from bloomery_b200.models.cpu_ref import CpuModel
    spec, eng, wc = _tiny_engine(mix=mix)
    assert eng.w.q["blk.0.attn_q.weight"].qtype == "Q8_F32"
    cpu = CpuModel(wc)
    g = torch.Generator().manual_seed(13)
    prompt = torch.randint(0, spec.vocab, (11,), generator=g).tolist()
    ref = cpu.forward(torch.tensor(prompt))
    eng.prefill(0, prompt, gemm=False)
    n_last = len(prompt) % 8 or 8
    err = ((eng.logits[:n_last].cpu() - ref[-n_last:]).abs().max() / ref[-n_last:].abs().max()).item()
    assert err < 2e-2, err


def test_engine_logits_band_and_graph_equals_eager():
    from bloomery_b200.models.cpu_ref import CpuModel
    spec, eng, wc = _tiny_engine(graphs=True)
    _, eng2, _ = _tiny_engine(graphs=False)
    cpu = CpuModel(wc)
    g = torch.Generator().manual_seed(12)
    prompt = torch.randint(0, spec.vocab, (19,), generator=g).tolist()
    ref = cpu.forward(torch.tensor(prompt))
    eng.prefill(0, prompt)
    eng2.prefill(0, prompt)
    n_last = len(prompt) % 8 or 8
    got = eng.logits[:n_last].cpu()
    want = ref[-n_last:]
    err = ((got - want).abs().max() / want.abs().max()).item()
    assert err < 2e-2, err
    assert torch.equal(eng.logits[:n_last], eng2.logits[:n_last])   # eager == replay, bit for bit
    # pass rows are independent: row bits equal the same token fed as a 1-row step
    eng.cut(0, len(prompt) - 1)
    eng.step([(0, prompt[-1], len(prompt) - 1)])
    assert torch.equal(eng.logits[0], eng2.logits[n_last - 1])


@pytest.mark.parametrize("scheme", ["fp8_b128", "nvfp4_modelopt"])
def test_engine_on_checkpoint_folder_logits_band(scheme, tmp_path):
    """A block-scaled safetensors folder loads into resident planes and decodes within the q8 band of the oracle."""
    from bloomery_b200.models import weights as W
    from bloomery_b200.models.cpu_ref import CpuModel
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_qwen3moe()
    spec.vocab = 4096
    W.write_folder(spec, str(tmp_path / "m"), scheme, seed=3)
    sp, wg, _ = W.open_model(str(tmp_path / "m"), DEV)
    _, wc, _ = W.open_model(str(tmp_path / "m"), "cpu")
    assert {"FP8_B128" if scheme == "fp8_b128" else "NVFP4", "BF16"} <= {q.qtype for q in wg.q.values()}
    eng = DecodeEngine(wg, n_slots=1, slot_ctx=256, use_graphs=True)
    g = torch.Generator().manual_seed(13)
    prompt = torch.randint(0, sp.vocab, (21,), generator=g).tolist()
    ref = CpuModel(wc).forward(torch.tensor(prompt))
    eng.prefill(0, prompt)
    n_last = len(prompt) % 8 or 8
    got, want = eng.logits[:n_last].cpu(), ref[-n_last:]
    err = ((got - want).abs().max() / ref.abs().max()).item()
    rms = ((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()).item()
    # 4-bit codes make a flipped q8 activation code weigh more than in the 8-bit schemes
    assert err < 6e-2 and rms < 2e-2, (err, rms)


def test_engine_fault_poisons_and_resets():
    from bloomery_b200.runtime.engine import EngineFault
    spec, eng, _ = _tiny_engine()
    with pytest.raises(EngineFault) as e:
        eng.step([(0, spec.vocab + 9, 0)])
    assert e.value.site == 1
    with pytest.raises(EngineFault):
        eng.step([(0, 1, 0)])                                  # poisoned until reset
    eng.reset_fault()
    eng.reset(0)
    assert len(eng.step([(0, 1, 0)])) == 1


def test_two_slots_one_pass():
    """Rows of different slots in one pass equal each slot stepped alone."""
    spec, eng, _ = _tiny_engine()
    a = [3, 99, 1234, 7]
    b = [500, 6, 42]
    eng.prefill(0, a)
    la = eng.logits[3].clone()
    eng.prefill(1, b)
    lb = eng.logits[2].clone()
    eng.reset(0); eng.reset(1)
    eng.prefill(0, a[:-1]); eng.prefill(1, b[:-1])
    eng.step([(0, a[-1], 3), (1, b[-1], 2)])
    assert torch.equal(eng.logits[0], la) and torch.equal(eng.logits[1], lb)


def test_two_pipeline_stages_equal_one_stage_bit_for_bit():
    """The stage axis: layers 0-1 and 2-3 as two engines with their own weights, KV and graphs (both on this GPU
    here), hidden rows copied across the boundary; picks and logits equal the one-stage engine's exactly."""
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import synth_tensors
    from bloomery_b200.parallel.pipeline import PipelineEngine, split_layers, stage_items
    spec, one, _ = _tiny_engine(graphs=True, n_slots=2)
    items = list(synth_tensors(spec, "cpu", seed=7))
    assert split_layers(48, 3, [1, 1, 2]) == [(0, 12), (12, 24), (24, 48)]
    pipe = PipelineEngine(spec, lambda lo, hi, f, l: stage_items(iter(items), spec, lo, hi, f, l), [DEV, DEV],
                          n_slots=2, slot_ctx=512, use_graphs=True)
    assert pipe.ranges == [(0, 2), (2, 4)] and "token_embd.weight" in pipe.stages[0].w.q
    assert not any(k.startswith("blk.3.") for k in pipe.stages[0].w.q) and pipe.stages[1].kv.k.shape[0] == 2
    g = torch.Generator().manual_seed(17)
    prompt = torch.randint(0, spec.vocab, (19,), generator=g).tolist()
    a, b = one.prefill(0, prompt, gemm=False), pipe.prefill(0, prompt)
    assert a == b
    n_last = len(prompt) % 8 or 8
    assert torch.equal(one.logits[:n_last], pipe.logits[:n_last])
    tok_a = tok_b = a
    for i in range(6):
        rows_a = [(0, tok_a, len(prompt) + i), (1, 5 + i, i)]
        pa, pb = one.step(rows_a), pipe.step([(0, tok_b, len(prompt) + i), (1, 5 + i, i)])
        assert pa == pb and torch.equal(one.logits[:2], pipe.logits[:2])
        tok_a, tok_b = pa[0], pb[0]
    pipe.cut(0, 10)
    one.cut(0, 10)
    assert one.step([(0, 7, 10)]) == pipe.step([(0, 7, 10)])


def test_overcommitted_kv_pool_spills_idle_slots_and_tokens_do_not_change():
    """Three slots of 256 positions over a pool of 6 pages (384 positions): the idle slot's pages go to pinned host
    memory when another slot needs them and come back when it runs again; every token equals the roomy engine's."""
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_qwen3moe()
    items = list(synth_tensors(spec, "cpu", seed=7))
    roomy = DecodeEngine(Weights.from_items(spec, iter(items), DEV), n_slots=3, slot_ctx=256, use_graphs=True)
    tight = DecodeEngine(Weights.from_items(spec, iter(items), DEV), n_slots=3, slot_ctx=256, use_graphs=True, kv_pages=6)
    g = torch.Generator().manual_seed(23)
    prompts = [torch.randint(0, spec.vocab, (n,), generator=g).tolist() for n in (150, 130, 100)]
    outs = {0: [], 1: []}
    for which, eng in enumerate((roomy, tight)):
        toks = [eng.prefill(sl, p, gemm=False) for sl, p in enumerate(prompts)]
        lens = [len(p) for p in prompts]
        for step in range(6):
            sl = step % 3                                    # one slot at a time: the others are idle and may spill
            toks[sl] = eng.step([(sl, toks[sl], lens[sl])])[0]
            lens[sl] += 1
            outs[which].append(toks[sl])
        outs[which] = toks + outs[which]
    assert outs[0] == outs[1]
    assert tight.kv.n_spills >= 2 and tight.kv.n_unspills >= 2 and roomy.kv.n_spills == 0


def _q8_rows(x):
    """q8_0 rows as the append launch writes them (scales first, then codes) and the f16 values they decode to."""
    n, hd = x.shape
    blk = x.float().reshape(n, hd // 32, 32)
    d = (blk.abs().amax(-1) / 127.0).half()
    df = d.float()
    q = torch.where(df[..., None] > 0, torch.round(blk / df[..., None].clamp_min(1e-30)), torch.zeros_like(blk)).clamp_(-127, 127)
    rows = torch.cat([d.view(torch.uint8).reshape(n, -1), q.to(torch.int8).view(torch.uint8).reshape(n, hd)], 1)
    return rows, (q * df[..., None]).reshape(n, hd).half()


@pytest.mark.parametrize("head,n_q,n_kv", [(128, 32, 4), (64, 8, 2), (128, 48, 4)])
def test_q8_0_kv_append_and_attention(head, n_q, n_kv):
    """Keys and values kept as q8_0 rows: the append launch writes the rows a plain PyTorch quantiser writes, and
    attention over them equals the f16 kernels over the decoded values."""
    from bloomery_b200.ops import decode as K
    torch.manual_seed(5)
    M, n_pages, max_pages, n_seg = 3, 40, 12, 5
    lens = [700, 65, 1]
    rb = head // 32 * 34
    kq = torch.zeros(n_pages, n_kv, 64, rb, dtype=torch.uint8, device=DEV)
    vq = torch.zeros_like(kq)
    kf = torch.zeros(n_pages, n_kv, 64, head, dtype=torch.float16, device=DEV)
    vf = torch.zeros_like(kf)
    table = torch.stack([torch.randperm(n_pages)[:max_pages] for _ in range(M)]).to(torch.int32).to(DEV)
    # fill the history of every row with random q8 rows (and their decoded f16 twins)
    for m, L in enumerate(lens):
        for pos in range(L - 1):
            page = int(table[m, pos // 64])
            for c, cf in ((kq, kf), (vq, vf)):
                rows, dec = _q8_rows(torch.randn(n_kv, head))
                c[page, :, pos % 64] = rows.to(DEV)
                cf[page, :, pos % 64] = dec.to(DEV)
    qkv = torch.randn(M, (n_q + 2 * n_kv) * head, device=DEV)
    gq, gk = 1 + 0.1 * torch.randn(head, device=DEV), 1 + 0.1 * torch.randn(head, device=DEV)
    inv = (1.0 / (1e6 ** (torch.arange(0, head, 2, dtype=torch.float64) / head))).float().to(DEV)
    pos = torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(M, dtype=torch.int32, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    outs = []
    for q8, kc, vc in ((True, kq, vq), (False, kf, vf)):
        q_out = torch.zeros(M, n_q, head, device=DEV)
        K.qk_norm_rope_append(qkv, gq, gk, inv, 1e-6, 1.0 / math.sqrt(head), head, n_q, n_kv, M, pos, seq, table, n_pages,
                              kc, vc, q_out, fault, 0, kv_q8=q8)
        if not q8:
            # the f16 twin gets the decoded values of the rows the q8 launch appended, so both caches hold the same numbers
            for m, L in enumerate(lens):
                page, off = int(table[m, (L - 1) // 64]), (L - 1) % 64
                for cq_, cf_ in ((kq, kf), (vq, vf)):
                    rows = cq_[page, :, off].cpu()
                    d = rows[:, :head // 16].contiguous().view(torch.float16).float()
                    codes = rows[:, head // 16:].contiguous().view(torch.int8).float().reshape(n_kv, head // 32, 32)
                    want_rows, _ = _q8_rows(cf_[page, :, off].float().cpu())
                    assert (rows[:, head // 16:].view(torch.int8).int() - want_rows[:, head // 16:].view(torch.int8).int()).abs().max() <= 1
                    cf_[page, :, off] = (codes * d[..., None]).reshape(n_kv, head).half().to(DEV)
        cells = M * n_q * n_seg
        out = torch.zeros(M, n_q * head, device=DEV)
        outq = torch.zeros(M, n_q * head, dtype=torch.int8, device=DEV)
        outds = torch.zeros(M, n_q * head // 32, 2, device=DEV)
        K.flash_decode(q_out, kc, vc, pos, seq, table, n_pages, head, n_q, n_kv, M, n_seg, max_pages * 64,
                       torch.zeros(cells * 2, device=DEV), torch.zeros(cells * head, device=DEV), out, outq, outds, fault, 0, kv_q8=q8)
        outs.append(out)
    torch.cuda.synchronize()
    assert (int(fault) & 0xFFFFFFFF) == 0xFFFFFFFF
    assert torch.allclose(outs[0], outs[1], rtol=1e-3, atol=1e-3), (outs[0] - outs[1]).abs().max()


def test_engine_with_q8_0_kv_stays_in_band_and_halves_the_cache():
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_qwen3moe()
    items = list(synth_tensors(spec, "cpu", seed=7))
    f16 = DecodeEngine(Weights.from_items(spec, iter(items), DEV), n_slots=1, slot_ctx=512)
    q8 = DecodeEngine(Weights.from_items(spec, iter(items), DEV), n_slots=1, slot_ctx=512, kv_type="q8_0")
    assert q8.kv.bytes * 64 == f16.kv.bytes * 34
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, spec.vocab, (90,), generator=g).tolist()
    a, b = f16.score(0, prompt), q8.score(0, prompt)
    n_last = len(prompt) % 8 or 8
    err = ((f16.logits[:n_last] - q8.logits[:n_last]).abs().max() / f16.logits[:n_last].abs().max()).item()
    assert err < 3e-2, err
    assert sum(int(x == y) for x, y in zip(a, b)) >= len(prompt) - 6
    assert q8.decode_chain(0, b[-1], len(prompt), 6) == q8.decode_chain(0, b[-1], len(prompt), 6)      # replay is stable
