"""The shared-memory staged decode kernels (csrc/decode_staged.cu): bit-equal to the register-streaming kernels
where both compute the same sums, and against a plain PyTorch fp32 reference for the fused attention launch."""
import math

import pytest
import torch

from bloomery_b200.formats import quant as Q

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _qw(w, t):
    from bloomery_b200.formats.resident import quantize_resident
    from bloomery_b200.ops.decode import QWeight
    res, wd = quantize_resident(w.reshape(-1, w.shape[-1]), t)
    res = res.to(DEV)
    if w.dim() == 3:
        res = res.reshape(w.shape[0], w.shape[1], -1)
    return QWeight(res, t, w.shape[-1]), wd.reshape(w.shape)


@pytest.fixture(autouse=True)
def _staged_on():
    from bloomery_b200.ops import decode as K
    K.set_staged(True)
    K.set_staged_parts("gemv,attn,moe,prefetch,cluster")
    yield
    K.set_staged(True)
    K.set_staged_parts("attn,prefetch")


@pytest.mark.parametrize("M", [1, 2, 5, 8])
@pytest.mark.parametrize("types", [("Q4_K", "Q4_K", "Q6_K"), ("Q8_0",), ("Q5_K", "Q6_K"), ("NVFP4", "FP8_B128"), ("Q3_K", "Q5_0", "Q2_K")])
def test_staged_gemv_equals_streaming_bits(M, types):
    from bloomery_b200.ops import decode as K
    torch.manual_seed(0)
    Kd = 2048
    rows = [517, 130, 66, 40][:len(types)]
    segs = [_qw(torch.randn(r, Kd) * 0.02, t)[0] for r, t in zip(rows, types)]
    width = sum(rows)
    x = torch.randn(M, Kd, device=DEV)
    gain = (1 + 0.1 * torch.randn(Kd)).to(DEV)
    resid = torch.randn(M, width, device=DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    outs = []
    for on in (True, False):
        K.set_staged(on)
        o = torch.zeros(M, width, device=DEV)
        K.gemv(segs, M, o, x=x, gain=gain, eps=1e-6, resid=resid, fault=fault)
        outs.append(o)
    assert torch.equal(outs[0], outs[1])
    assert int(fault) == -1
    # q8 rows in, no norm
    c, ds = Q.quantize_act_q8(x.cpu())
    outs = []
    for on in (True, False):
        K.set_staged(on)
        o = torch.zeros(M, width, device=DEV)
        K.gemv(segs, M, o, xq=c.to(DEV), xds=ds.to(DEV), fault=fault)
        outs.append(o)
    assert torch.equal(outs[0], outs[1])


def test_staged_gemv_o_proj_shape_and_fallback_for_big_matrices():
    from bloomery_b200.ops import decode as K
    torch.manual_seed(1)
    a, ad = _qw(torch.randn(2048, 4096) * 0.02, "Q4_K")
    x = torch.randn(3, 4096)
    c, ds = Q.quantize_act_q8(x)
    out = torch.zeros(3, 2048, device=DEV)
    K.gemv([a], 3, out, xq=c.to(DEV), xds=ds.to(DEV))
    ref = (Q.dequantize_act_q8(c, ds).double() @ ad.double().T).float()
    assert ((out.cpu() - ref).abs().max() / ref.abs().max()).item() < 1e-5
    # a matrix far beyond the stage (a vocabulary-sized head) silently takes the streaming kernel
    big, bd = _qw(torch.randn(60000, 1024) * 0.02, "Q6_K")
    x = torch.randn(1, 1024)
    gain = torch.ones(1024)
    o = torch.zeros(1, 60000, device=DEV)
    K.gemv([big], 1, o, x=x.to(DEV), gain=gain.to(DEV), eps=1e-6)
    assert torch.isfinite(o).all()


def _attn_case(head, n_q, n_kv, rows, n_seg, ctx, seed=5, qk_norm=True, cluster=0):
    """rows = [(seq, position)]; history of every sequence is random f16 rows below its first position in the pass."""
    from bloomery_b200.models.cpu_ref import rms_norm, rope_neox
    from bloomery_b200.ops import decode as K
    torch.manual_seed(seed)
    M = len(rows)
    n_seq = max(s for s, _ in rows if s >= 0) + 1
    max_pages = (ctx + 63) // 64
    n_pages = n_seq * max_pages + 3
    width = (n_q + 2 * n_kv) * head
    qkv = torch.randn(M, width)
    qg, kg = 1 + 0.1 * torch.randn(head), 1 + 0.1 * torch.randn(head)
    inv = (1.0 / (1e6 ** (torch.arange(0, head, 2, dtype=torch.float64) / head))).float()
    perm = torch.randperm(n_pages)
    table = torch.stack([perm[s * max_pages:(s + 1) * max_pages] for s in range(n_seq)]).to(torch.int32)
    kc = torch.zeros(n_pages, n_kv, 64, head, dtype=torch.float16)
    vc = torch.zeros(n_pages, n_kv, 64, head, dtype=torch.float16)
    first = {}
    for s, p in rows:
        if s >= 0:
            first[s] = min(first.get(s, p), p)
    hist_k = {s: torch.randn(n, n_kv, head).half() for s, n in first.items()}
    hist_v = {s: torch.randn(n, n_kv, head).half() for s, n in first.items()}
    for s, n in first.items():
        for t in range(n):
            pg = int(table[s, t // 64])
            kc[pg, :, t % 64] = hist_k[s][t]
            vc[pg, :, t % 64] = hist_v[s][t]
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32)
    seq = torch.tensor([s for s, _ in rows], dtype=torch.int32)
    d = lambda t: t.to(DEV)
    kc_d, vc_d = d(kc), d(vc)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    part_ml = torch.full((M * n_q * n_seg * 2,), float("nan"), device=DEV)      # poisoned scratch: nothing stale may be read
    part_acc = torch.full((M * n_q * n_seg * head,), float("nan"), device=DEV)
    tickets = torch.zeros(M * n_kv, dtype=torch.int32, device=DEV)
    out = torch.full((M, n_q * head), float("nan"), device=DEV)
    outq = torch.zeros(M, n_q * head, dtype=torch.int8, device=DEV)
    outds = torch.zeros(M, n_q * head // 32, 2, device=DEV)
    for _ in range(2):                              # twice: the tickets must come back to zero by themselves
        if cluster:
            K.attn_cluster(d(qkv), d(qg) if qk_norm else None, d(kg) if qk_norm else None, d(inv), 1e-6, 1 / math.sqrt(head),
                           head, n_q, n_kv, M, d(pos), d(seq), d(table), n_pages, kc_d, vc_d, cluster, ctx, out, outq, outds,
                           fault, 0)
            continue
        K.attn_fused(d(qkv), d(qg) if qk_norm else None, d(kg) if qk_norm else None, d(inv), 1e-6, 1 / math.sqrt(head), head,
                     n_q, n_kv, M, d(pos), d(seq), d(table), n_pages, kc_d, vc_d, n_seg, ctx, part_ml, part_acc, tickets,
                     out, outq, outds, fault, 0)
    assert int(tickets.abs().sum()) == 0
    q = qkv[:, :n_q * head].reshape(M, n_q, head)
    k = qkv[:, n_q * head:(n_q + n_kv) * head].reshape(M, n_kv, head)
    v = qkv[:, (n_q + n_kv) * head:].reshape(M, n_kv, head)
    ppos = pos.clamp(min=0)
    qr = rope_neox(rms_norm(q, qg, 1e-6) if qk_norm else q, ppos, inv) / math.sqrt(head)
    kr = rope_neox(rms_norm(k, kg, 1e-6) if qk_norm else k, ppos, inv)
    G = n_q // n_kv
    for m, (s, p) in enumerate(rows):
        if s < 0:
            assert float(out[m].abs().max()) == 0.0 and int(outq[m].abs().max()) == 0
            continue
        keys = [hist_k[s].float()]
        vals = [hist_v[s].float()]
        mine = sorted((pp, mm) for mm, (ss, pp) in enumerate(rows) if ss == s and pp <= p)
        assert [pp for pp, _ in mine] == list(range(first[s], p + 1)), "the case must append consecutive positions"
        for pp, mm in mine:
            keys.append(kr[mm].half().float()[None])
            vals.append(v[mm].half().float()[None])
        keys, vals = torch.cat(keys, 0), torch.cat(vals, 0)
        sc = torch.einsum("hd,shd->hs", qr[m], keys.repeat_interleave(G, 1))
        ref = torch.einsum("hs,shd->hd", torch.softmax(sc, -1), vals.repeat_interleave(G, 1)).reshape(-1)
        assert torch.allclose(out[m].cpu(), ref, rtol=2e-3, atol=2e-3), (m, (out[m].cpu() - ref).abs().max())
        pg, off = int(table[s, p // 64]), p % 64
        assert torch.allclose(kc_d[pg, :, off].cpu().float(), kr[m].half().float(), atol=2e-3, rtol=2e-3)
        assert torch.allclose(vc_d[pg, :, off].cpu().float(), v[m].half().float(), atol=1e-3, rtol=1e-3)
    live = [m for m, (s, _) in enumerate(rows) if s >= 0]
    c, ds = Q.quantize_act_q8(out[live].cpu())
    assert (outq[live].cpu() != c).float().mean() < 1e-3
    assert torch.allclose(outds[live].cpu(), ds, rtol=1e-4, atol=1e-6)
    assert int(fault) == -1
    return out


@pytest.mark.parametrize("head,n_q,n_kv", [(128, 32, 4), (64, 8, 2), (128, 64, 4)])
def test_attn_fused_rows_of_different_sequences(head, n_q, n_kv):
    # one key, a few tiles, many tiles; a padding row in between
    _attn_case(head, n_q, n_kv, [(0, 0), (1, 332), (-1, 0), (2, 699)], n_seg=9, ctx=704)


def test_attn_fused_rows_of_one_sequence_see_each_other():
    # a prompt pass: eight consecutive positions of one sequence, straddling a key tile and a page
    _attn_case(128, 32, 4, [(0, 60 + i) for i in range(8)], n_seg=5, ctx=256)
    _attn_case(128, 32, 4, [(0, i) for i in range(8)], n_seg=5, ctx=256, seed=6)        # from an empty cache
    _attn_case(64, 8, 2, [(1, 100 + i) for i in range(3)] + [(0, 31 + i) for i in range(3)], n_seg=3, ctx=192, seed=7)


@pytest.mark.parametrize("cluster", [8, 16])
@pytest.mark.parametrize("head,n_q,n_kv", [(128, 32, 4), (64, 8, 2), (128, 64, 4)])
def test_attn_cluster_form(head, n_q, n_kv, cluster):
    """Key segments over a thread-block cluster, merged through distributed shared memory."""
    if cluster == 16 and n_kv * 4 > 12:
        pytest.skip("more 16-CTA clusters than one B200 holds at once")
    _attn_case(head, n_q, n_kv, [(0, 0), (1, 332), (-1, 0), (2, 699)], n_seg=9, ctx=704, cluster=cluster)
    _attn_case(head, n_q, n_kv, [(0, 60 + i) for i in range(3)], n_seg=5, ctx=256, cluster=cluster, seed=8)


def test_attn_fused_without_qk_norm_and_with_one_segment():
    _attn_case(128, 8, 2, [(0, 200), (1, 17)], n_seg=1, ctx=256, qk_norm=False)


def test_attn_fused_bad_key_count_is_a_fault_word_not_a_trap():
    from bloomery_b200.ops import decode as K
    head, n_q, n_kv, M, n_seg, ctx = 128, 8, 2, 2, 4, 128
    d = DEV
    qkv = torch.randn(M, (n_q + 2 * n_kv) * head, device=d)
    inv = torch.ones(head // 2, device=d)
    table = torch.arange(4, dtype=torch.int32, device=d).reshape(2, 2)
    kc = torch.zeros(4, n_kv, 64, head, dtype=torch.float16, device=d)
    vc = torch.zeros_like(kc)
    pos = torch.tensor([5, ctx + 9], dtype=torch.int32, device=d)
    seq = torch.tensor([0, 1], dtype=torch.int32, device=d)
    fault = torch.full((1,), -1, dtype=torch.int32, device=d)
    out = torch.zeros(M, n_q * head, device=d)
    outq = torch.zeros(M, n_q * head, dtype=torch.int8, device=d)
    outds = torch.zeros(M, n_q * head // 32, 2, device=d)
    K.attn_fused(qkv, None, None, inv, 1e-6, 1.0, head, n_q, n_kv, M, pos, seq, table, 4, kc, vc, n_seg, ctx,
                 torch.zeros(M * n_q * n_seg * 2, device=d), torch.zeros(M * n_q * n_seg * head, device=d),
                 torch.zeros(M * n_kv, dtype=torch.int32, device=d), out, outq, outds, fault, 3)
    assert (int(fault) & 0xFFFFFFFF) == (3 << 8 | 5)
    assert torch.isnan(out[1]).all() and not torch.isnan(out[0]).any()


@pytest.mark.parametrize("gt,dt", [("Q4_K", "Q6_K"), ("Q8_0", "Q8_0"), ("NVFP4", "NVFP4"), ("Q5_K", "Q4_K")])
def test_staged_experts_equal_streaming_bits_and_router_routes(gt, dt):
    from bloomery_b200.ops import decode as K
    from bloomery_b200.ops.decode import QWeight, RouteRule
    torch.manual_seed(3)
    H, I, E, k, M = 1024, 512, 16, 4, 3
    gate, _ = _qw(torch.randn(E, I, H) * 0.03, gt)
    up, _ = _qw(torch.randn(E, I, H) * 0.03, gt)
    down, _ = _qw(torch.randn(E, H, I) * 0.03, dt)
    rw = torch.randn(E, H) * 0.05
    rq = QWeight(rw.contiguous().view(torch.uint8).reshape(E, -1).to(DEV), "F32", H)
    x = torch.randn(M, H, device=DEV)
    gain = (1 + 0.1 * torch.randn(H)).to(DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    rule = RouteRule(k)
    logits = torch.zeros(M, E, device=DEV)
    xq = torch.zeros(M, H, dtype=torch.int8, device=DEV)
    xds = torch.zeros(M, H // 32, 2, device=DEV)
    ids = torch.full((M, k), -7, dtype=torch.int32, device=DEV)
    wts = torch.zeros(M, k, device=DEV)
    heat = torch.zeros(E, dtype=torch.int32, device=DEV)
    ticket = torch.zeros(4, dtype=torch.int32, device=DEV)
    for _ in range(2):
        K.router(x, gain, 1e-6, rq, M, logits, xq, xds, None, fault, 0, rule=rule, ids=ids, wts=wts, heat=heat, ticket=ticket)
    assert int(ticket.abs().sum()) == 0 and int(heat.sum()) == 2 * M * k
    ids2 = torch.zeros_like(ids)
    wts2 = torch.zeros_like(wts)
    K.route_rows(logits, rule, M, ids2, wts2, None, fault, 0)
    assert torch.equal(ids, ids2) and torch.equal(wts, wts2)
    slot_map = torch.arange(E, dtype=torch.int32)
    slot_map[int(ids[0, 1])] = -1                      # one chosen expert lives elsewhere: its slot contributes nothing
    res = []
    for on in (True, False):
        K.set_staged(on)
        actq = torch.zeros(M, k, I, dtype=torch.int8, device=DEV)
        actds = torch.zeros(M, k, I // 32, 2, device=DEV)
        out = torch.zeros(M, H, device=DEV)
        sm = slot_map.to(DEV)
        if on:
            # routed inside the launch (warp 0): the ids and weights it publishes equal the router launch's
            ids3 = torch.full_like(ids, -9)
            wts3 = torch.zeros_like(wts)
            K.gate_up_staged(xq, xds, ids3, sm, gate, up, E, k, M, actq, actds, None, fault, 0, down=down, route_logits=logits,
                             rule=rule, wts=wts3)
            assert torch.equal(ids3, ids) and torch.equal(wts3, wts)
            K.down_staged(actq, actds, ids3, wts3, sm, down, E, k, M, x, None, out, fault, 0)
        else:
            K.gate_up_sel(xq, xds, ids, sm, gate, up, E, k, M, actq, actds, None, fault, 0)
            K.down_combine(actq, actds, ids, wts, sm, down, E, k, M, x, None, out, fault, 0)
        res.append((actq, actds, out))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    assert torch.equal(res[0][2], res[1][2])
    assert int(fault) == -1
    # an id beyond the expert count: fault word + NaN for that row, the other rows stay finite
    bad = ids.clone()
    bad[1, 0] = E + 2
    out = torch.zeros(M, H, device=DEV)
    actq = torch.zeros(M, k, I, dtype=torch.int8, device=DEV)
    actds = torch.zeros(M, k, I // 32, 2, device=DEV)
    K.set_staged(True)
    K.gate_up_staged(xq, xds, bad, None, gate, up, E, k, M, actq, actds, None, fault, 2, down=down)
    K.down_staged(actq, actds, bad, wts, None, down, E, k, M, x, None, out, fault, 2)
    assert (int(fault) & 0xFFFFFFFF) == (2 << 8 | 4)
    assert torch.isnan(out[1]).all() and not torch.isnan(out[0]).any()


@pytest.mark.parametrize("gt,dt,H,I,E,k", [("Q4_K", "Q6_K", 2048, 768, 128, 8), ("Q8_0", "Q8_0", 512, 256, 16, 4),
                                            ("NVFP4", "NVFP4", 1024, 512, 32, 6), ("Q5_K", "Q4_K", 1024, 512, 64, 8)])
def test_moe_cluster_launch_equals_the_three_launch_chain(gt, dt, H, I, E, k):
    """Router + routing + experts + combine of one row as ONE cluster launch: same picks and weights, the new residual
    row within float rounding of the chain's (the down projection is summed per slot before it is weighted)."""
    from bloomery_b200.ops import decode as K
    from bloomery_b200.ops.decode import QWeight, RouteRule
    torch.manual_seed(11)
    gate, _ = _qw(torch.randn(E, I, H) * 0.03, gt)
    up, _ = _qw(torch.randn(E, I, H) * 0.03, gt)
    down, _ = _qw(torch.randn(E, H, I) * 0.03, dt)
    rw = torch.randn(E, H) * 0.05
    rq = QWeight(rw.contiguous().view(torch.uint8).reshape(E, -1).to(DEV), "F32", H)
    if not K.moe_cluster_fits(rq, gate, up, down, k):
        pytest.skip("this device cannot hold one 16-CTA cluster per chosen expert")
    x = torch.randn(1, H, device=DEV)
    gain = (1 + 0.1 * torch.randn(H)).to(DEV)
    fault = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    rule = RouteRule(k)
    # the chain
    logits = torch.zeros(1, E, device=DEV)
    xq = torch.zeros(1, H, dtype=torch.int8, device=DEV)
    xds = torch.zeros(1, H // 32, 2, device=DEV)
    ids = torch.zeros(1, k, dtype=torch.int32, device=DEV)
    wts = torch.zeros(1, k, device=DEV)
    actq = torch.zeros(1, k, I, dtype=torch.int8, device=DEV)
    actds = torch.zeros(1, k, I // 32, 2, device=DEV)
    ref = torch.zeros(1, H, device=DEV)
    K.router(x, gain, 1e-6, rq, 1, logits, xq, xds, None, fault, 0)
    K.gate_up_sel(xq, xds, ids, None, gate, up, E, k, 1, actq, actds, None, fault, 0, route_logits=logits, rule=rule, wts=wts)
    K.down_combine(actq, actds, ids, wts, None, down, E, k, 1, x, None, ref, fault, 0)
    # the cluster launch, twice (its tickets must return to zero by themselves), on poisoned scratch
    parts = torch.full((k, H), float("nan"), device=DEV)
    tickets = torch.zeros(16, dtype=torch.int32, device=DEV)
    out = torch.full((1, H), float("nan"), device=DEV)
    lg2 = torch.zeros(1, E, device=DEV)
    ids2 = torch.full((1, k), -9, dtype=torch.int32, device=DEV)
    wts2 = torch.zeros(1, k, device=DEV)
    heat = torch.zeros(E, dtype=torch.int32, device=DEV)
    for _ in range(2):
        K.moe_cluster(x, gain, 1e-6, rq, rule, None, gate, up, down, k, None, parts, tickets, out, lg2, ids2, wts2, heat, fault, 0)
    assert int(fault) == -1 and int(tickets.abs().sum()) == 0 and int(heat.sum()) == 2 * k
    assert torch.equal(lg2, logits) and torch.equal(ids2, ids) and torch.equal(wts2, wts)
    scale = ref.abs().max().item()
    assert (out - ref).abs().max().item() < 2e-5 * max(scale, 1.0), (out - ref).abs().max().item()
    # one chosen expert lives elsewhere (slot map -1): its slot adds nothing; an extra addend rides along
    sm = torch.arange(E, dtype=torch.int32)
    sm[int(ids[0, 2])] = -1
    extra = torch.randn(1, H, device=DEV)
    K.gate_up_sel(xq, xds, ids, sm.to(DEV), gate, up, E, k, 1, actq, actds, None, fault, 0)
    K.down_combine(actq, actds, ids, wts, sm.to(DEV), down, E, k, 1, x, extra, ref, fault, 0)
    K.moe_cluster(x, gain, 1e-6, rq, rule, sm.to(DEV), gate, up, down, k, extra, parts, tickets, out, lg2, ids2, wts2, heat, fault, 0)
    assert (out - ref).abs().max().item() < 2e-5 * max(ref.abs().max().item(), 1.0)
    assert int(fault) == -1


def test_engine_tokens_do_not_depend_on_the_kernel_form():
    """Greedy tokens of the tiny model: staged kernels == streaming kernels (both under CUDA graphs)."""
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.ops import decode as K
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_qwen3moe()
    w = Weights.from_items(spec, synth_tensors(spec, DEV, seed=0), DEV)
    prompt = [(7 * i + 3) % spec.vocab for i in range(37)]
    toks = []
    for on in (True, False):
        K.set_staged(on)
        K.set_staged_parts("gemv,attn,moe,prefetch")       # the cluster launch sums the down rows in another order
        eng = DecodeEngine(w, n_slots=1, slot_ctx=256)
        first = eng.prefill(0, prompt, gemm=False)
        toks.append([first] + eng.decode_chain(0, first, len(prompt), 24))
    assert toks[0] == toks[1]
