"""tcgen05 / TMEM / TMA grouped GEMM against torch fp32 matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 512), (300, 768, 2048), (1000, 5120, 2048), (77, 2048, 768)])
def test_dense_gemm_f32_out(M, N, K):
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(0)
    A = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.5).bfloat16()
    C = torch.full((M, N), float("nan"), device=DEV)
    st = _status()
    G.gemm_bf16(A, B, G.TileTable.dense(M, DEV), out_f32=C, status=st)
    torch.cuda.synchronize()
    assert int(st) == 0
    ref = A.float() @ B.float().T
    assert torch.allclose(C, ref, rtol=1e-3, atol=1e-2), (C - ref).abs().max()


def test_dense_gemm_bf16_out_resid_and_rerun():
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(1)
    M, N, K = 513, 2048, 4096
    A = (torch.randn(M, K, device=DEV) * 0.1).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    R = torch.randn(M, N, device=DEV)
    C = torch.zeros(M, N, device=DEV)
    st = _status()
    tiles = G.TileTable.dense(M, DEV)
    G.gemm_bf16(A, B, tiles, out_f32=C, resid=R, status=st)
    ref = A.float() @ B.float().T + R
    assert torch.allclose(C, ref, rtol=1e-3, atol=2e-2)
    C2 = torch.zeros_like(C)
    G.gemm_bf16(A, B, tiles, out_f32=C2, resid=R, status=st)
    assert torch.equal(C, C2)                                   # bit-identical rerun
    Cb = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    G.gemm_bf16(A, B, tiles, out_bf16=Cb, status=st)
    assert torch.allclose(Cb.float(), (A.float() @ B.float().T), rtol=2e-2, atol=5e-2)
    assert int(st) == 0


def test_grouped_dual_swiglu_and_scatter():
    """The MoE prompt path: rows grouped by expert, gate/up fused with SwiGLU, down scattered with weights."""
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(2)
    E, H, I_, T, k = 8, 512, 256, 200, 2
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    ids[5, 1] = -1                                              # a slot served elsewhere
    wts = torch.rand(T, k, device=DEV)
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    Wg = (torch.randn(E, I_, H, device=DEV) * 0.1).bfloat16()
    Wu = (torch.randn(E, I_, H, device=DEV) * 0.1).bfloat16()
    Wd = (torch.randn(E, H, I_, device=DEV) * 0.1).bfloat16()
    n = T * k
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    cursor = torch.zeros(E, dtype=torch.int32, device=DEV)
    pos_of = torch.zeros(n, dtype=torch.int32, device=DEV)
    cap = n + 128
    dst_row = torch.full((cap,), -1, dtype=torch.int32, device=DEV)
    row_scale = torch.zeros(cap, device=DEV)
    tiles = G.TileTable(n, E, DEV)
    dst_row.fill_(7)                                            # the plan must clear the padding rows itself
    G.moe_plan(ids, wts, E, tiles, pos_of, dst_row, row_scale)
    torch.cuda.synchronize()
    flat = ids.flatten().cpu()
    cnt = torch.bincount(flat[flat >= 0], minlength=E)
    off = torch.cat([torch.zeros(1, dtype=torch.long), cnt.cumsum(0)])
    assert tiles.offsets.cpu().tolist() == off.tolist()
    want_tiles = [(e, int(off[e]) + r, int(off[e + 1])) for e in range(E) for r in range(0, int(cnt[e]), 128)]
    nmt = int(tiles.n_mtiles.item())
    assert nmt == len(want_tiles)
    assert [tuple(r[:3]) for r in tiles.mtiles.view(-1, 4)[:nmt].cpu().tolist()] == want_tiles
    dr = dst_row.cpu()
    assert (dr[int(off[E]):] == -1).all()
    for e in range(E):                                          # each expert's rows hold exactly its slots
        assert sorted(dr[int(off[e]):int(off[e + 1])].tolist()) == (flat == e).nonzero().flatten().tolist()
    po = pos_of.cpu()
    assert (po[flat < 0] == -1).all() and (dr[po[flat >= 0].long()] == (flat >= 0).nonzero().flatten()).all()
    Ap = torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV)
    G.gather_rows_bf16(x, dst_row, tiles.offsets[E:E + 1], cap, k, Ap)
    act = torch.zeros(cap, I_, dtype=torch.bfloat16, device=DEV)
    st = _status()
    G.gemm_bf16(Ap, Wg, tiles, out_bf16=act, B2=Wu, status=st)
    slot_out = torch.zeros(n, H, device=DEV)
    G.gemm_bf16(act, Wd, tiles, out_f32=slot_out, dst_row=dst_row, row_scale=row_scale, status=st)
    resid = torch.randn(T, H, device=DEV)
    y = torch.zeros(T, H, device=DEV)
    G.moe_combine(slot_out, pos_of, T, k, resid, y)
    torch.cuda.synchronize()
    assert int(st) == 0
    ref = resid.clone()
    xf = x.float()
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            if e < 0:
                continue
            g = xf[t] @ Wg[e].float().T
            u = xf[t] @ Wu[e].float().T
            a = (torch.nn.functional.silu(g) * u).bfloat16().float()
            ref[t] += wts[t, j] * (a @ Wd[e].float().T)
    assert torch.allclose(y, ref, rtol=2e-2, atol=2e-2), (y - ref).abs().max()


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K", "Q6_K", "Q8_0"])
def test_dequant_bf16_matches_oracle(t):
    from bloomery_b200.formats import quant as Q
    from bloomery_b200.formats.resident import to_resident
    from bloomery_b200.ops import gemm as G
    from bloomery_b200.ops.decode import QWeight
    torch.manual_seed(3)
    w = torch.randn(3, 40, 512) * 0.02
    raw = Q.quantize(w.reshape(-1, 512), t)
    qw = QWeight(to_resident(raw, t, 512).to(DEV).reshape(3, 40, -1), t, 512)
    out = G.dequant_bf16(qw)
    ref = Q.dequantize(raw, t, 512).reshape(3, 40, 512).bfloat16()
    assert torch.equal(out.cpu(), ref)


def test_rmsnorm_bf16():
    from bloomery_b200.models.cpu_ref import rms_norm
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(4)
    x = torch.randn(37, 2048, device=DEV)
    g = 1 + 0.1 * torch.randn(2048, device=DEV)
    out = torch.zeros(37, 2048, dtype=torch.bfloat16, device=DEV)
    G.rmsnorm_bf16(x, g, 1e-6, out)
    ref = rms_norm(x.cpu(), g.cpu(), 1e-6)
    assert torch.allclose(out.float().cpu(), ref, rtol=1e-2, atol=1e-2)


def test_gemm_prefill_matches_pass_path_in_band():
    """The GEMM prompt path against the 8-row pass path of the same engine: logits in a band,
    KV rows close, and decode continues from either."""
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.runtime.engine import DecodeEngine
    spec = tiny_qwen3moe()
    w = Weights.from_items(spec, synth_tensors(spec, DEV, seed=3), DEV)
    eng = DecodeEngine(w, n_slots=2, slot_ctx=1024)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, spec.vocab, (333,), generator=g).tolist()
    t_pass = eng.prefill(0, prompt, gemm=False)
    l_pass = eng.logits[(len(prompt) - 1) % 8].clone()
    t_gemm = eng.prefill(1, prompt, gemm=True)
    l_gemm = eng.logits[0].clone()
    err = ((l_pass - l_gemm).abs().max() / l_pass.abs().max()).item()
    assert err < 5e-2, err
    k0 = eng.kv.k[:, eng.kv.pages[0][0]].float()
    k1 = eng.kv.k[:, eng.kv.pages[1][0]].float()
    assert ((k0 - k1).abs().mean() / k0.abs().mean()).item() < 3e-2      # bf16 operands vs q8 operands
    # second micro-batch on top of the first (keys of both are attended)
    more = torch.randint(0, spec.vocab, (100,), generator=g).tolist()
    eng.prefill(0, more, start=len(prompt), gemm=False)
    l2_pass = eng.logits[(len(more) - 1) % 8].clone()
    eng.prefill(1, more, start=len(prompt), gemm=True)
    l2_gemm = eng.logits[0].clone()
    assert ((l2_pass - l2_gemm).abs().max() / l2_pass.abs().max()).item() < 5e-2
    assert len(eng.decode_chain(1, t_gemm, len(prompt) + len(more), 4)) == 4


def test_split_precision_router_logits_are_fp32_grade():
    from bloomery_b200.models.cpu_ref import rms_norm
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(6)
    T, H, E = 300, 2048, 128
    x = torch.randn(T, H, device=DEV) * 3
    g = 1 + 0.1 * torch.randn(H, device=DEV)
    W = torch.randn(E, H, device=DEV) * 0.05
    a3 = torch.zeros(T, 3 * H, dtype=torch.bfloat16, device=DEV)
    G.rmsnorm_hilo(x, g, 1e-6, a3)
    logits = torch.zeros(T, E, device=DEV)
    st = _status()
    G.gemm_bf16(a3, G.hilo_weights(W), G.TileTable.dense(T, DEV), out_f32=logits, status=st)
    ref = (rms_norm(x.cpu(), g.cpu(), 1e-6).double() @ W.cpu().double().T).float()
    err = ((logits.cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err < 2e-4 and int(st) == 0, err                     # plain bf16 operands would sit near 1e-2


@pytest.mark.parametrize("heads,Tq,pos0,T_pad", [(2, 128, 0, 128), (3, 256, 1000, 4096), (2, 384, 3700, 4096),
                                                (1, 128, 8100, 8320)])
def test_softmax_causal_rows(heads, Tq, pos0, T_pad):
    """Causal softmax of score rows (head-major) against torch fp32: masked keys exactly 0 inside the written span;
    covers the register path with every run in use and the re-reading path of rows longer than 8,192 keys."""
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(7)
    rows = heads * Tq
    S = torch.randn(rows, T_pad, device=DEV) * 4.0
    P = torch.full((rows, T_pad), float("nan"), device=DEV, dtype=torch.bfloat16)
    G.softmax_causal(S, rows, Tq, pos0, T_pad, P)
    torch.cuda.synchronize()
    tq = torch.arange(rows, device=DEV) % Tq
    n_valid = torch.clamp(pos0 + tq + 1, max=T_pad)
    col = torch.arange(T_pad, device=DEV)
    mask = col[None, :] < n_valid[:, None]
    ref = torch.softmax(S.masked_fill(~mask, float("-inf")), dim=-1)
    last = torch.clamp((tq | 127), max=Tq - 1)
    n_write = torch.clamp((pos0 + last + 1 + 63) // 64 * 64, max=T_pad)
    wr = col[None, :] < n_write[:, None]
    got = P.float()
    assert not torch.isnan(got[wr]).any()
    assert torch.all(got[wr & ~mask] == 0)
    assert torch.allclose(got[wr], ref[wr], rtol=1e-2, atol=1e-5), (got[wr] - ref[wr]).abs().max()
    assert torch.allclose(got.masked_fill(~wr, 0).sum(-1), torch.ones(rows, device=DEV), atol=2e-2)


@pytest.mark.parametrize("n_kv,head,n_keys,T_pad", [(2, 128, 200, 256), (4, 128, 64, 128), (1, 64, 321, 384)])
def test_kv_gather_rows_and_transposed_values(n_kv, head, n_keys, T_pad):
    """Paged f16 cache -> contiguous bf16 keys [n_kv, T_pad, head] and transposed values [n_kv, head, T_pad]
    through a shuffled block table; positions past the last key are zero."""
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(3)
    n_pages = 12
    k_cache = torch.randn(n_pages, n_kv, 64, head, device=DEV).half()
    v_cache = torch.randn(n_pages, n_kv, 64, head, device=DEV).half()
    table = torch.randperm(n_pages, device=DEV)[: (T_pad + 63) // 64].to(torch.int32).contiguous()
    Kb = torch.full((n_kv, T_pad, head), float("nan"), device=DEV, dtype=torch.bfloat16)
    Vt = torch.full((n_kv, head, T_pad), float("nan"), device=DEV, dtype=torch.bfloat16)
    G.kv_gather_bf16(k_cache, v_cache, table, n_pages, n_kv, head, n_keys, T_pad, Kb, Vt)
    torch.cuda.synchronize()
    t = torch.arange(T_pad, device=DEV)
    pages = table.long()[t // 64]
    k_ref = k_cache[pages, :, t % 64].permute(1, 0, 2).float()          # [n_kv, T_pad, head]
    v_ref = v_cache[pages, :, t % 64].permute(1, 0, 2).float()
    k_ref[:, n_keys:] = 0
    v_ref[:, n_keys:] = 0
    assert torch.equal(Kb.float(), k_ref.bfloat16().float())
    assert torch.equal(Vt.float(), v_ref.bfloat16().float().transpose(1, 2))
