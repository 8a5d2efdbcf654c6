"""Quantised-weight tcgen05 GEMM (weights expanded in flight) against torch fp32 matmul of the same dequantised
weights and bf16 activations."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _weight(t, shape, K, seed):
    from bloomery_b200.formats.resident import quantize_resident, resident_type
    from bloomery_b200.ops.decode import QWeight
    g = torch.Generator().manual_seed(seed)
    rows = 1
    for d in shape:
        rows *= d
    w = torch.randn(rows, K, generator=g) * 0.05
    res, ref = quantize_resident(w, t)
    return QWeight(res.to(DEV).reshape(*shape, -1).contiguous(), resident_type(t), K), ref.reshape(*shape, K).to(DEV)


@pytest.mark.parametrize("t", ["Q4_K", "Q5_K", "Q6_K", "Q8_0", "FP8_B128", "NVFP4", "IQ4_NL"])
@pytest.mark.parametrize("rows,tile", [(300, 128), (45, 32), (128, 128), (64, 64), (100, 64)])
def test_dense_qgemm(t, rows, tile):
    from bloomery_b200.ops import gemm as G
    N, K = 200, 1024                                            # N not a multiple of 128: the last weight tile is ragged
    qw, ref_w = _weight(t, (N,), K, 1)
    torch.manual_seed(2)
    X = (torch.randn(rows, K, device=DEV) * 0.5).bfloat16()
    R = torch.randn(rows, N, device=DEV)
    C = torch.full((rows, N), float("nan"), device=DEV)
    st = _status()
    tiles = G.TileTable.dense(rows, DEV, tile)
    G.qgemm(X, qw, tiles, out_f32=C, resid=R, status=st)
    torch.cuda.synchronize()
    assert int(st) == 0
    ref = X.float() @ ref_w.bfloat16().float().T + R
    # tiles below 128 tokens use the short expander (scale and offset of a block rounded to bf16 before the FMA)
    # (and NVFP4 rounds its group scale to bf16 at every tile size)
    tol = dict(rtol=1e-3, atol=1e-2) if tile == 128 and t != "NVFP4" else dict(rtol=1e-2, atol=3e-2)
    assert torch.allclose(C, ref, **tol), (C - ref).abs().max()
    C2 = torch.zeros_like(C)
    G.qgemm(X, qw, tiles, out_f32=C2, resid=R, status=st)
    assert torch.equal(C, C2)                                   # bit-identical rerun


@pytest.mark.parametrize("gt,dt", [("Q4_K", "Q6_K"), ("FP8_B128", "FP8_B128"), ("NVFP4", "NVFP4")])
@pytest.mark.parametrize("tile,T", [(128, 700), (32, 24)])
def test_grouped_dual_swiglu_and_scatter_quantised(tile, T, gt, dt):
    """The MoE path on quantised experts: rows grouped by expert, gate/up fused with SwiGLU (Q4_K), down (Q6_K)
    scattered with the router weights; prompt-sized tiles and decode-batch tiles."""
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(3)
    E, k, H, I_ = 8, 2, 512, 256
    wg, ref_g = _weight(gt, (E, I_), H, 4)
    wu, ref_u = _weight(gt, (E, I_), H, 5)
    wd, ref_d = _weight(dt, (E, H), I_, 6)
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    ids[5, 1] = -1
    wts = torch.rand(T, k, device=DEV)
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    n = T * k
    cap = n + 128
    pos_of = torch.zeros(n, dtype=torch.int32, device=DEV)
    dst_row = torch.zeros(cap, dtype=torch.int32, device=DEV)
    row_scale = torch.zeros(cap, device=DEV)
    tiles = G.TileTable(n, E, DEV, tile)
    G.moe_plan(ids, wts, E, tiles, pos_of, dst_row, row_scale)
    Ap = torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV)
    G.gather_rows_bf16(x, dst_row, tiles.offsets[E:E + 1], cap, k, Ap)
    act = torch.zeros(cap, I_, dtype=torch.bfloat16, device=DEV)
    st = _status()
    G.qgemm(Ap, wg, tiles, out_bf16=act, W2=wu, status=st)
    slot_out = torch.zeros(n, H, device=DEV)
    G.qgemm(act, wd, tiles, out_f32=slot_out, dst_row=dst_row, row_scale=row_scale, status=st)
    resid = torch.randn(T, H, device=DEV)
    y = torch.zeros(T, H, device=DEV)
    G.moe_combine(slot_out, pos_of, T, k, resid, y)
    torch.cuda.synchronize()
    assert int(st) == 0
    ref = resid.clone()
    xf = x.float()
    Wg, Wu, Wd = ref_g.bfloat16().float(), ref_u.bfloat16().float(), ref_d.bfloat16().float()
    for t_ in range(T):
        for j in range(k):
            e = int(ids[t_, j])
            if e < 0:
                continue
            a = (torch.nn.functional.silu(xf[t_] @ Wg[e].T) * (xf[t_] @ Wu[e].T)).bfloat16().float()
            ref[t_] += wts[t_, j] * (a @ Wd[e].T)
    assert torch.allclose(y, ref, rtol=2e-2, atol=2e-2), (y - ref).abs().max()


def _fp8_acts(X):
    """Device quantisation of bf16 rows and the fp32 values the codes stand for."""
    from bloomery_b200.formats.planes import e4m3_decode
    from bloomery_b200.ops import gemm as G
    rows, K = X.shape
    codes = torch.zeros(rows, K, dtype=torch.uint8, device=DEV)
    scales = torch.zeros(rows, K // 128, device=DEV)
    G.fp8_rows(X, codes, scales)
    vals = e4m3_decode(codes.cpu()).to(DEV).reshape(rows, K // 128, 128) * scales[:, :, None]
    return codes, scales, vals.reshape(rows, K)


def test_fp8_rows_quantise_within_half_a_step_and_fuse_the_norm():
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(11)
    X = (torch.randn(37, 1024, device=DEV) * torch.rand(37, 1, device=DEV) * 3).bfloat16()
    X[3, 128:256] = 0                                            # an all-zero block keeps scale 1 and codes 0
    codes, scales, vals = _fp8_acts(X)
    amax = X.float().reshape(37, 8, 128).abs().amax(-1)
    assert torch.allclose(scales, torch.where(amax > 0, amax / 448, torch.ones_like(amax)), rtol=1e-6)
    err = (vals - X.float()).abs().reshape(37, 8, 128)
    # E4M3 keeps 3 mantissa bits: half a step is 1/16 of the value's power of two, at most 1/16 of the block maximum
    assert bool((err <= amax[:, :, None] / 16 * 1.001 + 1e-12).all())
    assert int(codes[3, 128:256].max()) == 0
    xf = torch.randn(5, 512, device=DEV)
    gain = torch.rand(512, device=DEV) + 0.5
    c2 = torch.zeros(5, 512, dtype=torch.uint8, device=DEV)
    s2 = torch.zeros(5, 4, device=DEV)
    G.fp8_rows(xf, c2, s2, gain=gain, eps=1e-6)
    normed = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * gain
    assert torch.allclose(s2, normed.reshape(5, 4, 128).abs().amax(-1) / 448, rtol=1e-4)


@pytest.mark.parametrize("rows", [45, 32, 7])
def test_fp8_block_scaled_dense_gemm(rows):
    from bloomery_b200.ops import gemm as G
    N, K = 200, 1024                                            # N not a multiple of 128: the last weight tile is ragged
    qw, ref_w = _weight("FP8_B128", (N,), K, 1)
    torch.manual_seed(2)
    X = (torch.randn(rows, K, device=DEV) * 0.5).bfloat16()
    codes, scales, xv = _fp8_acts(X)
    R = torch.randn(rows, N, device=DEV)
    C = torch.full((rows, N), float("nan"), device=DEV)
    st = _status()
    tiles = G.TileTable.dense(rows, DEV, 32)
    G.fp8_gemm(codes, scales, qw, tiles, out_f32=C, resid=R, status=st)
    torch.cuda.synchronize()
    assert int(st) == 0
    ref = xv.double() @ ref_w.double().T + R.double()            # the quantised operands' own values, exact products
    assert torch.allclose(C.double(), ref, rtol=1e-4, atol=1e-4), (C.double() - ref).abs().max()
    C2 = torch.zeros_like(C)
    G.fp8_gemm(codes, scales, qw, tiles, out_f32=C2, resid=R, status=st)
    assert torch.equal(C, C2)
    plain = X.float() @ ref_w.T + R                               # and the activation rounding stays a small error
    assert float((C - plain).abs().max()) < 0.05 * float(plain.abs().max())


def test_fp8_block_scaled_grouped_dual_and_scatter():
    from bloomery_b200.ops import gemm as G
    torch.manual_seed(3)
    E, k, H, I_, T = 8, 2, 512, 256, 24
    wg, ref_g = _weight("FP8_B128", (E, I_), H, 4)
    wu, ref_u = _weight("FP8_B128", (E, I_), H, 5)
    wd, ref_d = _weight("FP8_B128", (E, H), I_, 6)
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    ids[5, 1] = -1
    wts = torch.rand(T, k, device=DEV)
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    n = T * k
    cap = n + 128
    pos_of = torch.zeros(n, dtype=torch.int32, device=DEV)
    dst_row = torch.zeros(cap, dtype=torch.int32, device=DEV)
    row_scale = torch.zeros(cap, device=DEV)
    tiles = G.TileTable(n, E, DEV, 32)
    G.moe_plan(ids, wts, E, tiles, pos_of, dst_row, row_scale)
    Ap = torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV)
    G.gather_rows_bf16(x, dst_row, tiles.offsets[E:E + 1], cap, k, Ap)
    ac, asc, _ = _fp8_acts(Ap)
    act = torch.zeros(cap, I_, dtype=torch.bfloat16, device=DEV)
    st = _status()
    G.fp8_gemm(ac, asc, wg, tiles, out_bf16=act, W2=wu, status=st)
    bc, bsc, _ = _fp8_acts(act)
    slot_out = torch.zeros(n, H, device=DEV)
    G.fp8_gemm(bc, bsc, wd, tiles, out_f32=slot_out, dst_row=dst_row, row_scale=row_scale, status=st)
    resid = torch.randn(T, H, device=DEV)
    y = torch.zeros(T, H, device=DEV)
    G.moe_combine(slot_out, pos_of, T, k, resid, y)
    torch.cuda.synchronize()
    assert int(st) == 0
    ref = resid.clone()
    xf = x.float()
    for t_ in range(T):
        for j in range(k):
            e = int(ids[t_, j])
            if e < 0:
                continue
            a = torch.nn.functional.silu(xf[t_] @ ref_g[e].T) * (xf[t_] @ ref_u[e].T)
            ref[t_] += wts[t_, j] * (a @ ref_d[e].T)
    # activations rounded to E4M3 twice (in front of gate / up and in front of down): a few percent of the expert sum
    assert float((y - ref).abs().max()) < 0.06 * float((ref - resid).abs().max()) + 1e-3, (y - ref).abs().max()
