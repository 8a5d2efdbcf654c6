"""Kernel micro-benchmark: each decode / prefill kernel alone at Qwen3-30B-A3B layer shapes, over a
few layers of random weights, replayed from a CUDA graph and timed with CUDA events.

    python -m bloomery_b200.ops.kernel_bench {all|qkv|o|router|gateup|gateup_ids|down|rope|flash|gemm|gemmdist|mla|sampler|gap|flash_mma} [replays] [context]

It is also the small workload the ncu summaries under ``profiles/`` were captured on.
"""
import sys

import torch
from bloomery_b200.ops import decode as K
from bloomery_b200.ops.decode import QWeight
from bloomery_b200.formats.resident import resident_row_bytes
dev = "cuda:0"
torch.manual_seed(0)
NL = 6
H, QR, KVR, E, I, k = 2048, 4096, 512, 128, 768, 8
def rw(rows, K_, t, stack=None):
    rb = resident_row_bytes(t, K_)
    shape = (rows, rb) if stack is None else (stack, rows, rb)
    d = torch.randint(0, 256, shape, dtype=torch.uint8, device=dev)
    return QWeight(d, t, K_)
layers = []
for l in range(NL):
    layers.append(dict(q=rw(QR, H, "Q4_K"), k=rw(KVR, H, "Q4_K"), v=rw(KVR, H, "Q6_K"), o=rw(H, QR, "Q4_K"),
                       r=QWeight((torch.randn(E, H, device=dev) * 0.05).view(torch.uint8).reshape(E, -1), "F32", H),
                       g=rw(I, H, "Q4_K", E), u=rw(I, H, "Q4_K", E), d=rw(H, I, "Q6_K", E)))
M = 1
x = torch.randn(8, H, device=dev); gain = torch.ones(H, device=dev)
qkv = torch.zeros(8, QR + 2 * KVR, device=dev)
xq = torch.zeros(8, QR, dtype=torch.int8, device=dev); xds = torch.ones(8, QR // 32, 2, device=dev)
fault = torch.full((1,), -1, dtype=torch.int32, device=dev)
logits = torch.zeros(8, E, device=dev); ids = torch.zeros(8, k, dtype=torch.int32, device=dev); wts = torch.zeros(8, k, device=dev)
hq = torch.zeros(8, H, dtype=torch.int8, device=dev); hds = torch.zeros(8, H // 32, 2, device=dev)
cnt = torch.zeros(1, dtype=torch.int32, device=dev)
actq = torch.zeros(8, k, I, dtype=torch.int8, device=dev); actds = torch.zeros(8, k, I // 32, 2, device=dev)
which = sys.argv[1] if len(sys.argv) > 1 else "all"
if which == "gateup_ids":
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(8)]).to(torch.int32).to(dev)
import math
n_q, n_kv, hd, ctx = 32, 4, 128, (int(sys.argv[3]) if len(sys.argv) > 3 else 4096)
n_pages = ctx // 64
kc = torch.randn(n_pages, n_kv, 64, hd, device=dev).half(); vc = torch.randn(n_pages, n_kv, 64, hd, device=dev).half()
table = torch.arange(n_pages, dtype=torch.int32, device=dev)[None].contiguous()
fpos = torch.tensor([ctx - 2], dtype=torch.int32, device=dev); fseq = torch.zeros(1, dtype=torch.int32, device=dev)
fq = torch.randn(8, n_q, hd, device=dev) / math.sqrt(hd)
n_seg = 37
pml = torch.zeros(8 * n_q * n_seg * 2, device=dev); pacc = torch.zeros(8 * n_q * n_seg * hd, device=dev)
if which == "gemm":
    from bloomery_b200.ops import gemm as G
    A = (torch.randn(4096, 2048, device=dev) * 0.1).bfloat16(); B = (torch.randn(5120, 2048, device=dev) * 0.1).bfloat16()
    C = torch.zeros(4096, 5120, device=dev, dtype=torch.bfloat16); tt = G.TileTable.dense(4096, dev); gst = torch.zeros(1, dtype=torch.int32, device=dev)
if which == "gemmdist":
    # the several-GPU epilogue on one GPU: o_proj-shaped product whose rows are added into two "owners" (both local here)
    from bloomery_b200.ops import gemm as G
    A = (torch.randn(4096, 4096, device=dev) * 0.1).bfloat16(); B = (torch.randn(2048, 4096, device=dev) * 0.1).bfloat16()
    own = [torch.zeros(2048, 2048, device=dev) for _ in range(2)]
    tt = G.TileTable.dense(4096, dev); gst = torch.zeros(1, dtype=torch.int32, device=dev)
if which == "mla":
    mq, mctx = 128, 4096
    mcache = torch.randn(mctx // 64, 64, 576, device=dev).half()
    mtable = torch.arange(mctx // 64, dtype=torch.int32, device=dev)[None].contiguous()
    mpos = torch.tensor([mctx - 2], dtype=torch.int32, device=dev); mseq = torch.zeros(1, dtype=torch.int32, device=dev)
    mqlat = torch.randn(8, mq, 576, device=dev) * 0.05
    mseg = 37
    mml = torch.zeros(8 * mq * mseg * 2, device=dev); macc = torch.zeros(8 * mq * mseg * 512, device=dev)
    mvb = (torch.randn(mq, 128, 512, device=dev) * 0.05).bfloat16()
    moq = torch.zeros(8, mq * 128, dtype=torch.int8, device=dev); mods = torch.zeros(8, mq * 128 // 32, 2, device=dev)
if which == "rope":
    r_inv = (1.0 / (1e6 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))).float().to(dev)
    r_g = torch.ones(hd, device=dev)
    r_q = torch.zeros(8, n_q, hd, device=dev)
    qkv.normal_()
if which == "sampler":
    V = 151936
    slog = torch.randn(1, V, device=dev) * 3
    spar = torch.tensor([[0.8, 40, 0.95, 0.05, 1.1, 0.0, 0.0, 64]], device=dev)
    ssd = torch.tensor([1234], dtype=torch.int64, device=dev); sdr = torch.zeros(1, dtype=torch.int64, device=dev)
    srec = torch.randint(0, V, (1, 64), dtype=torch.int32, device=dev); snrec = torch.tensor([64], dtype=torch.int32, device=dev)
    swork = torch.zeros(1, V, device=dev); sout = torch.zeros(1, dtype=torch.int32, device=dev)
if which == "flash_mma":
    K.set_flash_mma(True)
reps = int(sys.argv[2]) if len(sys.argv) > 2 else 4
def chain():
    for l in layers:
        if which in ("all", "qkv"): K.gemv([l["q"], l["k"], l["v"]], M, qkv, x=x, gain=gain, fault=fault)
        if which in ("all", "o"): K.gemv([l["o"]], M, x, xq=xq, xds=xds, resid=x, fault=fault)
        if which in ("all", "router"): K.router(x, gain, 1e-6, l["r"], M, logits, hq, hds, None, fault, 0)
        if which in ("all", "gateup"): K.gate_up_sel(hq, hds, ids, None, l["g"], l["u"], E, k, M, actq, actds, None, fault, 0, route_logits=logits, rule=K.RouteRule(k), wts=wts)
        if which == "gateup_ids": K.gate_up_sel(hq, hds, ids, None, l["g"], l["u"], E, k, M, actq, actds, None, fault, 0)
        if which == "rope": K.qk_norm_rope_append(qkv, r_g, r_g, r_inv, 1e-6, 1.0 / math.sqrt(hd), hd, n_q, n_kv, 1, fpos, fseq, table, n_pages, kc, vc, r_q, fault, 0)
        if which in ("all", "flash", "flash_mma"): K.flash_decode(fq, kc, vc, fpos, fseq, table, n_pages, hd, n_q, n_kv, 1, n_seg, ctx, pml, pacc, None, xq, xds, fault, 0)
        if which == "gemm": G.gemm_bf16(A, B, tt, out_bf16=C, status=gst)
        if which == "gemmdist": G.gemm_bf16_dist([A.data_ptr()], 4096, 4096, B, tt, owners=[o.data_ptr() for o in own], rows_per_owner=2048, ldc=2048, status=gst)
        if which == "mla": K.mla_flash_decode(mqlat, mcache, mpos, mseq, mtable, mctx // 64, mq, 1, mseg, mctx, mml, macc, mvb, 128, None, moq, mods, fault, 0)
        if which == "gap":
            for _ in range(8): K.fill_u32(cnt, 0)           # eight empty nodes: the number printed is 8 node gaps
        if which == "sampler": K.sample_rows(slog, V, 1, spar, ssd, sdr, sout, recent=srec, n_recent=snrec, work=swork)
        if which in ("all", "down"): K.down_combine(actq, actds, ids, wts, None, l["d"], E, k, M, x, None, x, fault, 0)
g = torch.cuda.CUDAGraph()
s = torch.cuda.Stream()
with torch.cuda.stream(s):
    chain(); s.synchronize()
    with torch.cuda.graph(g, stream=s):
        chain()
torch.cuda.synchronize()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
for _ in range(3): g.replay()
e0.record()
for _ in range(reps): g.replay()
e1.record(); torch.cuda.synchronize()
print(which, "us per layer-chain:", e0.elapsed_time(e1) * 1000 / reps / NL)
