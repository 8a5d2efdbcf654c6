"""Kernel micro-benchmark: each decode / prefill kernel alone (or the whole per-layer decode chain) at
Qwen3-30B-A3B layer shapes, over a few layers of random weights, replayed from a CUDA graph and timed with
CUDA events.

    python -m bloomery_b200.ops.kernel_bench NAME [replays] [context] [--no-staged] [--rows M]

NAME: chain (the six launches of a layer in order) | qkv | attn | o | router | gateup | down | rope | flash |
flash_mma | gemm | gemmdist | pflash | prope | mplan | qgu | qdown | qo | qq | bgu | bdown | mla | sampler | sampler_split | gap.  ``--no-staged`` runs the register-streaming kernels
instead of the shared-memory staged ones.  It is also the small workload the ncu summaries under ``profiles/``
were captured on.
"""
import math
import sys

NL = 6
H, QR, KVR, E, I, TOPK = 2048, 4096, 512, 128, 768, 8


def main(argv=None) -> int:
    import torch
    from bloomery_b200.ops import decode as K
    from bloomery_b200.ops.decode import QWeight
    from bloomery_b200.formats.resident import resident_row_bytes

    argv = list(sys.argv[1:] if argv is None else argv)
    staged = "--no-staged" not in argv
    rows = 1
    if "--rows" in argv:
        i = argv.index("--rows")
        rows = int(argv[i + 1])
        del argv[i:i + 2]
    global TOPK
    if "--topk" in argv:
        i = argv.index("--topk")
        TOPK = int(argv[i + 1])
        del argv[i:i + 2]
    wtype = None                       # --wtype T: the expert stacks of every layer in resident type T (e.g. FP8_B128, NVFP4)
    if "--wtype" in argv:
        i = argv.index("--wtype")
        wtype = argv[i + 1]
        del argv[i:i + 2]
    if "--dbg" in argv:
        i = argv.index("--dbg")
        from bloomery_b200.ops._lib import cuda
        import ctypes
        cuda().bl_set_stage_debug(ctypes.c_int(int(argv[i + 1])))
        print("stage debug flags", argv[i + 1])
        del argv[i:i + 2]
    probe = None
    if "--probe" in argv:
        argv.remove("--probe")
        probe = torch.zeros(16, dtype=torch.int64, device="cuda:0")
    argv = [a for a in argv if a != "--no-staged"]
    which = argv[0] if argv else "chain"
    if which in ("fgu", "fdown"):
        wtype = "FP8_B128"             # f* = FP8 weights against E4M3 activations on the tensor cores (no expansion)
    reps = int(argv[1]) if len(argv) > 1 else 4
    ctx = int(argv[2]) if len(argv) > 2 else 4096
    K.set_staged(staged)
    dev = "cuda:0"
    torch.manual_seed(0)
    M = rows

    def rw(n_rows, k_, t, stack=None):
        rb = resident_row_bytes(t, k_)
        shape = (n_rows, rb) if stack is None else (stack, n_rows, rb)
        return QWeight(torch.randint(0, 256, shape, dtype=torch.uint8, device=dev), t, k_)

    layers = []
    for _ in range(NL):
        layers.append(dict(q=rw(QR, H, "Q4_K"), k=rw(KVR, H, "Q4_K"), v=rw(KVR, H, "Q6_K"), o=rw(H, QR, "Q4_K"),
                           r=QWeight((torch.randn(E, H, device=dev) * 0.05).view(torch.uint8).reshape(E, -1), "F32", H),
                           g=rw(I, H, wtype or "Q4_K", E), u=rw(I, H, wtype or "Q4_K", E), d=rw(H, I, wtype or "Q6_K", E)))
    x = torch.randn(8, H, device=dev)
    gain = torch.ones(H, device=dev)
    qkv = torch.randn(8, QR + 2 * KVR, device=dev)
    xq = torch.zeros(8, QR, dtype=torch.int8, device=dev)
    xds = torch.ones(8, QR // 32, 2, device=dev)
    fault = torch.full((1,), -1, dtype=torch.int32, device=dev)
    logits = torch.zeros(8, E, device=dev)
    # distinct experts per row, so the expert launches stream eight different matrices as a real step does
    ids = torch.stack([torch.randperm(E)[:TOPK] for _ in range(8)]).to(torch.int32).to(dev)
    wts = torch.full((8, TOPK), 1.0 / TOPK, device=dev)
    hq = torch.zeros(8, H, dtype=torch.int8, device=dev)
    hds = torch.zeros(8, H // 32, 2, device=dev)
    cnt = torch.zeros(1, dtype=torch.int32, device=dev)
    actq = torch.zeros(8, TOPK, I, dtype=torch.int8, device=dev)
    actds = torch.zeros(8, TOPK, I // 32, 2, device=dev)
    tickets = torch.zeros(64, dtype=torch.int32, device=dev)
    n_q, n_kv, hd = 32, 4, 128
    n_pages = (ctx + 63) // 64
    kc = torch.randn(n_pages, n_kv, 64, hd, device=dev).half()
    vc = torch.randn(n_pages, n_kv, 64, hd, device=dev).half()
    table = torch.arange(n_pages, dtype=torch.int32, device=dev)[None].contiguous()
    fpos = torch.full((8,), ctx - 2, dtype=torch.int32, device=dev)
    fseq = torch.zeros(8, dtype=torch.int32, device=dev)
    fq = torch.randn(8, n_q, hd, device=dev) / math.sqrt(hd)
    n_seg = 37
    pml = torch.zeros(8 * n_q * n_seg * 2, device=dev)
    pacc = torch.zeros(8 * n_q * n_seg * hd, device=dev)
    r_inv = (1.0 / (1e6 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))).float().to(dev)
    r_g = torch.ones(hd, device=dev)
    r_q = torch.zeros(8, n_q, hd, device=dev)
    rule = K.RouteRule(TOPK)
    cparts = torch.zeros(TOPK, H, device=dev)
    x2 = torch.zeros(8, H, device=dev)
    extra = {}
    if which == "gemm":
        from bloomery_b200.ops import gemm as G
        extra = dict(G=G, A=(torch.randn(4096, 2048, device=dev) * 0.1).bfloat16(), B=(torch.randn(5120, 2048, device=dev) * 0.1).bfloat16(),
                     C=torch.zeros(4096, 5120, device=dev, dtype=torch.bfloat16), tt=G.TileTable.dense(4096, dev),
                     gst=torch.zeros(1, dtype=torch.int32, device=dev))
    if which == "pflash":
        # prompt flash attention of `ctx` tokens (32 query heads over 4 key/value heads of 128)
        from bloomery_b200.ops import gemm as G
        tp = (ctx + 127) // 128 * 128
        extra = dict(G=G, pq=(torch.randn(n_q, ctx, hd, device=dev) * 0.3).bfloat16(), pk=(torch.randn(n_kv, tp, hd, device=dev)).bfloat16(),
                     pv=(torch.randn(n_kv, hd, tp, device=dev)).bfloat16(), po=torch.zeros(ctx, n_q * hd, device=dev, dtype=torch.bfloat16),
                     gst=torch.zeros(1, dtype=torch.int32, device=dev))
    if which == "prope":
        # prompt RMSNorm + RoPE + KV append of `ctx` rows
        from bloomery_b200.ops import gemm as G
        extra = dict(G=G, rqkv=torch.randn(ctx, (n_q + 2 * n_kv) * hd, device=dev), rpos=torch.arange(ctx, dtype=torch.int32, device=dev),
                     rseq=torch.zeros(ctx, dtype=torch.int32, device=dev), rqb=torch.zeros(n_q, ctx, hd, device=dev, dtype=torch.bfloat16))
    if which == "mplan":
        # routed-slot plan (count, offsets, tile table, scatter) of `ctx` tokens x 8 experts of 128
        from bloomery_b200.ops import gemm as G
        n = ctx * TOPK
        extra = dict(G=G, mids=torch.stack([torch.randperm(E, device=dev)[:TOPK] for _ in range(ctx)]).to(torch.int32).contiguous(),
                     mwts=torch.rand(ctx, TOPK, device=dev), mtt=G.TileTable(n, E, dev), mpos_of=torch.zeros(n, dtype=torch.int32, device=dev),
                     mdst=torch.zeros(n + 128, dtype=torch.int32, device=dev), mscale=torch.zeros(n + 128, device=dev))
    if which in ("qgu", "qdown", "bgu", "bdown", "fgu", "fdown"):
        # expert products of `ctx` tokens x 8 experts of 128: q* = quantised weights expanded inside the GEMM,
        # b* = expansion launch + bf16 GEMM; --rows picks the token tile (32 or 128) of the q* forms
        from bloomery_b200.ops import gemm as G
        n = ctx * TOPK
        tr = 32 if rows == 32 or which[0] == "f" else 128
        mids = torch.stack([torch.randperm(E, device=dev)[:TOPK] for _ in range(ctx)]).to(torch.int32).contiguous()
        tt = G.TileTable(n, E, dev, tr if which[0] in "qf" else 128)
        dst = torch.zeros(n + 128, dtype=torch.int32, device=dev)
        scale = torch.zeros(n + 128, device=dev)
        G.moe_plan(mids, torch.rand(ctx, TOPK, device=dev), E, tt, torch.zeros(n, dtype=torch.int32, device=dev), dst, scale)
        extra = dict(G=G, tt=tt, dst=dst, scale=scale, gst=torch.zeros(1, dtype=torch.int32, device=dev),
                     xa=(torch.randn(n + 128, H, device=dev) * 0.3).bfloat16(), act=torch.zeros(n + 128, I, device=dev, dtype=torch.bfloat16),
                     so=torch.zeros(n, H, device=dev), wg=torch.zeros(E, I, H, device=dev, dtype=torch.bfloat16),
                     wu=torch.zeros(E, I, H, device=dev, dtype=torch.bfloat16), wd=torch.zeros(E, H, I, device=dev, dtype=torch.bfloat16))
        if which[0] == "f":
            extra.update(xa8=torch.randint(0, 120, (n + 128, H), dtype=torch.uint8, device=dev), xas=torch.rand(n + 128, H // 128, device=dev),
                         act8=torch.randint(0, 120, (n + 128, I), dtype=torch.uint8, device=dev), acts=torch.rand(n + 128, I // 128, device=dev))
        M = 1
    if which in ("qo", "qq"):
        # dense products of a decode batch of --rows tokens (one tile): o projection / q projection, weights quantised
        from bloomery_b200.ops import gemm as G
        tr = 64 if rows > 32 else 32
        extra = dict(G=G, tt=G.TileTable.dense(rows, dev, tr), gst=torch.zeros(1, dtype=torch.int32, device=dev),
                     xo=(torch.randn(rows, QR, device=dev) * 0.3).bfloat16(), xh=(torch.randn(rows, H, device=dev) * 0.3).bfloat16(),
                     oo=torch.zeros(rows, H, device=dev), oq=torch.zeros(rows, QR, device=dev))
        M = 1
    if which == "gemmdist":
        # the several-GPU epilogue on one GPU: o_proj-shaped product whose rows are added into two "owners" (both local here)
        from bloomery_b200.ops import gemm as G
        extra = dict(G=G, A=(torch.randn(4096, 4096, device=dev) * 0.1).bfloat16(), B=(torch.randn(2048, 4096, device=dev) * 0.1).bfloat16(),
                     own=[torch.zeros(2048, 2048, device=dev) for _ in range(2)], tt=G.TileTable.dense(4096, dev),
                     gst=torch.zeros(1, dtype=torch.int32, device=dev))
    if which == "mla":
        mq, mctx, mseg = 128, 4096, 37
        extra = dict(mq=mq, mctx=mctx, mseg=mseg, mcache=torch.randn(mctx // 64, 64, 576, device=dev).half(),
                     mtable=torch.arange(mctx // 64, dtype=torch.int32, device=dev)[None].contiguous(),
                     mpos=torch.tensor([mctx - 2], dtype=torch.int32, device=dev), mseq=torch.zeros(1, dtype=torch.int32, device=dev),
                     mqlat=torch.randn(8, mq, 576, device=dev) * 0.05, mml=torch.zeros(8 * mq * mseg * 2, device=dev),
                     macc=torch.zeros(8 * mq * mseg * 512, device=dev), mvb=(torch.randn(mq, 128, 512, device=dev) * 0.05).bfloat16(),
                     moq=torch.zeros(8, mq * 128, dtype=torch.int8, device=dev), mods=torch.zeros(8, mq * 128 // 32, 2, device=dev))
    if which in ("sampler", "sampler_split"):
        V = 151936
        extra = dict(V=V, slog=torch.randn(1, V, device=dev) * 3, spar=torch.tensor([[0.8, 40, 0.95, 0.05, 1.1, 0.0, 0.0, 64]], device=dev),
                     ssd=torch.tensor([1234], dtype=torch.int64, device=dev), sdr=torch.zeros(1, dtype=torch.int64, device=dev),
                     srec=torch.randint(0, V, (1, 64), dtype=torch.int32, device=dev), snrec=torch.tensor([64], dtype=torch.int32, device=dev),
                     swork=torch.zeros(1, V, device=dev), sout=torch.zeros(1, dtype=torch.int32, device=dev))
    if which == "flash_mma":
        K.set_flash_mma(True)
    X = extra

    def attn(l):
        if which == "attn_cluster" or (staged and which == "chain2"):
            K.attn_cluster(qkv, r_g, r_g, r_inv, 1e-6, 1.0 / math.sqrt(hd), hd, n_q, n_kv, M, fpos, fseq, table, n_pages, kc, vc,
                           K.attn_cluster_size(n_kv, M) or 8, ctx, None, xq, xds, fault, 0)
        elif staged:
            K.attn_fused(qkv, r_g, r_g, r_inv, 1e-6, 1.0 / math.sqrt(hd), hd, n_q, n_kv, M, fpos, fseq, table, n_pages, kc, vc,
                         n_seg, ctx, pml, pacc, tickets, None, xq, xds, fault, 0)
        else:
            K.qk_norm_rope_append(qkv, r_g, r_g, r_inv, 1e-6, 1.0 / math.sqrt(hd), hd, n_q, n_kv, M, fpos, fseq, table, n_pages,
                                  kc, vc, r_q, fault, 0)
            K.flash_decode(r_q, kc, vc, fpos, fseq, table, n_pages, hd, n_q, n_kv, M, n_seg, ctx, pml, pacc, None, xq, xds, fault, 0)

    def router(l):
        if which == "router_ticket":
            K.router(x, gain, 1e-6, l["r"], M, logits, hq, hds, None, fault, 0, rule=rule, ids=ids, wts=wts, ticket=tickets[40:])
        else:
            K.router(x, gain, 1e-6, l["r"], M, logits, hq, hds, None, fault, 0)

    def gateup(l, routed=True):
        if staged and routed:
            K.gate_up_staged(hq, hds, ids, None, l["g"], l["u"], E, TOPK, M, actq, actds, None, fault, 0, down=l["d"],
                             route_logits=logits, rule=rule, wts=wts)
        elif staged:
            K.gate_up_staged(hq, hds, ids, None, l["g"], l["u"], E, TOPK, M, actq, actds, None, fault, 0, down=l["d"])
        elif routed:
            K.gate_up_sel(hq, hds, ids, None, l["g"], l["u"], E, TOPK, M, actq, actds, None, fault, 0, route_logits=logits, rule=rule, wts=wts)
        else:
            K.gate_up_sel(hq, hds, ids, None, l["g"], l["u"], E, TOPK, M, actq, actds, None, fault, 0)

    def down(l):
        (K.down_staged if staged else K.down_combine)(actq, actds, ids, wts, None, l["d"], E, TOPK, M, x, None, x, fault, 0)

    def chain():
        for l in layers:
            if which in ("chain", "chain2", "qkv"): K.gemv([l["q"], l["k"], l["v"]], M, qkv, x=x, gain=gain, fault=fault)
            if which in ("chain", "chain2", "attn", "attn_cluster"): attn(l)
            if which in ("chain", "chain2", "o"): K.gemv([l["o"]], M, x, xq=xq, xds=xds, resid=x, fault=fault)
            if which in ("chain", "chain2", "router", "router_ticket"): router(l)
            if which in ("chain", "chain2", "gateup"): gateup(l)
            if which == "gateup_ids": gateup(l, routed=False)
            if which in ("chain", "chain2", "down"): down(l)
            if which in ("cluster", "chain_cluster"):
                if which == "chain_cluster":
                    K.gemv([l["q"], l["k"], l["v"]], M, qkv, x=x, gain=gain, fault=fault)
                    attn(l)
                    K.gemv([l["o"]], M, x, xq=xq, xds=xds, resid=x, fault=fault)
                K.moe_cluster(x, gain, 1e-6, l["r"], rule, None, l["g"], l["u"], l["d"], TOPK, None, cparts, tickets[44:], x2,
                              logits, ids, wts, None, fault, 0)
            if which == "rope": K.qk_norm_rope_append(qkv, r_g, r_g, r_inv, 1e-6, 1.0 / math.sqrt(hd), hd, n_q, n_kv, 1, fpos, fseq, table, n_pages, kc, vc, r_q, fault, 0)
            if which in ("flash", "flash_mma"): K.flash_decode(fq, kc, vc, fpos, fseq, table, n_pages, hd, n_q, n_kv, 1, n_seg, ctx, pml, pacc, None, xq, xds, fault, 0)
            if which == "gemm": X["G"].gemm_bf16(X["A"], X["B"], X["tt"], out_bf16=X["C"], status=X["gst"])
            if which == "pflash": X["G"].flash_prefill(X["pq"], X["pk"], X["pv"], X["po"], 0, X["gst"])
            if which == "prope": X["G"].qk_norm_rope_append_prefill(X["rqkv"], r_g, r_g, r_inv, 1e-6, 1.0 / math.sqrt(hd), hd, n_q, n_kv, ctx, X["rpos"], X["rseq"], table, n_pages, kc, vc, X["rqb"], fault, 0)
            if which == "mplan": X["G"].moe_plan(X["mids"], X["mwts"], E, X["mtt"], X["mpos_of"], X["mdst"], X["mscale"])
            if which == "qo": X["G"].qgemm(X["xo"], l["o"], X["tt"], out_f32=X["oo"], status=X["gst"])
            if which == "qq": X["G"].qgemm(X["xh"], l["q"], X["tt"], out_f32=X["oq"], status=X["gst"])
            if which == "qgu": X["G"].qgemm(X["xa"], l["g"], X["tt"], out_bf16=X["act"], W2=l["u"], status=X["gst"])
            if which == "qdown": X["G"].qgemm(X["act"], l["d"], X["tt"], out_f32=X["so"], dst_row=X["dst"], row_scale=X["scale"], status=X["gst"])
            if which == "fgu": X["G"].fp8_gemm(X["xa8"], X["xas"], l["g"], X["tt"], out_bf16=X["act"], W2=l["u"], status=X["gst"])
            if which == "fdown": X["G"].fp8_gemm(X["act8"], X["acts"], l["d"], X["tt"], out_f32=X["so"], dst_row=X["dst"], row_scale=X["scale"], status=X["gst"])
            if which == "bgu":
                X["G"].dequant_bf16(l["g"], X["wg"]); X["G"].dequant_bf16(l["u"], X["wu"])
                X["G"].gemm_bf16(X["xa"], X["wg"], X["tt"], out_bf16=X["act"], B2=X["wu"], status=X["gst"])
            if which == "bdown":
                X["G"].dequant_bf16(l["d"], X["wd"])
                X["G"].gemm_bf16(X["act"], X["wd"], X["tt"], out_f32=X["so"], dst_row=X["dst"], row_scale=X["scale"], status=X["gst"])
            if which == "gemmdist": X["G"].gemm_bf16_dist([X["A"].data_ptr()], 4096, 4096, X["B"], X["tt"], owners=[o.data_ptr() for o in X["own"]], rows_per_owner=2048, ldc=2048, status=X["gst"])
            if which == "mla": K.mla_flash_decode(X["mqlat"], X["mcache"], X["mpos"], X["mseq"], X["mtable"], X["mctx"] // 64, X["mq"], 1, X["mseg"], X["mctx"], X["mml"], X["macc"], X["mvb"], 128, None, X["moq"], X["mods"], fault, 0)
            if which == "gap":
                for _ in range(8): K.fill_u32(cnt, 0)           # eight empty nodes: the number printed is 8 node gaps
            if which == "sampler": K.sample_rows(X["slog"], X["V"], 1, X["spar"], X["ssd"], X["sdr"], X["sout"], recent=X["srec"], n_recent=X["snrec"], work=X["swork"], split=False)
            if which == "sampler_split": K.sample_rows(X["slog"], X["V"], 1, X["spar"], X["ssd"], X["sdr"], X["sout"], recent=X["srec"], n_recent=X["snrec"], work=X["swork"], split=True, cap=40)

    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        chain()
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            chain()
    torch.cuda.synchronize()
    if probe is not None:
        # one eager pass of the last layer with the phase probe armed: cycles between the marks of block (0, 0, 0)
        from bloomery_b200.ops._lib import cuda
        import ctypes
        g.replay()
        cuda().bl_set_stage_probe(ctypes.c_void_p(probe.data_ptr()))
        with torch.cuda.stream(s):
            chain()
            s.synchronize()
        cuda().bl_set_stage_probe(ctypes.c_void_p(0))
        marks = probe.cpu().tolist()
        live = [m for m in marks if m]
        print("probe cycles between marks:", [b - a for a, b in zip(live, live[1:])])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        g.replay()
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    word = int(fault.cpu().item()) & 0xFFFFFFFF
    print(which, "staged" if staged else "streaming", f"rows={M} ctx={ctx}", "us per layer:", round(e0.elapsed_time(e1) * 1000 / reps / NL, 2),
          "fault word:", hex(word))
    return 0


if __name__ == "__main__":
    sys.exit(main())
