"""N-GPU arm of ``bench.py``: the same single-request decode, heads and experts sharded over
the ranks, reductions fused into the kernels.  Timed on the device, max over ranks."""
from __future__ import annotations

import json
import time

import torch
import torch.distributed as dist

from . import dist as D
from .sharded import ShardedEngine, local_spec, shard_items


def run_batch_distributed(args, rank: int, local: int, world: int) -> int:
    """``--batch B`` on N GPUs: B sequences per pass, experts split over the ranks, rows and attention replicated."""
    from bench import METRIC, ClockSampler
    from ..models.spec import NAMED
    from ..models.weights import Weights, synth_tensors
    from .batch_dist import ShardedBatchDecode
    D.init("nccl")
    dev = f"cuda:{local}"
    spec = NAMED[args.model]()
    mix = getattr(args, "mix", "") or "Q4_K_M"
    B, steps, warm = args.batch, args.steps, max(3, args.warmup)
    t0 = time.time()
    lspec = local_spec(spec, world, attn=False)
    w = Weights.from_items(lspec, synth_tensors(spec, dev, seed=0, mix=mix, shard=(rank, world), shard_attn=False), dev)
    torch.cuda.synchronize()
    t_load = time.time() - t0
    ctx = (args.prompt + warm + 2 * steps + 64 + 63) // 64 * 64
    eng = ShardedEngine(w, spec, rank, world, fused=True, n_slots=B, slot_ctx=ctx, use_graphs=True, attn_replicated=True)
    eng.gemm_threshold = 0
    bd = ShardedBatchDecode(eng, rank, world, max_rows=max(16, B))
    g = torch.Generator().manual_seed(1234)
    rows = []
    dist.barrier()
    t0 = time.time()
    for slot in range(B):
        prompt = torch.randint(0, spec.vocab, (args.prompt,), generator=g).tolist()
        rows.append((slot, bd.prefill(slot, prompt), args.prompt))     # passes of up to 64 positions of the one sequence
    torch.cuda.synchronize()
    t_prompts = time.time() - t0
    for slot in range(B):
        eng.kv.ensure(slot, args.prompt + warm + 2 * steps + 8)
    M = bd.set_rows(rows)
    bd.counters[2:3].zero_()
    dist.barrier()
    for _ in range(warm):
        bd.launch(M, advance=True)
    torch.cuda.synchronize()
    bd.counters[2:3].zero_()
    dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    with torch.cuda.stream(bd._stream):
        e0.record()
    for _ in range(steps):
        bd.launch(M, advance=True)
    with torch.cuda.stream(bd._stream):
        e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = D.max_over_ranks(e0.elapsed_time(e1), dev)
    sampler.stop_flag.set()
    sampler.join()
    eng.check_fault()
    bad = int(bd.status.item())
    hist = bd.hist[:min(steps, bd.hist_cap) * M].view(-1, M)[:, :B]
    tmax, tmin = hist.clone().long(), hist.clone().long()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
    same = bool((tmax == tmin).all().item())
    tok_s = B * steps / (ms / 1e3)
    # end to end: host rows in, picks out, every pass (every rank feeds the same rows)
    pos = args.prompt + warm + steps
    cur = [(slot, int(hist[-1, slot]), pos) for slot in range(B)]
    n_e2e = min(steps, 32)
    for _ in range(2):
        picks = bd.step(cur)
        cur = [(s_, t_, p_ + 1) for (s_, _, p_), t_ in zip(cur, picks)]
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        picks = bd.step(cur)
        cur = [(s_, t_, p_ + 1) for (s_, _, p_), t_ in zip(cur, picks)]
    torch.cuda.synchronize()
    e2e_s = D.max_over_ranks(time.perf_counter() - t0, dev)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": (f"{mix.lower()} weights against e4m3 activations (1x128 scales) on tcgen05 kind::f8f6f4, fp32 promotion every 128 values, f16 KV"
                      if mix == "FP8_B128" and bd.fp8_native else
                      "bf16 weights and activations on tcgen05 kind::f16, fp32 accumulate, f16 KV" if mix == "BF16" else
                      f"{mix.lower()} weights expanded to bf16 inside the tcgen05 GEMM, fp32 accumulate, f16 KV"),
            "data": f"synthetic: seeded random token ids, random-init N(0,0.02) weights quantised {mix} on the card",
            "config": {"model": spec.name, "global_batch": B, "seq_len": args.prompt + warm + steps, "prompt_tokens": args.prompt,
                       "parallelism": f"ep{world} experts; rows and attention replicated; one rank-ordered all-reduce of the "
                                      f"experts' partial rows per layer over NVLink peer memory",
                       "graph": "one CUDA graph per pass", "rows_per_pass": M, "symmetric_memory": bd.sym.how,
                       "note": "aggregate tokens/s of B concurrent sequences"},
            "clocks": sampler.summary(),
            "e2e": {"value": B * n_e2e / e2e_s, "unit": "tok/s", "steps": n_e2e,
                    "h2d_bytes_per_step": int(bd.params_host.numel() * 4) * world,
                    "d2h_bytes_per_step": int(bd.tokens_out_host.numel() * 4) * world},
            "gpu_launches": bd.launches_per_step * steps * world, "launches_per_step": bd.launches_per_step,
            "per_sequence_tok_s": tok_s / B, "ranks_agree": same, "wait_ran_out": bool(bad), "prompts_s": t_prompts,
            "load_s": t_load, "weights_gb_per_rank": w.n_bytes / 1e9}), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


def run_distributed(args, rank: int, local: int, world: int) -> int:
    if getattr(args, "batch", 1) > 1:
        return run_batch_distributed(args, rank, local, world)
    from bench import BASELINE_TOKS, METRIC, ClockSampler
    from ..models.spec import NAMED
    from ..models.weights import Weights, synth_tensors
    from ..ops import decode as K
    D.init("nccl")
    dev = f"cuda:{local}"
    if args.no_pdl:
        K.set_pdl(False)
    spec = NAMED[args.model]()
    if getattr(args, "layers", 0):
        import dataclasses
        spec = dataclasses.replace(spec, n_layer=args.layers, n_mtp=0)
    # decode of a few rows: attention whole on every rank, FFN half split, one reduction per layer (--tp-attn: heads split too)
    rep = not getattr(args, "tp_attn", False)
    lspec = local_spec(spec, world, attn=not rep)
    steps, warm = args.steps, max(3, args.warmup)
    t0 = time.time()
    mix = getattr(args, "mix", "") or "Q4_K_M"
    # every rank builds only its own share (a model that fits no single card is never built whole)
    w = Weights.from_items(lspec, synth_tensors(spec, dev, seed=0, mix=mix, shard=(rank, world), shard_attn=not rep), dev)
    torch.cuda.synchronize()
    t_load = time.time() - t0
    fused = not getattr(args, "nccl_baseline", False)
    ctx = max(args.prompt, getattr(args, 'ttft', 0) or 0) + warm + 2 * steps + 64
    # the fused arm replays one CUDA graph per step.  The NCCL arm runs eager: captured into the step graph its
    # all-reduces did not come back on two B200s (the run sat until its time limit), so that form is not used.
    eng = ShardedEngine(w, spec, rank, world, fused=fused, n_slots=1, slot_ctx=(ctx + 63) // 64 * 64,
                        use_graphs=fused, attn_replicated=rep)
    if rep:
        eng.gemm_threshold = 0          # prompts of this engine take the pass path; the head-split engine below times TTFT
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, spec.vocab, (args.prompt,), generator=g).tolist()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.time()
    first = eng.prefill(0, prompt, gemm=False if eng.gemm_threshold else None)
    torch.cuda.synchronize()
    ttft_prompt_ms = (time.time() - t0) * 1e3
    pos = len(prompt)
    toks = eng.decode_chain(0, first, pos, warm)
    pos += warm
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eng.kv.ensure(0, pos + steps + 1)
    eng.set_rows([(0, toks[-1], pos)])
    eng.counters[2:3].zero_()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    e0.record()
    for _ in range(steps):
        eng.launch(1, True, True)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = D.max_over_ranks(e0.elapsed_time(e1), dev)
    sampler.stop_flag.set()
    sampler.join()
    eng.check_fault()
    out_tokens = eng.hist[:steps].cpu().tolist()
    pos += steps
    # every rank must have produced the same text
    t = torch.tensor(out_tokens[:64], dtype=torch.int64, device=dev)
    tmax, tmin = t.clone(), t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
    same = bool((tmax == tmin).all().item())
    tok_s = steps / (ms / 1e3)

    tok = out_tokens[-1]
    for _ in range(3):
        tok = eng.step([(0, tok, pos)])[0]
        pos += 1
    n_e2e = min(steps, 128)
    eng.kv.ensure(0, pos + n_e2e + 1)
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        tok = eng.step([(0, tok, pos)])[0]
        pos += 1
    torch.cuda.synchronize()
    e2e_s = D.max_over_ranks(time.perf_counter() - t0, dev)
    extra = {}
    eng_p = eng
    if getattr(args, "ttft", 0) and fused and rep and not (spec.mla or spec.n_shared):
        # the prompt path splits the heads as well (all-gather / reduce-scatter inside the GEMMs): its own engine
        lspec_tp = local_spec(spec, world)
        w_tp = Weights.from_items(lspec_tp, synth_tensors(spec, dev, seed=0, mix=mix, shard=(rank, world)), dev)
        eng_p = ShardedEngine(w_tp, spec, rank, world, fused=True, n_slots=1, slot_ctx=(ctx + 63) // 64 * 64, use_graphs=True)
    if getattr(args, "ttft", 0) and fused and eng_p.gemm_threshold:
        # time to first token of a long prompt through the several-GPU GEMM path (collectives inside the GEMMs)
        p2 = torch.randint(0, spec.vocab, (args.ttft,), generator=g).tolist()
        ts = []
        for _ in range(3):
            eng_p.reset(0)
            torch.cuda.synchronize()
            dist.barrier()
            t0 = time.perf_counter()
            eng_p.prefill(0, p2, gemm=True)
            torch.cuda.synchronize()
            ts.append(D.max_over_ranks((time.perf_counter() - t0) * 1e3, dev))
        # the token after the prompt must be the same on every rank and (up to a bf16 arg-max flip) equal to the
        # one the 8-row pass path gives
        eng_p.reset(0)
        tok_gemm = eng_p.prefill(0, p2, gemm=True)
        eng_p.reset(0)
        tok_steps = eng_p.prefill(0, p2[:512], gemm=False)
        eng_p.reset(0)
        tok_gemm_512 = eng_p.prefill(0, p2[:512], gemm=True)
        tt = torch.tensor([tok_gemm, tok_gemm_512], dtype=torch.int64, device=dev)
        tmx, tmn = tt.clone(), tt.clone()
        dist.all_reduce(tmx, op=dist.ReduceOp.MAX)
        dist.all_reduce(tmn, op=dist.ReduceOp.MIN)
        extra = {"ttft_ms_p50": sorted(ts)[1], "ttft_prompt_tokens": args.ttft,
                 "prefill_ranks_agree": bool((tmx == tmn).all().item()),
                 "prefill_token_equals_pass_path_512": tok_gemm_512 == tok_steps,
                 "prefill_tok_s": args.ttft / (sorted(ts)[1] / 1e3),
                 "prefill_path": "tcgen05 GEMM; all-gather as peer TMA loads, reduce-scatter and expert combine as adds "
                                 "into the owner's rows from the GEMM epilogue"}
    if rank == 0:
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": tok_s / BASELINE_TOKS if args.model == "qwen3-30b-a3b" else None,
            "dtype": f"{mix.lower()} weights, int8 dot / fp32 accumulate, f16 KV",
            "data": f"synthetic: seeded random token ids, random-init N(0,0.02) weights quantised {mix} on the card",
            "config": {"model": spec.name, "global_batch": 1, "seq_len": args.prompt + warm + steps,
                       "prompt_tokens": args.prompt, "parallelism": (f"ep{world} experts (FFN width split), attention replicated: one reduction per layer" if rep
                                       else f"tp{world} attention + ep{world} experts"),
                       "ttft_engine": f"tp{world} attention + ep{world} experts",
                       "reductions": "fused: producer pushes partial rows to peer HBM, consumer prologue sums"
                       if fused else "nccl all_reduce (baseline)",
                       "l2": "weights exceed L2; no flush needed", "graph": "one CUDA graph per decode step" if fused else "eager",
                       "pdl": not args.no_pdl, "symmetric_memory": eng.arena.how},
            "clocks": sampler.summary(),
            "e2e": {"value": n_e2e / e2e_s, "unit": "tok/s", "steps": n_e2e,
                    "h2d_bytes_per_step": int(eng.params_host.numel() * 4) * world,
                    "d2h_bytes_per_step": int(eng.tokens_out_host.numel() * 4) * world},
            "gpu_launches": eng.launches_per_step * steps * world, "launches_per_step": eng.launches_per_step,
            **({"smoke_only_layers": args.layers} if getattr(args, "layers", 0) else {}),
            "ranks_agree": same, "ttft_ms_prompt": ttft_prompt_ms, "load_s": t_load,
            "weights_gb_per_rank": w.n_bytes / 1e9, **extra,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0
