#!/usr/bin/env python
"""Headline benchmark: single-request greedy decode tokens/s on the Qwen3-30B-A3B shape
(48 layers, hidden 2048, 32 q / 4 kv heads of 128, 128 experts top-8, moe_inter 768,
vocab 151936) with Q4_K_M weights, after a 512-token random prompt.

    python bench.py --gpus N --steps K --warmup W          # own arm
    python bench.py --impl reference ...                   # reference arm

A step is one decode step (one token).  The device-timed value replays the decode graph
K times back to back (the next step's input stays on the card) between two CUDA events;
the end-to-end value drives the public ``DecodeEngine.step`` call once per token, which
copies that step's token/position/slot words from pinned host memory and reads the pick
(and the fault word) back every step.  Weights (about 17 GB) are far larger than L2, so
every step streams them from HBM; no explicit L2 flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_TOKS = 164.1   # Qwen3-30B-A3B Q4_K_M decode, reference on 1x RTX 3090 (docs/numbers.md:70)
METRIC = "decode tok/s (whole box, max over ranks)"


def reference_arm(args) -> int:
    why = ("reference is a Rust/cuda-oxide workspace (no setup.py/pyproject; pip: 'not installable'); "
           "no cargo/rustc on this image and it has no sm_100 target")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons through nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)
            except Exception:
                pass
            self.stop_flag.wait(0.1)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(s[0]) for s in self.samples)
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(self.samples[0][1]), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(float(s[2]) for s in self.samples)}


def _pool_threads() -> int:
    from bloomery_b200.ops._lib import host
    return int(host().blh_pool_size())


def cpu_arm(args) -> int:
    """``--cpu``: the tiny Qwen3-MoE shape on the host engine (quantised weights, q8 activation sites, the C++ expert
    leg's arithmetic), 64 seeded prompt ids then 32 greedy tokens; wall-clock, since no device is involved."""
    import torch
    from bloomery_b200.models.cpu_ref import CpuModel, greedy_pick
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.models.weights import Weights, synth_tensors
    spec = tiny_qwen3moe()
    w = Weights.from_items(spec, synth_tensors(spec, "cpu", seed=0, mix="Q4_K_M"), "cpu")
    from bloomery_b200.runtime.host_model import HostDecoder
    m = HostDecoder(w, ctx=256)                 # the native host step: quantised row dots on q8 activations, C++ throughout
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, spec.vocab, (64,), generator=g).tolist()
    n_gen = 32
    best = None
    for _ in range(max(3, min(args.warmup, 8))):      # the fastest of several runs: a shared host's other tenants are noise
        m.reset()
        t0 = time.perf_counter()
        for t in prompt[:-1]:
            m.step(t, want_logits=False)
        tok = greedy_pick(m.step(prompt[-1]))
        t1 = time.perf_counter()
        out = [tok]
        for _ in range(n_gen - 1):
            tok = greedy_pick(m.step(tok))
            out.append(tok)
        t2 = time.perf_counter()
        run = (t1 - t0, t2 - t1, out)
        if best is None or run[1] < best[1]:
            best = (min(run[0], best[0]) if best else run[0], run[1], run[2])
        else:
            best = (min(run[0], best[0]), best[1], best[2])
    # the oracle (plain PyTorch on the dequantised weights) on the same prompt: how many of the ids agree
    oracle = CpuModel(w)
    want = oracle.generate(prompt, n_gen)
    ttft, dec, out = best
    tok_s = (n_gen - 1) / dec
    print(json.dumps({
        "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": 0, "steps": n_gen - 1, "warmup": 1,
        "ms_per_step": dec / (n_gen - 1) * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "q4_k_m weights, q8 activation sites, int8 dots (VNNI / AVX2 / scalar), fp32 accumulate (host)",
        "data": "synthetic: seeded random ids, N(0,0.02) weights",
        "config": {"model": spec.name, "global_batch": 1, "seq_len": 64 + n_gen, "prompt_tokens": 64, "parallelism": "cpu",
                   "engine": "native host step (csrc/host/model_cpu.cpp)", "threads": _pool_threads()},
        "oracle_agreement": sum(int(a == b) for a, b in zip(out, want)) / n_gen,
        "ttft_ms_prompt": ttft * 1e3, "prefill_tok_s": 64 / ttft, "tokens": out[:8], "gpu_launches": 0,
        "e2e": {"value": n_gen / (ttft + dec), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
    return 0


def batch_arm(args, spec, w, dev, local, steps, warm, t_load) -> int:
    """``--batch B``: B sequences, one token each per pass, through the batched tensor-core decode."""
    import torch
    from bloomery_b200.runtime.batch_decode import BatchDecode
    from bloomery_b200.runtime.engine import DecodeEngine
    B = args.batch
    mix = args.mix or "Q4_K_M"
    ctx = (args.prompt + warm + 2 * steps + 64 + 63) // 64 * 64
    eng = DecodeEngine(w, n_slots=B, slot_ctx=ctx)
    bd = BatchDecode(eng, max_rows=max(16, B))
    g = torch.Generator().manual_seed(1234)
    rows = []
    t0 = time.time()
    for slot in range(B):
        prompt = torch.randint(0, spec.vocab, (args.prompt,), generator=g).tolist()
        rows.append((slot, eng.prefill(slot, prompt), args.prompt))
    torch.cuda.synchronize()
    t_prompts = time.time() - t0
    for slot in range(B):
        eng.kv.ensure(slot, args.prompt + warm + 2 * steps + 8)
    M = bd.set_rows(rows)
    bd.counters[2:3].zero_()
    for _ in range(warm):
        bd.launch(M, advance=True)
    torch.cuda.synchronize()
    bd.counters[2:3].zero_()
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
    ms = e0.elapsed_time(e1)
    sampler.stop_flag.set()
    sampler.join()
    eng.check_fault()
    if int(bd.status.item()) != 0:
        raise RuntimeError("a bounded wait inside the GEMM kernel ran out")
    tok_s = B * steps / (ms / 1e3)
    hist = bd.hist[:min(steps, bd.hist_cap) * M].view(-1, M)[:, :B].cpu()
    pos = args.prompt + warm + steps
    # end to end through the public call: host rows in, picks out, every pass
    cur = [(slot, int(hist[-1, slot]), pos) for slot in range(B)]
    n_e2e = min(steps, 64)
    for _ in range(2):
        picks = bd.step(cur)
        cur = [(s_, t_, p_ + 1) for (s_, _, p_), t_ in zip(cur, picks)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        picks = bd.step(cur)
        cur = [(s_, t_, p_ + 1) for (s_, _, p_), t_ in zip(cur, picks)]
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    # weight bytes one pass reads: every matrix once, routed experts only when some row chose them (at 64 rows of top-8
    # out of 128 nearly all are chosen: counted in full)
    active = sum(qw.n_bytes for name, qw in w.q.items() if not (name == "token_embd.weight" and "output.weight" in w.q))
    gbs = active / (ms / steps / 1e3) / 1e9
    peak, peak_src = 6650.0, "fallback"
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as fh:
            peak, peak_src = float(json.load(fh)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        pass
    line = {
        "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": (f"{mix.lower()} weights against e4m3 activations (1x128 scales) on tcgen05 kind::f8f6f4, fp32 promotion every 128 values, f16 KV"
                  if mix == "FP8_B128" and bd.fp8_native else
                  "bf16 weights and activations on tcgen05 kind::f16, fp32 accumulate, f16 KV" if mix == "BF16" else
                  f"{mix.lower()} weights expanded to bf16 inside the tcgen05 GEMM, fp32 accumulate, f16 KV"),
        "data": f"synthetic: seeded random token ids, random-init N(0,0.02) weights quantised {mix} on the card",
        "config": {"model": spec.name, "global_batch": B, "seq_len": args.prompt + warm + steps, "prompt_tokens": args.prompt,
                   "parallelism": "single", "l2": "weights (17 GB) exceed L2; no flush needed",
                   "graph": "one CUDA graph per pass", "rows_per_pass": M,
                   "note": "aggregate tokens/s of B concurrent sequences; the published reference figure is single-sequence"},
        "clocks": sampler.summary(),
        "e2e": {"value": B * n_e2e / e2e_s, "unit": "tok/s", "steps": n_e2e,
                "h2d_bytes_per_step": int(bd.params_host.numel() * 4), "d2h_bytes_per_step": int(bd.tokens_out_host.numel() * 4)},
        "gpu_launches": bd.launches_per_step * steps, "launches_per_step": bd.launches_per_step,
        "per_sequence_tok_s": tok_s / B, "prompts_s": t_prompts, "load_s": t_load, "weights_gb": w.n_bytes / 1e9,
        "weight_gb_per_pass": active / 1e9, "hbm_gbs_effective": gbs, "roofline_frac": gbs / peak,
        "roofline_peak": f"{peak:.0f} GB/s HBM copy rate ({peak_src})",
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="own")
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--flash-mma", action="store_true", help="decode attention segments on tensor-core tiles")
    ap.add_argument("--ttft", type=int, default=4096, help="also time a prompt of this many tokens (0 = skip)")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--staged-parts", dest="staged_parts", default="", help="ablation: which launches take the staged form (gemv,attn,moe,prefetch)")
    ap.add_argument("--attn-clusters", dest="attn_clusters", type=int, default=-1, help="ablation: 1 / 0 = cluster form of the attention launch on / off")
    ap.add_argument("--no-predict-down", dest="no_predict_down", action="store_true")
    ap.add_argument("--predict", type=int, default=-1, help="ablation: experts the side-stream prediction prefetches per layer (0 = off)")
    ap.add_argument("--no-staged", dest="no_staged", action="store_true",
                    help="register-streaming decode kernels instead of the shared-memory staged ones")
    ap.add_argument("--batch", type=int, default=1,
                    help="sequences decoded together (16..64: the batched tensor-core pass; the value is the total of all sequences)")
    ap.add_argument("--mix", default="", help="weight type recipe of the synthetic model (Q4_K_M, Q8_0, FP8_B128, NVFP4, IQ4_XS, ...)")
    ap.add_argument("--layers", type=int, default=0,
                    help="smoke runs only: cut the model to this many layers (the line is marked and is not a benchmark)")
    ap.add_argument("--cpu", action="store_true",
                    help="the CPU configuration: tiny Qwen3-MoE (Q4_K_M), 64-id prompt, 32 greedy tokens on the host engine, no GPU")
    ap.add_argument("--tp-attn", dest="tp_attn", action="store_true",
                    help="N > 1: split the attention heads over the ranks for decode too (two reductions per layer)")
    ap.add_argument("--nccl-baseline", dest="nccl_baseline", action="store_true",
                    help="N > 1: do the per-layer reductions with NCCL all_reduce instead of the fused kernels")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.cpu:
        return cpu_arm(args)

    import torch
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        print(json.dumps({"error": f"--gpus {args.gpus} but WORLD_SIZE={world}"}))
        return 1
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        from bloomery_b200.parallel.bench_dist import run_distributed
        return run_distributed(args, rank, local, world)

    from bloomery_b200.models.spec import NAMED
    from bloomery_b200.models.weights import Weights, synth_tensors
    from bloomery_b200.ops import decode as K
    from bloomery_b200.runtime.engine import DecodeEngine

    if args.flash_mma:
        from bloomery_b200.ops import decode as _K
        _K.set_flash_mma(True)
    if args.no_pdl:
        K.set_pdl(False)
    if args.no_staged:
        K.set_staged(False)
    if args.staged_parts:
        K.set_staged_parts(args.staged_parts)
    spec = NAMED[args.model]()
    steps, warm = args.steps, max(3, args.warmup)
    t0 = time.time()
    w = Weights.from_items(spec, synth_tensors(spec, dev, seed=0, mix=args.mix or "Q4_K_M"), dev)
    torch.cuda.synchronize()
    t_load = time.time() - t0
    if args.batch > 1:
        return batch_arm(args, spec, w, dev, local, steps, warm, t_load)
    ctx = max(args.prompt, args.ttft) + warm + 2 * steps + 64
    eng = DecodeEngine(w, n_slots=1, slot_ctx=(ctx + 63) // 64 * 64)
    if args.attn_clusters >= 0:
        eng.attn_clusters = bool(args.attn_clusters)
    if args.predict >= 0:
        eng.predict_experts = args.predict
    if args.no_predict_down:
        eng.predict_down = False
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, spec.vocab, (args.prompt,), generator=g).tolist()

    # prompt (timed as TTFT of this prompt length: prefill passes + first pick)
    torch.cuda.synchronize()
    t0 = time.time()
    first = eng.prefill(0, prompt)
    torch.cuda.synchronize()
    ttft_prompt_ms = (time.time() - t0) * 1e3

    # ---- device-timed decode: W warm-up steps, then exactly K steps between two events
    pos = len(prompt)
    toks = eng.decode_chain(0, first, pos, warm)
    pos += warm
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eng.kv.ensure(0, pos + steps + 1)
    eng.set_rows([(0, toks[-1], pos)])
    eng.counters[2:3].zero_()
    torch.cuda.synchronize()
    sampler.start()
    e0.record()
    for _ in range(steps):
        eng.launch(1, True, True)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    sampler.stop_flag.set()
    sampler.join()
    eng.check_fault()
    out_tokens = eng.hist[:steps].cpu().tolist()
    pos += steps
    tok_s = steps / (ms / 1e3)

    # ---- end to end through the public step call: H2D of the step's words, D2H of the pick
    tok = out_tokens[-1]
    for _ in range(3):
        tok = eng.step([(0, tok, pos)])[0]
        pos += 1
    n_e2e = min(steps, 128)
    eng.kv.ensure(0, pos + n_e2e + 1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        tok = eng.step([(0, tok, pos)])[0]
        pos += 1
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e = {"value": n_e2e / e2e_s, "unit": "tok/s", "steps": n_e2e,
           "h2d_bytes_per_step": int(eng.params_host.numel() * 4), "d2h_bytes_per_step": int(eng.tokens_out_host.numel() * 4)}

    extra = {}
    if args.ttft:
        eng.reset(0)
        p2 = torch.randint(0, spec.vocab, (args.ttft,), generator=g).tolist()
        ts = []
        for _ in range(3):
            eng.reset(0)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.prefill(0, p2)
            torch.cuda.synchronize()
            ts.append((time.perf_counter() - t0) * 1e3)
        extra["ttft_ms_p50"] = sorted(ts)[1]
        extra["ttft_prompt_tokens"] = args.ttft
        extra["prefill_tok_s"] = args.ttft / (sorted(ts)[1] / 1e3)
        # decode behind that prompt (the published reference figure is decode after 4,096 ids)
        n_deep = min(steps, 64)
        tk = eng.decode_chain(0, 1, args.ttft, 4)
        eng.kv.ensure(0, args.ttft + 4 + n_deep + 1)
        eng.set_rows([(0, tk[-1], args.ttft + 4)])
        eng.counters[2:3].zero_()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        d0.record()
        for _ in range(n_deep):
            eng.launch(1, True, True)
        d1.record()
        torch.cuda.synchronize()
        eng.check_fault()
        deep = n_deep / (d0.elapsed_time(d1) / 1e3)
        extra["decode_tok_s_after_prompt"] = {"context": args.ttft, "value": deep, "steps": n_deep, "vs_baseline": deep / BASELINE_TOKS}

    # bytes of weights one decode step has to read: everything but the routed experts it did not choose
    active = 0
    for name, qw in w.q.items():
        if name == "token_embd.weight" and "output.weight" in w.q:
            continue
        active += qw.n_bytes * (spec.n_used / spec.n_expert if "_exps." in name else 1.0)
    gbs = active / (ms / steps / 1e3) / 1e9
    peak, peak_src = 6650.0, "fallback"
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as fh:
            peak, peak_src = float(json.load(fh)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        pass

    line = {
        "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": tok_s / BASELINE_TOKS, "dtype": f"{(args.mix or 'Q4_K_M').lower()} weights, int8 dot / fp32 accumulate, f16 KV",
        "data": f"synthetic: seeded random token ids, random-init N(0,0.02) weights quantised {args.mix or 'Q4_K_M'} on the card",
        "config": {"model": spec.name, "global_batch": 1, "seq_len": args.prompt + warm + steps,
                   "prompt_tokens": args.prompt, "parallelism": "single", "l2": "weights (17 GB) exceed L2; no flush needed",
                   "graph": "one CUDA graph per decode step", "pdl": not args.no_pdl, "flash_mma": bool(args.flash_mma),
                   "staged_kernels": not args.no_staged},
        "clocks": sampler.summary(), "e2e": e2e,
        "gpu_launches": eng.launches_per_step * steps, "launches_per_step": eng.launches_per_step,
        "ttft_ms_prompt": ttft_prompt_ms, "load_s": t_load, "weights_gb": w.n_bytes / 1e9,
        "active_weight_gb_per_step": active / 1e9, "hbm_gbs_effective": gbs,
        "roofline_frac": gbs / peak, "roofline_peak": f"{peak:.0f} GB/s HBM copy rate ({peak_src})", **extra,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
