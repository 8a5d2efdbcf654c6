"""Process start: levers, flags, placement plan, early listener, load, ready.

Order follows the reference (``crates/gpu-gates/src/bin/bloomery_serve.rs``): levers are parsed
first and refused by name; flags resolve with their precedence; the listener binds *before*
the model loads and answers ``loading``; ``plan`` / ``need`` / ``ctx`` / ``parallel`` lines go to
stderr; JSON start events go to stdout; the exit code tells a supervisor what happened.
"""
from __future__ import annotations

import json
import os
import signal
import sys
import time
from typing import Any, Dict, List, Optional

from ..utils import events, flags, levers, records
from ..utils.exit_codes import Code, Refusal, WORDS


def _host_free_bytes() -> int:
    from ..utils import osshim
    try:
        return osshim.host_memory().available
    except OSError:
        return 8 << 30


def plan_for(opts: Dict[str, Any], spec, weights_bytes: int, n_visible: int, free_bytes: List[int]) -> Dict[str, Any]:
    """Context / slots / placement that fit (``docs/serving.md:84-87,200``): an unset context is the
    model's trained limit, else the largest multiple of 1,024 >= 4,096 that fits; a set context is
    never cut (refused with the largest that fits); 1,024 MiB margin per GPU."""
    pl = flags.placement(opts, n_visible, spec.n_layer)
    margin = int(levers.get("BLOOMERY_CARD_MARGIN"))
    budget = int(levers.get("BLOOMERY_CARD_BUDGET"))       # HBM bytes routed experts may take per GPU (0 = what fits)
    host_room = int(levers.get("BLOOMERY_HOST_ROOM"))      # pinned host bytes cold experts may take (0 = as needed)
    par = str(opts.get("parallel", "1"))
    auto = par == "auto"
    asked = int(opts.get("ctx") or 0)
    slot_ctx = int(opts.get("slot_ctx") or 0)
    if auto and asked:
        raise Refusal(Code.USAGE, "--parallel auto beside --ctx-size: auto counts slots of one request's context; name it with --slot-ctx")
    if slot_ctx and asked:
        raise Refusal(Code.USAGE, "--slot-ctx beside --ctx-size: one names a slot's share, the other the total")
    try:
        n_slots = 1 if auto else int(par)              # auto: the placement is chosen at one slot, the count follows
    except ValueError:
        raise Refusal(Code.USAGE, f"-np {par}: takes a count or auto") from None
    if n_slots < 1:
        raise Refusal(Code.USAGE, f"-np {par}: at least one slot")
    per_tok = spec.kv_bytes_per_token() // max(1, len(pl.devices) if pl.mode == "tp" else 1)
    if pl.devices:
        if pl.fit_targets_mib:
            # -fitt MiB[,MiB...]: what stays free on each device of the list (one value serves them all); the tightest
            # device decides, since every rank holds the same share
            t = pl.fit_targets_mib
            if len(t) not in (1, len(pl.devices)):
                raise Refusal(Code.USAGE, f"-fitt names {len(t)} targets for {len(pl.devices)} devices")
            keep = [(t[0] if len(t) == 1 else t[i]) << 20 for i in range(len(pl.devices))]
            dev_free = min(free_bytes[d] - k_ for d, k_ in zip(pl.devices, keep))
            margin = 0
        else:
            dev_free = min(free_bytes[d] for d in pl.devices)
        share = weights_bytes // (len(pl.devices) if pl.mode == "tp" else 1)
        room = dev_free - margin - share - (2 << 30)
        ebytes = int(opts.get("_expert_bytes") or weights_bytes * 0.9)
        over_budget = budget > 0 and spec.is_moe and ebytes // max(1, len(pl.devices) if pl.mode == "tp" else 1) > budget
        if over_budget and pl.host_experts == "none":
            # the expert budget is binding: as many experts per layer as it pays for stay on the card, the rest page from the host
            per_expert = ebytes // max(1, spec.n_expert)
            resident = max(0, budget // max(1, per_expert)) // 4 * 4
            pl.host_experts = f"fit:{min(resident, spec.n_expert)}"
            room = dev_free - margin - (weights_bytes - ebytes) - resident * per_expert - (2 << 30)
        if host_room > 0 and pl.host_experts != "none" and ebytes > host_room:
            raise Refusal(Code.NO_FIT, f"cold experts need {ebytes >> 20} MiB of pinned host memory, BLOOMERY_HOST_ROOM allows {host_room >> 20} MiB")
        if room <= 0 and pl.host_experts == "none" and pl.fit and spec.is_moe:
            # -fit on: keep as many routed experts per layer on the card as fit, the rest on the host
            expert_bytes = weights_bytes * 0.9 if not opts.get("_expert_bytes") else opts["_expert_bytes"]
            trunk = weights_bytes - int(expert_bytes)
            ctx_ask = asked or 4096 * n_slots
            left = dev_free - margin - (2 << 30) - trunk - ctx_ask * per_tok
            n_moe = max(1, spec.n_layer - spec.first_dense)
            per_slot = int(expert_bytes) // max(1, spec.n_expert) // 1 if n_moe else 0      # one expert slot in every layer
            fit_slots = max(0, left) // max(1, per_slot)
            resident = max(0, (int(fit_slots) - 1)) // 4 * 4
            if trunk + ctx_ask * per_tok + margin + (2 << 30) > dev_free:
                raise Refusal(Code.NO_FIT, f"the trunk of {trunk >> 20} MiB does not fit {dev_free >> 20} MiB even with every "
                                           f"routed expert on the host")
            pl.host_experts = f"fit:{min(resident, spec.n_expert)}"
            room = left - resident * per_slot + ctx_ask * per_tok      # what the context may use
        if room <= 0 and pl.host_experts == "none":
            raise Refusal(Code.NO_FIT, f"weights of {share >> 20} MiB per GPU do not fit {dev_free >> 20} MiB free "
                                       f"(margin {margin >> 20} MiB); try --cpu-moe or more devices")
        fit_tokens = max(0, room) // max(1, per_tok)
    else:
        fit_tokens = _host_free_bytes() // 2 // max(1, per_tok)
    source = "flag"
    if auto:
        # the most slots, up to 8, that hold one request's context: --slot-ctx when set, else the context one slot
        # takes with no flags -- and where that one slot already has to fit under the model's limit, one slot
        one = slot_ctx or min(spec.ctx_train, fit_tokens // 1024 * 1024)
        n_slots = 1 if (not slot_ctx and one < spec.ctx_train) else max(1, min(8, fit_tokens // max(1, one)))
        source = "auto"
    if asked:
        total = asked
        if total > fit_tokens:
            best = fit_tokens // 1024 * 1024
            raise Refusal(Code.NO_FIT, f"-c {asked} does not fit; the largest context that fits is {best}")
    elif slot_ctx:
        total = slot_ctx * n_slots
        if total > fit_tokens:
            best = fit_tokens // n_slots // 1024 * 1024
            raise Refusal(Code.NO_FIT, f"--slot-ctx {slot_ctx} x {n_slots} slots does not fit; the largest slot context that fits is {best}")
    else:
        total = min(spec.ctx_train * n_slots, fit_tokens // 1024 * 1024)
        if total < 4096:
            raise Refusal(Code.NO_FIT, "not even a context of 4,096 fits beside the weights")
    rule = "set" if (asked or slot_ctx) else None
    if not slot_ctx:
        slot_ctx = min(spec.ctx_train, total // n_slots)
    slot_ctx = slot_ctx // 64 * 64
    if rule is None:
        rule = "target" if slot_ctx >= spec.ctx_train // 64 * 64 else "fitted"
    return {"placement": pl, "n_slots": n_slots, "slot_ctx": slot_ctx, "ctx_total": slot_ctx * n_slots,
            "kv_bytes": slot_ctx * n_slots * per_tok, "weights_bytes": weights_bytes, "ctx_rule": rule, "slots_from": source}


def _inventory(path: str):
    """(spec, weights bytes, kind) of a model path: a GGUF file / split, or a checkpoint folder."""
    from ..formats.gguf import Gguf, GgufError
    from ..models.spec import ModelSpec
    try:
        if os.path.isdir(path):
            from ..formats.safetensors import Folder, SafetensorsError
            try:
                f = Folder(path)
            except SafetensorsError as exc:
                raise Refusal(Code.LOAD, str(exc)) from None
            if not f.config:
                raise Refusal(Code.LOAD, f"{path}: no config.json beside the tensors")
            nbytes = sum(f.info(n).end - f.info(n).begin for n in f.names())
            spec = ModelSpec.from_hf_config(f.config)
            f.close()
            return spec, nbytes, "folder"
        inv = Gguf.inventory(path)
        return ModelSpec.from_gguf(inv), sum(t.n_bytes for t in inv.tensors.values()), "gguf"
    except GgufError as exc:
        raise Refusal(Code.LOAD, str(exc)) from None
    except (ValueError, KeyError) as exc:
        raise Refusal(Code.UNSUPPORTED, str(exc)) from None


def _expert_bytes(path: str, kind: str) -> int:
    """Bytes of the routed-expert tensors of a model file (what may live on the host)."""
    try:
        if kind == "gguf":
            from ..formats.gguf import Gguf
            inv = Gguf.inventory(path)
            return sum(t.n_bytes for n, t in inv.tensors.items() if "_exps." in n)
        from ..formats.safetensors import Folder
        f = Folder(path)
        n = sum(f.info(t).end - f.info(t).begin for t in f.names() if ".mlp.experts." in t)
        f.close()
        return n
    except Exception:  # noqa: BLE001 - the plan falls back to its own estimate
        return 0


def open_engine(opts: Dict[str, Any], server, n_vis: int, template_src: Optional[str]):
    """Plan, load and build the engine the flags ask for: one GPU, several GPUs in lockstep, experts on the
    host beside a GPU, or the CPU alone.  Returns (engine, chat template source, bos text, eos text)."""
    import torch
    from .engine import CpuEngine, GpuEngine
    path = opts["model"]
    kinds = []
    for flag, key in (("-ctk", "cache_type_k"), ("-ctv", "cache_type_v")):
        kind = {"fp16": "f16"}.get(str(opts.get(key) or "f16").lower(), str(opts.get(key) or "f16").lower())
        if kind not in ("f16", "q8_0"):
            raise Refusal(Code.USAGE, f"{flag} {opts[key]}: the KV cache is f16 or q8_0 in this build")
        kinds.append(kind)
    if kinds[0] != kinds[1]:
        raise Refusal(Code.USAGE, f"-ctk {kinds[0]} with -ctv {kinds[1]}: keys and values share one cache type here")
    opts["_kv_type"] = kinds[0]
    spec, weights_bytes, kind = _inventory(path)
    free = [torch.cuda.mem_get_info(i)[0] for i in range(n_vis)]
    opts["_expert_bytes"] = _expert_bytes(path, kind)
    plan = plan_for(opts, spec, weights_bytes, n_vis, free)
    pl = plan["placement"]
    opts["_place_word"] = pl.word()
    if opts.get("_kv_type", "f16") != "f16" and len(pl.devices) > 1:
        raise Refusal(Code.USAGE, "-ctk q8_0: the several-GPU engines keep an f16 cache")
    records.write("plan", model=spec.name, devices=[f"CUDA{d}" for d in pl.devices], weights_bytes=weights_bytes,
                  kv_bytes=plan["kv_bytes"], ctx=plan["ctx_total"], slots=plan["n_slots"], place=pl.word())
    need = need_record(opts, spec, weights_bytes, plan)
    records.write("need", **need)
    ask_need_hook(need)
    records.write("ctx", asked=int(opts.get("ctx") or 0), served=plan["slot_ctx"], trained=spec.ctx_train, rule=plan["ctx_rule"])
    records.write("parallel", slots=plan["n_slots"], slot_ctx=plan["slot_ctx"], source=plan["slots_from"])
    if opts["plan"] or opts["dry_run"]:
        out = {"place": pl.word(), "devices": pl.devices, "slots": plan["n_slots"], "slot_ctx": plan["slot_ctx"],
               "weights_bytes": weights_bytes, "kv_bytes": plan["kv_bytes"]}
        print(json.dumps(out) if opts["json"] else "\n".join(f"{k}: {v}" for k, v in out.items()))
        server.state.stop_cause = "plan"
        server.state.stop_event.set()
        raise _PlanOnly()
    server.state.phase = "load"
    t0 = time.time()
    from ..models.weights import open_model
    from ..ops import decode as K
    from .tokenizer import from_folder, from_gguf
    name = opts.get("alias") or spec.name or os.path.basename(path.rstrip("/"))

    def surface(handle):
        if kind == "gguf":
            tk = from_gguf(handle, spec.vocab)
            tsrc = template_src if template_src is not None else handle.get("tokenizer.chat_template")
        else:
            tk = from_folder(path, spec.vocab)
            tsrc = template_src
            tc = os.path.join(path, "tokenizer_config.json")
            if tsrc is None and os.path.exists(tc):
                tsrc = json.load(open(tc, encoding="utf-8")).get("chat_template")
        bos = tk.decode([tk.bos_id], skip_special=False) if tk.bos_id >= 0 else ""
        eos = tk.decode([tk.eos_id], skip_special=False) if tk.eos_id >= 0 else ""
        return tk, tsrc, bos, eos

    if not pl.devices:
        if n_vis == 0 and str(opts.get("dev") or "").lower() != "none" and str(opts.get("ngl", "")) != "0":
            raise Refusal(Code.NO_DEVICE, "no CUDA device is visible; -dev none starts the CPU-only engine on a model that fits host RAM")
        _, w, handle = open_model(path, "cpu")
        records.write("setup", phase="load", seconds=round(time.time() - t0, 3), page_cache=getattr(handle, "page_cache", None))
        tk, tsrc, bos, eos = surface(handle)
        from ..runtime.host_model import covers
        if bool(levers.get("BLOOMERY_HOST_NATIVE")) and covers(w.spec):
            from .engine import NativeCpuEngine
            return NativeCpuEngine(w, tk, plan["n_slots"], plan["slot_ctx"], name), tsrc, bos, eos
        return CpuEngine(w, tk, plan["n_slots"], plan["slot_ctx"], name), tsrc, bos, eos
    from ..ops import host_ops
    host_ops.pool_configure(int(levers.get("BLOOMERY_THREADS")), bool(levers.get("BLOOMERY_PIN")), int(levers.get("BLOOMERY_SPIN")))
    K.set_pdl(bool(levers.get("BLOOMERY_PDL")))
    K.set_staged(bool(levers.get("BLOOMERY_STAGED")))
    K.set_staged_parts(str(levers.get("BLOOMERY_STAGED_PARTS")))
    K.set_flash_mma(bool(levers.get("BLOOMERY_FLASH_MMA")))
    graphs = bool(levers.get("BLOOMERY_GRAPHS"))
    bound = float(levers.get("BLOOMERY_ENGINE_BOUND"))
    if pl.mode == "tp" and len(pl.devices) > 1:
        if kind != "gguf":
            raise Refusal(Code.UNSUPPORTED, "several GPUs in lockstep are served from GGUF files; load the folder on one GPU")
        from ..parallel import serve_tp as TP
        port = int(levers.get("BLOOMERY_TP_PORT")) or (29600 + os.getpid() % 2000)
        followers = TP.spawn_followers(path, pl.devices, port, plan["n_slots"], plan["slot_ctx"])
        ctl = TP.init_groups(0, len(pl.devices), pl.devices[0], port)
        dec, _, handle = TP.open_rank(path, 0, len(pl.devices), pl.devices[0], plan["n_slots"], plan["slot_ctx"],
                                      fused=bool(levers.get("BLOOMERY_FUSED_COMM")), use_graphs=graphs)
        import torch.distributed as dist
        dist.barrier()
        records.write("setup", phase="load", seconds=round(time.time() - t0, 3))
        tk, tsrc, bos, eos = surface(handle)
        eng = TP.leader_engine(dec, tk, name, TP.Lockstep(ctl))
        eng.followers = followers
    else:
        dev = f"cuda:{pl.devices[0]}"
        torch.cuda.set_device(pl.devices[0])
        _, w, handle = open_model(path, dev)
        records.write("setup", phase="load", seconds=round(time.time() - t0, 3))
        kw = dict(n_slots=plan["n_slots"], slot_ctx=plan["slot_ctx"], use_graphs=graphs, engine_bound_s=bound)
        if opts.get("_kv_type", "f16") != "f16":
            if spec.mla:
                raise Refusal(Code.USAGE, "-ctk q8_0: the latent cache of this model is f16")
            kw["kv_type"] = opts["_kv_type"]
        if pl.host_experts != "none" and spec.is_moe:
            from ..runtime.tiered import TieredEngine
            if pl.host_experts == "all":
                resident = 0
            elif pl.host_experts.startswith("fit:"):
                resident = int(pl.host_experts.split(":")[1])
            elif pl.host_experts.startswith("first:"):
                n_host_layers = min(spec.n_layer, int(pl.host_experts.split(":")[1]))
                resident = spec.n_expert * (spec.n_layer - n_host_layers) // spec.n_layer // 4 * 4
            else:
                resident = 0
            records.write("setup", phase="tier", seconds=0.0, resident_per_layer=resident, host=pl.host_experts)
            dec = TieredEngine(w, resident, residency=str(levers.get("BLOOMERY_RESIDENCY")), **kw)
            server.state.residency = dec.tiered          # POST /residency/reset forgets the heat counts
        else:
            from ..runtime.engine import DecodeEngine
            dec = DecodeEngine(w, **kw)
        dec.ubatch = int(opts.get("ubatch") or levers.get("BLOOMERY_UBATCH"))
        if opts.get("prefill") == "steps" or str(levers.get("BLOOMERY_PREFILL")) == "steps":
            dec.gemm_threshold = 0
        if str(levers.get("BLOOMERY_KV_HOST")) != "spill":
            dec.kv.allow_spill = False
        dec.kv.floor_positions = int(levers.get("BLOOMERY_KV_FLOOR"))
        trace_dir = str(levers.get("BLOOMERY_ROUTE_TRACE"))
        if trace_dir and spec.is_moe:
            from ..runtime.route_trace import RouteTraceWriter
            dec.route_trace = RouteTraceWriter(os.path.join(trace_dir, f"{name}.blrt"), spec.n_layer, spec.n_used)
        tk, tsrc, bos, eos = surface(handle)
        eng = GpuEngine(dec, tk, name)
    from ..runtime.watchdog import Watchdog
    eng.dec.watchdog = Watchdog(name, bound_s=bound, report=lambda site, age: records.write(
        "watchdog", model=name, site=site, seconds=round(age, 1))).start()
    if bool(levers.get("BLOOMERY_AUTOTUNE")) and not (pl.mode == "tp" and len(pl.devices) > 1):
        from ..runtime.autotune import CostStore, tune_decode_launch
        from ..build import source_hash
        store = CostStore(os.path.join(os.path.expanduser("~"), ".cache", "bloomery_b200", "costs.json"))
        got = tune_decode_launch(eng.dec, store, build=source_hash())
        records.write("setup", phase="autotune", seconds=0.0, winner=got["winner"], raced=got["raced"])
    if not opts.get("no_warmup"):
        t1 = time.time()
        eng.step([(0, max(0, tk.bos_id), 0)], want_logits=False)
        eng.reset(0)
        records.write("setup", phase="warmup", seconds=round(time.time() - t1, 3))
    return eng, tsrc, bos, eos


def need_record(opts: Dict[str, Any], spec, weights_bytes: int, plan: Dict[str, Any]) -> Dict[str, Any]:
    """What the placed load asks of the machine (``docs/serving.md`` "Starting under a broker" of the reference): host
    bytes it will pin (cold experts and the upload ring), the prompt cache beside them, the bytes per card, the worker
    threads and the CPUs the process may run on."""
    from ..utils import osshim
    pl = plan["placement"]
    ebytes = int(opts.get("_expert_bytes") or 0)
    pinned = 2 * (256 << 20)                                         # the two-slot upload ring
    if pl.host_experts != "none" and spec.is_moe:
        resident = int(pl.host_experts.split(":")[1]) if pl.host_experts.startswith("fit:") else 0
        pinned += ebytes - ebytes // max(1, spec.n_expert) * resident            # the experts that stay on the host
    cache_mib = int(opts.get("cache_ram", -1))
    cache_ram = min(8 << 30, _host_free_bytes() // 2) if cache_mib < 0 else cache_mib << 20
    n_dev = max(1, len(pl.devices))
    share = (weights_bytes - (pinned - (512 << 20))) // (n_dev if pl.mode == "tp" else 1)
    allowed = osshim.mask_cpus()
    threads = int(levers.get("BLOOMERY_THREADS")) or len(allowed)
    return {"weights_bytes": weights_bytes, "kv_bytes_per_token": spec.kv_bytes_per_token(), "host_bytes": pinned,
            "fits": True, "bytes": pinned, "pinned": pinned, "cache_ram": cache_ram,
            "cards": [f"CUDA{d}:{share + plan['kv_bytes'] // n_dev}" for d in pl.devices], "threads": threads, "allowed": allowed}


def ask_need_hook(need: Dict[str, Any]) -> None:
    """``BLOOMERY_NEED_HOOK``: a broker's say before a card is opened.  The program gets the need line on its standard
    input; exit 0 goes on, 75 ends this process with 75 (the hook's last output line named) so the start can be queued
    and asked again, anything else is a named error."""
    hook = str(levers.get("BLOOMERY_NEED_HOOK") or "")
    if not hook:
        return
    if not os.path.isabs(hook):
        raise Refusal(Code.LEVER, f"BLOOMERY_NEED_HOOK={hook!r}: takes an absolute path")
    import subprocess
    line = "need " + " ".join(f"{k}={json.dumps(v, separators=(',', ':'))}" for k, v in need.items()) + "\n"
    try:
        done = subprocess.run([hook], input=line, capture_output=True, text=True, timeout=300)
    except (OSError, subprocess.TimeoutExpired) as exc:
        raise Refusal(Code.REFUSED, f"the need hook {hook} did not run: {exc}") from None
    last = ((done.stdout or "") + (done.stderr or "")).strip().splitlines()[-1:] or [""]
    if done.returncode == 0:
        return
    if done.returncode == int(Code.RETRY):
        raise Refusal(Code.RETRY, f"the need hook asks to start later: {last[0]}")
    raise Refusal(Code.REFUSED, f"the need hook {hook} exited {done.returncode}: {last[0]}")


def queue_depth_for(opts: Dict[str, Any], n_slots: int) -> int:
    """Requests that may wait for a slot: 64 minus the slot count unless ``--queue-depth`` names fewer; more is refused."""
    most = max(0, 64 - int(n_slots))
    asked = int(opts.get("queue_depth", -1))
    if asked < 0:
        return most
    if asked > most:
        raise Refusal(Code.USAGE, f"--queue-depth {asked}: with {n_slots} slot(s) the most is {most} (64 minus the slots)")
    return asked


def _views(server) -> None:
    """The start screen below the record lines, and the live view's keys, when a person is watching (stderr and stdin
    are terminals); a server under a supervisor gets neither."""
    from . import screen
    worker = server.state.worker
    ring = screen.Ring()
    if worker is not None:
        worker.request_lines = ring
    shown = [False]

    def on_key(ch: str) -> None:
        if ch != "d":
            return
        shown[0] = not shown[0]
        if shown[0]:
            m = worker.metrics if worker is not None else None
            counters = {k: (m.get(k) if m is not None else 0.0) for k in ("n_decode_total", "tokens_predicted_total", "prompt_tokens_total")}
            try:
                width = os.get_terminal_size(sys.stderr.fileno()).columns
            except (OSError, ValueError):
                width = 80
            sys.stderr.write(screen.live_view(ring, counters, width, screen.Style.of(os.environ)))
            sys.stderr.flush()
    keys = screen.watch_keys(on_key) if sys.stderr.isatty() else None
    screen.draw_if_armed(server.url, live_keys=keys is not None)


class _PlanOnly(Exception):
    pass


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    events.enable()
    try:
        levers.at_main()
        opts = flags.parse(argv)
        for note in opts.get("_config_notes", ()):
            print(f"bloomery-serve: {note}", file=sys.stderr)
        from . import screen
        screen.arm(os.environ, sys.stderr.isatty(), str(levers.get("BLOOMERY_SCREEN")))
        records.tap(screen.note)
        if opts["version"]:
            from .. import __version__
            print(f"bloomery_b200 {__version__}")
            return 0
        if opts["levers"]:
            print(levers.listing())
            return 0
        if opts["records_schema"]:
            print(records.schema())
            return 0
        # -np N --engine-slots P (P < N): the engine is planned and built for P sequences, N slots take it in turns
        turns = 0
        es = int(opts.get("engine_slots") or 0)
        if es:
            if opts["parallel"] == "auto" or es < 1 or es >= int(opts["parallel"]):
                raise Refusal(Code.USAGE, f"--engine-slots {es} takes a value below -np N (got -np {opts['parallel']})")
            if str(opts.get("park")) not in ("states", "ids"):
                raise Refusal(Code.USAGE, f"--park takes states or ids, got {opts['park']!r}")
            turns, opts["parallel"] = int(opts["parallel"]), str(es)

        def in_turns(eng):
            if not turns:
                return eng
            from .swap import SwapEngine
            return SwapEngine(eng, turns, str(opts["park"]), int(opts["park_ram"]) << 20)
        import torch
        n_vis = torch.cuda.device_count() if torch.cuda.is_available() else 0
        if opts["list_devices"]:
            devs = [{"id": f"CUDA{i}", "name": torch.cuda.get_device_name(i),
                     "free_mib": torch.cuda.mem_get_info(i)[0] >> 20, "total_mib": torch.cuda.mem_get_info(i)[1] >> 20}
                    for i in range(n_vis)]
            print(json.dumps(devs) if opts["json"] else "\n".join(f"{d['id']}: {d['name']} ({d['free_mib']} / {d['total_mib']} MiB free)" for d in devs) or "no CUDA device")
            return 0
        from .api import Server
        server = Server(opts)
        server.start()
        def on_signal(*_):
            if server.state.stop_event.is_set():            # a second signal ends the process at once
                print("bloomery-serve: second signal, leaving now", file=sys.stderr, flush=True)
                os._exit(1)
            server.state.stop_cause = "signal"
            server.state.stop_event.set()
        signal.signal(signal.SIGINT, on_signal)
        signal.signal(signal.SIGTERM, on_signal)
        from .engine import GpuEngine, MockEngine
        from .chat import ChatTemplate
        template_src = None
        if opts.get("chat_template_file"):
            with open(opts["chat_template_file"]) as fh:
                template_src = fh.read()
        elif opts.get("chat_template"):
            template_src = opts["chat_template"]
        cache_mib = int(opts.get("cache_ram", -1))
        cache_bytes = min(8 << 30, _host_free_bytes() // 2) if cache_mib < 0 else cache_mib << 20
        if opts["mock"]:
            eng = MockEngine(n_slots=4 if opts["parallel"] == "auto" else int(opts["parallel"]),      # nothing to count from: four
                             slot_ctx=int(opts.get("ctx") or 4096), fail_at=int(opts.get("mock_fail_at", -1)))
            opts["_place_word"] = "mock"
            server.ready(in_turns(eng), ChatTemplate(template_src), cache_bytes, queue_depth_for(opts, turns or eng.n_slots))
            _views(server)
            return server.wait()
        if not opts.get("model"):
            raise Refusal(Code.NO_MODEL, "no model was named; use -m FILE (a GGUF file, any shard of a split) or --mock")
        from . import preflight
        refusal = preflight.run(n_vis, str(opts.get("dev") or ""))
        if refusal:
            raise Refusal(Code.NO_DEVICE, refusal)
        if not os.path.exists(opts["model"]):
            raise Refusal(Code.NO_MODEL, f"{opts['model']}: no such file")
        server.state.phase = "plan"
        eng, template_src, bos, eos = open_engine(opts, server, n_vis, template_src)
        server.ready(in_turns(eng), ChatTemplate(template_src, bos, eos), cache_bytes, queue_depth_for(opts, turns or eng.n_slots))
        draft = str(levers.get("BLOOMERY_DRAFT")).lower()
        draft = "ngram" if draft == "lookup" else draft
        if turns and draft in ("mtp", "auto"):
            draft = ""            # the draft layer's KV rows are the engine's own slots, not the slots that take turns
        if draft == "ngram" and server.state.worker is not None:
            from ..runtime.speculative import NgramDraft, WidthChooser
            width = int(levers.get("BLOOMERY_MTP_WIDTH")) or 7
            server.state.worker.enable_drafting(NgramDraft(), WidthChooser(max_width=max(1, min(width, 7))))
        elif draft in ("mtp", "auto") and server.state.worker is not None and getattr(getattr(eng, "dec", None), "n_mtp", 0):
            from ..runtime.speculative import MtpDraft, WidthChooser
            if eng.dec.enable_mtp():
                width = int(levers.get("BLOOMERY_MTP_WIDTH")) or 1
                server.state.worker.enable_drafting(MtpDraft(eng), WidthChooser(max_width=max(1, min(width, 7))))
        _views(server)
        return server.wait()
    except _PlanOnly:
        return server.stop()
    except Refusal as r:
        word, nxt = WORDS.get(r.code, ("refused", ""))
        events.emit("error", code=int(r.code), word=word, message=str(r), next=nxt)
        print(f"error: {r}", file=sys.stderr)
        return int(r.code)
