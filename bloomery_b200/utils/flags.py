"""llama-server flag spellings, their ``LLAMA_ARG_*`` twins, ``--config`` files, and the
translation of the placement flags (``-dev``, ``-ts``, ``-ngl``, ``--cpu-moe``, ``-ncmoe``,
``-ot``, ``-fit``/``-fitt``/``-fitc``, ``--place``) into one placement request.

Counterpart of ``crates/gpu-gates/src/llama_place.rs:1-55`` and ``crates/serve/src/flag.rs``:
precedence is command line > config file > ``LLAMA_ARG_*`` > default
(``docs/serving.md:370-381``); an unknown *flag* is refused by name (exit 64) whereas an
unknown *request field* is ignored; ``-sm row`` / ``-sm tensor`` and partial ``-ngl`` are
refused by name.
"""
from __future__ import annotations

import dataclasses
import json
import os
import re
from typing import Any, Dict, List, Optional, Tuple

from .exit_codes import Code, Refusal


@dataclasses.dataclass
class Flag:
    names: Tuple[str, ...]
    dest: str
    kind: str = "str"            # str | int | float | bool | count
    default: Any = None
    env: Optional[str] = None
    help: str = ""


FLAGS: List[Flag] = [
    Flag(("-m", "--model-file", "--model"), "model", env="LLAMA_ARG_MODEL", help="GGUF file (any shard) or checkpoint folder, or a seat name"),
    Flag(("--hf", "-hf", "--hf-repo"), "hf", env="LLAMA_ARG_HF_REPO", help="<repo>[@rev][:quant] (needs network)"),
    Flag(("--host",), "host", default="127.0.0.1", env="LLAMA_ARG_HOST"),
    Flag(("--port",), "port", "int", 8080, env="LLAMA_ARG_PORT", help="0 = any free port"),
    Flag(("-c", "--ctx-size"), "ctx", "int", 0, env="LLAMA_ARG_CTX_SIZE", help="0 = the model's trained limit or what fits"),
    Flag(("-np", "--parallel"), "parallel", "str", "1", env="LLAMA_ARG_N_PARALLEL", help="slots: N, or auto = as many (up to 8) as hold one request's context"),
    Flag(("--slot-ctx",), "slot_ctx", "int", 0),
    Flag(("--queue-depth",), "queue_depth", "int", -1, help="requests that may wait; default and most: 64 minus the slot count"),
    Flag(("--engine-slots",), "engine_slots", "int", 0, help="sequences the engine holds; fewer than -np = the slots take it in turns"),
    Flag(("--park",), "park", default="states", help="what a slot that leaves the engine keeps: states or ids"),
    Flag(("--park-ram",), "park_ram", "int", 4096, help="MiB of parked slot states"),
    Flag(("-ub", "--ubatch-size"), "ubatch", "int", 4096, env="LLAMA_ARG_UBATCH"),
    Flag(("-b", "--batch-size"), "batch", "int", 4096, env="LLAMA_ARG_BATCH"),
    Flag(("-cram", "--cache-ram"), "cache_ram", "int", -1, env="LLAMA_ARG_CACHE_RAM", help="MiB of host prompt cache; -1 = min(8 GiB, half free)"),
    Flag(("--cache-type-k", "-ctk"), "cache_type_k", default="f16", env="LLAMA_ARG_CACHE_TYPE_K"),
    Flag(("--cache-type-v", "-ctv"), "cache_type_v", default="f16", env="LLAMA_ARG_CACHE_TYPE_V"),
    Flag(("--chat-template-file",), "chat_template_file", env="LLAMA_ARG_CHAT_TEMPLATE_FILE"),
    Flag(("--chat-template",), "chat_template", env="LLAMA_ARG_CHAT_TEMPLATE"),
    Flag(("--jinja",), "jinja", "bool", True),
    Flag(("-a", "--alias"), "alias", env="LLAMA_ARG_ALIAS"),
    Flag(("--api-key",), "api_key", env="LLAMA_API_KEY"),
    Flag(("--api-key-file",), "api_key_file", env="LLAMA_ARG_API_KEY_FILE"),
    Flag(("--slot-save-path",), "slot_save_path", env="LLAMA_ARG_SLOT_SAVE_PATH"),
    Flag(("--config",), "config"),
    Flag(("--plan",), "plan", "bool", False), Flag(("--levers",), "levers", "bool", False),
    Flag(("--list-devices",), "list_devices", "bool", False), Flag(("--recommend",), "recommend", "bool", False),
    Flag(("--dry-run",), "dry_run", "bool", False), Flag(("--json",), "json", "bool", False),
    Flag(("--version",), "version", "bool", False), Flag(("--records-schema",), "records_schema", "bool", False),
    Flag(("--autotune",), "autotune", default="on"), Flag(("--prefill",), "prefill", default="batch"),
    Flag(("-mm", "--mmproj"), "mmproj", env="LLAMA_ARG_MMPROJ"), Flag(("--no-mmproj",), "no_mmproj", "bool", False),
    Flag(("-n", "--n-predict", "--predict"), "n_predict", "int", -1, env="LLAMA_ARG_N_PREDICT"),
    Flag(("--temp",), "temp", "float", 0.8), Flag(("--top-k",), "top_k", "int", 40), Flag(("--top-p",), "top_p", "float", 0.95),
    Flag(("--min-p",), "min_p", "float", 0.05), Flag(("--repeat-penalty",), "repeat_penalty", "float", 1.0),
    Flag(("--repeat-last-n",), "repeat_last_n", "int", 64), Flag(("-s", "--seed"), "seed", "int", -1),
    Flag(("--no-warmup",), "no_warmup", "bool", False), Flag(("--metrics",), "metrics", "bool", True),
    Flag(("--slots",), "slots_endpoint", "bool", True), Flag(("--props",), "props_endpoint", "bool", True),
    Flag(("-t", "--threads"), "threads", "int", 0, env="LLAMA_ARG_THREADS"),
    Flag(("--draft", "--draft-max"), "draft_max", "int", 0), Flag(("--mock",), "mock", "bool", False),
    Flag(("--mock-fail-at",), "mock_fail_at", "int", -1),
    # placement
    Flag(("-dev", "--device"), "dev", env="LLAMA_ARG_DEVICE", help="comma list: CUDA0,CUDA1,... or none"),
    Flag(("-sm", "--split-mode"), "split_mode", default="layer", env="LLAMA_ARG_SPLIT_MODE"),
    Flag(("-mg", "--main-gpu"), "main_gpu", "int", 0, env="LLAMA_ARG_MAIN_GPU"),
    Flag(("-ts", "--tensor-split"), "tensor_split", env="LLAMA_ARG_TENSOR_SPLIT"),
    Flag(("-ngl", "--gpu-layers", "--n-gpu-layers"), "ngl", "str", "all", env="LLAMA_ARG_N_GPU_LAYERS"),
    Flag(("-cmoe", "--cpu-moe"), "cpu_moe", "bool", False, env="LLAMA_ARG_CPU_MOE"),
    Flag(("-ncmoe", "--n-cpu-moe"), "n_cpu_moe", "int", 0, env="LLAMA_ARG_N_CPU_MOE"),
    Flag(("-ot", "--override-tensor"), "override_tensor", env="LLAMA_ARG_OVERRIDE_TENSOR"),
    Flag(("-fit", "--fit"), "fit", default="off", env="LLAMA_ARG_FIT"),
    Flag(("-fitt", "--fit-target"), "fit_target", env="LLAMA_ARG_FIT_TARGET"),
    Flag(("-fitc", "--fit-ctx"), "fit_ctx", "int", 4096, env="LLAMA_ARG_FIT_CTX"), Flag(("-devd", "--device-draft"), "dev_draft"),
    Flag(("--place",), "place", default=""),
]
_BY_NAME = {n: f for f in FLAGS for n in f.names}


def _conv(f: Flag, raw: str):
    try:
        if f.kind == "int":
            return int(raw)
        if f.kind == "float":
            return float(raw)
        if f.kind == "bool":
            return str(raw).lower() in ("1", "true", "on", "yes")
    except ValueError:
        raise Refusal(Code.USAGE, f"{f.names[0]} takes a {f.kind}, got {raw!r}") from None
    return raw


# what a settings file may not hold: keys that ask the start to do something rather than set it
_CONFIG_ACTIONS = ("plan", "levers", "help", "version", "list-devices", "records-schema", "recommend", "dry-run", "json", "config")
# the entries whose value the start line may print (never a key)
_CONFIG_SHOWN = ("ctx-size", "ubatch-size", "cache-ram", "parallel", "alias", "host", "port", "api-key-file", "slot-save-path",
                 "chat-template-file")


def _read_config(path: str, cli: Dict[str, Any], notes: List[str]) -> Dict[str, Any]:
    """``--config FILE``: one JSON object whose keys are flags' long names without their dashes.  A string or a number is
    the flag's value, ``true`` gives a switch, a list gives the flag once for each value; the command line replaces an
    entry for the same flag.  ``notes`` gets one line an entry: what it was read as, or that a flag replaced it."""
    def pairs(items):
        seen = set()
        for k, _ in items:
            if k in seen:
                raise Refusal(Code.USAGE, f"--config {path}: the key {k!r} is named twice")
            seen.add(k)
        return dict(items)
    try:
        with open(path) as fh:
            raw = json.load(fh, object_pairs_hook=pairs)
    except (OSError, json.JSONDecodeError) as exc:
        raise Refusal(Code.USAGE, f"--config {path}: {exc}") from None
    if not isinstance(raw, dict):
        raise Refusal(Code.USAGE, f"--config {path}: the file is not one JSON object")
    cfg: Dict[str, Any] = {}
    for k, v in raw.items():
        if k.startswith("-"):
            raise Refusal(Code.USAGE, f"--config: the key {k!r} carries its dashes; keys are long names without them")
        if k in _CONFIG_ACTIONS:
            raise Refusal(Code.USAGE, f"--config: {k!r} asks the start to do something; a settings file only sets")
        f = _BY_NAME.get("--" + k)
        if f is None:
            raise Refusal(Code.USAGE, f"--config: unknown key {k!r}")
        if v is False or v is None or isinstance(v, dict) or (isinstance(v, list) and not v):
            raise Refusal(Code.USAGE, f"--config: {k!r} has no value to give (false, null, an object and an empty list are not values; "
                                      f"leave out a switch that is off)")
        if f.kind == "bool":
            if v is not True:
                raise Refusal(Code.USAGE, f"--config: {k!r} is a switch; its value is true")
            val: Any = True
        else:
            if v is True:
                raise Refusal(Code.USAGE, f"--config: {k!r} takes a value, not true")
            if isinstance(v, list):
                if any(isinstance(x, (dict, list, bool)) or x is None for x in v):
                    raise Refusal(Code.USAGE, f"--config: {k!r} lists something that is not a string or a number")
                val = ",".join(str(x) for x in v)              # the flag once for each value
            else:
                val = _conv(f, str(v)) if not isinstance(v, str) else _conv(f, v)
        if f.dest in cli:
            notes.append(f"config {k}: replaced by the command line")
            continue
        cfg[f.dest] = val
        notes.append(f"config {k}" + (f"={val}" if k in _CONFIG_SHOWN else (" on" if val is True else " set")))
    return cfg


def parse(argv: List[str], environ=None) -> Dict[str, Any]:
    """Resolve every flag with precedence CLI > --config > LLAMA_ARG_* > default."""
    env = os.environ if environ is None else environ
    cli: Dict[str, Any] = {}
    i = 0
    while i < len(argv):
        a = argv[i]
        name, eq, val = a.partition("=")
        f = _BY_NAME.get(name)
        if f is None:
            raise Refusal(Code.USAGE, f"unknown flag {a!r}")
        if f.dest == "config" and "config" in cli:
            raise Refusal(Code.USAGE, "--config given twice")
        if f.kind == "bool":
            cli[f.dest] = _conv(f, val) if eq else True
        else:
            if not eq:
                i += 1
                if i >= len(argv):
                    raise Refusal(Code.USAGE, f"{name} needs a value")
                val = argv[i]
            cli[f.dest] = _conv(f, val)
        i += 1
    # two sources of one thing on the command line are refused by name, never picked between
    if "model" in cli and "hf" in cli:
        raise Refusal(Code.USAGE, "the model is named twice: -m beside --hf")
    placed = [n for n, d in (("--cpu-moe", "cpu_moe"), ("-ncmoe", "n_cpu_moe"), ("-ot", "override_tensor")) if cli.get(d)]
    if len(placed) > 1:
        raise Refusal(Code.USAGE, f"the routed experts' place is named twice: {placed[0]} beside {placed[1]}")
    cfg: Dict[str, Any] = {}
    notes: List[str] = []
    if cli.get("config"):
        cfg = _read_config(cli["config"], cli, notes)
    if "api_key" in cli and not split_keys(str(cli["api_key"])):
        raise Refusal(Code.USAGE, "--api-key names no key")
    out: Dict[str, Any] = {}
    from_env: Dict[str, str] = {}
    set_above = set(cli) | set(cfg)
    if "model" not in set_above and "hf" not in set_above and env.get("LLAMA_ARG_MODEL") and env.get("LLAMA_ARG_HF_REPO"):
        raise Refusal(Code.USAGE, "the model is named twice: LLAMA_ARG_MODEL beside LLAMA_ARG_HF_REPO")
    # --place replaces the variables that name cards; a model named above replaces both of the model's variables
    displaced = {d: "--place" for d in _CARD_DESTS} if cli.get("place") or cfg.get("place") else {}
    if "model" in set_above or "hf" in set_above:
        displaced.update({"model": "the model named above", "hf": "the model named above"})
    for f in FLAGS:
        if f.dest in cli:
            out[f.dest] = cli[f.dest]
        elif f.dest in cfg:
            out[f.dest] = cfg[f.dest]
        elif f.env and f.env in env and f.dest not in displaced:
            out[f.dest] = _env_value(f, env[f.env])
            from_env[f.dest] = f.env
        elif f.dest not in out:
            out[f.dest] = f.default
        if f.env and f.env in env and f.dest not in from_env and f.dest != "api_key":
            by = displaced.get(f.dest) or ("the command line" if f.dest in cli else "the settings file")
            notes.append(f"{f.env}: replaced by {by}")
    # llama-server's "no limit" for the prompt cache is refused: the cache is host memory beside the load, so it always has
    # a budget (unset, the lesser of 8 GiB and half the host RAM the plan leaves)
    if ("cache_ram" in cli or "cache_ram" in cfg or "cache_ram" in from_env) and int(out["cache_ram"]) < 0:
        raise Refusal(Code.USAGE, f"{from_env.get('cache_ram', '--cache-ram')} {out['cache_ram']}: the prompt cache always has a "
                                  f"budget; give MiB, 0 to turn it off, or leave it unset")
    # keys add: the variable's keys count beside the command line's (no line prints one)
    if "LLAMA_API_KEY" in env:
        more = split_keys(env["LLAMA_API_KEY"])
        if not more:
            raise Refusal(Code.USAGE, "LLAMA_API_KEY names no key")
        if "api_key" not in from_env:
            out["api_key"] = join_keys(split_keys(str(out["api_key"] or "")) + more)
            notes.append(f"LLAMA_API_KEY: {len(more)} key(s) added to the command line's")
    known = {f.env for f in FLAGS if f.env}
    for name in sorted(env):
        if name.startswith("LLAMA_ARG_") and name not in known:
            notes.append(f"{name} is set: not a variable this server reads")
    out["_config_notes"] = notes
    out["_from_env"] = from_env
    return out


def split_keys(text: str) -> List[str]:
    """The keys of a comma-separated list; an item in double quotes may hold commas (a doubled quote inside is one)."""
    import csv
    rows = list(csv.reader([text], skipinitialspace=True)) if text else []
    return [k for k in (rows[0] if rows else []) if k]


def join_keys(keys: List[str]) -> str:
    return ",".join('"' + k.replace('"', '""') + '"' if ("," in k or '"' in k) else k for k in keys)


_CARD_DESTS = ("dev", "split_mode", "tensor_split", "main_gpu")
_SWITCH_ON, _SWITCH_OFF = ("on", "enabled", "true", "1"), ("off", "disabled", "false", "0")


def _env_value(f: Flag, raw: str):
    """A variable's value as its flag's: a refusal names the variable, and a switch takes llama-server's eight words only."""
    if f.kind == "bool":
        word = raw.strip().lower()
        if word in _SWITCH_ON:
            return True
        if word in _SWITCH_OFF:
            return False
        raise Refusal(Code.USAGE, f"{f.env}={raw!r}: a switch takes {', '.join(_SWITCH_ON)} or {', '.join(_SWITCH_OFF)}")
    try:
        return _conv(f, raw)
    except Refusal as exc:
        raise Refusal(exc.code, f"{f.env}: {exc}") from None


def _named(opts: Dict[str, Any], dest: str, flag: str) -> str:
    """The name a refusal gives a setting: its variable when the variable set it, else the flag."""
    return (opts.get("_from_env") or {}).get(dest) or flag


@dataclasses.dataclass
class Placement:
    """What the placement flags ask for, in this build's terms."""

    devices: List[int]                      # CUDA ordinals; empty = CPU only
    mode: str = "a"                         # a = one GPU (whole model), tp = TP attention + EP experts over devices, cpu
    expert_shares: Optional[List[float]] = None   # -ts: share of routed experts per device
    host_experts: str = "none"              # none | all (--cpu-moe) | first:N (-ncmoe N) | pattern
    host_pattern: Optional[str] = None
    fit: bool = False
    fit_targets_mib: Optional[List[int]] = None
    fit_ctx: int = 4096
    main_gpu: int = 0
    draft_device: Optional[int] = None

    def word(self) -> str:
        if not self.devices:
            return "cpu"
        base = self.mode if len(self.devices) == 1 else f"{self.mode}{len(self.devices)}"
        if self.host_experts != "none":
            base += f"+host[{self.host_experts}]"
        return base


def _devices(spec: Optional[str], n_visible: int, name: str = "-dev") -> List[int]:
    if spec is None or spec == "":
        return list(range(min(1, n_visible))) if n_visible else []
    if spec.lower() == "none":
        return []
    out = []
    for part in spec.split(","):
        m = re.fullmatch(r"(?i)(?:cuda)?(\d+)", part.strip())
        if not m:
            raise Refusal(Code.USAGE, f"{name} {spec!r}: {part!r} is not CUDA<n>")
        d = int(m.group(1))
        if d >= n_visible:
            raise Refusal(Code.NO_DEVICE, f"{name} names CUDA{d} but {n_visible} device(s) are visible")
        out.append(d)
    if len(set(out)) != len(out):
        raise Refusal(Code.USAGE, f"{name} {spec!r} names a device twice")
    return out


def placement(opts: Dict[str, Any], n_visible: int, n_layer: int = 0) -> Placement:
    sm = (opts.get("split_mode") or "layer").lower()
    if sm in ("row", "tensor"):
        raise Refusal(Code.USAGE, f"{_named(opts, 'split_mode', '-sm')} {sm} is not served: layers are never split row-wise; use --place tp")
    if sm not in ("none", "layer"):
        raise Refusal(Code.USAGE, f"{_named(opts, 'split_mode', '-sm')} {sm!r}: expected none or layer")
    ngl = str(opts.get("ngl", "all")).lower()
    if ngl not in ("all", "auto", "-1", "999") and not (ngl.isdigit() and (n_layer == 0 or int(ngl) >= n_layer)):
        if ngl == "0":
            devs: List[int] = []
        else:
            raise Refusal(Code.USAGE, f"{_named(opts, 'ngl', '-ngl')} {ngl}: only a full offload (or 0) is served; trunk layers are not split")
    devs = [] if ngl == "0" else _devices(opts.get("dev"), n_visible, _named(opts, "dev", "-dev"))
    from . import levers
    tp = int(levers.get("BLOOMERY_TP"))
    if tp > 0 and devs and not opts.get("dev"):
        # the lever names how many of the visible devices run in lockstep when -dev does not
        if tp > len(devs):
            raise Refusal(Code.USAGE, f"BLOOMERY_TP={tp}: only {len(devs)} device(s) are visible")
        devs = devs[:tp]
    pl = Placement(devices=devs, main_gpu=int(opts.get("main_gpu") or 0))
    word = (opts.get("place") or "").lower()
    if not devs:
        pl.mode = "cpu"
    elif word in ("", "a", "gate"):
        pl.mode = "a" if len(devs) == 1 or sm == "none" else "tp"
        if sm == "none":
            pl.devices = [devs[min(pl.main_gpu, len(devs) - 1)]]
    elif word in ("tp", "bp", "ep"):
        pl.mode = "tp"
    else:
        try:
            pl.devices = _devices(word, n_visible)
            pl.mode = "tp" if len(pl.devices) > 1 else "a"
        except Refusal:
            raise Refusal(Code.USAGE, f"--place {word!r}: expected a, gate, bp, tp or a device list") from None
    ts = opts.get("tensor_split")
    if ts:
        try:
            shares = [float(x) for x in re.split(r"[,/]", ts)]
        except ValueError:
            raise Refusal(Code.USAGE, f"{_named(opts, 'tensor_split', '-ts')} {ts!r}: expected numbers separated by commas") from None
        if len(shares) != len(pl.devices) or min(shares) < 0 or sum(shares) <= 0:
            raise Refusal(Code.USAGE, f"{_named(opts, 'tensor_split', '-ts')} {ts!r}: need one non-negative share per device ({len(pl.devices)})")
        tot = sum(shares)
        pl.expert_shares = [s / tot for s in shares]
    if opts.get("cpu_moe"):
        pl.host_experts = "all"
    elif int(opts.get("n_cpu_moe") or 0) > 0:
        pl.host_experts = f"first:{int(opts['n_cpu_moe'])}"
    ot = opts.get("override_tensor")
    if ot:
        pat, eq, where = ot.rpartition("=")
        if not eq or where.upper() != "CPU":
            raise Refusal(Code.USAGE, f"{_named(opts, 'override_tensor', '-ot')} {ot!r}: only <expert tensor pattern>=CPU is served")
        if "exps" not in pat and "expert" not in pat:
            raise Refusal(Code.USAGE, f"{_named(opts, 'override_tensor', '-ot')} {ot!r}: only routed-expert tensors may stay on the host")
        pl.host_experts, pl.host_pattern = "pattern", pat
    fit = str(opts.get("fit") or "off").lower()
    if fit not in ("on", "off"):
        raise Refusal(Code.USAGE, f"{_named(opts, 'fit', '-fit')} {fit!r}: expected on or off")
    pl.fit = fit == "on"
    if opts.get("fit_target"):
        try:
            pl.fit_targets_mib = [int(x) for x in str(opts["fit_target"]).split(",")]
        except ValueError:
            raise Refusal(Code.USAGE, f"{_named(opts, 'fit_target', '-fitt')} {opts['fit_target']!r}: expected MiB[,MiB...]") from None
    pl.fit_ctx = int(opts.get("fit_ctx") or 4096)
    if opts.get("dev_draft"):
        pl.draft_device = _devices(opts["dev_draft"], n_visible)[0]
    return pl


def usage() -> str:
    return "\n".join(f"  {', '.join(f.names):38s} {f.help}" for f in FLAGS)
