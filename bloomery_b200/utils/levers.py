"""Levers: typed ``BLOOMERY_*`` environment settings, parsed once at start, refused by name
on a bad value or a retired name, listed by ``--levers`` (``crates/levers/src/lib.rs:1-26``,
rows of ``registry.rs``)."""
from __future__ import annotations

import dataclasses
import os
from typing import Any, Callable, Dict, List, Optional

from .exit_codes import Code, Refusal


@dataclasses.dataclass(frozen=True)
class LeverSpec:
    name: str
    kind: str          # bool | int | float | bytes | word | str
    default: Any
    doc: str
    choices: Optional[tuple] = None
    phase: str = "start"


def _parse_bytes(v: str) -> int:
    v = v.strip()
    mult = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30, "t": 1 << 40}
    low = v.lower().rstrip("ib")
    if low and low[-1] in mult:
        return int(float(low[:-1]) * mult[low[-1]])
    return int(v)


_PARSERS: Dict[str, Callable[[str], Any]] = {
    "bool": lambda v: {"1": True, "0": False, "on": True, "off": False, "true": True, "false": False}[v.lower()],
    "int": int, "float": float, "bytes": _parse_bytes, "word": str, "str": str,
}

REGISTRY: List[LeverSpec] = [
    LeverSpec("BLOOMERY_DRAFT", "word", "auto", "speculative draft source (lookup = the n-gram lookup draft, also spelled ngram)", ("auto", "off", "mtp", "ngram", "lookup")),
    LeverSpec("BLOOMERY_SCREEN", "word", "on", "draw the start screen below the record lines when stderr is a terminal", ("on", "off")),
    LeverSpec("BLOOMERY_WATCH_CALLS", "word", "on", "hold a free reply's tool calls to their schemas from the call opener on", ("on", "off")),
    LeverSpec("BLOOMERY_RESIDENCY", "word", "mid", "hot-expert promotion rule", ("off", "low", "mid", "high")),
    LeverSpec("BLOOMERY_CARD_BUDGET", "bytes", 0, "HBM bytes routed experts may take per GPU (0 = what fits)"),
    LeverSpec("BLOOMERY_CARD_MARGIN", "bytes", 1 << 30, "HBM bytes the plan leaves free per GPU"),
    LeverSpec("BLOOMERY_HOST_ROOM", "bytes", 0, "pinned host bytes for cold experts (0 = as needed)"),
    LeverSpec("BLOOMERY_KV_FLOOR", "int", 8192, "positions a slot keeps on the card before KV may spill"),
    LeverSpec("BLOOMERY_KV_HOST", "word", "off", "KV pages beyond the margin", ("off", "spill")),
    LeverSpec("BLOOMERY_THREADS", "int", 0, "worker pool size of the host expert leg (0 = allowed CPUs)"),
    LeverSpec("BLOOMERY_PIN", "bool", True, "pin pool workers to CPUs"),
    LeverSpec("BLOOMERY_SPIN", "int", 20000, "pool spins before a worker parks"),
    LeverSpec("BLOOMERY_UBATCH", "int", 4096, "rows per prompt micro-batch"),
    LeverSpec("BLOOMERY_PREFILL", "word", "batch", "prompt path", ("batch", "steps")),
    LeverSpec("BLOOMERY_PREFILL_BF16", "word", "auto", "resident bf16 copy of the weights for the prompt path (auto = when it leaves a quarter of the card free)", ("auto", "0", "1")),
    LeverSpec("BLOOMERY_FP8_NATIVE", "bool", True, "batched pass: FP8 128x128 weights multiply E4M3 activations on the tensor cores (off = expand the weights to bf16 in flight)"),
    LeverSpec("BLOOMERY_NEED_HOOK", "str", "", "absolute path of a program run once per placed load with the need line on its standard input (exit 0 goes on, 75 = ask again later)"),
    LeverSpec("BLOOMERY_HOST_NATIVE", "bool", True, "-dev none: decode through the native host step where it covers the model (off = the plain PyTorch model)"),
    LeverSpec("BLOOMERY_PDL", "bool", True, "programmatic dependent launch between decode kernels"),
    LeverSpec("BLOOMERY_FLASH_MMA", "bool", False, "decode attention segments on tensor-core tiles (f16 queries and probabilities)"),
    LeverSpec("BLOOMERY_GRAPHS", "bool", True, "one CUDA graph per decode step"),
    LeverSpec("BLOOMERY_MTP_WIDTH", "int", 0, "draft ids per speculative pass (0 = chooser decides)"),
    LeverSpec("BLOOMERY_AUTOTUNE", "bool", True, "race equal kernel variants at load"),
    LeverSpec("BLOOMERY_POISON", "bool", False, "fill scratch with NaN so a missed cell shows"),
    LeverSpec("BLOOMERY_CHECK_FINITE", "bool", False, "check activations for non-finite values each layer"),
    LeverSpec("BLOOMERY_PROFILE", "int", 0, "CPU profiler level 0..2"),
    LeverSpec("BLOOMERY_STEP_STATS", "bool", False, "print per-step wait and residency statistics"),
    LeverSpec("BLOOMERY_TP", "int", 0, "tensor-parallel ranks (0 = from -dev / -ts)"),
    LeverSpec("BLOOMERY_FUSED_COMM", "bool", True, "reductions fused into kernels over NVLink (off = NCCL baseline)"),
    LeverSpec("BLOOMERY_ENGINE_BOUND", "float", 60.0, "seconds an engine-thread wait may last"),
    LeverSpec("BLOOMERY_ROUTE_TRACE", "str", "", "directory for per-position router traces"),
    LeverSpec("BLOOMERY_TP_PORT", "int", 0, "rendezvous port of the lockstep ranks on 127.0.0.1 (0 = derived from the pid)"),
    LeverSpec("BLOOMERY_STAGED", "bool", True, "decode kernels that stage their weight rows in shared memory with bulk copies"),
    LeverSpec("BLOOMERY_STAGED_PARTS", "str", "attn,prefetch", "which launches take the staged form: gemv, attn, moe, prefetch (L2 prefetches), cluster (one-row expert half as one cluster launch)"),
]
RETIRED = {"BLOOMERY_WORD_OPS": "stream memops are not used on this build", "BLOOMERY_TIER_LINK": "there is no host-page link: GPUs talk over NVLink",
           "BLOOMERY_TIER_NODES": "multi-machine tiers are not built", "BLOOMERY_TP_NODES": "TP ranks come from torchrun, not from a node list"}
_BY_NAME = {l.name: l for l in REGISTRY}
_values: Dict[str, Any] = {}


def at_main(environ=None) -> Dict[str, Any]:
    """Parse every lever once; refuse bad values, unknown and retired ``BLOOMERY_*`` names."""
    env = os.environ if environ is None else environ
    vals = {l.name: l.default for l in REGISTRY}
    for k, v in env.items():
        if not k.startswith("BLOOMERY_"):
            continue
        if k in RETIRED:
            raise Refusal(Code.LEVER, f"{k} is retired: {RETIRED[k]}")
        spec = _BY_NAME.get(k)
        if spec is None:
            raise Refusal(Code.LEVER, f"{k} is not a lever of this server (see --levers)")
        try:
            val = _PARSERS[spec.kind](v)
        except (ValueError, KeyError):
            raise Refusal(Code.LEVER, f"{k}={v!r}: expected a {spec.kind}") from None
        if spec.choices and val not in spec.choices:
            raise Refusal(Code.LEVER, f"{k}={v!r}: expected one of {', '.join(spec.choices)}")
        vals[k] = val
    launch_queues(env)
    _values.clear()
    _values.update(vals)
    return vals


LAUNCH_QUEUES = ("0.25x", "0.5x", "2x", "4x")


def launch_queues(env) -> str:
    """The CUDA driver's ``CUDA_SCALE_LAUNCH_QUEUES``: unset it becomes ``2x`` (a deeper launch queue per stream, so the
    host thread of a prompt batch's many launches does not wait on it); NVIDIA's other values are kept; anything else
    stops the start with a message, where the driver would ignore it.  Must run before the first CUDA call of the
    process (the driver reads the variable when it initialises)."""
    name = "CUDA_SCALE_LAUNCH_QUEUES"
    v = env.get(name)
    if v is None:
        env[name] = "2x"
        return "2x"
    if v not in LAUNCH_QUEUES:
        raise Refusal(Code.LEVER, f"{name}={v!r}: the driver takes {', '.join(LAUNCH_QUEUES)}")
    return v


def get(name: str):
    if not _values:
        at_main()
    return _values[name]


def listing() -> str:
    rows = [f"{l.name:28s} {l.kind:6s} default={l.default!s:12s} {l.doc}" + (f" [{'|'.join(l.choices)}]" if l.choices else "")
            for l in REGISTRY]
    return "\n".join(rows)
