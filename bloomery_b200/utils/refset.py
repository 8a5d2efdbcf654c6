"""Reference sets: greedy continuations of fixed prompts, stored with the identity of the model they
were made from, so another engine (or another build) can be checked against them later.

A set is a JSON file: ``{"schema": "bloomery.refset/1", "model_sha256": ..., "arch": ..., "cases": [{"prompt": [...],
"greedy": [...]}]}``.  ``check`` refuses a set made from another model file before comparing a token
(the reference keeps readers and identity checks for its oracle sets in ``crates/refset/src/lib.rs:1-50``;
its sets come from external oracles, these come from the plain PyTorch model in ``models/cpu_ref.py``).

    python -m bloomery_b200.utils.refset make  MODEL OUT.json [--cases 4] [--prompt-len 32] [--new 16]
    python -m bloomery_b200.utils.refset check MODEL SET.json [--device cuda:0]
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from typing import Callable, Dict, List, Sequence

SCHEMA = "bloomery.refset/1"


class RefsetError(ValueError):
    pass


def model_identity(path: str) -> str:
    """SHA-256 over the model's file(s): a GGUF file (all shards of a split) or every file of a folder, by name order."""
    h = hashlib.sha256()
    if os.path.isdir(path):
        files = sorted(os.path.join(path, n) for n in os.listdir(path) if n.endswith((".safetensors", ".json")))
    else:
        from ..formats.gguf import split_paths
        files = split_paths(path) or [path]
    for fp in files:
        h.update(os.path.basename(fp).encode())
        with open(fp, "rb") as f:
            for chunk in iter(lambda: f.read(1 << 20), b""):
                h.update(chunk)
    return h.hexdigest()


def make(path: str, generate: Callable[[List[int], int], List[int]], vocab: int, arch: str, n_cases: int = 4,
         prompt_len: int = 32, n_new: int = 16, seed: int = 0) -> Dict[str, object]:
    import random
    rng = random.Random(seed)
    cases = []
    for _ in range(n_cases):
        prompt = [rng.randrange(vocab) for _ in range(prompt_len)]
        cases.append({"prompt": prompt, "greedy": [int(t) for t in generate(prompt, n_new)]})
    return {"schema": SCHEMA, "model_sha256": model_identity(path), "arch": arch, "cases": cases}


def read(set_path: str) -> Dict[str, object]:
    try:
        doc = json.load(open(set_path))
    except (OSError, ValueError) as exc:
        raise RefsetError(f"{set_path}: {exc}") from None
    if doc.get("schema") != SCHEMA or not isinstance(doc.get("cases"), list):
        raise RefsetError(f"{set_path}: not a {SCHEMA} file")
    for c in doc["cases"]:
        if not isinstance(c.get("prompt"), list) or not isinstance(c.get("greedy"), list):
            raise RefsetError(f"{set_path}: a case lacks prompt / greedy ids")
    return doc


def check(doc: Dict[str, object], path: str, generate: Callable[[List[int], int], List[int]], min_agree: float = 1.0):
    """Compare ``generate`` with the set; returns (agreeing tokens, total).  Raises when the set was made from
    another model or the agreement is below ``min_agree`` (tokens count up to the first difference of a case:
    after it the two texts are different sequences)."""
    if doc["model_sha256"] != model_identity(path):
        raise RefsetError("the set was made from another model file (sha256 differs)")
    agree = total = 0
    for c in doc["cases"]:
        want: Sequence[int] = c["greedy"]
        got = generate(list(c["prompt"]), len(want))
        n = 0
        while n < len(want) and n < len(got) and int(got[n]) == int(want[n]):
            n += 1
        agree += n
        total += len(want)
    if total and agree / total < min_agree:
        raise RefsetError(f"{agree} of {total} tokens agree, below {min_agree:.2f}")
    return agree, total


def _generator(path: str, device: str):
    from ..models.weights import open_model
    spec, w, _ = open_model(path, device)
    if device == "cpu":
        from ..models.cpu_ref import CpuModel
        m = CpuModel(w)

        def gen(prompt, n):
            m.reset()
            return m.generate(prompt, n)
    else:
        from ..runtime.engine import DecodeEngine
        eng = DecodeEngine(w, n_slots=1, slot_ctx=4096)

        def gen(prompt, n):
            eng.reset(0)
            first = eng.prefill(0, prompt, gemm=False)
            return [first] + eng.decode_chain(0, first, len(prompt), n - 1) if n > 1 else [first]
    return spec, gen


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="refset")
    ap.add_argument("cmd", choices=["make", "check"])
    ap.add_argument("model")
    ap.add_argument("set")
    ap.add_argument("--cases", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=32)
    ap.add_argument("--new", type=int, default=16)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--min-agree", type=float, default=0.9)
    a = ap.parse_args(argv)
    spec, gen = _generator(a.model, a.device)
    if a.cmd == "make":
        doc = make(a.model, gen, spec.vocab, spec.arch, a.cases, a.prompt_len, a.new)
        json.dump(doc, open(a.set, "w"))
        print(f"wrote {len(doc['cases'])} cases to {a.set}")
        return 0
    try:
        agree, total = check(read(a.set), a.model, gen, a.min_agree)
    except RefsetError as exc:
        print(f"refset: {exc}", file=sys.stderr)
        return 1
    print(f"{agree} of {total} tokens agree")
    return 0


if __name__ == "__main__":
    sys.exit(main())
