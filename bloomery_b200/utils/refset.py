"""Reference sets: greedy continuations of fixed prompts, stored with the identity of the model they
were made from, so another engine (or another build) can be checked against them later.

A set is a JSON file: ``{"schema": "bloomery.refset/1", "model_sha256": ..., "arch": ..., "cases": [{"prompt": [...],
"greedy": [...]}]}``.  ``check`` refuses a set made from another model file before comparing a token
(the reference keeps readers and identity checks for its oracle sets in ``crates/refset/src/lib.rs:1-50``;
its sets come from external oracles, these come from the plain PyTorch model in ``models/cpu_ref.py``).

A second kind, ``"kind": "logits"``, keeps for every position of every case the oracle's ``top`` most likely ids with
their log-probabilities.  ``check_logits`` runs the positions teacher-forced and reports the mean and the largest KL
divergence over that support (the tail's mass as one bucket), and sorts every position where the arg-max differs by the
flip rule: when the oracle's lead of its first over its second id is under ``flip_margin`` nats the difference is a
flip (two engines that round differently may pick either), otherwise it is a miss; misses fail the check, flips only
count.

    python -m bloomery_b200.utils.refset make  MODEL OUT.json [--cases 4] [--prompt-len 32] [--new 16] [--logits]
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


def make_logits(path: str, logits: Callable[[List[int]], "object"], vocab: int, arch: str, n_cases: int = 4,
                prompt_len: int = 32, top: int = 16, seed: int = 0) -> Dict[str, object]:
    """``logits(ids)`` -> [len(ids), vocab] teacher-forced logits of the oracle."""
    import random

    import torch
    rng = random.Random(seed)
    cases = []
    for _ in range(n_cases):
        prompt = [rng.randrange(vocab) for _ in range(prompt_len)]
        lp = torch.log_softmax(torch.as_tensor(logits(prompt)).double(), dim=-1)
        v, i = lp.topk(top, dim=-1)
        cases.append({"prompt": prompt, "top_ids": i.tolist(), "top_logp": [[round(x, 6) for x in row] for row in v.tolist()]})
    return {"schema": SCHEMA, "kind": "logits", "model_sha256": model_identity(path), "arch": arch, "top": top, "cases": cases}


def check_logits(doc: Dict[str, object], path: str, logits: Callable[[List[int]], "object"], max_mean_kld: float = 0.05,
                 flip_margin: float = 0.05) -> Dict[str, float]:
    """Returns ``{"mean_kld", "max_kld", "positions", "flips", "misses"}``; raises on another model, a mean divergence above
    ``max_mean_kld``, or a miss."""
    import math

    import torch
    if doc.get("kind") != "logits":
        raise RefsetError("not a logits set")
    if doc["model_sha256"] != model_identity(path):
        raise RefsetError("the set was made from another model file (sha256 differs)")
    klds, flips, misses = [], 0, 0
    for c in doc["cases"]:
        got = torch.log_softmax(torch.as_tensor(logits(list(c["prompt"]))).double(), dim=-1)
        ids = torch.tensor(c["top_ids"])
        want = torch.tensor(c["top_logp"], dtype=torch.float64)
        if got.shape[0] != ids.shape[0]:
            raise RefsetError(f"{got.shape[0]} positions where the set holds {ids.shape[0]}")
        q = got.gather(1, ids)
        p = want.exp()
        # the support's terms, then the rest of the mass as one bucket
        kl = (p * (want - q)).sum(1)
        p_tail, q_tail = (1 - p.sum(1)).clamp_min(1e-12), (1 - q.exp().sum(1)).clamp_min(1e-12)
        kl = kl + p_tail * (p_tail.log() - q_tail.log())
        klds += kl.clamp_min(0).tolist()
        pick = got.argmax(1)
        for t in torch.nonzero(pick != ids[:, 0]).flatten().tolist():
            if float(want[t, 0] - want[t, 1]) < flip_margin:
                flips += 1
            else:
                misses += 1
    out = {"mean_kld": sum(klds) / max(1, len(klds)), "max_kld": max(klds, default=0.0), "positions": len(klds),
           "flips": flips, "misses": misses}
    if misses:
        raise RefsetError(f"{misses} of {len(klds)} positions pick another id where the oracle's lead is {flip_margin} nats or more")
    if not math.isfinite(out["mean_kld"]) or out["mean_kld"] > max_mean_kld:
        raise RefsetError(f"mean KL divergence {out['mean_kld']:.4f} is above {max_mean_kld}")
    return out


def _logits_fn(path: str, device: str):
    """Teacher-forced logits of a model file: the plain PyTorch model on the CPU, the decode engine row by row on a card."""
    import torch
    from ..models.weights import open_model
    spec, w, _ = open_model(path, device)
    if device == "cpu":
        from ..models.cpu_ref import CpuModel
        m = CpuModel(w)

        def fn(ids):
            m.reset()
            return m.forward(torch.tensor(ids))
    else:
        from ..runtime.engine import DecodeEngine
        eng = DecodeEngine(w, n_slots=1, slot_ctx=4096)

        def fn(ids):
            eng.reset(0)
            rows = []
            for pos, tok in enumerate(ids):
                eng.step([(0, int(tok), pos)])
                rows.append(eng.logits[0].float().cpu().clone())
            return torch.stack(rows)
    return spec, fn


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
    ap.add_argument("--logits", action="store_true", help="make: keep the oracle's top log-probabilities instead of greedy ids")
    ap.add_argument("--max-kld", type=float, default=0.05)
    ap.add_argument("--flip-margin", type=float, default=0.05)
    a = ap.parse_args(argv)
    if a.cmd == "make" and a.logits:
        spec, fn = _logits_fn(a.model, a.device)
        doc = make_logits(a.model, fn, spec.vocab, spec.arch, a.cases, a.prompt_len)
        json.dump(doc, open(a.set, "w"))
        print(f"wrote {len(doc['cases'])} cases of log-probabilities to {a.set}")
        return 0
    if a.cmd == "check":
        try:
            peek = json.load(open(a.set))
        except (OSError, ValueError) as exc:
            print(f"refset: {a.set}: {exc}", file=sys.stderr)
            return 1
        if isinstance(peek, dict) and peek.get("kind") == "logits":
            _, fn = _logits_fn(a.model, a.device)
            try:
                got = check_logits(peek, a.model, fn, a.max_kld, a.flip_margin)
            except RefsetError as exc:
                print(f"refset: {exc}", file=sys.stderr)
                return 1
            print(f"mean KLD {got['mean_kld']:.5f}, max {got['max_kld']:.5f} over {got['positions']} positions, {got['flips']} flips")
            return 0
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
