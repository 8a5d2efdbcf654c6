"""Interleaved A/B timing of two commands: the variants run alternately (A B, B A, A B, ...) so that clock drift, a
warming card or a noisy neighbour hits both alike, and the answer is the medians, their ratio and how many rounds each
side won -- not two numbers taken minutes apart.

Each command prints its own figure; the harness reads the last match of ``--pattern`` (default: the ``us per layer``
line of ``ops/kernel_bench.py``, else the ``"value"`` of a ``bench.py`` JSON line) from its output.

    python -m bloomery_b200.ops.ab --rounds 5 \\
        "python -m bloomery_b200.ops.kernel_bench qgu 4 64 --rows 32" \\
        "python -m bloomery_b200.ops.kernel_bench fgu 4 64 --rows 32"

The reference's counterpart is its A/B runner among the timing scripts (``tools/ref/*.sh``: interleaved arms on one
leased machine).
"""
from __future__ import annotations

import argparse
import json
import re
import shlex
import statistics
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

PATTERNS = (r"us per layer:\s*([0-9.eE+-]+)", r'"value":\s*([0-9.eE+-]+)')


class AbError(RuntimeError):
    pass


def figure(text: str, pattern: Optional[str] = None) -> float:
    """The last figure a command printed."""
    for pat in ((pattern,) if pattern else PATTERNS):
        hits = re.findall(pat, text)
        if hits:
            return float(hits[-1])
    raise AbError("the command printed no figure the pattern matches")


def run_once(cmd: str, pattern: Optional[str], timeout: float) -> float:
    try:
        done = subprocess.run(shlex.split(cmd), capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        raise AbError(f"{cmd!r} ran past {timeout:.0f} s") from None
    if done.returncode != 0:
        raise AbError(f"{cmd!r} exited {done.returncode}: {done.stderr.strip()[-300:]}")
    return figure(done.stdout + "\n" + done.stderr, pattern)


def compare(a: Sequence[float], b: Sequence[float], higher_is_better: bool = False) -> Dict[str, object]:
    """Medians, spread and the per-round outcomes of two interleaved series (round i pairs a[i] with b[i])."""
    if len(a) != len(b) or not a:
        raise AbError("two series of the same, non-zero length")
    better = (lambda x, y: x > y) if higher_is_better else (lambda x, y: x < y)
    wins_a = sum(1 for x, y in zip(a, b) if better(x, y))
    wins_b = sum(1 for x, y in zip(a, b) if better(y, x))
    med_a, med_b = statistics.median(a), statistics.median(b)
    spread = lambda s: (max(s) - min(s)) / statistics.median(s) if statistics.median(s) else 0.0        # noqa: E731
    n = len(a)
    # two-sided sign test: the chance of a split at least this lopsided if the arms were the same
    k = max(wins_a, wins_b)
    decided = wins_a + wins_b
    from math import comb
    p = min(1.0, 2 * sum(comb(decided, i) for i in range(k, decided + 1)) / 2 ** decided) if decided else 1.0
    return {"rounds": n, "median_a": med_a, "median_b": med_b, "ratio_b_over_a": med_b / med_a if med_a else float("nan"),
            "spread_a": spread(a), "spread_b": spread(b), "wins_a": wins_a, "wins_b": wins_b, "sign_test_p": p,
            "winner": "same" if p > 0.1 or wins_a == wins_b else ("a" if wins_a > wins_b else "b")}


def interleave(cmd_a: str, cmd_b: str, rounds: int, pattern: Optional[str] = None, timeout: float = 900.0,
               run=run_once) -> Dict[str, List[float]]:
    a: List[float] = []
    b: List[float] = []
    for r in range(rounds):
        order = (("a", cmd_a), ("b", cmd_b)) if r % 2 == 0 else (("b", cmd_b), ("a", cmd_a))
        for which, cmd in order:
            (a if which == "a" else b).append(run(cmd, pattern, timeout))
    return {"a": a, "b": b}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ab", description=__doc__.split("\n\n")[0])
    ap.add_argument("a")
    ap.add_argument("b")
    ap.add_argument("--rounds", type=int, default=5)
    ap.add_argument("--pattern", default=None, help="regular expression with one group: the figure")
    ap.add_argument("--higher-is-better", action="store_true")
    ap.add_argument("--timeout", type=float, default=900.0)
    args = ap.parse_args(argv)
    try:
        series = interleave(args.a, args.b, args.rounds, args.pattern, args.timeout)
        out = compare(series["a"], series["b"], args.higher_is_better)
    except AbError as exc:
        print(f"ab: {exc}", file=sys.stderr)
        return 1
    out.update(series)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
