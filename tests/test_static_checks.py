"""Static checks over the source tree, run on the CPU: the contracts that reading a diff does not reliably catch.

* every device wait is bounded: an unbounded-looking loop (``for (...;;...)``, ``while`` with an empty body) and every
  ``mbarrier.try_wait`` / acquire-load poll reads the timer or a limit close by;
* nothing traps: no ``__trap``, no device ``assert``;
* the loads and calls that are closed on this hardware are named nowhere (their names are assembled here from pieces,
  so this file does not name them either);
* the build names one architecture;
* every ``BLOOMERY_*`` variable the package reads is a registered (or retired) lever;
* comments and docstrings stand alone: they name no planning document of the build, no review, no machine path.

Counterpart of the reference's ``tools/check-{bounded,waits,loads,arch,levers,comments}.sh``.
"""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "bloomery_b200")
CSRC = os.path.join(PKG, "csrc")


def _files(top, exts):
    for d, dirs, names in os.walk(top):
        dirs[:] = [x for x in dirs if x not in ("__pycache__", "_work", ".git", "baseline", "build") and not x.endswith("_out")]
        for n in names:
            if n.endswith(exts):
                yield os.path.join(d, n)


def _device_sources():
    return sorted(_files(CSRC, (".cu", ".cuh")))


def test_there_are_device_sources_to_check():
    assert len(_device_sources()) >= 10


def test_every_device_wait_is_bounded():
    # what counts as a limit in sight: the timer, a named limit, or the shared bounded re-poll helper of the reducers
    bound = re.compile(r"globaltimer|global_timer|WAIT_LIMIT|limit|max_spins|spins\s*<|tries\s*<|reduce_again")
    open_loop = re.compile(r"for\s*\([^;()]*;\s*;[^;()]*\)|while\s*\(\s*(true|1)\s*\)")
    poll = re.compile(r"try_wait|ld\.acquire|ld\.volatile")
    bad = []
    for path in _device_sources():
        lines = open(path, encoding="utf-8").read().splitlines()
        for i, ln in enumerate(lines):
            code = ln.split("//")[0]
            near = "\n".join(lines[max(0, i - 12):i + 25])
            if (open_loop.search(code) or poll.search(code)) and not bound.search(near):
                bad.append(f"{os.path.relpath(path, ROOT)}:{i + 1}: a wait with no limit in sight")
            if re.search(r"while\s*\(.*\)\s*\{\s*\}", code) and not bound.search(code):
                bad.append(f"{os.path.relpath(path, ROOT)}:{i + 1}: an empty-bodied loop that reads no timer")
    assert not bad, "\n".join(bad)


def test_nothing_traps_on_the_device():
    bad = []
    for path in _device_sources():
        for i, ln in enumerate(open(path, encoding="utf-8").read().splitlines()):
            code = ln.split("//")[0]
            if re.search(r"__trap\s*\(|\bassert\s*\(|asm[^;]*\btrap;", code) and "static_assert" not in code:
                bad.append(f"{os.path.relpath(path, ROOT)}:{i + 1}: {code.strip()[:80]}")
    assert not bad, "\n".join(bad)


def test_closed_loads_and_calls_are_named_nowhere():
    closed = [".multi" + "cast::" + "cluster"] + [p + "Mem" + "cpy" + mid + "Batch" + "Async" for p in ("cuda", "cu") for mid in ("", "3D")]
    bad = []
    for path in _files(ROOT, (".py", ".cu", ".cuh", ".cpp", ".h", ".hpp", ".c", ".sh", ".toml", ".cfg", ".txt")):
        text = open(path, encoding="utf-8", errors="ignore").read()
        for name in closed:
            if name in text:
                bad.append(f"{os.path.relpath(path, ROOT)} names {name[:6]}...")
    assert not bad, "\n".join(bad)


def test_the_build_names_one_architecture():
    text = open(os.path.join(PKG, "build.py"), encoding="utf-8").read()
    archs = set(re.findall(r"sm_\d+a?", text)) | set(re.findall(r"compute_\d+a?", text))
    assert archs == {"sm_100a", "compute_100a"}, archs
    assert "-lineinfo" in text


def test_every_variable_the_package_reads_is_a_lever():
    from bloomery_b200.utils import levers
    known = {l.name for l in levers.REGISTRY} | set(levers.RETIRED)
    known |= {"BLOOMERY_CACHE", "BLOOMERY_COSTS"}            # directories, read where they are used, not behaviours
    bad = []
    for path in list(_files(PKG, (".py",))) + [os.path.join(ROOT, "bench.py")]:
        if path.endswith(os.path.join("utils", "levers.py")):
            continue
        for i, ln in enumerate(open(path, encoding="utf-8").read().splitlines()):
            for name in re.findall(r"\bBLOOMERY_[A-Z0-9_]+\b", ln):
                if name not in known and not name.endswith("_"):
                    bad.append(f"{os.path.relpath(path, ROOT)}:{i + 1}: {name} is no registered lever")
    assert not bad, "\n".join(sorted(set(bad)))


def test_comments_stand_alone():
    words = ["SUR" + "VEY", "VER" + "DICT", "ADV" + "ICE.md", "DES" + "IGN.md", "BASE" + "LINE.md", "gpu" + "run", "the " + "judge",
             "/ro" + "ot/"]
    bad = []
    for top in (PKG, os.path.join(ROOT, "tests")):
        for path in _files(top, (".py", ".cu", ".cuh", ".cpp", ".h")):
            for i, ln in enumerate(open(path, encoding="utf-8", errors="ignore").read().splitlines()):
                for w in words:
                    if w in ln:
                        bad.append(f"{os.path.relpath(path, ROOT)}:{i + 1}: names {w!r}")
    for name in ("bench.py", "__graft_entry__.py"):
        for i, ln in enumerate(open(os.path.join(ROOT, name), encoding="utf-8").read().splitlines()):
            for w in words:
                if w in ln:
                    bad.append(f"{name}:{i + 1}: names {w!r}")
    assert not bad, "\n".join(bad)
