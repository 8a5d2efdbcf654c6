"""What a server checks before it loads anything: that the CPU runs the host library, that the NVIDIA driver runs the
CUDA code, and what it says when no card is in view.

The verdicts are pure functions of what the caller read (the CPU's feature words, the driver's version string, the
listed cards), so they are tested without the hardware; the readers beside them only read (``/proc/cpuinfo``,
``/proc/driver/nvidia/version``, torch's device list) and change nothing.  A refusal is of the class ``no-device``
(``utils/exit_codes.py``) and names the missing CPU feature, the driver version, or the cards that are listed but not
visible.  (The reference: ``crates/serve/src/preflight.rs`` -- ``cpu_gate``, ``driver``, ``no_card``.)
"""
from __future__ import annotations

import os
import re
from typing import Iterable, List, Optional, Sequence, Tuple

# libbloomery_host.so is compiled with -mavx2 -mfma -mf16c: x86-64-v3's vector part
CPU_NEEDS = ("avx2", "fma", "f16c")
# sm_100a cubins of CUDA 12.8+ load on the R570 branch and later
DRIVER_MIN = (570, 0)


def cpu_gate(flags: Iterable[str], machine: str = "x86_64") -> Optional[str]:
    """None when the CPU runs the host code, else the message of the refusal."""
    if machine not in ("x86_64", "AMD64"):
        return None                                   # the host library is built without the x86 vector paths elsewhere
    have = set(flags)
    lacks = [f for f in CPU_NEEDS if f not in have]
    if lacks:
        return (f"this CPU lacks {', '.join(lacks)}: the host library is built for x86-64-v3 "
                f"(AVX2, FMA, F16C) and would stop on an illegal instruction")
    return None


def parse_driver(text: str) -> Optional[Tuple[int, int]]:
    """(major, minor) of the first version-looking number in a driver string ('580.159', 'NVRM version: ... 570.86.15 ...')."""
    m = re.search(r"(\d{3})\.(\d+)(?:\.\d+)?", text or "")
    return (int(m.group(1)), int(m.group(2))) if m else None


def driver_gate(version_text: Optional[str], need: Tuple[int, int] = DRIVER_MIN) -> Optional[str]:
    """None when the driver is new enough (or unreadable: the load itself will tell), else the refusal's message."""
    if not version_text:
        return None
    v = parse_driver(version_text)
    if v is None:
        return None
    if v < need:
        return (f"the NVIDIA driver is {v[0]}.{v[1]}; this build's sm_100a code needs R{need[0]} or later "
                f"(update the driver, or run with -dev none)")
    return None


def no_card(visible: int, listed: Sequence[str], asked: str = "") -> Optional[str]:
    """The message when no card is in view: names what nvidia-smi lists (a container without the devices mapped, a
    CUDA_VISIBLE_DEVICES that hides them) or says that the machine has none.  None when a card is visible."""
    if visible > 0:
        return None
    hidden = os.environ.get("CUDA_VISIBLE_DEVICES")
    if listed:
        why = f" (CUDA_VISIBLE_DEVICES={hidden!r} hides them)" if hidden is not None else " (are the devices mapped into this container?)"
        return f"no CUDA device is visible, but the driver lists {len(listed)}: {', '.join(listed)}{why}"
    tail = f"; -dev {asked} cannot be served" if asked and asked != "none" else ""
    return f"no CUDA device on this machine{tail}; use -dev none for the CPU engine"


def read_cpu_flags(path: str = "/proc/cpuinfo") -> List[str]:
    try:
        with open(path) as fh:
            for ln in fh:
                if ln.startswith("flags"):
                    return ln.split(":", 1)[1].split()
    except OSError:
        pass
    return []


def read_driver(path: str = "/proc/driver/nvidia/version") -> Optional[str]:
    try:
        with open(path) as fh:
            return fh.read()
    except OSError:
        return None


def run(n_visible: int, dev_word: str = "") -> Optional[str]:
    """All gates in order on what this machine reports; the first refusal's message, or None."""
    import platform
    flags = read_cpu_flags()
    if flags:
        msg = cpu_gate(flags, platform.machine())
        if msg:
            return msg
    if dev_word == "none":
        return None
    msg = driver_gate(read_driver())
    if msg:
        return msg
    return no_card(n_visible, [], dev_word)
