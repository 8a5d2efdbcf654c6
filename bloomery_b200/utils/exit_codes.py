"""Exit-code table of the server (``crates/serve/src/exit.rs:60-95`` in the reference):
a supervisor tells a refusal that clears by itself from one that needs a human."""
from __future__ import annotations

import enum


class Code(enum.IntEnum):
    OK = 0
    REFUSED = 1
    USAGE = 64
    UNSUPPORTED = 65
    NO_MODEL = 66
    NO_DEVICE = 69
    ENGINE = 70
    NETWORK = 74
    RETRY = 75
    DENIED = 77
    LEVER = 78
    NO_FIT = 80
    CARD_BUSY = 81
    DISK_SHORT = 82
    LOAD = 83


WORDS = {
    Code.OK: ("ok", ""), Code.REFUSED: ("refused", "read the message"),
    Code.USAGE: ("usage", "run with --help; the message names the flag or value"),
    Code.UNSUPPORTED: ("unsupported", "run with --recommend --json for what this machine serves"),
    Code.NO_MODEL: ("no-model", "name a model with --model or -m; the message lists what exists"),
    Code.NO_DEVICE: ("no-device", "the message names the driver, device or CPU feature that is missing"),
    Code.ENGINE: ("engine", "restart the server; the crash block names the failure"),
    Code.NETWORK: ("network", "check the connection"), Code.RETRY: ("retry", "retry later"),
    Code.DENIED: ("denied", "check the credentials"),
    Code.LEVER: ("lever", "the message names the lever and the kind of value it takes"),
    Code.NO_FIT: ("no-fit", "choose a smaller variant, a smaller context or fewer slots"),
    Code.CARD_BUSY: ("card-busy", "retry when the process holding the card ends"),
    Code.DISK_SHORT: ("disk-short", "free disk space"), Code.LOAD: ("load", "the model file could not be loaded"),
}


class Refusal(Exception):
    """A start-up refusal that carries its exit code."""

    def __init__(self, code: Code, message: str):
        super().__init__(message)
        self.code = code
