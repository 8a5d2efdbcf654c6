"""Slot files: a sequence state on disk (``POST /slots/{id}?action=save|restore``).

Format (``crates/serve/src/slotfile.rs:1-24`` names the same parts): magic ``BLSLOT01``,
version u32, n_vocab u32, token count u64, the ids as i32, then the engine payload as a
length-prefixed blob (torch-serialised tensors).  A file written for another vocabulary or
version is refused by name."""
from __future__ import annotations

import io
import struct
from typing import List, Tuple

import numpy as np

from .engine import Saved

MAGIC = b"BLSLOT01"
VERSION = 1


def _landed(payload) -> None:
    """A snapshot's device-to-host copies run behind the caller; wait for them before the bytes are serialised."""
    from ..runtime.kv import snap_ready
    if isinstance(payload, dict):
        snap_ready(payload)
        for v in payload.values():
            if isinstance(v, (dict, list)):
                _landed(v)
    elif isinstance(payload, list):
        for v in payload:
            _landed(v)


def write_slot_file(path: str, n_vocab: int, ids: List[int], saved: Saved) -> int:
    import torch
    buf = io.BytesIO()
    _landed(saved.payload if saved is not None else None)
    torch.save(saved.payload if saved is not None else None, buf)
    blob = buf.getvalue()
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<IIQ", VERSION, n_vocab, len(ids)))
        f.write(np.asarray(ids, dtype=np.int32).tobytes())
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        return f.tell()


def read_slot_file(path: str, n_vocab: int) -> Tuple[List[int], Saved]:
    import torch
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError(f"{path}: not a slot file")
        version, vocab, n = struct.unpack("<IIQ", f.read(16))
        if version != VERSION:
            raise ValueError(f"{path}: slot file version {version}, this build reads {VERSION}")
        if vocab != n_vocab:
            raise ValueError(f"{path}: written for a vocabulary of {vocab}, the model has {n_vocab}")
        ids = np.frombuffer(f.read(4 * n), dtype=np.int32).tolist()
        (nb,) = struct.unpack("<Q", f.read(8))
        payload = torch.load(io.BytesIO(f.read(nb)), weights_only=False)
    return ids, Saved(tuple(ids), payload, nb)
