"""Safetensors files and checkpoint folders.

A file is an 8-byte little-endian header length, a JSON header
(``name -> {dtype, shape, data_offsets}``) and one data region; a folder is either one
``model.safetensors`` or ``model.safetensors.index.json`` naming the shard of every tensor,
beside ``config.json``.  Tensors are memory-mapped and handed out as torch views without a
copy (the reference: ``crates/safetensors/src/lib.rs`` ``Safetensors`` / ``Folder``).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# dtype tag -> (bytes per element, torch dtype used for the view)
_DTYPES = {
    "F64": (8, torch.float64), "F32": (4, torch.float32), "F16": (2, torch.float16),
    "BF16": (2, torch.bfloat16), "I64": (8, torch.int64), "I32": (4, torch.int32),
    "I16": (2, torch.int16), "I8": (1, torch.int8), "U8": (1, torch.uint8),
    "BOOL": (1, torch.bool), "F8_E4M3": (1, torch.uint8), "F8_E5M2": (1, torch.uint8),
    "F8_E8M0": (1, torch.uint8), "U16": (2, torch.int16), "U32": (4, torch.int32),
}
_TAG_OF = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
           torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
           torch.uint8: "U8", torch.bool: "BOOL"}
_MAX_HEADER = 100 << 20


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


class Safetensors:
    """One memory-mapped file."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than its own length field")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file")
        try:
            header = json.loads(self._f.read(hlen))
        except Exception as e:  # noqa: BLE001
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        self.tensors: Dict[str, TensorInfo] = {}
        spans: List[Tuple[int, int, str]] = []
        for name, d in header.items():
            try:
                dtype, shape, (b, e) = d["dtype"], tuple(int(x) for x in d["shape"]), d["data_offsets"]
            except Exception:  # noqa: BLE001
                raise SafetensorsError(f"{path}: malformed entry for {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: {name!r} has unknown dtype {dtype}")
            info = TensorInfo(name, dtype, shape, int(b), int(e))
            if info.begin > info.end or self._base + info.end > size:
                raise SafetensorsError(f"{path}: {name!r} lies outside the file")
            if info.numel * _DTYPES[dtype][0] != info.end - info.begin:
                raise SafetensorsError(f"{path}: {name!r} shape {shape} does not match its {info.end - info.begin} bytes")
            self.tensors[name] = info
            spans.append((info.begin, info.end, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: {n0!r} and {n1!r} overlap")

    def names(self) -> List[str]:
        return list(self.tensors)

    def raw(self, name: str) -> torch.Tensor:
        """The tensor's bytes as a uint8 view of the mapping."""
        t = self.tensors[name]
        if t.end == t.begin:
            return torch.empty(0, dtype=torch.uint8)
        arr = np.frombuffer(self._mm, dtype=np.uint8, count=t.end - t.begin, offset=self._base + t.begin)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # a read-only mapping: callers copy before they write
            return torch.from_numpy(arr)

    def tensor(self, name: str) -> torch.Tensor:
        """Typed view (8-bit float types come back as their uint8 codes)."""
        t = self.tensors[name]
        return self.raw(name).view(_DTYPES[t.dtype][1]).reshape(t.shape)

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass          # views still alive; the mapping goes with them
            self._mm = None
        self._f.close()


class Folder:
    """A checkpoint folder: config.json + one file or an index over shards."""

    INDEX = "model.safetensors.index.json"
    SINGLE = "model.safetensors"

    def __init__(self, path: str):
        self.path = path
        cfg = os.path.join(path, "config.json")
        self.config: dict = json.load(open(cfg)) if os.path.exists(cfg) else {}
        self._files: Dict[str, Safetensors] = {}
        self.where: Dict[str, str] = {}
        idx = os.path.join(path, self.INDEX)
        if os.path.exists(idx):
            wm = json.load(open(idx)).get("weight_map")
            if not isinstance(wm, dict) or not wm:
                raise SafetensorsError(f"{idx}: no weight_map")
            for shard in sorted(set(wm.values())):
                if os.path.basename(shard) != shard:
                    raise SafetensorsError(f"{idx}: shard name {shard!r} leaves the folder")
                if not os.path.exists(os.path.join(path, shard)):
                    raise SafetensorsError(f"{path}: shard {shard} named by the index is missing")
            self.where = dict(wm)
        elif os.path.exists(os.path.join(path, self.SINGLE)):
            st = self._open(self.SINGLE)
            self.where = {n: self.SINGLE for n in st.names()}
        else:
            raise SafetensorsError(f"{path}: neither {self.INDEX} nor {self.SINGLE}")

    def _open(self, shard: str) -> Safetensors:
        st = self._files.get(shard)
        if st is None:
            st = self._files[shard] = Safetensors(os.path.join(self.path, shard))
        return st

    def names(self) -> List[str]:
        return list(self.where)

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def info(self, name: str) -> TensorInfo:
        st = self._open(self.where[name])
        if name not in st.tensors:
            raise SafetensorsError(f"{self.path}: index places {name!r} in {self.where[name]}, which lacks it")
        return st.tensors[name]

    def tensor(self, name: str) -> torch.Tensor:
        self.info(name)
        return self._open(self.where[name]).tensor(name)

    def close(self) -> None:
        for st in self._files.values():
            st.close()
        self._files.clear()


def write_file(path: str, tensors: Dict[str, torch.Tensor], dtypes: Optional[Dict[str, str]] = None,
               metadata: Optional[Dict[str, str]] = None) -> None:
    """Fixture writer.  ``dtypes`` overrides the tag of uint8 tensors (``F8_E4M3`` planes)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        tag = (dtypes or {}).get(name) or _TAG_OF[t.dtype]
        b = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": tag, "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_folder(path: str, tensors: Dict[str, torch.Tensor], config: dict, shards: int = 1,
                 dtypes: Optional[Dict[str, str]] = None) -> None:
    os.makedirs(path, exist_ok=True)
    json.dump(config, open(os.path.join(path, "config.json"), "w"))
    names = list(tensors)
    if shards <= 1:
        write_file(os.path.join(path, Folder.SINGLE), tensors, dtypes)
        return
    per = (len(names) + shards - 1) // shards
    wm = {}
    for i in range(shards):
        part = names[i * per:(i + 1) * per]
        if not part:
            continue
        fn = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        write_file(os.path.join(path, fn), {n: tensors[n] for n in part}, dtypes)
        wm.update({n: fn for n in part})
    json.dump({"metadata": {}, "weight_map": wm}, open(os.path.join(path, Folder.INDEX), "w"))
