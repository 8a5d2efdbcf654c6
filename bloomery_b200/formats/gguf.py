"""GGUF v3 reader (mmap, strict + header-only inventory, split shards) and writer.

Counterpart of the reference's ``crates/gguf`` (``lib.rs:1-41``: ``Gguf::open``,
``Split``, ``inventory_of``; ``write.rs``).  Tensor dims are kept in ggml ``ne[]``
order (fastest first) exactly as the file stores them; ``TensorInfo.shape`` gives
the row-major (slowest first) view the rest of the framework uses.

Values are never converted on load: ``Gguf.tensor_bytes`` returns a zero-copy
uint8 view of the mapped file for every block type.
"""
from __future__ import annotations

import dataclasses
import hashlib
import mmap
import os
import re
import struct
from typing import Any, BinaryIO, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .quant import QTYPE_BY_ID, QTYPES, QType

GGUF_MAGIC = 0x46554747  # "GGUF" little-endian
GGUF_VERSION = 3
DEFAULT_ALIGNMENT = 32

# metadata value types
_T_U8, _T_I8, _T_U16, _T_I16, _T_U32, _T_I32, _T_F32, _T_BOOL, _T_STR, _T_ARR, _T_U64, _T_I64, _T_F64 = range(13)
_SCALAR_FMT = {
    _T_U8: "<B", _T_I8: "<b", _T_U16: "<H", _T_I16: "<h", _T_U32: "<I", _T_I32: "<i",
    _T_F32: "<f", _T_BOOL: "<?", _T_U64: "<Q", _T_I64: "<q", _T_F64: "<d",
}
_NP_DTYPE = {
    _T_U8: np.uint8, _T_I8: np.int8, _T_U16: np.uint16, _T_I16: np.int16, _T_U32: np.uint32,
    _T_I32: np.int32, _T_F32: np.float32, _T_BOOL: np.bool_, _T_U64: np.uint64, _T_I64: np.int64,
    _T_F64: np.float64,
}


class GgufError(ValueError):
    """A malformed or unsupported file; the message names the offending field."""


@dataclasses.dataclass
class TensorInfo:
    name: str
    ne: Tuple[int, ...]          # ggml order: ne[0] is the row length
    qtype: QType
    offset: int                  # from the start of the data section
    shard: int = 0

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(reversed(self.ne))

    @property
    def n_values(self) -> int:
        n = 1
        for d in self.ne:
            n *= d
        return n

    @property
    def row_bytes(self) -> int:
        return self.qtype.row_bytes(self.ne[0])

    @property
    def n_bytes(self) -> int:
        return self.n_values // self.ne[0] * self.row_bytes


class _Cursor:
    def __init__(self, buf, pos: int = 0):
        self.buf, self.pos = buf, pos

    def take(self, n: int) -> bytes:
        if self.pos + n > len(self.buf):
            raise GgufError(f"file ends inside the header at byte {self.pos}")
        b = self.buf[self.pos:self.pos + n]
        self.pos += n
        return b

    def scalar(self, t: int):
        fmt = _SCALAR_FMT.get(t)
        if fmt is None:
            raise GgufError(f"unknown metadata value type {t}")
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.scalar(_T_U64)
        if n > 1 << 30:
            raise GgufError(f"string of {n} bytes in the header")
        return bytes(self.take(n)).decode("utf-8", errors="replace")

    def value(self, t: int):
        if t == _T_STR:
            return self.string()
        if t == _T_ARR:
            et = self.scalar(_T_U32)
            n = self.scalar(_T_U64)
            if et == _T_STR:
                return [self.string() for _ in range(n)]
            if et == _T_ARR:
                return [self.value(_T_ARR) for _ in range(n)]
            dt = _NP_DTYPE.get(et)
            if dt is None:
                raise GgufError(f"unknown array element type {et}")
            raw = self.take(n * np.dtype(dt).itemsize)
            return np.frombuffer(raw, dtype=dt).copy()
        return self.scalar(t)


class _Shard:
    def __init__(self, path: str, header_only: bool):
        self.path = path
        self.file = open(path, "rb")
        size = os.fstat(self.file.fileno()).st_size
        if size < 24:
            raise GgufError(f"{path}: {size} bytes is too short for a GGUF header")
        self.map = mmap.mmap(self.file.fileno(), 0, access=mmap.ACCESS_READ)
        cur = _Cursor(self.map)
        magic = cur.scalar(_T_U32)
        if magic != GGUF_MAGIC:
            raise GgufError(f"{path}: magic {magic:#x} is not GGUF")
        self.version = cur.scalar(_T_U32)
        if self.version not in (2, 3):
            raise GgufError(f"{path}: GGUF version {self.version} is not supported")
        n_tensors = cur.scalar(_T_U64)
        n_kv = cur.scalar(_T_U64)
        self.meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = cur.string()
            t = cur.scalar(_T_U32)
            self.meta[key] = cur.value(t)
        self.tensors: List[TensorInfo] = []
        for _ in range(n_tensors):
            name = cur.string()
            nd = cur.scalar(_T_U32)
            if nd > 8:
                raise GgufError(f"{path}: tensor {name} has {nd} dims")
            ne = tuple(cur.scalar(_T_U64) for _ in range(nd))
            tid = cur.scalar(_T_U32)
            qt = QTYPE_BY_ID.get(tid)
            if qt is None:
                raise GgufError(f"{path}: tensor {name} has unknown ggml type {tid}")
            off = cur.scalar(_T_U64)
            self.tensors.append(TensorInfo(name, ne, qt, off))
        self.alignment = int(self.meta.get("general.alignment", DEFAULT_ALIGNMENT))
        self.data_start = (cur.pos + self.alignment - 1) // self.alignment * self.alignment
        if not header_only:
            for t in self.tensors:
                if t.ne and t.ne[0] % t.qtype.block_values:
                    raise GgufError(f"{path}: {t.name} row length {t.ne[0]} not a multiple of {t.qtype.block_values}")
                if t.offset % self.alignment:
                    raise GgufError(f"{path}: {t.name} offset {t.offset} is not {self.alignment}-aligned")
                if self.data_start + t.offset + t.n_bytes > size:
                    raise GgufError(f"{path}: {t.name} runs past the end of the file")

    def close(self):
        try:
            self.map.close()
        except BufferError:
            pass  # views still alive; the OS unmaps at exit
        self.file.close()


_SPLIT_RE = re.compile(r"^(.*)-(\d{5})-of-(\d{5})\.gguf$")


def split_paths(path: str) -> List[str]:
    """All shard paths of a split file given any one of them (``Split`` in the reference)."""
    m = _SPLIT_RE.match(path)
    if not m:
        return [path]
    stem, _, total = m.group(1), int(m.group(2)), int(m.group(3))
    return [f"{stem}-{i:05d}-of-{total:05d}.gguf" for i in range(1, total + 1)]


class Gguf:
    """An opened GGUF model (one file or every shard of a split)."""

    def __init__(self, path: str, header_only: bool = False):
        self.paths = split_paths(path)
        self.shards = [_Shard(p, header_only) for p in self.paths]
        self.meta: Dict[str, Any] = dict(self.shards[0].meta)
        self.tensors: Dict[str, TensorInfo] = {}
        for i, sh in enumerate(self.shards):
            for t in sh.tensors:
                if t.name in self.tensors:
                    raise GgufError(f"tensor {t.name} appears in two shards")
                t.shard = i
                self.tensors[t.name] = t
        n_split = int(self.meta.get("split.count", len(self.shards)) or len(self.shards))
        if n_split != len(self.shards) and len(self.shards) > 1:
            raise GgufError(f"split.count {n_split} but {len(self.shards)} shard files")

    @classmethod
    def open(cls, path: str) -> "Gguf":
        return cls(path, header_only=False)

    @classmethod
    def inventory(cls, path: str) -> "Gguf":
        """Header-only open: names, dims, types; no bounds checks of the data section."""
        return cls(path, header_only=True)

    def close(self):
        for s in self.shards:
            s.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # metadata helpers -----------------------------------------------------------------
    @property
    def arch(self) -> str:
        return str(self.meta.get("general.architecture", ""))

    def get(self, key: str, default=None):
        return self.meta.get(key, default)

    def arch_get(self, key: str, default=None):
        return self.meta.get(f"{self.arch}.{key}", default)

    # data -----------------------------------------------------------------------------
    def tensor_bytes(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        sh = self.shards[t.shard]
        start = sh.data_start + t.offset
        return np.frombuffer(sh.map, dtype=np.uint8, count=t.n_bytes, offset=start)

    def tensor_rows(self, name: str) -> torch.Tensor:
        """uint8 [n_rows, row_bytes] view (zero copy; read-only memory)."""
        t = self.tensors[name]
        arr = self.tensor_bytes(name).reshape(-1, t.row_bytes)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            return torch.from_numpy(arr)

    def tensor_f32(self, name: str) -> torch.Tensor:
        from .quant import dequantize
        t = self.tensors[name]
        rows = self.tensor_rows(name).clone()
        return dequantize(rows, t.qtype.name, t.ne[0]).reshape(t.shape)

    def sha256(self, name: str) -> str:
        return hashlib.sha256(self.tensor_bytes(name).tobytes()).hexdigest()


# --------------------------------------------------------------------------------------
# writer
# --------------------------------------------------------------------------------------

def _w_str(f: BinaryIO, s: str):
    b = s.encode("utf-8")
    f.write(struct.pack("<Q", len(b)))
    f.write(b)


def _w_value(f: BinaryIO, v):
    if isinstance(v, bool):
        f.write(struct.pack("<I", _T_BOOL)); f.write(struct.pack("<?", v))
    elif isinstance(v, int):
        if 0 <= v < 1 << 32:
            f.write(struct.pack("<I", _T_U32)); f.write(struct.pack("<I", v))
        elif v < 0 and v >= -(1 << 31):
            f.write(struct.pack("<I", _T_I32)); f.write(struct.pack("<i", v))
        else:
            f.write(struct.pack("<I", _T_U64 if v >= 0 else _T_I64)); f.write(struct.pack("<Q" if v >= 0 else "<q", v))
    elif isinstance(v, float):
        f.write(struct.pack("<I", _T_F32)); f.write(struct.pack("<f", v))
    elif isinstance(v, str):
        f.write(struct.pack("<I", _T_STR)); _w_str(f, v)
    elif isinstance(v, np.ndarray):
        et = {np.dtype(k): t for t, k in _NP_DTYPE.items()}[v.dtype]
        f.write(struct.pack("<I", _T_ARR)); f.write(struct.pack("<I", et)); f.write(struct.pack("<Q", v.size))
        f.write(v.tobytes())
    elif isinstance(v, (list, tuple)):
        f.write(struct.pack("<I", _T_ARR))
        if len(v) and isinstance(v[0], str):
            f.write(struct.pack("<I", _T_STR)); f.write(struct.pack("<Q", len(v)))
            for s in v:
                _w_str(f, s)
        elif len(v) and isinstance(v[0], float):
            f.write(struct.pack("<I", _T_F32)); f.write(struct.pack("<Q", len(v)))
            f.write(np.asarray(v, np.float32).tobytes())
        else:
            f.write(struct.pack("<I", _T_I32)); f.write(struct.pack("<Q", len(v)))
            f.write(np.asarray(v, np.int32).tobytes())
    else:
        raise GgufError(f"cannot write metadata value of type {type(v).__name__}")


class GgufWriter:
    """Collects metadata and tensors, then writes one GGUF v3 file."""

    def __init__(self, arch: str, alignment: int = DEFAULT_ALIGNMENT):
        self.meta: Dict[str, Any] = {"general.architecture": arch, "general.alignment": alignment}
        self.alignment = alignment
        self._tensors: List[Tuple[str, Tuple[int, ...], QType, np.ndarray]] = []

    def set(self, key: str, value):
        self.meta[key] = value

    def add(self, name: str, shape: Sequence[int], qtype: str, data) -> None:
        """``shape`` is row-major (slowest first); ``data`` is the raw block bytes."""
        qt = QTYPES[qtype]
        if isinstance(data, torch.Tensor):
            data = data.detach().cpu().contiguous().view(torch.uint8).numpy()
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        n_rows = 1
        for d in shape[:-1]:
            n_rows *= d
        want = n_rows * qt.row_bytes(shape[-1])
        if data.size != want:
            raise GgufError(f"{name}: {data.size} bytes given, {want} expected for {qtype} {tuple(shape)}")
        self._tensors.append((name, tuple(reversed(tuple(shape))), qt, data))

    def add_f32(self, name: str, t: torch.Tensor):
        self.add(name, tuple(t.shape), "F32", t.detach().float().cpu().contiguous().numpy().view(np.uint8))

    def add_quantized(self, name: str, w: torch.Tensor, qtype: str):
        from .quant import quantize
        w2 = w.reshape(-1, w.shape[-1])
        self.add(name, tuple(w.shape), qtype, quantize(w2, qtype))

    def write(self, path: str) -> None:
        a = self.alignment
        with open(path, "wb") as f:
            f.write(struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(self._tensors), len(self.meta)))
            for k, v in self.meta.items():
                _w_str(f, k)
                _w_value(f, v)
            off = 0
            for name, ne, qt, data in self._tensors:
                _w_str(f, name)
                f.write(struct.pack("<I", len(ne)))
                for d in ne:
                    f.write(struct.pack("<Q", d))
                f.write(struct.pack("<I", qt.ggml_id))
                f.write(struct.pack("<Q", off))
                off += (data.size + a - 1) // a * a
            pad = (-f.tell()) % a
            f.write(b"\0" * pad)
            for _, _, _, data in self._tensors:
                f.write(data.tobytes())
                f.write(b"\0" * ((-data.size) % a))
