"""NVFP4 block scales that a ModelOpt checkpoint stores compressed, read back as the plain ``weight_scale`` bytes
(one E4M3 byte per 16 values, ``rows x cols`` row-major).

A row's scale bytes cluster in a narrow window, so both encodings store a base byte per row and a 4-bit code per scale
(``byte = base + code``, two codes a byte, low nibble first) and list apart, as whole bytes, the few scales the 16-wide
window misses.  ``quantized_layers[...].weight_scale_encoding`` names the encoding:

``csf``
    ``<scale>.nvfp4_csf_fixed`` U8 ``[rows / 16, 16 * (1 + cols / 2)]``: per slab of 16 rows its 16 base bytes, then the
    slab's codes row by row.  ``<scale>.nvfp4_csf_exceptions`` U32, strictly increasing: the low 24 bits are the flat
    position ``r * cols + c``, the high 8 the byte there.

``csf_32x2_v1``
    blocks of 32 rows x 2 columns (the last block of an odd ``cols`` is one column wide), grouped in tiles of 4 block
    rows x 2 block columns taken row-major, 32 tiles a page.  ``.csf32_bases`` U8 ``[rows]``; ``.csf32_codes`` U8
    ``[rows * cols / 2]``: the blocks in stream order (inside a tile the first block column's block rows, then the
    second's), a block's codes row-major; ``.csf32_exceptions`` U16 records, a block's in increasing place
    (low byte ``2 * row + col`` inside the block, high byte the byte there); ``.csf32_offsets`` U16
    ``[blocks + pages]``: per page the running count of its blocks' records, starting at 0, with one closing entry;
    ``.csf32_page_bases`` U32: twice the number of records before each page.

Everything a rule does not allow is refused with the part's name: a base above 240, a part of the wrong size, a page
base or first prefix that does not match, prefixes that fall or run past the records, a record outside its block or out
of order, an exception out of range or out of order, records or codes left over.  The encoders below write the
same layouts (fixtures, and a way to shrink a plain checkpoint).

Counterpart of the reference's ``crates/hf/src/csf.rs`` (the layouts are those of the published decoders it cites,
FlashInfer's ``_csf_blocks.py`` and vLLM's ``csf_scales.py``).
"""
from __future__ import annotations

from typing import Dict, Tuple

import numpy as np

MAX_BASE = 240                     # base + 15 must stay a byte
BLOCK_ROWS, TILE_BLOCK_ROWS, TILE_BLOCK_COLS, PAGE_TILES = 32, 4, 2, 32


class CsfError(ValueError):
    def __init__(self, name: str, what: str):
        super().__init__(f"{name}: {what}")
        self.name, self.what = name, what


def _nibbles(codes: np.ndarray) -> np.ndarray:
    """u8 [n] -> u8 [2n], low nibble first."""
    out = np.empty(codes.size * 2, dtype=np.uint8)
    out[0::2] = codes & 15
    out[1::2] = codes >> 4
    return out


def _pack(nib: np.ndarray) -> np.ndarray:
    return (nib[0::2] | (nib[1::2] << 4)).astype(np.uint8)


# ---------------------------------------------------------------------------------------------------------- csf
def decode_csf(name: str, fixed: np.ndarray, exceptions: np.ndarray, rows: int, cols: int) -> np.ndarray:
    fixed = np.ascontiguousarray(fixed, dtype=np.uint8).reshape(-1)
    exceptions = np.ascontiguousarray(exceptions).astype(np.uint32).reshape(-1)
    if rows <= 0 or rows % 16 or cols <= 0 or cols % 2:
        raise CsfError(name, f"{rows} by {cols} scales: csf needs rows a multiple of 16 and even columns")
    slab = 16 * (1 + cols // 2)
    if fixed.size != rows // 16 * slab:
        raise CsfError(name, f"{fixed.size} bytes; {rows} by {cols} scales are {rows // 16} slabs of {slab}")
    slabs = fixed.reshape(rows // 16, slab)
    bases = slabs[:, :16].reshape(rows)
    if int(bases.max()) > MAX_BASE:
        r = int(np.argmax(bases > MAX_BASE))
        raise CsfError(name, f"row {r} base {int(bases[r])} is above {MAX_BASE}")
    out = (bases[:, None] + _nibbles(slabs[:, 16:].reshape(-1)).reshape(rows, cols)).astype(np.uint8)
    if exceptions.size:
        at = (exceptions & 0xFFFFFF).astype(np.int64)
        bad = np.flatnonzero((at >= rows * cols) | (np.diff(at, prepend=-1) <= 0))
        if bad.size:
            i = int(bad[0])
            raise CsfError(name, f"exception {i} at position {int(at[i])}: positions are increasing and below {rows * cols}")
        out.reshape(-1)[at] = (exceptions >> 24).astype(np.uint8)
    return out


def _row_bases(scale: np.ndarray) -> np.ndarray:
    """The base of every row: the 16-wide window that holds the most of the row's bytes (lowest such on a tie)."""
    rows = scale.shape[0]
    bases = np.zeros(rows, dtype=np.uint8)
    for r in range(rows):
        hist = np.bincount(scale[r], minlength=256)
        win = np.convolve(hist, np.ones(16, dtype=np.int64))[15:15 + MAX_BASE + 1]      # win[b] = bytes in [b, b + 15]
        bases[r] = int(np.argmax(win))
    return bases


def encode_csf(scale: np.ndarray) -> Dict[str, np.ndarray]:
    """Plain scale bytes [rows, cols] -> {"nvfp4_csf_fixed", "nvfp4_csf_exceptions"}."""
    scale = np.ascontiguousarray(scale, dtype=np.uint8)
    rows, cols = scale.shape
    if rows % 16 or cols % 2:
        raise CsfError("encode", f"{rows} by {cols} scales: csf needs rows a multiple of 16 and even columns")
    bases = _row_bases(scale)
    delta = scale.astype(np.int32) - bases[:, None]
    miss = (delta < 0) | (delta > 15)
    codes = np.where(miss, 0, delta).astype(np.uint8)
    fixed = np.concatenate([bases.reshape(rows // 16, 16), _pack(codes.reshape(-1)).reshape(rows // 16, 16 * cols // 2)], axis=1)
    at = np.flatnonzero(miss.reshape(-1)).astype(np.uint32)
    words = at | (scale.reshape(-1)[at].astype(np.uint32) << 24)
    return {"nvfp4_csf_fixed": fixed, "nvfp4_csf_exceptions": words.astype(np.uint32)}


# ---------------------------------------------------------------------------------------------------- csf_32x2_v1
def _stream(rows: int, cols: int):
    """The blocks in stream order: (tile, first row, first column, width)."""
    block_rows, block_cols = rows // BLOCK_ROWS, (cols + 1) // 2
    tile_cols = (block_cols + TILE_BLOCK_COLS - 1) // TILE_BLOCK_COLS
    tile_rows = (block_rows + TILE_BLOCK_ROWS - 1) // TILE_BLOCK_ROWS
    for tile in range(tile_rows * tile_cols):
        r, c = tile // tile_cols * TILE_BLOCK_ROWS, tile % tile_cols * TILE_BLOCK_COLS
        for bc in range(c, min(block_cols, c + TILE_BLOCK_COLS)):
            for br in range(r, min(block_rows, r + TILE_BLOCK_ROWS)):
                yield tile, br * BLOCK_ROWS, 2 * bc, min(2, cols - 2 * bc)


def decode_csf32(name: str, bases: np.ndarray, codes: np.ndarray, page_bases: np.ndarray, offsets: np.ndarray,
                 exceptions: np.ndarray, rows: int, cols: int) -> np.ndarray:
    bases = np.ascontiguousarray(bases, dtype=np.uint8).reshape(-1)
    codes = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
    page_bases = np.ascontiguousarray(page_bases).astype(np.uint32).reshape(-1).astype(np.int64)
    offsets = np.ascontiguousarray(offsets).astype(np.uint16).reshape(-1).astype(np.int64)
    exceptions = np.ascontiguousarray(exceptions).astype(np.uint16).reshape(-1).astype(np.int64)
    if rows <= 0 or rows % BLOCK_ROWS or cols <= 0:
        raise CsfError(name, f"{rows} by {cols} scales: csf32 needs rows a multiple of 32")
    size = rows * cols
    block_rows, block_cols = rows // BLOCK_ROWS, (cols + 1) // 2
    tile_cols = (block_cols + TILE_BLOCK_COLS - 1) // TILE_BLOCK_COLS
    tiles = (block_rows + TILE_BLOCK_ROWS - 1) // TILE_BLOCK_ROWS * tile_cols
    pages = (tiles + PAGE_TILES - 1) // PAGE_TILES
    blocks = block_rows * block_cols
    for part, have, want in (("bases", bases.size, rows), ("codes", codes.size, size // 2), ("page bases", page_bases.size, pages),
                             ("offsets", offsets.size, blocks + pages)):
        if have != want:
            raise CsfError(name, f"{part} hold {have} entries; {rows} by {cols} scales need {want}")
    if size % 2:
        raise CsfError(name, f"{rows} by {cols} scales: an odd number of codes")
    if int(bases.max()) > MAX_BASE:
        r = int(np.argmax(bases > MAX_BASE))
        raise CsfError(name, f"row {r} base {int(bases[r])} is above {MAX_BASE}")
    nib = _nibbles(codes)
    out = np.zeros((rows, cols), dtype=np.uint8)
    field = entry = origin = page_end = 0
    last_tile = -1
    for block, (tile, r0, c0, w) in enumerate(_stream(rows, cols)):
        if tile != last_tile and tile % PAGE_TILES == 0:
            if tile > 0:
                entry += 1                       # the closing entry of the page before
                origin += page_end
            page = tile // PAGE_TILES
            if int(page_bases[page]) != 2 * origin or int(offsets[entry]) != 0:
                raise CsfError(name, f"page {page}: base {int(page_bases[page])} and first prefix {int(offsets[entry])}; "
                                     f"the records before it make {2 * origin} and 0")
        last_tile = tile
        out[r0:r0 + BLOCK_ROWS, c0:c0 + w] = bases[r0:r0 + BLOCK_ROWS, None] + nib[field:field + BLOCK_ROWS * w].reshape(BLOCK_ROWS, w)
        field += BLOCK_ROWS * w
        lo, hi = int(offsets[entry]), int(offsets[entry + 1])
        if hi < lo or origin + hi > exceptions.size:
            raise CsfError(name, f"block {block}: prefixes {lo} to {hi} from record {origin} of {exceptions.size}")
        prev = -1
        for rec in exceptions[origin + lo:origin + hi]:
            at = int(rec) & 0xFF
            if at // 2 >= BLOCK_ROWS or at % 2 >= w or at <= prev:
                raise CsfError(name, f"block {block}: record at {at} is outside its {BLOCK_ROWS} by {w} block or out of order")
            prev = at
            out[r0 + at // 2, c0 + at % 2] = int(rec) >> 8
        page_end = hi
        entry += 1
    if origin + page_end != exceptions.size or field != size:
        raise CsfError(name, f"{origin + page_end} of {exceptions.size} records and {field} of {size} codes read")
    return out


def encode_csf32(scale: np.ndarray) -> Dict[str, np.ndarray]:
    """Plain scale bytes [rows, cols] -> the five ``csf32_*`` parts."""
    scale = np.ascontiguousarray(scale, dtype=np.uint8)
    rows, cols = scale.shape
    if rows % BLOCK_ROWS or (rows * cols) % 2:
        raise CsfError("encode", f"{rows} by {cols} scales: csf32 needs rows a multiple of 32 and an even byte count")
    bases = _row_bases(scale)
    nib, recs, offsets, page_bases = [], [], [], []
    in_page = before = 0
    last_tile = -1
    for tile, r0, c0, w in _stream(rows, cols):
        if tile != last_tile and tile % PAGE_TILES == 0:
            if tile > 0:
                offsets.append(in_page)          # the closing entry
                before += in_page
            page_bases.append(2 * before)
            in_page = 0
        last_tile = tile
        offsets.append(in_page)
        blk = scale[r0:r0 + BLOCK_ROWS, c0:c0 + w].astype(np.int32)
        delta = blk - bases[r0:r0 + BLOCK_ROWS, None]
        miss = (delta < 0) | (delta > 15)
        nib.append(np.where(miss, 0, delta).astype(np.uint8).reshape(-1))
        for i, j in zip(*np.nonzero(miss)):
            recs.append((2 * int(i) + int(j)) | (int(blk[i, j]) << 8))
            in_page += 1
    offsets.append(in_page)
    if max(offsets, default=0) > 0xFFFF:
        raise CsfError("encode", "a page holds more records than a 16-bit prefix counts")
    return {"csf32_bases": bases, "csf32_codes": _pack(np.concatenate(nib)), "csf32_page_bases": np.asarray(page_bases, dtype=np.uint32),
            "csf32_offsets": np.asarray(offsets, dtype=np.uint16), "csf32_exceptions": np.asarray(recs, dtype=np.uint16)}


# ------------------------------------------------------------------------------------------------------- folders
SUFFIXES = {"csf": ("nvfp4_csf_fixed", "nvfp4_csf_exceptions"),
            "csf_32x2_v1": ("csf32_bases", "csf32_codes", "csf32_page_bases", "csf32_offsets", "csf32_exceptions")}


def encoding_of(folder, scale: str):
    """The encoding whose parts ``folder`` holds for the scale tensor ``scale``, or None when it is stored plain."""
    for enc, parts in SUFFIXES.items():
        if f"{scale}.{parts[0]}" in folder:
            return enc
    return None


def weight_scale(folder, scale: str, encoding: str, rows: int, cols: int) -> np.ndarray:
    """The logical scale bytes [rows, cols] of ``scale`` (``<stem>.weight_scale``) from its compressed parts."""
    if encoding not in SUFFIXES:
        raise CsfError(scale, f"scale encoding {encoding!r} is not read (csf, csf_32x2_v1)")
    want = {"nvfp4_csf_exceptions": 4, "csf32_page_bases": 4, "csf32_offsets": 2, "csf32_exceptions": 2}
    parts = []
    for suffix in SUFFIXES[encoding]:
        name = f"{scale}.{suffix}"
        if name not in folder:
            raise CsfError(name, "the checkpoint has no such tensor")
        t = folder.tensor(name)
        width = want.get(suffix, 1)
        if t.element_size() != width:
            raise CsfError(name, f"elements of {t.element_size()} bytes where the encoding stores {width}")
        parts.append(t.contiguous().reshape(-1).numpy())
    name = f"{scale}.{SUFFIXES[encoding][0]}"
    if encoding == "csf":
        return decode_csf(name, parts[0], parts[1].view(np.uint32), rows, cols)
    return decode_csf32(name, parts[0], parts[1], parts[2].view(np.uint32), parts[3].view(np.uint16), parts[4].view(np.uint16), rows, cols)
