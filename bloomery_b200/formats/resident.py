"""Resident (in-HBM) layouts of quantised weights.

Values are never re-quantised on load; some block types are only re-laid so that every
16-byte vector load of the kernels is aligned (the reference does the same in
``crates/gpu/src/weights.rs`` / ``planes.rs``: "resident formats per type").

  Q4_K, Q5_K          file blocks unchanged (144 / 176 bytes, both multiples of 16)
  Q6_K                210-byte file blocks padded to 224: ql[128] qh[64] sc[16] d pad[14]
  Q2_K                84-byte file blocks re-laid to 96: qs[64] scales[16] d dmin pad[12]
  Q3_K                110-byte file blocks re-laid to 128: qs[64] hmask[32] sc[16] d pad[14]; the sixteen 6-bit
                      scales are unpacked to signed bytes with the 32 already subtracted (same values)
  Q8_0                per row: K int8 codes, then K/32 f16 scales, padded to 16 bytes
  Q4_0 Q4_1 Q5_0 Q5_1 per row: nibble codes K/2, fifth bits K/8 (5-bit types), f16 d per block, f16 m per block
                      (_1 types), padded to 16 bytes; nibble order inside a block as in the file
  F32 / F16 / BF16    unchanged
  NVFP4, FP8_B128     rows built from checkpoint planes by ``formats/planes.py``
  IQ4_NL, IQ4_XS,     decoded at load to Q8_F32 rows: K int8 codes, then K/32 f32 scales, padded to 16.  Every code of
  MXFP4, IQ2_XXS      these types is a small integer of a code book and every 32 values share one scale, so the rows
                      hold the same values (9 bits per weight on the card whatever the file's rate)

Works on CPU and CUDA tensors (the repack of a 30 B-parameter model runs on the card).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .quant import QTYPES

# weight-type ids shared with csrc/quant_units.cuh (equal to the ggml ids)
WT = {"F32": 0, "F16": 1, "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14, "BF16": 30, "NVFP4": 40, "FP8_B128": 41, "Q8_F32": 50}
INT_DOT_TYPES = ("Q4_K", "Q5_K", "Q6_K", "Q8_0", "Q2_K", "Q3_K", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "NVFP4", "FP8_B128", "Q8_F32")      # dotted against q8 activations
PLANE_TYPES = ("NVFP4", "FP8_B128")
FLOAT_TYPES = ("F32", "F16", "BF16")


# file types that are decoded to another resident type at load (value-preserving)
LOAD_AS = {"IQ4_NL": "Q8_F32", "IQ4_XS": "Q8_F32", "MXFP4": "Q8_F32", "IQ2_XXS": "Q8_F32"}


class UnsupportedType(ValueError):
    pass


def resident_type(file_qtype: str) -> str:
    """The type of the rows that :func:`to_resident` makes of a file type."""
    return LOAD_AS.get(file_qtype, file_qtype)


_Q32 = {"Q4_0": (4, False), "Q4_1": (4, True), "Q5_0": (5, False), "Q5_1": (5, True)}     # bits, has a min


def _q32_fields(qtype: str):
    """Byte ranges of d, m, qh, qs inside one file block."""
    bits, has_min = _Q32[qtype]
    o = 2
    m = (o, o + 2) if has_min else None
    o += 2 if has_min else 0
    qh = (o, o + 4) if bits == 5 else None
    o += 4 if bits == 5 else 0
    return (0, 2), m, qh, (o, o + 16), o + 16


def resident_row_bytes(qtype: str, k: int) -> int:
    if qtype == "Q4_K":
        return k // 256 * 144
    if qtype == "Q5_K":
        return k // 256 * 176
    if qtype == "Q6_K":
        return k // 256 * 224
    if qtype == "Q8_0":
        return (k + k // 16 + 15) // 16 * 16
    if qtype == "Q8_F32":
        return (k + k // 8 + 15) // 16 * 16
    if qtype == "Q2_K":
        return k // 256 * 96
    if qtype == "Q3_K":
        return k // 256 * 128
    if qtype in _Q32:
        bits, has_min = _Q32[qtype]
        return (k // 2 + (k // 8 if bits == 5 else 0) + k // 16 * (2 if has_min else 1) + 15) // 16 * 16
    if qtype == "F32":
        return 4 * k
    if qtype in ("F16", "BF16"):
        return 2 * k
    if qtype == "NVFP4":
        return (k // 2 + k // 16 + 4 + 15) // 16 * 16
    if qtype == "FP8_B128":
        return (k + k // 32 + 15) // 16 * 16
    raise UnsupportedType(f"no resident layout for block type {qtype}")


def quantize_resident(w: torch.Tensor, qtype: str, values: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """f32 [rows, K] -> (resident rows, the f32 values those rows decode to, or None when ``values`` is off).
    Fixtures and tests."""
    from . import planes, quant
    k = w.shape[-1]
    chunk = 1 << 15                     # rows per pass: the block-scaled quantisers make several full-size temporaries
    if qtype in PLANE_TYPES and w.shape[0] > chunk:
        parts = [quantize_resident(w[i:i + chunk], qtype, values) for i in range(0, w.shape[0], chunk)]
        return torch.cat([p[0] for p in parts], 0), (torch.cat([p[1] for p in parts], 0) if values else None)
    if qtype == "NVFP4":
        res = planes.nvfp4_resident(*planes.nvfp4_quantize(w))
        return res, (planes.resident_dequantize(res, qtype, k) if values else None)
    if qtype == "FP8_B128":
        res = planes.fp8_b128_resident(*planes.fp8_b128_quantize(w))
        return res, (planes.resident_dequantize(res, qtype, k) if values else None)
    raw = quant.quantize(w, qtype)
    return to_resident(raw, qtype, k), (quant.dequantize(raw, qtype, k) if values else None)


def to_resident(raw: torch.Tensor, qtype: str, k: int) -> torch.Tensor:
    """uint8 [rows, file_row_bytes] -> uint8 [rows, resident_row_bytes] (same device)."""
    if raw.dtype != torch.uint8 or raw.dim() != 2:
        raise ValueError("to_resident takes uint8 [rows, row_bytes]")
    rows = raw.shape[0]
    if raw.shape[1] != QTYPES[qtype].row_bytes(k):
        raise ValueError(f"{qtype}: row of {raw.shape[1]} bytes does not match k={k}")
    if qtype in ("Q4_K", "Q5_K", "F32", "F16", "BF16"):
        return raw.contiguous()
    if qtype in LOAD_AS:
        from .quant import code_scale_form
        codes, scales = code_scale_form(raw, qtype, k)
        out = torch.zeros(rows, resident_row_bytes("Q8_F32", k), dtype=torch.uint8, device=raw.device)
        out[:, :k] = codes.view(torch.uint8)
        out[:, k:k + k // 8] = scales.contiguous().view(torch.uint8).reshape(rows, k // 8)
        return out
    if qtype == "Q6_K":
        nsb = k // 256
        out = torch.zeros(rows, nsb, 224, dtype=torch.uint8, device=raw.device)
        out[..., :210] = raw.reshape(rows, nsb, 210)
        return out.reshape(rows, nsb * 224)
    if qtype == "Q2_K":
        nsb = k // 256
        blk = raw.reshape(rows, nsb, 84)
        out = torch.zeros(rows, nsb, 96, dtype=torch.uint8, device=raw.device)
        out[..., 0:64], out[..., 64:80], out[..., 80:84] = blk[..., 16:80], blk[..., 0:16], blk[..., 80:84]
        return out.reshape(rows, nsb * 96)
    if qtype == "Q3_K":
        nsb = k // 256
        blk = raw.reshape(rows, nsb, 110)
        sb = blk[..., 96:108].to(torch.int32)
        lo4 = torch.cat([sb[..., 0:8] & 0xF, sb[..., 0:8] >> 4], -1)
        hi2 = torch.cat([(sb[..., 8:12] >> s) & 3 for s in (0, 2, 4, 6)], -1)
        sc = ((lo4 | (hi2 << 4)) - 32).to(torch.int8).view(torch.uint8)
        out = torch.zeros(rows, nsb, 128, dtype=torch.uint8, device=raw.device)
        out[..., 0:64], out[..., 64:96], out[..., 96:112], out[..., 112:114] = blk[..., 32:96], blk[..., 0:32], sc, blk[..., 108:110]
        return out.reshape(rows, nsb * 128)
    if qtype in _Q32:
        d, m, qh, qs, bb = _q32_fields(qtype)
        nb = k // 32
        blk = raw.reshape(rows, nb, bb)
        out = torch.zeros(rows, resident_row_bytes(qtype, k), dtype=torch.uint8, device=raw.device)
        o = k // 2
        out[:, :o] = blk[..., qs[0]:qs[1]].reshape(rows, o)
        if qh:
            out[:, o:o + k // 8] = blk[..., qh[0]:qh[1]].reshape(rows, k // 8)
            o += k // 8
        out[:, o:o + 2 * nb] = blk[..., d[0]:d[1]].reshape(rows, 2 * nb)
        o += 2 * nb
        if m:
            out[:, o:o + 2 * nb] = blk[..., m[0]:m[1]].reshape(rows, 2 * nb)
        return out
    if qtype == "Q8_0":
        nb = k // 32
        blk = raw.reshape(rows, nb, 34)
        out = torch.zeros(rows, resident_row_bytes("Q8_0", k), dtype=torch.uint8, device=raw.device)
        out[:, :k] = blk[..., 2:].reshape(rows, k)
        out[:, k:k + 2 * nb] = blk[..., :2].reshape(rows, 2 * nb)
        return out
    raise UnsupportedType(f"no resident layout for block type {qtype}")


def decode_q8_f32(res: torch.Tensor, k: int) -> torch.Tensor:
    """f32 values of Q8_F32 rows (code * scale, exact)."""
    rows = res.shape[0]
    codes = res[:, :k].contiguous().view(torch.int8).float().reshape(rows, k // 32, 32)
    scales = res[:, k:k + k // 8].contiguous().view(torch.float32).reshape(rows, k // 32)
    return (codes * scales[..., None]).reshape(rows, k)


def from_resident(res: torch.Tensor, qtype: str, k: int) -> torch.Tensor:
    """Inverse of :func:`to_resident` (used by tests and by slot files)."""
    rows = res.shape[0]
    if qtype in ("Q4_K", "Q5_K", "F32", "F16", "BF16"):
        return res
    if qtype == "Q6_K":
        nsb = k // 256
        return res.reshape(rows, nsb, 224)[..., :210].reshape(rows, nsb * 210).contiguous()
    if qtype == "Q2_K":
        nsb = k // 256
        r = res.reshape(rows, nsb, 96)
        out = torch.empty(rows, nsb, 84, dtype=torch.uint8, device=res.device)
        out[..., 16:80], out[..., 0:16], out[..., 80:84] = r[..., 0:64], r[..., 64:80], r[..., 80:84]
        return out.reshape(rows, nsb * 84)
    if qtype == "Q3_K":
        nsb = k // 256
        r = res.reshape(rows, nsb, 128)
        sc = r[..., 96:112].view(torch.int8).to(torch.int32) + 32          # back to the 6-bit codes
        lo, hi = sc & 0xF, sc >> 4
        packed = torch.zeros(rows, nsb, 12, dtype=torch.int32, device=res.device)
        packed[..., 0:8] = lo[..., 0:8] | (lo[..., 8:16] << 4)
        for j in range(4):
            packed[..., 8:12] |= hi[..., 4 * j:4 * j + 4] << (2 * j)
        out = torch.empty(rows, nsb, 110, dtype=torch.uint8, device=res.device)
        out[..., 32:96], out[..., 0:32], out[..., 96:108], out[..., 108:110] = r[..., 0:64], r[..., 64:96], packed.to(torch.uint8), r[..., 112:114]
        return out.reshape(rows, nsb * 110)
    if qtype in _Q32:
        d, m, qh, qs, bb = _q32_fields(qtype)
        nb = k // 32
        out = torch.empty(rows, nb, bb, dtype=torch.uint8, device=res.device)
        o = k // 2
        out[..., qs[0]:qs[1]] = res[:, :o].reshape(rows, nb, 16)
        if qh:
            out[..., qh[0]:qh[1]] = res[:, o:o + k // 8].reshape(rows, nb, 4)
            o += k // 8
        out[..., d[0]:d[1]] = res[:, o:o + 2 * nb].reshape(rows, nb, 2)
        o += 2 * nb
        if m:
            out[..., m[0]:m[1]] = res[:, o:o + 2 * nb].reshape(rows, nb, 2)
        return out.reshape(rows, nb * bb)
    if qtype == "Q8_0":
        nb = k // 32
        out = torch.empty(rows, nb, 34, dtype=torch.uint8, device=res.device)
        out[..., 2:] = res[:, :k].reshape(rows, nb, 32)
        out[..., :2] = res[:, k:k + 2 * nb].reshape(rows, nb, 2)
        return out.reshape(rows, nb * 34)
    raise UnsupportedType(qtype)
