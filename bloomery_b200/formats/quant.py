"""Block quantization formats (GGUF K-quants and legacy quants) as vectorised torch code.

Every routine here runs on CPU or CUDA tensors alike, so the same code is the
byte-exact *oracle* for the CUDA kernels in ``csrc/`` and the fast on-device
fixture quantizer used by ``bench.py`` (30 B values quantised on the GPU in
seconds).  Block layouts follow the ggml on-disk format that the reference
reads in ``crates/gguf/src/quant.rs`` (scalar dequant for every type) and
``crates/gguf/src/qtype.rs`` (``QROWS`` type-facts table).

Layouts (bytes per block / values per block):
  Q4_0 18/32, Q4_1 20/32, Q5_0 22/32, Q5_1 24/32, Q8_0 34/32,
  Q2_K 84/256, Q3_K 110/256, Q4_K 144/256, Q5_K 176/256, Q6_K 210/256,
  F16, BF16, F32.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict

import torch

QK_K = 256


@dataclasses.dataclass(frozen=True)
class QType:
    """One row of the type-facts table (``crates/gguf/src/qtype.rs`` ``QROWS``)."""

    name: str
    ggml_id: int
    block_values: int
    block_bytes: int

    def row_bytes(self, k: int) -> int:
        if k % self.block_values:
            raise ValueError(f"{self.name}: row length {k} is not a multiple of {self.block_values}")
        return k // self.block_values * self.block_bytes


# ggml type ids are part of the GGUF file format.
QTYPES: Dict[str, QType] = {
    q.name: q
    for q in [
        QType("F32", 0, 1, 4),
        QType("F16", 1, 1, 2),
        QType("Q4_0", 2, 32, 18),
        QType("Q4_1", 3, 32, 20),
        QType("Q5_0", 6, 32, 22),
        QType("Q5_1", 7, 32, 24),
        QType("Q8_0", 8, 32, 34),
        QType("Q2_K", 10, 256, 84),
        QType("Q3_K", 11, 256, 110),
        QType("Q4_K", 12, 256, 144),
        QType("Q5_K", 13, 256, 176),
        QType("Q6_K", 14, 256, 210),
        QType("IQ2_XXS", 16, 256, 66),
        QType("IQ4_NL", 20, 32, 18),
        QType("IQ4_XS", 23, 256, 136),
        QType("I8", 24, 1, 1),
        QType("I32", 26, 1, 4),
        QType("BF16", 30, 1, 2),
        QType("MXFP4", 39, 32, 17),
        QType("NVFP4", 40, 64, 36),
    ]
}
QTYPE_BY_ID: Dict[int, QType] = {q.ggml_id: q for q in QTYPES.values()}


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """fp32 [...]-> uint8 [..., 2] little-endian half bytes."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def _bytes_f16(b: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 2] -> fp32 [...]"""
    return b.contiguous().view(torch.float16).reshape(b.shape[:-1]).to(torch.float32)


def _nearest_int(x: torch.Tensor) -> torch.Tensor:
    return torch.round(x)


# --------------------------------------------------------------------------------------
# Q8_0
# --------------------------------------------------------------------------------------

def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    amax = x.abs().amax(-1)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = _nearest_int(x * inv[..., None]).clamp_(-127, 127).to(torch.int8)
    out = torch.empty(rows, k // 32, 34, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = q.view(torch.uint8)
    return out.reshape(rows, -1)


def dequantize_q8_0(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    blk = b.reshape(rows, k // 32, 34)
    d = _bytes_f16(blk[..., 0:2])
    q = blk[..., 2:].contiguous().view(torch.int8).float()
    return (q * d[..., None]).reshape(rows, k)


# --------------------------------------------------------------------------------------
# Q4_0 / Q4_1 / Q5_0 / Q5_1
# --------------------------------------------------------------------------------------

def quantize_q4_0(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    idx = x.abs().argmax(-1, keepdim=True)
    mx = torch.gather(x, -1, idx).squeeze(-1)  # signed value of max magnitude
    d = mx / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (x * inv[..., None] + 8.5).floor().clamp_(0, 15).to(torch.uint8)
    out = torch.empty(rows, k // 32, 18, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(rows, -1)


def dequantize_q4_0(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    blk = b.reshape(rows, k // 32, 18)
    d = _bytes_f16(blk[..., 0:2])
    qs = blk[..., 2:]
    q = torch.cat([qs & 0xF, qs >> 4], -1).float() - 8.0
    return (q * d[..., None]).reshape(rows, k)


def quantize_q4_1(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    mn, mx = x.amin(-1), x.amax(-1)
    d = (mx - mn) / 15.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = ((x - mn[..., None]) * inv[..., None] + 0.5).floor().clamp_(0, 15).to(torch.uint8)
    out = torch.empty(rows, k // 32, 20, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:4] = _f16_bytes(mn)
    out[..., 4:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(rows, -1)


def dequantize_q4_1(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    blk = b.reshape(rows, k // 32, 20)
    d = _bytes_f16(blk[..., 0:2])
    m = _bytes_f16(blk[..., 2:4])
    qs = blk[..., 4:]
    q = torch.cat([qs & 0xF, qs >> 4], -1).float()
    return (q * d[..., None] + m[..., None]).reshape(rows, k)


def _pack_bits32(bits: torch.Tensor) -> torch.Tensor:
    """bits uint8 [..., 32] (0/1) -> uint8 [..., 4] little-endian u32."""
    b = bits.reshape(*bits.shape[:-1], 4, 8).to(torch.int32)
    sh = torch.arange(8, device=bits.device, dtype=torch.int32)
    return (b << sh).sum(-1).to(torch.uint8)


def _unpack_bits32(b: torch.Tensor) -> torch.Tensor:
    sh = torch.arange(8, device=b.device, dtype=torch.uint8)
    return ((b[..., None] >> sh) & 1).reshape(*b.shape[:-1], 32)


def quantize_q5_0(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    idx = x.abs().argmax(-1, keepdim=True)
    mx = torch.gather(x, -1, idx).squeeze(-1)
    d = mx / -16.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = (x * inv[..., None] + 16.5).floor().clamp_(0, 31).to(torch.uint8)
    out = torch.empty(rows, k // 32, 22, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:6] = _pack_bits32(q >> 4)
    lo = q & 0xF
    out[..., 6:] = lo[..., :16] | (lo[..., 16:] << 4)
    return out.reshape(rows, -1)


def dequantize_q5_0(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    blk = b.reshape(rows, k // 32, 22)
    d = _bytes_f16(blk[..., 0:2])
    hi = _unpack_bits32(blk[..., 2:6])
    qs = blk[..., 6:]
    q = (torch.cat([qs & 0xF, qs >> 4], -1) | (hi << 4)).float() - 16.0
    return (q * d[..., None]).reshape(rows, k)


def quantize_q5_1(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    mn, mx = x.amin(-1), x.amax(-1)
    d = (mx - mn) / 31.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = ((x - mn[..., None]) * inv[..., None] + 0.5).floor().clamp_(0, 31).to(torch.uint8)
    out = torch.empty(rows, k // 32, 24, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:4] = _f16_bytes(mn)
    out[..., 4:8] = _pack_bits32(q >> 4)
    lo = q & 0xF
    out[..., 8:] = lo[..., :16] | (lo[..., 16:] << 4)
    return out.reshape(rows, -1)


def dequantize_q5_1(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    blk = b.reshape(rows, k // 32, 24)
    d = _bytes_f16(blk[..., 0:2])
    m = _bytes_f16(blk[..., 2:4])
    hi = _unpack_bits32(blk[..., 4:8])
    qs = blk[..., 8:]
    q = (torch.cat([qs & 0xF, qs >> 4], -1) | (hi << 4)).float()
    return (q * d[..., None] + m[..., None]).reshape(rows, k)


# --------------------------------------------------------------------------------------
# K-quant helpers: 6-bit (scale, min) pairs packed into 12 bytes
# --------------------------------------------------------------------------------------

def pack_scale_min_k4(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """sc, mn: uint8 [..., 8] with values < 64 -> uint8 [..., 12]."""
    out = torch.empty(*sc.shape[:-1], 12, dtype=torch.uint8, device=sc.device)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0xF) | ((mn[..., 4:8] & 0xF) << 4)
    return out


def unpack_scale_min_k4(q: torch.Tensor):
    """uint8 [..., 12] -> (sc, mn) uint8 [..., 8]."""
    sc_lo = q[..., 0:4] & 63
    mn_lo = q[..., 4:8] & 63
    sc_hi = (q[..., 8:12] & 0xF) | ((q[..., 0:4] >> 6) << 4)
    mn_hi = (q[..., 8:12] >> 4) | ((q[..., 4:8] >> 6) << 4)
    return torch.cat([sc_lo, sc_hi], -1), torch.cat([mn_lo, mn_hi], -1)


def _kquant_scale_min(x: torch.Tensor, nmax: int):
    """Per 32-value sub-block affine fit: x ~ scale * q - mn, q in [0, nmax], mn >= 0.

    A plain range fit (the reference's quantizer and llama.cpp search over
    candidate scales; a fixture needs only a valid encoding of nearby values).
    """
    lo = torch.clamp(x.amin(-1), max=0.0)
    hi = torch.clamp(x.amax(-1), min=0.0)
    scale = (hi - lo) / float(nmax)
    return scale, -lo


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    nsb = k // QK_K
    x = w.float().reshape(rows, nsb, 8, 32)
    scale, mn = _kquant_scale_min(x, 15)
    d = scale.amax(-1) / 63.0
    dmin = mn.amax(-1) / 63.0
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_dm = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = _nearest_int(scale * inv_d[..., None]).clamp_(0, 63).to(torch.uint8)
    mq = _nearest_int(mn * inv_dm[..., None]).clamp_(0, 63).to(torch.uint8)
    # re-encode against the values the decoder will see (half-rounded d, dmin)
    d16 = d.to(torch.float16).float()
    dm16 = dmin.to(torch.float16).float()
    eff = d16[..., None] * sc.float()
    off = dm16[..., None] * mq.float()
    inv_eff = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = _nearest_int((x + off[..., None]) * inv_eff[..., None]).clamp_(0, 15).to(torch.uint8)
    out = torch.empty(rows, nsb, 144, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:4] = _f16_bytes(dmin)
    out[..., 4:16] = pack_scale_min_k4(sc, mq)
    q = q.reshape(rows, nsb, 4, 2, 32)
    out[..., 16:] = (q[..., 0, :] | (q[..., 1, :] << 4)).reshape(rows, nsb, 128)
    return out.reshape(rows, -1)


def dequantize_q4_k(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    nsb = k // QK_K
    blk = b.reshape(rows, nsb, 144)
    d = _bytes_f16(blk[..., 0:2])
    dmin = _bytes_f16(blk[..., 2:4])
    sc, mn = unpack_scale_min_k4(blk[..., 4:16])
    qs = blk[..., 16:].reshape(rows, nsb, 4, 32)
    q = torch.stack([qs & 0xF, qs >> 4], 3).reshape(rows, nsb, 8, 32).float()
    y = q * (d[..., None] * sc.float())[..., None] - (dmin[..., None] * mn.float())[..., None]
    return y.reshape(rows, k)


def quantize_q5_k(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    nsb = k // QK_K
    x = w.float().reshape(rows, nsb, 8, 32)
    scale, mn = _kquant_scale_min(x, 31)
    d = scale.amax(-1) / 63.0
    dmin = mn.amax(-1) / 63.0
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_dm = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = _nearest_int(scale * inv_d[..., None]).clamp_(0, 63).to(torch.uint8)
    mq = _nearest_int(mn * inv_dm[..., None]).clamp_(0, 63).to(torch.uint8)
    d16 = d.to(torch.float16).float()
    dm16 = dmin.to(torch.float16).float()
    eff = d16[..., None] * sc.float()
    off = dm16[..., None] * mq.float()
    inv_eff = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = _nearest_int((x + off[..., None]) * inv_eff[..., None]).clamp_(0, 31).to(torch.uint8)
    out = torch.empty(rows, nsb, 176, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:4] = _f16_bytes(dmin)
    out[..., 4:16] = pack_scale_min_k4(sc, mq)
    hi = (q >> 4).to(torch.int32)  # [rows, nsb, 8, 32]
    sh = torch.arange(8, device=w.device, dtype=torch.int32).reshape(1, 1, 8, 1)
    out[..., 16:48] = (hi << sh).sum(2).to(torch.uint8)
    lo = (q & 0xF).reshape(rows, nsb, 4, 2, 32)
    out[..., 48:] = (lo[..., 0, :] | (lo[..., 1, :] << 4)).reshape(rows, nsb, 128)
    return out.reshape(rows, -1)


def dequantize_q5_k(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    nsb = k // QK_K
    blk = b.reshape(rows, nsb, 176)
    d = _bytes_f16(blk[..., 0:2])
    dmin = _bytes_f16(blk[..., 2:4])
    sc, mn = unpack_scale_min_k4(blk[..., 4:16])
    qh = blk[..., 16:48]
    qs = blk[..., 48:].reshape(rows, nsb, 4, 32)
    lo = torch.stack([qs & 0xF, qs >> 4], 3).reshape(rows, nsb, 8, 32)
    sh = torch.arange(8, device=b.device, dtype=torch.uint8).reshape(1, 1, 8, 1)
    hi = (qh[:, :, None, :] >> sh) & 1
    q = (lo | (hi << 4)).float()
    y = q * (d[..., None] * sc.float())[..., None] - (dmin[..., None] * mn.float())[..., None]
    return y.reshape(rows, k)


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    nsb = k // QK_K
    x = w.float().reshape(rows, nsb, 16, 16)
    idx = x.abs().argmax(-1, keepdim=True)
    mx = torch.gather(x, -1, idx).squeeze(-1)
    scale = mx / -32.0  # per 16 values, signed
    idx2 = scale.abs().argmax(-1, keepdim=True)
    smax = torch.gather(scale, -1, idx2).squeeze(-1)
    d = smax / -128.0
    inv_d = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    sc = _nearest_int(scale * inv_d[..., None]).clamp_(-128, 127)
    d16 = d.to(torch.float16).float()
    eff = d16[..., None] * sc
    inv_eff = torch.where(eff != 0, 1.0 / eff, torch.zeros_like(eff))
    q = (_nearest_int(x * inv_eff[..., None]).clamp_(-32, 31) + 32).to(torch.uint8)
    q = q.reshape(rows, nsb, 2, 4, 32)  # half n, quarter (0,32,64,96), l
    lo = q & 0xF
    hi = q >> 4
    out = torch.empty(rows, nsb, 210, dtype=torch.uint8, device=w.device)
    ql = torch.stack([lo[:, :, :, 0] | (lo[:, :, :, 2] << 4), lo[:, :, :, 1] | (lo[:, :, :, 3] << 4)], 3)
    out[..., 0:128] = ql.reshape(rows, nsb, 128)
    qh = hi[:, :, :, 0] | (hi[:, :, :, 1] << 2) | (hi[:, :, :, 2] << 4) | (hi[:, :, :, 3] << 6)
    out[..., 128:192] = qh.reshape(rows, nsb, 64)
    out[..., 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[..., 208:210] = _f16_bytes(d)
    return out.reshape(rows, -1)


def dequantize_q6_k(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    nsb = k // QK_K
    blk = b.reshape(rows, nsb, 210)
    ql = blk[..., 0:128].reshape(rows, nsb, 2, 2, 32)
    qh = blk[..., 128:192].reshape(rows, nsb, 2, 32)
    sc = blk[..., 192:208].contiguous().view(torch.int8).float()
    d = _bytes_f16(blk[..., 208:210])
    q0 = (ql[:, :, :, 0] & 0xF) | (((qh >> 0) & 3) << 4)
    q1 = (ql[:, :, :, 1] & 0xF) | (((qh >> 2) & 3) << 4)
    q2 = (ql[:, :, :, 0] >> 4) | (((qh >> 4) & 3) << 4)
    q3 = (ql[:, :, :, 1] >> 4) | (((qh >> 6) & 3) << 4)
    q = torch.stack([q0, q1, q2, q3], 3).reshape(rows, nsb, 16, 16).float() - 32.0
    y = q * (d[..., None] * sc)[..., None]
    return y.reshape(rows, k)


def dequantize_q2_k(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    nsb = k // QK_K
    blk = b.reshape(rows, nsb, 84)
    scales = blk[..., 0:16]
    qs = blk[..., 16:80].reshape(rows, nsb, 2, 32)
    d = _bytes_f16(blk[..., 80:82])
    dmin = _bytes_f16(blk[..., 82:84])
    sh = torch.tensor([0, 2, 4, 6], device=b.device, dtype=torch.uint8).reshape(1, 1, 1, 4, 1)
    q = ((qs[:, :, :, None, :] >> sh) & 3).reshape(rows, nsb, 16, 16).float()
    dl = d[..., None] * (scales & 0xF).float()
    ml = dmin[..., None] * (scales >> 4).float()
    return (q * dl[..., None] - ml[..., None]).reshape(rows, k)


def quantize_q2_k(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    nsb = k // QK_K
    x = w.float().reshape(rows, nsb, 16, 16)
    lo = torch.clamp(x.amin(-1), max=0.0)
    hi = torch.clamp(x.amax(-1), min=0.0)
    scale, mn = (hi - lo) / 3.0, -lo
    d = scale.amax(-1) / 15.0
    dmin = mn.amax(-1) / 15.0
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_dm = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = _nearest_int(scale * inv_d[..., None]).clamp_(0, 15).to(torch.uint8)
    mq = _nearest_int(mn * inv_dm[..., None]).clamp_(0, 15).to(torch.uint8)
    eff = d.to(torch.float16).float()[..., None] * sc.float()
    off = dmin.to(torch.float16).float()[..., None] * mq.float()
    inv_eff = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
    q = _nearest_int((x + off[..., None]) * inv_eff[..., None]).clamp_(0, 3).to(torch.uint8)
    q = q.reshape(rows, nsb, 2, 4, 32)
    out = torch.empty(rows, nsb, 84, dtype=torch.uint8, device=w.device)
    out[..., 0:16] = sc | (mq << 4)
    out[..., 16:80] = (q[:, :, :, 0] | (q[:, :, :, 1] << 2) | (q[:, :, :, 2] << 4) | (q[:, :, :, 3] << 6)).reshape(rows, nsb, 64)
    out[..., 80:82] = _f16_bytes(d)
    out[..., 82:84] = _f16_bytes(dmin)
    return out.reshape(rows, -1)


def dequantize_q3_k(b: torch.Tensor, k: int) -> torch.Tensor:
    rows = b.shape[0]
    nsb = k // QK_K
    blk = b.reshape(rows, nsb, 110)
    hmask = blk[..., 0:32]
    qs = blk[..., 32:96].reshape(rows, nsb, 2, 32)
    sb = blk[..., 96:108].to(torch.int32)
    d = _bytes_f16(blk[..., 108:110])
    # 16 6-bit scales: low 4 bits in bytes 0..7 (two nibbles), high 2 bits in bytes 8..11
    lo4 = torch.cat([sb[..., 0:8] & 0xF, sb[..., 0:8] >> 4], -1)
    hi2 = torch.cat([(sb[..., 8:12] >> s) & 3 for s in (0, 2, 4, 6)], -1)
    sc = ((lo4 | (hi2 << 4)) - 32).float()
    sh = torch.tensor([0, 2, 4, 6], device=b.device, dtype=torch.uint8).reshape(1, 1, 1, 4, 1)
    q = ((qs[:, :, :, None, :] >> sh) & 3).reshape(rows, nsb, 8, 32).to(torch.int32)
    hb = torch.arange(8, device=b.device, dtype=torch.uint8).reshape(1, 1, 8, 1)
    h = ((hmask[:, :, None, :] >> hb) & 1).to(torch.int32)
    q = (q - 4 * (1 - h)).reshape(rows, nsb, 16, 16).float()
    return (q * (d[..., None] * sc)[..., None]).reshape(rows, k)


def quantize_q3_k(w: torch.Tensor) -> torch.Tensor:
    rows, k = w.shape
    nsb = k // QK_K
    x = w.float().reshape(rows, nsb, 16, 16)
    idx = x.abs().argmax(-1, keepdim=True)
    mx = torch.gather(x, -1, idx).squeeze(-1)
    scale = mx / -4.0
    idx2 = scale.abs().argmax(-1, keepdim=True)
    smax = torch.gather(scale, -1, idx2).squeeze(-1)
    d = smax / -32.0
    inv_d = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    sc = _nearest_int(scale * inv_d[..., None]).clamp_(-32, 31)
    eff = d.to(torch.float16).float()[..., None] * sc
    inv_eff = torch.where(eff != 0, 1.0 / eff, torch.zeros_like(eff))
    q = (_nearest_int(x * inv_eff[..., None]).clamp_(-4, 3) + 4).to(torch.uint8)  # 0..7
    q = q.reshape(rows, nsb, 8, 32)
    hbit = (q >> 2).to(torch.int32)
    sh = torch.arange(8, device=w.device, dtype=torch.int32).reshape(1, 1, 8, 1)
    out = torch.empty(rows, nsb, 110, dtype=torch.uint8, device=w.device)
    out[..., 0:32] = (hbit << sh).sum(2).to(torch.uint8)
    lo = (q & 3).reshape(rows, nsb, 2, 4, 32)
    out[..., 32:96] = (lo[:, :, :, 0] | (lo[:, :, :, 1] << 2) | (lo[:, :, :, 2] << 4) | (lo[:, :, :, 3] << 6)).reshape(rows, nsb, 64)
    s6 = (sc + 32).to(torch.uint8)  # 0..63, [rows,nsb,16]
    out[..., 96:104] = (s6[..., 0:8] & 0xF) | ((s6[..., 8:16] & 0xF) << 4)
    h = s6 >> 4
    out[..., 104:108] = h[..., 0:4] | (h[..., 4:8] << 2) | (h[..., 8:12] << 4) | (h[..., 12:16] << 6)
    out[..., 108:110] = _f16_bytes(d)
    return out.reshape(rows, -1)


# --------------------------------------------------------------------------------------
# plain float types
# --------------------------------------------------------------------------------------

def _q_plain(dtype):
    def q(w: torch.Tensor) -> torch.Tensor:
        return w.to(dtype).contiguous().view(torch.uint8).reshape(w.shape[0], -1)

    return q


def _dq_plain(dtype):
    def dq(b: torch.Tensor, k: int) -> torch.Tensor:
        return b.contiguous().view(dtype).reshape(b.shape[0], k).float()

    return dq


# --------------------------------------------------------------------------------------
# Non-linear 4-bit types (IQ4_NL, IQ4_XS), MXFP4 and the grid type IQ2_XXS.
#   IQ4_NL   32 values: f16 d, 16 bytes of nibbles (value j low nibble of byte j, value j + 16 high); d * kvalues[q]
#   IQ4_XS  256 values: f16 d, u16 scales_h, scales_l[4], qs[128]; 6-bit scale ls per 32, d * (ls - 32) * kvalues[q]
#   MXFP4    32 values: E8M0 byte, 16 bytes of nibbles (same order); 2^(E-128) * kvalues_mxfp4[q]
#   IQ2_XXS 256 values: f16 d, eight (idx u32, aux u32) pairs; per 8 values a grid byte and a 7-bit sign index, per 32
#           a 4-bit scale s in aux[28:32]; d * (0.5 + s) * 0.25 * grid * sign
# The encoders are plain nearest-code searches (fixtures and tests); the decoders are the file format.
# --------------------------------------------------------------------------------------

def _nibbles(qs: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 16] -> int64 codes [..., 32] in value order (low nibbles first)."""
    q = qs.to(torch.int64)
    return torch.cat([q & 0xF, q >> 4], -1)


def _pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """int codes [..., 32] -> uint8 [..., 16]."""
    return (codes[..., :16] | (codes[..., 16:] << 4)).to(torch.uint8)


def _nearest_code(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """index of the table value nearest to every x."""
    return (x[..., None] - table).abs().argmin(-1)


def dequantize_iq4_nl(b: torch.Tensor, k: int) -> torch.Tensor:
    from .iq_tables import KVALUES_IQ4NL
    rows = b.shape[0]
    blk = b.reshape(rows, k // 32, 18)
    d = _bytes_f16(blk[..., 0:2])
    lut = torch.tensor(KVALUES_IQ4NL, dtype=torch.float32, device=b.device)
    return (lut[_nibbles(blk[..., 2:])] * d[..., None]).reshape(rows, k)


def quantize_iq4_nl(w: torch.Tensor) -> torch.Tensor:
    from .iq_tables import KVALUES_IQ4NL
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    lut = torch.tensor(KVALUES_IQ4NL, dtype=torch.float32, device=w.device)
    # the value of largest magnitude lands on the table's end of the same sign
    idx = x.abs().argmax(-1, keepdim=True)
    mx = x.gather(-1, idx).squeeze(-1)
    d = (mx / torch.where(mx < 0, lut[0], lut[15])).to(torch.float16).float()
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    codes = _nearest_code(x * inv[..., None], lut)
    out = torch.empty(rows, k // 32, 18, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:] = _pack_nibbles(codes)
    return out.reshape(rows, -1)


def _iq4_xs_scales(blk: torch.Tensor) -> torch.Tensor:
    """6-bit sub-block scales [..., 8] of IQ4_XS blocks [..., 136]."""
    sh = blk[..., 2].to(torch.int64) | (blk[..., 3].to(torch.int64) << 8)
    sl = blk[..., 4:8].to(torch.int64)
    ib = torch.arange(8, device=blk.device)
    lo = (sl[..., ib // 2] >> (4 * (ib % 2))) & 0xF
    hi = (sh[..., None] >> (2 * ib)) & 3
    return lo | (hi << 4)


def dequantize_iq4_xs(b: torch.Tensor, k: int) -> torch.Tensor:
    from .iq_tables import KVALUES_IQ4NL
    rows = b.shape[0]
    blk = b.reshape(rows, k // 256, 136)
    d = _bytes_f16(blk[..., 0:2])
    dl = d[..., None] * (_iq4_xs_scales(blk) - 32).float()                     # [rows, nsb, 8]
    lut = torch.tensor(KVALUES_IQ4NL, dtype=torch.float32, device=b.device)
    v = lut[_nibbles(blk[..., 8:].reshape(rows, k // 256, 8, 16))]           # [rows, nsb, 8, 32]
    return (v * dl[..., None]).reshape(rows, k)


def quantize_iq4_xs(w: torch.Tensor) -> torch.Tensor:
    from .iq_tables import KVALUES_IQ4NL
    rows, k = w.shape
    nsb = k // 256
    x = w.float().reshape(rows, nsb, 8, 32)
    lut = torch.tensor(KVALUES_IQ4NL, dtype=torch.float32, device=w.device)
    idx = x.abs().argmax(-1, keepdim=True)
    mx = x.gather(-1, idx).squeeze(-1)                                       # signed extreme of every sub-block
    dl = mx / torch.where(mx < 0, lut[0], lut[15])                           # ideal sub-block scale (>= 0)
    d = (dl.amax(-1) / 31.0).to(torch.float16).float()                       # ls - 32 in 0 .. 31
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    ls = (torch.round(dl * inv[..., None]).clamp_(0, 31) + 32).to(torch.int64)
    eff = d[..., None] * (ls - 32).float()
    inv_eff = torch.where(eff != 0, 1.0 / eff, torch.zeros_like(eff))
    codes = _nearest_code(x * inv_eff[..., None], lut)
    out = torch.zeros(rows, nsb, 136, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    sh = torch.zeros(rows, nsb, dtype=torch.int64, device=w.device)
    for ib in range(8):
        sh |= (ls[..., ib] >> 4) << (2 * ib)
    out[..., 2] = (sh & 0xFF).to(torch.uint8)
    out[..., 3] = (sh >> 8).to(torch.uint8)
    out[..., 4:8] = ((ls[..., 0::2] & 0xF) | ((ls[..., 1::2] & 0xF) << 4)).to(torch.uint8)
    out[..., 8:] = _pack_nibbles(codes).reshape(rows, nsb, 128)
    return out.reshape(rows, -1)


def dequantize_mxfp4(b: torch.Tensor, k: int) -> torch.Tensor:
    from .iq_tables import KVALUES_MXFP4, e8m0_half
    rows = b.shape[0]
    blk = b.reshape(rows, k // 32, 17)
    d = e8m0_half(blk[..., 0])
    lut = torch.tensor(KVALUES_MXFP4, dtype=torch.float32, device=b.device)
    return (lut[_nibbles(blk[..., 1:])] * d[..., None]).reshape(rows, k)


def quantize_mxfp4(w: torch.Tensor) -> torch.Tensor:
    from .iq_tables import KVALUES_MXFP4, e8m0_half
    rows, k = w.shape
    x = w.float().reshape(rows, k // 32, 32)
    amax = x.abs().amax(-1).clamp_min(1e-30)
    # smallest power-of-two block scale whose largest code (12 * half scale) covers the block
    e = (torch.ceil(torch.log2(amax / 12.0)) + 128).clamp_(2, 254).to(torch.uint8)
    d = e8m0_half(e)
    lut = torch.tensor(KVALUES_MXFP4, dtype=torch.float32, device=w.device)
    mag = _nearest_code((x / d[..., None]).abs(), lut[:8])
    codes = mag | ((x < 0) & (mag > 0)).to(torch.int64) << 3
    out = torch.empty(rows, k // 32, 17, dtype=torch.uint8, device=w.device)
    out[..., 0] = e
    out[..., 1:] = _pack_nibbles(codes)
    return out.reshape(rows, -1)


def _iq2_xxs_fields(b: torch.Tensor, k: int):
    rows = b.shape[0]
    blk = b.reshape(rows, k // 256, 66)
    d = _bytes_f16(blk[..., 0:2])
    words = blk[..., 2:].reshape(rows, k // 256, 8, 8).to(torch.int64)
    gidx = words[..., 0:4]                                                   # [rows, nsb, 8, 4] grid entries
    aux = words[..., 4] | (words[..., 5] << 8) | (words[..., 6] << 16) | (words[..., 7] << 24)
    sidx = torch.stack([(aux >> (7 * l)) & 127 for l in range(4)], -1)      # [rows, nsb, 8, 4]
    scale = aux >> 28                                                        # [rows, nsb, 8]
    return d, gidx, sidx, scale


def dequantize_iq2_xxs(b: torch.Tensor, k: int) -> torch.Tensor:
    from .iq_tables import iq2_signs, iq2xxs_grid
    rows = b.shape[0]
    d, gidx, sidx, scale = _iq2_xxs_fields(b, k)
    grid = iq2xxs_grid().to(b.device).float()
    signs = iq2_signs().to(b.device)
    db = d[..., None] * (0.5 + scale.float()) * 0.25                        # [rows, nsb, 8]
    v = grid[gidx] * signs[sidx]                                             # [rows, nsb, 8, 4, 8]
    return (v * db[..., None, None]).reshape(rows, k)


def quantize_iq2_xxs(w: torch.Tensor) -> torch.Tensor:
    """Nearest grid entry per eight values (exhaustive over the 256 entries), even sign parity by flipping the value
    with the least at stake, one 4-bit scale per 32 values."""
    from .iq_tables import iq2xxs_grid
    rows, k = w.shape
    nsb = k // 256
    x = w.float().reshape(rows, nsb, 8, 4, 8)
    grid = iq2xxs_grid().to(w.device).float()                                # [256, 8]
    amax32 = x.abs().amax((-1, -2))                                          # [rows, nsb, 8]
    # db * 43 covers the sub-block's largest magnitude; db = d * (0.5 + s) / 4 with s <= 15
    db_ideal = amax32 / 43.0
    d = (db_ideal.amax(-1) * 4.0 / 15.5).to(torch.float16).float()
    inv_d = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    s = torch.round(db_ideal * 4.0 * inv_d[..., None] - 0.5).clamp_(0, 15).to(torch.int64)
    db = d[..., None] * (0.5 + s.float()) * 0.25
    inv_db = torch.where(db != 0, 1.0 / db, torch.zeros_like(db))
    mag = x.abs() * inv_db[..., None, None]                                  # in grid units
    err = ((mag[..., None, :] - grid) ** 2).sum(-1)                          # [rows, nsb, 8, 4, 256]
    gidx = err.argmin(-1)
    neg = x < 0
    odd = neg.sum(-1) % 2 == 1
    # an odd number of minus signs cannot be stored: flip the sign of the value whose product with its grid magnitude
    # is smallest
    stake = mag * grid[gidx]
    flip = torch.nn.functional.one_hot(stake.argmin(-1), 8).bool() & odd[..., None]
    neg = neg ^ flip
    bits = (neg[..., :7].to(torch.int64) << torch.arange(7, device=w.device)).sum(-1)   # the eighth follows from parity
    aux = (s << 28)
    for l in range(4):
        aux = aux | (bits[..., l] << (7 * l))
    out = torch.zeros(rows, nsb, 66, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _f16_bytes(d)
    words = torch.zeros(rows, nsb, 8, 8, dtype=torch.int64, device=w.device)
    words[..., 0:4] = gidx
    for j in range(4):
        words[..., 4 + j] = (aux >> (8 * j)) & 0xFF
    out[..., 2:] = words.to(torch.uint8).reshape(rows, nsb, 64)
    return out.reshape(rows, -1)


def code_scale_form(b: torch.Tensor, qtype: str, k: int):
    """Blocks of IQ4_NL / IQ4_XS / MXFP4 / IQ2_XXS as (int8 codes [rows, k], f32 scales [rows, k / 32]) with
    value = code * scale exactly: every code of these types is a small integer and every 32 values share one scale."""
    from .iq_tables import KVALUES_IQ4NL, KVALUES_MXFP4, e8m0_half, iq2_signs, iq2xxs_grid
    rows = b.shape[0]
    if qtype == "IQ4_NL":
        blk = b.reshape(rows, k // 32, 18)
        lut = torch.tensor(KVALUES_IQ4NL, dtype=torch.int8, device=b.device)
        return lut[_nibbles(blk[..., 2:])].reshape(rows, k), _bytes_f16(blk[..., 0:2])
    if qtype == "MXFP4":
        blk = b.reshape(rows, k // 32, 17)
        lut = torch.tensor(KVALUES_MXFP4, dtype=torch.int8, device=b.device)
        return lut[_nibbles(blk[..., 1:])].reshape(rows, k), e8m0_half(blk[..., 0])
    if qtype == "IQ4_XS":
        blk = b.reshape(rows, k // 256, 136)
        lut = torch.tensor(KVALUES_IQ4NL, dtype=torch.int8, device=b.device)
        dl = _bytes_f16(blk[..., 0:2])[..., None] * (_iq4_xs_scales(blk) - 32).float()
        return lut[_nibbles(blk[..., 8:].reshape(rows, k // 256, 8, 16))].reshape(rows, k), dl.reshape(rows, k // 32)
    if qtype == "IQ2_XXS":
        d, gidx, sidx, scale = _iq2_xxs_fields(b, k)
        codes = (iq2xxs_grid().to(b.device).float()[gidx] * iq2_signs().to(b.device)[sidx]).to(torch.int8)
        db = d[..., None] * (0.5 + scale.float()) * 0.25
        return codes.reshape(rows, k), db.reshape(rows, k // 32)
    raise ValueError(f"{qtype} has no code * scale form")


QUANTIZE: Dict[str, Callable[[torch.Tensor], torch.Tensor]] = {
    "F32": _q_plain(torch.float32),
    "F16": _q_plain(torch.float16),
    "BF16": _q_plain(torch.bfloat16),
    "Q8_0": quantize_q8_0,
    "Q4_0": quantize_q4_0,
    "Q4_1": quantize_q4_1,
    "Q5_0": quantize_q5_0,
    "Q5_1": quantize_q5_1,
    "Q2_K": quantize_q2_k,
    "Q3_K": quantize_q3_k,
    "Q4_K": quantize_q4_k,
    "Q5_K": quantize_q5_k,
    "Q6_K": quantize_q6_k,
    "IQ4_NL": quantize_iq4_nl,
    "IQ4_XS": quantize_iq4_xs,
    "MXFP4": quantize_mxfp4,
    "IQ2_XXS": quantize_iq2_xxs,
}

DEQUANTIZE: Dict[str, Callable[[torch.Tensor, int], torch.Tensor]] = {
    "F32": _dq_plain(torch.float32),
    "F16": _dq_plain(torch.float16),
    "BF16": _dq_plain(torch.bfloat16),
    "Q8_0": dequantize_q8_0,
    "Q4_0": dequantize_q4_0,
    "Q4_1": dequantize_q4_1,
    "Q5_0": dequantize_q5_0,
    "Q5_1": dequantize_q5_1,
    "Q2_K": dequantize_q2_k,
    "Q3_K": dequantize_q3_k,
    "Q4_K": dequantize_q4_k,
    "Q5_K": dequantize_q5_k,
    "Q6_K": dequantize_q6_k,
    "IQ4_NL": dequantize_iq4_nl,
    "IQ4_XS": dequantize_iq4_xs,
    "MXFP4": dequantize_mxfp4,
    "IQ2_XXS": dequantize_iq2_xxs,
}


def quantize(w: torch.Tensor, qtype: str) -> torch.Tensor:
    """[rows, k] float -> uint8 [rows, row_bytes] in the named block format."""
    if w.dim() != 2:
        raise ValueError("quantize takes a 2-D [rows, k] tensor")
    QTYPES[qtype].row_bytes(w.shape[1])
    return QUANTIZE[qtype](w)


def dequantize(b: torch.Tensor, qtype: str, k: int) -> torch.Tensor:
    """uint8 [rows, row_bytes] -> fp32 [rows, k]."""
    if b.dtype != torch.uint8 or b.dim() != 2:
        raise ValueError("dequantize takes a 2-D uint8 tensor")
    if b.shape[1] != QTYPES[qtype].row_bytes(k):
        raise ValueError(f"{qtype}: {b.shape[1]} bytes per row does not match k={k}")
    return DEQUANTIZE[qtype](b, k)


# --------------------------------------------------------------------------------------
# q8 activation form used by every integer-dot kernel
# --------------------------------------------------------------------------------------

def quantize_act_q8(x: torch.Tensor):
    """fp32 [m, k] -> (codes int8 [m, k], ds fp32 [m, k/32, 2]).

    One scale ``d`` and one scaled code sum ``s = d * sum(q)`` per 32 values,
    the 32-value activation form of the reference (``crates/gpu/src/gemm/gemm32.rs``
    doc, ``Q8Blocks32``).  ``d = amax/127``; codes round to nearest even like
    ``__float2int_rn`` on the card.
    """
    m, k = x.shape
    xb = x.float().reshape(m, k // 32, 32)
    amax = xb.abs().amax(-1)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(xb * inv[..., None]).clamp_(-127, 127)
    s = d * q.sum(-1)
    return q.to(torch.int8).reshape(m, k), torch.stack([d, s], -1)


def dequantize_act_q8(codes: torch.Tensor, ds: torch.Tensor) -> torch.Tensor:
    m, k = codes.shape
    return (codes.float().reshape(m, k // 32, 32) * ds[..., 0:1]).reshape(m, k)
