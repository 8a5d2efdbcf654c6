"""Block-scaled float checkpoints: FP8 128x128 blocks and NVFP4, as stored by checkpoint
folders, and their resident row layouts.

Stored forms (the reference: ``crates/hf/src/modelopt.rs``, ``crates/hf/src/quant_config.rs``,
``crates/gguf/src/quant.rs`` FP8_B128):

  transformers ``fp8``          ``W.weight`` F8_E4M3 [N, K], ``W.weight_scale_inv`` F32 [ceil(N/128), ceil(K/128)]
  ModelOpt NVFP4                ``W.weight`` U8 [N, K/2] (two E2M1 codes per byte, low nibble first),
                                ``W.weight_scale`` F8_E4M3 [N, K/16], ``W.weight_scale_2`` F32 scalar (a multiplier)
  compressed-tensors            ``W.weight_packed`` U8 [N, K/2], ``W.weight_scale`` F8_E4M3 [N, K/16],
  ``nvfp4-pack-quantized``      ``W.weight_global_scale`` F32 scalar (a DIVISOR)

Resident rows (what the kernels read; values are never re-quantised):

  FP8_B128   K code bytes, then K/128 f32 scales (the block scale replicated into the row), pad to 16
  NVFP4      K/2 code bytes, K/16 E4M3 scale bytes, one f32 tensor scale, pad to 16
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
E4M3_MAX = 448.0


class PlaneError(ValueError):
    pass


def e4m3_decode(codes: torch.Tensor) -> torch.Tensor:
    """uint8 codes -> f32 (the one NaN encoding S.1111.111 decodes to NaN)."""
    c = codes.to(torch.int32)
    s, e, m = c >> 7, (c >> 3) & 15, c & 7
    v = torch.where(e == 0, m.float() * 2.0 ** -9, (1.0 + m.float() / 8.0) * torch.exp2((e - 7).float()))
    v = torch.where((e == 15) & (m == 7), torch.full_like(v, float("nan")), v)
    return torch.where(s == 1, -v, v)


_E4M3_TABLE: Optional[torch.Tensor] = None


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """f32 -> nearest finite E4M3 code (ties to the even code), saturating at +-448."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        _E4M3_TABLE = e4m3_decode(torch.arange(0, 127, dtype=torch.uint8))     # non-negative finite, ascending
    tab = _E4M3_TABLE.to(x.device)
    a = x.abs().clamp(max=E4M3_MAX).float()
    hi = torch.searchsorted(tab, a.contiguous()).clamp(max=126)
    lo = (hi - 1).clamp(min=0)
    dlo, dhi = a - tab[lo], tab[hi] - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    code = torch.where(pick_hi, hi, lo).to(torch.uint8)
    return code | ((x < 0).to(torch.uint8) << 7)


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    c = codes.to(torch.int64)
    v = E2M1_VALUES.to(codes.device)[c & 7]
    return torch.where((c & 8) != 0, -v, v)


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    tab = E2M1_VALUES.to(x.device)
    a = x.abs().clamp(max=6.0)
    idx = (a.unsqueeze(-1) - tab).abs().argmin(-1)
    return (idx | ((x < 0).to(torch.int64) << 3)).to(torch.uint8)


# ------------------------------------------------------------------------------------
# FP8 128x128
# ------------------------------------------------------------------------------------
def fp8_b128_quantize(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """f32 [N, K] -> (codes uint8 [N, K], scale_inv f32 [ceil(N/128), ceil(K/128)]) — a fixture writer."""
    n, k = w.shape
    nb, kb = (n + 127) // 128, (k + 127) // 128
    pad = torch.zeros(nb * 128, kb * 128, device=w.device)
    pad[:n, :k] = w
    blk = pad.reshape(nb, 128, kb, 128)
    amax = blk.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale = amax / E4M3_MAX
    codes = e4m3_encode(blk / scale[:, None, :, None]).reshape(nb * 128, kb * 128)[:n, :k].contiguous()
    return codes, scale


def fp8_b128_dequantize(codes: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    n, k = codes.shape
    s = scale_inv.float().repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :k]
    return e4m3_decode(codes) * s


def fp8_b128_resident(codes: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    """Resident rows.  Refuses NaN codes and non-finite scales, and a K that is not a multiple of 128."""
    n, k = codes.shape
    if k % 128:
        raise PlaneError(f"FP8_B128 rows must be a multiple of 128 values, got {k}")
    if scale_inv.shape != ((n + 127) // 128, k // 128):
        raise PlaneError(f"FP8 scale plane {tuple(scale_inv.shape)} does not cover {n}x{k} in 128x128 blocks")
    if bool(((codes & 0x7F) == 0x7F).any()):
        raise PlaneError("FP8 codes hold a NaN byte (0x7F/0xFF)")
    if not bool(torch.isfinite(scale_inv).all()):
        raise PlaneError("FP8 scale plane holds a non-finite scale")
    rb = (k + k // 32 + 15) // 16 * 16
    out = torch.zeros(n, rb, dtype=torch.uint8, device=codes.device)
    out[:, :k] = codes
    rows_scale = scale_inv.float().repeat_interleave(128, 0)[:n].contiguous()      # [n, k/128]
    out[:, k:k + 4 * (k // 128)] = rows_scale.view(torch.uint8).reshape(n, -1)
    return out


# ------------------------------------------------------------------------------------
# NVFP4
# ------------------------------------------------------------------------------------
def nvfp4_quantize(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """f32 [N, K] -> (packed uint8 [N, K/2], scales E4M3 uint8 [N, K/16], tensor scale f32 scalar)."""
    n, k = w.shape
    if k % 16:
        raise PlaneError("NVFP4 rows are a multiple of 16 values")
    g = w.reshape(n, k // 16, 16).float()
    amax = g.abs().amax(-1)
    tscale = (w.abs().max().clamp(min=1e-12) / (6.0 * E4M3_MAX)).float()
    sc_codes = e4m3_encode(amax / 6.0 / tscale)
    sc = e4m3_decode(sc_codes) * tscale
    codes = e2m1_encode(g / sc.clamp(min=1e-30).unsqueeze(-1)).reshape(n, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, sc_codes, tscale.reshape(())


def nvfp4_dequantize(packed: torch.Tensor, scales: torch.Tensor, tscale) -> torch.Tensor:
    n, kh = packed.shape
    codes = torch.stack([packed & 15, packed >> 4], -1).reshape(n, kh * 2)
    sc = e4m3_decode(scales).repeat_interleave(16, 1) * float(tscale)
    return e2m1_decode(codes) * sc


def nvfp4_resident(packed: torch.Tensor, scales: torch.Tensor, tscale) -> torch.Tensor:
    """Resident rows; ``tscale`` is the MULTIPLIER (callers invert a compressed-tensors divisor)."""
    n, kh = packed.shape
    k = kh * 2
    if k % 64:
        raise PlaneError(f"NVFP4 resident rows are a multiple of 64 values, got {k}")
    if scales.shape != (n, k // 16):
        raise PlaneError(f"NVFP4 scale plane {tuple(scales.shape)} does not match {n}x{k}")
    if bool(((scales & 0x7F) == 0x7F).any()):
        raise PlaneError("NVFP4 scale plane holds a NaN byte")
    ts = torch.as_tensor(tscale, dtype=torch.float32).reshape(-1)
    if ts.numel() not in (1, n) or not bool(torch.isfinite(ts).all()):
        raise PlaneError("NVFP4 tensor scale must be one finite f32 (or one per row)")
    rb = (k // 2 + k // 16 + 4 + 15) // 16 * 16
    out = torch.zeros(n, rb, dtype=torch.uint8, device=packed.device)
    out[:, :kh] = packed
    out[:, kh:kh + k // 16] = scales
    out[:, kh + k // 16:kh + k // 16 + 4] = ts.to(packed.device).expand(n).contiguous().view(torch.uint8).reshape(n, 4)
    return out


def resident_dequantize(res: torch.Tensor, qtype: str, k: int) -> torch.Tensor:
    """Oracle decode of resident rows (both types)."""
    n = res.shape[0]
    if qtype == "FP8_B128":
        sc = res[:, k:k + 4 * (k // 128)].contiguous().view(torch.float32).reshape(n, k // 128)
        return e4m3_decode(res[:, :k]) * sc.repeat_interleave(128, 1)
    if qtype == "NVFP4":
        kh = k // 2
        ts = res[:, kh + k // 16:kh + k // 16 + 4].contiguous().view(torch.float32).reshape(n, 1)
        packed = res[:, :kh]
        codes = torch.stack([packed & 15, packed >> 4], -1).reshape(n, k)
        # the kernels' order of operations: (group scale * tensor scale * 0.5) * (2 * E2M1 value), all f32
        sc = (e4m3_decode(res[:, kh:kh + k // 16]) * ts * 0.5).repeat_interleave(16, 1)
        return sc * (e2m1_decode(codes) * 2.0)
    raise PlaneError(qtype)


# ------------------------------------------------------------------------------------
# Checkpoint naming -> one linear layer's resident rows
# ------------------------------------------------------------------------------------
def mxfp8_dequantize(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """OCP MXFP8 (E4M3 codes [N, K], one E8M0 byte per 32 values [N, K / 32]) -> bf16 [N, K], exactly: a 3-bit mantissa
    times a power of two always fits bf16 while the exponent stays in its range."""
    n, k = codes.shape
    if k % 32 or tuple(scales.shape) != (n, k // 32):
        raise PlaneError(f"MXFP8 codes {tuple(codes.shape)} with scales {tuple(scales.shape)}: one scale byte per 32 values")
    if bool((scales == 255).any()):
        raise PlaneError("MXFP8 scale byte 255 (NaN)")
    out = torch.empty(n, k, dtype=torch.bfloat16, device=codes.device)
    for r0 in range(0, n, 8192):                       # rows per pass: the decode makes full-size f32 temporaries
        c = codes[r0:r0 + 8192]
        sc = torch.exp2(scales[r0:r0 + 8192].to(torch.float32) - 127.0)
        v = e4m3_decode(c.view(torch.uint8)).reshape(c.shape[0], k // 32, 32) * sc[:, :, None]
        out[r0:r0 + 8192] = v.reshape(c.shape[0], k).to(torch.bfloat16)
    return out


def mxfp4_resident(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """OCP MXFP4 as checkpoints pack it (two E2M1 codes a byte, the even value in the low nibble, [N, K / 2]; one E8M0
    byte per 32 values [N, K / 32]) -> resident ``Q8_F32`` rows: the doubled code values are small integers and half
    the block scale puts the factor back, so value = code * scale exactly (the form the GGUF MXFP4 blocks load as)."""
    from .iq_tables import KVALUES_MXFP4, e8m0_half
    from .resident import resident_row_bytes
    n, k = packed.shape[0], packed.shape[1] * 2
    if k % 32 or tuple(scales.shape) != (n, k // 32):
        raise PlaneError(f"MXFP4 codes {tuple(packed.shape)} with scales {tuple(scales.shape)}: one scale byte per 32 values")
    if bool((scales == 255).any()):
        raise PlaneError("MXFP4 scale byte 255 (NaN)")
    lut = torch.tensor(KVALUES_MXFP4, dtype=torch.int8, device=packed.device)
    p8 = packed.view(torch.uint8).to(torch.int64)
    codes = torch.stack([lut[p8 & 15], lut[p8 >> 4]], dim=-1).reshape(n, k)
    out = torch.zeros(n, resident_row_bytes("Q8_F32", k), dtype=torch.uint8, device=packed.device)
    out[:, :k] = codes.view(torch.uint8)
    out[:, k:k + k // 8] = e8m0_half(scales.view(torch.uint8)).contiguous().view(torch.uint8).reshape(n, k // 8)
    return out


def resident_k_slice(res: torch.Tensor, qtype: str, k: int, lo: int, hi: int) -> torch.Tensor:
    """Columns [lo, hi) of resident FP8_B128 / NVFP4 rows [N, row bytes] as resident rows of width ``hi - lo`` (what a
    rank that holds a slice of a matrix's input width loads): codes and scales of the span, the row's tensor scale kept."""
    from .resident import resident_row_bytes
    n = res.shape[0]
    if not 0 <= lo < hi <= k:
        raise PlaneError(f"columns {lo}..{hi} of {k}")
    w = hi - lo
    out = torch.zeros(n, resident_row_bytes(qtype, w), dtype=torch.uint8, device=res.device)
    if qtype == "FP8_B128":
        if lo % 128 or hi % 128:
            raise PlaneError(f"FP8_B128: a slice of columns {lo}..{hi} does not align to 128-value blocks")
        out[:, :w] = res[:, lo:hi]
        out[:, w:w + w // 32] = res[:, k + lo // 32:k + hi // 32]
        return out
    if qtype == "NVFP4":
        if lo % 16 or hi % 16:
            raise PlaneError(f"NVFP4: a slice of columns {lo}..{hi} does not align to 16-value groups")
        out[:, :w // 2] = res[:, lo // 2:hi // 2]
        out[:, w // 2:w // 2 + w // 16] = res[:, k // 2 + lo // 16:k // 2 + hi // 16]
        out[:, w // 2 + w // 16:w // 2 + w // 16 + 4] = res[:, k // 2 + k // 16:k // 2 + k // 16 + 4]
        return out
    raise PlaneError(f"{qtype} rows are not plane rows")


def detect_scheme(config: dict) -> str:
    """'fp8_b128', 'nvfp4_modelopt', 'nvfp4_ct', 'mxfp4_ct', 'mxfp8' or 'plain' from config.json's quantization block."""
    q = config.get("quantization_config") or config.get("quantization") or {}
    method = str(q.get("quant_method", "")).lower()
    if method == "fp8":
        bs = q.get("weight_block_size")
        if bs and list(bs) != [128, 128]:
            raise PlaneError(f"fp8 block size {bs} is not 128x128")
        return "fp8_b128"
    if method == "mxfp8":
        return "mxfp8"
    if method == "modelopt" or "nvfp4" in str(q.get("quant_algo", "")).lower():
        return "nvfp4_modelopt"
    if method == "compressed-tensors":
        fmt = str(q.get("format", "")).lower()
        if fmt == "mxfp4-pack-quantized":
            return "mxfp4_ct"
        if fmt != "nvfp4-pack-quantized":
            raise PlaneError(f"compressed-tensors format {q.get('format')!r} is not read")
        return "nvfp4_ct"
    if method:
        raise PlaneError(f"quantization method {method!r} is not read")
    return "plain"


def linear_resident(folder, stem: str, scheme: str) -> Tuple[torch.Tensor, str, int]:
    """(resident rows, type name, K) of the linear layer ``stem`` (no ``.weight`` suffix)."""
    if scheme == "fp8_b128" and f"{stem}.weight_scale_inv" in folder:
        codes = folder.tensor(f"{stem}.weight")
        return fp8_b128_resident(codes, folder.tensor(f"{stem}.weight_scale_inv")), "FP8_B128", codes.shape[1]
    if scheme == "nvfp4_modelopt" and f"{stem}.weight_scale" in folder:
        packed = folder.tensor(f"{stem}.weight")
        ts = folder.tensor(f"{stem}.weight_scale_2").float().reshape(-1)
        return nvfp4_resident(packed, folder.tensor(f"{stem}.weight_scale"), ts), "NVFP4", packed.shape[1] * 2
    if scheme == "nvfp4_modelopt" and f"{stem}.weight_scale_2" in folder:
        # the block scales are stored compressed (formats/csf.py): a base byte per row and 4-bit codes
        from . import csf
        enc = csf.encoding_of(folder, f"{stem}.weight_scale")
        if enc is None:
            raise PlaneError(f"{stem}: NVFP4 weight without block scales (plain, csf or csf_32x2_v1)")
        packed = folder.tensor(f"{stem}.weight")
        n, k = packed.shape[0], packed.shape[1] * 2
        try:
            scales = torch.from_numpy(csf.weight_scale(folder, f"{stem}.weight_scale", enc, n, k // 16))
        except csf.CsfError as exc:
            raise PlaneError(str(exc)) from None
        ts = folder.tensor(f"{stem}.weight_scale_2").float().reshape(-1)
        return nvfp4_resident(packed, scales, ts), "NVFP4", k
    if scheme == "mxfp4_ct" and f"{stem}.weight_packed" in folder:
        packed = folder.tensor(f"{stem}.weight_packed")
        return mxfp4_resident(packed, folder.tensor(f"{stem}.weight_scale")), "Q8_F32", packed.shape[1] * 2
    if scheme == "mxfp8" and f"{stem}.weight_scale" in folder:
        # value-preserving load as bf16 rows (twice the bytes of the file: no kernel here reads 32-wide E8M0 scales)
        w = mxfp8_dequantize(folder.tensor(f"{stem}.weight"), folder.tensor(f"{stem}.weight_scale"))
        return w.contiguous().view(torch.uint8).reshape(w.shape[0], -1), "BF16", w.shape[1]
    if scheme == "nvfp4_ct" and f"{stem}.weight_packed" in folder:
        packed = folder.tensor(f"{stem}.weight_packed")
        div = folder.tensor(f"{stem}.weight_global_scale").float().reshape(-1)
        if bool((div == 0).any()):
            raise PlaneError(f"{stem}: global scale divisor is zero")
        return nvfp4_resident(packed, folder.tensor(f"{stem}.weight_scale"), 1.0 / div), "NVFP4", packed.shape[1] * 2
    w = folder.tensor(f"{stem}.weight")
    tag = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32"}.get(w.dtype)
    if tag is None:
        raise PlaneError(f"{stem}.weight has dtype {w.dtype}, which no scheme here explains")
    w = w.reshape(1, -1) if w.dim() == 1 else w.reshape(-1, w.shape[-1])
    return w.contiguous().view(torch.uint8).reshape(w.shape[0], -1), tag, w.shape[1]
