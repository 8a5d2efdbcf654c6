"""Code books of the non-linear GGUF block types (data of the file format, ggml-common.h).

* ``KVALUES_IQ4NL``: the 16 code values of IQ4_NL / IQ4_XS.
* ``KVALUES_MXFP4``: the E2M1 code values of MXFP4, doubled (the halved block scale puts the factor back).
* IQ2_XXS grid: 256 entries of eight magnitudes, each one of 8 / 25 / 43.  Stored here as base-3 numbers (digit j =
  level of magnitude j, least significant first) and expanded on first use.
* sign patterns of IQ2_XXS: a 7-bit index gives seven sign bits, the eighth makes the number of minus signs even.

The reference keeps the same tables in ``crates/gguf/src/iq_tables.rs``.
"""
from __future__ import annotations

import functools

import torch

KVALUES_IQ4NL = (-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113)
KVALUES_MXFP4 = (0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12)
IQ2XXS_LEVELS = (8, 25, 43)

_IQ2XXS_BASE3 = (
    0, 2, 4, 6, 8, 10, 12, 18, 20, 24, 26, 28, 30, 36, 42, 46,
    48, 54, 56, 62, 74, 82, 84, 90, 94, 108, 138, 150, 162, 164, 182, 218,
    244, 246, 252, 262, 264, 270, 272, 276, 288, 298, 300, 306, 318, 324, 326, 330,
    342, 356, 376, 378, 388, 412, 414, 432, 462, 480, 486, 490, 492, 498, 510, 514,
    516, 522, 524, 546, 570, 594, 650, 660, 730, 732, 738, 748, 756, 774, 786, 792,
    796, 810, 816, 828, 846, 854, 864, 912, 922, 972, 978, 990, 994, 1006, 1026, 1068,
    1100, 1134, 1148, 1216, 1218, 1224, 1242, 1270, 1296, 1300, 1368, 1414, 1458, 1460, 1466, 1488,
    1504, 1512, 1514, 1564, 1572, 1620, 1622, 1702, 1704, 1710, 1728, 1742, 1782, 1810, 1830, 1926,
    1950, 1962, 2010, 2136, 2188, 2190, 2196, 2202, 2206, 2208, 2214, 2220, 2228, 2232, 2242, 2244,
    2250, 2268, 2286, 2314, 2322, 2326, 2350, 2358, 2382, 2390, 2400, 2430, 2436, 2448, 2484, 2500,
    2522, 2532, 2592, 2674, 2676, 2682, 2700, 2704, 2754, 2796, 2800, 2810, 2866, 2898, 2916, 2922,
    2926, 2932, 2934, 2970, 2976, 3000, 3026, 3072, 3142, 3222, 3224, 3248, 3322, 3360, 3402, 3412,
    3418, 3450, 3510, 3570, 3648, 3654, 3672, 3696, 3726, 3766, 3822, 3852, 3888, 3892, 3978, 3980,
    4026, 4160, 4374, 4376, 4382, 4402, 4430, 4458, 4470, 4482, 4546, 4618, 4620, 4626, 4630, 4644,
    4662, 4698, 4730, 4764, 4786, 4806, 4824, 4862, 4944, 5032, 5106, 5112, 5124, 5130, 5176, 5198,
    5238, 5296, 5346, 5366, 5376, 5464, 5644, 5688, 5834, 5868, 5890, 5920, 5994, 6090, 6354, 6402,
)


@functools.lru_cache(maxsize=None)
def iq2xxs_grid() -> torch.Tensor:
    """uint8 [256, 8]: the eight magnitudes of every grid entry."""
    g = torch.empty(256, 8, dtype=torch.uint8)
    for i, c in enumerate(_IQ2XXS_BASE3):
        for j in range(8):
            g[i, j] = IQ2XXS_LEVELS[c % 3]
            c //= 3
    return g


@functools.lru_cache(maxsize=None)
def iq2_signs() -> torch.Tensor:
    """float [128, 8] of +1 / -1: bit j of the 7-bit index flips value j; the eighth sign keeps the parity even."""
    s = torch.ones(128, 8)
    for i in range(128):
        full = i | ((bin(i).count("1") & 1) << 7)
        for j in range(8):
            if full >> j & 1:
                s[i, j] = -1.0
    return s


def e8m0_half(e: torch.Tensor) -> torch.Tensor:
    """uint8 exponent bytes -> f32 of half the E8M0 scale, 2^(E - 128); E = 0 and 1 are the two subnormals."""
    e = e.to(torch.int32)
    bits = torch.where(e >= 2, (e - 1) << 23, torch.where(e == 1, torch.full_like(e, 0x00400000), torch.full_like(e, 0x00200000)))
    return bits.view(torch.float32)
