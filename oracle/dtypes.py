"""Bit-level dtype helpers for the oracle (test infrastructure, see oracle/__init__.py).

FP8 is the OCP e4m3 "fn" format used by the reference for compact KV
(`torch.float8_e4m3fn`: 1 sign, 4 exponent (bias 7), 3 mantissa bits, no infinities,
0x7f/0xff = NaN, max finite 448).  The reference's GPU store rounds to nearest even and
saturates out-of-range values to +-448, while its CPU cast turns them into NaN
(fastdms/layers/compact_attention.py:185-209 store into an fp8 pointer;
fastdms/engine/compact_kv.py:1085-1087 `.to(compact_dtype)`).  `encode_e4m3` takes the
saturating behaviour by default; both agree for |x| <= 448, which is the domain the parity
tests stay in.
"""
from __future__ import annotations

import numpy as np


def _build_e4m3_table() -> np.ndarray:
    tab = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if (b & 0x80) else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-6)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        tab[b] = v
    return tab


E4M3_TABLE = _build_e4m3_table()
_E4M3_POS = E4M3_TABLE[:127].astype(np.float64)  # 0 .. 448, strictly increasing, index == byte code


def decode_e4m3(raw: np.ndarray) -> np.ndarray:
    """uint8 bytes -> float32 values."""
    return E4M3_TABLE[np.asarray(raw, dtype=np.uint8)]


def encode_e4m3(x: np.ndarray, saturate: bool = True) -> np.ndarray:
    """float32 -> e4m3 bytes, round-to-nearest-even.  Out-of-range: +-448 (saturate) or NaN."""
    x = np.asarray(x, dtype=np.float32)
    ax = np.abs(x).astype(np.float64)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    # nearest representable magnitude; ties go to the even code (codes are consecutive integers,
    # so "even mantissa" == "even byte code").
    hi = np.searchsorted(_E4M3_POS, ax, side="left")  # first code with value >= ax
    hi = np.clip(hi, 0, 126)
    lo = np.clip(hi - 1, 0, 126)
    d_hi = np.abs(_E4M3_POS[hi] - ax)
    d_lo = np.abs(ax - _E4M3_POS[lo])
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & (lo % 2 == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    # overflow: anything that would round above 448 (the next binade step would be 480 -> tie at 464)
    over = ax > 464.0
    if saturate:
        code = np.where(over, np.uint8(126), code)
    else:
        code = np.where(over, np.uint8(127), code)
    code = np.where(np.isnan(x), np.uint8(127), code)
    return (code | sign).astype(np.uint8)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    b = np.asarray(bits).astype(np.uint16).astype(np.uint32) << 16
    return b.view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit pattern (uint16)."""
    u = np.ascontiguousarray(np.asarray(x, dtype=np.float32)).view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    r = ((u + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    return np.where(nan, np.uint16(0x7FC0), r)


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round float32 values to `dtype` and return them as float32 again."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "f32":
        return x
    if dtype == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits(x))
    if dtype == "f16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "e4m3":
        return decode_e4m3(encode_e4m3(x))
    raise ValueError(f"unknown dtype {dtype!r}")
