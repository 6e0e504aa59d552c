"""numpy restatement of the reference's rotary embedding for decode (test oracle).

Follows obkv_accel/triton_rope.py:141-165 (fused_rope_ref): half format — channel i pairs with
channel i + 64 — in fp32 with every product and sum rounded on its own, the result rounded to the
rows' own type.  bf16 rows travel as their 16-bit patterns (numpy has no bf16).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(F32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, as torch's .to(bfloat16) does; returns the 16-bit patterns."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1)))
    out = (rounded >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def to_f32(x: np.ndarray, dtype: str) -> np.ndarray:
    return bf16_to_f32(x) if dtype == "bf16" else x.astype(F32)


def from_f32(x: np.ndarray, dtype: str) -> np.ndarray:
    return f32_to_bf16(x) if dtype == "bf16" else x.astype(np.float16 if dtype == "f16" else F32)


def rope_rows(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, dtype: str) -> np.ndarray:
    """x [...,128] of `dtype` ("f16", "bf16" as bit patterns, "f32"), cos / sin [...,64] fp32 ->
    rotated rows in the same representation."""
    xf = to_f32(x, dtype)
    lo, hi = xf[..., :64], xf[..., 64:]
    c, s = cos.astype(F32), sin.astype(F32)
    out_lo = ((lo * c).astype(F32) - (hi * s).astype(F32)).astype(F32)
    out_hi = ((hi * c).astype(F32) + (lo * s).astype(F32)).astype(F32)
    return from_f32(np.concatenate([out_lo, out_hi], axis=-1), dtype)


def fused_rope(q: np.ndarray, k: np.ndarray, cos_half: np.ndarray, sin_half: np.ndarray, dtype: str, cs_dtype: str):
    """(q_out, k_out) of fused_rope_ref for rows of `dtype` and tables of `cs_dtype`."""
    c, s = to_f32(cos_half, cs_dtype), to_f32(sin_half, cs_dtype)
    return rope_rows(q, c, s, dtype), rope_rows(k, c, s, dtype)
