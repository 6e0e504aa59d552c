"""numpy restatement of the reference dequantise-then-attend decode path (test oracle).

Follows, in the reference project:
  obkv_accel/trizone_decompress.py:185-333   packed cache -> fp16 (K, V) + per-head masks
  obkv_accel/triton_k_kernel.py:1433-1456    k_mixed_qk_dot_ref (scores = q.K^/sqrt(D))
  obkv_accel/triton_v_kernel.py:1858-1882    v_dequant_weighted_sum_ref
  obkv_accel/fast_decode.py:1701-1784        one softmax over Zone A | Zone B | Zone C

The dequantised K^ and V^ are rounded to fp16 exactly as the reference does
before the fp32 attention arithmetic.
"""
from __future__ import annotations

import numpy as np

from .ref_packing import unpack_k, unpack_v

F32 = np.float32


def k_scores(q: np.ndarray, layer: dict, T_eff: int, D: int = 128) -> np.ndarray:
    """q [H_q,D] -> scores [H_q,T_eff] fp32 (no mask), triton_k_kernel.py:1433."""
    K = unpack_k(layer, D)[0].astype(F32)            # [H,T_k,D]
    g = q.shape[0] // K.shape[0]
    Kx = np.repeat(K, g, axis=0)[:, :T_eff]
    return (np.einsum("hd,htd->ht", q.astype(F32), Kx) / F32(np.sqrt(F32(D)))).astype(F32)


def v_weighted_sum(w: np.ndarray, layer: dict, new_v_only, D: int = 128) -> np.ndarray:
    """w [H_q,T_k] fp32 stripe weights -> out [H_q,D] fp32 (Zone A + Zone B)."""
    V = unpack_v(layer, new_v_only, D)[0].astype(F32)  # [H,T_k,D]
    g = w.shape[0] // V.shape[0]
    valid = np.isfinite(layer["softmax_mask"])       # pad columns carry no value
    ww = np.where(valid, w[:, :V.shape[1]], F32(0))
    return np.einsum("ht,htd->hd", ww, np.repeat(V, g, axis=0)).astype(F32)


def decode_attention(q: np.ndarray, layer: dict, new_v_only, new_k=None, new_v=None, D: int = 128):
    """softmax(q.K^T/sqrt(D) + mask).V^ over the stripe plus an optional fp tail.

    q [H_q,D]; new_k/new_v [H,n_new,D] (Zone C, decode-appended tokens, unmasked).
    Returns out [H_q,D] fp32, and the row statistics (m [H_q], l [H_q]).
    """
    qf = q.astype(F32)
    K = unpack_k(layer, D)[0].astype(F32)
    V = unpack_v(layer, new_v_only, D)[0].astype(F32)
    H = K.shape[0]
    g = qf.shape[0] // H
    inv = F32(1.0) / F32(np.sqrt(F32(D)))
    s = np.einsum("hd,htd->ht", qf, np.repeat(K, g, axis=0)) * inv + layer["softmax_mask"]
    Vx = np.repeat(V, g, axis=0)
    if new_k is not None and new_k.shape[1] > 0:
        s_new = np.einsum("hd,htd->ht", qf * inv, np.repeat(new_k.astype(F32), g, axis=0))
        s = np.concatenate([s, s_new], axis=1)
        Vx = np.concatenate([Vx, np.repeat(new_v.astype(F32), g, axis=0)], axis=1)
    m = s.max(axis=1)
    safe_m = np.where(np.isfinite(m), m, F32(0))
    p = np.exp(s - safe_m[:, None]).astype(F32)
    l = p.sum(axis=1)
    out = np.einsum("ht,htd->hd", p, Vx) / np.maximum(l, F32(1e-30))[:, None]
    return out.astype(F32), m.astype(F32), l.astype(F32)


def lse_combine(m: np.ndarray, l: np.ndarray, o: np.ndarray):
    """Merge split-sequence partials.  m,l [S,R]; o [S,R,D] un-normalised.

    out = sum_i o_i e^{m_i-M} / sum_i l_i e^{m_i-M}, M = max_i m_i.
    """
    M = m.max(axis=0)
    safe = np.where(np.isfinite(M), M, F32(0))
    w = np.where(np.isfinite(m), np.exp(m - safe[None]), F32(0)).astype(F32)
    L = (l * w).sum(axis=0)
    O = (o * w[..., None]).sum(axis=0)
    return (O / np.maximum(L, F32(1e-30))[:, None]).astype(F32), M.astype(F32), L.astype(F32)
