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


def row_window_mask(layer: dict, lo: int, hi: int, g: int) -> np.ndarray:
    """Additive mask [H_q, T_k] that keeps, per head, the live rows lo <= i < hi of its own row
    order (its 2-, 4-, 8-bit rows, then its fp16 rows) and removes every other stripe column:
    the share of one rank when a head's rows are split across ranks (no reference counterpart;
    the reference attends over all rows on one device)."""
    T_k, max_t_v = int(layer["T_eff_k"]), int(layer["T_eff"])
    t_v = np.asarray(layer["T_eff_per_head"]).astype(np.int64)[:, None]
    col = np.arange(T_k)[None]
    live_idx = np.where(col < max_t_v, col, t_v + (col - max_t_v))
    keep = (live_idx >= lo) & (live_idx < hi)
    return np.repeat(np.where(keep, F32(0), F32(-np.inf)), g, axis=0)


def part_mask(layer: dict, part: int, parts: int, g: int) -> np.ndarray:
    """Additive mask [H_q, T_k] that keeps, per head, part `part` of `parts` of each of its phases
    (its 2-bit rows, its 4-bit rows, its 8-bit rows, its fp16 rows; cut points rounded down to
    multiples of 32 rows, the last part takes the rest): one rank's share when the ranks that
    share a head split its rows (no reference counterpart)."""
    T_k, max_t_v = int(layer["T_eff_k"]), int(layer["T_eff"])
    sb = np.asarray(layer["seg_bounds_per_head"]).astype(np.int64)
    n16 = np.asarray(layer["n_v16_per_head"]).astype(np.int64)
    H = sb.shape[0]
    keep = np.zeros((H, T_k), bool)
    cut = lambda n, i: n if i >= parts else (n * i // parts) & ~31
    for h in range(H):
        t_v = int(sb[h].sum())
        base = 0
        for p, n in enumerate([int(sb[h, 0]), int(sb[h, 1]), int(sb[h, 2]), int(n16[h])]):
            lo, hi = base + cut(n, part), base + cut(n, part + 1)
            if p < 3:
                keep[h, lo:hi] = True
            else:
                keep[h, max_t_v + (lo - t_v):max_t_v + (hi - t_v)] = True
            base += n
    return np.repeat(np.where(keep, F32(0), F32(-np.inf)), g, axis=0)


def decode_attention(q: np.ndarray, layer: dict, new_v_only, new_k=None, new_v=None, D: int = 128, rows=None,
                     seq_part=None):
    """softmax(q.K^T/sqrt(D) + mask).V^ over the stripe plus an optional fp tail.

    q [H_q,D]; new_k/new_v [H,n_new,D] (Zone C, decode-appended tokens, unmasked);
    rows = (lo, hi): only that window of every head's live rows (see row_window_mask);
    seq_part = (i, n): only part i of n of every head's rows (see part_mask).
    Returns out [H_q,D] fp32, and the row statistics (m [H_q], l [H_q]).
    """
    qf = q.astype(F32)
    K = unpack_k(layer, D)[0].astype(F32)
    V = unpack_v(layer, new_v_only, D)[0].astype(F32)
    H = K.shape[0]
    g = qf.shape[0] // H
    inv = F32(1.0) / F32(np.sqrt(F32(D)))
    s = np.einsum("hd,htd->ht", qf, np.repeat(K, g, axis=0)) * inv + layer["softmax_mask"]
    if rows is not None:
        s = s + row_window_mask(layer, int(rows[0]), int(rows[1]), g)
    if seq_part is not None:
        s = s + part_mask(layer, int(seq_part[0]), int(seq_part[1]), g)
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
