"""numpy restatement of the reference quantise-and-bitpack path (test oracle).

Follows, in the reference project:
  obkv_accel/bitpack.py:13-47        quarter-split / half-split byte layouts
  obkv_accel/packing.py:141-165      asymmetric uniform quantisation
  obkv_accel/packing.py:177-391      K per-channel mixed packing (one head)
  obkv_accel/packing.py:399-578      K per-head packing to a shared-max layout
  obkv_accel/packing.py:715-778      V per-token segment packing
  obkv_accel/packing.py:801-1013     one head: evict, split fp16 tokens, pack
  obkv_accel/packing.py:1019-1317    pad + stack heads on the K stripe canvas
  obkv_fast.py:1098-1166             per-head select + pack driver

All arithmetic is IEEE fp32 with one rounding per operation (numpy does not
contract multiply-add), round-half-to-even, fp16 conversion round-to-nearest:
the same semantics the reference gets from PyTorch's CPU kernels.

A packed layer is a plain dict of numpy arrays whose keys and shapes mirror
the reference ``PackedKVLayer`` fields (leading batch dim of 1 kept).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
F16 = np.float16
U8 = np.uint8


# ── bit layouts (bitpack.py:13-47) ───────────────────────────────────────────

def bitpack2(codes: np.ndarray) -> np.ndarray:
    """[..., L] codes in 0..3 -> [..., L/4] bytes, quarter-split."""
    L = codes.shape[-1]
    assert L % 4 == 0
    s = L // 4
    c = codes.astype(U8)
    return (c[..., 0:s] | (c[..., s:2 * s] << 2) | (c[..., 2 * s:3 * s] << 4)
            | (c[..., 3 * s:] << 6)).astype(U8)


def bitpack4(codes: np.ndarray) -> np.ndarray:
    """[..., L] codes in 0..15 -> [..., L/2] bytes, half-split."""
    L = codes.shape[-1]
    assert L % 2 == 0
    s = L // 2
    c = codes.astype(U8)
    return (c[..., 0:s] | (c[..., s:] << 4)).astype(U8)


def bitunpack2(b: np.ndarray) -> np.ndarray:
    return np.concatenate([b & 3, (b >> 2) & 3, (b >> 4) & 3, (b >> 6) & 3], axis=-1).astype(U8)


def bitunpack4(b: np.ndarray) -> np.ndarray:
    return np.concatenate([b & 15, (b >> 4) & 15], axis=-1).astype(U8)


# ── quantisation (packing.py:141-165) ────────────────────────────────────────

def quantize(x: np.ndarray, n_bits: int, axis: int):
    """codes u8 (same shape as x), scale fp16, zero-point fp16 (keepdims on axis)."""
    xf = x.astype(F32)
    qmax = F32(2 ** n_bits - 1)
    if xf.shape[axis] == 0:
        raise ValueError("cannot quantise along an empty axis")
    lo = xf.min(axis=axis, keepdims=True)
    hi = xf.max(axis=axis, keepdims=True)
    scale = np.maximum((hi - lo) / qmax, F32(1e-8)).astype(F32)
    zp = np.rint(np.clip(F32(0) - lo / scale, F32(0), qmax)).astype(F32)
    q = np.rint(np.clip(xf / scale + zp, F32(0), qmax)).astype(F32)
    return q.astype(U8), scale.astype(F16), zp.astype(F16)


def _pad_to(n: int, align: int) -> int:
    return 0 if n == 0 else ((n + align - 1) // align) * align


def stable_order(bits: np.ndarray) -> np.ndarray:
    return np.argsort(bits, kind="stable")


# ── V: per-token segments (packing.py:715-778) ───────────────────────────────

def pack_v_segments(V: np.ndarray, v_bits: np.ndarray):
    """V [1,H,T,D] fp16, v_bits [T] in {2,4,8} -> dict of segments."""
    order = stable_order(v_bits)
    Vs = V[:, :, order, :]
    bs = v_bits[order]
    n2, n4, n8 = int((bs == 2).sum()), int((bs == 4).sum()), int((bs == 8).sum())
    assert n2 + n4 + n8 == V.shape[2]
    out = {"V_2bit": None, "V_4bit": None, "V_8bit": None}
    sc, zp = [], []
    if n2:
        c, s, z = quantize(Vs[:, :, :n2], 2, 3)
        out["V_2bit"] = bitpack2(c); sc.append(s); zp.append(z)
    if n4:
        c, s, z = quantize(Vs[:, :, n2:n2 + n4], 4, 3)
        out["V_4bit"] = bitpack4(c); sc.append(s); zp.append(z)
    if n8:
        c, s, z = quantize(Vs[:, :, n2 + n4:], 8, 3)
        out["V_8bit"] = c; sc.append(s); zp.append(z)
    out["V_scale"] = np.concatenate(sc, axis=2)
    out["V_zp"] = np.concatenate(zp, axis=2)
    out["sort_idx"] = order.astype(np.int64)
    out["seg_bounds"] = (n2, n4, n8)
    return out


# ── K: per-channel mixed packing, one bit-map for all heads (packing.py:177-391) ──

def pack_k_mixed(K: np.ndarray, k_bits: np.ndarray, sub_2_target=None, sub_4_target=None,
                 n_ch_8_target=None):
    """K [1,H,T,D] fp16, k_bits [D] in {0,2,4,8,16} -> dict."""
    H, T = K.shape[1], K.shape[2]
    kb = np.minimum(k_bits.astype(np.int64), 8)
    keep = np.nonzero(kb > 0)[0]
    order = stable_order(kb[keep])
    ch_sort_idx = keep[order].astype(np.int64)
    bs = kb[keep][order]
    n2, n4, n8 = int((bs == 2).sum()), int((bs == 4).sum()), int((bs == 8).sum())
    Ks = K[:, :, :, ch_sort_idx]
    n2p = 4 * int(sub_2_target) if sub_2_target is not None else _pad_to(n2, 4)
    n4p = 2 * int(sub_4_target) if sub_4_target is not None else _pad_to(n4, 2)
    n8o = int(n_ch_8_target) if n_ch_8_target is not None else n8
    assert n2p >= _pad_to(n2, 4) and n4p >= _pad_to(n4, 2) and n8o >= n8

    def seg(lo, n, n_pad):
        s = np.zeros((1, H, T, n_pad), dtype=F16)
        s[..., :n] = Ks[..., lo:lo + n]
        return s

    out = {"K_2bit": None, "K_4bit": None, "K_8bit": None}
    sc, zp, perm = [], [], []
    if n2p:
        c, s, z = quantize(seg(0, n2, n2p), 2, 2)
        out["K_2bit"] = bitpack2(c); sc.append(s); zp.append(z)
        perm += [ch_sort_idx[:n2], np.zeros(n2p - n2, np.int64)]
    if n4p:
        c, s, z = quantize(seg(n2, n4, n4p), 4, 2)
        out["K_4bit"] = bitpack4(c); sc.append(s); zp.append(z)
        perm += [ch_sort_idx[n2:n2 + n4], np.zeros(n4p - n4, np.int64)]
    if n8o:
        c, s, z = quantize(seg(n2 + n4, n8, n8o), 8, 2)
        out["K_8bit"] = c; sc.append(s); zp.append(z)
        perm += [ch_sort_idx[n2 + n4:], np.zeros(n8o - n8, np.int64)]
    if sc:
        out["K_ch_scale"] = np.concatenate(sc, axis=3)
        out["K_ch_zp"] = np.concatenate(zp, axis=3)
        out["K_ch_perm_padded_idx"] = np.concatenate(perm).astype(np.int64)
    else:
        out["K_ch_scale"] = np.zeros((1, H, 1, 0), F16)
        out["K_ch_zp"] = np.zeros((1, H, 1, 0), F16)
        out["K_ch_perm_padded_idx"] = np.zeros(0, np.int64)
    out["K_ch_sort_idx"] = ch_sort_idx
    out["K_ch_seg_bounds"] = (n2, n4, n8)
    return out


# ── K: one bit-map per head, shared-max channel layout (packing.py:399-578) ──

def pack_k_mixed_per_head(K: np.ndarray, k_bits_ph: np.ndarray):
    """K [1,H,T,D] fp16, k_bits_ph [H,D] -> dict with per-head index tables."""
    H = K.shape[1]
    kb = np.minimum(k_bits_ph.astype(np.int64), 8)
    n2h = [(kb[h] == 2).sum().item() for h in range(H)]
    n4h = [(kb[h] == 4).sum().item() for h in range(H)]
    n8h = [(kb[h] == 8).sum().item() for h in range(H)]
    m2, m4, m8 = max(n2h), max(n4h), max(n8h)
    sub2, sub4 = _pad_to(m2, 4) // 4, _pad_to(m4, 2) // 2
    heads = [pack_k_mixed(K[:, h:h + 1], k_bits_ph[h],
                          sub_2_target=sub2 if sub2 else None,
                          sub_4_target=sub4 if sub4 else None,
                          n_ch_8_target=m8 if m8 else None) for h in range(H)]

    def cat(key):
        parts = [hd[key] for hd in heads]
        return None if all(p is None for p in parts) else np.concatenate(parts, axis=1)

    d_pad = 4 * sub2 + 2 * sub4 + m8
    d_kept_max = max(a + b + c for a, b, c in zip(n2h, n4h, n8h))
    sort_ph = np.zeros((H, d_kept_max), np.int64)
    for h, hd in enumerate(heads):
        sort_ph[h, :hd["K_ch_sort_idx"].size] = hd["K_ch_sort_idx"]
    out = {
        "K_2bit": cat("K_2bit"), "K_4bit": cat("K_4bit"), "K_8bit": cat("K_8bit"),
        "K_ch_scale": (np.concatenate([hd["K_ch_scale"] for hd in heads], axis=1)
                       if d_pad else np.zeros((1, H, 1, 0), F16)),
        "K_ch_zp": (np.concatenate([hd["K_ch_zp"] for hd in heads], axis=1)
                    if d_pad else np.zeros((1, H, 1, 0), F16)),
        "K_ch_sort_idx_per_head": sort_ph,
        "K_ch_perm_padded_idx_per_head": (
            np.stack([hd["K_ch_perm_padded_idx"] for hd in heads]) if d_pad
            else np.zeros((H, 0), np.int64)),
        "K_ch_seg_bounds_per_head": np.array(list(zip(n2h, n4h, n8h)), np.int32).reshape(H, 3),
        "K_ch_seg_bounds": (m2, m4, m8),
    }
    return out


# ── one (sequence, layer): select, pack per head, stack on the stripe ────────

def pack_kv(K: np.ndarray, V: np.ndarray, v_bits: np.ndarray, k_bits: np.ndarray, gqa_factor: int):
    """Composite the reference runs per layer (obkv_fast.py:1098-1166 ->
    packing.py:801 with deferred K -> packing.py:1019).

    K, V [1,H,T,D] fp16; v_bits [H,T] in {0,2,4,8,16}; k_bits [H,D] in
    {0,2,4,8,16}.  Returns (layer dict, new_v_only or None).
    """
    H, T, D = K.shape[1], K.shape[2], K.shape[3]
    per = []
    for h in range(H):
        vb = v_bits[h]
        keep = np.nonzero(vb > 0)[0]
        vbk = vb[keep]
        comp = keep[vbk != 16]
        v16 = keep[vbk == 16]
        if comp.size:
            pv = pack_v_segments(V[:, h:h + 1][:, :, comp], vb[comp])
            k_comp = K[:, h:h + 1][:, :, comp][:, :, pv["sort_idx"]]
        else:
            pv = {"V_2bit": None, "V_4bit": None, "V_8bit": None,
                  "V_scale": np.zeros((1, 1, 0, 1), F16), "V_zp": np.zeros((1, 1, 0, 1), F16),
                  "sort_idx": np.zeros(0, np.int64), "seg_bounds": (0, 0, 0)}
            k_comp = np.zeros((1, 1, 0, D), F16)
        per.append({
            "pv": pv, "t_v": int(comp.size), "n16": int(v16.size),
            "k_rows": np.concatenate([k_comp, K[:, h:h + 1][:, :, v16]], axis=2),
            "v16": V[:, h:h + 1][:, :, v16] if v16.size else None,
        })
    max_tv = max(p["t_v"] for p in per)
    max_n16 = max(p["n16"] for p in per)
    T_k = max_tv + max_n16
    segs = [p["pv"]["seg_bounds"] for p in per]
    mx = tuple(max(s[i] for s in segs) for i in range(3))

    def stack_v(key, n_max, width, idx):
        if n_max == 0:
            return None
        out = np.zeros((1, H, n_max, width), U8)
        for h, p in enumerate(per):
            n = segs[h][idx]
            if n:
                out[0, h, :n] = p["pv"][key][0, 0]
        return out

    layer = {
        "V_2bit": stack_v("V_2bit", mx[0], D // 4, 0),
        "V_4bit": stack_v("V_4bit", mx[1], D // 2, 1),
        "V_8bit": stack_v("V_8bit", mx[2], D, 2),
    }
    v_scale = np.zeros((1, H, max_tv, 1), F16)
    v_zp = np.zeros((1, H, max_tv, 1), F16)
    canvas = np.zeros((1, H, T_k, D), F16)
    for h, p in enumerate(per):
        v_scale[0, h, :p["t_v"]] = p["pv"]["V_scale"][0, 0]
        v_zp[0, h, :p["t_v"]] = p["pv"]["V_zp"][0, 0]
        canvas[0, h, :p["t_v"]] = p["k_rows"][0, 0, :p["t_v"]]
        canvas[0, h, max_tv:max_tv + p["n16"]] = p["k_rows"][0, 0, p["t_v"]:]
    layer["V_scale"], layer["V_zp"] = v_scale, v_zp
    if T_k > 0:
        layer.update(pack_k_mixed_per_head(canvas, k_bits))
    else:
        layer.update({"K_2bit": None, "K_4bit": None, "K_8bit": None})
    if "K_ch_perm_padded_idx_per_head" in layer:
        layer["K_ch_perm_padded_idx_for_Q"] = np.repeat(
            layer["K_ch_perm_padded_idx_per_head"], gqa_factor, axis=0)
    mask = np.zeros((H, T_k), F32)
    for h, p in enumerate(per):
        mask[h, p["t_v"]:max_tv] = -np.inf
        mask[h, max_tv + p["n16"]:] = -np.inf
    layer["softmax_mask"] = np.repeat(mask, gqa_factor, axis=0)
    layer["seg_bounds"] = mx
    layer["seg_bounds_per_head"] = np.array(segs, np.int32).reshape(H, 3)
    layer["T_eff"] = max_tv
    layer["T_eff_k"] = T_k
    layer["n_v16"] = max_n16
    layer["T_eff_per_head"] = np.array([p["t_v"] for p in per], np.int32)
    layer["T_eff_k_per_head"] = np.array([p["t_v"] + p["n16"] for p in per], np.int32)
    layer["n_v16_per_head"] = np.array([p["n16"] for p in per], np.int32)
    new_v_only = None
    if max_n16:
        new_v_only = np.zeros((1, H, max_n16, D), F16)
        for h, p in enumerate(per):
            if p["n16"]:
                new_v_only[0, h, :p["n16"]] = p["v16"][0, 0]
    return layer, new_v_only


# ── dequantisation (packing.py:581-709, 1427-1444; trizone_decompress.py:91-146) ──

def unpack_k(layer: dict, D: int) -> np.ndarray:
    """Packed K stripe -> [1,H,T_k,D] fp16 in original channel order."""
    sc, zp = layer["K_ch_scale"].astype(F32), layer["K_ch_zp"].astype(F32)
    H = sc.shape[1]
    T_k = layer["T_eff_k"]
    m2, m4, m8 = layer["K_ch_seg_bounds"]
    p2, p4 = _pad_to(m2, 4), _pad_to(m4, 2)
    parts = []
    if layer["K_2bit"] is not None and p2:
        parts.append((bitunpack2(layer["K_2bit"]).astype(F32) - zp[..., :p2]) * sc[..., :p2])
    if layer["K_4bit"] is not None and p4:
        parts.append((bitunpack4(layer["K_4bit"]).astype(F32) - zp[..., p2:p2 + p4]) * sc[..., p2:p2 + p4])
    if layer["K_8bit"] is not None and m8:
        parts.append((layer["K_8bit"].astype(F32) - zp[..., p2 + p4:p2 + p4 + m8]) * sc[..., p2 + p4:p2 + p4 + m8])
    out = np.zeros((1, H, T_k, D), F16)
    if not parts:
        return out
    srt = np.concatenate(parts, axis=3).astype(F16)
    sb, si = layer["K_ch_seg_bounds_per_head"], layer["K_ch_sort_idx_per_head"]
    for h in range(H):
        n2, n4, n8 = (int(x) for x in sb[h])
        cols = np.concatenate([np.arange(n2), p2 + np.arange(n4), p2 + p4 + np.arange(n8)]).astype(np.int64)
        if cols.size:
            out[0, h][:, si[h, :cols.size]] = srt[0, h][:, cols]
    return out


def unpack_v(layer: dict, new_v_only, D: int) -> np.ndarray:
    """Zone A (dequantised) ++ Zone B (fp16) on the stripe -> [1,H,T_k,D] fp16."""
    H = layer["V_scale"].shape[1]
    max_tv, max_n16 = layer["T_eff"], layer["n_v16"]
    out = np.zeros((1, H, max_tv + max_n16, D), F16)
    sc, zp = layer["V_scale"].astype(F32), layer["V_zp"].astype(F32)
    for h in range(H):
        n2, n4, n8 = (int(x) for x in layer["seg_bounds_per_head"][h])
        off = 0
        for n, key, un in ((n2, "V_2bit", bitunpack2), (n4, "V_4bit", bitunpack4), (n8, "V_8bit", lambda b: b)):
            if n:
                codes = un(layer[key][0, h, :n]).astype(F32)
                out[0, h, off:off + n] = ((codes - zp[0, h, off:off + n]) * sc[0, h, off:off + n]).astype(F16)
                off += n
    if max_n16:
        out[0, :, max_tv:] = new_v_only[0]
    return out
