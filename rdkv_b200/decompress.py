"""Packed cache -> fp16 (K, V): drop-ins for the reference's decompressor.

Mirrors ``unpack_k_mixed`` (obkv_accel/packing.py:581-709), ``unpack_v_segment``
(:1427-1444) and ``unpack_trizone_to_past_kv`` with its helpers
(obkv_accel/trizone_decompress.py:43-333): same names, arguments and results, computed
by one CUDA launch per layer (``rdkv_unpack_layer``).  Tensors must be on a CUDA device.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch
from torch import Tensor

from ._lib import LayerView, check, lib, ptr, require_cuda, stream_ptr
from .packing import PackedKVLayer, TriZoneCache, _squeeze_h, layer_view


def _is_perhead_layout(pl: PackedKVLayer) -> bool:
    """True when ``pl`` came out of ``_pad_and_stack_per_head_layers`` (trizone_decompress.py:86-88)."""
    return pl.seg_bounds_per_head is not None


def _launch(view: LayerView, H_kv: int, D: int, rows: int, device, *, want_k: bool, want_v: bool,
            sort_idx: Optional[Tensor] = None, sort_stride: int = 0, ch_counts: Optional[Tensor] = None,
            n_ch=(0, 0, 0)) -> Tuple[Optional[Tensor], Optional[Tensor]]:
    k_out = torch.empty((1, H_kv, rows, D), dtype=torch.float16, device=device) if want_k else None
    v_out = torch.empty((1, H_kv, rows, D), dtype=torch.float16, device=device) if want_v else None
    if rows > 0:
        check(lib().rdkv_unpack_layer(C.byref(view), H_kv, D, ptr(sort_idx), sort_stride, ptr(ch_counts),
                                      int(n_ch[0]), int(n_ch[1]), int(n_ch[2]), ptr(k_out), ptr(v_out),
                                      rows * D, rows, stream_ptr(device)), "rdkv_unpack_layer")
    return k_out, v_out


def _k_channel_maps(pl: PackedKVLayer):
    """(sort_idx int64, head stride, per-head counts int32 or None, shared counts)."""
    n_ch = tuple(int(x) for x in pl.K_ch_seg_bounds)
    if pl.K_ch_seg_bounds_per_head is not None:
        assert pl.K_ch_sort_idx_per_head is not None, "per-head layout requires K_ch_sort_idx_per_head"
        si = pl.K_ch_sort_idx_per_head.to(torch.int64).contiguous()
        cnt = pl.K_ch_seg_bounds_per_head.to(torch.int32).contiguous()
        return si, si.stride(0), cnt, n_ch
    si = pl.K_ch_sort_idx
    if si is None or si.numel() == 0:
        return None, 0, None, n_ch
    return si.to(torch.int64).contiguous(), 0, None, n_ch


def unpack_k_mixed(packed: PackedKVLayer, D: int) -> Tensor:
    """Reverse of pack_k_mixed / pack_k_mixed_per_head: ``[1, H_kv, T_eff, D]`` fp16 with the kept
    channels scattered back to their original positions and zeros elsewhere (packing.py:581-709)."""
    if packed.K_ch_scale is None:
        raise ValueError("unpack_k_mixed: K_ch_scale missing")
    require_cuda(packed.K_ch_scale, "K_ch_scale")
    H_kv = _squeeze_h(packed.K_ch_scale).shape[0]
    T_eff = int(packed.T_eff_k) if packed.T_eff_k > 0 else int(packed.T_eff)
    device = packed.K_ch_scale.device
    si, stride, cnt, n_ch = _k_channel_maps(packed)
    if si is None or sum(n_ch) == 0:
        return torch.zeros(1, H_kv, T_eff, D, dtype=torch.float16, device=device)
    view, keep = layer_view(packed, t_k=T_eff)
    k, _ = _launch(view, H_kv, D, T_eff, device, want_k=True, want_v=False, sort_idx=si, sort_stride=stride,
                   ch_counts=cnt, n_ch=n_ch)
    del keep
    return k


def unpack_v_segment(V_packed: Tensor, V_scale: Tensor, V_zp: Tensor, n_bits: int) -> Tensor:
    """Reverse of one V segment: unpack + dequantise -> fp16 ``[..., N, D]`` (packing.py:1427-1444)."""
    if n_bits not in (2, 4, 8):
        raise ValueError(f"Unsupported n_bits={n_bits}")
    require_cuda(V_packed, "V_packed")
    lead = V_packed.shape[:-2]
    n, width = int(V_packed.shape[-2]), int(V_packed.shape[-1])
    D = width * (8 // n_bits)
    heads = 1
    for x in lead:
        heads *= int(x)
    codes = V_packed.reshape(heads, n, width).contiguous()
    sc = V_scale.reshape(heads, n).to(torch.float16).contiguous()
    zp = V_zp.reshape(heads, n).to(torch.float16).contiguous()
    out = torch.empty((heads, n, D), dtype=torch.float16, device=V_packed.device)
    if heads == 0 or n == 0:
        return out.reshape(*lead, n, D)
    v = LayerView()
    name = {2: "v2", 4: "v4", 8: "v8"}[n_bits]
    setattr(v, name, codes.data_ptr())
    setattr(v, name + "_head_stride", codes.stride(0))
    setattr(v, name + "_bytes", codes.numel())
    v.v_scale, v.v_zp, v.v_meta_head_stride, v.v_meta_bytes = sc.data_ptr(), zp.data_ptr(), sc.stride(0), sc.numel() * 2
    v.n2, v.n4, v.n8 = (n if n_bits == 2 else 0), (n if n_bits == 4 else 0), (n if n_bits == 8 else 0)
    v.max_t_v, v.t_k = n, n
    check(lib().rdkv_unpack_layer(C.byref(v), heads, D, None, 0, None, 0, 0, 0, None, ptr(out), n * D, n,
                                  stream_ptr(out.device)), "rdkv_unpack_layer")
    return out.reshape(*lead, n, D)


def _v_stripe(pl: PackedKVLayer, V16: Optional[Tensor], head_dim: int, rows: int, *, with_zone_b: bool) -> Tensor:
    H_kv = _squeeze_h(pl.V_scale).shape[0]
    device = pl.V_scale.device
    view, keep = layer_view(pl, V16 if with_zone_b else None, t_k=rows)
    _, v = _launch(view, H_kv, head_dim, rows, device, want_k=False, want_v=True)
    del keep
    return v


def _unpack_v_zone_a(pl: PackedKVLayer) -> Tensor:
    """Shared layout: the 2/4/8-bit V segments dequantised and concatenated along T, in ``sort_idx``
    order: ``[1, H_kv, T_v, D]`` fp16 (trizone_decompress.py:43-83)."""
    N_2, N_4, N_8 = (int(x) for x in pl.seg_bounds)
    T_v = int(pl.T_eff)
    assert N_2 + N_4 + N_8 == T_v, f"V seg_bounds {(N_2, N_4, N_8)} must sum to T_v={T_v}"
    H_kv = pl.V_scale.shape[1]
    if T_v == 0:
        return torch.empty(1, H_kv, 0, 1, dtype=torch.float16, device=pl.V_scale.device)
    for t, n_bits in ((pl.V_2bit, 2), (pl.V_4bit, 4), (pl.V_8bit, 8)):
        if t is not None and t.numel() > 0:
            D = int(t.shape[-1]) * (8 // n_bits)
            break
    else:
        return torch.empty(1, H_kv, 0, 1, dtype=torch.float16, device=pl.V_scale.device)
    return _v_stripe(pl, None, D, T_v, with_zone_b=False)


def _unpack_v_perhead(pl: PackedKVLayer, *, head_dim: int) -> Tensor:
    """Per-head layout: ``[1, H_kv, max_T_v, head_dim]`` fp16, head h's rows ``[0, T_v_h)`` dequantised
    and the rest zeros (trizone_decompress.py:91-144)."""
    return _v_stripe(pl, None, head_dim, int(pl.T_eff), with_zone_b=False)


def unpack_trizone_to_past_kv(dual_cache: TriZoneCache, *, head_dim: int, device: Optional[torch.device] = None,
                              dtype: torch.dtype = torch.float16, return_masks: bool = False,
                              H_q: Optional[int] = None, max_new_tokens: int = 0,
                              mask_dtype: torch.dtype = torch.float16):
    """Reverse a ``TriZoneCache`` into HF legacy ``past_key_values``: a tuple of ``(K_i, V_i)``, each
    ``[1, H_kv, T_eff_k_i, head_dim]``; with ``return_masks`` also the per-layer ``[1, H_q, 1,
    T_eff_k_i + max_new_tokens]`` additive masks of the per-head layout (``None`` for shared-layout
    layers).  Same contract as trizone_decompress.py:185-333."""
    past_kv: List[Tuple[Tensor, Tensor]] = []
    masks_list: List[Optional[Tensor]] = []
    for i, pl in enumerate(dual_cache.packed):
        K_full = unpack_k_mixed(pl, D=head_dim)
        V16 = dual_cache.new_v_only[i] if i < len(dual_cache.new_v_only) else None
        per_head = _is_perhead_layout(pl)
        if per_head:
            rows = int(pl.T_eff) + int(pl.n_v16)
            V_full = _v_stripe(pl, V16, head_dim, rows, with_zone_b=True)
        else:
            n16 = int(V16.shape[2]) if V16 is not None and V16.numel() > 0 else 0
            rows = int(pl.T_eff) + n16
            if rows == 0:
                V_full = torch.empty(1, K_full.shape[1], 0, head_dim, dtype=torch.float16, device=K_full.device)
            else:
                V_full = _v_stripe(pl, V16, head_dim, rows, with_zone_b=True)
        assert K_full.shape[2] == V_full.shape[2], (
            f"layer {i}: K T-dim {K_full.shape[2]} != V T-dim {V_full.shape[2]} "
            f"(T_v={pl.T_eff}, n_v16={pl.n_v16}, T_eff_k={pl.T_eff_k})")
        assert K_full.shape[3] == head_dim and V_full.shape[3] == head_dim
        if device is not None:
            K_full, V_full = K_full.to(device), V_full.to(device)
        past_kv.append((K_full.to(dtype).contiguous(), V_full.to(dtype).contiguous()))
        if return_masks:
            if per_head and pl.softmax_mask is not None:
                mask_2d = pl.softmax_mask
                mask_H_q = int(mask_2d.shape[0])
                if H_q is not None:
                    assert H_q == mask_H_q, f"layer {i}: caller H_q={H_q} != softmax_mask H_q={mask_H_q}"
                target = device if device is not None else mask_2d.device
                mask_4d = mask_2d.to(device=target, dtype=mask_dtype).view(1, mask_H_q, 1, int(mask_2d.shape[1]))
                if max_new_tokens > 0:
                    pad = torch.zeros(1, mask_H_q, 1, max_new_tokens, dtype=mask_dtype, device=target)
                    mask_4d = torch.cat([mask_4d, pad], dim=-1)
                masks_list.append(mask_4d.contiguous())
            else:
                masks_list.append(None)
    if return_masks:
        return tuple(past_kv), masks_list
    return tuple(past_kv)
