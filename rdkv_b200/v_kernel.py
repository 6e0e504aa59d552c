"""V side of decode attention: softmax weights times per-token quantised V.

Drop-in for the reference's ``v_dequant_weighted_sum_dispatch[_into]``
(obkv_accel/triton_v_kernel.py:1274-1313, 1729-1760).  Weight columns follow the
reference: a head's 2/4/8-bit rows use head-local column offsets, the fp16
"Zone B" rows start at column ``max_T_v``.  ``out`` is fully overwritten and the
summation order is fixed (the reference's default kernel uses atomics).
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, lib, ptr, require_cuda, stream_ptr
from .packing import layer_identity, layer_view

D = 128


def _num_kv_heads(packed_layer) -> int:
    sc = packed_layer.V_scale
    return sc.shape[1] if sc.dim() == 4 else sc.shape[0]


def v_dequant_weighted_sum_dispatch_into(attn_weights_old: torch.Tensor, packed_layer, out: torch.Tensor,
                                         V16=None, n_v16_per_head=None, max_T_v: int = 0) -> None:
    """out[h_q, :] = sum_t w[h_q, t] * dequant(V)[h_q // g, t, :] (+ fp16 Zone B rows)."""
    w = attn_weights_old
    require_cuda(w, "attn_weights_old")
    require_cuda(out, "out")
    if w.dtype != torch.float32 or out.dtype != torch.float32:
        raise ValueError("attn_weights_old and out must be float32")
    if w.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("attn_weights_old and out need unit column stride")
    H_q = w.shape[0]
    table = _weights_table(packed_layer, V16, n_v16_per_head, max_T_v, H_q)
    if table is not None and out.is_contiguous() and w.shape[1] >= table.max_t_k:
        # the weighted-sum half of the fused tensor-core kernel (one CTA per KV head, fixed order)
        check(lib().rdkv_decode_weighted_sum(ptr(table.views), 1, H_q, table.H_kv, table.unit_rows,
                                             table.k_row_bytes_max, ptr(w), w.stride(0), ptr(out), ptr(table.status),
                                             stream_ptr(w.device)), "rdkv_decode_weighted_sum")
        return
    view, _keep = layer_view(packed_layer, V16, n_v16_per_head,
                             max_T_v=int(max_T_v) if V16 is not None else None)
    check(lib().rdkv_v_weighted_sum(C.byref(view), ptr(w), w.stride(0), H_q, _num_kv_heads(packed_layer),
                                    ptr(out), out.stride(0), stream_ptr(w.device)), "rdkv_v_weighted_sum")


def v_dequant_weighted_sum_dispatch(attn_weights_old: torch.Tensor, packed_layer, V16=None,
                                    n_v16_per_head=None, max_T_v: int = 0) -> torch.Tensor:
    """Allocating form: returns ``[H_q, 128]`` fp32."""
    out = torch.empty((attn_weights_old.shape[0], D), dtype=torch.float32, device=attn_weights_old.device)
    v_dequant_weighted_sum_dispatch_into(attn_weights_old, packed_layer, out, V16=V16,
                                         n_v16_per_head=n_v16_per_head, max_T_v=max_T_v)
    return out


def _weights_table(packed_layer, V16, n_v16_per_head, max_T_v, H_q: int):
    """One-view table of the layer (+ its fp16 rows) for the fused kernel's weighted-sum mode,
    cached on the layer; None when the call is outside what that kernel takes."""
    from .decode import DecodeTable
    if n_v16_per_head is not None and n_v16_per_head is not getattr(packed_layer, "n_v16_per_head", None):
        return None                                        # caller-supplied counts: scalar kernel
    if V16 is not None and int(max_T_v) != int(packed_layer.T_eff):
        return None
    key = (H_q, None if V16 is None else (V16.data_ptr(), tuple(V16.shape), tuple(V16.stride())),
           layer_identity(packed_layer))
    cached = getattr(packed_layer, "_rdkv_v_table", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    table = None
    try:
        if H_q % _num_kv_heads(packed_layer) == 0 and (int(packed_layer.n_v16) == 0 or V16 is not None):
            nv = None if V16 is None else (V16 if V16.dim() == 4 else V16.unsqueeze(0))
            table = DecodeTable([packed_layer], [nv], H_q)
            if table.k_row_bytes_max > 224:
                table = None
    except (ValueError, AttributeError):
        table = None
    try:
        packed_layer._rdkv_v_table = (key, table)
    except AttributeError:
        pass
    return table
