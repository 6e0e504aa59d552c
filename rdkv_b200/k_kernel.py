"""K side of decode attention: q·K scores over pruned, per-channel quantised K.

Drop-in for the reference's ``k_mixed_qk_dot_into`` / ``k_mixed_qk_dot``
(obkv_accel/triton_k_kernel.py:1211-1427): same arguments, same output
convention (only ``out[:, :T_eff]`` is written), no allocation in the ``_into``
form, launch on the current stream.  ``out`` may be a column slice of a wider
buffer (any row stride, unit column stride, unaligned base).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from ._lib import check, lib, ptr, q_dtype_tag, require_cuda, stream_ptr
from .packing import _pad_to, layer_identity, layer_view

D = 128
SQRT_D = math.sqrt(float(D))
INV_SQRT_D = 1.0 / SQRT_D


def _num_kv_heads(packed_layer) -> int:
    sc = packed_layer.K_ch_scale
    return sc.shape[1] if sc.dim() == 4 else sc.shape[0]


def k_mixed_qk_dot_into(Q: torch.Tensor, packed_layer, T_eff: int, out: torch.Tensor, T_alloc=None) -> None:
    """scores[h_q, t] = q[h_q] · dequant(K)[h_q // g, t] / sqrt(128) for t < T_eff.

    Q [H_q,128] fp16/bf16/fp32; out [H_q, >=T_eff] fp32.  ``T_alloc`` is accepted
    for signature compatibility (row counts come from the tensors themselves).
    """
    require_cuda(Q, "Q")
    require_cuda(out, "out")
    H_q = Q.shape[0]
    assert Q.shape[1] == D, f"Q head_dim {Q.shape[1]} != {D}"
    if out.dtype != torch.float32 or out.stride(1) != 1:
        raise ValueError("out must be float32 with unit column stride")
    n2, n4, n8 = packed_layer.K_ch_seg_bounds
    if _pad_to(n2, 4) + _pad_to(n4, 2) + n8 == 0:
        out[:H_q, :T_eff].zero_()
        return
    if T_eff <= 0:
        return
    table = _scores_table(packed_layer, H_q)
    if table is not None and int(T_eff) <= table.max_t_k:
        # the score half of the fused tensor-core kernel; its one-view table is kept on the layer
        # object, as the reference keeps its pre-squeezed views on the cache object
        # (obkv_accel/fast_decode.py:813-816)
        if not Q.is_contiguous():
            Q = Q.contiguous()
        rows = 256
        check(lib().rdkv_decode_scores(ptr(table.views), 1, ptr(Q), q_dtype_tag(Q), H_q, table.H_kv, rows,
                                       -(-int(T_eff) // rows), table.k_row_bytes_max, int(T_eff), ptr(out),
                                       out.stride(0), ptr(table.status), stream_ptr(Q.device)), "rdkv_decode_scores")
        return
    if Q.stride(1) != 1:
        Q = Q.contiguous()
    view, _keep = layer_view(packed_layer)
    check(lib().rdkv_k_scores(C.byref(view), ptr(Q), q_dtype_tag(Q), Q.stride(0), H_q, _num_kv_heads(packed_layer),
                              int(T_eff), ptr(out), out.stride(0), stream_ptr(Q.device)), "rdkv_k_scores")


def _scores_table(packed_layer, H_q: int):
    """One-view table of the layer for the fused kernel's score mode, cached on the layer; None
    when the layer's shape is outside what that kernel takes (the scalar kernel then runs)."""
    from .decode import DecodeTable
    key = (H_q, layer_identity(packed_layer))
    cached = getattr(packed_layer, "_rdkv_k_table", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    table = None
    try:
        if H_q % _num_kv_heads(packed_layer) == 0:
            table = DecodeTable([packed_layer], [None], H_q, k_only=True)
            if table.k_row_bytes_max > 224:
                table = None
    except (ValueError, AttributeError):
        table = None
    try:
        packed_layer._rdkv_k_table = (key, table)
    except AttributeError:
        pass
    return table


def k_mixed_qk_dot(Q: torch.Tensor, packed_layer, T_eff: int) -> torch.Tensor:
    """Allocating form: returns ``[H_q, T_eff]`` fp32."""
    out = torch.empty((Q.shape[0], T_eff), dtype=torch.float32, device=Q.device)
    k_mixed_qk_dot_into(Q, packed_layer, T_eff, out)
    return out
