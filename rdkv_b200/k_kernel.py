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
from .packing import _pad_to, layer_view

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
    if Q.stride(1) != 1:
        Q = Q.contiguous()
    view, _keep = layer_view(packed_layer)
    check(lib().rdkv_k_scores(C.byref(view), ptr(Q), q_dtype_tag(Q), Q.stride(0), H_q, _num_kv_heads(packed_layer),
                              int(T_eff), ptr(out), out.stride(0), stream_ptr(Q.device)), "rdkv_k_scores")


def k_mixed_qk_dot(Q: torch.Tensor, packed_layer, T_eff: int) -> torch.Tensor:
    """Allocating form: returns ``[H_q, T_eff]`` fp32."""
    out = torch.empty((Q.shape[0], T_eff), dtype=torch.float32, device=Q.device)
    k_mixed_qk_dot_into(Q, packed_layer, T_eff, out)
    return out
