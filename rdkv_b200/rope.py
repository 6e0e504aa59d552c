"""Rotary position embedding of a decode step's query and key rows.

Drop-in for the reference's ``fused_rope`` (obkv_accel/triton_rope.py:111-138): same name,
arguments and in-place behaviour.  Inside a decode step the rotation is part of the attention
launch (:func:`rdkv_b200.decode.packed_decode_attention` with ``rope=``); this call is for
callers that keep the two steps apart.
"""
from __future__ import annotations

from torch import Tensor

from ._lib import HEAD_DIM, check, lib, ptr, q_dtype_tag, require_cuda, stream_ptr


def fused_rope(q: Tensor, k: Tensor, cos_half: Tensor, sin_half: Tensor):
    """Rotate q [H_q,128] and k [H_kv,128] (fp16 / bf16 / fp32) in place, half format:
    (x[i], x[i+64]) -> (x[i]·cos[i] − x[i+64]·sin[i], x[i+64]·cos[i] + x[i]·sin[i]) with fp32
    arithmetic; cos_half / sin_half [64].  Returns (q, k).  One launch."""
    for name, t in (("q", q), ("k", k), ("cos_half", cos_half), ("sin_half", sin_half)):
        require_cuda(t, name)
    if q.dim() != 2 or k.dim() != 2 or q.shape[1] != HEAD_DIM or k.shape[1] != HEAD_DIM:
        raise ValueError(f"q and k must be [heads,{HEAD_DIM}], got {tuple(q.shape)} and {tuple(k.shape)}")
    if cos_half.shape[0] != HEAD_DIM // 2 or sin_half.shape[0] != HEAD_DIM // 2 or cos_half.dtype != sin_half.dtype:
        raise ValueError(f"cos_half and sin_half must hold {HEAD_DIM // 2} values of one dtype")
    if q.stride(1) != 1 or k.stride(1) != 1:
        raise ValueError("q and k rows must be contiguous")
    cos_half, sin_half = cos_half.contiguous(), sin_half.contiguous()
    check(lib().rdkv_rope(ptr(q), q_dtype_tag(q), q.shape[0], q.stride(0), ptr(k), q_dtype_tag(k), k.shape[0],
                          k.stride(0), ptr(cos_half), ptr(sin_half), q_dtype_tag(cos_half), stream_ptr(q.device)),
          "rdkv_rope")
    return q, k
