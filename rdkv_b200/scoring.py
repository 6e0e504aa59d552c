"""Importance scores that feed the bit allocator.

Drop-ins for the reference's ``_score_one_layer`` (obkv_fast.py:854-896) and
``apply_score_pooling`` (obkv_fast.py:208-246): same names, arguments and return shapes.
"""
from __future__ import annotations

import torch
from torch import Tensor

from ._lib import check, lib, ptr, q_dtype_tag, require_cuda, stream_ptr


def _score_one_layer(aw: Tensor, q: Tensor, o, v: Tensor, head_dim: int, v_score_type: str = "attn_linear",
                     k: Tensor = None, k_score_type: str = "think"):
    """aw [B,H_kv,g,W,T], q [B,H_kv,g,W,D], v / k [B,H_kv,T,D] ->
    (layer_token [B,H_kv,T] = sum_{g,w} aw, layer_channel [B,H_kv,D] = mean(q^2) * mean_t(k^2)), fp32.
    ``o`` and ``v`` are accepted for signature compatibility (unused, as in the reference)."""
    if v_score_type != "attn_linear":
        raise ValueError(f"Unsupported v_score_type={v_score_type!r}; expected 'attn_linear'.")
    if k_score_type != "think":
        raise ValueError(f"Unsupported k_score_type={k_score_type!r}; expected 'think'.")
    if k is None:
        raise ValueError("k_score_type='think' requires the keys tensor (k=...).")
    require_cuda(aw, "aw"); require_cuda(q, "q"); require_cuda(k, "k")
    B, H, g, W, T = aw.shape
    D = int(q.shape[-1])
    if tuple(q.shape) != (B, H, g, W, D) or tuple(k.shape) != (B, H, T, D) or D != int(head_dim):
        raise ValueError("q must be [B,H_kv,g,W,D] and k [B,H_kv,T,D]")
    aw, q = aw.contiguous(), q.contiguous()
    if k.stride(3) != 1 or k.stride(0) != H * k.stride(1):
        k = k.contiguous()
    dev = aw.device
    token = torch.empty((B, H, T), dtype=torch.float32, device=dev)
    channel = torch.empty((B, H, D), dtype=torch.float32, device=dev)
    scratch = torch.empty(lib().rdkv_score_scratch_words(B * H, T, D), dtype=torch.float32, device=dev)
    check(lib().rdkv_score_layer(ptr(aw), q_dtype_tag(aw), ptr(q), q_dtype_tag(q), ptr(k), q_dtype_tag(k),
                                 k.stride(1), k.stride(2), B * H, g * W, T, D, ptr(scratch), ptr(token),
                                 ptr(channel), stream_ptr(dev)), "rdkv_score_layer")
    return token, channel


def obs_window_scores(q_obs: Tensor, k: Tensor, *, causal: bool = True, normalise: bool = False, check_status: bool = False):
    """Token and channel scores of a prefilled layer from the observation window's queries and the
    layer's keys in one step: what the reference computes with a matmul, a masked softmax and
    ``_score_one_layer`` (obkv_fast.py:1443-1466), without materialising the ``[H_q,W,T]`` weights.

    q_obs [B,H_q,W,128] (the last W query positions, after RoPE), k [B,H_kv,T,128], both fp16 or both
    bf16 -> (layer_token [B,H_kv,T], layer_channel [B,H_kv,128]) fp32, as ``_score_one_layer`` returns
    them.  ``causal``: window position w sees keys up to T-W+w (the reference's ``obs_mask``).
    ``normalise``: divide the token scores by the number of window positions that can see each key
    (the reference's ``correct_norm``, obkv_fast.py:1342-1344, 1461).  ``check_status``: wait for the kernels
    and raise if one of their bounded waits (for the staged operands, for the tensor-core products)
    ran out, in which case the scores are invalid; without it the call returns at once."""
    require_cuda(q_obs, "q_obs"); require_cuda(k, "k")
    if q_obs.dim() != 4 or k.dim() != 4 or q_obs.shape[-1] != 128 or k.shape[-1] != 128:
        raise ValueError("q_obs must be [B,H_q,W,128] and k [B,H_kv,T,128]")
    if q_obs.dtype != k.dtype or q_obs.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("q_obs and k must both be fp16 or both bf16")
    B, H_q, W, D = q_obs.shape
    H, T = int(k.shape[1]), int(k.shape[2])
    if k.shape[0] != B or H_q % H != 0:
        raise ValueError(f"k must be [{B},H_kv,T,128] with H_kv dividing {H_q}")
    g = H_q // H
    if g * W > 256:
        raise ValueError(f"g*W = {g * W} rows per KV head: at most 256")
    if causal and W > T:
        raise ValueError("the observation window is longer than the sequence")
    if q_obs.stride(3) != 1 or q_obs.stride(0) != H_q * q_obs.stride(1):
        q_obs = q_obs.contiguous()
    if k.stride(3) != 1 or k.stride(0) != H * k.stride(1):
        k = k.contiguous()
    dev = q_obs.device
    token = torch.empty((B, H, T), dtype=torch.float32, device=dev)
    channel = torch.empty((B, H, D), dtype=torch.float32, device=dev)
    scratch = torch.empty(lib().rdkv_obs_scratch_words(B * H, g, W, T), dtype=torch.float32, device=dev)
    check(lib().rdkv_obs_scores(ptr(q_obs), ptr(k), q_dtype_tag(q_obs), q_obs.stride(1), q_obs.stride(2), k.stride(1),
                                k.stride(2), B * H, g, W, T, 1 if causal else 0, ptr(scratch), ptr(token), ptr(channel),
                                stream_ptr(dev)), "rdkv_obs_scores")
    if check_status:
        status = int(scratch[-1:].view(torch.int32).item())    # (the last scratch word)
        if status != 0:
            raise RuntimeError(f"rdkv_obs_scores: a device-side wait ran out (status {status}: 1 = operands, "
                               f"2 = products); the scores are invalid")
    if normalise:
        norm = torch.full((T,), float(W), dtype=torch.float32, device=dev)
        if causal:
            norm[T - W:] = torch.arange(W, 0, -1, dtype=torch.float32, device=dev)
        token = token / norm
    return token, channel


def apply_score_pooling(scores: Tensor, pool_type: str, kernel_size: int, padding_mode: str = "zero") -> Tensor:
    """Sliding-window average (``pool_type == "avg"``) or maximum of a score row / of the rows of a
    2-D score tensor; ``padding_mode`` "zero" or "reflect" (the window shrinks to ``2*len-1`` taps
    on very short rows, as in the reference)."""
    require_cuda(scores, "scores")
    if scores.dim() not in (1, 2):
        raise ValueError(f"Expected score tensor rank 1 or 2, got shape={tuple(scores.shape)}.")
    x = scores.reshape(1, -1) if scores.dim() == 1 else scores
    if x.dtype != torch.float32:
        x = x.float()
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, n = int(x.shape[0]), int(x.shape[1])
    reflect = padding_mode == "reflect"
    if reflect and n <= 0:
        raise ValueError("Cannot reflect-pool an empty score sequence.")
    taps = min(int(kernel_size), 2 * n - 1) if reflect else int(kernel_size)
    out_len = n + 2 * (taps // 2) - taps + 1
    out = torch.empty((rows, out_len), dtype=torch.float32, device=x.device)
    check(lib().rdkv_score_pool(ptr(x), x.stride(0), rows, n, 0 if pool_type == "avg" else 1, int(kernel_size),
                                1 if reflect else 0, ptr(out), out.stride(0), out_len, stream_ptr(x.device)),
          "rdkv_score_pool")
    out = out.to(scores.dtype) if scores.dtype != torch.float32 else out
    return out[0] if scores.dim() == 1 else out
