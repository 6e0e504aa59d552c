"""Batched Lagrangian bit allocator on the GPU.

Drop-in for the reference's ``knapsack_bit_allocation_batched`` and its scalar
twin (knapsack_solver.py:39-248): same arguments, same LongTensor result, and
bit-for-bit the same choices as the reference produces on CPU.  The whole
multiplier search (lambda_hi doubling, lambda = 0 shortcut, bisection with
per-row freeze) runs inside one kernel pair, one CTA per row.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Union

import torch

from ._lib import check, lib, ptr, require_cuda, stream_ptr

# Default distortion tables of the reference (knapsack_solver.py:23-34): normalised
# quantisation MSE per bit-width from its calibration runs.
DEFAULT_EPSILON: Dict[int, float] = {0: 1.0, 2: 0.25, 4: 0.011, 8: 0.000057, 16: 0.0}
DEFAULT_EPSILON_K: Dict[int, float] = {0: 1.0, 2: 0.277, 4: 0.011, 8: 0.000061, 16: 0.0}
DEFAULT_EPSILON_V: Dict[int, float] = {0: 1.0, 2: 0.312, 4: 0.0138, 8: 0.000048, 16: 0.0}

BITS = torch.tensor([0, 2, 4, 8, 16], dtype=torch.float32)


def knapsack_bit_allocation_batched(scores: torch.Tensor, budget_per_token: Union[float, torch.Tensor],
                                    epsilon: Optional[Dict[int, float]] = None, max_iters: int = 64,
                                    tol: float = 0.01, bit_options: Optional[torch.Tensor] = None
                                    ) -> torch.Tensor:
    """scores [B,T] (CUDA) -> LongTensor [B,T] with values from ``bit_options``.

    Each row minimises sum_t score_t*eps(b_t) subject to mean(b_t) ~ budget via
    cost(t,b) = score_t*eps(b) + lambda*b and a 1-D search over lambda.
    """
    if epsilon is None:
        epsilon = DEFAULT_EPSILON
    bits = bit_options if bit_options is not None else BITS
    assert scores.dim() == 2, f"knapsack_bit_allocation_batched expects [B, T]; got {tuple(scores.shape)}"
    require_cuda(scores, "scores")
    s = scores.detach().float()
    if s.stride(1) != 1:
        s = s.contiguous()
    B, T = s.shape
    dev = s.device
    if torch.is_tensor(budget_per_token):
        assert budget_per_token.shape == (B,), (
            f"budget_per_token tensor must be [B={B}]; got {tuple(budget_per_token.shape)}")
        budget = budget_per_token.detach().float().to(dev).contiguous()
    else:
        budget = torch.full((B,), float(budget_per_token), dtype=torch.float32, device=dev)
    opt = [float(b) for b in bits.tolist()]
    eps = [float(epsilon[int(b)]) for b in opt]
    n = len(opt)
    out = torch.empty((B, T), dtype=torch.int64, device=dev)
    if B == 0 or T == 0:
        return out
    scratch = torch.empty(3 * B, dtype=torch.int32, device=dev)
    c_bits = (C.c_float * n)(*opt)
    c_eps = (C.c_float * n)(*eps)
    check(lib().rdkv_knapsack_batched(ptr(s), s.stride(0), B, T, ptr(budget), c_bits, c_eps, n, int(max_iters),
                                      float(tol), ptr(out), ptr(scratch), stream_ptr(dev)),
          "rdkv_knapsack_batched")
    return out


def knapsack_bit_allocation(scores: torch.Tensor, budget_per_token: float,
                            epsilon: Optional[Dict[int, float]] = None, max_iters: int = 64,
                            tol: float = 0.01, bit_options: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-row form (reference: knapsack_solver.py:39-118): scores [T] -> LongTensor [T]."""
    return knapsack_bit_allocation_batched(scores.reshape(1, -1), float(budget_per_token), epsilon=epsilon,
                                           max_iters=max_iters, tol=tol, bit_options=bit_options)[0]
