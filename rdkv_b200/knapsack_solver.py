"""Batched Lagrangian bit allocator on the GPU.

Drop-in for the reference's ``knapsack_bit_allocation_batched`` and its scalar
twin (knapsack_solver.py:39-248): same arguments, same LongTensor result, and
bit-for-bit the same choices as the reference produces on CPU.  The whole
multiplier search (lambda_hi doubling, lambda = 0 shortcut, bisection with
per-row freeze) runs inside one kernel pair, one CTA per row.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Dict, Optional, Tuple, Union

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
    """Single-row form (reference: knapsack_solver.py:39-118): scores [T] -> LongTensor [T].

    Its own kernel, not the batched one: the reference's scalar solver bisects the multiplier in
    Python floats (double precision), compares means and the tolerance in double and has no floor
    under lambda_hi, so on some rows it settles on another multiplier than the batched solver."""
    if epsilon is None:
        epsilon = DEFAULT_EPSILON
    bits = bit_options if bit_options is not None else BITS
    require_cuda(scores, "scores")
    s = scores.detach().float().reshape(1, -1).contiguous()
    T = s.shape[1]
    out = torch.empty((1, T), dtype=torch.int64, device=s.device)
    if T == 0:
        return out[0]
    opt = [float(b) for b in bits.tolist()]
    eps = [float(epsilon[int(b)]) for b in opt]
    budget = torch.tensor([float(budget_per_token)], dtype=torch.float64, device=s.device)
    check(lib().rdkv_knapsack_rows(ptr(s), s.stride(0), 1, T, ptr(budget), (C.c_float * len(opt))(*opt),
                                   (C.c_float * len(opt))(*eps), len(opt), int(max_iters), float(tol), ptr(out),
                                   stream_ptr(s.device)), "rdkv_knapsack_rows")
    return out[0]


# ── distortion tables from a calibration file, and the bit budgets ──────────────────────────────
def _read_calibration(path: str) -> Dict[int, dict]:
    with open(path, "r") as f:
        return {int(bits): stats for bits, stats in json.load(f).items()}


def load_epsilon_from_calibration(path: str) -> Dict[int, float]:
    """One distortion table for K and V from a calibration JSON ({bits: {"K_mean", "V_mean", ...}}):
    the average of the two means per bit-width (reference: knapsack_solver.py:370-381)."""
    return {bits: (st["K_mean"] + st["V_mean"]) / 2.0 for bits, st in _read_calibration(path).items()}


def load_epsilon_kv_from_calibration(path: str) -> Tuple[Dict[int, float], Dict[int, float]]:
    """(epsilon_K, epsilon_V) from a calibration JSON (reference: knapsack_solver.py:384-404).
    K: 0 bits costs 1 (channel eviction), 16 bits costs 0, and 2/4/8 bits take the per-channel
    figure ``K_per_channel_mean`` where the file has it, else ``K_mean``.  V: ``V_mean`` of the
    widths 0, 2, 4, 8, 16 the file lists."""
    table = _read_calibration(path)
    eps_k: Dict[int, float] = {0: 1.0}
    eps_v: Dict[int, float] = {}
    for bits, st in table.items():
        if bits in (2, 4, 8):
            eps_k[bits] = st.get("K_per_channel_mean", st["K_mean"])
        if bits in (0, 2, 4, 8, 16):
            eps_v[bits] = st["V_mean"]
    eps_k[16] = 0.0
    return eps_k, eps_v


def total_budget_bits(token_budget: int, head_dim: int) -> int:
    """Bits one head may spend on K and V together: ``token_budget`` tokens at fp16
    (reference: obkv_fast.py:979)."""
    return 2 * int(token_budget) * int(head_dim) * 16


def v_average_bits(token_budget: int, head_dim: int, seq_len: int, k_budget_ratio: float) -> float:
    """Average bits per V element over the whole sequence, the budget of the V allocation
    (reference: obkv_fast.py:979-981)."""
    return (1.0 - k_budget_ratio) * total_budget_bits(token_budget, head_dim) / (int(seq_len) * int(head_dim))


def k_average_bits_per_head(token_budget: int, head_dim: int, k_budget_ratio: float,
                            kept_tokens_per_head: torch.Tensor) -> torch.Tensor:
    """Average bits per K element of every head, the budgets of the K allocation: the K share of
    the bits over the tokens the head actually kept (at least one), fp32, on the tensor's device
    (reference: obkv_fast.py:983, 1033-1035 — the same expression, a Python number divided by an
    fp32 tensor)."""
    k_budget_bits = k_budget_ratio * total_budget_bits(token_budget, head_dim)
    return k_budget_bits / (int(head_dim) * kept_tokens_per_head.clamp(min=1).float())
