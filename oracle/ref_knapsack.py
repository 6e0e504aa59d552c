"""numpy restatement of the reference Lagrangian bit allocator (test oracle).

Follows knapsack_solver.py:121-248 (knapsack_bit_allocation_batched) in the
reference project, including its batch-wide loop exits:
  * lambda_hi = max(score)*0.375, floored at 1e-8, doubled (at most 40 rounds)
    for rows whose mean bits at lambda_hi still exceed the budget; the doubling
    loop stops for EVERY row once no row needs it or all rows reached 1e12;
  * rows whose mean at lambda = 0 is within budget return that solution;
  * bisection for max_iters rounds; a row is frozen at the first round whose
    relative budget error is < tol (compared in fp32); rows that never converge
    return the last round's choice.
cost = score*eps[n] + lambda*bits[n] with every product and the sum rounded to
fp32 separately; ties go to the lowest option index.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32

DEFAULT_BITS = (0, 2, 4, 8, 16)


def _solve(scores: np.ndarray, lam: np.ndarray, eps: np.ndarray, bits: np.ndarray) -> np.ndarray:
    """[B,T] chosen bit value (fp32) per unit for per-row multipliers lam [B]."""
    out = np.empty(scores.shape, F32)
    step = max(1, (1 << 22) // max(1, scores.shape[1]))
    for b0 in range(0, scores.shape[0], step):
        s = scores[b0:b0 + step]
        cost = (s[:, :, None] * eps[None, None, :]).astype(F32) + \
               (lam[b0:b0 + step, None, None] * bits[None, None, :]).astype(F32)
        out[b0:b0 + step] = bits[np.argmin(cost, axis=2)]
    return out


def _mean(x: np.ndarray) -> np.ndarray:
    # sums of small integers are exact in fp32 below 2^24; one IEEE division
    return (x.sum(axis=1, dtype=np.float64).astype(F32) / F32(x.shape[1])).astype(F32)


def knapsack_batched(scores, budget, epsilon: dict, max_iters: int = 64, tol: float = 0.01,
                     bit_options=DEFAULT_BITS) -> np.ndarray:
    scores = np.ascontiguousarray(scores, dtype=F32)
    B, T = scores.shape
    bits = np.asarray(bit_options, dtype=F32)
    eps = np.asarray([epsilon[int(b)] for b in bits], dtype=F32)
    budget = np.broadcast_to(np.asarray(budget, dtype=F32), (B,)).astype(F32)
    tol32 = F32(tol)

    lam_lo = np.zeros(B, F32)
    lam_hi = np.maximum(scores.max(axis=1) * F32(0.375), F32(1e-8)).astype(F32)
    for _ in range(40):
        need = _mean(_solve(scores, lam_hi, eps, bits)) > budget
        if not need.any():
            break
        lam_hi = np.where(need, lam_hi * F32(2.0), lam_hi).astype(F32)
        if (lam_hi >= F32(1e12)).all():
            break

    bits_lo = _solve(scores, lam_lo, eps, bits)
    converged = _mean(bits_lo) <= budget
    final = bits_lo.copy()
    bits_mid = bits_lo.copy()
    for _ in range(max_iters):
        lam_mid = ((lam_lo + lam_hi) / F32(2.0)).astype(F32)
        bits_mid = _solve(scores, lam_mid, eps, bits)
        avg = _mean(bits_mid)
        rel = (np.abs(avg - budget) / np.maximum(budget, F32(1e-8))).astype(F32)
        just = (rel < tol32) & ~converged
        final[just] = bits_mid[just]
        converged |= just
        if converged.all():
            break
        high = avg > budget
        lam_lo = np.where(high, lam_mid, lam_lo).astype(F32)
        lam_hi = np.where(high, lam_hi, lam_mid).astype(F32)
    final[~converged] = bits_mid[~converged]
    return final.astype(np.int64)


def knapsack_scalar(scores, budget: float, epsilon: dict, max_iters: int = 64, tol: float = 0.01,
                    bit_options=DEFAULT_BITS) -> np.ndarray:
    """The reference's single-row solver (knapsack_solver.py:39-118): same cost and argmin as the
    batched one, but the multiplier is a Python float (double) that enters the cost as its fp32
    rounding, the means (fp32) are compared with the budget in double, lambda_hi starts at
    max(score)*0.375 without a floor and is doubled while the mean exceeds the budget and it is
    below 1e12, and the tolerance test runs in double."""
    s = np.ascontiguousarray(scores, dtype=F32).reshape(1, -1)
    bits = np.asarray(bit_options, dtype=F32)
    eps = np.asarray([epsilon[int(b)] for b in bits], dtype=F32)
    budget = float(budget)

    def solve(lam: float) -> np.ndarray:
        return _solve(s, np.asarray([lam], dtype=F32), eps, bits)

    def mean(b: np.ndarray) -> float:
        return float(_mean(b)[0])

    lam_lo, lam_hi = 0.0, float(s.max()) * 0.375
    rounds = 0
    while mean(solve(lam_hi)) > budget and lam_hi < 1e12 and rounds < 200:
        lam_hi *= 2.0
        rounds += 1
    lo = solve(lam_lo)
    if mean(lo) <= budget:
        return lo[0].astype(np.int64)
    mid = lo
    for _ in range(max_iters):
        lam_mid = (lam_lo + lam_hi) / 2.0
        mid = solve(lam_mid)
        avg = mean(mid)
        if abs(avg - budget) / max(budget, 1e-8) < tol:
            break
        if avg > budget:
            lam_lo = lam_mid
        else:
            lam_hi = lam_mid
    return mid[0].astype(np.int64)
