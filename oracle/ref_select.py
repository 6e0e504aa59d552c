"""numpy restatement of the reference's per-layer select-and-pack composite (test oracle).

Follows obkv_fast.py:899-1186 (_perhead_select_and_pack_joint) in the reference project: score
pooling, V allocation over the whole sequence at v_avg bits, per-head K budgets from the tokens
each head kept, K allocation, eviction of the channels that got 0 bits, packing.  Test
infrastructure only; the product path is rdkv_b200.packing.select_and_pack.
"""
from __future__ import annotations

import numpy as np

from .ref_knapsack import knapsack_batched
from .ref_packing import pack_kv
from .ref_scoring import score_pooling

F32 = np.float32


def budgets(token_budget: int, head_dim: int, seq_len: int, k_budget_ratio: float, kept_per_head: np.ndarray):
    """(v_avg as a Python float, k_avg per head as fp32): obkv_fast.py:979-981, 983, 1033-1035.  The
    reference divides a Python number by an fp32 tensor, which torch evaluates as
    reciprocal(tensor) * fp32(number)."""
    total = 2 * token_budget * head_dim * 16
    v_avg = (1.0 - k_budget_ratio) * total / (seq_len * head_dim)
    denom = (F32(head_dim) * np.maximum(kept_per_head, 1).astype(F32)).astype(F32)
    k_avg = ((F32(1.0) / denom).astype(F32) * F32(k_budget_ratio * total)).astype(F32)
    return v_avg, k_avg


def select_and_pack(K, V, token_scores, channel_scores, *, gqa_factor, token_budget, k_budget_ratio,
                    pool_kernel_size=5, pool_padding="reflect", pool_type="avg", eps_V, eps_K):
    """K, V [1,H_kv,T,D] fp16, token_scores [H_kv,T], channel_scores [H_kv,D] ->
    (layer dict, new_v_only, v_bits, k_bits)."""
    H, T = token_scores.shape
    D = K.shape[3]
    pooled = (score_pooling(token_scores, pool_type, pool_kernel_size, pool_padding)
              if pool_kernel_size > 1 else token_scores).astype(F32)
    v_avg, _ = budgets(token_budget, D, T, k_budget_ratio, np.ones(H))
    v_bits = knapsack_batched(pooled, v_avg, eps_V)
    _, k_avg = budgets(token_budget, D, T, k_budget_ratio, (v_bits > 0).sum(axis=1))
    k_bits = knapsack_batched(channel_scores.astype(F32), k_avg, eps_K)
    K = np.where((k_bits == 0)[None, :, None, :], np.zeros_like(K), K)
    layer, nv = pack_kv(K, V, v_bits, k_bits, gqa_factor)
    return layer, nv, v_bits, k_bits
