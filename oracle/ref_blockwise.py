"""numpy restatement of the reference's blockwise-decode helpers (test oracle).

Follows, in the reference project (obkv_accel/blockwise_decode.py):
  :89-140   plan_block_compressions   which blocks are compressed, and whose queries score them
  :756-792  _score_block              token scores (column sums of softmax(q.k/sqrt(D))) and the
                                      channel statistic mean(q^2) * mean(k^2)
  :659-678  _logical_layer_bits       bits a packed block stands for
Test infrastructure only; the product path is rdkv_b200.blockwise.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def plan_block_compressions(generated_tokens: int, block_size: int):
    """List of (block_id, token_start, token_end, query_source_block, is_final_flush, self_causal)."""
    if generated_tokens < 0 or block_size <= 0:
        raise ValueError("generated_tokens must be non-negative and block_size positive")
    plan, start, b = [], 0, 0
    while generated_tokens - start >= 2 * block_size:      # a complete successor exists: compressed while generating
        plan.append((b, start, start + block_size - 1, b + 1, 0, 0))
        start += block_size
        b += 1
    while generated_tokens - start > block_size:           # drained at the end with a partial successor
        plan.append((b, start, start + block_size - 1, b + 1, 1, 0))
        start += block_size
        b += 1
    if start < generated_tokens:                           # the last block scores itself, causally
        plan.append((b, start, generated_tokens - 1, b, 1, 1))
    return plan


def score_block(queries: np.ndarray, keys: np.ndarray, num_kv_groups: int, causal: bool):
    """queries [H_q,Q,D], keys [1,H_kv,T,D] -> (token [H_kv,T], channel [H_kv,D]) fp32."""
    h_kv, t_len, d = keys.shape[1], keys.shape[2], keys.shape[3]
    q_len = queries.shape[1]
    qg = queries.astype(F32).reshape(h_kv, num_kv_groups, q_len, d)
    k = keys[0].astype(F32)
    logits = np.einsum("hgqd,htd->hgqt", qg, k).astype(F32) * F32(1.0 / np.sqrt(d))
    if causal:
        if q_len != t_len:
            raise ValueError("self-scored final flush requires equal query/key lengths")
        hidden = np.arange(t_len)[None, :] > np.arange(q_len)[:, None]
        logits = np.where(hidden[None, None], F32(-np.inf), logits)
    e = np.exp(logits - logits.max(axis=-1, keepdims=True)).astype(F32)
    att = e / e.sum(axis=-1, keepdims=True)
    token = att.sum(axis=(1, 2)).astype(F32)
    channel = ((qg ** 2).mean(axis=(1, 2)) * (k ** 2).mean(axis=1)).astype(F32)
    return token, channel


def logical_layer_bits(v_bits: np.ndarray, k_bits: np.ndarray, head_dim: int) -> int:
    """v_bits [H_kv,T], k_bits [H_kv,D]: V bits times head_dim plus each head's K bits per kept token."""
    kept = (v_bits > 0).sum(axis=1).astype(np.int64)
    return int(v_bits.astype(np.int64).sum() * head_dim + (k_bits.astype(np.int64).sum(axis=1) * kept).sum())
