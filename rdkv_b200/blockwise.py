"""Blockwise recompression of decode-generated KV (first slice).

The reference's experimental decoder keeps the tokens it generates in blocks of 64 or 128,
compresses each complete block with the prefill machinery (scores from the queries of the NEXT
block, or causal self-scores for the last one) and attends over the prompt layer plus all
compressed blocks plus the uncompressed tail (obkv_accel/blockwise_decode.py).  Built here:

* ``plan_block_compressions``  — the block schedule (blockwise_decode.py:89-140), host logic;
* ``_score_block`` / ``_channel_score`` — block scoring on the GPU (:756-810);
* ``compress_block``           — one block through ``select_and_pack`` per layer, with the
                                 reference's logical-bit accounting (:812-1121, :659-678);
* ``multi_source_attention``   — one softmax over any number of packed sources (+ tail) for a
                                 decode step: every source is a view of ONE DecodeTable, the
                                 fused kernel writes a record per (source, head) and the combine
                                 kernel merges them (the reference scores every source into one
                                 buffer and runs one softmax, :1985-2121).

Not built: slot banks, CUDA-graph replay of the block loop, the model-side decode loop.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from ._lib import check, lib, ptr, q_dtype_tag, require_cuda, stream_ptr
from .packing import PackedKVLayer, select_and_pack


@dataclass(frozen=True)
class BlockwiseRDKVConfig:
    """Knobs of the blockwise decoder, field for field the reference's (blockwise_decode.py:46-71)."""
    block_size: int
    block_budget_tokens: int
    k_budget_ratio: float
    obs_window: int
    pool_kernel_size: int
    pool_padding: str
    v_bit_options: Optional[Tensor]
    k_bit_options: Optional[Tensor]
    epsilon_v: Dict[int, float]
    epsilon_k: Dict[int, float]
    correctness_check: bool = False

    def validate(self) -> None:
        if self.block_size <= 0:
            raise ValueError("decode block size must be positive")
        if self.block_budget_tokens <= 0:
            raise ValueError("decode block budget must be positive")
        if self.block_budget_tokens > self.block_size:
            raise ValueError(f"decode block budget cannot exceed decode block size "
                             f"({self.block_budget_tokens} > {self.block_size})")
        if not 0.0 < self.k_budget_ratio < 1.0:
            raise ValueError("k_budget_ratio must be strictly between 0 and 1")


def plan_block_compressions(generated_tokens: int, block_size: int) -> List[Dict[str, Any]]:
    """Which blocks of the generated tokens get compressed, in order, and whose queries score them.

    A complete block is scored by the queries of its successor.  While generation runs, block b is
    compressed once block b+1 is complete too; at the end every remaining complete block with a
    (possibly partial) successor is drained the same way, marked as part of the final flush, and
    the last block scores itself under a causal mask.  Same records as the reference's planner
    (blockwise_decode.py:89-140)."""
    if generated_tokens < 0 or block_size <= 0:
        raise ValueError("generated_tokens must be non-negative and block_size positive")
    n_full = generated_tokens // block_size
    rest = generated_tokens - n_full * block_size
    # blocks with a successor of any length: all full blocks but the last when nothing follows it
    n_scored_by_next = n_full if rest > 0 else max(n_full - 1, 0)
    # of those, the ones whose successor is complete as well were compressed during generation
    n_in_flight = max(n_full - 1, 0)
    events = []
    for b in range(n_scored_by_next):
        events.append({"block_id": b, "token_start": b * block_size, "token_end": (b + 1) * block_size - 1,
                       "query_source_block": b + 1, "is_final_flush": b >= n_in_flight,
                       "query_mode": "next_block"})
    start = n_scored_by_next * block_size
    if start < generated_tokens:
        events.append({"block_id": n_scored_by_next, "token_start": start, "token_end": generated_tokens - 1,
                       "query_source_block": n_scored_by_next, "is_final_flush": True,
                       "query_mode": "self_causal"})
    return events


def _block_scores(queries: Tensor, keys: Tensor, num_kv_groups: int, causal: bool, want_token: bool):
    require_cuda(queries, "queries"); require_cuda(keys, "keys")
    if queries.dim() != 3 or keys.dim() != 4 or keys.shape[0] != 1:
        raise ValueError("queries must be [H_q,Q,D] and keys [1,H_kv,T,D]")
    h_kv, t_len, head_dim = int(keys.shape[1]), int(keys.shape[2]), int(keys.shape[3])
    q_len = int(queries.shape[1])
    if int(queries.shape[0]) != h_kv * num_kv_groups or int(queries.shape[2]) != head_dim:
        raise ValueError(f"queries {tuple(queries.shape)} do not match {h_kv} KV heads x {num_kv_groups} groups x {head_dim}")
    if causal and q_len != t_len:
        raise ValueError(f"self-scored final flush requires equal query/key lengths, got Q={q_len}, T={t_len}")
    if queries.stride(2) != 1:
        queries = queries.contiguous()
    if keys.stride(3) != 1:
        keys = keys.contiguous()
    dev = keys.device
    token = torch.empty((h_kv, t_len), dtype=torch.float32, device=dev) if want_token else None
    channel = torch.empty((h_kv, head_dim), dtype=torch.float32, device=dev)
    check(lib().rdkv_block_scores(ptr(queries), q_dtype_tag(queries), queries.stride(0), queries.stride(1),
                                  ptr(keys), q_dtype_tag(keys), keys.stride(1), keys.stride(2), h_kv, num_kv_groups,
                                  q_len, t_len, head_dim, 1 if causal else 0, ptr(token), ptr(channel),
                                  stream_ptr(dev)), "rdkv_block_scores")
    return token, channel


def _score_block(queries: Tensor, keys: Tensor, *, num_kv_groups: int, causal: bool) -> Tuple[Tensor, Tensor]:
    """queries [H_q,Q,D], keys [1,H_kv,T,D] -> (token scores [H_kv,T], channel scores [H_kv,D]), fp32
    (reference: blockwise_decode.py:756-792)."""
    return _block_scores(queries, keys, num_kv_groups, causal, True)


def _channel_score(queries: Tensor, keys: Tensor, *, num_kv_groups: int) -> Tensor:
    """The channel statistic alone (reference: blockwise_decode.py:794-810)."""
    return _block_scores(queries, keys, num_kv_groups, False, False)[1]


def _logical_layer_bits_tensor(packed: PackedKVLayer, head_dim: int) -> Tensor:
    """Bits a packed layer stands for, from the allocator's decisions, without a host read: V bits
    times head_dim, plus every head's K bits per kept token (reference: blockwise_decode.py:665-678)."""
    v_bits, k_bits = packed.allocation_v_bits, packed.allocation_k_bits
    if v_bits is None or k_bits is None:
        raise RuntimeError("packed block is missing allocator decisions")
    kept = (v_bits > 0).sum(dim=1).to(torch.int64)
    return v_bits.to(torch.int64).sum() * int(head_dim) + (k_bits.to(torch.int64).sum(dim=1) * kept).sum()


def _logical_layer_bits(packed: PackedKVLayer, head_dim: int) -> int:
    return int(_logical_layer_bits_tensor(packed, head_dim).item())


@dataclass
class CompressedDecodeBlock:
    """One compressed block of generated tokens, all layers (reference: blockwise_decode.py:74-86)."""
    block_id: int
    token_start: int
    token_end: int
    packed: Tuple[PackedKVLayer, ...]
    new_v_only: List[Optional[Tensor]]
    logical_bits_per_layer: Tensor                 # int64 [layers], on the device
    fp16_equivalent_tokens_per_layer: Tensor       # float64 [layers]
    extra: Dict[str, Any] = field(default_factory=dict)


def compress_block(*, target_kv: Sequence[Tensor], query_block: Sequence[Tensor],
                   token_scores_by_layer: Sequence[Tensor], block_id: int, token_start: int, token_end: int,
                   config: BlockwiseRDKVConfig, num_kv_groups: int, model_dtype: torch.dtype = torch.float16
                   ) -> CompressedDecodeBlock:
    """Compress one block of generated tokens, layer by layer (reference: _compress_block,
    blockwise_decode.py:812-1121, default path): ``target_kv[l]`` [1,H_kv,T,2*D] holds the block's
    keys and values side by side, ``query_block[l]`` [H_q,Q,D] the scoring queries,
    ``token_scores_by_layer[l]`` [H_kv,T] the token scores (from :func:`_score_block`).  Each layer
    goes through the channel statistic and :func:`rdkv_b200.packing.select_and_pack` with the
    block's budget; the allocator's decisions are kept on the layer for the bit accounting."""
    packed_layers, v16_layers, bits = [], [], []
    head_dim = int(target_kv[0].shape[-1] // 2)
    h_kv = int(target_kv[0].shape[1])
    for kv, queries, token_scores in zip(target_kv, query_block, token_scores_by_layer):
        keys = kv[..., :head_dim].to(dtype=model_dtype)
        values = kv[..., head_dim:].to(dtype=model_dtype)
        channel_scores = _channel_score(queries, keys, num_kv_groups=num_kv_groups)
        packed, new_v_only, _ = select_and_pack(
            keys, values, token_scores, channel_scores, gqa_factor=num_kv_groups,
            token_budget=config.block_budget_tokens, k_budget_ratio=config.k_budget_ratio,
            obs_window=config.obs_window, pool_kernel_size=config.pool_kernel_size,
            pool_padding=config.pool_padding, pool_type="avg", v_bit_options=config.v_bit_options,
            k_bit_options=config.k_bit_options, eps_V=config.epsilon_v, eps_K=config.epsilon_k,
            retain_allocation_metadata=True)
        if config.correctness_check:
            for t in (packed.K_ch_scale, packed.K_ch_zp, packed.V_scale, packed.V_zp, new_v_only):
                if t is not None and t.is_floating_point() and not bool(torch.isfinite(t).all()):
                    raise FloatingPointError("non-finite packed metadata")
        bits.append(_logical_layer_bits_tensor(packed, head_dim))
        packed_layers.append(packed)
        v16_layers.append(new_v_only)
    logical = torch.stack(bits)
    return CompressedDecodeBlock(block_id=block_id, token_start=token_start, token_end=token_end,
                                 packed=tuple(packed_layers), new_v_only=v16_layers, logical_bits_per_layer=logical,
                                 fp16_equivalent_tokens_per_layer=logical.double() / (2 * h_kv * head_dim * 16))


def multi_source_attention(q: Tensor, sources: Sequence[Tuple[PackedKVLayer, Optional[Tensor]]], *,
                           new_k: Optional[Tensor] = None, new_v: Optional[Tensor] = None, n_new=0,
                           table=None):
    """Attention of one decode step of one layer over several packed sources — the prompt's layer
    and the compressed decode blocks — and the uncompressed tail, with ONE softmax over all of them.

    q [H_q,128]; sources: (PackedKVLayer, new_v_only) pairs of the same head layout; new_k / new_v
    [1,H_kv,cap,128] with n_new live rows.  Every source is a view of one DecodeTable (pass the
    returned table back in while the sources stay the same): one fused launch writes a record per
    (source, query head), the tail kernel one more, the combine kernel merges them.
    Returns (out [H_q,128] fp32, table)."""
    from .decode import DecodeTable, lse_combine, packed_decode_attention, tail_attention_partial
    from ._lib import HEAD_DIM, PARTIAL_STRIDE
    require_cuda(q, "q")
    H_q = int(q.shape[0])
    n_src = len(sources)
    if table is None:
        table = DecodeTable([s[0] for s in sources], [s[1] for s in sources], H_q)
    if table.n_views != n_src:
        raise ValueError("the table was built for another number of sources")
    H_kv = table.H_kv
    has_tail = new_k is not None
    recs = getattr(table, "_ms_records", None)
    if recs is None or recs.shape[0] != n_src + 1:
        recs = torch.empty((n_src + 1, H_q, PARTIAL_STRIDE), dtype=torch.float32, device=q.device)
        table._ms_records = recs
    q_rep = q.reshape(1, H_q, HEAD_DIM).expand(n_src, H_q, HEAD_DIM).contiguous()
    packed_decode_attention(q_rep, table, out_partial=recs[:n_src].view(n_src * H_q, PARTIAL_STRIDE))
    n_rec = n_src
    if has_tail:
        if new_v is None:
            raise ValueError("new_k needs new_v")
        tail_attention_partial(q.reshape(1, H_q, HEAD_DIM), new_k, new_v, n_new, H_kv, recs[n_src])
        n_rec += 1
    out = lse_combine(recs[:n_rec].permute(1, 0, 2))
    return out, table
