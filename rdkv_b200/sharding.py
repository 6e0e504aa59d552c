"""Sharding of the packed-KV decode path over the GPUs of one node.

One process per GPU (torch.distributed, NCCL over NVLink).  Two ways to cut the work:

* KV-head sharding — rank r packs and serves KV heads [r*H_kv/N, (r+1)*H_kv/N) and their
  query heads.  Heads are independent, so attention needs no collective; an all-gather of
  the [B, H_q_local, 128] outputs is only needed if every rank wants the full result.
* sequence split — the ranks of a group serve the same heads of the SAME packed layer (packed
  once, exactly as the reference packs it) and each attends over its own part of every head's
  rows — its share of the head's 2-bit, 4-bit, 8-bit and fp16 rows, so that the parts read about
  the same bytes (`part_rows`); the fused kernel writes one merged (m, l, o) record per query head,
  the ranks exchange the records with one all-gather into local memory per decode step (all
  layers and sequences together) and the log-sum-exp combine kernel merges them.  A rank reads
  only its window's bytes; in this implementation every rank of the group keeps the whole packed
  layer in memory.

The reference has no distributed code; the oracle for both is the single-device result on
the same (sharded, unsplit) inputs.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

PARTIAL_STRIDE = 132


def head_shard(rank: int, world: int, H_kv: int) -> Tuple[int, int]:
    """KV heads [h0, h1) owned by `rank` when `world` ranks share H_kv heads evenly."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    if H_kv % world:
        raise ValueError(f"{world} ranks cannot share {H_kv} KV heads evenly")
    per = H_kv // world
    return rank * per, (rank + 1) * per


def shard_heads(K: Tensor, V: Tensor, v_bits: Tensor, k_bits: Tensor, rank: int, world: int):
    """Slices of one layer's inputs for this rank: K,V [1,H_kv,T,D], v_bits [H_kv,T], k_bits [H_kv,D]."""
    h0, h1 = head_shard(rank, world, K.shape[1])
    return K[:, h0:h1], V[:, h0:h1], v_bits[h0:h1], k_bits[h0:h1]


def row_window(part: int, n_parts: int, rows: int) -> Tuple[int, int]:
    """Live-row window [lo, hi) of sequence part `part` when heads of up to `rows` live rows are
    split into `n_parts` equal parts (multiples of 64 rows, so that windows start on tile-friendly
    boundaries; the last part takes what is left)."""
    if n_parts <= 0 or not 0 <= part < n_parts:
        raise ValueError(f"bad part {part} of {n_parts}")
    per = max(64, ((-(-max(rows, 1) // n_parts) + 63) // 64) * 64)
    lo = min(part * per, rows)
    hi = rows if part == n_parts - 1 else min((part + 1) * per, rows)
    return lo, max(lo, hi)


def part_cut(n: int, i: int, parts: int) -> int:
    """First row of part i when a phase of n rows is shared out over `parts` parts (multiples of
    32 rows; the last part takes what is left).  The kernel computes the same."""
    return n if i >= parts else (n * i // parts) & ~31


def part_rows(counts: Sequence[int], part: int, parts: int):
    """Rows of a head that part `part` of `parts` attends over: for each of the head's phases
    (counts = its 2-bit, 4-bit, 8-bit, fp16 row counts) the (first, end) rows in the head's own
    row order."""
    if parts < 1 or not 0 <= part < parts:
        raise ValueError(f"bad part {part} of {parts}")
    out, base = [], 0
    for n in counts:
        n = int(n)
        out.append((base + part_cut(n, part, parts), base + part_cut(n, part + 1, parts)))
        base += n
    return out


def grid(rank: int, world: int, seq_parts: int) -> Tuple[int, int, int]:
    """(head_rank, head_world, seq_part) of a rank in a head-shards x sequence-parts grid;
    ranks of one sequence group are adjacent."""
    if world % seq_parts:
        raise ValueError(f"world size {world} is not a multiple of {seq_parts} sequence parts")
    return rank // seq_parts, world // seq_parts, rank % seq_parts


def check_group_consistency(n_rows: int, group=None) -> None:
    """Host-side agreement check before the first exchange: every rank of the group must
    bring the same number of records.  Raises on every rank if they disagree."""
    world = dist.get_world_size(group)
    sizes = [None] * world
    dist.all_gather_object(sizes, int(n_rows), group=group)
    if len(set(sizes)) != 1:
        raise ValueError(f"sequence-split group disagrees on the record count: {sizes}")


def combine_across_ranks(local_record: Tensor, group=None, *, combine: Optional[Callable] = None,
                         gathered: Optional[Tensor] = None) -> Tensor:
    """All-gather the merged per-head records [n_rows,132] of the group's ranks into local
    memory and merge them in rank order.  Returns [n_rows,128] fp32.

    `combine(records [n_rows, S, 132]) -> [n_rows,128]` defaults to the CUDA combine kernel."""
    world = dist.get_world_size(group)
    if local_record.dim() != 2 or local_record.shape[1] != PARTIAL_STRIDE:
        raise ValueError("local_record must be [n_rows, 132]")
    n_rows = local_record.shape[0]
    if gathered is None:
        gathered = torch.empty((world * n_rows, PARTIAL_STRIDE), dtype=local_record.dtype,
                               device=local_record.device)
    dist.all_gather_into_tensor(gathered, local_record.contiguous(), group=group)
    records = gathered.view(world, n_rows, PARTIAL_STRIDE).permute(1, 0, 2)   # [n_rows, S, 132] view, no copy
    if combine is None:
        from .decode import lse_combine
        combine = lse_combine
    return combine(records)


def sequence_split_attention(q: Tensor, table, group=None, *, part: Optional[int] = None,
                             n_parts: Optional[int] = None, record: Optional[Tensor] = None,
                             gathered: Optional[Tensor] = None) -> Tensor:
    """Decode attention when the ranks of `group` split the live rows of the same heads: fused
    kernel on this rank's part of every (view, head) -> one record per query head ->
    ONE all-gather for the whole step -> combine.  q [n_views,H_q,128]; returns
    [n_views,H_q,128] fp32 on every rank of the group.  `part` / `n_parts` default to the
    rank and size of the group."""
    from .decode import packed_decode_attention
    n_parts = dist.get_world_size(group) if n_parts is None else n_parts
    part = dist.get_rank(group) if part is None else part
    n_rows = table.n_views * table.H_q
    if record is None:
        record = torch.empty((n_rows, PARTIAL_STRIDE), dtype=torch.float32, device=q.device)
    packed_decode_attention(q, table, out_partial=record, seq_part=(part, n_parts))
    return combine_across_ranks(record, group, gathered=gathered).view(table.n_views, table.H_q, 128)
