"""Seeded synthetic K/V/q and bit allocations with the shapes and value
distributions of the benchmark configurations.

No dataset or checkpoint is involved: K ~ N(0,1) with four fixed outlier
channels per head scaled x10, V ~ N(0,1), q ~ N(0,1)/sqrt(D); token and channel
importances are lognormal.  The prescribed allocation ranks importances and
hands out bit-widths in fixed fractions of the token budget N
(N/8 fp16, N/4 8-bit, 3N/8 4-bit, N/4 2-bit, rest evicted) and of the 128
channels (16 at 8-bit, 24 at 4-bit, 24 at 2-bit, 64 pruned).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

OUTLIER_BASE = (3, 37, 71, 105)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def make_kv(H_kv: int, T: int, D: int = 128, *, seed: int, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """K, V [1,H_kv,T,D] fp16."""
    g = _gen(seed, device)
    K = torch.randn(H_kv, T, D, generator=g, device=device, dtype=torch.float32)
    V = torch.randn(H_kv, T, D, generator=g, device=device, dtype=torch.float32)
    for h in range(H_kv):
        for c in OUTLIER_BASE:
            K[h, :, (16 * h + c) % D] *= 10.0
    return K.half().unsqueeze(0), V.half().unsqueeze(0)


def make_q(H_q: int, D: int = 128, *, seed: int, device="cpu", dtype=torch.float16, batch: Optional[int] = None):
    g = _gen(seed, device)
    shape = (H_q, D) if batch is None else (batch, H_q, D)
    return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) / math.sqrt(D)).to(dtype)


def rank_to_bits(importance: torch.Tensor, counts: Sequence[Tuple[int, int]]) -> torch.Tensor:
    """importance [R,L]; counts = [(bit, n), ...] handed out in descending rank order."""
    order = torch.argsort(importance, dim=1, descending=True, stable=True)
    ranked = torch.zeros(importance.shape[1], dtype=torch.long, device=importance.device)
    pos = 0
    for bit, n in counts:
        ranked[pos:pos + n] = bit
        pos += n
    bits = torch.zeros_like(order)
    bits.scatter_(1, order, ranked.unsqueeze(0).expand_as(order))
    return bits


def make_v_bits(H_kv: int, T: int, N: int, *, seed: int, device="cpu",
                per_head_N: Optional[Sequence[int]] = None) -> torch.Tensor:
    """[H_kv,T] long in {0,2,4,8,16}; the config-0 bit mix over a budget of N tokens.

    ``per_head_N`` gives ragged heads a different budget each (coverage of the
    per-head padding, mask and stripe layout).
    """
    g = _gen(seed + 7919, device)
    imp = torch.exp(torch.randn(H_kv, T, generator=g, device=device))
    if per_head_N is None:
        per_head_N = [N] * H_kv
    rows = []
    for h in range(H_kv):
        n = int(per_head_N[h])
        n16, n8, n2 = n // 8, n // 4, n // 4
        n4 = n - n16 - n8 - n2
        rows.append(rank_to_bits(imp[h:h + 1], [(16, n16), (8, n8), (4, n4), (2, n2)]))
    return torch.cat(rows, dim=0)


def make_k_bits(H_kv: int, D: int = 128, *, seed: int, device="cpu",
                mix: Sequence[Tuple[int, int]] = ((8, 16), (4, 24), (2, 24))) -> torch.Tensor:
    """[H_kv,D] long; top channels by lognormal importance get the given (bit, count) mix."""
    g = _gen(seed + 104729, device)
    imp = torch.exp(torch.randn(H_kv, D, generator=g, device=device))
    return rank_to_bits(imp, list(mix))


def make_scores(rows: int, T: int, *, seed: int, sigma: float = 1.5, device="cpu") -> torch.Tensor:
    """Allocator input: lognormal(0, sigma) importances [rows,T] fp32."""
    g = _gen(seed, device)
    return torch.exp(sigma * torch.randn(rows, T, generator=g, device=device, dtype=torch.float32))


ALLOC_EPSILON = {0: 1.0, 2: 0.12, 4: 0.02, 8: 0.0012, 16: 0.0}


def unit_seed(config: int, layer: int = 0, sequence: int = 0) -> int:
    return 1000 * config + 17 * layer + sequence
