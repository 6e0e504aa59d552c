"""rdkv_b200 — B200-native (sm_100a) packed-KV decode path.

Operators (all CUDA, no CPU or PyTorch fallback):
  packing          quantise + bit-pack of K (per channel) and V (per token)
  knapsack_solver  batched Lagrangian bit allocator
  k_kernel         q·K scores over packed K
  v_kernel         softmax-weighted sum over packed V
  decode           fused split-sequence decode attention + log-sum-exp combine
  sharding         KV-head / sequence sharding across GPUs
"""
from .packing import PackedKVLayer, TriZoneCache, DualZoneCache  # noqa: F401

__all__ = ["PackedKVLayer", "TriZoneCache", "DualZoneCache"]
