"""Packed-cache containers and the prefill quantise-and-bitpack operators.

Host-side mirror of the reference's packing module (obkv_accel/packing.py): same
function names, argument meaning, return tuples and error behaviour, so that a
caller of the reference can switch imports.  All arithmetic runs in the CUDA
library (rdkv_partition_by_bits / rdkv_pack_v / rdkv_pack_k); torch is used for
allocation and for index bookkeeping only.  Tensors must be on a CUDA device.

Layouts (reference: obkv_accel/packing.py:1-20, obkv_accel/bitpack.py):
  4-bit half-split     byte[i] = c[i] | c[i+L/2] << 4
  2-bit quarter-split  byte[i] = c[i] | c[i+L/4] << 2 | c[i+L/2] << 4 | c[i+3L/4] << 6
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch import Tensor

from . import _lib
from ._lib import LayerView, check, lib, ptr, require_cuda, stream_ptr


# ── containers (reference: obkv_accel/packing.py:43-135) ─────────────────────

@dataclass
class PackedKVLayer:
    """One layer of packed cache; field names and shapes as in the reference.

    K: ``K_2bit/K_4bit/K_8bit [1,H_kv,T_k,bytes]`` u8 in the shared-max channel
    layout, ``K_ch_scale/K_ch_zp [1,H_kv,1,D_pad]`` fp16, index tables int64.
    V: ``V_2bit [1,H_kv,N2,D/4]``, ``V_4bit [..,N4,D/2]``, ``V_8bit [..,N8,D]`` u8,
    ``V_scale/V_zp [1,H_kv,T_v,1]`` fp16 in head-local row order.
    """
    K_2bit: Optional[Tensor]
    K_4bit: Optional[Tensor]
    K_8bit: Optional[Tensor]
    K_ch_scale: Tensor
    K_ch_zp: Tensor
    K_ch_sort_idx: Tensor
    K_ch_seg_bounds: Tuple[int, int, int]
    K_ch_perm_padded_idx: Tensor
    V_2bit: Optional[Tensor]
    V_4bit: Optional[Tensor]
    V_8bit: Optional[Tensor]
    V_scale: Tensor
    V_zp: Tensor
    sort_idx: Tensor
    seg_bounds: Tuple[int, int, int]
    T_eff: int
    seg_bounds_per_head: Optional[Tensor] = None
    T_eff_per_head: Optional[Tensor] = None
    softmax_mask: Optional[Tensor] = None
    n_fp16_per_head: Optional[Tensor] = None
    fp16_gap_mask: Optional[Tensor] = None
    K_ch_sort_idx_per_head: Optional[Tensor] = None
    K_ch_perm_padded_idx_per_head: Optional[Tensor] = None
    K_ch_seg_bounds_per_head: Optional[Tensor] = None
    K_ch_perm_padded_idx_for_Q: Optional[Tensor] = None
    T_eff_k: int = 0
    n_v16: int = 0
    T_eff_k_per_head: Optional[Tensor] = None
    n_v16_per_head: Optional[Tensor] = None
    allocation_v_bits: Optional[Tensor] = None
    allocation_k_bits: Optional[Tensor] = None
    deferred_k_for_stack: Optional[Tensor] = None


@dataclass
class TriZoneCache:
    """Packed layers + per-layer fp16 Zone-B values + decode-appended tail."""
    packed: Tuple[PackedKVLayer, ...]
    new_v_only: List[Optional[Tensor]]
    new_both_k: List[Optional[Tensor]]
    new_both_v: List[Optional[Tensor]]
    original_seq_len: int

    @property
    def new_k(self):
        return self.new_both_k

    @property
    def new_v(self):
        return self.new_both_v


DualZoneCache = TriZoneCache


def _pad_to(n: int, align: int) -> int:
    return 0 if n == 0 else ((n + align - 1) // align) * align


_seg_padded_len = _pad_to


def _as_fp16_rows(x: Tensor, name: str) -> Tensor:
    require_cuda(x, name)
    if x.dtype != torch.float16:
        raise ValueError(f"{name} must be float16, got {x.dtype}")
    if x.dim() != 4 or x.shape[0] != 1:
        raise AssertionError(f"Expected {name} [1,H,T,D], got {tuple(x.shape)}")
    if x.stride(3) != 1 and x.shape[3] > 1:
        x = x.contiguous()
    return x


# ── C-ABI wrappers ───────────────────────────────────────────────────────────

def partition_by_bits(bits: Tensor, mode: int, fill: bool = True) -> Tuple[Tensor, Tensor]:
    """Stable class partition of integer bit maps ``[R,L]``.

    Returns ``(order int32 [R,L], counts int32 [R,4])``; mode 0 = tokens
    (classes 2,4,8,16), mode 1 = channels (16 counted as 8).  ``fill=False``: the entries of
    ``order`` past a row's kept count are left uninitialised (for callers that go by ``counts``).
    """
    require_cuda(bits, "bits")
    if bits.dim() != 2:
        raise ValueError("bits must be [rows, len]")
    if bits.dtype not in (torch.int8, torch.int16, torch.int32, torch.int64):
        bits = bits.to(torch.int64)
    if bits.stride(1) != 1 and bits.shape[1] > 1:
        bits = bits.contiguous()
    R, L = bits.shape
    order = torch.empty((R, L), dtype=torch.int32, device=bits.device)
    counts = torch.zeros((R, 4), dtype=torch.int32, device=bits.device)
    if R and L:
        check(lib().rdkv_partition_by_bits(ptr(bits), bits.element_size(), bits.stride(0), R, L,
                                           mode if fill else mode + 4,
                                           ptr(order), ptr(counts), stream_ptr(bits.device)),
              "rdkv_partition_by_bits")
    return order, counts


def _launch_pack_v(V: Tensor, order: Optional[Tensor], order_rs: int, counts: Optional[Tensor],
                   counts_rs: int, n_identity: int, identity_bits: int, mx: Sequence[int], max_t_v: int,
                   override: int = 0):
    """Allocates the outputs and runs rdkv_pack_v; returns (v2, v4, v8, v16, scale, zp)."""
    _, H, _, D = V.shape
    dev = V.device
    m2, m4, m8, m16 = (int(x) for x in mx)
    u8 = dict(dtype=torch.uint8, device=dev)
    v2 = torch.empty((1, H, m2, D // 4), **u8) if m2 else None
    v4 = torch.empty((1, H, m4, D // 2), **u8) if m4 else None
    v8 = torch.empty((1, H, m8, D), **u8) if m8 else None
    v16 = torch.empty((1, H, m16, D), dtype=torch.float16, device=dev) if m16 else None
    scale = torch.empty((1, H, max_t_v, 1), dtype=torch.float16, device=dev)
    zp = torch.empty_like(scale)
    check(lib().rdkv_pack_v(ptr(V), V.stride(1), V.stride(2), H, D, ptr(order), order_rs, ptr(counts),
                            counts_rs, n_identity, identity_bits, m2, m4, m8, m16, ptr(v2), ptr(v4), ptr(v8),
                            ptr(v16), ptr(scale), ptr(zp), max_t_v, override, stream_ptr(dev)),
          "rdkv_pack_v")
    return v2, v4, v8, v16, scale, zp


def _launch_pack_k(K: Tensor, tok_order, tok_order_rs, tok_counts, tok_counts_rs, max_t_v: int, t_k: int,
                   ch_order: Tensor, ch_order_rs: int, ch_counts: Tensor, ch_counts_rs: int,
                   n2p: int, n4p: int, n8p: int, d_kept_max: int, gqa: int, override: int = 0):
    """Allocates outputs + scratch and runs rdkv_pack_k.

    Returns (k2, k4, k8, scale, zp, sort_idx [H,d_kept_max], perm [H,d_pad], perm_q or None,
    seg_bounds int32 [H,3]).
    """
    _, H, _, D = K.shape
    dev = K.device
    d_pad = n2p + n4p + n8p
    u8 = dict(dtype=torch.uint8, device=dev)
    i64 = dict(dtype=torch.int64, device=dev)
    if override:
        k2 = k4 = None
        k8 = torch.empty((1, H, t_k, d_pad), **u8)
    else:
        k2 = torch.empty((1, H, t_k, n2p // 4), **u8) if n2p else None
        k4 = torch.empty((1, H, t_k, n4p // 2), **u8) if n4p else None
        k8 = torch.empty((1, H, t_k, n8p), **u8) if n8p else None
    scale = torch.empty((1, H, 1, d_pad), dtype=torch.float16, device=dev)
    zp = torch.empty_like(scale)
    sort_idx = torch.empty((H, d_kept_max), **i64)
    perm = torch.empty((H, d_pad), **i64)
    perm_q = torch.empty((H * gqa, d_pad), **i64) if gqa > 0 else None
    seg_bounds = torch.empty((H, 3), dtype=torch.int32, device=dev)
    if d_pad > 0:
        slabs = lib().rdkv_pack_k_slabs(t_k)
        scratch = torch.empty(H * slabs * 2 * d_pad, dtype=torch.float32, device=dev)
        check(lib().rdkv_pack_k(ptr(K), K.stride(1), K.stride(2), H, D, ptr(tok_order), tok_order_rs,
                                ptr(tok_counts), tok_counts_rs, max_t_v, t_k, ptr(ch_order), ch_order_rs,
                                ptr(ch_counts), ch_counts_rs, n2p, n4p, n8p, d_kept_max, gqa, ptr(scratch),
                                ptr(k2), ptr(k4), ptr(k8), ptr(scale), ptr(zp), ptr(sort_idx), ptr(perm),
                                ptr(perm_q), ptr(seg_bounds), override, stream_ptr(dev)),
              "rdkv_pack_k")
    else:
        seg_bounds.zero_()
    return k2, k4, k8, scale, zp, sort_idx, perm, perm_q, seg_bounds


# ── reference-named operators ────────────────────────────────────────────────

def quantize_and_pack(x: Tensor, n_bits: int, dim: int) -> Tuple[Tensor, Tensor, Tensor]:
    """Asymmetric uniform quantisation along ``dim`` of a ``[1,H,T,D]`` fp16 tensor
    (reference: obkv_accel/packing.py:141-165).  Returns (codes u8 like x, scale
    fp16, zero_point fp16, both keepdim along ``dim``).  dim 3 = per token, dim 2 =
    per channel; other layouts are not part of the packed-cache path.
    """
    x = _as_fp16_rows(x, "x")
    if n_bits not in (2, 4, 8):
        raise ValueError(f"Unsupported n_bits={n_bits}")
    _, H, T, D = x.shape
    dim = dim % 4
    if T == 0 or D == 0:
        raise ValueError("cannot quantise an empty tensor")
    if dim == 3:
        if D % 4:
            raise ValueError("per-token quantisation needs D % 4 == 0")
        _, _, v8, _, scale, zp = _launch_pack_v(x, None, 0, None, 0, T, 8, (0, 0, T, 0), T, override=n_bits)
        return v8, scale, zp
    if dim == 2:
        dev = x.device
        ch_order = torch.arange(D, dtype=torch.int32, device=dev).view(1, D)
        ch_counts = torch.tensor([[0, 0, D, 0]], dtype=torch.int32, device=dev)
        _, _, k8, scale, zp, *_ = _launch_pack_k(x, None, 0, None, 0, T, T, ch_order, 0, ch_counts, 0,
                                                 0, 0, D, D, 0, override=n_bits)
        return k8, scale, zp
    raise ValueError("quantize_and_pack supports dim=2 (per channel) and dim=3 (per token)")


def pack_v_segments(V: Tensor, v_bits: Tensor, *, segment_counts: Optional[Tuple[int, int, int]] = None):
    """Sort tokens by bit-width (stable) and pack each V segment
    (reference: obkv_accel/packing.py:715-778).  V [1,H,T,D] fp16, v_bits [T] in {2,4,8}.

    Returns (V_2bit, V_4bit, V_8bit, V_scale, V_zp, sort_idx, (N_2, N_4, N_8)); a
    segment with no tokens is None.
    """
    V = _as_fp16_rows(V, "V")
    T, D = V.shape[2], V.shape[3]
    if D % 4:
        raise AssertionError("head dim must be a multiple of 4")
    order, counts = partition_by_bits(v_bits.reshape(1, -1).to(V.device), 0)
    if segment_counts is None:
        n2, n4, n8 = (int(c) for c in counts[0, :3].tolist())
    else:
        n2, n4, n8 = map(int, segment_counts)
    assert n2 + n4 + n8 == T, f"Segment sizes {n2}+{n4}+{n8} != T_eff={T}"
    v2, v4, v8, _, scale, zp = _launch_pack_v(V, order, 0, counts, 0, 0, 0, (n2, n4, n8, 0), T)
    return v2, v4, v8, scale, zp, order[0].to(torch.int64), (n2, n4, n8)


def pack_k_mixed(K: Tensor, k_bits: Tensor, *, sub_2_target: Optional[int] = None,
                 sub_4_target: Optional[int] = None, n_ch_8_target: Optional[int] = None,
                 segment_counts: Optional[Tuple[int, int, int]] = None):
    """Per-channel mixed-precision K packing with one bit map for all heads
    (reference: obkv_accel/packing.py:177-391).  K [1,H,T,D] fp16, k_bits [D] in
    {0,2,4,8,16} (0 pruned, 16 packed as 8).

    Returns (K_2bit, K_4bit, K_8bit, K_ch_scale, K_ch_zp, ch_sort_idx,
    ch_perm_padded_idx, (N_ch_2, N_ch_4, N_ch_8)).
    """
    K = _as_fp16_rows(K, "K")
    H, T, D = K.shape[1], K.shape[2], K.shape[3]
    if T == 0:
        raise ValueError("pack_k_mixed needs at least one token row")
    ch_order, ch_counts = partition_by_bits(k_bits.reshape(1, -1).to(K.device), 1)
    if segment_counts is None:
        n2, n4, n8 = (int(c) for c in ch_counts[0, :3].tolist())
    else:
        n2, n4, n8 = map(int, segment_counts)
    n2p = 4 * int(sub_2_target) if sub_2_target is not None else _pad_to(n2, 4)
    n4p = 2 * int(sub_4_target) if sub_4_target is not None else _pad_to(n4, 2)
    n8o = int(n_ch_8_target) if n_ch_8_target is not None else n8
    assert n2p >= _pad_to(n2, 4), f"sub_2_target={sub_2_target} too small for N_ch_2={n2}"
    assert n4p >= _pad_to(n4, 2), f"sub_4_target={sub_4_target} too small for N_ch_4={n4}"
    assert n8o >= n8, f"n_ch_8_target={n_ch_8_target} < N_ch_8={n8}"
    k2, k4, k8, scale, zp, sort_idx, perm, _, _ = _launch_pack_k(
        K, None, 0, None, 0, T, T, ch_order, 0, ch_counts, 0, n2p, n4p, n8o, n2 + n4 + n8, 0)
    return k2, k4, k8, scale, zp, sort_idx[0].contiguous(), perm[0].contiguous(), (n2, n4, n8)


pack_k_mixed_single_head = pack_k_mixed


def _pack_k_per_head(K: Tensor, tok_order, tok_counts, max_t_v: int, t_k: int, ch_order: Tensor,
                     ch_counts: Tensor, ch_host: Sequence[Sequence[int]], gqa: int):
    """Shared-max channel layout over per-head bit maps; ``ch_host`` = host copy of the counts."""
    m2 = max(r[0] for r in ch_host)
    m4 = max(r[1] for r in ch_host)
    m8 = max(r[2] for r in ch_host)
    d_kept_max = max(r[0] + r[1] + r[2] for r in ch_host)
    n2p, n4p = _pad_to(m2, 4), _pad_to(m4, 2)
    tok_rs = tok_order.stride(0) if tok_order is not None else 0
    res = _launch_pack_k(K, tok_order, tok_rs, tok_counts, 4 if tok_counts is not None else 0, max_t_v, t_k,
                         ch_order, ch_order.stride(0), ch_counts, 4, n2p, n4p, m8, d_kept_max, gqa)
    return res, (m2, m4, m8)


def pack_k_mixed_per_head(K: Tensor, k_bits_ph: Tensor):
    """Per-head K bit maps packed to a shared-max channel layout
    (reference: obkv_accel/packing.py:399-578).  K [1,H,T,D] fp16, k_bits_ph [H,D].

    Returns the 9-tuple (K_2bit, K_4bit, K_8bit, K_ch_scale, K_ch_zp,
    K_ch_sort_idx_per_head, K_ch_perm_padded_idx_per_head,
    K_ch_seg_bounds_per_head, (max_N_ch_2, max_N_ch_4, max_N_ch_8)).
    """
    K = _as_fp16_rows(K, "K")
    H, T = K.shape[1], K.shape[2]
    assert k_bits_ph.dim() == 2 and k_bits_ph.shape[0] == H, (
        f"k_bits_ph must be [H_kv={H}, D], got {tuple(k_bits_ph.shape)}")
    if T == 0:
        raise ValueError("pack_k_mixed_per_head needs at least one token row")
    ch_order, ch_counts = partition_by_bits(k_bits_ph.to(K.device), 1)
    ch_host = ch_counts.cpu().tolist()
    (k2, k4, k8, scale, zp, sort_idx, perm, _, seg_bounds), mx = _pack_k_per_head(
        K, None, None, T, T, ch_order, ch_counts, ch_host, 0)
    return k2, k4, k8, scale, zp, sort_idx, perm, seg_bounds, mx


def _empty_packed_layer(H_kv: int, D: int, device, dtype) -> PackedKVLayer:
    e_v = torch.empty(1, H_kv, 0, 1, dtype=dtype, device=device)
    e_k = torch.empty(1, H_kv, 1, 0, dtype=dtype, device=device)
    e_i = torch.empty(0, dtype=torch.long, device=device)
    return PackedKVLayer(None, None, None, e_k, e_k.clone(), e_i, (0, 0, 0), e_i.clone(),
                         None, None, None, e_v, e_v.clone(), e_i.clone(), (0, 0, 0), 0)


def _softmax_mask(t_v: Tensor, n16: Tensor, max_t_v: int, t_k: int, gqa: int) -> Tensor:
    """Additive fp32 mask [H_q, t_k]: 0 on a head's live rows, -inf on stripe padding
    (reference: obkv_accel/packing.py:1236-1257)."""
    col = torch.arange(t_k, device=t_v.device).view(1, -1)
    live = (col < t_v.view(-1, 1)) | ((col >= max_t_v) & (col < max_t_v + n16.view(-1, 1)))
    mask = torch.zeros(live.shape, dtype=torch.float32, device=t_v.device)
    mask.masked_fill_(~live, float("-inf"))
    return mask.repeat_interleave(gqa, dim=0).contiguous()


def pack_kv(K: Tensor, V: Tensor, v_bits: Tensor, k_bits: Tensor, gqa_factor: int, *,
            build_mask: bool = True, retain_allocation_metadata: bool = False
            ) -> Tuple[PackedKVLayer, Optional[Tensor]]:
    """Select, quantise and pack one layer in the per-head stripe layout.

    The composite the reference runs per layer after bit allocation
    (obkv_fast.py:1098-1166: per-head ``build_packed_layer`` with deferred K, then
    ``_pad_and_stack_per_head_layers``), as one device pass with a single host
    read of the segment counts.

    K, V [1,H_kv,T,D] fp16; v_bits [H_kv,T] in {0,2,4,8,16} (0 evicted, 16 kept
    fp16); k_bits [H_kv,D] in {0,2,4,8,16}.  Returns (PackedKVLayer, new_v_only
    [1,H_kv,max_n_v16,D] fp16 or None).
    """
    K = _as_fp16_rows(K, "K")
    V = _as_fp16_rows(V, "V")
    H, T, D = K.shape[1], K.shape[2], K.shape[3]
    dev = K.device
    if tuple(v_bits.shape) != (H, T) or tuple(k_bits.shape) != (H, D):
        raise ValueError(f"v_bits must be [{H},{T}] and k_bits [{H},{D}]")
    tok_order, tok_counts = partition_by_bits(v_bits.to(dev), 0)
    ch_order, ch_counts = partition_by_bits(k_bits.to(dev), 1)
    host = torch.cat([tok_counts, ch_counts], dim=0).cpu().tolist()        # the one host read
    tok_host, ch_host = host[:H], host[H:]
    mx = [max(r[i] for r in tok_host) for i in range(4)]
    t_v_h = [r[0] + r[1] + r[2] for r in tok_host]
    max_t_v, max_n16 = max(t_v_h), mx[3]
    t_k = max_t_v + max_n16
    if t_k == 0:
        raise RuntimeError("pack_kv: every head kept zero tokens")
    v2, v4, v8, v16, v_scale, v_zp = _launch_pack_v(V, tok_order, tok_order.stride(0), tok_counts, 4, 0, 0,
                                                    mx, max_t_v)
    (k2, k4, k8, k_scale, k_zp, sort_ph, perm_ph, perm_q, seg_ch), ch_mx = _pack_k_per_head(
        K, tok_order, tok_counts, max_t_v, t_k, ch_order, ch_counts, ch_host, gqa_factor)
    t_v = tok_counts[:, :3].sum(dim=1).to(torch.int32)
    n16 = tok_counts[:, 3].contiguous()
    # legacy single-head field: V sort order of the first non-empty head, as ranks inside
    # that head's compressed-token list
    h0 = next((h for h in range(H) if t_v_h[h] + tok_host[h][3] > 0), 0)
    is_comp = (v_bits[h0].to(dev) > 0) & (v_bits[h0].to(dev) != 16)
    rank = torch.cumsum(is_comp.to(torch.int64), 0) - 1
    sort_idx = rank[tok_order[h0, :t_v_h[h0]].to(torch.int64)]
    layer = PackedKVLayer(
        K_2bit=k2, K_4bit=k4, K_8bit=k8, K_ch_scale=k_scale, K_ch_zp=k_zp,
        K_ch_sort_idx=sort_ph[0], K_ch_seg_bounds=ch_mx, K_ch_perm_padded_idx=perm_ph[0],
        V_2bit=v2, V_4bit=v4, V_8bit=v8, V_scale=v_scale, V_zp=v_zp, sort_idx=sort_idx,
        seg_bounds=(mx[0], mx[1], mx[2]), T_eff=max_t_v,
        seg_bounds_per_head=tok_counts[:, :3].contiguous(), T_eff_per_head=t_v,
        softmax_mask=_softmax_mask(t_v, n16, max_t_v, t_k, gqa_factor) if build_mask else None,
        K_ch_sort_idx_per_head=sort_ph, K_ch_perm_padded_idx_per_head=perm_ph,
        K_ch_seg_bounds_per_head=seg_ch, K_ch_perm_padded_idx_for_Q=perm_q,
        T_eff_k=t_k, n_v16=max_n16, T_eff_k_per_head=(t_v + n16).to(torch.int32), n_v16_per_head=n16,
        allocation_v_bits=v_bits.to(device=dev, dtype=torch.int16) if retain_allocation_metadata else None,
        allocation_k_bits=k_bits.to(device=dev, dtype=torch.int16) if retain_allocation_metadata else None,
    )
    return layer, v16


class PackedLayerBatch:
    """Result of :func:`pack_kv_layers`: every layer of a cache packed in one pass.

    The packed bytes of all layers live in a few tall tensors (one per field, leading
    dimension = layer); ``batch[i]`` / ``batch.layer(i)`` gives layer ``i`` as the
    ``(PackedKVLayer, new_v_only)`` pair :func:`pack_kv` would have returned, made of
    views into them (same shapes, same bytes; the views are strided along the head axis
    when another layer needed more rows).
    """

    def __init__(self, n_layers: int):
        self.n_layers = n_layers
        self._cache: dict = {}
        self._make = None

    def __len__(self) -> int:
        return self.n_layers

    def layer(self, i: int) -> Tuple[PackedKVLayer, Optional[Tensor]]:
        if not 0 <= i < self.n_layers:
            raise IndexError(i)
        if i not in self._cache:
            self._cache[i] = self._make(i)
        return self._cache[i]

    __getitem__ = layer

    def __iter__(self):
        return (self.layer(i) for i in range(self.n_layers))


def select_and_pack(K: Tensor, V: Tensor, layer_scores: Tensor, channel_scores: Tensor, *, gqa_factor: int,
                    token_budget: int, k_budget_ratio: float, obs_window: int = 0, pool_kernel_size: int = 5,
                    pool_padding: str = "reflect", pool_type: str = "avg", v_bit_options: Optional[Tensor] = None,
                    k_bit_options: Optional[Tensor] = None, eps_V: Optional[dict] = None,
                    eps_K: Optional[dict] = None, build_mask: bool = True,
                    retain_allocation_metadata: bool = False) -> Tuple[PackedKVLayer, Optional[Tensor], int]:
    """One layer of the prefill: pool the token scores, allocate V bits per head, derive every head's
    K budget from the tokens it kept, allocate K bits, drop the evicted channels and pack — the
    reference's per-layer composite ``_perhead_select_and_pack_joint`` (obkv_fast.py:899-1186) with
    its arguments and its return ``(packed_layer, new_v_only, T_eff)``.

    K, V [1,H_kv,T,D] fp16, layer_scores [H_kv,T], channel_scores [H_kv,D], all on the GPU.
    Everything stays on the device: the only host read is the one of the segment counts inside
    :func:`pack_kv` (the reference reads them too: the shared-max bounds are Python ints).
    ``obs_window`` is accepted for signature compatibility (unused, as in the reference);
    ``retain_allocation_metadata`` keeps the allocator's decisions on the layer
    (``allocation_v_bits`` / ``allocation_k_bits``), as the blockwise decoder's accounting wants.
    """
    from .knapsack_solver import (DEFAULT_EPSILON_K, DEFAULT_EPSILON_V, k_average_bits_per_head,
                                  knapsack_bit_allocation_batched, v_average_bits)
    from .scoring import apply_score_pooling
    assert K.dim() == 4 and V.dim() == 4, f"K/V must be [1,H_kv,T,D], got {tuple(K.shape)}/{tuple(V.shape)}"
    assert layer_scores.dim() == 2, f"layer_scores must be [H_kv,T], got {tuple(layer_scores.shape)}"
    assert channel_scores.dim() == 2, f"channel_scores must be [H_kv, D], got {tuple(channel_scores.shape)}"
    require_cuda(K, "K"); require_cuda(layer_scores, "layer_scores"); require_cuda(channel_scores, "channel_scores")
    H_kv, T = int(layer_scores.shape[0]), int(layer_scores.shape[1])
    head_dim = int(K.shape[3])
    pooled = (apply_score_pooling(layer_scores, pool_type, pool_kernel_size, pool_padding)
              if pool_kernel_size > 1 else layer_scores).float()
    v_bits = knapsack_bit_allocation_batched(
        pooled, v_average_bits(token_budget, head_dim, T, k_budget_ratio),
        epsilon=DEFAULT_EPSILON_V if eps_V is None else eps_V, bit_options=v_bit_options)       # [H_kv,T]
    kept = (v_bits > 0).sum(dim=1)                                                               # stays on the device
    k_bits = knapsack_bit_allocation_batched(
        channel_scores.float(), k_average_bits_per_head(token_budget, head_dim, k_budget_ratio, kept),
        epsilon=DEFAULT_EPSILON_K if eps_K is None else eps_K, bit_options=k_bit_options)       # [H_kv,D]
    K = torch.where((k_bits == 0)[None, :, None, :], torch.zeros_like(K), K)                   # evicted channels
    layer, new_v_only = pack_kv(K, V, v_bits, k_bits, gqa_factor, build_mask=build_mask,
                                retain_allocation_metadata=retain_allocation_metadata)
    return layer, new_v_only, int(layer.T_eff)


_PACK_JOB_DTYPE = None


def _pack_job_dtype():
    """numpy record type with the layout of ``rdkv_pack_job`` (built once)."""
    global _PACK_JOB_DTYPE
    if _PACK_JOB_DTYPE is None:
        _PACK_JOB_DTYPE = np.dtype(_lib.PackJob)
    return _PACK_JOB_DTYPE


def pack_kv_layers(Ks: Sequence[Tensor], Vs: Sequence[Tensor], v_bits: Tensor, k_bits: Tensor, gqa_factor: int, *,
                   build_mask: bool = True, launch_events: Optional[list] = None,
                   k_passes: int = 0) -> PackedLayerBatch:
    """:func:`pack_kv` for all layers of a cache at once (the reference packs a prefilled
    cache layer by layer: obkv_accel/packing.py:1323-1421, obkv_fast.py:1098-1166).

    Ks, Vs: per-layer [1,H_kv,T,D] fp16 tensors; v_bits [L,H_kv,T], k_bits [L,H_kv,D] in
    {0,2,4,8,16}.  Two partition launches, ONE host read of all segment counts, three
    packing launches whose third grid dimension is the layer.  Layer ``i`` of the result
    is bit-identical to ``pack_kv(Ks[i], Vs[i], v_bits[i], k_bits[i], gqa_factor)``.
    Layers whose K bit maps lead to different padded channel widths cannot share tall
    tensors; they are then packed one by one.  ``launch_events``: a list that receives two
    (start, end) pairs of CUDA events per call, around the two partition launches and around
    the packing launches (for measurements).  ``k_passes``: 1 = K packed in one pass over the kept
    rows (held in the shared memory of a cluster of CTAs; raises if they do not fit), 3 = in three
    (the rows are read twice), 0 = one pass where it fits; the bytes are the same.
    """
    import ctypes as C
    from ._lib import PackJob
    L = len(Ks)
    if L == 0 or len(Vs) != L:
        raise ValueError("pack_kv_layers needs as many V as K tensors, at least one")
    Ks = [_as_fp16_rows(k, "K") for k in Ks]
    Vs = [_as_fp16_rows(v, "V") for v in Vs]
    H, T, D = Ks[0].shape[1], Ks[0].shape[2], Ks[0].shape[3]
    dev = Ks[0].device
    if any(tuple(k.shape) != (1, H, T, D) for k in Ks) or any(tuple(v.shape) != (1, H, T, D) for v in Vs):
        raise ValueError("every layer must have the same [1,H_kv,T,D] shape")
    if tuple(v_bits.shape) != (L, H, T) or tuple(k_bits.shape) != (L, H, D):
        raise ValueError(f"v_bits must be [{L},{H},{T}] and k_bits [{L},{H},{D}]")
    v_bits, k_bits = v_bits.to(dev), k_bits.to(dev)
    if launch_events is not None:
        pev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        pev[0].record()
    tok_order, tok_counts = partition_by_bits(v_bits.reshape(L * H, T), 0, fill=False)   # (read through the counts only)
    ch_order, ch_counts = partition_by_bits(k_bits.reshape(L * H, D), 1, fill=False)
    if launch_events is not None:
        pev[1].record()
        launch_events.append(pev)
    host = torch.cat([tok_counts, ch_counts], dim=0).cpu().numpy()          # the one host read
    tok_h = host[:L * H].reshape(L, H, 4)
    ch_h = host[L * H:].reshape(L, H, 4)
    mx = tok_h.max(axis=1)                                                   # [L,4] per-layer segment maxima
    t_v_h = tok_h[:, :, :3].sum(axis=2)                                      # [L,H]
    max_t_v = t_v_h.max(axis=1)
    t_k = max_t_v + mx[:, 3]
    if int(t_k.min()) == 0:
        raise RuntimeError("pack_kv_layers: a layer kept zero tokens in every head")
    cm = ch_h[:, :, :3].max(axis=1)                                          # [L,3]
    n2p = (cm[:, 0] + 3) // 4 * 4
    n4p = (cm[:, 1] + 1) // 2 * 2
    n8p = cm[:, 2]
    dk = ch_h[:, :, :3].sum(axis=2).max(axis=1)
    batch = PackedLayerBatch(L)
    uniform = (n2p == n2p[0]).all() and (n4p == n4p[0]).all() and (n8p == n8p[0]).all() and (dk == dk[0]).all()
    if not uniform or int(n2p[0] + n4p[0] + n8p[0]) == 0:
        done = [pack_kv(Ks[i], Vs[i], v_bits[i], k_bits[i], gqa_factor, build_mask=build_mask) for i in range(L)]
        batch._make = lambda i: done[i]
        return batch
    N2P, N4P, N8P, DK = int(n2p[0]), int(n4p[0]), int(n8p[0]), int(dk[0])
    d_pad = N2P + N4P + N8P
    R2, R4, R8, R16 = (int(x) for x in mx.max(axis=0))
    RM, RK = int(max_t_v.max()), int(t_k.max())
    u8 = dict(dtype=torch.uint8, device=dev)
    f16 = dict(dtype=torch.float16, device=dev)
    i64 = dict(dtype=torch.int64, device=dev)
    V2 = torch.empty((L, H, R2, D // 4), **u8) if R2 else None
    V4 = torch.empty((L, H, R4, D // 2), **u8) if R4 else None
    V8 = torch.empty((L, H, R8, D), **u8) if R8 else None
    V16 = torch.empty((L, H, R16, D), **f16) if R16 else None
    VS = torch.empty((L, H, max(RM, 1), 1), **f16)
    VZ = torch.empty_like(VS)
    K2 = torch.empty((L, H, RK, N2P // 4), **u8) if N2P else None
    K4 = torch.empty((L, H, RK, N4P // 2), **u8) if N4P else None
    K8 = torch.empty((L, H, RK, N8P), **u8) if N8P else None
    KS = torch.empty((L, H, 1, d_pad), **f16)
    KZ = torch.empty_like(KS)
    SORT = torch.empty((L, H, DK), **i64)
    PERM = torch.empty((L, H, d_pad), **i64)
    PERMQ = torch.empty((L, H * gqa_factor, d_pad), **i64)
    SEG = torch.empty((L, H, 3), dtype=torch.int32, device=dev)
    slabs = [lib().rdkv_pack_k_slabs(int(x)) for x in t_k]
    max_slabs = max(slabs)
    SCR = torch.empty((L, H * max_slabs * 2 * d_pad), dtype=torch.float32, device=dev)

    # base address and per-layer byte stride of every tall tensor, read once
    def span(t: Optional[Tensor]):
        return (0, 0) if t is None else (t.data_ptr(), t.stride(0) * t.element_size())

    outs = {"v2": span(V2), "v4": span(V4), "v8": span(V8), "v16": span(V16), "v_scale": span(VS), "v_zp": span(VZ),
            "k2": span(K2), "k4": span(K4), "k8": span(K8), "k_scale": span(KS), "k_zp": span(KZ),
            "sort_idx": span(SORT), "perm": span(PERM), "perm_q": span(PERMQ), "seg_bounds": span(SEG),
            "scratch": span(SCR)}
    to_p, tc_p, co_p, cc_p = tok_order.data_ptr(), tok_counts.data_ptr(), ch_order.data_ptr(), ch_counts.data_ptr()
    # the job table, column by column (a numpy record array with the layout of rdkv_pack_job)
    jobs = np.zeros(L, dtype=_pack_job_dtype())
    layer_idx = np.arange(L, dtype=np.int64)
    jobs["K"], jobs["V"] = [k.data_ptr() for k in Ks], [v.data_ptr() for v in Vs]
    jobs["k_head_stride"], jobs["k_row_stride"] = [k.stride(1) for k in Ks], [k.stride(2) for k in Ks]
    jobs["v_head_stride"], jobs["v_row_stride"] = [v.stride(1) for v in Vs], [v.stride(2) for v in Vs]
    jobs["tok_order"], jobs["tok_counts"] = to_p + layer_idx * (H * T * 4), tc_p + layer_idx * (H * 16)
    jobs["ch_order"], jobs["ch_counts"] = co_p + layer_idx * (H * D * 4), cc_p + layer_idx * (H * 16)
    jobs["tok_order_row_stride"], jobs["ch_order_row_stride"] = T, D
    jobs["D"], jobs["gqa"] = D, gqa_factor
    jobs["max_n2"], jobs["max_n4"], jobs["max_n8"], jobs["max_n16"] = mx[:, 0], mx[:, 1], mx[:, 2], mx[:, 3]
    jobs["max_t_v"], jobs["t_k"] = max_t_v, t_k
    jobs["rows2"], jobs["rows4"], jobs["rows8"], jobs["rows16"] = R2, R4, R8, R16
    jobs["rows_meta"], jobs["rows_k"] = max(RM, 1), RK
    jobs["n_ch2_pad"], jobs["n_ch4_pad"], jobs["n_ch8"], jobs["d_kept_max"] = N2P, N4P, N8P, DK
    for name, (p0, step) in outs.items():
        if p0:
            jobs[name] = p0 + layer_idx * step
    jobs_host = torch.from_numpy(jobs.view(np.uint8))
    jobs_dev = jobs_host.to(dev)
    if launch_events is not None:
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        ev[0].record()
    check(lib().rdkv_pack_kv_batched(jobs_dev.data_ptr(), L, H, D, int(mx.sum(axis=1).max()), RK, d_pad,
                                     int(k_passes), N2P // 4 + (N4P // 2 + 1) // 2 + (N8P + 3) // 4, stream_ptr(dev)),
          "rdkv_pack_kv_batched")
    if launch_events is not None:
        ev[1].record()
        launch_events.append(ev)
    keep = (jobs_dev, jobs_host, Ks, Vs, SCR)                                # alive until the kernels have run

    def make(i: int) -> Tuple[PackedKVLayer, Optional[Tensor]]:
        _ = keep
        m2, m4, m8, m16 = (int(x) for x in mx[i])
        tv, tk = int(max_t_v[i]), int(t_k[i])

        def cut(t: Optional[Tensor], rows: int) -> Optional[Tensor]:
            return None if (t is None or rows == 0) else t[i:i + 1, :, :rows]

        cnt = tok_counts[i * H:(i + 1) * H]
        t_v = cnt[:, :3].sum(dim=1).to(torch.int32)
        n16 = cnt[:, 3].contiguous()
        order_i = tok_order[i * H:(i + 1) * H]
        h0 = next((h for h in range(H) if int(t_v_h[i, h]) + int(tok_h[i, h, 3]) > 0), 0)
        is_comp = (v_bits[i, h0] > 0) & (v_bits[i, h0] != 16)
        rank = torch.cumsum(is_comp.to(torch.int64), 0) - 1
        sort_idx = rank[order_i[h0, :int(t_v_h[i, h0])].to(torch.int64)]
        layer = PackedKVLayer(
            K_2bit=cut(K2, tk), K_4bit=cut(K4, tk), K_8bit=cut(K8, tk), K_ch_scale=KS[i:i + 1], K_ch_zp=KZ[i:i + 1],
            K_ch_sort_idx=SORT[i, 0], K_ch_seg_bounds=(int(cm[i, 0]), int(cm[i, 1]), int(cm[i, 2])),
            K_ch_perm_padded_idx=PERM[i, 0],
            V_2bit=cut(V2, m2), V_4bit=cut(V4, m4), V_8bit=cut(V8, m8), V_scale=VS[i:i + 1, :, :tv], V_zp=VZ[i:i + 1, :, :tv],
            sort_idx=sort_idx, seg_bounds=(m2, m4, m8), T_eff=tv,
            seg_bounds_per_head=cnt[:, :3].contiguous(), T_eff_per_head=t_v,
            softmax_mask=_softmax_mask(t_v, n16, tv, tk, gqa_factor) if build_mask else None,
            K_ch_sort_idx_per_head=SORT[i], K_ch_perm_padded_idx_per_head=PERM[i],
            K_ch_seg_bounds_per_head=SEG[i], K_ch_perm_padded_idx_for_Q=PERMQ[i],
            T_eff_k=tk, n_v16=m16, T_eff_k_per_head=(t_v + n16).to(torch.int32), n_v16_per_head=n16,
        )
        return layer, cut(V16, m16)

    batch._make = make
    return batch


def build_packed_layer(K: Tensor, V: Tensor, v_bits: Tensor, k_bits: Tensor, *,
                       gqa_factor: Optional[int] = None,
                       v_segment_counts: Optional[Tuple[int, int, int]] = None,
                       defer_k_for_per_head_stack: bool = False
                       ) -> Tuple[PackedKVLayer, int, Optional[Tensor]]:
    """Pack one layer whose heads share one token bit map
    (reference: obkv_accel/packing.py:801-1013).

    K, V [1,H_kv,T,D] fp16; v_bits [T] in {0,2,4,8,16}; k_bits [D] (shared) or
    [H_kv,D] (per head, needs gqa_factor).  K rows are laid out as [compressed
    tokens in V segment order ; fp16-V tokens ascending].  Returns
    (PackedKVLayer, T_eff_k, v16_V).
    """
    K = _as_fp16_rows(K, "K")
    V = _as_fp16_rows(V, "V")
    H, T, D = K.shape[1], K.shape[2], K.shape[3]
    dev = K.device
    v_bits = v_bits.to(dev)
    tok_order, tok_counts = partition_by_bits(v_bits.reshape(1, -1), 0)
    n2, n4, n8, n16 = (int(c) for c in tok_counts[0].tolist())
    if v_segment_counts is not None:
        assert tuple(map(int, v_segment_counts)) == (n2, n4, n8), (
            f"Segment sizes {tuple(v_segment_counts)} != counted {(n2, n4, n8)}")
    t_v = n2 + n4 + n8
    t_k = t_v + n16
    if t_k == 0:
        return _empty_packed_layer(H, D, dev, torch.float16), 0, None
    v2, v4, v8, v16, v_scale, v_zp = _launch_pack_v(V, tok_order, 0, tok_counts, 0, 0, 0, (n2, n4, n8, n16), t_v)
    is_comp = (v_bits > 0) & (v_bits != 16)
    rank = torch.cumsum(is_comp.to(torch.int64), 0) - 1
    sort_idx = rank[tok_order[0, :t_v].to(torch.int64)]
    common = dict(V_2bit=v2, V_4bit=v4, V_8bit=v8, V_scale=v_scale, V_zp=v_zp, sort_idx=sort_idx,
                  seg_bounds=(n2, n4, n8), T_eff=t_v, T_eff_k=t_k, n_v16=n16)
    e_k = torch.empty(1, H, 1, 0, dtype=torch.float16, device=dev)
    e_i = torch.empty(0, dtype=torch.long, device=dev)
    if defer_k_for_per_head_stack:
        if k_bits.dim() != 1 or H != 1:
            raise ValueError("deferred K packing expects one head and 1-D k_bits")
        rows = K.index_select(2, tok_order[0, :t_k].to(torch.int64)).contiguous()
        packed = PackedKVLayer(None, None, None, e_k, e_k.clone(), e_i, (0, 0, 0), e_i.clone(),
                               deferred_k_for_stack=rows, **common)
        return packed, t_k, v16
    k_bits = k_bits.to(dev)
    if k_bits.dim() == 2:
        assert tuple(k_bits.shape) == (H, D), f"k_bits 2D must be [H_kv={H}, D={D}], got {tuple(k_bits.shape)}"
        assert gqa_factor is not None, "build_packed_layer: gqa_factor is required when k_bits is 2D (per-head)"
        ch_order, ch_counts = partition_by_bits(k_bits, 1)
        ch_host = ch_counts.cpu().tolist()
        (k2, k4, k8, k_scale, k_zp, sort_ph, perm_ph, perm_q, seg_ch), ch_mx = _pack_k_per_head(
            K, tok_order.expand(H, -1), tok_counts.expand(H, -1).contiguous(), t_v, t_k, ch_order, ch_counts,
            ch_host, int(gqa_factor))
        packed = PackedKVLayer(k2, k4, k8, k_scale, k_zp, sort_ph[0], ch_mx, perm_ph[0],
                               K_ch_sort_idx_per_head=sort_ph, K_ch_perm_padded_idx_per_head=perm_ph,
                               K_ch_seg_bounds_per_head=seg_ch, K_ch_perm_padded_idx_for_Q=perm_q, **common)
        return packed, t_k, v16
    ch_order, ch_counts = partition_by_bits(k_bits.reshape(1, -1), 1)
    c2, c4, c8 = (int(c) for c in ch_counts[0, :3].tolist())
    n2p, n4p = _pad_to(c2, 4), _pad_to(c4, 2)
    k2, k4, k8, k_scale, k_zp, sort_ph, perm_ph, _, _ = _launch_pack_k(
        K, tok_order, 0, tok_counts, 0, t_v, t_k, ch_order, 0, ch_counts, 0, n2p, n4p, c8, c2 + c4 + c8, 0)
    packed = PackedKVLayer(k2, k4, k8, k_scale, k_zp, sort_ph[0].contiguous(), (c2, c4, c8),
                           perm_ph[0].contiguous(), **common)
    return packed, t_k, v16


def _pad_and_stack_per_head_layers(layers: List[PackedKVLayer], per_head_v16_V: List[Optional[Tensor]],
                                   H_q: int, gqa_factor: int, head_dim: int, device, dtype, *,
                                   k_bits_per_head: Optional[Tensor] = None,
                                   v_bits_per_head: Optional[Tensor] = None,
                                   retain_allocation_metadata: bool = False
                                   ) -> Tuple[PackedKVLayer, Optional[Tensor]]:
    """Stack single-head layers (from ``build_packed_layer`` with deferred K) into the
    per-head stripe layout (reference: obkv_accel/packing.py:1019-1317).

    V segments, scale/zp and fp16 values are zero-padded to the per-layer maxima.
    With ``k_bits_per_head`` K is quantised once over the zero-padded stripe canvas
    ``[1,H_kv,max_T_v + max_n_v16,D]``, so pad rows take part in the per-channel range as
    they do in the reference.  Without it (the reference's shared layout: one K bit map
    for all heads, every inner layer carrying its own packed K) the inner layers' K
    bytes are copied into the stripe, their scales and zero points stacked, and the
    channel tables of the first non-empty head serve all heads.
    """
    H = len(layers)
    assert H_q == H * gqa_factor, f"H_q={H_q}, H_kv={H}, gqa={gqa_factor}"
    D = head_dim
    t_v_h = [int(pl.T_eff) for pl in layers]
    n16_h = [int(pl.n_v16) for pl in layers]
    seg_h = [tuple(int(x) for x in pl.seg_bounds) for pl in layers]
    max_t_v, max_n16 = max(t_v_h), max(n16_h)
    t_k = max_t_v + max_n16
    mx = tuple(max(s[i] for s in seg_h) for i in range(3))
    u8 = dict(dtype=torch.uint8, device=device)

    def stack(field: str, idx: int, width: int):
        if mx[idx] == 0:
            return None
        out = torch.zeros((1, H, mx[idx], width), **u8)
        for h, pl in enumerate(layers):
            if seg_h[h][idx]:
                out[0, h, :seg_h[h][idx]] = getattr(pl, field)[0, 0]
        return out

    v2, v4, v8 = stack("V_2bit", 0, D // 4), stack("V_4bit", 1, D // 2), stack("V_8bit", 2, D)
    v_scale = torch.zeros((1, H, max_t_v, 1), dtype=torch.float16, device=device)
    v_zp = torch.zeros_like(v_scale)
    canvas = torch.zeros((1, H, max(t_k, 1), D), dtype=torch.float16, device=device)[:, :, :t_k]
    new_v_only = torch.zeros((1, H, max_n16, D), dtype=torch.float16, device=device) if max_n16 else None
    for h, pl in enumerate(layers):
        if t_v_h[h]:
            v_scale[0, h, :t_v_h[h]] = pl.V_scale[0, 0]
            v_zp[0, h, :t_v_h[h]] = pl.V_zp[0, 0]
        if n16_h[h]:
            new_v_only[0, h, :n16_h[h]] = per_head_v16_V[h][0, 0]
    if t_k == 0:
        raise RuntimeError("every head kept zero tokens")
    ref_pl = next((pl for pl in layers if pl.T_eff_k > 0 or pl.T_eff > 0), layers[0])
    i32 = dict(dtype=torch.int32, device=device)
    t_v_t, n16_t = torch.tensor(t_v_h, **i32), torch.tensor(n16_h, **i32)
    if k_bits_per_head is None:
        # shared layout: copy every head's packed K rows ([compressed; fp16-V rows]) into the stripe
        n2c, n4c, n8c = (int(x) for x in ref_pl.K_ch_seg_bounds)
        d_pad = _pad_to(n2c, 4) + _pad_to(n4c, 2) + n8c

        def stack_k(field: str, width: int):
            if width == 0:
                return None
            out = torch.zeros((1, H, t_k, width), **u8)
            for h, pl in enumerate(layers):
                cur = getattr(pl, field)
                if cur is None:
                    continue
                if t_v_h[h]:
                    out[0, h, :t_v_h[h]] = cur[0, 0, :t_v_h[h]]
                if n16_h[h]:
                    out[0, h, max_t_v:max_t_v + n16_h[h]] = cur[0, 0, t_v_h[h]:t_v_h[h] + n16_h[h]]
            return out

        def stack_ch(field: str):
            parts = []
            for pl in layers:
                t = getattr(pl, field)
                parts.append(t if t.shape[3] == d_pad else torch.zeros((1, 1, 1, d_pad), dtype=torch.float16, device=device))
            return torch.cat(parts, dim=1).contiguous()

        packed = PackedKVLayer(
            K_2bit=stack_k("K_2bit", _pad_to(n2c, 4) // 4), K_4bit=stack_k("K_4bit", _pad_to(n4c, 2) // 2),
            K_8bit=stack_k("K_8bit", n8c), K_ch_scale=stack_ch("K_ch_scale"), K_ch_zp=stack_ch("K_ch_zp"),
            K_ch_sort_idx=ref_pl.K_ch_sort_idx, K_ch_seg_bounds=ref_pl.K_ch_seg_bounds,
            K_ch_perm_padded_idx=ref_pl.K_ch_perm_padded_idx,
            V_2bit=v2, V_4bit=v4, V_8bit=v8, V_scale=v_scale, V_zp=v_zp, sort_idx=ref_pl.sort_idx,
            seg_bounds=mx, T_eff=max_t_v, seg_bounds_per_head=torch.tensor(seg_h, **i32).view(H, 3),
            T_eff_per_head=t_v_t, softmax_mask=_softmax_mask(t_v_t, n16_t, max_t_v, t_k, gqa_factor),
            T_eff_k=t_k, n_v16=max_n16, T_eff_k_per_head=t_v_t + n16_t, n_v16_per_head=n16_t,
            allocation_v_bits=(v_bits_per_head.to(device=device, dtype=torch.int16)
                               if retain_allocation_metadata and v_bits_per_head is not None else None),
        )
        return packed, new_v_only
    for h, pl in enumerate(layers):
        if t_v_h[h] + n16_h[h] == 0:
            continue
        rows = pl.deferred_k_for_stack
        if rows is None:
            raise ValueError("inner layers must carry deferred_k_for_stack (defer_k_for_per_head_stack=True)")
        canvas[0, h, :t_v_h[h]] = rows[0, 0, :t_v_h[h]]
        if n16_h[h]:
            canvas[0, h, max_t_v:max_t_v + n16_h[h]] = rows[0, 0, t_v_h[h]:]
    k2, k4, k8, k_scale, k_zp, sort_ph, perm_ph, seg_ch, ch_mx = pack_k_mixed_per_head(
        canvas, k_bits_per_head.to(device))
    packed = PackedKVLayer(
        K_2bit=k2, K_4bit=k4, K_8bit=k8, K_ch_scale=k_scale, K_ch_zp=k_zp, K_ch_sort_idx=sort_ph[0],
        K_ch_seg_bounds=ch_mx, K_ch_perm_padded_idx=perm_ph[0],
        V_2bit=v2, V_4bit=v4, V_8bit=v8, V_scale=v_scale, V_zp=v_zp, sort_idx=ref_pl.sort_idx,
        seg_bounds=mx, T_eff=max_t_v, seg_bounds_per_head=torch.tensor(seg_h, **i32).view(H, 3),
        T_eff_per_head=t_v_t, softmax_mask=_softmax_mask(t_v_t, n16_t, max_t_v, t_k, gqa_factor),
        K_ch_sort_idx_per_head=sort_ph, K_ch_perm_padded_idx_per_head=perm_ph,
        K_ch_seg_bounds_per_head=seg_ch,
        K_ch_perm_padded_idx_for_Q=perm_ph.repeat_interleave(gqa_factor, dim=0),
        T_eff_k=t_k, n_v16=max_n16, T_eff_k_per_head=t_v_t + n16_t, n_v16_per_head=n16_t,
        allocation_v_bits=(v_bits_per_head.to(device=device, dtype=torch.int16)
                           if retain_allocation_metadata and v_bits_per_head is not None else None),
        allocation_k_bits=(k_bits_per_head.to(device=device, dtype=torch.int16)
                           if retain_allocation_metadata else None),
    )
    return packed, new_v_only


def build_packed_cache(past_key_values, v_bits: Tensor, k_bits: Tensor, *, original_seq_len: int,
                       gqa_factor: Optional[int] = None) -> TriZoneCache:
    """Pack every layer of an HF-style ``((K, V), ...)`` cache with one token bit map
    (reference: obkv_accel/packing.py:1323-1421).  k_bits: [D], [L,D], [H_kv,D] or
    [L,H_kv,D] with the reference's shape dispatch."""
    L = len(past_key_values)
    H = int(past_key_values[0][0].shape[1])
    if k_bits.dim() == 1:
        per_layer = False
    elif k_bits.dim() == 2:
        if k_bits.shape[0] == H and k_bits.shape[0] != L:
            per_layer = False
        elif k_bits.shape[0] == L:
            per_layer = True
        elif k_bits.shape[0] == H:
            per_layer = False
        else:
            raise ValueError(f"k_bits 2D shape {tuple(k_bits.shape)} matches neither num_layers={L} nor H_kv={H}")
    elif k_bits.dim() == 3:
        assert tuple(k_bits.shape[:2]) == (L, H), f"k_bits 3D must be [L={L}, H_kv={H}, D]"
        per_layer = True
    else:
        raise ValueError(f"k_bits must be 1D/2D/3D, got shape {tuple(k_bits.shape)}")
    packed, v16s = [], []
    for i, (K, V) in enumerate(past_key_values):
        layer, _, v16 = build_packed_layer(K, V, v_bits, k_bits[i] if per_layer else k_bits,
                                           gqa_factor=gqa_factor)
        packed.append(layer)
        v16s.append(v16)
    return TriZoneCache(tuple(packed), v16s, [None] * L, [None] * L, int(original_seq_len))


# ── kernel-facing view of a layer ────────────────────────────────────────────

def _squeeze_h(t: Optional[Tensor]) -> Optional[Tensor]:
    if t is not None and t.dim() == 4 and t.shape[0] == 1:
        return t[0]
    return t


def layer_identity(pl) -> tuple:
    """Identity of everything a cached ``rdkv_layer_view`` of this layer captures: address and
    shape of every tensor field it points into and the host scalars it copies.  A cache of views
    keyed by this notices a field that was re-assigned (a deferred K filled in later, a re-pack, a
    grown ``T_eff``); values rewritten in place keep the key, and are read by the kernels anyway."""
    def ident(t):
        return None if t is None else (t.data_ptr(), tuple(t.shape), tuple(t.stride()))
    tensors = tuple(ident(getattr(pl, f, None)) for f in (
        "K_2bit", "K_4bit", "K_8bit", "K_ch_scale", "K_ch_zp", "K_ch_perm_padded_idx_for_Q",
        "K_ch_perm_padded_idx_per_head", "K_ch_perm_padded_idx", "V_2bit", "V_4bit", "V_8bit", "V_scale", "V_zp",
        "seg_bounds_per_head", "n_v16_per_head", "softmax_mask"))
    scalars = (tuple(int(x) for x in pl.K_ch_seg_bounds), tuple(int(x) for x in pl.seg_bounds),
               int(pl.T_eff), int(pl.T_eff_k), int(pl.n_v16))
    return tensors + scalars


def layer_view(pl: PackedKVLayer, V16: Optional[Tensor] = None, n_v16_per_head: Optional[Tensor] = None,
               max_T_v: Optional[int] = None, *, use_mask: bool = False, t_k: Optional[int] = None
               ) -> Tuple[LayerView, list]:
    """Fill a ``rdkv_layer_view`` from a PackedKVLayer (+ optional Zone-B values).

    Accepts ``[1,H_kv,...]`` or squeezed ``[H_kv,...]`` fields, like the reference
    wrappers do (triton_k_kernel.py:1190-1200).  Returns the struct and the list of
    tensors it points into (keep them alive while the view is in use).
    """
    v = LayerView()
    keep = []

    def put(name, t, stride_name=None, stride_dim=0, bytes_=False, extent_name=None):
        t = _squeeze_h(t)
        if t is None or t.numel() == 0:
            setattr(v, name, None)
            if stride_name:
                setattr(v, stride_name, 0)
            return None
        require_cuda(t, name)
        if t.stride(-1) != 1:
            t = t.contiguous()
        keep.append(t)
        setattr(v, name, t.data_ptr())
        if stride_name:
            setattr(v, stride_name, t.stride(stride_dim) * (t.element_size() if bytes_ else 1))
        if extent_name:
            # last addressable byte + 1, relative to the base pointer
            last = sum((n - 1) * st for n, st in zip(t.shape, t.stride()))
            setattr(v, extent_name, (last + 1) * t.element_size())
        return t

    n2c, n4c, n8c = (int(x) for x in pl.K_ch_seg_bounds)
    v.n_ch2_pad, v.n_ch4_pad, v.n_ch8 = _pad_to(n2c, 4), _pad_to(n4c, 2), n8c
    put("k2", pl.K_2bit if v.n_ch2_pad else None, "k2_head_stride", 0, True, "k2_bytes")
    put("k4", pl.K_4bit if v.n_ch4_pad else None, "k4_head_stride", 0, True, "k4_bytes")
    put("k8", pl.K_8bit if v.n_ch8 else None, "k8_head_stride", 0, True, "k8_bytes")
    sc = _squeeze_h(pl.K_ch_scale)
    put("k_scale", sc.reshape(sc.shape[0], -1) if sc is not None and sc.numel() else None)
    zp = _squeeze_h(pl.K_ch_zp)
    put("k_zp", zp.reshape(zp.shape[0], -1) if zp is not None and zp.numel() else None)
    perm_q = pl.K_ch_perm_padded_idx_for_Q
    if perm_q is not None:
        H_kv = sc.shape[0]
        g = perm_q.shape[0] // H_kv
        put("k_perm", perm_q)
        v.k_perm_head_stride = g * perm_q.stride(0)
    elif pl.K_ch_perm_padded_idx_per_head is not None:
        put("k_perm", pl.K_ch_perm_padded_idx_per_head, "k_perm_head_stride", 0)
    else:
        put("k_perm", pl.K_ch_perm_padded_idx)
        v.k_perm_head_stride = 0
    put("v2", pl.V_2bit, "v2_head_stride", 0, True, "v2_bytes")
    put("v4", pl.V_4bit, "v4_head_stride", 0, True, "v4_bytes")
    put("v8", pl.V_8bit, "v8_head_stride", 0, True, "v8_bytes")
    vs = _squeeze_h(pl.V_scale)
    vz = _squeeze_h(pl.V_zp)
    put("v_scale", vs.reshape(vs.shape[0], -1) if vs.numel() else None, "v_meta_head_stride", 0, False,
        "v_meta_bytes")
    put("v_zp", vz.reshape(vz.shape[0], -1) if vz.numel() else None)
    if pl.seg_bounds_per_head is not None:
        sb = pl.seg_bounds_per_head
        if sb.dtype != torch.int32 or not sb.is_contiguous():
            sb = sb.to(torch.int32).contiguous()
        put("v_seg_bounds", sb)
    v.n2, v.n4, v.n8 = (int(x) for x in pl.seg_bounds)
    v.max_t_v = int(pl.T_eff if max_T_v is None else max_T_v)
    if V16 is not None and V16.numel() > 0:
        t = put("v16", V16, "v16_head_stride", 0, False, "v16_bytes")
        v.n_v16_shared = int(t.shape[-2])
        nv = n_v16_per_head if n_v16_per_head is not None else pl.n_v16_per_head
        if nv is not None:
            if nv.dtype != torch.int32 or not nv.is_contiguous():
                nv = nv.to(torch.int32).contiguous()
            put("n_v16", nv)
    if use_mask and pl.softmax_mask is not None and pl.softmax_mask.numel():
        put("mask", pl.softmax_mask, "mask_row_stride", 0)
    full = int(pl.T_eff_k) if pl.T_eff_k > 0 else int(pl.T_eff)
    v.t_k = int(full if t_k is None else t_k)
    return v, keep
