"""Fused packed-KV decode attention.

Replaces the attention block of the reference decode loop
(obkv_accel/fast_decode.py:1701-1784: K kernel -> mask add -> softmax -> V kernel)
with one split-sequence kernel launch over any number of (sequence, layer)
pairs followed by a log-sum-exp combine.  Softmax semantics are the
reference's: one softmax per query head over its live Zone-A and Zone-B rows;
stripe padding is excluded through the per-head row counts read on the device
(and through ``softmax_mask`` too when ``use_mask`` is set).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch
from torch import Tensor

from ._lib import HEAD_DIM, PARTIAL_STRIDE, LayerView, check, lib, ptr, q_dtype_tag, require_cuda, stream_ptr
from .packing import PackedKVLayer, layer_view


class DecodeTable:
    """Device-resident array of ``rdkv_layer_view`` records, one per (sequence, layer).

    The table holds references to every tensor it points into.  Per-head row
    counts stay in the layers' own int32 device tensors, so a caller may rewrite
    payloads and counts in place between launches.
    """

    def __init__(self, layers: Sequence[PackedKVLayer], new_v_only: Sequence[Optional[Tensor]], H_q: int,
                 *, use_mask: bool = False, device=None, n_chunks: Optional[int] = None,
                 k_only: bool = False):
        if len(layers) == 0:
            raise ValueError("DecodeTable needs at least one layer")
        if len(new_v_only) != len(layers):
            raise ValueError("new_v_only must have one entry per layer")
        sc = layers[0].K_ch_scale
        self.H_kv = int(sc.shape[1] if sc.dim() == 4 else sc.shape[0])
        self.H_q = int(H_q)
        if self.H_q % self.H_kv:
            raise ValueError(f"H_q={H_q} is not a multiple of H_kv={self.H_kv}")
        self.device = torch.device(device) if device is not None else layers[0].K_ch_scale.device
        self._keep: List = []
        self.source = list(zip(layers, new_v_only))
        views = (LayerView * len(layers))()
        max_t_k = 0
        for i, (pl, nv) in enumerate(zip(layers, new_v_only)):
            n2, n4, n8 = pl.K_ch_seg_bounds
            if n2 + n4 + n8 == 0 or n2 > 128 or n4 > 128 or n8 > 128:
                raise ValueError("layer has no kept K channels or more than 128 in a segment")
            if int(pl.n_v16) > 0 and nv is None and not k_only:
                raise ValueError(f"layer {i} has fp16 rows but no new_v_only tensor")
            v, keep = layer_view(pl, nv if (nv is not None and int(pl.n_v16) > 0) else None, use_mask=use_mask)
            views[i] = v
            self._keep.append(keep)
            max_t_k = max(max_t_k, int(v.t_k))
        self.n_views = len(layers)
        self.max_t_k = max_t_k
        self.k_row_bytes_max = max(
            sum(int(t.shape[-1]) for t in (pl.K_2bit, pl.K_4bit, pl.K_8bit) if t is not None) for pl in layers)
        for pl, nv in zip(layers, new_v_only):
            for t, align in ((pl.V_2bit, 4), (pl.V_4bit, 4), (pl.V_8bit, 4), (nv, 8)):
                if t is not None and t.numel() and t.data_ptr() % align:
                    raise ValueError(f"packed V tensors must be {align}-byte aligned")
        # uniform chunks of the partial-record calls: only when there are fewer units than CTA slots
        # (a chunk pays the per-CTA prologue and merge again; see unit_plan)
        n_hgrp = (self.H_q // self.H_kv + 7) // 8
        units = self.n_views * self.H_kv * n_hgrp
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        want = max(1, min(4, (self.CTAS_PER_SM * sms) // units))
        n_chunks = max(1, min(want if n_chunks is None else int(n_chunks), -(-max(max_t_k, 1) // 128)))
        self.chunk_rows = max(64, ((-(-max(max_t_k, 1) // n_chunks) + 63) // 64) * 64)
        self.n_chunks = max(1, -(-max(max_t_k, 1) // self.chunk_rows))
        raw = bytes(views)
        host = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
        self.views = host.to(self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._partials: Optional[Tensor] = None
        self.unit_rows = ((max(max_t_k, 1) + 63) // 64) * 64
        self._sms = sms
        self._n_hgrp = n_hgrp

    CTAS_PER_SM = 3                      # resident CTAs of the fused kernel per SM

    def unit_plan(self, n_views: int):
        """(v_main, k, rows): of a launch over ``n_views`` views the first ``v_main`` views run one CTA
        per unit, the units of the remaining views are cut into ``k`` uniform chunks of ``rows`` rows.
        Measured on B200: a CTA per whole unit is the most efficient shape (a chunk pays the per-CTA
        prologue and merge again), so units are cut — all of them, uniformly — only when there are
        fewer units than CTA slots.  Tried and dropped: cutting just the units of a mostly empty last
        wave (on a stream of lower priority), and equal segments of one flat row axis over all units
        with a loop over items in the CTA — both slower than the idle tail they remove."""
        slots = self._sms * self.CTAS_PER_SM
        hy = self.H_kv * self._n_hgrp
        units = n_views * hy
        k_max = max(1, min(4, self.unit_rows // 256))
        if units <= slots:
            k = max(1, min(k_max, slots // max(units, 1)))
            return (n_views, 1, self.unit_rows) if k == 1 else (0, k, self._chunk_rows_for(k))
        return n_views, 1, self.unit_rows

    def _chunk_rows_for(self, k: int) -> int:
        return max(64, ((-(-self.unit_rows // k) + 63) // 64) * 64)

    def chunk_workspace(self, k: int) -> Tensor:
        """Records of chunked units: [n_views*H_q, k, 132] fp32 (grown on demand)."""
        cache = self.__dict__.setdefault("_chunk_ws", {})
        if k not in cache:
            cache[k] = torch.empty((self.n_views * self.H_q, k, PARTIAL_STRIDE), dtype=torch.float32, device=self.device)
        return cache[k]

    def workspace(self) -> Optional[Tensor]:
        """Split-sequence partial records [n_views*H_q, n_chunks, 132] fp32 (allocated once);
        None when one chunk covers every head (results are written directly)."""
        if self.n_chunks == 1:
            return None
        if self._partials is None:
            self._partials = torch.empty((self.n_views * self.H_q, self.n_chunks, PARTIAL_STRIDE),
                                         dtype=torch.float32, device=self.device)
        return self._partials

    def check_status(self) -> None:
        """Host read (synchronises) of the kernel's status word; raises if a launch reported a problem."""
        st = int(self.status.item())
        if st:
            raise RuntimeError(f"rdkv_b200: fused decode kernel reported status {st} "
                               "(1 = staging wait ran out, 2 = a view did not fit the launch)")


def lse_combine(partials: Tensor, out: Optional[Tensor] = None, *, out_ml: Optional[Tensor] = None,
                out_partial: Optional[Tensor] = None) -> Optional[Tensor]:
    """Merge split-sequence records ``[n_rows, n_splits, 132]`` (m, l, -, -, o[128]) in
    split-index order.  Returns ``out [n_rows,128]`` fp32 (normalised); ``out_partial``
    ``[n_rows,132]`` receives the merged un-normalised record instead when given."""
    require_cuda(partials, "partials")
    if partials.dim() != 3 or partials.shape[2] != PARTIAL_STRIDE or partials.dtype != torch.float32:
        raise ValueError("partials must be float32 [n_rows, n_splits, 132]")
    if partials.stride(2) != 1:
        partials = partials.contiguous()
    n_rows, n_splits = partials.shape[0], partials.shape[1]
    if out is None and out_partial is None:
        out = torch.empty((n_rows, HEAD_DIM), dtype=torch.float32, device=partials.device)
    check(lib().rdkv_lse_combine(ptr(partials), n_rows, n_splits, partials.stride(0), partials.stride(1),
                                 ptr(out), ptr(out_ml), ptr(out_partial), stream_ptr(partials.device)),
          "rdkv_lse_combine")
    return out


def _launch_fused(q: Tensor, table: DecodeTable, partials: Optional[Tensor], out: Optional[Tensor],
                  v0: int = 0, v1: Optional[int] = None, n_chunks: Optional[int] = None,
                  chunk_rows: Optional[int] = None) -> None:
    """Launch the fused kernel on views [v0, v1) of the table (all of them by default) with uniform
    chunks (the table's, or the given ones); q, partials ([n_views*H_q, n_chunks, 132]) and out are
    the full-table tensors, the range is cut by pointer offsets.  ``out`` may be a pinned host
    tensor (device-addressable)."""
    require_cuda(q, "q")
    if q.shape[-1] != HEAD_DIM or q.numel() != table.n_views * table.H_q * HEAD_DIM:
        raise ValueError(f"q must be [{table.n_views},{table.H_q},{HEAD_DIM}], got {tuple(q.shape)}")
    if not q.is_contiguous():
        q = q.contiguous()
    v1 = table.n_views if v1 is None else v1
    if not 0 <= v0 <= v1 <= table.n_views:
        raise ValueError(f"view range [{v0},{v1}) outside the table of {table.n_views} views")
    rows = v0 * table.H_q                                  # first query-head row of the range

    def off(t: Optional[Tensor], per_row: int) -> Optional[int]:
        return None if t is None else t.data_ptr() + rows * per_row * t.element_size()

    n_chunks = table.n_chunks if n_chunks is None else n_chunks
    chunk_rows = table.chunk_rows if chunk_rows is None else chunk_rows
    check(lib().rdkv_decode_attn_partial(table.views.data_ptr() + v0 * C.sizeof(LayerView), v1 - v0,
                                         off(q, HEAD_DIM), q_dtype_tag(q), table.H_q,
                                         table.H_kv, chunk_rows, n_chunks, table.k_row_bytes_max,
                                         off(partials, n_chunks * PARTIAL_STRIDE), off(out, HEAD_DIM),
                                         ptr(table.status), stream_ptr(q.device)),
          "rdkv_decode_attn_partial")


def _launch_units(q: Tensor, table: DecodeTable, out: Tensor, v0: int = 0, v1: Optional[int] = None,
                  phases: int = 3) -> None:
    """One CTA per unit on views [v0, v1), or uniform chunks of every unit when there are fewer
    units than CTA slots (DecodeTable.unit_plan); chunk records are merged by the combine kernel.
    phases: 1 = fused launches, 2 = merge, 3 = both."""
    v1 = table.n_views if v1 is None else v1
    v_main, k, rows_k = table.unit_plan(v1 - v0)
    if phases & 1 and v_main > 0:
        _launch_fused(q, table, None, out, v0, v0 + v_main, 1, table.unit_rows)
    if v_main < v1 - v0:
        a = v0 + v_main
        if k == 1:
            if phases & 1:
                _launch_fused(q, table, None, out, a, v1, 1, table.unit_rows)
            return
        ws = table.chunk_workspace(k)
        if phases & 1:
            _launch_fused(q, table, ws, None, a, v1, k, rows_k)
        if phases & 2:
            rows = slice(a * table.H_q, v1 * table.H_q)
            check(lib().rdkv_lse_combine(ws[rows].data_ptr(), (v1 - a) * table.H_q, k, ws.stride(0), ws.stride(1),
                                         out.data_ptr() + a * table.H_q * HEAD_DIM * 4, None, None,
                                         stream_ptr(q.device)), "rdkv_lse_combine")



def decode_attention_phases(q: Tensor, table: DecodeTable, out: Tensor, *, phases: int = 3) -> Tensor:
    """The two phases of :func:`packed_decode_attention` separately (for measurements):
    ``phases=1`` runs the fused kernel alone, ``phases=2`` the merge of the records of split
    units / chunks (if the table's launch shape has any), 3 both."""
    _launch_units(q, table, out, phases=phases)
    return out


def decode_attention_partial(q: Tensor, table: DecodeTable, out: Optional[Tensor] = None) -> Tensor:
    """The fused kernel alone in uniform-chunk mode: returns the per-chunk records, or ``out``
    itself when a single chunk covers every head (the kernel then writes normalised results)."""
    if table.n_chunks == 1:
        if out is None:
            out = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=torch.float32, device=q.device)
        _launch_fused(q, table, None, out)
        return out
    part = table.workspace()
    _launch_fused(q, table, part, None)
    return part


def tail_attention_partial(q: Tensor, new_k: Tensor, new_v: Tensor, n_new, H_kv: int,
                           out_partial: Optional[Tensor] = None) -> Tensor:
    """(m, l, o) records of plain attention over the uncompressed tail (Zone C: tokens
    appended while decoding; reference obkv_accel/fast_decode.py:863-866, 1719-1784).

    q [n_views,H_q,128]; new_k, new_v [n_views,H_kv,cap,128] fp16/bf16/fp32 (same dtype and
    strides); n_new: live rows per head, an int or an int32 device tensor [n_views].
    Returns [n_views*H_q, 132] fp32 records for :func:`lse_combine`.
    """
    require_cuda(q, "q"); require_cuda(new_k, "new_k"); require_cuda(new_v, "new_v")
    if q.dim() != 3 or q.shape[-1] != HEAD_DIM:
        raise ValueError("q must be [n_views,H_q,128]")
    n_views, H_q = int(q.shape[0]), int(q.shape[1])
    if new_k.dim() != 4 or tuple(new_k.shape[:2]) != (n_views, H_kv) or new_k.shape[-1] != HEAD_DIM:
        raise ValueError(f"new_k must be [{n_views},{H_kv},cap,{HEAD_DIM}], got {tuple(new_k.shape)}")
    if new_v.shape != new_k.shape or new_v.dtype != new_k.dtype or new_v.stride() != new_k.stride():
        raise ValueError("new_v must match new_k in shape, dtype and strides")
    if new_k.stride(-1) != 1:
        raise ValueError("tail rows must be contiguous along the channel axis")
    if not q.is_contiguous():
        q = q.contiguous()
    cap = int(new_k.shape[2])
    per_view = None
    if isinstance(n_new, Tensor):
        require_cuda(n_new, "n_new")
        if n_new.dtype != torch.int32 or n_new.numel() != n_views or not n_new.is_contiguous():
            raise ValueError("n_new tensor must be contiguous int32 [n_views]")
        per_view, n_int = n_new, 0
    else:
        n_int = int(n_new)
        if not 0 <= n_int <= cap:
            raise ValueError(f"n_new={n_int} outside [0, {cap}]")
    if out_partial is None:
        out_partial = torch.empty((n_views * H_q, PARTIAL_STRIDE), dtype=torch.float32, device=q.device)
    check(lib().rdkv_tail_attn_partial(ptr(q), q_dtype_tag(q), n_views, H_q, H_kv, ptr(new_k), ptr(new_v),
                                       q_dtype_tag(new_k), new_k.stride(0), new_k.stride(1), new_k.stride(2),
                                       n_int, ptr(per_view), ptr(out_partial), stream_ptr(q.device)),
          "rdkv_tail_attn_partial")
    return out_partial


def packed_decode_attention(q: Tensor, table: DecodeTable, *, out: Optional[Tensor] = None,
                            out_partial: Optional[Tensor] = None, new_k: Optional[Tensor] = None,
                            new_v: Optional[Tensor] = None, n_new=0) -> Tensor:
    """softmax(q·K̂ᵀ/√128)·V̂ over every view of ``table``.

    q [n_views,H_q,128] fp16/bf16/fp32 -> out [n_views,H_q,128] fp32.  With
    ``out_partial`` ([n_views*H_q,132] fp32) the merged un-normalised (m, l, o)
    record per query head is written instead, for a later combine across
    sequence shards.  ``new_k`` / ``new_v`` [n_views,H_kv,cap,128] with ``n_new`` live
    rows add the uncompressed tail of decode-appended tokens (Zone C) to the same
    softmax, as the reference's attention block does (fast_decode.py:1719-1784).
    One launch when a single chunk covers every head and there is no tail, else the
    fused kernel plus the combine; no allocation after the first call, no host
    synchronisation.
    """
    if new_k is not None:
        if new_v is None:
            raise ValueError("new_k needs new_v")
        n_rows = table.n_views * table.H_q
        ws = getattr(table, "_tail_ws", None)
        if ws is None:
            ws = torch.empty((2, n_rows, PARTIAL_STRIDE), dtype=torch.float32, device=table.device)
            table._tail_ws = ws
        packed_decode_attention(q, table, out_partial=ws[0])          # packed zones: merged record
        tail_attention_partial(q.reshape(table.n_views, table.H_q, HEAD_DIM), new_k, new_v, n_new, table.H_kv, ws[1])
        both = ws.permute(1, 0, 2)                                       # [n_rows, 2, 132]
        if out_partial is not None:
            lse_combine(both, None, out_partial=out_partial)
            return out_partial
        if out is None:
            out = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=torch.float32, device=q.device)
        lse_combine(both, out.view(-1, HEAD_DIM))
        return out
    if out_partial is not None:
        if table.n_chunks == 1:
            _launch_fused(q, table, out_partial, None)
        else:
            part = table.workspace()
            _launch_fused(q, table, part, None)
            lse_combine(part, None, out_partial=out_partial)
        return out_partial
    if out is None:
        out = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=torch.float32, device=q.device)
    if not out.is_contiguous() or out.dtype != torch.float32:
        raise ValueError("out must be contiguous float32 [n_views,H_q,128]")
    _launch_units(q, table, out)
    return out


class _HostIO:
    """Device staging buffer for the queries and the streams of the host-buffer call, kept on the table."""

    def __init__(self, table: DecodeTable, q_dtype: torch.dtype, n_slices: int, growing: bool):
        dev = table.device
        self.q = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=q_dtype, device=dev)
        self.out: Optional[Tensor] = None                  # device-side results; only for pageable out_host
        self.key = (q_dtype, n_slices, growing)
        n = table.n_views
        if growing and n_slices > 1:
            # ranges of 1 : 2 : 4 : ... : rest — the first upload, the only one no kernel hides, is short
            unit = max(1, n // (2 ** n_slices - 1))
            sizes = [unit * 2 ** i for i in range(n_slices - 1)]
            sizes.append(n - sum(sizes))
        else:
            step = -(-n // n_slices)
            sizes = [min(step, n - a) for a in range(0, n, step)]
        self.ranges, a = [], 0
        for sz in sizes:
            if sz > 0:
                self.ranges.append((a, a + sz))
                a += sz
        self.streams = [torch.cuda.Stream(device=dev) for _ in self.ranges]


def packed_decode_attention_host(q_host: Tensor, table: DecodeTable, out_host: Tensor, *,
                                 slices: Optional[int] = None) -> Tensor:
    """Host-buffer form of :func:`packed_decode_attention`: ``q_host`` [n_views,H_q,128]
    (fp16/bf16/fp32) and ``out_host`` [n_views,H_q,128] fp32 live in host memory.

    The views are cut into ``slices`` ranges (default: two when each is at least one full wave of
    CTAs); every range uploads its queries and runs the
    kernel on a stream of its own, so the upload of one range overlaps the kernel of another.
    With a pinned ``out_host`` the kernels write their results straight into it (pinned host
    memory is addressable from the device), so the results cross the bus while the kernels
    run and no separate download is needed; a pageable ``out_host`` gets a copy per range.
    Returns after the results have arrived in ``out_host``.
    """
    if q_host.is_cuda or out_host.is_cuda:
        raise ValueError("packed_decode_attention_host takes host tensors; use packed_decode_attention on the device")
    if tuple(q_host.shape) != (table.n_views, table.H_q, HEAD_DIM) or not q_host.is_contiguous():
        raise ValueError(f"q_host must be contiguous [{table.n_views},{table.H_q},{HEAD_DIM}]")
    if tuple(out_host.shape) != tuple(q_host.shape) or out_host.dtype != torch.float32 or not out_host.is_contiguous():
        raise ValueError("out_host must be contiguous float32 with q_host's shape")
    q_dtype_tag(q_host)
    growing = False
    if slices is None:                                     # two ranges when each is at least a full wave of CTAs (measured best)
        waves = (table.n_views * table.H_kv * table._n_hgrp) // (table._sms * table.CTAS_PER_SM)
        slices = 2 if waves >= 2 else 1
    n_slices = max(1, min(int(slices), table.n_views))
    io: Optional[_HostIO] = getattr(table, "_host_io", None)
    if io is None or io.key != (q_host.dtype, n_slices, growing):
        io = _HostIO(table, q_host.dtype, n_slices, growing)
        table._host_io = io
    direct = out_host.is_pinned()
    if not direct and io.out is None:
        io.out = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=torch.float32, device=table.device)
    out = out_host if direct else io.out
    cur = torch.cuda.current_stream(table.device)
    for (a, b), st in zip(io.ranges, io.streams):
        st.wait_stream(cur)
        with torch.cuda.stream(st):
            io.q[a:b].copy_(q_host[a:b], non_blocking=True)
            _launch_units(io.q, table, out, a, b)
            if not direct:
                out_host[a:b].copy_(io.out[a:b], non_blocking=True)
    for st in io.streams[:len(io.ranges)]:
        cur.wait_stream(st)
    cur.synchronize()
    return out_host


def packed_layer_attention(q: Tensor, packed_layer: PackedKVLayer, new_v_only: Optional[Tensor] = None,
                           *, use_mask: bool = False) -> Tensor:
    """Single (sequence, layer) convenience form: q [H_q,128] -> [H_q,128] fp32.

    The one-entry table is cached on the layer object, as the reference decode
    loop caches its pre-squeezed views on the cache object
    (obkv_accel/fast_decode.py:813-816).
    """
    key = (q.shape[0], None if new_v_only is None else new_v_only.data_ptr(), use_mask)
    cached = getattr(packed_layer, "_rdkv_table", None)
    if cached is None or cached[0] != key:
        cached = (key, DecodeTable([packed_layer], [new_v_only], q.shape[0], use_mask=use_mask))
        packed_layer._rdkv_table = cached
    return packed_decode_attention(q.reshape(1, q.shape[0], HEAD_DIM), cached[1])[0]
