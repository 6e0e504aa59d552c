"""Fused packed-KV decode attention.

Replaces the attention block of the reference decode loop
(obkv_accel/fast_decode.py:1701-1784: K kernel -> mask add -> softmax -> V kernel)
with one split-sequence kernel launch over any number of (sequence, layer)
pairs (units cut into chunks are merged by the last of their CTAs to finish).  Softmax semantics are the
reference's: one softmax per query head over its live Zone-A and Zone-B rows;
stripe padding is excluded through the per-head row counts read on the device
(and through ``softmax_mask`` too when ``use_mask`` is set).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from ._lib import (HEAD_DIM, PARTIAL_STRIDE, LayerView, TailArgs, check, lib, ptr, q_dtype_tag, require_cuda,
                   stream_ptr)
from .packing import PackedKVLayer, layer_identity, layer_view


class DecodeTable:
    """Device-resident array of ``rdkv_layer_view`` records, one per (sequence, layer).

    The table holds references to every tensor it points into.  Payloads, scales, zero
    points of V are read from the layers' own tensors at every launch, so a caller may
    rewrite them in place between launches.  The per-head row counts and the K scales,
    zero points and channel permutation are read from a snapshot the table keeps on the
    device: call :meth:`refresh` after rewriting those in place (or build the table with
    ``live_counts=True``, which makes every CTA read the layers' own tensors for them).
    The table also keeps tensor maps of the layers' V tensors (their addresses and extents as of
    construction), through which the kernel stages the 8-bit and fp16 rows of a tile: rewriting
    payloads in place is fine, a V tensor that moves or grows needs a new table.
    """

    def __init__(self, layers: Sequence[PackedKVLayer], new_v_only: Sequence[Optional[Tensor]], H_q: int,
                 *, use_mask: bool = False, device=None, n_chunks: Optional[int] = None,
                 k_only: bool = False, live_counts: bool = False, persistent: Optional[bool] = None):
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
        n_hgrp = (self.H_q // self.H_kv + 7) // 8
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.unit_rows = ((max(max_t_k, 1) + 63) // 64) * 64
        self._sms = sms
        self._n_hgrp = n_hgrp
        # chunks per unit: None = chosen per launch by plan(); an int forces uniform chunks
        self.n_chunks: Optional[int] = None if n_chunks is None else max(1, int(n_chunks))
        self.chunk_rows: Optional[int] = None
        raw = bytes(views)
        host = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
        self.views = host.to(self.device)
        # tensor maps of the views' V tensors (encoded on the host from the records above; the kernel's
        # staging warp brings a tile's V rows in with one tiled TMA box each where a map exists)
        with torch.cuda.device(self.device):
            maps_host = torch.zeros(int(lib().rdkv_decode_v_map_bytes(self.n_views)), dtype=torch.uint8)
            self.n_v_maps = int(lib().rdkv_decode_encode_v_maps(host.data_ptr(), self.n_views, maps_host.data_ptr()))
        if self.n_v_maps < 0:
            raise RuntimeError("rdkv_decode_encode_v_maps failed")
        self.v_maps = maps_host.to(self.device) if self.n_v_maps > 0 else None
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # snapshot of every head's row counts (one round trip less in the kernel's prologue) and the
        # arrival counters of chunked units (zero between launches)
        L = lib()
        self.nkb_max = max(L.rdkv_decode_k_blocks(int(vw.n_ch2_pad), int(vw.n_ch4_pad), int(vw.n_ch8)) for vw in views)
        n_units = self.n_views * self.H_kv
        self._unit_rec_bytes = int(L.rdkv_decode_prepared_bytes(1, self.nkb_max, 0))
        self.unit_recs = torch.empty(L.rdkv_decode_prepared_bytes(n_units, self.nkb_max, 0), dtype=torch.uint8, device=self.device)
        self.k_slots = torch.empty(L.rdkv_decode_prepared_bytes(n_units, self.nkb_max, 1), dtype=torch.uint8, device=self.device)
        self.unit_ctr = torch.zeros(self.n_views * self.H_kv * n_hgrp, dtype=torch.int32, device=self.device)
        # item counters of the persistent form: a pair per launch that may be in flight at the same time
        self.work_ctr = torch.zeros(2 * self.WORK_CTR_SLOTS, dtype=torch.int32, device=self.device)
        self._ws = {}
        # live_counts: the kernel reads the layers' count / scale / permutation tensors itself at every
        # launch (no snapshot to refresh; one more round trip per CTA)
        self.live_counts = bool(live_counts)
        self.use_mask = bool(use_mask)
        self.refresh()
        # the persistent form of the kernel needs every unit's byte ranges on whole 16-byte blocks
        # (flag bit 0 of its prepared record; read back once, here)
        self.persistent = None if persistent is None else bool(persistent)
        self._all_fast = False
        if not self.live_counts:
            recs = self.unit_recs.view(torch.int32).view(n_units, self._unit_rec_bytes // 4)
            self._all_fast = bool(((recs[:, 4] & 3) == 3).all().item())   # (bit 1: the V rows come through tensor maps)

    CTAS_PER_SM = 3                      # resident CTAs of the fused kernel per SM
    WORK_CTR_SLOTS = 64                  # launches of one table that may overlap (view ranges on streams of their own)
    # The persistent form (one resident CTA per slot draws items from a counter) is used for launches
    # of whole units that fill the CTA slots at least this many times over.  Measured on B200
    # (2048-row units): 2 % faster at 9 rounds, 3 % faster at 2.3 rounds than two rounds of whole units
    # plus the leftover units in chunks (a chunk costs 5 - 8 us of prologue, merge and record
    # traffic on top of its rows); no better than one CTA per item where whole units and chunks mix.
    PERSISTENT_MIN_ROUNDS = 2
    # cost model of a launch (SM cycles, measured on B200): a CTA spends ROW_COST per live row it
    # attends over plus a fixed cost (prologue, first tile, merge of its warps, result): FIXED_WHOLE
    # when it has a whole unit, FIXED_CHUNK when it has a chunk (record + arrival counter on top)
    ROW_COST = 17.6
    FIXED_WHOLE = 13000.0
    FIXED_CHUNK = 11000.0
    MERGE_PER_CHUNK = 1500.0             # per chunk of a unit: its record read back by the unit's last CTA, contention on the counter

    def refresh(self) -> None:
        """Rebuild the table's snapshot of the per-head quantities (one small launch on the current
        stream, capturable): V row counts, K scales, zero points and channel permutation.  Call it
        after rewriting a layer's ``seg_bounds_per_head`` / ``n_v16_per_head`` / ``K_ch_scale`` /
        ``K_ch_zp`` / ``K_ch_perm_padded_idx_for_Q`` in place; packed payloads and V scales / zero
        points are always read from the layers' own tensors."""
        if hasattr(self, "_host_io"):
            del self._host_io                              # recorded launch plans of the host-buffer call
        if self.live_counts or self.nkb_max > 24:
            self.live_counts = True
            return
        with torch.cuda.device(self.device):
            check(lib().rdkv_decode_prepare(self.views.data_ptr(), self.n_views, self.H_kv, self.nkb_max,
                                            self.unit_recs.data_ptr(), self.k_slots.data_ptr(),
                                            self.v_maps.data_ptr() if self.v_maps is not None else None,
                                            stream_ptr(self.device)), "rdkv_decode_prepare")

    def plan(self, n_views: int, rows: Optional[int] = None):
        """(k, chunk_rows, n_whole) for a launch over ``n_views`` views whose heads have up to ``rows``
        live rows to attend over (default: whole heads): the first ``n_whole`` units (view, KV head,
        group of query heads) get one CTA each, every other unit is cut into ``k`` chunks of
        ``chunk_rows`` rows, merged by the last of its CTAs to finish.

        A CTA per whole unit is the most efficient shape (a chunk pays the fixed cost again), but
        units that do not fill the last round of CTA slots leave SMs idle.  Three shapes are
        costed with the measured constants and the cheapest is taken: all units whole; all units
        in k chunks (few units); full rounds of whole units followed by the leftover units cut
        finely enough to fill one more round."""
        rows = self.unit_rows if rows is None else max(64, ((rows + 63) // 64) * 64)
        units = max(1, n_views * self.H_kv * self._n_hgrp)
        if self.n_chunks is not None:
            k = max(1, min(self.n_chunks, -(-rows // 64)))
            cr = self.chunk_rows if (self.chunk_rows and self.chunk_rows * k >= rows) else self._chunk_rows_for(k, rows)
            return k, cr, (units if k == 1 else 0)
        slots = self._sms * self.CTAS_PER_SM
        k_max = max(1, min(16, rows // 128))
        whole = rows * self.ROW_COST + self.FIXED_WHOLE

        def chunk_cost(k):                                  # (the unit's last CTA also reads all k records)
            return self._chunk_rows_for(k, rows) * self.ROW_COST + self.FIXED_CHUNK + k * self.MERGE_PER_CHUNK

        best = (-(-units // slots) * whole, 1, units)                       # all whole
        full, left = divmod(units, slots)
        if full >= self.PERSISTENT_MIN_ROUNDS and self.persistent is not False and self._can_persist():
            return 1, self._chunk_rows_for(1, rows), units                  # many rounds: whole units, persistent form
        if left and k_max > 1:
            for k in range(2, k_max + 1):                                   # full rounds whole + leftover in k chunks
                cost = full * whole + -(-left * k // slots) * chunk_cost(k)
                if cost < best[0] * 0.98:
                    best = (cost, k, full * slots)
        _, k, n_whole = best
        return k, self._chunk_rows_for(k, rows), n_whole

    def _can_persist(self) -> bool:
        return (not self.live_counts) and self._all_fast and not self.use_mask

    def unit_plan(self, n_views: int):
        """(v_main, k, rows) form of :meth:`plan`: ``v_main`` = views whose units all stay whole."""
        k, rows, n_whole = self.plan(n_views)
        return n_whole // (self.H_kv * self._n_hgrp), k, rows

    def _chunk_rows_for(self, k: int, rows: Optional[int] = None) -> int:
        rows = self.unit_rows if rows is None else rows
        return max(64, ((-(-rows // k) + 63) // 64) * 64)

    def chunk_workspace(self, k: int) -> Tensor:
        """Records of chunked units: [n_views*H_q, k, 132] fp32 (grown on demand)."""
        if k not in self._ws:
            self._ws[k] = torch.empty((self.n_views * self.H_q, k, PARTIAL_STRIDE), dtype=torch.float32, device=self.device)
        return self._ws[k]

    def workspace(self) -> Optional[Tensor]:
        """Split-sequence partial records [n_views*H_q, n_chunks, 132] fp32 of the table's launch
        shape (allocated once); None when one chunk covers every head."""
        k = self.plan(self.n_views)[0]
        return None if k == 1 else self.chunk_workspace(k)

    def check_status(self) -> None:
        """Host read (synchronises) of the kernel's status word; raises if a launch reported a problem."""
        st = int(self.status.item())
        if st:
            raise RuntimeError(f"rdkv_b200: fused decode kernel reported status {st} "
                               "(bit 0 = a staging wait ran out, bit 1 = a view did not fit the launch, "
                               "bit 2 = a tail buffer had no row left for the new token)")


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

    if n_chunks is None or chunk_rows is None:
        n_chunks, chunk_rows = table.plan(v1 - v0)[:2]
    check(lib().rdkv_decode_attn_partial(table.views.data_ptr() + v0 * C.sizeof(LayerView), v1 - v0,
                                         off(q, HEAD_DIM), q_dtype_tag(q), table.H_q,
                                         table.H_kv, chunk_rows, n_chunks, table.k_row_bytes_max,
                                         off(partials, n_chunks * PARTIAL_STRIDE), off(out, HEAD_DIM),
                                         ptr(table.status), stream_ptr(q.device)),
          "rdkv_decode_attn_partial")


def _launch_units(q: Tensor, table: DecodeTable, out: Optional[Tensor], v0: int = 0, v1: Optional[int] = None,
                  *, out_record: Optional[Tensor] = None, rows: Optional[Tuple[int, int]] = None,
                  seq_part: Optional[Tuple[int, int]] = None, plan: Optional[Tuple[int, int, int]] = None,
                  ctr_slot: int = 0, tail: Optional[TailArgs] = None, tail_rows: int = 0) -> None:
    """ONE launch of the fused kernel on views [v0, v1): whole units, or uniform chunks merged inside
    the kernel (DecodeTable.plan).  The result is the normalised ``out`` [n_views,H_q,128] or the
    un-normalised record per query head ``out_record`` [n_views*H_q,132]; ``seq_part`` = (i, n)
    restricts every head to part i of n of its rows (phase by phase), ``rows`` = (begin, end) to
    that window of the rows that leaves; ``tail`` (with up to ``tail_rows`` live rows per head)
    adds the uncompressed tail and the token being decoded.  q, out, out_record are the full-table
    tensors, the view range is cut by pointer offsets; ``out`` and ``q`` may be pinned host memory
    (addressable from the device)."""
    if not (q.is_cuda or q.is_pinned()):
        raise ValueError("q must be a CUDA tensor or pinned host memory")
    if q.shape[-1] != HEAD_DIM or q.numel() != table.n_views * table.H_q * HEAD_DIM:
        raise ValueError(f"q must be [{table.n_views},{table.H_q},{HEAD_DIM}], got {tuple(q.shape)}")
    if not q.is_contiguous():
        q = q.contiguous()
    v1 = table.n_views if v1 is None else v1
    if not 0 <= v0 <= v1 <= table.n_views:
        raise ValueError(f"view range [{v0},{v1}) outside the table of {table.n_views} views")
    if (out is None) == (out_record is None):
        raise ValueError("exactly one of out and out_record")
    r0, r1 = (0, 0x7fffffff) if rows is None else (int(rows[0]), int(rows[1]))
    if not 0 <= r0 <= r1:
        raise ValueError(f"bad row window [{r0},{r1})")
    sp_i, sp_n = (0, 1) if seq_part is None else (int(seq_part[0]), int(seq_part[1]))
    if sp_n < 1 or not 0 <= sp_i < sp_n:
        raise ValueError(f"bad sequence part {sp_i} of {sp_n}")
    all_rows = table.unit_rows + (tail_rows if tail is not None else 0)
    part_rows = all_rows if sp_n == 1 else -(-all_rows // sp_n) + 160   # a part's rows, at most
    live = min(r1, part_rows) - r0
    k, rows_k, n_whole = plan if plan is not None else table.plan(
        v1 - v0, None if (rows is None and sp_n == 1 and all_rows == table.unit_rows) else live)
    hy = table.H_kv * table._n_hgrp
    if plan is not None:                                   # a plan of the whole table: its whole units are the table's first
        n_whole -= v0 * hy
    n_whole = min(max(n_whole, 0), (v1 - v0) * hy)
    qrow = v0 * table.H_q                                  # first query-head row of the range

    def off(t: Optional[Tensor], per_row: int) -> Optional[int]:
        return None if t is None else t.data_ptr() + qrow * per_row * t.element_size()

    ws = table.chunk_workspace(k) if k > 1 else None
    # persistent form (one resident CTA per slot draws the items): when the table allows it and the
    # launch is whole units filling the CTA slots several times over (or the table asks for it)
    items = n_whole + ((v1 - v0) * hy - n_whole) * k
    can = table._can_persist() and (q.data_ptr() + qrow * HEAD_DIM * q.element_size()) % 16 == 0
    want = (table.persistent if table.persistent is not None
            else (k == 1 and items >= table.PERSISTENT_MIN_ROUNDS * table._sms * table.CTAS_PER_SM))
    persistent = can and want and ctr_slot < table.WORK_CTR_SLOTS and tail is None
    fn = (lib().rdkv_decode_attn_tail if tail is not None
          else lib().rdkv_decode_attn_persistent if persistent else lib().rdkv_decode_attn)
    extra = (table.work_ctr.data_ptr() + 8 * ctr_slot,) if persistent else ()
    tail_arg = ()
    if tail is not None:                                   # this range's views of the per-view tail tensors
        es = 2
        tv = TailArgs.from_buffer_copy(tail)
        for name, per_view in (("new_k", tv.view_stride * es), ("new_v", tv.view_stride * es),
                               ("n_new_per_view", 4), ("rope_cos", tv.rope_view_stride * _ELEM_SIZE[tv.rope_dtype]),
                               ("rope_sin", tv.rope_view_stride * _ELEM_SIZE[tv.rope_dtype]),
                               ("k_cur", table.H_kv * HEAD_DIM * es), ("v_cur", table.H_kv * HEAD_DIM * es)):
            base = getattr(tv, name)
            if base:
                setattr(tv, name, base + v0 * per_view)
        tail_arg = (C.byref(tv),)
    with torch.cuda.device(table.device):
        check(fn(table.views.data_ptr() + v0 * C.sizeof(LayerView), v1 - v0,
                                     off(q, HEAD_DIM), q_dtype_tag(q), table.H_q, table.H_kv, rows_k, k, n_whole, r0, r1, sp_i, sp_n,
                                     table.k_row_bytes_max,
                                     None if table.live_counts else table.unit_recs.data_ptr() + v0 * table.H_kv * table._unit_rec_bytes,
                                     None if table.live_counts else table.k_slots.data_ptr() + v0 * table.H_kv * table.nkb_max * 512,
                                     0 if table.live_counts else table.nkb_max,
                                     off(ws, k * PARTIAL_STRIDE), table.unit_ctr.data_ptr() + v0 * hy * 4, *extra,
                                     off(out, HEAD_DIM), off(out_record, PARTIAL_STRIDE),
                                     ptr(table.status), *tail_arg, stream_ptr(table.device)),
              "rdkv_decode_attn")


_ELEM_SIZE = {0: 2, 1: 2, 2: 4}                           # bytes per element of RDKV_F16 / RDKV_BF16 / RDKV_F32


def _tail_args(table: DecodeTable, new_k: Optional[Tensor], new_v: Optional[Tensor], n_new, k_cur: Optional[Tensor],
               v_cur: Optional[Tensor], rope, append: bool) -> Optional[Tuple[TailArgs, int, list]]:
    """The argument record of the one-launch form for these tail tensors, the most tail rows a head
    has, and the tensors the record points into (kept alive by the caller until the launch is
    queued); None when the tensors do not fit it (other types than fp16 / bf16, rows that are not
    contiguous, unaligned addresses)."""
    n_views, H_kv = table.n_views, table.H_kv
    ref = new_k if new_k is not None else k_cur
    if ref is None or ref.dtype not in (torch.float16, torch.bfloat16):
        return None
    ta, keep = TailArgs(), []
    ta.dtype = q_dtype_tag(ref)
    rows = 0
    if new_k is not None:
        require_cuda(new_k, "new_k"); require_cuda(new_v, "new_v")
        if new_k.dim() != 4 or tuple(new_k.shape[:2]) != (n_views, H_kv) or new_k.shape[-1] != HEAD_DIM:
            raise ValueError(f"new_k must be [{n_views},{H_kv},cap,{HEAD_DIM}], got {tuple(new_k.shape)}")
        if new_v.shape != new_k.shape or new_v.dtype != new_k.dtype or new_v.stride() != new_k.stride():
            raise ValueError("new_v must match new_k in shape, dtype and strides")
        cap = int(new_k.shape[2])
        if (new_k.stride(3) != 1 or (cap > 1 and new_k.stride(2) != HEAD_DIM) or new_k.stride(0) % 8 or new_k.stride(1) % 8
                or new_k.data_ptr() % 16 or new_v.data_ptr() % 16):
            return None
        ta.new_k, ta.new_v, ta.cap = new_k.data_ptr(), new_v.data_ptr(), cap
        ta.view_stride, ta.head_stride = new_k.stride(0), new_k.stride(1)
        keep += [new_k, new_v]
        if isinstance(n_new, Tensor):
            require_cuda(n_new, "n_new")
            if n_new.dtype != torch.int32 or n_new.numel() != n_views or not n_new.is_contiguous():
                raise ValueError("n_new tensor must be contiguous int32 [n_views]")
            ta.n_new_per_view, rows = n_new.data_ptr(), cap
            keep.append(n_new)
        else:
            rows = int(n_new)
            if not 0 <= rows <= cap:
                raise ValueError(f"n_new={rows} outside [0, {cap}]")
            ta.n_new = rows
    if k_cur is not None:
        if v_cur is None:
            raise ValueError("k_cur needs v_cur")
        for name, t in (("k_cur", k_cur), ("v_cur", v_cur)):
            require_cuda(t, name)
            if tuple(t.shape) != (n_views, H_kv, HEAD_DIM) or t.dtype != ref.dtype or not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous [{n_views},{H_kv},{HEAD_DIM}] of the tail's dtype")
        ta.k_cur, ta.v_cur = k_cur.data_ptr(), v_cur.data_ptr()
        keep += [k_cur, v_cur]
        if append:
            if new_k is None:
                raise ValueError("append=True needs the tail buffers new_k / new_v")
            if not isinstance(n_new, Tensor) and int(n_new) >= int(new_k.shape[2]):
                raise ValueError("the tail buffers are full: no row left for the new token")
            ta.append = 1
    if rope is not None:
        cos, sin = rope
        require_cuda(cos, "rope cos"); require_cuda(sin, "rope sin")
        if cos.shape != sin.shape or cos.dtype != sin.dtype or cos.shape[-1] != HEAD_DIM // 2 or not (
                cos.is_contiguous() and sin.is_contiguous()):
            raise ValueError("rope = (cos, sin): contiguous [64] or [n_views,64] tensors of one dtype")
        if cos.dim() == 2 and cos.shape[0] != n_views or cos.dim() > 2:
            raise ValueError(f"rope tables must be [64] or [{n_views},64]")
        ta.rope_cos, ta.rope_sin, ta.rope_dtype = cos.data_ptr(), sin.data_ptr(), q_dtype_tag(cos)
        ta.rope_view_stride = HEAD_DIM // 2 if cos.dim() == 2 else 0
        keep += [cos, sin]
    return ta, rows, keep


def decode_attention_partial(q: Tensor, table: DecodeTable, out: Optional[Tensor] = None) -> Tensor:
    """The fused kernel alone, writing per-chunk records and leaving them unmerged (the input of
    :func:`lse_combine`): returns ``[n_views*H_q, k, 132]``, or ``out`` itself when a single chunk
    covers every head (the kernel then writes normalised results)."""
    k, rows_k = table.plan(table.n_views)[:2]
    if k == 1:
        if out is None:
            out = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=torch.float32, device=q.device)
        _launch_fused(q, table, None, out, n_chunks=1, chunk_rows=rows_k)
        return out
    part = table.chunk_workspace(k)
    _launch_fused(q, table, part, None, n_chunks=k, chunk_rows=rows_k)
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
                                       n_int, ptr(per_view), cap, ptr(out_partial), stream_ptr(q.device)),
          "rdkv_tail_attn_partial")
    return out_partial


def packed_decode_attention(q: Tensor, table: DecodeTable, *, out: Optional[Tensor] = None,
                            out_partial: Optional[Tensor] = None, new_k: Optional[Tensor] = None,
                            new_v: Optional[Tensor] = None, n_new=0,
                            rows: Optional[Tuple[int, int]] = None,
                            seq_part: Optional[Tuple[int, int]] = None, k_cur: Optional[Tensor] = None,
                            v_cur: Optional[Tensor] = None, rope: Optional[Tuple[Tensor, Tensor]] = None,
                            append: bool = True, one_launch: Optional[bool] = None) -> Tensor:
    """softmax(q·K̂ᵀ/√128)·V̂ over every view of ``table``.

    q [n_views,H_q,128] fp16/bf16/fp32 -> out [n_views,H_q,128] fp32.  With
    ``out_partial`` ([n_views*H_q,132] fp32) the merged un-normalised (m, l, o)
    record per query head is written instead, for a later combine across
    sequence shards; ``seq_part`` = (i, n) restricts every head to part i of n of its
    rows, shared out phase by phase (the share of one sequence-split rank), ``rows`` =
    (begin, end) to that window of the rows that leaves.  ``new_k`` / ``new_v``
    [n_views,H_kv,cap,128] with ``n_new`` live rows add the uncompressed tail of
    decode-appended tokens (Zone C) to the same softmax, as the reference's attention
    block does (fast_decode.py:1719-1784).  ``k_cur`` / ``v_cur`` [n_views,H_kv,128]: the
    key and value row of the token being decoded; it joins the softmax and, with
    ``append``, its rows are written to row ``n_new`` of the tail buffers (the caller
    counts ``n_new`` up for the next step).  ``rope`` = (cos, sin), [64] or
    [n_views,64]: the queries and ``k_cur`` are rotated first (half format, as
    fused_rope does in place, triton_rope.py:35-108; q itself is not written), so the
    call covers fast_decode.py:1699-1784 of a layer.
    Always one launch (chunked units are merged inside the kernel) when the tail buffers
    are fp16 / bf16 with contiguous rows; other tail buffers (``one_launch=False`` forces
    this form, which takes neither ``k_cur`` nor ``rope``) take the fused kernel, the tail
    kernel and the combine.  No allocation after the first call, no host synchronisation.
    """
    if new_k is not None and new_v is None:
        raise ValueError("new_k needs new_v")
    if new_k is not None or k_cur is not None or rope is not None:
        fused = None if one_launch is False else _tail_args(table, new_k, new_v, n_new, k_cur, v_cur, rope, append)
        if fused is None and (k_cur is not None or rope is not None or one_launch):
            raise ValueError("the one-launch form needs fp16 / bf16 tail buffers with contiguous, 16-byte aligned rows")
        if fused is not None:
            ta, tail_rows, _keep = fused
            if out_partial is not None:
                if (out_partial.dtype != torch.float32 or not out_partial.is_contiguous()
                        or out_partial.numel() != table.n_views * table.H_q * PARTIAL_STRIDE):
                    raise ValueError(f"out_partial must be contiguous float32 [{table.n_views * table.H_q},{PARTIAL_STRIDE}]")
                _launch_units(q, table, None, out_record=out_partial, rows=rows, seq_part=seq_part, tail=ta,
                              tail_rows=tail_rows)
                return out_partial
            if out is None:
                out = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=torch.float32, device=q.device)
            if (not out.is_contiguous() or out.dtype != torch.float32
                    or out.numel() != table.n_views * table.H_q * HEAD_DIM):
                raise ValueError(f"out must be contiguous float32 [{table.n_views},{table.H_q},{HEAD_DIM}]")
            _launch_units(q, table, out, rows=rows, seq_part=seq_part, tail=ta, tail_rows=tail_rows)
            return out
    if new_k is not None:
        n_rows = table.n_views * table.H_q
        ws = getattr(table, "_tail_ws", None)
        if ws is None:
            ws = torch.empty((2, n_rows, PARTIAL_STRIDE), dtype=torch.float32, device=table.device)
            table._tail_ws = ws
        _launch_units(q, table, None, out_record=ws[0], rows=rows, seq_part=seq_part)      # packed zones: merged record
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
        if (out_partial.dtype != torch.float32 or not out_partial.is_contiguous()
                or out_partial.numel() != table.n_views * table.H_q * PARTIAL_STRIDE):
            raise ValueError(f"out_partial must be contiguous float32 [{table.n_views * table.H_q},{PARTIAL_STRIDE}]")
        _launch_units(q, table, None, out_record=out_partial, rows=rows, seq_part=seq_part)
        return out_partial
    if out is None:
        out = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=torch.float32, device=q.device)
    if (not out.is_contiguous() or out.dtype != torch.float32
            or out.numel() != table.n_views * table.H_q * HEAD_DIM):
        raise ValueError(f"out must be contiguous float32 [{table.n_views},{table.H_q},{HEAD_DIM}]")
    _launch_units(q, table, out, rows=rows, seq_part=seq_part)
    return out


class _HostIO:
    """Device staging buffer for the queries and the streams of the host-buffer call, kept on the table."""
    MAX_GRAPHS = 8

    def __init__(self, table: DecodeTable, q_dtype: torch.dtype, n_slices: int, growing: bool):
        dev = table.device
        self.q = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=q_dtype, device=dev)
        self.out: Optional[Tensor] = None                  # device-side results; only for pageable out_host
        self.key = (q_dtype, n_slices, growing)
        n = table.n_views
        if growing and n_slices > 1:
            # ranges of 1 : 2 : 4 : ... : rest — the first upload, the only one no kernel hides, is short
            unit = max(1, n // (2 ** n_slices - 1))
            sizes, left = [], n
            for i in range(n_slices - 1):
                sizes.append(min(unit * 2 ** i, left))
                left -= sizes[-1]
            sizes.append(left)
        else:
            step = -(-n // n_slices)
            sizes = [min(step, n - a) for a in range(0, n, step)]
        self.ranges, a = [], 0
        for sz in sizes:
            if sz > 0:
                self.ranges.append((a, a + sz))
                a += sz
        self.streams = [torch.cuda.Stream(device=dev) for _ in self.ranges]
        self.capture_stream = torch.cuda.Stream(device=dev)
        self.graphs: dict = {}                             # (buffers, table, plan) -> the ranges' copies and launches, recorded
        self.seen: set = set()
        self.replays: dict = {}                            # the call's arguments as given -> its recording (shortcut of the next call)


def _issue_host_ranges(io: "_HostIO", q_host: Tensor, out_host: Tensor, table: DecodeTable, out: Tensor,
                       direct: bool, plan, in_place: int = 0) -> None:
    """Every range on its own stream, forked from and joined to the current stream: upload of the
    range's queries, its launch, and (pageable results only) its download.  The first ``in_place``
    ranges read their queries straight from the (pinned) host buffer instead of uploading them."""
    cur = torch.cuda.current_stream(table.device)
    for slot, ((a, b), st) in enumerate(zip(io.ranges, io.streams)):
        st.wait_stream(cur)
        with torch.cuda.stream(st):
            if slot < in_place:
                _launch_units(q_host, table, out, a, b, plan=plan, ctr_slot=slot)
            else:
                io.q[a:b].copy_(q_host[a:b], non_blocking=True)
                _launch_units(io.q, table, out, a, b, plan=plan, ctr_slot=slot)
            if not direct:
                out_host[a:b].copy_(io.out[a:b], non_blocking=True)
    for st in io.streams[:len(io.ranges)]:
        cur.wait_stream(st)


def packed_decode_attention_host(q_host: Tensor, table: DecodeTable, out_host: Tensor, *,
                                 slices: Optional[int] = None, graph: Optional[bool] = None,
                                 growing: Optional[bool] = None, in_place: Optional[int] = None) -> Tensor:
    """Host-buffer form of :func:`packed_decode_attention`: ``q_host`` [n_views,H_q,128]
    (fp16/bf16/fp32) and ``out_host`` [n_views,H_q,128] fp32 live in host memory.

    The views are cut into ``slices`` ranges (default: one or two, by the waves of CTAs the table
    fills); every range uploads its queries and runs the
    kernel on a stream of its own, so the upload of one range overlaps the kernel of another.
    With a pinned ``out_host`` the kernels write their results straight into it (pinned host
    memory is addressable from the device), so the results cross the bus while the kernels
    run and no separate download is needed; a pageable ``out_host`` gets a copy per range.

    With both buffers pinned, the second call with the same two buffers records the copies and
    launches of all ranges as one CUDA graph, and that call and later ones replay it: a step then
    costs one graph launch on the host instead of a dozen stream operations (``graph=False``
    keeps the stream form; the graph holds the buffers' addresses, the table's and its launch
    plan; a few recordings are kept per table, for callers that alternate between buffers;
    :meth:`DecodeTable.refresh` drops them).  The kernels of the first ``in_place`` ranges
    (default: one in the graph form) read their queries from the pinned buffer itself, so the
    step does not start with an upload that nothing hides.
    Returns after the results have arrived in ``out_host``.
    """
    io: Optional[_HostIO] = getattr(table, "_host_io", None)
    call_key = (q_host.data_ptr(), out_host.data_ptr(), q_host.dtype, q_host.numel(), out_host.numel(), out_host.dtype,
                slices, graph, growing, in_place)
    if io is not None:                                     # a call seen before with a recording: nothing else to do
        g = io.replays.get(call_key)
        if g is not None:
            g.replay()
            torch.cuda.current_stream(table.device).synchronize()
            return out_host
    if q_host.is_cuda or out_host.is_cuda:
        raise ValueError("packed_decode_attention_host takes host tensors; use packed_decode_attention on the device")
    if tuple(q_host.shape) != (table.n_views, table.H_q, HEAD_DIM) or not q_host.is_contiguous():
        raise ValueError(f"q_host must be contiguous [{table.n_views},{table.H_q},{HEAD_DIM}]")
    if tuple(out_host.shape) != tuple(q_host.shape) or out_host.dtype != torch.float32 or not out_host.is_contiguous():
        raise ValueError("out_host must be contiguous float32 with q_host's shape")
    q_dtype_tag(q_host)
    direct = out_host.is_pinned()
    use_graph = (direct and q_host.is_pinned()) if graph is None else bool(graph)
    if use_graph and not (direct and q_host.is_pinned()):
        raise ValueError("graph=True needs pinned q_host and out_host")
    waves = (table.n_views * table.H_kv * table._n_hgrp) // (table._sms * table.CTAS_PER_SM)
    if slices is None:
        # measured best.  Stream form: two ranges when each is at least a full wave of CTAs (the
        # host's per-range work is in the way of more).  Graph form: two ranges for a table of one
        # to three waves; ONE for a larger table, whose kernel then reads its queries from the pinned
        # buffer itself (in_place) and writes its results into the other: a launch of many waves deals
        # most of its items out statically, which cutting it into ranges would undo.
        slices = ((2 if 1 <= waves <= 3 else 1) if use_graph else (2 if waves >= 2 else 1))
    growing = False if growing is None else bool(growing)  # ranges of 1 : 2 : 4 : ... instead of equal ones
    n_slices = max(1, min(int(slices), table.n_views))
    if io is None or io.key != (q_host.dtype, n_slices, growing):
        io = _HostIO(table, q_host.dtype, n_slices, growing)
        table._host_io = io
    if not direct and io.out is None:
        io.out = torch.empty((table.n_views, table.H_q, HEAD_DIM), dtype=torch.float32, device=table.device)
    out = out_host if direct else io.out
    cur = torch.cuda.current_stream(table.device)
    plan = table.plan(table.n_views)                       # the device call's launch shape: same results bit for bit
    # leading ranges whose kernels read the queries from the pinned host buffer itself: no upload to wait for
    n_in_place = (1 if use_graph else 0) if in_place is None else int(in_place)
    if n_in_place and not q_host.is_pinned():
        raise ValueError("in_place needs a pinned q_host")
    if use_graph:
        key = (q_host.data_ptr(), out_host.data_ptr(), table.views.data_ptr(), plan, n_in_place)
        g = io.graphs.get(key)
        if g is None and key in io.seen:                   # second call with these buffers: record, then replay
            if len(io.graphs) >= _HostIO.MAX_GRAPHS:       # a caller that keeps changing buffers: forget the oldest
                old = io.graphs.pop(next(iter(io.graphs)))
                io.replays = {k: v for k, v in io.replays.items() if v is not old}
            g = torch.cuda.CUDAGraph()
            io.capture_stream.wait_stream(cur)
            with torch.cuda.graph(g, stream=io.capture_stream, capture_error_mode="thread_local"):
                _issue_host_ranges(io, q_host, out_host, table, out, direct, plan, n_in_place)
            cur.wait_stream(io.capture_stream)
            io.graphs[key] = g
        if g is not None:
            if len(io.replays) >= 4 * _HostIO.MAX_GRAPHS:
                io.replays.clear()
            io.replays[call_key] = g
            g.replay()
            cur.synchronize()
            return out_host
        if len(io.seen) >= 4 * _HostIO.MAX_GRAPHS:
            io.seen.clear()
        io.seen.add(key)
    _issue_host_ranges(io, q_host, out_host, table, out, direct, plan, n_in_place)
    cur.synchronize()
    return out_host


def packed_layer_attention(q: Tensor, packed_layer: PackedKVLayer, new_v_only: Optional[Tensor] = None,
                           *, use_mask: bool = False) -> Tensor:
    """Single (sequence, layer) convenience form: q [H_q,128] -> [H_q,128] fp32.

    The one-entry table is cached on the layer object, as the reference decode
    loop caches its pre-squeezed views on the cache object
    (obkv_accel/fast_decode.py:813-816).
    """
    key = (q.shape[0], use_mask, layer_identity(packed_layer),
           None if new_v_only is None else (new_v_only.data_ptr(), tuple(new_v_only.shape), tuple(new_v_only.stride())))
    cached = getattr(packed_layer, "_rdkv_table", None)
    if cached is None or cached[0] != key:
        # (live_counts: a caller may rewrite the per-head counts in place between calls)
        cached = (key, DecodeTable([packed_layer], [new_v_only], q.shape[0], use_mask=use_mask, live_counts=True))
        packed_layer._rdkv_table = cached
    return packed_decode_attention(q.reshape(1, q.shape[0], HEAD_DIM), cached[1])[0]
