"""Decode-attention parity (through the C ABI): K-side scores, V-side weighted sum,
the fused split-sequence kernel and the log-sum-exp combine against golden vectors
produced by the reference's dequantise-then-attend code and against the numpy oracle.
Tolerance for attention outputs: |err| <= 2e-3 + 1e-2*|ref|."""
import numpy as np
import pytest
import torch

from conftest import sub
from helpers import assert_attn_close, cuda, layer_to_np, to_np

pytestmark = pytest.mark.gpu


def _packed(g):
    from rdkv_b200.packing import pack_kv
    return pack_kv(cuda(g["K"]), cuda(g["V"]), cuda(g["v_bits"]), cuda(g["k_bits"]), int(g["g"]))


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
@pytest.mark.parametrize("qdtype", [torch.float16, torch.float32])
def test_k_scores_match_golden(golden_layers, tag, qdtype):
    from rdkv_b200.k_kernel import k_mixed_qk_dot, k_mixed_qk_dot_into
    g = sub(golden_layers, tag)
    pl, _ = _packed(g)
    q = cuda(g["q"]).to(qdtype)
    s = k_mixed_qk_dot(q, pl, pl.T_eff_k)
    live = np.isfinite(g["softmax_mask"])
    np.testing.assert_allclose(to_np(s)[live], g["k_scores"][live], atol=2e-3, rtol=1e-3)
    # _into form writes only [:, :T_eff] of a wider, offset, unaligned buffer
    buf = torch.full((q.shape[0], pl.T_eff_k + 13), 7.0, device="cuda")
    view = buf[:, 3:3 + pl.T_eff_k]
    k_mixed_qk_dot_into(q, pl, pl.T_eff_k - 5, view)
    assert torch.all(buf[:, :3] == 7.0) and torch.all(buf[:, 3 + pl.T_eff_k - 5:] == 7.0)
    assert torch.equal(view[:, :pl.T_eff_k - 5], s[:, :pl.T_eff_k - 5])


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
def test_two_stage_attention_matches_golden(golden_layers, tag):
    """scores -> masked softmax (torch) -> V-side kernel, the reference's call sequence."""
    from rdkv_b200.k_kernel import k_mixed_qk_dot
    from rdkv_b200.v_kernel import v_dequant_weighted_sum_dispatch, v_dequant_weighted_sum_dispatch_into
    g = sub(golden_layers, tag)
    pl, nv = _packed(g)
    q = cuda(g["q"])
    s = k_mixed_qk_dot(q.float(), pl, pl.T_eff_k) + pl.softmax_mask
    w_all = torch.softmax(torch.cat([s, torch.zeros(s.shape[0], 5, device="cuda")], dim=1), dim=-1)
    w = torch.softmax(s, dim=-1)
    V16 = nv[0] if nv is not None else None
    out = v_dequant_weighted_sum_dispatch(w, pl, V16=V16, n_v16_per_head=pl.n_v16_per_head, max_T_v=pl.T_eff)
    assert_attn_close(to_np(out), g["attn_out"], tag)
    # strided weight view (column slice of a wider buffer) and preallocated output
    out2 = torch.empty_like(out)
    v_dequant_weighted_sum_dispatch_into(w_all[:, :pl.T_eff_k] * (w_all.sum(1, keepdim=True) / w_all[:, :pl.T_eff_k].sum(1, keepdim=True)),
                                         pl, out2, V16=V16, n_v16_per_head=pl.n_v16_per_head, max_T_v=pl.T_eff)
    assert_attn_close(to_np(out2), g["attn_out"], tag + " strided")


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
@pytest.mark.parametrize("use_mask", [False, True])
def test_fused_attention_matches_golden(golden_layers, tag, use_mask):
    from rdkv_b200.decode import packed_layer_attention
    g = sub(golden_layers, tag)
    pl, nv = _packed(g)
    out = packed_layer_attention(cuda(g["q"]), pl, nv, use_mask=use_mask)
    assert_attn_close(to_np(out), g["attn_out"], tag)


def test_fused_batch_of_views_and_partials():
    """Several (sequence, layer) views in one launch, bf16 queries; merged partial records
    recombine to the same output; config-0 shape against the oracle."""
    from oracle import ref_attention as RA
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, lse_combine, packed_decode_attention
    from rdkv_b200.packing import pack_kv
    layers, nvs, wants = [], [], []
    H_kv, g = 8, 4
    shapes = [(4096, 1024, None), (1024, 512, [512, 448, 384, 512, 320, 512, 256, 512]), (700, 200, None)]
    qs = synth.make_q(H_kv * g, seed=9, batch=len(shapes), dtype=torch.bfloat16)
    for i, (T, N, ragged) in enumerate(shapes):
        seed = synth.unit_seed(0, i, 3)
        K, V = synth.make_kv(H_kv, T, seed=seed)
        vb = synth.make_v_bits(H_kv, T, N, seed=seed, per_head_N=ragged)
        kb = synth.make_k_bits(H_kv, seed=seed)
        pl, nv = pack_kv(K.cuda(), V.cuda(), vb.cuda(), kb.cuda(), g)
        layers.append(pl)
        nvs.append(nv)
        ol, onv = RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g)
        wants.append(RA.decode_attention(qs[i].float().numpy(), ol, onv))
    table = DecodeTable(layers, nvs, H_kv * g)
    out = packed_decode_attention(qs.cuda(), table)
    for i, (w_out, _, _) in enumerate(wants):
        assert_attn_close(to_np(out[i]), w_out, f"view {i}")
    # merged un-normalised records: normalise on the host and compare; m and l match the oracle
    rec = torch.empty((len(shapes) * H_kv * g, 132), device="cuda")
    packed_decode_attention(qs.cuda(), table, out_partial=rec)
    r = to_np(rec).reshape(len(shapes), H_kv * g, 132)
    for i, (w_out, w_m, w_l) in enumerate(wants):
        assert_attn_close(r[i, :, 4:] / r[i, :, 1:2], w_out, f"partial {i}")
        lse_got = r[i, :, 0] + np.log(r[i, :, 1])
        np.testing.assert_allclose(lse_got, w_m + np.log(w_l), atol=2e-3)
    # combining a record with an empty one (m=-inf, l=0) is the identity
    empty = torch.zeros_like(rec)
    empty[:, 0] = float("-inf")
    both = torch.stack([rec, empty], dim=1)
    again = lse_combine(both)
    assert_attn_close(to_np(again).reshape(len(shapes), H_kv * g, 128)[0], wants[0][0], "combine identity")


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
def test_uncompressed_tail_matches_reference_vectors(golden_layers, tag):
    """One softmax over the packed zones and the tokens appended while decoding, against the
    reference's formula (fast_decode.py:1719-1784) evaluated on the reference's own dequantised
    cache: fp16 and fp32 tail buffers, the tail as a row count and as a per-view tensor."""
    from rdkv_b200.decode import DecodeTable, packed_decode_attention
    g = sub(golden_layers, tag)
    H_q = g["q"].shape[0]
    pl, nv = _packed(g)
    n = g["tail_k"].shape[1]
    for dt in (torch.float16, torch.float32):
        cap = n + 5
        new_k = torch.zeros((1, g["tail_k"].shape[0], cap, 128), dtype=dt, device="cuda")
        new_v = torch.zeros_like(new_k)
        new_k[0, :, :n] = cuda(g["tail_k"]).to(dt)
        new_v[0, :, :n] = cuda(g["tail_v"]).to(dt)
        table = DecodeTable([pl], [nv], H_q)
        for count in (n, torch.tensor([n], dtype=torch.int32, device="cuda")):
            out = packed_decode_attention(cuda(g["q"]).reshape(1, H_q, 128), table, new_k=new_k, new_v=new_v, n_new=count)
            assert_attn_close(to_np(out[0]), g["attn_out_tail"], f"{tag} tail {dt}")
        table.check_status()


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_uncompressed_tail_joins_the_softmax(kv_dtype):
    """Zone C (decode-appended fp rows) is part of the same softmax as the packed zones:
    several views with different tail lengths (per-view count tensor and shared int),
    single-chunk and split-sequence tables, against the oracle."""
    from oracle import ref_attention as RA
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, packed_decode_attention, tail_attention_partial
    from rdkv_b200.packing import pack_kv
    H_kv, g, cap = 4, 4, 40
    shapes = [(1024, 384, None), (640, 256, [256, 100, 7, 200]), (512, 128, None)]
    tails = [33, 0, 40]
    qs = synth.make_q(H_kv * g, seed=21, batch=len(shapes), dtype=torch.float16)
    gen = torch.Generator().manual_seed(77)
    new_k = torch.randn(len(shapes), H_kv, cap, 128, generator=gen).to(kv_dtype)
    new_v = torch.randn(len(shapes), H_kv, cap, 128, generator=gen).to(kv_dtype)
    layers, nvs, wants, ols = [], [], [], []
    for i, (T, N, ragged) in enumerate(shapes):
        seed = synth.unit_seed(3, i, 9)
        K, V = synth.make_kv(H_kv, T, seed=seed)
        vb = synth.make_v_bits(H_kv, T, N, seed=seed, per_head_N=ragged)
        kb = synth.make_k_bits(H_kv, seed=seed)
        pl, nv = pack_kv(K.cuda(), V.cuda(), vb.cuda(), kb.cuda(), g)
        layers.append(pl); nvs.append(nv)
        ol, onv = RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g)
        ols.append((ol, onv))
        wants.append(RA.decode_attention(qs[i].float().numpy(), ol, onv,
                                         new_k[i, :, :tails[i]].float().numpy(), new_v[i, :, :tails[i]].float().numpy())[0])
    n_dev = torch.tensor(tails, dtype=torch.int32, device="cuda")
    for n_chunks in (1, 3):
        table = DecodeTable(layers, nvs, H_kv * g)
        table.n_chunks, table.chunk_rows = n_chunks, 64 * (-(-table.max_t_k // (64 * n_chunks)))
        out = packed_decode_attention(qs.cuda(), table, new_k=new_k.cuda(), new_v=new_v.cuda(), n_new=n_dev)
        for i, w in enumerate(wants):
            assert_attn_close(to_np(out[i]), w, f"chunks {n_chunks} view {i}")
        table.check_status()
    # shared integer count: every view uses the first 12 tail rows
    table = DecodeTable(layers[:1], nvs[:1], H_kv * g)
    out = packed_decode_attention(qs[:1].cuda(), table, new_k=new_k[:1].cuda(), new_v=new_v[:1].cuda(), n_new=12)
    ol, onv = ols[0]
    want = RA.decode_attention(qs[0].float().numpy(), ol, onv, new_k[0, :, :12].float().numpy(), new_v[0, :, :12].float().numpy())[0]
    assert_attn_close(to_np(out[0]), want, "shared count")
    # an empty tail record is (-inf, 0, 0): combining it changes nothing
    rec = tail_attention_partial(qs[:1].cuda(), new_k[:1].cuda(), new_v[:1].cuda(), 0, H_kv)
    assert torch.all(rec[:, 0] == float("-inf")) and torch.all(rec[:, 1] == 0) and torch.all(rec[:, 4:] == 0)
    with pytest.raises(ValueError):
        packed_decode_attention(qs[:1].cuda(), table, new_k=new_k[:1].cuda())


def test_whole_units_and_uniform_chunks():
    """One CTA per unit against uniform chunks of every unit merged inside the kernel by the last
    CTA of the unit to finish (two and three chunks, more CTAs than one wave), and what the launch
    plan picks by itself for many and for few units.  All shapes against each other and the oracle."""
    from oracle import ref_attention as RA
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, packed_decode_attention
    from rdkv_b200.packing import pack_kv
    H_kv, g, T, N = 4, 4, 1024, 560
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    n_views = (3 * sms) // H_kv + 9                        # a few units more than one wave of CTAs
    layers, nvs = [], []
    for i in range(n_views):
        seed = synth.unit_seed(6, i % 7, i)
        K, V = synth.make_kv(H_kv, T, seed=seed)
        vb = synth.make_v_bits(H_kv, T, N, seed=seed)
        kb = synth.make_k_bits(H_kv, seed=seed)
        pl, nv = pack_kv(K.cuda(), V.cuda(), vb.cuda(), kb.cuda(), g, build_mask=False)
        layers.append(pl); nvs.append(nv)
        if i == n_views - 1:
            last = RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g)
    q = synth.make_q(H_kv * g, seed=5, batch=n_views, dtype=torch.float16)
    want_last = RA.decode_attention(q[n_views - 1].float().numpy(), *last)[0]
    outs = []
    for lo, forced in ((0, 1), (0, 2), (0, 3), (0, None), (n_views - 20, None)):
        table = DecodeTable(layers[lo:], nvs[lo:], H_kv * g, n_chunks=forced)
        k, rows, n_whole = table.plan(n_views - lo)
        assert k == forced if forced else (k > 1 if lo else k >= 1)
        assert k * rows >= table.unit_rows and 0 <= n_whole <= (n_views - lo) * H_kv
        if forced is None and lo == 0:                     # a few units more than one round of CTAs: only those are cut
            assert k > 1 and n_whole == 3 * sms
        for rep in range(2):                               # twice: the arrival counters must be back at zero
            out = packed_decode_attention(q[lo:].cuda(), table)
            assert_attn_close(to_np(out[-1]), want_last, f"last view, {k} chunks, call {rep}")
        assert int(table.unit_ctr.abs().sum().item()) == 0
        outs.append(out[-20:])
        table.check_status()
    for o in outs[1:]:
        assert_attn_close(to_np(outs[0]), to_np(o), "whole units vs chunks")


def test_row_windows_merge_to_the_unsplit_result():
    """Sequence split on one GPU: every window of the heads' live rows gives the oracle's record for
    that window, and the windows' records merge to the unsplit result (ragged heads, windows that
    cut phases anywhere, windows past a short head's end)."""
    from oracle import ref_attention as RA
    from oracle import ref_packing as RP
    from rdkv_b200 import sharding, synth
    from rdkv_b200.decode import DecodeTable, lse_combine, packed_decode_attention
    from rdkv_b200.packing import pack_kv
    H_kv, g, T = 4, 4, 2048
    layers, nvs, ols = [], [], []
    for i, ragged in enumerate(([700, 333, 512, 64], None)):
        seed = synth.unit_seed(7, i, 3)
        K, V = synth.make_kv(H_kv, T, seed=seed)
        vb = synth.make_v_bits(H_kv, T, 640, seed=seed, per_head_N=ragged)
        kb = synth.make_k_bits(H_kv, seed=seed)
        pl, nv = pack_kv(K.cuda(), V.cuda(), vb.cuda(), kb.cuda(), g, build_mask=False)
        layers.append(pl); nvs.append(nv)
        ols.append(RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g))
    q = synth.make_q(H_kv * g, seed=11, batch=2, dtype=torch.float16)
    table = DecodeTable(layers, nvs, H_kv * g)
    want = packed_decode_attention(q.cuda(), table)
    for i, (ol, onv) in enumerate(ols):
        assert_attn_close(to_np(want[i]), RA.decode_attention(q[i].float().numpy(), ol, onv)[0], f"unsplit view {i}")
    for parts in (2, 3):
        recs = []
        for part in range(parts):
            win = sharding.row_window(part, parts, table.unit_rows)
            rec = torch.empty((2 * H_kv * g, 132), device="cuda")
            packed_decode_attention(q.cuda(), table, out_partial=rec, rows=win)
            recs.append(rec)
            for i, (ol, onv) in enumerate(ols):                # the window alone against the oracle's window
                o, m, l = RA.decode_attention(q[i].float().numpy(), ol, onv, rows=win)
                r = to_np(rec).reshape(2, H_kv * g, 132)[i]
                live = l > 0
                got = np.where(live[:, None], r[:, 4:] / np.maximum(r[:, 1], 1e-30)[:, None], 0)
                assert_attn_close(got[live], o[live], f"window {win} view {i}")
                assert np.array_equal(np.isfinite(r[:, 0]), live)
        got = lse_combine(torch.stack(recs, dim=1)).view(2, H_kv * g, 128)
        assert float((got - want).abs().max()) < 2e-4, parts
        # the sequence split proper: part i of n of every phase of every head, alone against the
        # oracle's part, with and without a row window inside the part, and merged
        recs = []
        for part in range(parts):
            rec = torch.empty((2 * H_kv * g, 132), device="cuda")
            packed_decode_attention(q.cuda(), table, out_partial=rec, seq_part=(part, parts))
            recs.append(rec)
            for i, (ol, onv) in enumerate(ols):
                o, m, l = RA.decode_attention(q[i].float().numpy(), ol, onv, seq_part=(part, parts))
                r = to_np(rec).reshape(2, H_kv * g, 132)[i]
                live = l > 0
                got_i = np.where(live[:, None], r[:, 4:] / np.maximum(r[:, 1], 1e-30)[:, None], 0)
                assert_attn_close(got_i[live], o[live], f"part {part}/{parts} view {i}")
                assert np.array_equal(np.isfinite(r[:, 0]), live)
        got = lse_combine(torch.stack(recs, dim=1)).view(2, H_kv * g, 128)
        assert float((got - want).abs().max()) < 2e-4, parts
        halves = [torch.empty((2 * H_kv * g, 132), device="cuda") for _ in range(2)]
        packed_decode_attention(q.cuda(), table, out_partial=halves[0], seq_part=(0, parts), rows=(0, 128))
        packed_decode_attention(q.cuda(), table, out_partial=halves[1], seq_part=(0, parts), rows=(128, 1 << 20))
        both = lse_combine(torch.stack(halves, dim=1))     # two windows of part 0 = part 0
        r0 = recs[0]
        alone = torch.where(r0[:, 1:2] > 0, r0[:, 4:] / r0[:, 1:2].clamp_min(1e-30), torch.zeros_like(r0[:, 4:]))
        assert float((both - alone).abs().max()) < 2e-4, parts
    table.check_status()
    with pytest.raises(ValueError):
        packed_decode_attention(q.cuda(), table, rows=(5, 2))


def test_persistent_form_equals_the_one_item_form():
    """One resident CTA per slot walking the work items gives bit for bit what one CTA per item
    gives: whole units, chunked units, a mix, sequence parts and un-normalised records, ragged heads
    and heads without rows, few items and more items than CTA slots, called twice."""
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, packed_decode_attention
    from rdkv_b200.packing import pack_kv
    H_kv, g, T = 4, 4, 1024
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    base = []
    for i, ragged in enumerate((None, [400, 64, 0, 333], [17, 512, 256, 1], None, [0, 0, 480, 480])):
        seed = synth.unit_seed(8, i, 5)
        K, V = synth.make_kv(H_kv, T, seed=seed)
        vb = synth.make_v_bits(H_kv, T, 512, seed=seed, per_head_N=ragged)
        kb = synth.make_k_bits(H_kv, seed=seed)
        base.append(pack_kv(K.cuda(), V.cuda(), vb.cuda(), kb.cuda(), g, build_mask=False))
    for n_views in (3, (3 * sms) // H_kv + 7):
        layers = [base[i % len(base)][0] for i in range(n_views)]
        nvs = [base[i % len(base)][1] for i in range(n_views)]
        q = synth.make_q(H_kv * g, seed=13, batch=n_views, dtype=torch.bfloat16).cuda()
        for forced in (None, 1, 3):
            one = DecodeTable(layers, nvs, H_kv * g, n_chunks=forced, persistent=False)
            per = DecodeTable(layers, nvs, H_kv * g, n_chunks=forced, persistent=True)
            assert per._all_fast
            for rep in range(2):
                a = packed_decode_attention(q, one)
                b = packed_decode_attention(q, per)
                assert torch.equal(a, b), (n_views, forced, rep, float((a - b).abs().max()))
            ra = torch.empty((n_views * H_kv * g, 132), device="cuda")
            rb = torch.empty_like(ra)
            packed_decode_attention(q, one, out_partial=ra, seq_part=(1, 2))
            packed_decode_attention(q, per, out_partial=rb, seq_part=(1, 2))
            assert torch.equal(ra, rb), (n_views, forced)
            one.check_status(); per.check_status()
            assert int(per.unit_ctr.abs().sum().item()) == 0


def test_v_rows_through_tensor_maps_equal_the_lane_copies():
    """The 8-bit and fp16 V rows of a tile reach shared memory as one tiled TMA box where the table
    has tensor maps, and by 16-byte copies of the staging warp at the same pitch where it has none:
    both ways, in both kernel forms, give the same bits (ragged heads, heads without rows)."""
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, packed_decode_attention
    from rdkv_b200.packing import pack_kv
    H_kv, g, T = 4, 4, 2048
    layers, nvs = [], []
    for i, ragged in enumerate((None, [700, 64, 0, 333], [17, 1024, 256, 1], [0, 0, 480, 480])):
        seed = synth.unit_seed(11, i, 3)
        K, V = synth.make_kv(H_kv, T, seed=seed)
        vb = synth.make_v_bits(H_kv, T, 1024, seed=seed, per_head_N=ragged)
        kb = synth.make_k_bits(H_kv, seed=seed)
        pl, nv = pack_kv(K.cuda(), V.cuda(), vb.cuda(), kb.cuda(), g, build_mask=False)
        layers.append(pl); nvs.append(nv)
    q = synth.make_q(H_kv * g, seed=5, batch=len(layers), dtype=torch.float16).cuda()
    for persistent in (False, True):
        mapped = DecodeTable(layers, nvs, H_kv * g, persistent=persistent)
        assert mapped.n_v_maps > 0 and mapped._all_fast
        want = packed_decode_attention(q, mapped)
        plain = DecodeTable(layers, nvs, H_kv * g, persistent=False)
        plain.v_maps = None                                   # a table without maps: rows by lane copies
        plain.refresh()
        recs = plain.unit_recs.view(torch.int32).view(-1, plain._unit_rec_bytes // 4)
        assert int((recs[:, 4] & 2).sum().item()) == 0 or int(recs[:, 14::16].max().item()) < 0
        got = packed_decode_attention(q, plain)
        assert torch.equal(want, got), (persistent, float((want - got).abs().max()))
        mapped.check_status(); plain.check_status()


def test_cached_views_follow_reassigned_fields_and_counts_rewritten_in_place():
    """The one-view tables that the layer-level operators cache on the layer object are keyed by the
    identity of every tensor they point into: a field that is re-assigned (another packing of the
    same shape) is seen by the next call; per-head counts rewritten in place are read at launch."""
    import dataclasses
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, packed_decode_attention, packed_layer_attention
    from rdkv_b200.k_kernel import k_mixed_qk_dot
    from rdkv_b200.packing import pack_kv
    from rdkv_b200.v_kernel import v_dequant_weighted_sum_dispatch
    H_kv, g, T, N = 2, 4, 512, 256
    packs = []
    for i in range(2):
        seed = synth.unit_seed(9, i, 1)
        K, V = synth.make_kv(H_kv, T, seed=seed)
        packs.append(pack_kv(K.cuda(), V.cuda(), synth.make_v_bits(H_kv, T, N, seed=seed).cuda(),
                             synth.make_k_bits(H_kv, seed=seed).cuda(), g))
    (pa, nva), (pb, nvb) = packs
    q = synth.make_q(H_kv * g, seed=3).cuda()
    w = torch.softmax(torch.randn(H_kv * g, pa.T_eff_k, device="cuda"), dim=-1)
    want_b = packed_layer_attention(q, pb, nvb).clone()
    want_sb = k_mixed_qk_dot(q, pb, pb.T_eff_k).clone()
    want_vb = v_dequant_weighted_sum_dispatch(w, pb, V16=nvb[0], n_v16_per_head=pb.n_v16_per_head, max_T_v=pb.T_eff).clone()
    out_a = packed_layer_attention(q, pa, nva).clone()
    k_mixed_qk_dot(q, pa, pa.T_eff_k)
    v_dequant_weighted_sum_dispatch(w, pa, V16=nva[0], n_v16_per_head=pa.n_v16_per_head, max_T_v=pa.T_eff)
    assert not torch.equal(out_a, want_b)
    for f in dataclasses.fields(pb):                        # the same object now holds the other packing
        setattr(pa, f.name, getattr(pb, f.name))
    assert torch.equal(packed_layer_attention(q, pa, nvb), want_b)
    assert torch.equal(k_mixed_qk_dot(q, pa, pa.T_eff_k), want_sb)
    assert torch.equal(v_dequant_weighted_sum_dispatch(w, pa, V16=nvb[0], n_v16_per_head=pa.n_v16_per_head,
                                                       max_T_v=pa.T_eff), want_vb)
    # counts rewritten in place: the layer-level call reads them at every launch; a table snapshots
    # them and follows after refresh()
    table = DecodeTable([pb], [nvb], H_kv * g)
    before = packed_decode_attention(q[None], table).clone()
    pb.seg_bounds_per_head[0, 2] -= 32                      # head 0 loses its last 32 8-bit rows
    layer_level = packed_layer_attention(q, pb, nvb).clone()
    assert not torch.equal(layer_level, before[0])
    assert torch.equal(packed_decode_attention(q[None], table), before)        # snapshot: unchanged until refreshed
    table.refresh()
    assert torch.equal(packed_decode_attention(q[None], table)[0], layer_level)
    pb.seg_bounds_per_head[0, 2] += 32


def test_host_buffer_call_equals_device_call():
    """The host-buffer form (view ranges on separate streams, copies overlapped with the
    kernels) returns bit-for-bit what the device call returns, for one-chunk tables and
    for split-sequence tables, whatever the number of ranges."""
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, packed_decode_attention, packed_decode_attention_host
    from rdkv_b200.packing import pack_kv
    H_kv, g = 4, 4
    layers, nvs = [], []
    for i in range(7):
        seed = synth.unit_seed(5, i, 1)
        T, N = 1536 + 64 * i, 640 + 32 * i
        K, V = synth.make_kv(H_kv, T, seed=seed)
        pl, nv = pack_kv(K.cuda(), V.cuda(), synth.make_v_bits(H_kv, T, N, seed=seed).cuda(),
                         synth.make_k_bits(H_kv, seed=seed).cuda(), g)
        layers.append(pl)
        nvs.append(nv)
    q = synth.make_q(H_kv * g, seed=2, batch=7, dtype=torch.bfloat16)
    for n_chunks in (1, 3):                                # one chunk per head (direct write) / split sequence
        table = DecodeTable(layers, nvs, H_kv * g)
        table.n_chunks, table.chunk_rows = n_chunks, 64 * (-(-table.max_t_k // (64 * n_chunks)))
        want = packed_decode_attention(q.cuda(), table).cpu()
        q_host = q.pin_memory()
        for slices in (1, 3, 7, 50):
            for pinned in (True, False):                   # pinned: written by the kernels; pageable: copied per range
                out_host = torch.full((7, H_kv * g, 128), float("nan"))
                if pinned:
                    out_host = out_host.pin_memory()
                got = packed_decode_attention_host(q_host, table, out_host, slices=slices)
                assert got is out_host
                assert torch.equal(out_host, want), (n_chunks, slices, pinned)
        table.check_status()
    with pytest.raises(ValueError):
        packed_decode_attention_host(q.cuda(), table, out_host)


def test_host_buffer_call_replayed_as_a_graph_follows_the_buffers_contents():
    """With pinned buffers the second call records the ranges' copies and launches as one graph and
    later calls replay it: every call returns what the device call returns for the queries that
    are in the buffer at that time; other buffers drop the recording."""
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, packed_decode_attention, packed_decode_attention_host
    from rdkv_b200.packing import pack_kv
    H_kv, g = 4, 4
    layers, nvs = [], []
    for i in range(9):
        seed = synth.unit_seed(6, i, 1)
        T, N = 1280 + 64 * i, 512 + 32 * i
        K, V = synth.make_kv(H_kv, T, seed=seed)
        pl, nv = pack_kv(K.cuda(), V.cuda(), synth.make_v_bits(H_kv, T, N, seed=seed).cuda(),
                         synth.make_k_bits(H_kv, seed=seed).cuda(), g)
        layers.append(pl)
        nvs.append(nv)
    table = DecodeTable(layers, nvs, H_kv * g)
    q_host = torch.empty((9, H_kv * g, 128), dtype=torch.bfloat16).pin_memory()
    out_host = torch.empty((9, H_kv * g, 128)).pin_memory()
    for step in range(5):                                  # stream form, recording, three replays
        q = synth.make_q(H_kv * g, seed=10 + step, batch=9, dtype=torch.bfloat16)
        q_host.copy_(q)
        out_host.fill_(float("nan"))
        packed_decode_attention_host(q_host, table, out_host, slices=3)
        assert torch.equal(out_host, packed_decode_attention(q.cuda(), table).cpu()), step
        assert len(table._host_io.graphs) == (1 if step >= 1 else 0)
    other = torch.empty_like(out_host).pin_memory()
    packed_decode_attention_host(q_host, table, other, slices=3)
    assert torch.equal(other, out_host)
    for in_place in (0, 2, 3):                             # ranges whose kernels read the pinned queries themselves
        for _ in range(3):
            other.fill_(float("nan"))
            packed_decode_attention_host(q_host, table, other, slices=3, in_place=in_place)
            assert torch.equal(other, out_host), in_place
    table.refresh()                                        # drops the recordings
    assert not hasattr(table, "_host_io")
    packed_decode_attention_host(q_host, table, out_host, slices=3, graph=False)
    assert torch.equal(other, out_host)
    with pytest.raises(ValueError):
        packed_decode_attention_host(q_host, table, torch.empty_like(out_host), graph=True)
    table.check_status()


def test_lse_combine_matches_oracle():
    from oracle import ref_attention as RA
    from rdkv_b200.decode import lse_combine
    rng = np.random.default_rng(3)
    S, R = 5, 37
    m = rng.normal(size=(S, R)).astype(np.float32) * 4
    m[1, :7] = -np.inf
    m[:, 9] = -np.inf                      # a row with no live token anywhere
    l = rng.uniform(0.5, 30, size=(S, R)).astype(np.float32)
    l[~np.isfinite(m)] = 0
    o = rng.normal(size=(S, R, 128)).astype(np.float32) * l[..., None]
    o[~np.isfinite(m)] = 0
    rec = np.zeros((R, S, 132), np.float32)
    rec[:, :, 0], rec[:, :, 1], rec[:, :, 4:] = m.T, l.T, o.transpose(1, 0, 2)
    want, wM, wL = RA.lse_combine(m, l, o)
    ml = torch.empty((R, 2), device="cuda")
    got = lse_combine(cuda(rec), out_ml=ml)
    want[9] = 0
    np.testing.assert_allclose(to_np(got), want, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(to_np(ml)[:, 1], wL, rtol=2e-5)
    assert np.array_equal(to_np(ml)[:, 0], wM)


def test_full_size_linearity_and_permutation():
    """Config-3 unit size (budget 2048, g=4) and config-4 unit size (budget 8192, g=8):
    properties that need no oracle pass — linearity of the V side in the weights, a
    softmax row summing to one (l check) and agreement of fused vs two-stage paths."""
    from rdkv_b200 import synth
    from rdkv_b200.decode import packed_layer_attention
    from rdkv_b200.k_kernel import k_mixed_qk_dot
    from rdkv_b200.packing import pack_kv
    from rdkv_b200.v_kernel import v_dequant_weighted_sum_dispatch
    for (H_kv, g, T, N) in ((8, 4, 8192, 2048), (2, 8, 16384, 8192)):
        seed = synth.unit_seed(3 if g == 4 else 4)
        K, V = synth.make_kv(H_kv, T, seed=seed, device="cuda")
        vb = synth.make_v_bits(H_kv, T, N, seed=seed, device="cuda")
        kb = synth.make_k_bits(H_kv, seed=seed, device="cuda")
        pl, nv = pack_kv(K, V, vb, kb, g)
        q = synth.make_q(H_kv * g, seed=seed + 1, device="cuda")
        fused = packed_layer_attention(q, pl, nv)
        s = k_mixed_qk_dot(q, pl, pl.T_eff_k) + pl.softmax_mask
        w = torch.softmax(s, dim=-1)
        two = v_dequant_weighted_sum_dispatch(w, pl, V16=nv[0], n_v16_per_head=pl.n_v16_per_head, max_T_v=pl.T_eff)
        assert_attn_close(to_np(fused), to_np(two), f"fused vs two-stage g={g}")
        w2 = torch.softmax(s * 0.5, dim=-1)
        a = v_dequant_weighted_sum_dispatch(w, pl, V16=nv[0], n_v16_per_head=pl.n_v16_per_head, max_T_v=pl.T_eff)
        b = v_dequant_weighted_sum_dispatch(w2, pl, V16=nv[0], n_v16_per_head=pl.n_v16_per_head, max_T_v=pl.T_eff)
        ab = v_dequant_weighted_sum_dispatch(0.25 * w + 0.75 * w2, pl, V16=nv[0],
                                             n_v16_per_head=pl.n_v16_per_head, max_T_v=pl.T_eff)
        # (the weights enter the tensor-core product as fp16 pairs, as in the reference's V kernel:
        #  linear up to that rounding)
        assert_attn_close(to_np(ab), to_np(0.25 * a + 0.75 * b), f"linearity g={g}")
        # an exact reference for this size on the GPU-resident dequantised values of one head
        from oracle import ref_packing as RP
        layer = {k: to_np(v) if torch.is_tensor(v) else v for k, v in vars(pl).items()}
        Khat = RP.unpack_k(layer, 128)[0, 0].astype(np.float32)
        Vhat = RP.unpack_v(layer, to_np(nv), 128)[0, 0].astype(np.float32)
        qq = to_np(q[:g].float())
        sc = qq @ Khat.T / np.sqrt(np.float32(128)) + layer["softmax_mask"][:g]
        p = np.exp(sc - sc.max(1, keepdims=True))
        ref = (p / p.sum(1, keepdims=True)) @ Vhat
        assert_attn_close(to_np(fused[:g]), ref, f"head 0 vs dequantise-then-attend g={g}")
