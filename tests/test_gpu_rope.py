"""Rotary embedding of a decode step (through the C ABI) against vectors from the reference's own
fused_rope_ref, bit for bit, and the one-launch attention block (rotation, new token, uncompressed
tail, packed zones) against the oracle."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from helpers import assert_attn_close, cuda, to_np

pytestmark = pytest.mark.gpu

_DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def _tensor(bits, tag):
    t = torch.from_numpy(np.ascontiguousarray(bits))
    return (t.view(torch.int16).view(torch.bfloat16) if tag == "bf16" else t).cuda()


def _bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)   # fp16 and bf16 alike: the 16-bit patterns


@pytest.mark.parametrize("tag", ["f16", "bf16"])
@pytest.mark.parametrize("cs", ["same", "f32"])
def test_fused_rope_is_bit_exact(tag, cs):
    from rdkv_b200.rope import fused_rope
    g = load_golden("rope.npz")
    key = f"{tag}_{cs}_"
    cs_tag = tag if cs == "same" else "f32"
    q, k = _tensor(g[key + "q"], tag), _tensor(g[key + "k"], tag)
    cos, sin = _tensor(g[key + "cos"], cs_tag), _tensor(g[key + "sin"], cs_tag)
    q2, k2 = fused_rope(q, k, cos, sin)
    assert q2 is q and k2 is k                             # in place, as the reference's kernel
    assert np.array_equal(_bits(q), g[key + "q_out"].view(np.uint16))
    assert np.array_equal(_bits(k), g[key + "k_out"].view(np.uint16))
    # rows of a wider tensor (row stride > 128)
    wide = torch.zeros(12, 200, dtype=_DT[tag], device="cuda")
    wide[:, :128] = _tensor(g[key + "q"], tag)
    fused_rope(wide[:, :128], k2[:0], cos, sin)
    assert torch.equal(wide[:, :128], q) and torch.all(wide[:, 128:] == 0)
    with pytest.raises(ValueError):
        fused_rope(q[:, :64], k, cos, sin)


def _case(kv_dtype, n_views, tails, cap, seed, H_kv=4, g=4):
    """Packed layers, tail buffers, the new token's rows and rotation tables for n_views views, and
    per view the oracle's result of the whole block."""
    from oracle import ref_attention as RA
    from oracle import ref_packing as RP
    from oracle import ref_rope as RR
    from rdkv_b200 import synth
    from rdkv_b200.packing import pack_kv
    tag = "bf16" if kv_dtype == torch.bfloat16 else "f16"
    gen = torch.Generator().manual_seed(seed)
    q = synth.make_q(H_kv * g, seed=seed, batch=n_views, dtype=kv_dtype)
    new_k = torch.randn(n_views, H_kv, cap, 128, generator=gen).to(kv_dtype)
    new_v = torch.randn(n_views, H_kv, cap, 128, generator=gen).to(kv_dtype)
    k_cur = torch.randn(n_views, H_kv, 128, generator=gen).to(kv_dtype)
    v_cur = torch.randn(n_views, H_kv, 128, generator=gen).to(kv_dtype)
    pos = torch.rand(n_views, 64, generator=gen) * 500.0
    cos, sin = torch.cos(pos), torch.sin(pos)              # fp32 tables, one per view
    as_np = lambda t: (t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy())
    f32 = lambda bits: RR.to_f32(bits, tag)
    layers, nvs, wants, k_rot = [], [], [], []
    for i in range(n_views):
        T, N = 768 + 128 * (i % 3), 256 + 64 * (i % 4)
        s = synth.unit_seed(11, i, seed)
        K, V = synth.make_kv(H_kv, T, seed=s)
        vb, kb = synth.make_v_bits(H_kv, T, N, seed=s), synth.make_k_bits(H_kv, seed=s)
        pl, nv = pack_kv(K.cuda(), V.cuda(), vb.cuda(), kb.cuda(), g)
        layers.append(pl); nvs.append(nv)
        ol, onv = RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g)
        q_r, k_r = RR.fused_rope(as_np(q[i]), as_np(k_cur[i]), cos[i].numpy(), sin[i].numpy(), tag, "f32")
        k_rot.append(k_r)
        tk = np.concatenate([f32(as_np(new_k[i, :, :tails[i]])), f32(k_r)[:, None]], axis=1)
        tv = np.concatenate([f32(as_np(new_v[i, :, :tails[i]])), f32(as_np(v_cur[i]))[:, None]], axis=1)
        wants.append(RA.decode_attention(f32(q_r), ol, onv, tk, tv)[0])
    return dict(q=q, new_k=new_k, new_v=new_v, k_cur=k_cur, v_cur=v_cur, cos=cos, sin=sin, layers=layers, nvs=nvs,
                wants=wants, k_rot=k_rot, H_q=H_kv * g, as_np=as_np)


@pytest.mark.parametrize("kv_dtype", [torch.float16, torch.bfloat16])
def test_one_launch_block_with_rotation_new_token_and_tail(kv_dtype):
    """Rotation of q and the new key row, the new token, 1024 / 0 / 333 / 40 tail rows and the packed
    zones in one launch: against the oracle; the appended rows are the rotated key row and the value
    row bit for bit; whole units and chunked units; per-view counts on the device."""
    from rdkv_b200.decode import DecodeTable, packed_decode_attention
    tails, cap = [1024, 0, 333, 40], 1030
    c = _case(kv_dtype, 4, tails, cap, seed=5)
    n_dev = torch.tensor(tails, dtype=torch.int32, device="cuda")
    for n_chunks in (None, 3):
        new_k, new_v = c["new_k"].cuda(), c["new_v"].cuda()
        table = DecodeTable(c["layers"], c["nvs"], c["H_q"], n_chunks=n_chunks)
        q_dev = c["q"].cuda()
        out = packed_decode_attention(q_dev, table, new_k=new_k, new_v=new_v, n_new=n_dev, k_cur=c["k_cur"].cuda(),
                                      v_cur=c["v_cur"].cuda(), rope=(c["cos"].cuda(), c["sin"].cuda()))
        assert torch.equal(q_dev.cpu(), c["q"])            # the caller's queries are not written
        for i, w in enumerate(c["wants"]):
            assert_attn_close(to_np(out[i]), w, f"{kv_dtype} chunks {n_chunks} view {i}")
            assert np.array_equal(_bits(new_k[i, :, tails[i]]), c["k_rot"][i].view(np.uint16)), (n_chunks, i)
            assert torch.equal(new_v[i, :, tails[i]].cpu(), c["v_cur"][i])
            assert torch.equal(new_k[i, :, :tails[i]].cpu(), c["new_k"][i, :, :tails[i]])
        table.check_status()


def test_one_launch_block_with_more_query_heads_than_a_cta_takes():
    """16 query heads per KV head: two CTAs per (view, KV head), each with eight of the heads; both
    seed their softmax with the new token, one of them appends its rows."""
    from rdkv_b200.decode import DecodeTable, packed_decode_attention
    tails, cap = [70, 5], 80
    c = _case(torch.float16, 2, tails, cap, seed=13, H_kv=2, g=16)
    new_k, new_v = c["new_k"].cuda(), c["new_v"].cuda()
    table = DecodeTable(c["layers"], c["nvs"], c["H_q"])
    out = packed_decode_attention(c["q"].cuda(), table, new_k=new_k, new_v=new_v,
                                  n_new=torch.tensor(tails, dtype=torch.int32, device="cuda"), k_cur=c["k_cur"].cuda(),
                                  v_cur=c["v_cur"].cuda(), rope=(c["cos"].cuda(), c["sin"].cuda()))
    for i, w in enumerate(c["wants"]):
        assert_attn_close(to_np(out[i]), w, f"g=16 view {i}")
        assert np.array_equal(_bits(new_k[i, :, tails[i]]), c["k_rot"][i].view(np.uint16))
    table.check_status()


def test_one_launch_block_equals_the_separate_steps():
    """The same block as separate steps (fused_rope on copies, append by hand, packed zones + tail
    kernel + combine) and in one launch; a shared integer count; sequence parts merged afterwards."""
    from rdkv_b200.decode import DecodeTable, lse_combine, packed_decode_attention
    from rdkv_b200.rope import fused_rope
    n = 200
    c = _case(torch.float16, 2, [n, n], n + 8, seed=9)
    table = DecodeTable(c["layers"], c["nvs"], c["H_q"])
    cos, sin = c["cos"][0].cuda(), c["sin"][0].cuda()     # one table for both views
    k1, v1 = c["new_k"].cuda(), c["new_v"].cuda()
    one = packed_decode_attention(c["q"].cuda(), table, new_k=k1, new_v=v1, n_new=n, k_cur=c["k_cur"].cuda(),
                                  v_cur=c["v_cur"].cuda(), rope=(cos, sin))
    q2, kc = c["q"].cuda().clone(), c["k_cur"].cuda().clone()
    fused_rope(q2.view(-1, 128), kc.view(-1, 128), cos, sin)
    k2, v2 = c["new_k"].cuda(), c["new_v"].cuda()
    k2[:, :, n], v2[:, :, n] = kc, c["v_cur"].cuda()
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    sep = packed_decode_attention(q2, table, new_k=k2, new_v=v2, n_new=n + 1, one_launch=False)
    np.testing.assert_allclose(to_np(one), to_np(sep), rtol=2e-2, atol=2e-3)
    again = packed_decode_attention(q2, table, new_k=k2, new_v=v2, n_new=n + 1)     # tail only, one launch
    np.testing.assert_allclose(to_np(again), to_np(sep), rtol=2e-2, atol=2e-3)
    # two sequence parts of the same block, merged by the combine kernel
    recs = torch.empty((2, 2 * c["H_q"], 132), device="cuda")
    for part in range(2):
        packed_decode_attention(q2, table, new_k=k2, new_v=v2, n_new=n + 1, seq_part=(part, 2), out_partial=recs[part])
    merged = lse_combine(recs.permute(1, 0, 2).contiguous())
    np.testing.assert_allclose(to_np(merged).reshape(2, c["H_q"], 128), to_np(again), rtol=2e-2, atol=2e-3)
    with pytest.raises(ValueError):                        # fp32 tail buffers take the separate kernels only
        packed_decode_attention(q2, table, new_k=k2.float(), new_v=v2.float(), n_new=n, k_cur=kc, v_cur=kc)
    table.check_status()
