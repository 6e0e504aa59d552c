"""Bit-exact parity of the CUDA quantise-and-bitpack path (through the C ABI) with
the reference-generated golden vectors and with the numpy oracle."""
import numpy as np
import pytest
import torch

from conftest import assert_layer_equal, sub
from helpers import cuda, layer_to_np, to_np

pytestmark = pytest.mark.gpu


def _pack_kv_gpu(K, V, v_bits, k_bits, g, **kw):
    from rdkv_b200.packing import pack_kv
    return pack_kv(cuda(K), cuda(V), cuda(v_bits), cuda(k_bits), g, **kw)


def test_reference_unit_case_segment_packing(golden_unit):
    """Inputs of the reference's own segment-count test: pack_k_mixed and pack_v_segments
    with and without precomputed counts give the golden tensors."""
    from rdkv_b200.packing import pack_k_mixed, pack_v_segments
    g = sub(golden_unit, "t1")
    for counts in (None, (2, 2, 3)):
        k = pack_k_mixed(cuda(g["keys"]), cuda(g["k_bits"]), segment_counts=counts)
        for name, got in zip(["K_2bit", "K_4bit", "K_8bit", "K_ch_scale", "K_ch_zp", "K_ch_sort_idx",
                              "K_ch_perm_padded_idx"], k[:7]):
            assert np.array_equal(to_np(got), g[name]), name
        assert k[7] == (2, 2, 3)
    for counts in (None, (2, 2, 2)):
        v = pack_v_segments(cuda(g["values"]), cuda(g["v_bits"]), segment_counts=counts)
        for name, got in zip(["V_2bit", "V_4bit", "V_8bit", "V_scale", "V_zp", "sort_idx"], v[:6]):
            assert np.array_equal(to_np(got), g[name]), name
        assert v[6] == (2, 2, 2)


def test_reference_unit_case_deferred_k_stack(golden_unit):
    """The reference's ragged-head test (bits {0,2,4,8,16}, D=8) through the same call
    sequence: per-head build_packed_layer with deferred K, then pad-and-stack."""
    from rdkv_b200.packing import _pad_and_stack_per_head_layers, build_packed_layer
    g = sub(golden_unit, "t2")
    keys, values = cuda(g["keys"]), cuda(g["values"])
    v_bits, k_bits = cuda(g["v_bits"]), cuda(g["k_bits"])
    layers, v16s = [], []
    for h in range(2):
        kept = (v_bits[h] > 0).nonzero(as_tuple=True)[0]
        kb = v_bits[h].index_select(0, kept)
        counts = tuple(int((kb == b).sum()) for b in (2, 4, 8))
        layer, _, v16 = build_packed_layer(keys[:, h:h + 1].index_select(2, kept),
                                           values[:, h:h + 1].index_select(2, kept), kb, k_bits[h],
                                           v_segment_counts=counts, defer_k_for_per_head_stack=True)
        assert layer.deferred_k_for_stack is not None
        layers.append(layer)
        v16s.append(v16)
    packed, nv = _pad_and_stack_per_head_layers(layers, v16s, H_q=4, gqa_factor=2, head_dim=8,
                                                device=keys.device, dtype=keys.dtype, k_bits_per_head=k_bits)
    assert_layer_equal(layer_to_np(packed), g, "stack.")
    assert np.array_equal(to_np(nv), g["new_v_only"])
    assert packed.deferred_k_for_stack is None
    # the one-pass composite gives the same layer
    packed2, nv2 = _pack_kv_gpu(g["keys"], g["values"], g["v_bits"], g["k_bits"], 2)
    assert_layer_equal(layer_to_np(packed2), g, "pack_kv.")
    assert np.array_equal(to_np(nv2), g["new_v_only"])
    assert np.array_equal(to_np(packed2.sort_idx), g["sort_idx"])
    assert np.array_equal(to_np(packed2.K_ch_sort_idx), g["K_ch_sort_idx"])
    assert np.array_equal(to_np(packed2.K_ch_perm_padded_idx), g["K_ch_perm_padded_idx"])


def test_shared_layout_stacking_matches_reference_vectors():
    """The reference's shared layout (one K bit map for all heads, every head's K quantised on its own
    rows, packed bytes copied into the stripe: packing.py:1019-1317 without k_bits_per_head): layer
    fields bit for bit, and the fused kernel, the two-stage operators and the decompressor on such a
    layer against the reference's dequantise-then-attend output."""
    from conftest import load_golden
    from helpers import assert_attn_close
    from rdkv_b200.decode import packed_layer_attention
    from rdkv_b200.decompress import unpack_trizone_to_past_kv
    from rdkv_b200.packing import TriZoneCache, _pad_and_stack_per_head_layers, build_packed_layer
    g = load_golden("legacy.npz")
    K, V, v_bits, k_bits = cuda(g["K"]), cuda(g["V"]), cuda(g["v_bits"]), cuda(g["k_bits"])
    H = K.shape[1]
    layers, v16s = [], []
    for h in range(H):
        kept = (v_bits[h] > 0).nonzero(as_tuple=True)[0]
        kb = v_bits[h].index_select(0, kept)
        counts = tuple(int((kb == b).sum()) for b in (2, 4, 8))
        layer, _, v16 = build_packed_layer(K[:, h:h + 1].index_select(2, kept), V[:, h:h + 1].index_select(2, kept),
                                           kb, k_bits, v_segment_counts=counts)
        layers.append(layer)
        v16s.append(v16)
    packed, nv = _pad_and_stack_per_head_layers(layers, v16s, H_q=2 * H, gqa_factor=2, head_dim=128,
                                                device=K.device, dtype=K.dtype)
    assert_layer_equal(layer_to_np(packed), g, "shared.")
    assert np.array_equal(to_np(nv), g["new_v_only"])
    assert packed.K_ch_perm_padded_idx_for_Q is None and packed.K_ch_sort_idx_per_head is None
    for name in ("K_ch_sort_idx", "K_ch_perm_padded_idx", "sort_idx"):
        assert np.array_equal(to_np(getattr(packed, name)), g[name]), name
    out = packed_layer_attention(cuda(g["q"]), packed, nv, use_mask=True)
    assert_attn_close(to_np(out), g["attn_out"], "shared layout, fused kernel")
    cache = TriZoneCache(packed=(packed,), new_v_only=[nv], new_both_k=[None], new_both_v=[None], original_seq_len=0)
    (K_hat, V_hat), = unpack_trizone_to_past_kv(cache, head_dim=128)
    assert np.array_equal(to_np(K_hat), g["K_hat"]) and np.array_equal(to_np(V_hat), g["V_hat"])


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
def test_pack_kv_matches_golden(golden_layers, tag):
    g = sub(golden_layers, tag)
    packed, nv = _pack_kv_gpu(g["K"], g["V"], g["v_bits"], g["k_bits"], int(g["g"]))
    assert_layer_equal(layer_to_np(packed), g, tag + ".")
    if "new_v_only" in g:
        assert np.array_equal(to_np(nv), g["new_v_only"])
    else:
        assert nv is None
    assert np.array_equal(to_np(packed.sort_idx), g["sort_idx"])


def test_quantize_and_pack_both_axes(golden_layers):
    from oracle import ref_packing as RP
    from rdkv_b200.packing import quantize_and_pack
    g = sub(golden_layers, "even")
    x = g["K"][:, :, :200]
    for bits in (2, 4, 8):
        for dim in (2, 3):
            c, s, z = quantize_and_pack(cuda(x), bits, dim)
            rc, rs, rz = RP.quantize(x, bits, dim)
            assert np.array_equal(to_np(c), rc), (bits, dim)
            assert np.array_equal(to_np(s), rs) and np.array_equal(to_np(z), rz), (bits, dim)


def test_build_packed_layer_shared_and_per_head_k(golden_layers):
    """Heads sharing one token map: [D] and [H,D] channel maps against the oracle."""
    from oracle import ref_packing as RP
    from rdkv_b200.packing import build_packed_layer
    from rdkv_b200 import synth
    g = sub(golden_layers, "ragged")
    K, V = g["K"], g["V"]
    H = K.shape[1]
    v_bits = g["v_bits"][0]
    kb_ph = g["k_bits"]
    # per-head channel maps
    pl, t_k, v16 = build_packed_layer(cuda(K), cuda(V), cuda(v_bits), cuda(kb_ph), gqa_factor=2)
    want, want_nv = RP.pack_kv(K, V, np.repeat(v_bits[None], H, 0), kb_ph, 2)
    got = layer_to_np(pl)
    for f in ["K_2bit", "K_4bit", "K_8bit", "K_ch_scale", "K_ch_zp", "V_2bit", "V_4bit", "V_8bit", "V_scale",
              "V_zp", "K_ch_perm_padded_idx_for_Q", "K_ch_seg_bounds_per_head", "K_ch_sort_idx_per_head"]:
        assert np.array_equal(got[f], want[f]), f
    assert t_k == want["T_eff_k"] and np.array_equal(to_np(v16), want_nv)
    # one channel map for all heads
    pl1, _, _ = build_packed_layer(cuda(K), cuda(V), cuda(v_bits), cuda(kb_ph[0]))
    want1, _ = RP.pack_kv(K, V, np.repeat(v_bits[None], H, 0), np.repeat(kb_ph[:1], H, 0), 2)
    got1 = layer_to_np(pl1)
    for f in ["K_2bit", "K_4bit", "K_8bit", "K_ch_scale", "K_ch_zp", "V_8bit", "V_scale"]:
        assert np.array_equal(got1[f], want1[f]), f
    assert np.array_equal(got1["K_ch_perm_padded_idx"], want1["K_ch_perm_padded_idx_per_head"][0])


def test_config0_layer_matches_oracle():
    """Llama-3.1-8B layer shape: 8 KV heads, context 4096, budget 1024, 64 kept channels."""
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    seed = synth.unit_seed(0)
    K, V = synth.make_kv(8, 4096, seed=seed)
    v_bits = synth.make_v_bits(8, 4096, 1024, seed=seed)
    k_bits = synth.make_k_bits(8, seed=seed)
    packed, nv = _pack_kv_gpu(K.numpy(), V.numpy(), v_bits.numpy(), k_bits.numpy(), 4)
    want, want_nv = RP.pack_kv(K.numpy(), V.numpy(), v_bits.numpy(), k_bits.numpy(), 4)
    assert_layer_equal(layer_to_np(packed), want, "cfg0.")
    assert np.array_equal(to_np(nv), want_nv)
    assert tuple(packed.K_2bit.shape) == (1, 8, 1024, 6) and tuple(packed.V_4bit.shape) == (1, 8, 384, 64)


def test_quotients_on_and_next_to_half_integers():
    """Values built so that (x - lo) / scale lands exactly on, or one fp16 step off, a half-integer for
    most elements: the rounding then depends on the last bit of the IEEE quotient.  Integer-valued rows
    with a power-of-two-ish range give exact ties; fp16 neighbours of those give the near misses."""
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    rng = np.random.default_rng(20250607)
    H, T, D = 2, 512, 128
    seed = synth.unit_seed(11)
    v_bits = synth.make_v_bits(H, T, 384, seed=seed).numpy()
    k_bits = synth.make_k_bits(H, seed=seed).numpy()

    def tie_tensor():
        # per (head, token): integers in [0, 2*qmax] for some qmax -> scale 2 (8-bit: 510/255), quotient k/2
        base = rng.integers(0, 511, size=(1, H, T, D)).astype(np.float32)
        base[..., 0] = 0.0
        base[..., 1] = 510.0          # V rows: lo 0, hi 510 -> scale 2 at 8 bits, 34 at 4 bits, 170 at 2 bits
        base[:, :, 0, :] = 0.0
        base[:, :, 1, :] = 510.0        # K channels: same range along the token axis
        x = base.astype(np.float16)
        nudge = rng.integers(-1, 2, size=x.shape).astype(np.int16)          # one fp16 step down / none / up
        nudge[..., :2] = 0
        nudge[:, :, :2, :] = 0
        nudge[base == 0.0] = 0        # (0 minus one step would be a NaN pattern)
        y = (x.view(np.int16) + nudge).view(np.float16)
        return np.ascontiguousarray(y)

    K, V = tie_tensor(), tie_tensor()
    packed, nv = _pack_kv_gpu(K, V, v_bits, k_bits, 4)
    want, want_nv = RP.pack_kv(K, V, v_bits, k_bits, 4)
    assert_layer_equal(layer_to_np(packed), want, "ties.")
    assert np.array_equal(to_np(nv), want_nv)


def test_pack_kv_layers_equals_per_layer_packing():
    """All layers in one pass: every layer bit-identical to pack_kv on that layer (tall
    shared tensors, ragged and per-layer different segment counts, strided head views),
    the decode kernel reads the views, and differing K widths fall back to per-layer packing."""
    from rdkv_b200 import synth
    from rdkv_b200.decode import DecodeTable, packed_decode_attention
    from rdkv_b200.packing import pack_kv, pack_kv_layers
    H, T, g = 4, 1536, 4
    Ks, Vs, vbs, kbs = [], [], [], []
    budgets = [(512, None), (384, [384, 200, 0, 333]), (640, [640, 640, 17, 512]), (64, None)]
    for i, (N, ragged) in enumerate(budgets):
        seed = synth.unit_seed(7, i)
        K, V = synth.make_kv(H, T, seed=seed)
        Ks.append(K.cuda()); Vs.append(V.cuda())
        vbs.append(synth.make_v_bits(H, T, N, seed=seed, per_head_N=ragged))
        kbs.append(synth.make_k_bits(H, seed=seed))
    v_bits, k_bits = torch.stack(vbs).cuda(), torch.stack(kbs).cuda()
    singles = [pack_kv(Ks[i], Vs[i], v_bits[i], k_bits[i], g) for i in range(4)]
    for k_passes in (0, 1, 3):                             # K in one pass over the kept rows (cluster) / in three
        batch = pack_kv_layers(Ks, Vs, v_bits, k_bits, g, k_passes=k_passes)
        assert len(batch) == 4
        for i, ((pl, nv), (wl, wnv)) in enumerate(zip(batch, singles)):
            assert_layer_equal(layer_to_np(pl), layer_to_np(wl), f"k_passes {k_passes} layer {i}.")
            for f in ("K_ch_sort_idx", "K_ch_perm_padded_idx", "sort_idx"):
                assert torch.equal(getattr(pl, f), getattr(wl, f)), f
            assert (nv is None) == (wnv is None) and (nv is None or torch.equal(nv, wnv))
    # the fused kernel reads the (strided) views of the batch exactly as it reads single layers
    q = synth.make_q(H * g, seed=3, batch=4, dtype=torch.float16).cuda()
    got = packed_decode_attention(q, DecodeTable([b[0] for b in batch], [b[1] for b in batch], H * g))
    want = packed_decode_attention(q, DecodeTable([b[0] for b in singles], [b[1] for b in singles], H * g))
    assert torch.equal(got, want)
    # a layer whose K bit map pads to other widths: per-layer fallback, same results
    kb2 = k_bits.clone()
    kb2[1, :, :] = 0
    kb2[1, :, :40] = 8
    batch2 = pack_kv_layers(Ks, Vs, v_bits, kb2, g, build_mask=False)
    for i in range(4):
        wl, wnv = pack_kv(Ks[i], Vs[i], v_bits[i], kb2[i], g, build_mask=False)
        assert_layer_equal(layer_to_np(batch2[i][0]), layer_to_np(wl), f"fallback layer {i}.")
    with pytest.raises(ValueError):
        pack_kv_layers(Ks, Vs[:3], v_bits, k_bits, g)


def test_edge_cases():
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    from rdkv_b200.packing import pack_kv
    K, V = synth.make_kv(2, 64, seed=5)
    # a head with no kept token, a head with only fp16 tokens, single segment classes
    v_bits = torch.zeros(2, 64, dtype=torch.long)
    v_bits[1, 5:9] = 16
    k_bits = torch.zeros(2, 128, dtype=torch.long)
    k_bits[0, :3] = 2
    k_bits[1, 7] = 16
    packed, nv = pack_kv(K.cuda(), V.cuda(), v_bits.cuda(), k_bits.cuda(), 1)
    want, want_nv = RP.pack_kv(K.numpy(), V.numpy(), v_bits.numpy(), k_bits.numpy(), 1)
    assert_layer_equal(layer_to_np(packed), want, "edge.")
    assert np.array_equal(to_np(nv), want_nv)
    # all heads empty -> error, like the reference's "kept zero tokens" failure
    with pytest.raises(RuntimeError):
        pack_kv(K.cuda(), V.cuda(), torch.zeros(2, 64, dtype=torch.long).cuda(), k_bits.cuda(), 1)
    # every channel pruned: no K segments, empty scale
    v_bits[0, :10] = 4
    packed, _ = pack_kv(K.cuda(), V.cuda(), v_bits.cuda(), torch.zeros(2, 128, dtype=torch.long).cuda(), 1)
    assert packed.K_2bit is None and packed.K_8bit is None and packed.K_ch_scale.shape[-1] == 0


def test_unaligned_strided_inputs():
    """K and V as views into wider buffers (rows start 6 bytes off, row stride not a multiple of 8
    bytes): the element-wise load paths and the unstaged K pass, per layer and all layers at once."""
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    from rdkv_b200.packing import pack_kv, pack_kv_layers
    H, T = 3, 300
    Ks, Vs, vbs, kbs, wants = [], [], [], [], []
    for layer in range(2):
        seed = synth.unit_seed(12, layer)
        K, V = synth.make_kv(H, T, seed=seed)
        vb = synth.make_v_bits(H, T, 120, seed=seed, per_head_N=[120, 90, 77])
        kb = synth.make_k_bits(H, seed=seed)
        views = []
        for x in (K, V):
            wide = torch.zeros(1, H, T, 128 + 6, dtype=x.dtype, device="cuda")
            wide[..., 3:131] = x.cuda()
            views.append(wide[..., 3:131])
            assert views[-1].data_ptr() % 8 == 6 and views[-1].stride(2) == 134
        Ks.append(views[0]); Vs.append(views[1]); vbs.append(vb.cuda()); kbs.append(kb.cuda())
        wants.append(RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), 2))
        packed, nv = pack_kv(views[0], views[1], vbs[-1], kbs[-1], 2)
        assert_layer_equal(layer_to_np(packed), wants[-1][0], f"unaligned{layer}.")
        assert np.array_equal(to_np(nv), wants[-1][1])
    for k_passes in (1, 3):
        batch = pack_kv_layers(Ks, Vs, torch.stack(vbs), torch.stack(kbs), 2, k_passes=k_passes)
        for layer in range(2):
            packed, nv = batch[layer]
            assert_layer_equal(layer_to_np(packed), wants[layer][0], f"unaligned.batched{layer}.{k_passes}.")
            assert np.array_equal(to_np(nv), wants[layer][1])


def test_one_pass_and_three_pass_k_packing_agree_at_full_size():
    """Two config-1 layers (8 heads x 32768 tokens, budget 4096, ragged heads in the second): the
    cluster kernel that reads the kept K rows once and the three-pass kernels write the same bytes;
    rows that do not fit a cluster's shared memory are refused when one pass is demanded."""
    from rdkv_b200 import synth
    from rdkv_b200.packing import pack_kv_layers
    H, T = 8, 32768
    Ks, Vs, vbs, kbs = [], [], [], []
    for layer, ragged in enumerate((None, [4096, 4000, 3000, 4096, 1, 4095, 2048, 777])):
        seed = synth.unit_seed(1, layer)
        K, V = synth.make_kv(H, T, seed=seed, device="cuda")
        Ks.append(K); Vs.append(V)
        vbs.append(synth.make_v_bits(H, T, 4096, seed=seed, device="cuda", per_head_N=ragged))
        kbs.append(synth.make_k_bits(H, seed=seed, device="cuda"))
    one = pack_kv_layers(Ks, Vs, torch.stack(vbs), torch.stack(kbs), 4, build_mask=False, k_passes=1)
    three = pack_kv_layers(Ks, Vs, torch.stack(vbs), torch.stack(kbs), 4, build_mask=False, k_passes=3)
    for layer in range(2):
        assert_layer_equal(layer_to_np(one[layer][0]), layer_to_np(three[layer][0]), f"layer {layer}.")
    big = synth.make_v_bits(H, T, 30000, seed=3, device="cuda")
    with pytest.raises((RuntimeError, ValueError)):
        pack_kv_layers(Ks[:1], Vs[:1], big[None], kbs[0][None], 4, build_mask=False, k_passes=1)
    assert len(pack_kv_layers(Ks[:1], Vs[:1], big[None], kbs[0][None], 4, build_mask=False)) == 1   # falls back by itself


def test_full_size_properties():
    """Config-1 layer (8 heads x 32768 tokens, budget 4096): size-independent checks —
    byte-exact round trip of the codes through dequantise/requantise and range bounds."""
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    from rdkv_b200.packing import pack_kv, quantize_and_pack
    seed = synth.unit_seed(1)
    K, V = synth.make_kv(8, 32768, seed=seed, device="cuda")
    v_bits = synth.make_v_bits(8, 32768, 4096, seed=seed, device="cuda")
    k_bits = synth.make_k_bits(8, seed=seed, device="cuda")
    packed, nv = pack_kv(K, V, v_bits, k_bits, 4)
    assert packed.T_eff == 3584 and packed.n_v16 == 512 and packed.T_eff_k == 4096
    assert tuple(packed.V_2bit.shape) == (1, 8, 1024, 32) and tuple(packed.K_4bit.shape) == (1, 8, 4096, 12)
    # fp16 rows are bit copies of the selected V rows, in ascending token order
    for h in (0, 7):
        ids = (v_bits[h] == 16).nonzero(as_tuple=True)[0]
        assert torch.equal(nv[0, h], V[0, h, ids])
    # idempotence: dequantised 8-bit V rows re-quantise to the same codes/scale/zp
    layer = {k: to_np(v) if torch.is_tensor(v) else v for k, v in vars(packed).items()}
    Vhat = RP.unpack_v(layer, to_np(nv), 128)
    n2, n4, n8 = (int(x) for x in layer["seg_bounds_per_head"][3])
    rows8 = torch.from_numpy(Vhat[:, 3:4, n2 + n4:n2 + n4 + n8]).cuda().contiguous()
    c, s, z = quantize_and_pack(rows8, 8, 3)
    codes = to_np(c).astype(np.float32)
    zp = to_np(z).astype(np.float32)
    again = ((codes - zp) * to_np(s).astype(np.float32)).astype(np.float16)
    assert np.abs(again.astype(np.float32) - Vhat[:, 3:4, n2 + n4:n2 + n4 + n8].astype(np.float32)).max() <= \
        float(to_np(s).astype(np.float32).max()) * 1.01
    # K codes of the whole layer agree with the oracle on a sample of heads
    want, _ = RP.pack_kv(to_np(K[:, 2:4]), to_np(V[:, 2:4]), to_np(v_bits[2:4]), to_np(k_bits[2:4]), 4)
    # (heads 2..3 packed alone see the same stripe extents because every head keeps 4096 tokens)
    for f in ["K_2bit", "K_4bit", "K_8bit"]:
        assert np.array_equal(to_np(getattr(packed, f))[:, 2:4], want[f]), f
    assert np.array_equal(to_np(packed.V_scale)[:, 2:4], want["V_scale"])


@pytest.mark.parametrize("tag", ["a", "b"])
def test_select_and_pack_matches_the_reference_composite(tag):
    """select_and_pack (pooling -> V allocation -> per-head K budget -> K allocation -> eviction ->
    pack, all on the device) against the reference's own _perhead_select_and_pack_joint run on CPU:
    every field of the packed layer, the fp16 rows and T_eff, bit for bit."""
    from conftest import load_golden
    from rdkv_b200.knapsack_solver import DEFAULT_EPSILON_K, DEFAULT_EPSILON_V
    from rdkv_b200.packing import select_and_pack
    g = sub(load_golden("select.npz"), tag)
    gq, budget, pool = (int(x) for x in g["args"])
    pl, nv, t_eff = select_and_pack(
        cuda(g["K"]), cuda(g["V"]), cuda(g["token_scores"]), cuda(g["channel_scores"]), gqa_factor=gq,
        token_budget=budget, k_budget_ratio=float(g["k_budget_ratio"]), obs_window=32, pool_kernel_size=pool,
        pool_padding="reflect", pool_type="avg", v_bit_options=None, k_bit_options=None,
        eps_V=DEFAULT_EPSILON_V, eps_K=DEFAULT_EPSILON_K)
    assert_layer_equal(layer_to_np(pl), g, tag + ".")
    assert t_eff == int(g["t_eff"])
    if "new_v_only" in g:
        assert np.array_equal(to_np(nv), g["new_v_only"])
    else:
        assert nv is None
