"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own
Python code (PyTorch CPU kernels) on seeded inputs.

    python tests/golden/make_golden.py /path/to/reference/checkout [layers] [scoring] [unpack] [select] [blockwise] [rope] [legacy] [obs]
    (or RDKV_REFERENCE=/path/to/reference/checkout in the environment; no part named = all)

The reference checkout is only needed to (re)generate the files; the tests read
the committed .npz files and never import the reference.  Inputs are stored
next to the outputs, so the vectors do not depend on a torch RNG stream.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("RDKV_REFERENCE", "")
if not os.path.isdir(REF):
    raise SystemExit("give the path of the reference checkout (argument or RDKV_REFERENCE)")
sys.dont_write_bytecode = True
sys.path.insert(0, REF)
sys.path.insert(0, ROOT)

import knapsack_solver as KS                                   # noqa: E402  (reference)
from obkv_accel import packing as P                            # noqa: E402  (reference)
from obkv_accel import trizone_decompress as TD                # noqa: E402  (reference)
from obkv_accel.triton_k_kernel import k_mixed_qk_dot_ref      # noqa: E402  (reference)

from rdkv_b200 import synth                                     # noqa: E402

LAYER_FIELDS = [
    "K_2bit", "K_4bit", "K_8bit", "K_ch_scale", "K_ch_zp", "K_ch_sort_idx", "K_ch_perm_padded_idx",
    "V_2bit", "V_4bit", "V_8bit", "V_scale", "V_zp", "sort_idx",
    "seg_bounds_per_head", "T_eff_per_head", "softmax_mask",
    "K_ch_sort_idx_per_head", "K_ch_perm_padded_idx_per_head", "K_ch_seg_bounds_per_head",
    "K_ch_perm_padded_idx_for_Q", "T_eff_k_per_head", "n_v16_per_head",
]
LAYER_SCALARS = ["K_ch_seg_bounds", "seg_bounds", "T_eff", "T_eff_k", "n_v16"]


def npy(t):
    return None if t is None else t.detach().cpu().numpy()


def layer_to_dict(pl, prefix=""):
    out = {}
    for f in LAYER_FIELDS:
        v = getattr(pl, f)
        if v is not None:
            out[prefix + f] = npy(v)
    for f in LAYER_SCALARS:
        out[prefix + f] = np.asarray(getattr(pl, f), dtype=np.int64)
    return out


def ref_pack_kv(K, V, v_bits, k_bits, g):
    """The reference's per-layer composite (obkv_fast.py:1098-1166), per-head deferred-K path."""
    H_kv, D = K.shape[1], K.shape[3]
    layers, v16s = [], []
    for h in range(H_kv):
        kept = (v_bits[h] > 0).nonzero(as_tuple=True)[0]
        if kept.numel() == 0:
            layers.append(P._empty_packed_layer(1, D, K.device, K.dtype))
            v16s.append(None)
            continue
        kb = v_bits[h][kept]
        counts = tuple(int((kb == b).sum()) for b in (2, 4, 8))
        layer, _, v16 = P.build_packed_layer(
            K[:, h:h + 1].index_select(2, kept).contiguous(),
            V[:, h:h + 1].index_select(2, kept).contiguous(),
            kb, k_bits[h], v_segment_counts=counts, defer_k_for_per_head_stack=True)
        layers.append(layer)
        v16s.append(v16)
    return P._pad_and_stack_per_head_layers(
        layers, v16s, H_q=H_kv * g, gqa_factor=g, head_dim=D, device=K.device, dtype=K.dtype,
        k_bits_per_head=k_bits)


def ref_pack_kv_legacy(K, V, v_bits, k_bits_shared, g):
    """The shared-layout form of the same composite: one K bit map [D] for all heads, every head's K
    quantised on its own rows by build_packed_layer, the packed bytes copied into the stripe
    (packing.py:1019-1317 with k_bits_per_head=None)."""
    H_kv, D = K.shape[1], K.shape[3]
    layers, v16s = [], []
    for h in range(H_kv):
        kept = (v_bits[h] > 0).nonzero(as_tuple=True)[0]
        kb = v_bits[h][kept]
        counts = tuple(int((kb == b).sum()) for b in (2, 4, 8))
        layer, _, v16 = P.build_packed_layer(
            K[:, h:h + 1].index_select(2, kept).contiguous(),
            V[:, h:h + 1].index_select(2, kept).contiguous(),
            kb, k_bits_shared, v_segment_counts=counts)
        layers.append(layer)
        v16s.append(v16)
    return P._pad_and_stack_per_head_layers(
        layers, v16s, H_q=H_kv * g, gqa_factor=g, head_dim=D, device=K.device, dtype=K.dtype)


def make_legacy():
    """Shared-layout stacking on a ragged layer: the stacked layer's fields, the fp16 rows and the
    dequantise-then-attend output."""
    H_kv, g, T, N = 4, 2, 256, 96
    seed = synth.unit_seed(21, 0)
    K, V = synth.make_kv(H_kv, T, seed=seed)
    v_bits = synth.make_v_bits(H_kv, T, N, seed=seed, per_head_N=[96, 64, 17, 80])
    k_bits = synth.make_k_bits(1, seed=seed)[0]
    pl, nv = ref_pack_kv_legacy(K, V, v_bits, k_bits, g)
    q = synth.make_q(H_kv * g, seed=seed)
    out = {"K": npy(K), "V": npy(V), "v_bits": npy(v_bits), "k_bits": npy(k_bits), "q": npy(q), "new_v_only": npy(nv)}
    out.update(layer_to_dict(pl))
    attn, K_hat, V_hat = ref_attend(q, pl, nv, 128)
    out.update(attn_out=npy(attn), K_hat=npy(K_hat), V_hat=npy(V_hat))
    np.savez_compressed(os.path.join(HERE, "legacy.npz"), **out)
    print("legacy.npz", os.path.getsize(os.path.join(HERE, "legacy.npz")), "bytes")


def ref_attend(q, pl, new_v_only, D, tail_k=None, tail_v=None):
    """Reference dequantise-then-attend (trizone_decompress.py:185 + fp32 softmax attention).  With
    tail_k / tail_v [H_kv,n,D] (tokens appended while decoding, kept uncompressed) the softmax runs
    over the packed zones and the tail together, as the reference's attention block computes it
    (fast_decode.py:1719-1784: scores of the tail use q/sqrt(D), one softmax over the concatenation,
    out = weights_old . V_old + weights_new . V_new)."""
    cache = P.TriZoneCache(packed=(pl,), new_v_only=[new_v_only], new_both_k=[None], new_both_v=[None],
                           original_seq_len=0)
    (K_hat, V_hat), = TD.unpack_trizone_to_past_kv(cache, head_dim=D)
    g = q.shape[0] // K_hat.shape[1]
    Kx = K_hat[0].float().repeat_interleave(g, 0)
    Vx = V_hat[0].float().repeat_interleave(g, 0)
    s = torch.einsum("hd,htd->ht", q.float(), Kx) / (D ** 0.5) + pl.softmax_mask
    if tail_k is not None:
        s_new = torch.bmm((q.float() / (D ** 0.5)).unsqueeze(1), tail_k.float().repeat_interleave(g, 0).transpose(1, 2)).squeeze(1)
        w = torch.softmax(torch.cat([s, s_new], dim=-1), dim=-1)
        w_old, w_new = w[:, :s.shape[1]], w[:, s.shape[1]:]
        out = torch.einsum("ht,htd->hd", w_old, Vx) + torch.bmm(w_new.unsqueeze(1), tail_v.float().repeat_interleave(g, 0)).squeeze(1)
        return out, K_hat, V_hat
    w = torch.softmax(s, dim=-1)
    return torch.einsum("ht,htd->hd", w, Vx), K_hat, V_hat


def case_unit_tests():
    """The two packing pins of the reference's own unit tests (tests/test_blockwise_rdkv.py:119-228)."""
    out = {}
    torch.manual_seed(1)
    keys = torch.randn(1, 1, 7, 8, dtype=torch.float16)
    k_bits = torch.tensor([0, 2, 4, 8, 16, 2, 4, 8])
    values = torch.randn(1, 1, 6, 8, dtype=torch.float16)
    v_bits = torch.tensor([2, 4, 8, 2, 8, 4])
    rk = P.pack_k_mixed(keys.clone(), k_bits)
    rv = P.pack_v_segments(values.clone(), v_bits)
    out.update(t1_keys=npy(keys), t1_k_bits=npy(k_bits), t1_values=npy(values), t1_v_bits=npy(v_bits))
    for name, t in zip(["K_2bit", "K_4bit", "K_8bit", "K_ch_scale", "K_ch_zp", "K_ch_sort_idx",
                        "K_ch_perm_padded_idx"], rk[:7]):
        out["t1_" + name] = npy(t)
    out["t1_K_ch_seg_bounds"] = np.asarray(rk[7], np.int64)
    for name, t in zip(["V_2bit", "V_4bit", "V_8bit", "V_scale", "V_zp", "sort_idx"], rv[:6]):
        out["t1_" + name] = npy(t)
    out["t1_seg_bounds"] = np.asarray(rv[6], np.int64)

    torch.manual_seed(11)
    keys = torch.randn(1, 2, 7, 8, dtype=torch.float16)
    values = torch.randn_like(keys)
    v_bits = torch.tensor([[2, 4, 8, 16, 0, 2, 4], [4, 16, 2, 8, 0, 4, 2]])
    k_bits = torch.tensor([[2, 4, 8, 0, 16, 2, 4, 8], [4, 2, 0, 8, 16, 4, 2, 8]])
    pl, nv = ref_pack_kv(keys, values, v_bits, k_bits, 2)
    out.update(t2_keys=npy(keys), t2_values=npy(values), t2_v_bits=npy(v_bits), t2_k_bits=npy(k_bits),
               t2_new_v_only=npy(nv))
    out.update(layer_to_dict(pl, "t2_"))
    return out


def case_layer(tag, H_kv, g, T, N, seed, per_head_N=None, k_mix=((8, 16), (4, 24), (2, 24))):
    K, V = synth.make_kv(H_kv, T, seed=seed)
    v_bits = synth.make_v_bits(H_kv, T, N, seed=seed, per_head_N=per_head_N)
    k_bits = synth.make_k_bits(H_kv, seed=seed, mix=k_mix)
    q = synth.make_q(H_kv * g, seed=seed + 1)
    pl, nv = ref_pack_kv(K, V, v_bits, k_bits, g)
    att, _, _ = ref_attend(q, pl, nv, 128)
    scores = k_mixed_qk_dot_ref(q, pl, pl.T_eff_k)
    gen = torch.Generator().manual_seed(seed + 5)
    tail_k = torch.randn(H_kv, 19, 128, generator=gen).half()       # decode-appended tokens (Zone C)
    tail_v = torch.randn(H_kv, 19, 128, generator=gen).half()
    att_tail, _, _ = ref_attend(q, pl, nv, 128, tail_k, tail_v)
    out = {f"{tag}_K": npy(K), f"{tag}_V": npy(V), f"{tag}_v_bits": npy(v_bits), f"{tag}_k_bits": npy(k_bits),
           f"{tag}_q": npy(q), f"{tag}_attn_out": npy(att), f"{tag}_k_scores": npy(scores),
           f"{tag}_tail_k": npy(tail_k), f"{tag}_tail_v": npy(tail_v), f"{tag}_attn_out_tail": npy(att_tail),
           f"{tag}_g": np.asarray(g)}
    if nv is not None:
        out[f"{tag}_new_v_only"] = npy(nv)
    out.update(layer_to_dict(pl, tag + "_"))
    return out


def case_knapsack():
    out = {}
    eps = synth.ALLOC_EPSILON
    cases = {
        "v": dict(scores=synth.make_scores(6, 2048, seed=2000), budget=2.0, max_iters=60),
        "vrow": dict(scores=synth.make_scores(5, 1024, seed=2001),
                     budget=torch.tensor([0.5, 1.0, 2.0, 6.0, 20.0]), max_iters=60),
        "k": dict(scores=synth.make_scores(8, 128, seed=2002), budget=2.64, max_iters=60),
        "kdef": dict(scores=synth.make_scores(4, 128, seed=2003), budget=4.0, max_iters=64),
        "zeros": dict(scores=torch.zeros(2, 64), budget=2.0, max_iters=60),
        "nozero": dict(scores=synth.make_scores(3, 256, seed=2004), budget=1.0, max_iters=12,
                       bit_options=torch.tensor([2., 4., 8.])),
        "tiny": dict(scores=synth.make_scores(3, 7, seed=2005), budget=3.0, max_iters=60),
        "tight": dict(scores=synth.make_scores(2, 4096, seed=2006), budget=2.0, max_iters=60, tol=1e-5),
    }
    for name, c in cases.items():
        kw = dict(epsilon=eps, max_iters=c["max_iters"], tol=c.get("tol", 0.01))
        if "bit_options" in c:
            kw["bit_options"] = c["bit_options"]
        res = KS.knapsack_bit_allocation_batched(c["scores"], c["budget"], **kw)
        out[f"{name}_scores"] = npy(c["scores"])
        out[f"{name}_budget"] = np.asarray(c["budget"], dtype=np.float32)
        out[f"{name}_max_iters"] = np.asarray(c["max_iters"])
        out[f"{name}_tol"] = np.asarray(c.get("tol", 0.01), dtype=np.float64)
        out[f"{name}_bit_options"] = npy(c.get("bit_options", torch.tensor([0., 2., 4., 8., 16.])))
        out[f"{name}_bits"] = npy(res)
    # the scalar form (knapsack_solver.py:39-118: bisection in Python floats, no clamp of lambda_hi),
    # row by row, on rows that converge early, late, never, and on an all-zero row
    sc = torch.cat([synth.make_scores(3, 512, seed=2010), torch.zeros(1, 512), synth.make_scores(2, 512, seed=2011, sigma=0.3)])
    budgets = [2.0, 0.7, 9.0, 2.0, 2.0, 15.5]
    out["scalar_scores"] = npy(sc)
    out["scalar_budget"] = np.asarray(budgets, np.float32)
    out["scalar_bits"] = np.stack([npy(KS.knapsack_bit_allocation(sc[i], budgets[i], epsilon=eps, max_iters=60))
                                   for i in range(sc.shape[0])])
    out["scalar_tight_bits"] = np.stack([npy(KS.knapsack_bit_allocation(sc[i], budgets[i], epsilon=eps, max_iters=60, tol=1e-6))
                                         for i in range(sc.shape[0])])
    # default-epsilon call, as the reference's smoke test makes it
    s = synth.make_scores(2, 512, seed=2007, sigma=1.0)
    out["defeps_scores"] = npy(s)
    out["defeps_bits"] = npy(KS.knapsack_bit_allocation_batched(s, 2.0))
    return out


def main():
    torch.set_num_threads(os.cpu_count() or 1)
    np.savez_compressed(os.path.join(HERE, "packing_unit.npz"), **case_unit_tests())
    layers = {}
    layers.update(case_layer("even", H_kv=2, g=4, T=384, N=128, seed=synth.unit_seed(0, 0, 1)))
    layers.update(case_layer("ragged", H_kv=3, g=2, T=320, N=96, seed=synth.unit_seed(0, 1, 2),
                             per_head_N=[96, 84, 72], k_mix=((8, 9), (4, 21), (2, 30))))
    layers.update(case_layer("gqa8", H_kv=1, g=8, T=200, N=64, seed=synth.unit_seed(4, 0, 0),
                             k_mix=((8, 128),)))
    np.savez_compressed(os.path.join(HERE, "layers.npz"), **layers)
    np.savez_compressed(os.path.join(HERE, "knapsack.npz"), **case_knapsack())
    for f in ("packing_unit.npz", "layers.npz", "knapsack.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


def make_scoring():
    """Scoring / pooling vectors from the reference's own functions (obkv_fast.py:208-246, 854-896)."""
    import obkv_fast as ref_fast
    out = {}
    g = torch.Generator().manual_seed(1234)
    B, H, gq, W, T, D = 1, 2, 4, 8, 203, 128
    for tag, dt in (("f32", torch.float32), ("f16", torch.float16)):
        aw = torch.softmax(torch.randn(B, H, gq, W, T, generator=g) * 3, dim=-1).to(dt)
        q = torch.randn(B, H, gq, W, D, generator=g).to(dt)
        k = torch.randn(B, H, T, D, generator=g).to(dt)
        v = torch.randn(B, H, T, D, generator=g).to(dt)
        tok, ch = ref_fast._score_one_layer(aw, q, None, v, D, k=k)
        out[f"score_{tag}_aw"] = aw.float().numpy(); out[f"score_{tag}_q"] = q.float().numpy()
        out[f"score_{tag}_k"] = k.float().numpy()
        out[f"score_{tag}_token"] = tok.numpy(); out[f"score_{tag}_channel"] = ch.numpy()
    x = torch.randn(3, 57, generator=g)
    out["pool_x"] = x.numpy()
    for pt in ("avg", "max"):
        for mode in ("zero", "reflect"):
            for ks in (5, 4, 1):
                out[f"pool_{pt}_{mode}_{ks}"] = ref_fast.apply_score_pooling(x, pt, ks, mode).numpy()
    short = torch.randn(2, generator=g)
    out["pool_short_x"] = short.numpy()
    out["pool_short_avg_reflect_5"] = ref_fast.apply_score_pooling(short, "avg", 5, "reflect").numpy()
    one = torch.randn(1, generator=g)
    out["pool_one_x"] = one.numpy()
    out["pool_one_avg_reflect_5"] = ref_fast.apply_score_pooling(one, "avg", 5, "reflect").numpy()
    np.savez_compressed(os.path.join(HERE, "scoring.npz"), **out)


LAYER_CASES = {
    "even": dict(H_kv=2, g=4, T=384, N=128, seed=synth.unit_seed(0, 0, 1)),
    "ragged": dict(H_kv=3, g=2, T=320, N=96, seed=synth.unit_seed(0, 1, 2), per_head_N=[96, 84, 72],
                   k_mix=((8, 9), (4, 21), (2, 30))),
    "gqa8": dict(H_kv=1, g=8, T=200, N=64, seed=synth.unit_seed(4, 0, 0), k_mix=((8, 128),)),
}


def make_unpack():
    """Decompressor vectors: the reference's unpack_trizone_to_past_kv (trizone_decompress.py:185) on the
    layers of layers.npz (same seeds), and unpack_v_segment (packing.py:1427) on one segment of each width."""
    out = {}
    for tag, c in LAYER_CASES.items():
        K, V = synth.make_kv(c["H_kv"], c["T"], seed=c["seed"])
        v_bits = synth.make_v_bits(c["H_kv"], c["T"], c["N"], seed=c["seed"], per_head_N=c.get("per_head_N"))
        k_bits = synth.make_k_bits(c["H_kv"], seed=c["seed"], mix=c.get("k_mix", ((8, 16), (4, 24), (2, 24))))
        pl, nv = ref_pack_kv(K, V, v_bits, k_bits, c["g"])
        cache = P.TriZoneCache(packed=(pl,), new_v_only=[nv], new_both_k=[None], new_both_v=[None], original_seq_len=0)
        ((K_hat, V_hat),), masks = TD.unpack_trizone_to_past_kv(cache, head_dim=128, return_masks=True, max_new_tokens=3)
        out[f"{tag}_K_hat"] = npy(K_hat); out[f"{tag}_V_hat"] = npy(V_hat)
        out[f"{tag}_zone_a"] = npy(TD._unpack_v_perhead(pl, head_dim=128))
        if masks[0] is not None:
            out[f"{tag}_mask"] = npy(masks[0].float())
    g = torch.Generator().manual_seed(99)
    x = torch.randn(1, 2, 37, 128, generator=g).half()
    for bits in (2, 4, 8):
        codes, sc, zp = P.quantize_and_pack(x, bits, 3)
        out[f"seg{bits}_codes"] = npy(codes); out[f"seg{bits}_scale"] = npy(sc); out[f"seg{bits}_zp"] = npy(zp)
        out[f"seg{bits}_out"] = npy(P.unpack_v_segment(codes, sc, zp, bits))
    np.savez_compressed(os.path.join(HERE, "unpack.npz"), **out)
    print("unpack.npz", os.path.getsize(os.path.join(HERE, "unpack.npz")), "bytes")


def make_select():
    """The reference's per-layer composite _perhead_select_and_pack_joint (obkv_fast.py:899-1186) on CPU:
    pooling -> V allocation -> per-head K budget -> K allocation -> channel eviction -> pack."""
    import obkv_fast as ref_fast
    out = {}
    cases = {
        "a": dict(H_kv=2, g=4, T=512, budget=128, kr=0.5, pool=5, seed=7001),
        "b": dict(H_kv=3, g=2, T=384, budget=64, kr=0.35, pool=1, seed=7002),
    }
    for tag, c in cases.items():
        K, V = synth.make_kv(c["H_kv"], c["T"], seed=c["seed"])
        gen = torch.Generator().manual_seed(c["seed"] + 1)
        tok = torch.exp(1.2 * torch.randn(c["H_kv"], c["T"], generator=gen))
        if tag == "b":
            tok[1] *= 1e-3                                  # a head that keeps much less: another K budget
        ch = torch.exp(torch.randn(c["H_kv"], 128, generator=gen))
        pl, nv, t_eff = ref_fast._perhead_select_and_pack_joint(
            K, V, tok, ch, gqa_factor=c["g"], token_budget=c["budget"], k_budget_ratio=c["kr"], obs_window=32,
            pool_kernel_size=c["pool"], pool_padding="reflect", pool_type="avg", v_bit_options=None,
            k_bit_options=None, eps_V=dict(KS.DEFAULT_EPSILON_V), eps_K=dict(KS.DEFAULT_EPSILON_K))
        out.update({f"{tag}_K": npy(K), f"{tag}_V": npy(V), f"{tag}_token_scores": npy(tok), f"{tag}_channel_scores": npy(ch),
                    f"{tag}_args": np.asarray([c["g"], c["budget"], c["pool"]], np.int64),
                    f"{tag}_k_budget_ratio": np.asarray(c["kr"], np.float64), f"{tag}_t_eff": np.asarray(t_eff, np.int64)})
        if nv is not None:
            out[f"{tag}_new_v_only"] = npy(nv)
        out.update(layer_to_dict(pl, tag + "_"))
    np.savez_compressed(os.path.join(HERE, "select.npz"), **out)
    print("select.npz", os.path.getsize(os.path.join(HERE, "select.npz")), "bytes")


def make_blockwise():
    """Blockwise recompression: the reference's planner, block scoring and _compress_block on CPU
    (obkv_accel/blockwise_decode.py:89-140, 756-810, 812-1121), and attention over several packed
    sources plus a tail, evaluated on the reference's own dequantised caches."""
    import obkv_fast as ref_fast                                # noqa: F401  (resolves the decoder's lazy import)
    from obkv_accel import blockwise_decode as BD
    out = {}
    # planner: the reference tests' cases and a sweep
    cases = [(512, 64), (128, 64), (192, 64), (127, 64), (0, 64), (1, 64), (64, 64), (65, 64), (129, 128), (700, 128)]
    out["plan_cases"] = np.asarray(cases, np.int64)
    for n, bs in cases:
        ev = BD.plan_block_compressions(n, bs)
        out[f"plan_{n}_{bs}"] = np.asarray(
            [[e["block_id"], e["token_start"], e["token_end"], e["query_source_block"], int(e["is_final_flush"]),
              int(e["query_mode"] == "self_causal")] for e in ev], np.int64).reshape(-1, 6)
    # block scoring: the shapes of the reference's own test (seed 7) and block-sized ones
    torch.manual_seed(7)
    q = torch.randn(4, 5, 8); k = torch.randn(1, 2, 4, 8)
    tok, ch = BD._score_block(q, k, num_kv_groups=2, causal=False)
    out.update(score_t_q=npy(q), score_t_k=npy(k), score_t_token=npy(tok), score_t_channel=npy(ch))
    gen = torch.Generator().manual_seed(31)
    for tag, (hkv, g, Q, T, dt, causal) in {"next": (2, 4, 64, 64, torch.float16, False),
                                            "self": (2, 4, 37, 37, torch.float16, True),
                                            "wide": (1, 8, 128, 128, torch.float32, False)}.items():
        q = torch.randn(hkv * g, Q, 128, generator=gen).to(dt)
        k = torch.randn(1, hkv, T, 128, generator=gen).to(dt)
        tok, ch = BD._score_block(q, k, num_kv_groups=g, causal=causal)
        out.update({f"score_{tag}_q": npy(q.float()), f"score_{tag}_k": npy(k.float()), f"score_{tag}_token": npy(tok),
                    f"score_{tag}_channel": npy(ch), f"score_{tag}_args": np.asarray([g, int(causal), int(dt == torch.float16)])})
    # one block of 64 generated tokens, two layers, through the reference's _compress_block
    hkv, g, T, D = 2, 2, 64, 128
    cfg = BD.BlockwiseRDKVConfig(block_size=64, block_budget_tokens=8, k_budget_ratio=0.5, obs_window=32,
                                 pool_kernel_size=5, pool_padding="reflect", v_bit_options=None, k_bit_options=None,
                                 epsilon_v=dict(KS.DEFAULT_EPSILON_V), epsilon_k=dict(KS.DEFAULT_EPSILON_K))
    kvs, qs, toks = [], [], []
    for layer in range(2):
        K, V = synth.make_kv(hkv, T, seed=8100 + layer)
        kvs.append(torch.cat([K, V], dim=-1))
        qb = torch.randn(hkv * g, 64, D, generator=gen).half()
        qs.append(qb)
        toks.append(BD._score_block(qb, K, num_kv_groups=g, causal=False)[0])
    block, _ = BD._compress_block(target_kv=kvs, query_block=qs, token_scores_by_layer=toks, block_id=0, token_start=0,
                                  token_end=63, query_source_block=1, is_final_flush=False, causal=False, config=cfg,
                                  num_kv_groups=g, model_dtype=torch.float16)
    out["block_args"] = np.asarray([hkv, g, T], np.int64)
    for layer in range(2):
        out[f"block_l{layer}_kv"] = npy(kvs[layer]); out[f"block_l{layer}_q"] = npy(qs[layer].float())
        out[f"block_l{layer}_token_scores"] = npy(toks[layer])
        out.update(layer_to_dict(block.packed[layer], f"block_l{layer}_"))
        if block.new_v_only[layer] is not None:
            out[f"block_l{layer}_new_v_only"] = npy(block.new_v_only[layer])
    out["block_logical_bits"] = np.asarray(block.logical_bits_per_layer, np.int64)
    # attention over the prompt's layer, the block's layer 0 and a tail: one softmax over everything
    Kp, Vp = synth.make_kv(hkv, 384, seed=8200)
    vbp = synth.make_v_bits(hkv, 384, 128, seed=8200)
    kbp = synth.make_k_bits(hkv, seed=8200)
    prompt, prompt_nv = ref_pack_kv(Kp, Vp, vbp, kbp, g)
    qd = synth.make_q(hkv * g, seed=8201)
    tail_k = torch.randn(hkv, 9, D, generator=gen).half(); tail_v = torch.randn(hkv, 9, D, generator=gen).half()
    ks, vs, masks = [], [], []
    for pl, nv in ((prompt, prompt_nv), (block.packed[0], block.new_v_only[0])):
        cache = P.TriZoneCache(packed=(pl,), new_v_only=[nv], new_both_k=[None], new_both_v=[None], original_seq_len=0)
        (K_hat, V_hat), = TD.unpack_trizone_to_past_kv(cache, head_dim=D)
        ks.append(K_hat[0].float().repeat_interleave(g, 0)); vs.append(V_hat[0].float().repeat_interleave(g, 0))
        masks.append(pl.softmax_mask)
    ks.append(tail_k.float().repeat_interleave(g, 0)); vs.append(tail_v.float().repeat_interleave(g, 0))
    masks.append(torch.zeros(hkv * g, 9))
    Kall, Vall, mall = torch.cat(ks, 1), torch.cat(vs, 1), torch.cat(masks, 1)
    w = torch.softmax(torch.einsum("hd,htd->ht", qd.float(), Kall) / (D ** 0.5) + mall, dim=-1)
    out.update(ms_K=npy(Kp), ms_V=npy(Vp), ms_v_bits=npy(vbp), ms_k_bits=npy(kbp), ms_q=npy(qd), ms_tail_k=npy(tail_k),
               ms_tail_v=npy(tail_v), ms_attn_out=npy(torch.einsum("ht,htd->hd", w, Vall)))
    np.savez_compressed(os.path.join(HERE, "blockwise.npz"), **out)
    print("blockwise.npz", os.path.getsize(os.path.join(HERE, "blockwise.npz")), "bytes")


def make_obs():
    """Token and channel scores of a layer from the observation window's queries and the keys: the
    reference's inline scoring step (obkv_fast.py:1443-1450: 16-bit matmul, scaling, causal mask of
    the window, softmax) followed by its _score_one_layer (:854-896), on seeded tensors."""
    import math
    import obkv_fast as ref_fast
    gen = torch.Generator().manual_seed(4321)
    out = {}
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()
    for tag, dt, (B, H, g, W, T) in (("f16", torch.float16, (1, 2, 4, 8, 300)), ("bf16", torch.bfloat16, (1, 2, 4, 8, 300)),
                                     ("f16w32", torch.float16, (2, 1, 4, 32, 1000))):
        D = 128
        q_obs = torch.randn(B, H * g, W, D, generator=gen).to(dt)
        k = (torch.randn(B, H, T, D, generator=gen) * 0.7).to(dt)
        k_exp = k.repeat_interleave(g, dim=1)
        query_positions = torch.arange(T - W, T)
        obs_mask = torch.arange(T).unsqueeze(0) > query_positions.unsqueeze(1)
        aw = torch.matmul(q_obs, k_exp.transpose(-1, -2)) * (1.0 / math.sqrt(D))
        aw.masked_fill_(obs_mask.unsqueeze(0).unsqueeze(0), float("-inf"))
        aw = aw.softmax(dim=-1)
        tok, ch = ref_fast._score_one_layer(aw.view(B, H, g, W, T), q_obs.view(B, H, g, W, D), None, k, D, k=k)
        out.update({f"{tag}_q": bits(q_obs), f"{tag}_k": bits(k), f"{tag}_token": tok.numpy(), f"{tag}_channel": ch.numpy(),
                    f"{tag}_shape": np.asarray([B, H, g, W, T], dtype=np.int64)})
    np.savez_compressed(os.path.join(HERE, "obs.npz"), **out)
    print("obs.npz", os.path.getsize(os.path.join(HERE, "obs.npz")), "bytes")


def make_rope():
    """fused_rope_ref (obkv_accel/triton_rope.py:141-165) on seeded rows: fp16 and bf16 rows (bf16
    stored as its 16-bit patterns), tables of the rows' type and fp32 tables."""
    from obkv_accel.triton_rope import fused_rope_ref
    gen = torch.Generator().manual_seed(77)
    out = {}
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()
    for tag, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        for cs_tag, cs_dt in (("same", dt), ("f32", torch.float32)):
            q = (torch.randn(12, 128, generator=gen) * 1.7).to(dt)
            k = (torch.randn(4, 128, generator=gen) * 2.3).to(dt)
            pos = torch.rand(64, generator=gen) * 900.0
            cos, sin = torch.cos(pos).to(cs_dt), torch.sin(pos).to(cs_dt)
            q2, k2 = fused_rope_ref(q, k, cos, sin)
            key = f"{tag}_{cs_tag}_"
            out.update({key + "q": bits(q), key + "k": bits(k), key + "cos": bits(cos), key + "sin": bits(sin),
                        key + "q_out": bits(q2), key + "k_out": bits(k2)})
    np.savez_compressed(os.path.join(HERE, "rope.npz"), **out)
    print("rope.npz", os.path.getsize(os.path.join(HERE, "rope.npz")), "bytes")


if __name__ == "__main__":
    parts = sys.argv[2:] or ["layers", "scoring", "unpack", "select", "blockwise", "rope", "legacy", "obs"]
    if "obs" in parts:
        make_obs()
    if "legacy" in parts:
        make_legacy()
    if "rope" in parts:
        make_rope()
    if "blockwise" in parts:
        make_blockwise()
    if "select" in parts:
        make_select()
    if "layers" in parts:
        main()
    if "scoring" in parts:
        make_scoring()
    if "unpack" in parts:
        make_unpack()
