"""The numpy oracle against vectors produced by the reference's own code (CPU only)."""
import numpy as np
import pytest

from conftest import assert_layer_equal, sub
from oracle import ref_attention as RA
from oracle import ref_knapsack as RK
from oracle import ref_packing as RP


def test_reference_unit_case_k_and_v(golden_unit):
    """Shapes and inputs of the reference's segment-count packing test (T=6/7, D=8, seed 1)."""
    g = sub(golden_unit, "t1")
    k = RP.pack_k_mixed(g["keys"], g["k_bits"])
    for f in ["K_2bit", "K_4bit", "K_8bit", "K_ch_scale", "K_ch_zp", "K_ch_sort_idx", "K_ch_perm_padded_idx"]:
        assert np.array_equal(k[f], g[f]), f
    assert tuple(g["K_ch_seg_bounds"]) == k["K_ch_seg_bounds"] == (2, 2, 3)
    v = RP.pack_v_segments(g["values"], g["v_bits"])
    for f in ["V_2bit", "V_4bit", "V_8bit", "V_scale", "V_zp", "sort_idx"]:
        assert np.array_equal(v[f], g[f]), f
    assert tuple(g["seg_bounds"]) == v["seg_bounds"] == (2, 2, 2)


def test_reference_unit_case_deferred_k_stack(golden_unit):
    """Ragged heads with every bit class {0,2,4,8,16} (reference test, seed 11, D=8)."""
    g = sub(golden_unit, "t2")
    layer, nv = RP.pack_kv(g["keys"], g["values"], g["v_bits"], g["k_bits"], 2)
    assert_layer_equal(layer, g, "t2.")
    assert np.array_equal(nv, g["new_v_only"])


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
def test_pack_kv_matches_reference(golden_layers, tag):
    g = sub(golden_layers, tag)
    layer, nv = RP.pack_kv(g["K"], g["V"], g["v_bits"], g["k_bits"], int(g["g"]))
    assert_layer_equal(layer, g, tag + ".")
    if "new_v_only" in g:
        assert np.array_equal(nv, g["new_v_only"])
    else:
        assert nv is None


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
def test_attention_matches_reference(golden_layers, tag):
    g = sub(golden_layers, tag)
    layer, nv = RP.pack_kv(g["K"], g["V"], g["v_bits"], g["k_bits"], int(g["g"]))
    out, _, _ = RA.decode_attention(g["q"], layer, nv)
    np.testing.assert_allclose(out, g["attn_out"], rtol=1e-5, atol=2e-6)
    s = RA.k_scores(g["q"], layer, layer["T_eff_k"])
    np.testing.assert_allclose(s, g["k_scores"], rtol=1e-5, atol=2e-6)


def test_two_stage_equals_fused(golden_layers):
    """scores -> masked softmax -> weighted sum reproduces the fused oracle."""
    g = sub(golden_layers, "ragged")
    layer, nv = RP.pack_kv(g["K"], g["V"], g["v_bits"], g["k_bits"], int(g["g"]))
    s = RA.k_scores(g["q"], layer, layer["T_eff_k"]) + layer["softmax_mask"]
    w = np.exp(s - s.max(axis=1, keepdims=True))
    w /= w.sum(axis=1, keepdims=True)
    out = RA.v_weighted_sum(w.astype(np.float32), layer, nv)
    np.testing.assert_allclose(out, g["attn_out"], rtol=1e-5, atol=2e-6)


def test_lse_combine_of_halves(golden_layers):
    g = sub(golden_layers, "even")
    layer, nv = RP.pack_kv(g["K"], g["V"], g["v_bits"], g["k_bits"], int(g["g"]))
    full, _, _ = RA.decode_attention(g["q"], layer, nv)
    # split the stripe in two by masking halves
    T_k = layer["T_eff_k"]
    parts = []
    for lo, hi in ((0, T_k // 3), (T_k // 3, T_k)):
        half = dict(layer)
        m = layer["softmax_mask"].copy()
        m[:, :lo] = -np.inf
        m[:, hi:] = -np.inf
        half["softmax_mask"] = m
        o, mm, ll = RA.decode_attention(g["q"], half, nv)
        parts.append((mm, ll, o * ll[:, None]))
    out, _, _ = RA.lse_combine(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]),
                               np.stack([p[2] for p in parts]))
    np.testing.assert_allclose(out, full, rtol=1e-5, atol=2e-6)


KNAP_CASES = ["v", "vrow", "k", "kdef", "zeros", "nozero", "tiny", "tight"]


@pytest.mark.parametrize("name", KNAP_CASES)
def test_knapsack_matches_reference(golden_knapsack, name):
    from rdkv_b200.synth import ALLOC_EPSILON
    g = sub(golden_knapsack, name)
    got = RK.knapsack_batched(g["scores"], g["budget"], ALLOC_EPSILON, max_iters=int(g["max_iters"]),
                              tol=float(g["tol"]), bit_options=tuple(g["bit_options"].tolist()))
    assert got.dtype == np.int64
    assert np.array_equal(got, g["bits"])


def test_knapsack_default_epsilon(golden_knapsack):
    from rdkv_b200.knapsack_solver import DEFAULT_EPSILON
    got = RK.knapsack_batched(golden_knapsack["defeps_scores"], 2.0, DEFAULT_EPSILON)
    assert np.array_equal(got, golden_knapsack["defeps_bits"])


def test_scoring_oracle_matches_reference_vectors():
    """Importance scoring and score pooling: the numpy restatement against vectors produced by the
    reference's own functions (pooling bit for bit; the score sums to fp32 summation-order noise)."""
    from conftest import load_golden
    from oracle import ref_scoring as RS
    g = load_golden("scoring.npz")
    for tag, dt in (("f32", np.float32), ("f16", np.float16)):
        tok, ch = RS.score_one_layer(g[f"score_{tag}_aw"].astype(dt), g[f"score_{tag}_q"].astype(dt),
                                     g[f"score_{tag}_k"].astype(dt))
        np.testing.assert_allclose(tok, g[f"score_{tag}_token"], rtol=2e-3 if dt == np.float16 else 1e-5, atol=1e-6)
        np.testing.assert_allclose(ch, g[f"score_{tag}_channel"], rtol=1e-5)
    for key in g:
        if key.startswith("pool_") and not key.endswith("_x"):
            parts = key.split("_")
            src = g["pool_x"] if parts[1] in ("avg", "max") else g[f"pool_{parts[1]}_x"]
            pt, mode, ks = parts[-3], parts[-2], int(parts[-1])
            got = RS.score_pooling(src, pt, ks, mode)
            assert got.shape == g[key].shape, key
            assert np.array_equal(got, g[key]), key


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
def test_dequantise_matches_reference(golden_layers, tag):
    """Oracle dequantisation against the reference's unpack_trizone_to_past_kv outputs (bit-exact fp16)."""
    from conftest import load_golden
    u = sub(load_golden("unpack.npz"), tag)
    g = sub(golden_layers, tag)
    layer, nv = RP.pack_kv(g["K"], g["V"], g["v_bits"], g["k_bits"], int(g["g"]))
    assert np.array_equal(RP.unpack_k(layer, 128).view(np.uint16), u["K_hat"].view(np.uint16))
    v_hat = RP.unpack_v(layer, nv, 128)
    assert np.array_equal(v_hat.view(np.uint16), u["V_hat"].view(np.uint16))
    assert np.array_equal(v_hat[:, :, :layer["T_eff"]].view(np.uint16), u["zone_a"].view(np.uint16))


def test_scalar_knapsack_matches_reference(golden_knapsack):
    """The single-row solver (double-precision bisection): rows that converge early, late and never, an
    all-zero row, and the same rows with a tolerance that is never met."""
    from rdkv_b200.synth import ALLOC_EPSILON
    g = golden_knapsack
    for i in range(g["scalar_scores"].shape[0]):
        got = RK.knapsack_scalar(g["scalar_scores"][i], float(g["scalar_budget"][i]), ALLOC_EPSILON, max_iters=60)
        assert np.array_equal(got, g["scalar_bits"][i]), i
        got = RK.knapsack_scalar(g["scalar_scores"][i], float(g["scalar_budget"][i]), ALLOC_EPSILON, max_iters=60, tol=1e-6)
        assert np.array_equal(got, g["scalar_tight_bits"][i]), i


@pytest.mark.parametrize("tag", ["even", "ragged", "gqa8"])
def test_attention_with_uncompressed_tail_matches_reference(golden_layers, tag):
    """One softmax over the packed zones and the tokens appended while decoding (Zone C): the oracle
    against the reference's formula evaluated on the reference's own dequantised cache."""
    g = sub(golden_layers, tag)
    layer, nv = RP.pack_kv(g["K"], g["V"], g["v_bits"], g["k_bits"], int(g["g"]))
    out, _, _ = RA.decode_attention(g["q"], layer, nv, g["tail_k"], g["tail_v"])
    np.testing.assert_allclose(out, g["attn_out_tail"], rtol=1e-5, atol=2e-6)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_select_and_pack_matches_reference(tag):
    """Pooling -> V allocation -> per-head K budget -> K allocation -> eviction -> pack: every field of
    the packed layer bit for bit against the reference's own per-layer composite."""
    from conftest import load_golden
    from oracle import ref_select as RSel
    from rdkv_b200.knapsack_solver import DEFAULT_EPSILON_K, DEFAULT_EPSILON_V
    g = sub(load_golden("select.npz"), tag)
    gq, budget, pool = (int(x) for x in g["args"])
    layer, nv, v_bits, k_bits = RSel.select_and_pack(
        g["K"], g["V"], g["token_scores"], g["channel_scores"], gqa_factor=gq, token_budget=budget,
        k_budget_ratio=float(g["k_budget_ratio"]), pool_kernel_size=pool, eps_V=DEFAULT_EPSILON_V, eps_K=DEFAULT_EPSILON_K)
    assert_layer_equal(layer, g, tag + ".")
    assert int(g["t_eff"]) == layer["T_eff"]
    if "new_v_only" in g:
        assert np.array_equal(nv, g["new_v_only"])
    else:
        assert nv is None


@pytest.mark.parametrize("tag", ["f16", "bf16"])
@pytest.mark.parametrize("cs", ["same", "f32"])
def test_rope_oracle_matches_reference_vectors(tag, cs):
    """fused_rope_ref of the reference (triton_rope.py:141-165) on seeded rows, bit for bit."""
    from oracle import ref_rope as RR
    from conftest import load_golden
    g = load_golden("rope.npz")
    key = f"{tag}_{cs}_"
    q_out, k_out = RR.fused_rope(g[key + "q"], g[key + "k"], g[key + "cos"], g[key + "sin"], tag,
                                 tag if cs == "same" else "f32")
    assert np.array_equal(q_out.view(np.uint16), g[key + "q_out"].view(np.uint16))
    assert np.array_equal(k_out.view(np.uint16), g[key + "k_out"].view(np.uint16))


@pytest.mark.parametrize("tag", ["f16", "bf16", "f16w32"])
def test_obs_window_scores_oracle_matches_reference_vectors(tag):
    """Scores from the observation window's queries and the keys (obkv_fast.py:1443-1450 + :854-896)."""
    from oracle import ref_scoring as RS
    from conftest import load_golden
    g = load_golden("obs.npz")
    B, H, gq, W, T = (int(x) for x in g[f"{tag}_shape"])
    tok, ch = RS.obs_window_scores(g[f"{tag}_q"], g[f"{tag}_k"], "bf16" if tag == "bf16" else "f16", gq)
    # (sums of 16-bit weights in another order: the last 16-bit place may differ)
    np.testing.assert_allclose(tok, g[f"{tag}_token"], rtol=1e-2 if tag == "bf16" else 2e-3, atol=1e-5)
    np.testing.assert_allclose(ch, g[f"{tag}_channel"], rtol=1e-5)
