"""Importance scoring and score pooling on the GPU (through the C ABI) against vectors produced by
the reference's own functions: pooling bit for bit, score sums to summation-order noise."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from helpers import cuda, to_np

pytestmark = pytest.mark.gpu


def test_score_one_layer_matches_reference_vectors():
    from rdkv_b200.scoring import _score_one_layer
    g = load_golden("scoring.npz")
    for tag, dt in (("f32", torch.float32), ("f16", torch.float16)):
        aw, q, k = (cuda(g[f"score_{tag}_{n}"]).to(dt) for n in ("aw", "q", "k"))
        tok, ch = _score_one_layer(aw, q, None, k, 128, k=k)
        assert tok.dtype == torch.float32 and tuple(tok.shape) == g[f"score_{tag}_token"].shape
        np.testing.assert_allclose(to_np(tok), g[f"score_{tag}_token"], rtol=2e-3 if dt == torch.float16 else 1e-5,
                                   atol=1e-6)
        np.testing.assert_allclose(to_np(ch), g[f"score_{tag}_channel"], rtol=1e-5)
        # a strided K (a slice of a longer context) gives the same channel scores
        k_wide = torch.zeros(k.shape[0], k.shape[1], k.shape[2] + 7, k.shape[3], dtype=dt, device="cuda")
        k_wide[:, :, :k.shape[2]] = k
        _, ch2 = _score_one_layer(aw, q, None, k, 128, k=k_wide[:, :, :k.shape[2]])
        assert torch.equal(ch, ch2)
    with pytest.raises(ValueError):
        _score_one_layer(aw, q, None, k, 128)


def test_score_one_layer_on_odd_shapes_matches_torch():
    """Token counts that are odd or not a multiple of the block, windows that are not a multiple of
    eight rows, head sizes other than 128, every dtype: against the same sums done by torch."""
    from rdkv_b200.scoring import _score_one_layer
    gen = torch.Generator(device="cuda").manual_seed(4)
    for (B, H, g, W, T, D), dt in (((1, 3, 2, 5, 1031, 128), torch.float16), ((2, 2, 4, 8, 4096, 96), torch.bfloat16),
                                   ((1, 2, 1, 3, 777, 64), torch.float32), ((1, 1, 7, 9, 2, 256), torch.float16)):
        aw = torch.softmax(torch.randn(B, H, g, W, T, device="cuda", generator=gen), -1).to(dt)
        q = torch.randn(B, H, g, W, D, device="cuda", generator=gen).to(dt)
        k = torch.randn(B, H, T, D, device="cuda", generator=gen).to(dt)
        tok, ch = _score_one_layer(aw, q, None, k, D, k=k)
        want_tok = aw.float().sum(dim=(2, 3)).to(dt).float()
        want_ch = q.float().pow(2).mean(dim=(2, 3)) * k.float().pow(2).mean(dim=2)
        torch.testing.assert_close(tok, want_tok, rtol={torch.float16: 2e-3, torch.bfloat16: 1e-2, torch.float32: 1e-5}[dt],
                                   atol=1e-6)
        torch.testing.assert_close(ch, want_ch, rtol=1e-5, atol=1e-7)
        assert torch.equal(tok, _score_one_layer(aw, q, None, k, D, k=k)[0])   # fixed summation order


@pytest.mark.parametrize("tag", ["f16", "bf16", "f16w32"])
def test_obs_window_scores_match_reference_vectors(tag):
    """Scores straight from the window's queries and the keys (no attention weights in memory) against
    vectors from the reference's scoring step (obkv_fast.py:1443-1450) and its _score_one_layer."""
    from rdkv_b200.scoring import obs_window_scores
    g = load_golden("obs.npz")
    B, H, gq, W, T = (int(x) for x in g[f"{tag}_shape"])
    dt = torch.bfloat16 if tag == "bf16" else torch.float16
    as_t = lambda a: (torch.from_numpy(np.ascontiguousarray(a)).view(torch.int16).view(torch.bfloat16)
                      if tag == "bf16" else torch.from_numpy(np.ascontiguousarray(a))).cuda()
    q, k = as_t(g[f"{tag}_q"]), as_t(g[f"{tag}_k"])
    assert q.dtype == dt
    tok, ch = obs_window_scores(q, k, check_status=True)
    # (the weights are rounded to 16 bits before they are summed, in another order than the reference's)
    np.testing.assert_allclose(to_np(tok), g[f"{tag}_token"], rtol=1.5e-2 if tag == "bf16" else 4e-3, atol=2e-5)
    np.testing.assert_allclose(to_np(ch), g[f"{tag}_channel"], rtol=1e-5)
    assert torch.equal(tok, obs_window_scores(q, k)[0])    # fixed summation order
    # a strided K (a slice of a longer context) and the normalised form
    k_wide = torch.zeros(B, H, T + 5, 128, dtype=dt, device="cuda")
    k_wide[:, :, :T] = k
    tok2, ch2 = obs_window_scores(q, k_wide[:, :, :T], normalise=True)
    norm = torch.full((T,), float(W), device="cuda")
    norm[T - W:] = torch.arange(W, 0, -1, device="cuda").float()
    assert torch.equal(tok2, tok / norm) and torch.equal(ch2, ch)
    with pytest.raises(ValueError):
        obs_window_scores(q.float(), k.float())


def test_obs_window_scores_at_full_size_against_the_two_step_path():
    """Config-1 shape (8 KV heads x 32768 keys, 4 x 32 window rows per head): the fused scores
    against torch's matmul + softmax followed by _score_one_layer on the same device."""
    from rdkv_b200.scoring import _score_one_layer, obs_window_scores
    gen = torch.Generator(device="cuda").manual_seed(8)
    B, H, gq, W, T = 1, 8, 4, 32, 32768
    q = torch.randn(B, H * gq, W, 128, device="cuda", generator=gen).half()
    k = (torch.randn(B, H, T, 128, device="cuda", generator=gen) * 0.5).half()
    tok, ch = obs_window_scores(q, k, check_status=True)
    aw = torch.matmul(q, k.repeat_interleave(gq, dim=1).transpose(-1, -2)) * (1.0 / 128 ** 0.5)
    mask = torch.arange(T, device="cuda")[None, :] > torch.arange(T - W, T, device="cuda")[:, None]
    aw = aw.masked_fill(mask[None, None], float("-inf")).softmax(dim=-1)
    want_tok, want_ch = _score_one_layer(aw.view(B, H, gq, W, T), q.view(B, H, gq, W, 128), None, k, 128, k=k)
    torch.testing.assert_close(tok, want_tok, rtol=1e-2, atol=1e-5)
    torch.testing.assert_close(ch, want_ch, rtol=1e-5, atol=1e-8)


@pytest.mark.parametrize("B,H,gq,W,T,dt,causal,k_pad", [
    (2, 3, 8, 32, 700, torch.float16, True, 0),      # 256 rows: two row blocks in the first pass, 256 columns in the second
    (2, 3, 8, 32, 513, torch.bfloat16, True, 0),
    (2, 3, 3, 20, 450, torch.float16, True, 0),      # window not a multiple of 8: queries staged by plain loads
    (2, 3, 5, 48, 300, torch.bfloat16, True, 0),     # 240 rows, a head's rows straddle the two row blocks
    (2, 3, 2, 24, 257, torch.float16, False, 0),     # 48 rows (zero rows up to 64 / 128), no mask
    (2, 3, 4, 32, 1000, torch.bfloat16, True, 4),    # key rows 132 elements apart: keys staged by unaligned plain loads
    (2, 3, 4, 32, 640, torch.float16, True, 8),      # key rows 136 elements apart: still a valid tensor map
    (1, 40, 4, 32, 3000, torch.float16, True, 0),    # many heads: few CTAs per head, each streams 3-4 tiles through the ring
    (1, 40, 2, 32, 3000, torch.bfloat16, False, 4),  # the same with keys staged by plain loads
    (1, 20, 8, 32, 2500, torch.float16, True, 0),    # two row blocks, several tiles per CTA
    (1, 1, 1, 1, 1, torch.float16, True, 0),
])
def test_obs_window_scores_over_shapes_and_layouts(B, H, gq, W, T, dt, causal, k_pad):
    """Both ways the operands reach shared memory (tensor maps / plain loads), one and two row
    blocks, ragged last tiles, one and several tiles per CTA: against torch's matmul + softmax and
    _score_one_layer on the device."""
    from rdkv_b200.scoring import _score_one_layer, obs_window_scores
    gen = torch.Generator(device="cuda").manual_seed(gq * 1000 + W + T)
    q = torch.randn(B, H * gq, W, 128, device="cuda", generator=gen).to(dt)
    k_store = (torch.randn(B, H, T, 128 + k_pad, device="cuda", generator=gen) * 0.6).to(dt)
    k = k_store[..., :128]
    tok, ch = obs_window_scores(q, k, causal=causal, check_status=True)
    aw = torch.matmul(q, k.repeat_interleave(gq, dim=1).transpose(-1, -2)) * (1.0 / 128 ** 0.5)
    if causal:
        mask = torch.arange(T, device="cuda")[None, :] > torch.arange(T - W, T, device="cuda")[:, None]
        aw = aw.masked_fill(mask[None, None], float("-inf"))
    aw = aw.softmax(dim=-1)
    kc = k.contiguous()
    want_tok, want_ch = _score_one_layer(aw.view(B, H, gq, W, T), q.view(B, H, gq, W, 128), None, kc, 128, k=kc)
    torch.testing.assert_close(tok, want_tok, rtol=3e-2 if dt == torch.bfloat16 else 1e-2, atol=2e-5)
    torch.testing.assert_close(ch, want_ch, rtol=1e-5, atol=1e-8)
    assert torch.equal(tok, obs_window_scores(q, k, causal=causal)[0])


def test_score_pooling_is_bit_exact():
    from rdkv_b200.scoring import apply_score_pooling
    g = load_golden("scoring.npz")
    n = 0
    for key in g:
        if key.startswith("pool_") and not key.endswith("_x"):
            parts = key.split("_")
            src = g["pool_x"] if parts[1] in ("avg", "max") else g[f"pool_{parts[1]}_x"]
            pt, mode, ks = parts[-3], parts[-2], int(parts[-1])
            got = to_np(apply_score_pooling(cuda(src), pt, ks, mode))
            assert got.shape == g[key].shape, key
            assert np.array_equal(got, g[key]), key
            n += 1
    assert n >= 14
    # config-2 sized rows: 8 heads x 32768 tokens, default avg / 5 / reflect, against torch on the same device
    x = torch.randn(8, 32768, device="cuda")
    want = torch.nn.functional.avg_pool1d(torch.nn.functional.pad(x.unsqueeze(1), (2, 2), mode="reflect"), 5, 1).squeeze(1)
    np.testing.assert_allclose(to_np(apply_score_pooling(x, "avg", 5, "reflect")), to_np(want), rtol=1e-6, atol=1e-7)
