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
