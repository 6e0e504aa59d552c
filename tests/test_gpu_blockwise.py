"""Blockwise recompression on the GPU (through the C ABI): block scoring against vectors from the
reference's _score_block, one block through compress_block bit for bit against the reference's
_compress_block, and attention over several packed sources plus a tail against the reference's
dequantised caches."""
import numpy as np
import pytest
import torch

from conftest import assert_layer_equal, load_golden, sub
from helpers import assert_attn_close, cuda, layer_to_np, to_np

pytestmark = pytest.mark.gpu


def test_block_scores_match_reference_vectors():
    from rdkv_b200.blockwise import _channel_score, _score_block
    g = load_golden("blockwise.npz")
    tok, ch = _score_block(cuda(g["score_t_q"]), cuda(g["score_t_k"]), num_kv_groups=2, causal=False)
    np.testing.assert_allclose(to_np(tok), g["score_t_token"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(to_np(ch), g["score_t_channel"], rtol=1e-5)
    for tag in ("next", "self", "wide"):
        gq, causal, half = (int(x) for x in g[f"score_{tag}_args"])
        dt = torch.float16 if half else torch.float32
        q, k = cuda(g[f"score_{tag}_q"]).to(dt), cuda(g[f"score_{tag}_k"]).to(dt)
        tok, ch = _score_block(q, k, num_kv_groups=gq, causal=bool(causal))
        np.testing.assert_allclose(to_np(tok), g[f"score_{tag}_token"], rtol=2e-5, atol=2e-6)
        np.testing.assert_allclose(to_np(ch), g[f"score_{tag}_channel"], rtol=1e-5)
        np.testing.assert_allclose(to_np(_channel_score(q, k, num_kv_groups=gq)), g[f"score_{tag}_channel"], rtol=1e-5)
    with pytest.raises(ValueError):                         # the causal form needs as many queries as keys
        _score_block(cuda(g["score_t_q"]), cuda(g["score_t_k"]), num_kv_groups=2, causal=True)
    # the causal case of the reference's test: the last key is seen by the last query only
    q = torch.ones(1, 4, 2, device="cuda")
    k = torch.tensor([[[[1.0, 0.0], [0.0, 1.0], [1.0, 1.0], [2.0, 0.0]]]], device="cuda")
    tok, _ = _score_block(q, k, num_kv_groups=1, causal=True)
    assert float(tok[0, 0]) > float(tok[0, 3]) and bool(torch.isfinite(tok).all())


def _config():
    from rdkv_b200.blockwise import BlockwiseRDKVConfig
    from rdkv_b200.knapsack_solver import DEFAULT_EPSILON_K, DEFAULT_EPSILON_V
    return BlockwiseRDKVConfig(block_size=64, block_budget_tokens=8, k_budget_ratio=0.5, obs_window=32,
                               pool_kernel_size=5, pool_padding="reflect", v_bit_options=None, k_bit_options=None,
                               epsilon_v=dict(DEFAULT_EPSILON_V), epsilon_k=dict(DEFAULT_EPSILON_K), correctness_check=True)


def _block(g):
    from rdkv_b200.blockwise import compress_block
    hkv, gq, T = (int(x) for x in g["block_args"])
    return compress_block(target_kv=[cuda(g[f"block_l{l}_kv"]) for l in range(2)],
                          query_block=[cuda(g[f"block_l{l}_q"]).half() for l in range(2)],
                          token_scores_by_layer=[cuda(g[f"block_l{l}_token_scores"]) for l in range(2)],
                          block_id=0, token_start=0, token_end=T - 1, config=_config(), num_kv_groups=gq), gq


def test_compress_block_matches_reference_block():
    """One 64-token block, two layers: every packed field and the logical bits, bit for bit, against
    the reference's _compress_block (K rows of 31 + 6..7 + 4 bytes: the unaligned widths)."""
    from rdkv_b200.blockwise import _logical_layer_bits
    g = load_golden("blockwise.npz")
    block, gq = _block(g)
    for l in range(2):
        assert_layer_equal(layer_to_np(block.packed[l]), sub(g, f"block_l{l}"), f"block layer {l}.")
        assert block.new_v_only[l] is None or f"block_l{l}_new_v_only" in g
        assert _logical_layer_bits(block.packed[l], 128) == int(g["block_logical_bits"][l])
    assert np.array_equal(to_np(block.logical_bits_per_layer), g["block_logical_bits"])


def test_attention_over_prompt_block_and_tail():
    """One softmax over the prompt's packed layer, a compressed decode block and the uncompressed
    tail, against the same softmax over the reference's dequantised caches."""
    from rdkv_b200.blockwise import multi_source_attention
    from rdkv_b200.packing import pack_kv
    g = load_golden("blockwise.npz")
    block, gq = _block(g)
    prompt = pack_kv(cuda(g["ms_K"]), cuda(g["ms_V"]), cuda(g["ms_v_bits"]), cuda(g["ms_k_bits"]), gq)
    sources = [prompt, (block.packed[0], block.new_v_only[0])]
    q = cuda(g["ms_q"])
    n = g["ms_tail_k"].shape[1]
    new_k = torch.zeros((1, g["ms_tail_k"].shape[0], n + 3, 128), dtype=torch.float16, device="cuda")
    new_v = torch.zeros_like(new_k)
    new_k[0, :, :n], new_v[0, :, :n] = cuda(g["ms_tail_k"]), cuda(g["ms_tail_v"])
    out, table = multi_source_attention(q, sources, new_k=new_k, new_v=new_v, n_new=n)
    assert_attn_close(to_np(out), g["ms_attn_out"], "prompt + block + tail")
    out2, table2 = multi_source_attention(q, sources, new_k=new_k, new_v=new_v, n_new=n, table=table)
    assert table2 is table and torch.equal(out, out2)
    table.check_status()
