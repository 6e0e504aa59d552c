"""Blockwise recompression, CPU side: the block schedule (product code and oracle) and the oracle's
block scoring against vectors produced by the reference's own functions, plus the reference's own
schedule test cases (tests/test_blockwise_rdkv.py:23-66) restated on the product's planner."""
import numpy as np
import pytest

from conftest import load_golden
from oracle import ref_blockwise as RB
from rdkv_b200.blockwise import BlockwiseRDKVConfig, plan_block_compressions


def _rows(events):
    return [(e["block_id"], e["token_start"], e["token_end"], e["query_source_block"], int(e["is_final_flush"]),
             int(e["query_mode"] == "self_causal")) for e in events]


def test_schedule_matches_reference_vectors():
    g = load_golden("blockwise.npz")
    for n, bs in g["plan_cases"].tolist():
        want = [tuple(r) for r in g[f"plan_{n}_{bs}"].tolist()]
        assert RB.plan_block_compressions(n, bs) == want, (n, bs)
        assert _rows(plan_block_compressions(n, bs)) == want, (n, bs)
    for bs in (1, 3, 64):                                   # product planner == oracle on a sweep
        for n in range(0, 6 * bs + 2):
            assert _rows(plan_block_compressions(n, bs)) == RB.plan_block_compressions(n, bs), (n, bs)
    with pytest.raises(ValueError):
        plan_block_compressions(-1, 64)
    with pytest.raises(ValueError):
        plan_block_compressions(10, 0)


def test_schedule_cases_of_the_reference_tests():
    plan = plan_block_compressions(512, 64)
    assert len(plan) == 8 and sum(not e["is_final_flush"] for e in plan) == 7
    assert plan[0]["token_start"] == 0 and plan[-1]["token_end"] == 511 and plan[-1]["query_mode"] == "self_causal"
    for n, blocks in ((128, 2), (192, 3)):
        plan = plan_block_compressions(n, 64)
        assert len(plan) == blocks and plan[-1]["is_final_flush"]
        assert [t for e in plan for t in range(e["token_start"], e["token_end"] + 1)] == list(range(n))
    plan = plan_block_compressions(127, 64)
    assert [(e["token_start"], e["token_end"]) for e in plan] == [(0, 63), (64, 126)]
    assert all(e["is_final_flush"] for e in plan)


def test_block_scoring_oracle_matches_reference_vectors():
    g = load_golden("blockwise.npz")
    tok, ch = RB.score_block(g["score_t_q"], g["score_t_k"], 2, False)
    np.testing.assert_allclose(tok, g["score_t_token"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ch, g["score_t_channel"], rtol=1e-5)
    for tag in ("next", "self", "wide"):
        gq, causal, half = (int(x) for x in g[f"score_{tag}_args"])
        tok, ch = RB.score_block(g[f"score_{tag}_q"], g[f"score_{tag}_k"], gq, bool(causal))
        np.testing.assert_allclose(tok, g[f"score_{tag}_token"], rtol=2e-5, atol=2e-6)
        np.testing.assert_allclose(ch, g[f"score_{tag}_channel"], rtol=1e-5)


def test_bit_accounting_and_config_validation():
    # the reference's accounting case: V (18 + 12) * D=2 = 60, K (2+4)*2 + (8+16)*2 = 60
    assert RB.logical_layer_bits(np.array([[0, 2, 16], [4, 0, 8]]), np.array([[2, 4], [8, 16]]), 2) == 120
    cfg = dict(block_size=64, block_budget_tokens=8, k_budget_ratio=0.5, obs_window=32, pool_kernel_size=5,
               pool_padding="reflect", v_bit_options=None, k_bit_options=None, epsilon_v={}, epsilon_k={})
    BlockwiseRDKVConfig(**cfg).validate()
    for bad in (dict(block_size=0), dict(block_budget_tokens=0), dict(block_budget_tokens=65), dict(k_budget_ratio=1.0)):
        with pytest.raises(ValueError):
            BlockwiseRDKVConfig(**{**cfg, **bad}).validate()
