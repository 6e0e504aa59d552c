"""Shared helpers for the parity tests."""
import numpy as np
import torch

from conftest import SCALAR_FIELDS, TENSOR_FIELDS

ATTN_ATOL, ATTN_RTOL = 2e-3, 1e-2     # tolerance stated for attention outputs (fp16 data, fp32 accumulate)


def to_np(t):
    return None if t is None else t.detach().cpu().numpy()


def layer_to_np(pl) -> dict:
    """rdkv_b200 PackedKVLayer -> dict of numpy arrays / ints (oracle dict format)."""
    d = {f: to_np(getattr(pl, f)) for f in TENSOR_FIELDS + ["K_ch_sort_idx", "K_ch_perm_padded_idx", "sort_idx"]}
    for f in SCALAR_FIELDS:
        d[f] = getattr(pl, f)
    return d


def cuda(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def assert_attn_close(got, want, what=""):
    got, want = np.asarray(got, dtype=np.float32), np.asarray(want, dtype=np.float32)
    err = np.abs(got - want)
    bound = ATTN_ATOL + ATTN_RTOL * np.abs(want)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    assert np.all(err <= bound), f"{what}: max abs err {err.max():.3e} (allowed {ATTN_ATOL} + {ATTN_RTOL}*|ref|)"
