import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name), allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


def sub(d, prefix):
    """Entries of d whose key starts with prefix + '_' , prefix stripped."""
    p = prefix + "_"
    return {k[len(p):]: v for k, v in d.items() if k.startswith(p)}


@pytest.fixture(scope="session")
def golden_layers():
    return load_golden("layers.npz")


@pytest.fixture(scope="session")
def golden_unit():
    return load_golden("packing_unit.npz")


@pytest.fixture(scope="session")
def golden_knapsack():
    return load_golden("knapsack.npz")


TENSOR_FIELDS = [
    "K_2bit", "K_4bit", "K_8bit", "K_ch_scale", "K_ch_zp",
    "V_2bit", "V_4bit", "V_8bit", "V_scale", "V_zp",
    "seg_bounds_per_head", "T_eff_per_head", "softmax_mask",
    "K_ch_sort_idx_per_head", "K_ch_perm_padded_idx_per_head", "K_ch_seg_bounds_per_head",
    "K_ch_perm_padded_idx_for_Q", "T_eff_k_per_head", "n_v16_per_head",
]
SCALAR_FIELDS = ["K_ch_seg_bounds", "seg_bounds", "T_eff", "T_eff_k", "n_v16"]


def assert_layer_equal(got: dict, want: dict, what=""):
    """Bit-exact comparison of a packed layer (dict of numpy arrays) with golden fields."""
    for f in TENSOR_FIELDS:
        g, w = got.get(f), want.get(f)
        if w is None:
            assert g is None or g.size == 0, f"{what}{f}: expected absent"
            continue
        assert g is not None, f"{what}{f}: missing"
        g = np.asarray(g)
        assert g.shape == w.shape, f"{what}{f}: shape {g.shape} != {w.shape}"
        assert g.dtype == w.dtype, f"{what}{f}: dtype {g.dtype} != {w.dtype}"
        if g.dtype.kind == "f":
            assert np.array_equal(g.view(f"u{g.dtype.itemsize}"), w.view(f"u{w.dtype.itemsize}")) or \
                np.array_equal(g, w), f"{what}{f}: values differ"
        else:
            assert np.array_equal(g, w), f"{what}{f}: values differ"
    for f in SCALAR_FIELDS:
        assert np.array_equal(np.asarray(got[f], dtype=np.int64), want[f]), f"{what}{f}: {got[f]} != {want[f]}"
