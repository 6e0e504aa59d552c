"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "rdkv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rdkv_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from rdkv_b200 import _lib
    from rdkv_b200.build import LIB_PATH, build
    build()
    handle = ctypes.CDLL(LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared, "ctypes binding and header disagree"


def test_struct_layout_and_version():
    from rdkv_b200 import _lib
    lib = _lib.lib()
    assert lib.rdkv_version() == _lib.ABI_VERSION
    assert lib.rdkv_sizeof_layer_view() == ctypes.sizeof(_lib.LayerView)
    assert lib.rdkv_sizeof_tail_args() == ctypes.sizeof(_lib.TailArgs)
    assert lib.rdkv_last_error_string(0) == b"ok"
    assert b"argument" in lib.rdkv_last_error_string(1)
    assert lib.rdkv_decode_stage_bytes(34) >= 4096 + 64 * 34 and lib.rdkv_decode_stage_bytes(34) % 128 == 0
    assert lib.rdkv_decode_v_map_bytes(3) == 3 * 4 * 128 and lib.rdkv_decode_v_map_bytes(-1) == -1
    assert lib.rdkv_decode_encode_v_maps(None, 1, None) == -1
    assert lib.rdkv_pack_k_slabs(1) == 2 and lib.rdkv_pack_k_slabs(10 ** 6) <= 65   # slabs + the block of final parameters
    assert lib.rdkv_sizeof_pack_job() == ctypes.sizeof(_lib.PackJob)


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected on the host before any launch."""
    from rdkv_b200 import _lib
    lib = _lib.lib()
    assert lib.rdkv_lse_combine(None, 1, 1, 132, 132, None, None, None, None) == 1
    assert lib.rdkv_partition_by_bits(None, 8, 0, 1, 1, 0, None, None, None) == 1
    v = _lib.LayerView()
    assert lib.rdkv_k_scores(ctypes.byref(v), None, 0, 128, 32, 8, 16, None, 16, None) == 1
    assert lib.rdkv_decode_attn_partial(1, 1, 1, 0, 30, 8, 256, 1, 34, 1, None, None, None) == 2   # H_q % H_kv != 0


def test_ops_refuse_cpu_tensors():
    import torch
    from rdkv_b200 import knapsack_solver, packing
    with pytest.raises(RuntimeError, match="CUDA"):
        knapsack_solver.knapsack_bit_allocation_batched(torch.ones(2, 8), 2.0)
    with pytest.raises(RuntimeError, match="CUDA"):
        packing.pack_v_segments(torch.zeros(1, 1, 4, 8, dtype=torch.float16), torch.tensor([2, 2, 4, 8]))
