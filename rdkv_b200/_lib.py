"""ctypes binding of the C-ABI library (include/rdkv_b200.h).

The library is the only compute path: if it cannot be loaded every operator
raises.  Nothing here falls back to PyTorch or to the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from .build import LIB_PATH

ABI_VERSION = 1

RDKV_F16, RDKV_BF16, RDKV_F32 = 0, 1, 2
PARTIAL_STRIDE = 132
HEAD_DIM = 128

_STATUS_EXC = {1: ValueError, 2: ValueError, 3: ValueError, 4: RuntimeError, 5: RuntimeError}


class TailArgs(C.Structure):
    """Mirror of ``rdkv_tail_args``; field order and types must match the header."""
    _fields_ = [
        ("new_k", C.c_void_p), ("new_v", C.c_void_p), ("view_stride", C.c_int64), ("head_stride", C.c_int64),
        ("dtype", C.c_int32), ("cap", C.c_int32), ("n_new", C.c_int32), ("rope_dtype", C.c_int32),
        ("n_new_per_view", C.c_void_p), ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("rope_view_stride", C.c_int64), ("k_cur", C.c_void_p), ("v_cur", C.c_void_p),
        ("append", C.c_int32), ("reserved", C.c_int32),
    ]


class LayerView(C.Structure):
    """Mirror of ``rdkv_layer_view``; field order and types must match the header."""
    _fields_ = [
        ("k2", C.c_void_p), ("k4", C.c_void_p), ("k8", C.c_void_p),
        ("k2_head_stride", C.c_int64), ("k4_head_stride", C.c_int64), ("k8_head_stride", C.c_int64),
        ("k_scale", C.c_void_p), ("k_zp", C.c_void_p), ("k_perm", C.c_void_p),
        ("k_perm_head_stride", C.c_int64),
        ("v2", C.c_void_p), ("v4", C.c_void_p), ("v8", C.c_void_p),
        ("v2_head_stride", C.c_int64), ("v4_head_stride", C.c_int64), ("v8_head_stride", C.c_int64),
        ("v_scale", C.c_void_p), ("v_zp", C.c_void_p), ("v_meta_head_stride", C.c_int64),
        ("v16", C.c_void_p), ("v16_head_stride", C.c_int64),
        ("v_seg_bounds", C.c_void_p), ("n2", C.c_int32), ("n4", C.c_int32), ("n8", C.c_int32),
        ("n_v16", C.c_void_p), ("n_v16_shared", C.c_int32),
        ("mask", C.c_void_p), ("mask_row_stride", C.c_int64),
        ("n_ch2_pad", C.c_int32), ("n_ch4_pad", C.c_int32), ("n_ch8", C.c_int32),
        ("max_t_v", C.c_int32), ("t_k", C.c_int32), ("reserved", C.c_int32),
        ("k2_bytes", C.c_int64), ("k4_bytes", C.c_int64), ("k8_bytes", C.c_int64),
        ("v2_bytes", C.c_int64), ("v4_bytes", C.c_int64), ("v8_bytes", C.c_int64), ("v16_bytes", C.c_int64),
        ("v_meta_bytes", C.c_int64),
    ]


class PackJob(C.Structure):
    """Mirror of ``rdkv_pack_job`` (one layer of a batched pack); field order and types must match the header."""
    _fields_ = [
        ("K", C.c_void_p), ("V", C.c_void_p),
        ("k_head_stride", C.c_int64), ("k_row_stride", C.c_int64),
        ("v_head_stride", C.c_int64), ("v_row_stride", C.c_int64),
        ("tok_order", C.c_void_p), ("tok_counts", C.c_void_p),
        ("ch_order", C.c_void_p), ("ch_counts", C.c_void_p),
        ("tok_order_row_stride", C.c_int64), ("ch_order_row_stride", C.c_int64),
        ("D", C.c_int32), ("gqa", C.c_int32),
        ("max_n2", C.c_int32), ("max_n4", C.c_int32), ("max_n8", C.c_int32), ("max_n16", C.c_int32),
        ("max_t_v", C.c_int32), ("t_k", C.c_int32),
        ("rows2", C.c_int32), ("rows4", C.c_int32), ("rows8", C.c_int32), ("rows16", C.c_int32),
        ("rows_meta", C.c_int32), ("rows_k", C.c_int32),
        ("n_ch2_pad", C.c_int32), ("n_ch4_pad", C.c_int32), ("n_ch8", C.c_int32), ("d_kept_max", C.c_int32),
        ("v2", C.c_void_p), ("v4", C.c_void_p), ("v8", C.c_void_p),
        ("v16", C.c_void_p), ("v_scale", C.c_void_p), ("v_zp", C.c_void_p),
        ("k2", C.c_void_p), ("k4", C.c_void_p), ("k8", C.c_void_p),
        ("k_scale", C.c_void_p), ("k_zp", C.c_void_p),
        ("sort_idx", C.c_void_p), ("perm", C.c_void_p), ("perm_q", C.c_void_p), ("seg_bounds", C.c_void_p),
        ("scratch", C.c_void_p),
    ]


_lib: Optional[C.CDLL] = None

_i, _i64, _p, _f = C.c_int, C.c_int64, C.c_void_p, C.c_float

_PROTOTYPES = {
    "rdkv_version": ([], _i),
    "rdkv_last_error_string": ([_i], C.c_char_p),
    "rdkv_last_cuda_error": ([], _i),
    "rdkv_sizeof_layer_view": ([], _i),
    "rdkv_sizeof_tail_args": ([], _i),
    "rdkv_k_scores": ([C.POINTER(LayerView), _p, _i, _i64, _i, _i, _i, _p, _i64, _p], _i),
    "rdkv_v_weighted_sum": ([C.POINTER(LayerView), _p, _i64, _i, _i, _p, _i64, _p], _i),
    "rdkv_decode_stage_bytes": ([_i], _i),
    "rdkv_decode_scores": ([_p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _p, _i64, _p, _p], _i),
    "rdkv_decode_weighted_sum": ([_p, _i, _i, _i, _i, _i, _p, _i64, _p, _p, _p], _i),
    "rdkv_decode_attn_partial": ([_p, _i, _p, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p], _i),
    "rdkv_decode_k_blocks": ([_i, _i, _i], _i),
    "rdkv_decode_prepared_bytes": ([_i64, _i, _i], _i64),
    "rdkv_decode_prepare": ([_p, _i, _i, _i, _p, _p, _p, _p], _i),
    "rdkv_decode_v_map_bytes": ([_i], _i64),
    "rdkv_decode_encode_v_maps": ([_p, _i, _p], _i),
    "rdkv_decode_attn": ([_p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p], _i),
    "rdkv_decode_attn_tail": ([_p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p, _p], _i),
    "rdkv_rope": ([_p, _i, _i, _i64, _p, _i, _i, _i64, _p, _p, _i, _p], _i),
    "rdkv_decode_attn_persistent": ([_p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p, _p], _i),
    "rdkv_tail_attn_partial": ([_p, _i, _i64, _i, _i, _p, _p, _i, _i64, _i64, _i64, _i, _p, _i, _p, _p], _i),
    "rdkv_lse_combine": ([_p, _i64, _i, _i64, _i64, _p, _p, _p, _p], _i),
    "rdkv_partition_by_bits": ([_p, _i, _i64, _i, _i, _i, _p, _p, _p], _i),
    "rdkv_pack_v": ([_p, _i64, _i64, _i, _i, _p, _i64, _p, _i64, _i, _i, _i, _i, _i, _i,
                     _p, _p, _p, _p, _p, _p, _i, _i, _p], _i),
    "rdkv_pack_k_slabs": ([_i], _i),
    "rdkv_pack_k": ([_p, _i64, _i64, _i, _i, _p, _i64, _p, _i64, _i, _i, _p, _i64, _p, _i64,
                     _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p], _i),
    "rdkv_obs_scratch_words": ([_i, _i, _i, _i], _i64),
    "rdkv_obs_scores": ([_p, _p, _i, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _i, _p, _p, _p, _p], _i),
    "rdkv_score_chunks": ([_i], _i),
    "rdkv_score_scratch_words": ([_i, _i, _i], _i64),
    "rdkv_score_layer": ([_p, _i, _p, _i, _p, _i, _i64, _i64, _i, _i, _i, _i, _p, _p, _p, _p], _i),
    "rdkv_score_pool": ([_p, _i64, _i, _i, _i, _i, _i, _p, _i64, _i, _p], _i),
    "rdkv_block_scores": ([_p, _i, _i64, _i64, _p, _i, _i64, _i64, _i, _i, _i, _i, _i, _i, _p, _p, _p], _i),
    "rdkv_unpack_layer": ([_p, _i, _i, _p, _i64, _p, _i, _i, _i, _p, _p, _i64, _i, _p], _i),
    "rdkv_sizeof_pack_job": ([], _i),
    "rdkv_pack_kv_batched": ([_p, _i, _i, _i, _i, _i, _i, _i, _i, _p], _i),
    "rdkv_knapsack_batched": ([_p, _i64, _i, _i, _p, C.POINTER(_f), C.POINTER(_f), _i, _i, _f, _p, _p, _p], _i),
    "rdkv_knapsack_rows": ([_p, _i64, _i, _i, _p, C.POINTER(_f), C.POINTER(_f), _i, _i, C.c_double, _p, _p], _i),
    "rdkv_knapsack_static_max_rows": ([], _i),
    "rdkv_knapsack_batched_static": ([_p, _i64, _i, _i, _p, C.POINTER(_f), C.POINTER(_f), _i, _i, _f, _p, _p], _i),
}

EXPORTED_SYMBOLS = tuple(_PROTOTYPES)


def lib() -> C.CDLL:
    """The loaded library; raises if the CUDA extension has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"rdkv_b200: CUDA extension not built ({LIB_PATH} missing). "
                "Run `python -m rdkv_b200.build`; there is no fallback path.")
        handle = C.CDLL(LIB_PATH)
        for name, (argtypes, restype) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
        if handle.rdkv_version() != ABI_VERSION:
            raise RuntimeError("rdkv_b200: library ABI version mismatch; rebuild it")
        if handle.rdkv_sizeof_layer_view() != C.sizeof(LayerView):
            raise RuntimeError("rdkv_b200: rdkv_layer_view layout mismatch between header and binding")
        if handle.rdkv_sizeof_tail_args() != C.sizeof(TailArgs):
            raise RuntimeError("rdkv_b200: rdkv_tail_args layout mismatch between header and binding")
        if handle.rdkv_sizeof_pack_job() != C.sizeof(PackJob):
            raise RuntimeError("rdkv_b200: rdkv_pack_job layout mismatch between header and binding")
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status == 0:
        return
    msg = lib().rdkv_last_error_string(status).decode()
    if status == 4:
        msg += f" [cudaError {lib().rdkv_last_cuda_error()}]"
    raise _STATUS_EXC.get(status, RuntimeError)(f"{what}: {msg}")


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"rdkv_b200: {name} must live on a CUDA device (no CPU path exists)")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    """The current stream of ``device`` for a launch.  The library launches on the CURRENT device, so
    a tensor that lives on another GPU is refused here (wrap the call in ``torch.cuda.device``)."""
    if device is not None:
        idx = torch.device(device).index
        if idx is not None and idx != torch.cuda.current_device():
            raise RuntimeError(f"rdkv_b200: tensors live on cuda:{idx} but the current device is "
                               f"cuda:{torch.cuda.current_device()}; make their device current for the call")
    return torch.cuda.current_stream(device).cuda_stream


def q_dtype_tag(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return RDKV_F16
    if t.dtype == torch.bfloat16:
        return RDKV_BF16
    if t.dtype == torch.float32:
        return RDKV_F32
    raise ValueError(f"query dtype {t.dtype} not supported (fp16, bf16, fp32)")
