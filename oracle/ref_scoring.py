"""CPU restatement (numpy) of the reference's importance scoring and score pooling.

TEST INFRASTRUCTURE ONLY: imported by tests/ and by nothing in the product path.
Follows obkv_fast.py:854-896 (_score_one_layer) and obkv_fast.py:208-246
(apply_score_pooling; torch's avg_pool1d / max_pool1d semantics: taps added in ascending
order in fp32 and divided once by the window size; zero padding counts as zeros for the
average and is no candidate for the maximum).  Pinned by tests/golden/scoring.npz, generated
from the reference's own functions.
"""
import numpy as np

F32 = np.float32


def score_one_layer(aw: np.ndarray, q: np.ndarray, k: np.ndarray):
    """aw [B,H,g,W,T], q [B,H,g,W,D], k [B,H,T,D] -> (token [B,H,T], channel [B,H,D]) fp32."""
    token = aw.astype(F32).sum(axis=(2, 3), dtype=F32).astype(aw.dtype).astype(F32)
    qn = np.square(q.astype(F32)).mean(axis=(2, 3), dtype=F32)
    kn = np.square(k.astype(F32)).mean(axis=2, dtype=F32)
    return token, (qn * kn).astype(F32)


def score_pooling(scores: np.ndarray, pool_type: str, kernel_size: int, padding_mode: str = "zero") -> np.ndarray:
    x = np.atleast_2d(scores).astype(F32)
    n = x.shape[1]
    reflect = padding_mode == "reflect"
    taps = min(kernel_size, 2 * n - 1) if reflect else kernel_size
    pad = taps // 2
    out_len = n + 2 * pad - taps + 1
    out = np.empty((x.shape[0], out_len), F32)
    for i in range(out_len):
        acc = np.full(x.shape[0], -np.inf if pool_type != "avg" else 0.0, F32)
        for w in range(taps):
            j = i - pad + w
            if reflect:
                if j < 0:
                    j = -j
                if j >= n:
                    j = 2 * (n - 1) - j
            if j < 0 or j >= n:
                continue
            acc = np.maximum(acc, x[:, j]) if pool_type != "avg" else (acc + x[:, j]).astype(F32)
        out[:, i] = acc if pool_type != "avg" else (acc / F32(taps)).astype(F32)
    return out[0] if scores.ndim == 1 else out
