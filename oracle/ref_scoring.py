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


def obs_window_scores(q_obs: np.ndarray, k: np.ndarray, dtype: str, g: int, causal: bool = True):
    """The reference's scoring step from the observation window's queries (obkv_fast.py:1443-1450)
    followed by score_one_layer: q_obs [B,H_q,W,D], k [B,H_kv,T,D] in `dtype` ("f16", or "bf16" as
    16-bit patterns) -> (token [B,H_kv,T], channel [B,H_kv,D]) fp32.  The scores are the 16-bit
    matmul result times 1/sqrt(D) rounded to 16 bits again, the window is causal (query i of the
    last W positions sees keys <= T-W+i), the softmax output is rounded to 16 bits."""
    from .ref_rope import from_f32, to_f32
    rd = lambda x: to_f32(from_f32(np.ascontiguousarray(x, dtype=F32), dtype), dtype)
    qf, kf = to_f32(q_obs, dtype), to_f32(k, dtype)
    B, H_q, W, D = qf.shape
    H, T = kf.shape[1], kf.shape[2]
    kx = np.repeat(kf, g, axis=1)
    s = rd(rd(np.einsum("bhwd,bhtd->bhwt", qf, kx)) * F32(1.0 / np.sqrt(D)))
    if causal:
        masked = np.arange(T)[None, :] > (T - W + np.arange(W))[:, None]
        s = np.where(masked[None, None], -np.inf, s)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp((s - m).astype(F32)).astype(F32)
    aw = rd(e / e.sum(axis=-1, keepdims=True, dtype=F32))
    tok = rd(aw.reshape(B, H, g * W, T).sum(axis=2, dtype=F32))
    qsq = (qf.reshape(B, H, g * W, D) ** 2).mean(axis=2, dtype=F32)
    ch = qsq * (kf ** 2).mean(axis=2, dtype=F32)
    return tok.astype(F32), ch.astype(F32)
