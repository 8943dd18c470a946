"""CPU restatement of the reference's weighted-median selection layer (cudaMedian/cudaCode/medimax.cu).
TEST INFRASTRUCTURE ONLY.

Input: a volume of per-bin weights, channel-last [N, H, W, K], assumed to sum to 1 over K ("handled from
outside", medimax.cu:73).  Forward (kMedianScore, medimax.cu:17-42): sequential fp32 running sum over the bins;
at the first bin c with  score < 0.5 <= score + p_c  the output is (c + alpha, p_c) with
alpha = (1 - 2 score - p_c) / (2 p_c) evaluated in double.  Pixels whose weights never reach 0.5 keep (0, 0).
Backward (kMedianScoreGrad, medimax.cu:44-100): gradient w.r.t. every bin.

Pinned by golden vectors produced by the reference's own kernels (tests/golden/median_reference_cuda.npz)."""
from __future__ import annotations

import numpy as np


def median_forward(vol: np.ndarray):
    """vol [N,H,W,K] float32 -> (out [N,2,H,W] float32, crossing index [N,H,W] int32, -1 where no crossing)."""
    vol = np.asarray(vol, dtype=np.float32)
    n, h, w, k = vol.shape
    score = np.zeros((n, h, w), dtype=np.float32)
    found = np.zeros((n, h, w), dtype=bool)
    idx = np.full((n, h, w), -1, dtype=np.int32)
    out = np.zeros((n, 2, h, w), dtype=np.float32)
    for c in range(k):
        p = vol[..., c]
        nxt = (score + p).astype(np.float32)                      # fp32 sum, as in medimax.cu:30
        hit = (~found) & (score < 0.5) & (nxt >= 0.5)
        if hit.any():
            s64 = score.astype(np.float64)
            p64 = p.astype(np.float64)
            with np.errstate(divide="ignore", invalid="ignore"):
                alpha = (1.0 - 2.0 * s64 - p64) / (2.0 * p64)     # :33, double arithmetic
            out[:, 0][hit] = (float(c) + alpha)[hit].astype(np.float32)      # :34
            out[:, 1][hit] = p[hit]                                         # :35
            idx[hit] = c
            found |= hit
        score = np.where(found, score, nxt)                       # threads that broke out stop summing
    return out, idx


def median_backward(vol: np.ndarray, grad: np.ndarray):
    """vol [N,H,W,K], grad [N,2,H,W] -> gradient w.r.t. vol [N,H,W,K] (float32)."""
    vol = np.asarray(vol, dtype=np.float32)
    grad = np.asarray(grad, dtype=np.float32)
    n, h, w, k = vol.shape
    g0 = grad[:, 0]
    g1 = grad[:, 1]
    out = np.zeros_like(vol)
    # first pass (:55-80): locate the crossing, remember pmid and alpha (alpha is stored in a float)
    score = np.zeros((n, h, w), dtype=np.float32)
    found = np.zeros((n, h, w), dtype=bool)
    pmid = np.ones((n, h, w), dtype=np.float32)
    for c in range(k):
        p = vol[..., c]
        nxt = (score + p).astype(np.float32)
        hit = (~found) & (score < 0.5) & (nxt >= 0.5)
        if hit.any():
            with np.errstate(divide="ignore", invalid="ignore"):
                alpha = ((1.0 - 2.0 * score.astype(np.float64) - p.astype(np.float64)) / (2.0 * p.astype(np.float64))).astype(np.float32)
                val = ((g0 * alpha).astype(np.float32) / (-p)).astype(np.float32) + g1          # :73, fp32 arithmetic
            out[..., c][hit] = val.astype(np.float32)[hit]
            pmid[hit] = p[hit]
            found |= hit
        score = np.where(found, score, nxt)
    # second pass (:82-99): bins strictly before / after the crossing
    score = np.zeros((n, h, w), dtype=np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        half = (g0.astype(np.float64) / (2.0 * pmid.astype(np.float64)))
    for c in range(k):
        p = vol[..., c]
        nxt = (score + p).astype(np.float32)
        before = nxt < 0.5
        after = (~before) & (score >= 0.5)
        out[..., c][before] = (-half).astype(np.float32)[before]
        out[..., c][after] = half.astype(np.float32)[after]
        score = nxt
    return out
