"""CPU restatement of the learnable weighted-median FILTER built around the reference's selection rule.
TEST INFRASTRUCTURE ONLY.

The reference ships only the selection on a weight vector that sums to one (cudaMedian/cudaCode/medimax.cu:17-100,
restated in oracle/median_ref.py).  The filter of the benchmark configuration wraps it as follows; everything that
is not the selection rule has NO reference counterpart (parity unpinned for those parts):
  * window: k x k taps in row-major offset order, replicate border;
  * the taps are sorted by value (stable: ties keep offset order) and the k*k normalised weights are permuted alike;
  * the reference scan (sequential fp32 running sum, first rank j with score < 0.5 <= score + p_j) selects rank j;
  * output = value of the selected tap (no interpolation); `tap` = its offset index;
  * gradient w.r.t. the weights: the reference's d/dp (with the upstream gradient of the output in the role of the
    position gradient, medimax.cu:73, :91-95) scattered back through the permutation and summed over all pixels;
  * gradient w.r.t. the input: passed through to the selected tap."""
from __future__ import annotations

import numpy as np

f32 = np.float32


def _windows(flow: np.ndarray, k: int):
    n, c, h, w = flow.shape
    r = k // 2
    ys = np.clip(np.arange(h)[:, None] + np.arange(-r, r + 1)[None, :], 0, h - 1)       # [h, k]
    xs = np.clip(np.arange(w)[:, None] + np.arange(-r, r + 1)[None, :], 0, w - 1)       # [w, k]
    win = flow[:, :, ys[:, None, :, None], xs[None, :, None, :]]                        # [n,c,h,w,k,k]
    return win.reshape(n, c, h, w, k * k), ys, xs


def wmedian_forward(flow, p, k: int = 7):
    """flow [N,C,H,W] fp32, p [k*k] fp32 (sums to 1) -> (out [N,C,H,W], tap [N,C,H,W] int32, aux dict for backward)."""
    flow = np.asarray(flow, f32)
    p = np.asarray(p, f32)
    win, ys, xs = _windows(flow, k)
    order = np.argsort(win, axis=-1, kind="stable")
    ps = p[order]                                                   # permuted weights, [N,C,H,W,K]
    K = k * k
    shape = flow.shape
    score = np.zeros(shape, f32)
    found = np.zeros(shape, bool)
    rank = np.full(shape, -1, np.int32)
    pmid = np.ones(shape, f32)
    alpha = np.zeros(shape, f32)
    for r in range(K):
        pr = ps[..., r]
        nxt = (score + pr).astype(f32)
        hit = (~found) & (score < 0.5) & (nxt >= 0.5)
        if hit.any():
            with np.errstate(divide="ignore", invalid="ignore"):
                a = ((1.0 - 2.0 * score.astype(np.float64) - pr.astype(np.float64)) / (2.0 * pr.astype(np.float64))).astype(f32)
            rank[hit] = r
            pmid[hit] = pr[hit]
            alpha[hit] = a[hit]
            found |= hit
        score = np.where(found, score, nxt)
    safe = np.maximum(rank, 0)
    tap = np.take_along_axis(order, safe[..., None].astype(np.int64), axis=-1)[..., 0].astype(np.int32)
    out = np.take_along_axis(win, tap[..., None].astype(np.int64), axis=-1)[..., 0]
    tap = np.where(rank >= 0, tap, -1).astype(np.int32)
    out = np.where(rank >= 0, out, flow).astype(f32)               # no crossing: the centre value passes through
    return out, tap, {"order": order, "rank": rank, "pmid": pmid, "alpha": alpha}


def wmedian_backward(flow, p, grad, k: int = 7):
    """Returns (g_flow [N,C,H,W] fp32, g_p [k*k] float64 summed over all pixels and channels)."""
    flow = np.asarray(flow, f32)
    grad = np.asarray(grad, f32)
    out, tap, aux = wmedian_forward(flow, p, k)
    K = k * k
    order, rank, pmid, alpha = aux["order"], aux["rank"], aux["pmid"], aux["alpha"]
    g0 = grad
    ranks = np.arange(K).reshape((1,) * 4 + (K,))
    rk = rank[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        half = (g0.astype(np.float64) / (2.0 * pmid.astype(np.float64))).astype(f32)          # medimax.cu:91-95
        mid = ((g0 * alpha).astype(f32) / (-pmid)).astype(f32)                                # :73 with g1 = 0
    has = rk >= 0
    d_sorted = np.where(ranks < rk, -half[..., None], np.where(ranks > rk, half[..., None], mid[..., None]))
    d_sorted = np.where(has, d_sorted, -half[..., None]).astype(np.float64)     # no crossing: every bin is "before"
    g_p = np.zeros(K, np.float64)
    np.add.at(g_p, order.reshape(-1), d_sorted.reshape(-1))
    # input gradient: pass-through to the selected tap (replicate border: clamped coordinates)
    n, c, h, w = flow.shape
    r = k // 2
    g_flow = np.zeros(flow.shape, np.float64)
    tt = np.where(tap >= 0, tap, (K - 1) // 2)
    dy, dx = tt // k - r, tt % k - r
    yy = np.clip(np.arange(h).reshape(1, 1, h, 1) + dy, 0, h - 1)
    xx = np.clip(np.arange(w).reshape(1, 1, 1, w) + dx, 0, w - 1)
    ni = np.broadcast_to(np.arange(n).reshape(n, 1, 1, 1), flow.shape)
    ci = np.broadcast_to(np.arange(c).reshape(1, c, 1, 1), flow.shape)
    np.add.at(g_flow, (ni, ci, yy, xx), grad.astype(np.float64))
    return g_flow.astype(f32), g_p
