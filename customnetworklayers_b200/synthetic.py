"""Seeded synthetic inputs of the benchmark configurations (CPU tensors; no CUDA needed).

They stand in for the optical-flow benchmark images the reference's paper was evaluated on, which are not
available offline: same shapes and value ranges, generated from a seed."""
from __future__ import annotations

import torch

def _gaussian_smooth(img: torch.Tensor, sigma: float = 2.0, radius: int = 6) -> torch.Tensor:
    xs = torch.arange(-radius, radius + 1, dtype=torch.float64)
    k = torch.exp(-0.5 * (xs / sigma) ** 2)
    k = (k / k.sum()).to(img.dtype)
    n = img.shape[0]
    pad = torch.nn.functional.pad
    r = min(radius, img.shape[-1] - 1)
    rh = min(radius, img.shape[-2] - 1)
    mode_w = "reflect" if r == radius else "replicate"
    mode_h = "reflect" if rh == radius else "replicate"
    out = torch.nn.functional.conv2d(pad(img, (radius, radius, 0, 0), mode=mode_w), k.view(1, 1, 1, -1))
    out = torch.nn.functional.conv2d(pad(out, (0, 0, radius, radius), mode=mode_h), k.view(1, 1, -1, 1))
    assert out.shape[0] == n
    return out


def make_inputs(n: int, ch: int, h: int, w: int, seed: int = 1234, conf_p: float = 0.3):
    """Seeded synthetic stand-in for optical-flow inpainting inputs (fp32 CPU tensors).

    flow b ~ U(-20, 20); init = b; c = Bernoulli(conf_p) * U(0,1); guide I ~ N(0,1) smoothed (sigma 2);
    wx = exp(-10 |I[h,w+1]-I[h,w]|), wy = exp(-10 |I[h+1,w]-I[h,w]|), last column / row = 1; upstream grad ~ N(0,1)."""
    gen = torch.Generator().manual_seed(seed)
    b = (torch.rand(n, ch, h, w, generator=gen) * 40.0 - 20.0).float()
    mask = (torch.rand(n, 1, h, w, generator=gen) < conf_p).float()
    c = (mask * torch.rand(n, 1, h, w, generator=gen)).float()
    guide = _gaussian_smooth(torch.randn(n, 1, h, w, generator=gen).float())
    wx = torch.ones(n, 1, h, w)
    wy = torch.ones(n, 1, h, w)
    if w > 1:
        wx[..., :, :-1] = torch.exp(-10.0 * (guide[..., :, 1:] - guide[..., :, :-1]).abs())
    if h > 1:
        wy[..., :-1, :] = torch.exp(-10.0 * (guide[..., 1:, :] - guide[..., :-1, :]).abs())
    grad = torch.randn(n, ch, h, w, generator=gen).float()
    return {"wx": wx.contiguous(), "wy": wy.contiguous(), "c": c.contiguous(), "b": b.contiguous(),
            "init": b.clone(), "grad": grad.contiguous()}


def make_median_volume(n: int, h: int, w: int, k: int, seed: int = 1238, peaky: bool = True):
    """Per-pixel weight vectors [n,h,w,k] that sum to 1 (fp32): U(0.5,1.5) weights, optionally sharpened so that the
    crossing bin varies over the whole range, plus an upstream gradient [n,2,h,w] ~ N(0,1)."""
    gen = torch.Generator().manual_seed(seed)
    vol = torch.rand(n, h, w, k, generator=gen) + 0.5
    if peaky:
        centre = torch.randint(0, k, (n, h, w, 1), generator=gen).float()
        bins = torch.arange(k).float().view(1, 1, 1, k)
        vol = vol * torch.exp(-0.5 * ((bins - centre) / max(1.0, k / 8.0)) ** 2) + 1e-3 * vol
    vol = (vol / vol.sum(dim=-1, keepdim=True)).float().contiguous()
    grad = torch.randn(n, 2, h, w, generator=gen).float()
    return vol, grad


def make_quadfit_inputs(n: int, c: int, h: int, w: int, seed: int = 1237, max_disp: float = 6.0):
    """Feature maps whose correlation peaks near the true displacement: feat1 is feat0 warped by a smooth integer-ish
    flow plus noise; the initial flow is the true one perturbed by up to half a pixel (and pushed out of the image
    in one corner).  Returns fp32 CPU tensors feat0, feat1 [n,c,h,w], flow [n,2,h,w], grad [n,3,h,w]."""
    gen = torch.Generator().manual_seed(seed)
    base = _gaussian_smooth(torch.randn(n * c, 1, h, w, generator=gen).float(), sigma=1.5, radius=4).view(n, c, h, w)
    feat0 = base / base.std() if base.numel() > 1 else base + 1.0
    dx = int(max_disp // 2)
    feat1 = torch.roll(feat0, shifts=(1, dx), dims=(2, 3)) + 0.05 * torch.randn(n, c, h, w, generator=gen)
    flow = torch.empty(n, 2, h, w)
    flow[:, 0] = dx + (torch.rand(n, h, w, generator=gen) - 0.5)
    flow[:, 1] = 1 + (torch.rand(n, h, w, generator=gen) - 0.5)
    flow[:, :, : max(1, h // 8), : max(1, w // 8)] -= 3.0 * max_disp          # leaves the image
    grad = torch.randn(n, 3, h, w, generator=gen).float()
    return feat0.float().contiguous(), feat1.float().contiguous(), flow.float().contiguous(), grad


def make_cost_patches(n: int, h: int, w: int, seed: int = 1237):
    """5-point stencils of a score to maximise: minus (quadratic bowl with sub-pixel minimum in (-0.5,0.5)^2 and
    curvature U(0.5,2) plus N(0,0.05) noise).  Returns cost5 [n,5,h,w] ordered (c00, c0+, c+0, c0-, c-0) and the
    true sub-pixel offsets [n,2,h,w]."""
    gen = torch.Generator().manual_seed(seed)
    off = torch.rand(n, 2, h, w, generator=gen) - 0.5
    curv = torch.rand(n, 2, h, w, generator=gen) * 1.5 + 0.5
    def bowl(dx, dy):
        v = curv[:, 0] * (dx - off[:, 0]) ** 2 + curv[:, 1] * (dy - off[:, 1]) ** 2
        return -(v + 0.05 * torch.randn(n, h, w, generator=gen))
    cost5 = torch.stack([bowl(0, 0), bowl(1, 0), bowl(0, 1), bowl(-1, 0), bowl(0, -1)], dim=1)
    return cost5.float().contiguous(), off.float()


def make_tgv_inputs(n: int, ch: int, h: int, w: int, seed: int = 1236, conf_p: float = 0.2, alpha0: float = 1.0,
                    alpha1: float = 2.0):
    """TGV stand-in inputs: dx = [alpha0*wx, alpha1*1], dy = [alpha0*wy, alpha1*1] as [n,2,h,w]; b ~ U(-20,20);
    c = Bernoulli(conf_p)*U(0,1); init = [b, 0, 0] as [n,3,ch,h,w]; upstream gradient ~ N(0,1) on all three planes."""
    I = make_inputs(n, ch, h, w, seed=seed, conf_p=conf_p)
    gen = torch.Generator().manual_seed(seed + 7)
    dx = torch.cat([alpha0 * I["wx"], torch.full_like(I["wx"], alpha1)], dim=1).contiguous()
    dy = torch.cat([alpha0 * I["wy"], torch.full_like(I["wy"], alpha1)], dim=1).contiguous()
    init = torch.zeros(n, 3, ch, h, w)
    init[:, 0] = I["b"]
    grad = torch.randn(n, 3, ch, h, w, generator=gen).float()
    return {"dx": dx, "dy": dy, "c": I["c"], "b": I["b"], "init": init.contiguous(), "grad": grad.contiguous()}


def make_hierarchy_inputs(n: int, h: int, w: int, levels: int = 3, seed: int = 1237):
    """Inputs of the coarse-to-fine stack: per level (coarse to fine, each half the next one's size) edge weights,
    confidence, integer match offsets uniform in +-64 px (scaled with the level) and 5-point cost stencils."""
    out = []
    for l in range(levels):
        s = 2 ** (levels - 1 - l)
        hl, wl = h // s, w // s
        I = make_inputs(n, 2, hl, wl, seed=seed + 10 * l)
        gen = torch.Generator().manual_seed(seed + 10 * l + 5)
        offsets = torch.randint(-64 // s, 64 // s + 1, (n, 2, hl, wl), generator=gen).float()
        cost5, _ = make_cost_patches(n, hl, wl, seed=seed + 10 * l + 7)
        out.append({"wx": I["wx"], "wy": I["wy"], "c": I["c"], "offsets": offsets.contiguous(), "cost5": cost5})
    grad = torch.randn(n, 2, h, w, generator=torch.Generator().manual_seed(seed + 99)).float()
    return out, grad


def make_median_filter_inputs(n: int, c: int, h: int, w: int, k: int = 7, seed: int = 1238):
    """Flow ~ U(-20,20) with 5 % of the pixels replaced by outliers ~ U(-200,200); k*k raw weights ~ U(0.5,1.5);
    upstream gradient ~ N(0,1).  Returns (flow, raw_weights, grad) as fp32 CPU tensors."""
    gen = torch.Generator().manual_seed(seed)
    flow = torch.rand(n, c, h, w, generator=gen) * 40.0 - 20.0
    outlier = torch.rand(n, c, h, w, generator=gen) < 0.05
    flow = torch.where(outlier, torch.rand(n, c, h, w, generator=gen) * 400.0 - 200.0, flow)
    weights = torch.rand(k * k, generator=gen) + 0.5
    grad = torch.randn(n, c, h, w, generator=gen)
    return flow.float().contiguous(), weights.float(), grad.float().contiguous()
