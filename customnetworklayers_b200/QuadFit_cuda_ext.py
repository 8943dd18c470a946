"""Drop-in for the reference's `QuadFit_cuda_ext` extension module (cudaQuadFit/QuadFit_cuda.cpp:117-122):
forward, backward, dummy, dummy_only over the C ABI.  The returned solution has three channels (fx, fy, score);
the reference's binding allocates two (QuadFit_cuda.cpp:57) while its kernel writes three (quadFit.cu:134)."""
from __future__ import annotations

import torch

from . import _lib
from .tvInpaint_cuda_ext import _check_input, _stream_ptr


def forward(feat0, feat1, flow):
    for t, nm in ((feat0, "feat0"), (feat1, "feat1"), (flow, "flow")):
        _check_input(t, nm)
    n, c, h, w = feat0.shape
    if feat1.shape != feat0.shape or flow.shape[0] != n or tuple(flow.shape[2:]) != (h, w) or flow.shape[1] < 2:
        raise RuntimeError("feat1 must match feat0 and flow must be [N,>=2,H,W]")
    out = torch.empty((n, 3, h, w), dtype=torch.float32, device=feat0.device)
    with torch.cuda.device(feat0.device):
        rc = _lib.load().cnl_quadfit_forward(feat0.data_ptr(), feat1.data_ptr(), flow.data_ptr(), flow.shape[1],
                                             out.data_ptr(), None, n, c, h, w, _stream_ptr(feat0.device))
    _lib.check(rc, "QuadFit forward")
    return [out]


def forward_with_location(feat0, feat1, flow):
    """forward plus the rounded integer location (x, y) per pixel as int32 [N,2,H,W] (-1 where outside)."""
    n, c, h, w = feat0.shape
    out = torch.empty((n, 3, h, w), dtype=torch.float32, device=feat0.device)
    loc = torch.empty((n, 2, h, w), dtype=torch.int32, device=feat0.device)
    with torch.cuda.device(feat0.device):
        rc = _lib.load().cnl_quadfit_forward(feat0.data_ptr(), feat1.data_ptr(), flow.data_ptr(), flow.shape[1],
                                             out.data_ptr(), loc.data_ptr(), n, c, h, w, _stream_ptr(feat0.device))
    _lib.check(rc, "QuadFit forward")
    return out, loc


def backward(grad_sol, feat0, feat1, flow):
    for t, nm in ((feat0, "feat0"), (feat1, "feat1"), (flow, "flow"), (grad_sol, "grad_sol")):
        _check_input(t, nm)
    n, c, h, w = feat0.shape
    if tuple(grad_sol.shape) != (n, 3, h, w):
        raise RuntimeError("grad_sol must be [N,3,H,W]")
    g0 = torch.empty_like(feat0)
    g1 = torch.empty_like(feat1)
    with torch.cuda.device(feat0.device):
        rc = _lib.load().cnl_quadfit_backward(feat0.data_ptr(), feat1.data_ptr(), flow.data_ptr(), flow.shape[1],
                                              grad_sol.data_ptr(), g0.data_ptr(), g1.data_ptr(), n, c, h, w,
                                              _stream_ptr(feat0.device))
    _lib.check(rc, "QuadFit backward")
    return [g0, g1]


def cost_forward(cost5):
    _check_input(cost5, "cost5")
    n, five, h, w = cost5.shape
    if five != 5:
        raise RuntimeError("cost5 must be [N,5,H,W]")
    out = torch.empty((n, 3, h, w), dtype=torch.float32, device=cost5.device)
    with torch.cuda.device(cost5.device):
        rc = _lib.load().cnl_quadfit_cost_forward(cost5.data_ptr(), out.data_ptr(), n, h, w, _stream_ptr(cost5.device))
    _lib.check(rc, "QuadFit cost forward")
    return out


def cost_backward(grad, cost5):
    _check_input(cost5, "cost5")
    _check_input(grad, "grad")
    n, _, h, w = cost5.shape
    g = torch.empty_like(cost5)
    with torch.cuda.device(cost5.device):
        rc = _lib.load().cnl_quadfit_cost_backward(cost5.data_ptr(), grad.data_ptr(), g.data_ptr(), n, h, w,
                                                   _stream_ptr(cost5.device))
    _lib.check(rc, "QuadFit cost backward")
    return g


def dummy():
    print("Input: not present just dummy:")
    return []


def dummy_only():
    print("Dummy call:")
    return None
