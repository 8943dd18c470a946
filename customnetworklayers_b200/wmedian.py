"""Learnable weighted-median filter: a k x k window whose k*k per-offset weights are learned, built around the
selection rule of the reference's median layer (cudaMedian/cudaCode/medimax.cu:17-100).  The reference ships only the
selection on a per-pixel weight vector (`median.py`); this module is the filter the benchmark configuration describes
(gather window, sort, permute the normalised weights, select)."""
from __future__ import annotations

import torch
from torch import nn
from torch.autograd import Function

from . import _lib
from .dist import allreduce_scalar_grads
from .tvInpaint_cuda_ext import _check_input, _stream_ptr


def forward(flow: torch.Tensor, p: torch.Tensor, k: int):
    """flow [N,C,H,W], p [k*k] normalised weights (CUDA fp32) -> (out [N,C,H,W], tap [N,C,H,W] int32,
    alpha [N,C,H,W] = interpolation factor of the selection rule at the crossing, kept for the backward pass)."""
    _check_input(flow, "flow")
    _check_input(p, "p")
    if p.numel() != k * k:
        raise RuntimeError("p must hold k*k weights")
    n, c, h, w = flow.shape
    out = torch.empty_like(flow)
    tap = torch.empty((n, c, h, w), dtype=torch.int32, device=flow.device)
    alpha = torch.empty_like(flow)
    with torch.cuda.device(flow.device):
        rc = _lib.load().cnl_wmedian_forward(flow.data_ptr(), p.data_ptr(), out.data_ptr(), tap.data_ptr(), alpha.data_ptr(),
                                             n, c, h, w, k, _stream_ptr(flow.device))
    _lib.check(rc, "weighted median forward")
    return out, tap, alpha


def backward(flow, p, tap, alpha, grad, k: int):
    """Returns (g_flow [N,C,H,W], g_p [k*k])."""
    for t, nm in ((flow, "flow"), (p, "p"), (alpha, "alpha"), (grad, "grad")):
        _check_input(t, nm)
    n, c, h, w = flow.shape
    lib = _lib.load()
    g_flow = torch.empty_like(flow)
    g_p = torch.empty(k * k, dtype=torch.float32, device=flow.device)
    scratch = torch.empty(lib.cnl_wmedian_scratch_bytes(k) // 8, dtype=torch.float64, device=flow.device)
    with torch.cuda.device(flow.device):
        rc = lib.cnl_wmedian_backward(flow.data_ptr(), p.data_ptr(), tap.data_ptr(), alpha.data_ptr(), grad.data_ptr(),
                                      g_flow.data_ptr(), g_p.data_ptr(), scratch.data_ptr(), n, c, h, w, k,
                                      _stream_ptr(flow.device))
    _lib.check(rc, "weighted median backward")
    return g_flow, g_p


class WeightedMedianFunction(Function):
    @staticmethod
    def forward(ctx, flow, p, k):
        flow, p = flow.contiguous(), p.contiguous()
        out, tap, alpha = forward(flow, p, k)
        ctx.save_for_backward(flow, p, tap, alpha)
        ctx.k = k
        return out

    @staticmethod
    def backward(ctx, grad):
        flow, p, tap, alpha = ctx.saved_tensors
        g_flow, g_p = backward(flow, p, tap, alpha, grad.contiguous(), ctx.k)
        return g_flow, g_p, None


class WeightedMedianFilter(nn.Module):
    """forward(flow [N,C,H,W]) -> filtered flow.  `weight` holds the k*k raw per-offset weights (row-major window
    offsets); they are normalised to sum to one before the selection, as the reference's rule expects."""

    def __init__(self, k: int = 7):
        super().__init__()
        self.k = k
        self.weight = nn.Parameter(torch.rand(k * k) + 0.5)

    def forward(self, flow):
        p = self.weight / self.weight.sum()
        return WeightedMedianFunction.apply(flow, p, self.k)

    def allreduce_parameter_grads(self) -> None:
        """Data-parallel step: sum the k*k weight gradients over all ranks (the only collective)."""
        if self.weight.grad is not None:
            allreduce_scalar_grads(self.weight.grad)
