"""Drop-in for the reference's `median_cuda_ext` extension module (cudaMedian/median_cuda.cpp:108-112):
forward, backward, dummy, dummy_only with the same arguments and return conventions, over the C ABI."""
from __future__ import annotations

import torch

from . import _lib
from .tvInpaint_cuda_ext import _check_input, _stream_ptr


def forward(in_vol: torch.Tensor):
    """median_forward (median_cuda.cpp:36-70): in_vol [N,H,W,K] -> [solution [N,2,H,W]] (position, crossing weight)."""
    _check_input(in_vol, "in_vol")
    n, h, w, k = in_vol.shape
    out = torch.empty((n, 2, h, w), dtype=torch.float32, device=in_vol.device)
    with torch.cuda.device(in_vol.device):
        rc = _lib.load().cnl_median_forward(in_vol.data_ptr(), out.data_ptr(), None, n, h, w, k, _stream_ptr(in_vol.device))
    _lib.check(rc, "median forward")
    return [out]


def forward_with_index(in_vol: torch.Tensor):
    """Like forward, and also returns the crossing bin per pixel as int32 [N,H,W] (-1: no crossing)."""
    _check_input(in_vol, "in_vol")
    n, h, w, k = in_vol.shape
    out = torch.empty((n, 2, h, w), dtype=torch.float32, device=in_vol.device)
    idx = torch.empty((n, h, w), dtype=torch.int32, device=in_vol.device)
    with torch.cuda.device(in_vol.device):
        rc = _lib.load().cnl_median_forward(in_vol.data_ptr(), out.data_ptr(), idx.data_ptr(), n, h, w, k,
                                            _stream_ptr(in_vol.device))
    _lib.check(rc, "median forward")
    return out, idx


def backward(in_grad: torch.Tensor, in_vol: torch.Tensor):
    """median_backward (median_cuda.cpp:72-106): gradient w.r.t. in_vol as [outGrad]."""
    _check_input(in_vol, "in_vol")
    _check_input(in_grad, "in_grad")
    n, h, w, k = in_vol.shape
    if tuple(in_grad.shape) != (n, 2, h, w):
        raise RuntimeError("in_grad must have shape [N,2,H,W]")
    g = torch.empty_like(in_vol)
    with torch.cuda.device(in_vol.device):
        rc = _lib.load().cnl_median_backward(in_vol.data_ptr(), in_grad.data_ptr(), g.data_ptr(), n, h, w, k,
                                             _stream_ptr(in_vol.device))
    _lib.check(rc, "median backward")
    return [g]


def dummy():
    print("Input: not present just dummy:")
    return []


def dummy_only():
    print("Dummy call:")
    return None
