"""Drop-in for the reference's `tgvInpaint_cuda_ext` extension module (cudaTGV/TGVInpaintFista_cuda.cpp:175-180):
forward, backward, dummy, dummy_only over the C ABI.  d_x = [wx, beta_x], d_y = [wy, beta_y] are N x 2 x H x W;
d_i, the solution and their gradients are N x 3C x H x W ordered u(C), v1(C), v2(C)."""
from __future__ import annotations

import torch

from . import _lib
from .tvInpaint_cuda_ext import _check_input, _stream_ptr


def _shapes(d_x, d_y, d_c, d_b, d_i):
    n, ch, h, w = d_b.shape
    if tuple(d_x.shape) != (n, 2, h, w) or tuple(d_y.shape) != (n, 2, h, w):
        raise RuntimeError("d_x and d_y must be [N,2,H,W] (edge weight, beta)")
    if tuple(d_c.shape) != (n, 1, h, w):
        raise RuntimeError("d_c must be [N,1,H,W]")
    if tuple(d_i.shape) != (n, 3 * ch, h, w):
        raise RuntimeError("d_i must be [N,3*C,H,W] (primary and two auxiliary planes per channel)")
    return n, ch, h, w


def forward(d_x, d_y, d_c, d_b, d_i, its: int, id: int):
    for t, nm in ((d_x, "d_x"), (d_y, "d_y"), (d_c, "d_c"), (d_b, "d_b"), (d_i, "d_i")):
        _check_input(t, nm)
    n, ch, h, w = _shapes(d_x, d_y, d_c, d_b, d_i)
    out = torch.empty_like(d_i)
    with torch.cuda.device(d_b.device):
        rc = _lib.load().cnl_tgv_forward(d_x.data_ptr(), d_y.data_ptr(), d_c.data_ptr(), d_b.data_ptr(), d_i.data_ptr(),
                                         out.data_ptr(), n, ch, h, w, int(its), int(id), _stream_ptr(d_b.device))
    _lib.check(rc, "tgvInpaint forward")
    return [out]


def backward(d_iGf, d_x, d_y, d_c, d_b, its: int, id: int):
    for t, nm in ((d_x, "d_x"), (d_y, "d_y"), (d_c, "d_c"), (d_b, "d_b"), (d_iGf, "d_iGf")):
        _check_input(t, nm)
    n, ch, h, w = _shapes(d_x, d_y, d_c, d_b, d_iGf)
    g = [torch.empty_like(d_x), torch.empty_like(d_y), torch.empty_like(d_c), torch.empty_like(d_b), torch.empty_like(d_iGf)]
    with torch.cuda.device(d_b.device):
        rc = _lib.load().cnl_tgv_backward(d_x.data_ptr(), d_y.data_ptr(), d_c.data_ptr(), d_b.data_ptr(), d_iGf.data_ptr(),
                                          g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), g[3].data_ptr(),
                                          g[4].data_ptr(), n, ch, h, w, int(its), int(id), _stream_ptr(d_b.device))
    _lib.check(rc, "tgvInpaint backward")
    return g


def dummy():
    print("Input: not present just dummy:")
    return []


def dummy_only():
    print("Dummy call:")
    return None


def release(id: int) -> None:
    _lib.check(_lib.load().cnl_tgv_release(int(id)), "tgvInpaint release")


def set_option(id: int, option: int, value: int) -> None:
    _lib.check(_lib.load().cnl_tgv_set_option(int(id), int(option), int(value)), "tgvInpaint set_option")


def read_history(id: int, like: torch.Tensor, its: int):
    """(hist [its_eff, ...like.shape], ckpt_y [K, ...], L [N]) of the last forward(id), as CUDA tensors."""
    lib = _lib.load()
    its_eff = 2 * (int(its) // 2)
    with torch.cuda.device(like.device):
        k = lib.cnl_tgv_num_checkpoints(int(id))
        if k < 0:
            raise RuntimeError("slot holds no forward pass")
        st = _stream_ptr(like.device)
        hist = torch.empty((its_eff,) + tuple(like.shape), dtype=torch.float32, device=like.device)
        ck = torch.empty((k,) + tuple(like.shape), dtype=torch.float32, device=like.device)
        L = torch.empty(like.shape[0], dtype=torch.float32, device=like.device)
        for g in range(its_eff):
            _lib.check(lib.cnl_tgv_read_state(int(id), 0, g, hist[g].data_ptr(), st), "read_state")
        for i in range(k):
            _lib.check(lib.cnl_tgv_read_state(int(id), 1, i, ck[i].data_ptr(), st), "read_state")
        _lib.check(lib.cnl_tgv_read_state(int(id), 2, 0, L.data_ptr(), st), "read_state")
    return hist, ck, L
