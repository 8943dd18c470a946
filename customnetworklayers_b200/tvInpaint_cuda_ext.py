"""Drop-in for the reference's `tvInpaint_cuda_ext` extension module (cudaTV/TVInpaintFista_cuda.cpp:145-150):
the same four exports -- forward, backward, dummy, dummy_only -- with the same argument order and return
conventions, backed by the C ABI of libcnl_b200.so instead of a pybind module.

Differences from the reference binding, all supersets:
  * a leading batch dimension N >= 1 is accepted (the reference refuses N != 1, :61-65);
  * failures raise RuntimeError carrying the library's message instead of printing and returning [] (:80-87);
  * work is enqueued on the current torch CUDA stream; nothing synchronises the host.
"""
from __future__ import annotations

import torch

from . import _lib


def _check_input(t: torch.Tensor, name: str) -> None:
    # CHECK_INPUT of the reference (TVInpaintFista_cuda.cpp:24-26) plus its fp32 test (:68)
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != torch.float32:
        raise RuntimeError("Input/Output type to cuda operator must be single/float")


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _check_out(t, like, name):
    _check_input(t, name)
    if t.shape != like.shape or t.device != like.device:
        raise RuntimeError(f"{name} must have the shape and device of the tensor it mirrors")


def forward(d_x, d_y, d_c, d_b, d_i, its: int, id: int, out=None):
    """tvInpaint_forward (TVInpaintFista_cuda.cpp:47-88): returns [solution] with the shape of d_b.

    `out` (optional, no reference counterpart): a tensor to receive the solution instead of a fresh allocation, for
    callers that keep their own buffers (the host-buffer pipeline does)."""
    for t, name in ((d_x, "d_x"), (d_y, "d_y"), (d_c, "d_c"), (d_b, "d_b"), (d_i, "d_i")):
        _check_input(t, name)
    n, ch, h, w = d_b.shape
    if d_i.shape != d_b.shape:
        raise RuntimeError("d_i must have the shape of d_b")
    for t, name in ((d_x, "d_x"), (d_y, "d_y"), (d_c, "d_c")):
        if tuple(t.shape) != (n, 1, h, w):
            raise RuntimeError(f"{name} must have shape [N,1,H,W] matching d_b")
    lib = _lib.load()
    if out is None:
        solution = torch.empty_like(d_b)
    else:
        _check_out(out, d_b, "out")
        solution = out
    with torch.cuda.device(d_b.device):
        rc = lib.cnl_tv_forward(d_x.data_ptr(), d_y.data_ptr(), d_c.data_ptr(), d_b.data_ptr(), d_i.data_ptr(),
                                solution.data_ptr(), n, ch, h, w, int(its), int(id), _stream_ptr(d_b.device))
    _lib.check(rc, "tvInpaint forward")
    return [solution]


def backward(d_iGf, d_x, d_y, d_c, d_b, its: int, id: int, generation=None, out=None):
    """tvInpaint_backward (TVInpaintFista_cuda.cpp:99-143): returns [gX, gY, gC, gB, gI].

    `generation` (optional, no reference counterpart): the value forward_count(id) had right after the forward pass
    this call belongs to; if another forward pass has replaced the slot's history since, the call raises instead of
    returning gradients of the wrong problem.
    `out` (optional, no reference counterpart): five tensors [gX, gY, gC, gB, gI] to fill instead of fresh allocations."""
    for t, name in ((d_x, "d_x"), (d_y, "d_y"), (d_c, "d_c"), (d_b, "d_b"), (d_iGf, "d_iGf")):
        _check_input(t, name)
    n, ch, h, w = d_b.shape
    if d_iGf.shape != d_b.shape:
        raise RuntimeError("d_iGf must have the shape of d_b")
    for t, name in ((d_x, "d_x"), (d_y, "d_y"), (d_c, "d_c")):
        if tuple(t.shape) != (n, 1, h, w):
            raise RuntimeError(f"{name} must have shape [N,1,H,W] matching d_b")
    lib = _lib.load()
    if generation is not None:
        with torch.cuda.device(d_b.device):
            now = lib.cnl_tv_forward_count(int(id))
        if now != int(generation):
            raise RuntimeError(f"tvInpaint backward: slot {id} holds forward pass {now}, not {generation}: another forward "
                               f"call on this id replaced the history (give each live layer its own id)")
    if out is None:
        g_x = torch.empty_like(d_x)
        g_y = torch.empty_like(d_y)
        g_c = torch.empty_like(d_c)
        g_b = torch.empty_like(d_b)
        g_i = torch.empty_like(d_b)
    else:
        g_x, g_y, g_c, g_b, g_i = out
        for t, like, name in ((g_x, d_x, "out[0]"), (g_y, d_y, "out[1]"), (g_c, d_c, "out[2]"), (g_b, d_b, "out[3]"),
                              (g_i, d_b, "out[4]")):
            _check_out(t, like, name)
    with torch.cuda.device(d_b.device):
        rc = lib.cnl_tv_backward(d_x.data_ptr(), d_y.data_ptr(), d_c.data_ptr(), d_b.data_ptr(), d_iGf.data_ptr(),
                                 g_x.data_ptr(), g_y.data_ptr(), g_c.data_ptr(), g_b.data_ptr(), g_i.data_ptr(),
                                 n, ch, h, w, int(its), int(id), _stream_ptr(d_b.device))
    _lib.check(rc, "tvInpaint backward")
    return [g_x, g_y, g_c, g_b, g_i]


def dummy():
    """tvInpaint_dummy (TVInpaintFista_cuda.cpp:28-32)."""
    print("Input: not present just dummy:")
    return []


def dummy_only():
    """tvInpaint_dummy_only (TVInpaintFista_cuda.cpp:34-38)."""
    print("Dummy call:")
    return None


# ---- additions without a reference counterpart ---------------------------------------------------------------
def release(id: int) -> None:
    """Frees the device buffers of slot `id` on the current device."""
    _lib.check(_lib.load().cnl_tv_release(int(id)), "tvInpaint release")


def forward_count(id: int, device=None) -> int:
    """Forward passes stored on slot `id` of `device` (default: current device) so far; see backward(generation=...)."""
    with torch.cuda.device(device):
        k = _lib.load().cnl_tv_forward_count(int(id))
    if k < 0:
        raise RuntimeError("tvInpaint forward_count: " + _lib.last_error())
    return k


def set_option(id: int, option: int, value: int) -> None:
    _lib.check(_lib.load().cnl_tv_set_option(int(id), int(option), int(value)), "tvInpaint set_option")


def lambda_grad(g_c: torch.Tensor, c_raw: torch.Tensor, out=None, scratch=None) -> torch.Tensor:
    """sum(g_c * c_raw) as a 1-element CUDA tensor: the gradient of a learned scalar lambda in c = lambda * c_raw.
    `out` (1 float) and `scratch` (cnl_dot_scratch_floats() floats) may be supplied by callers that keep their own."""
    _check_input(g_c, "g_c")
    _check_input(c_raw, "c_raw")
    if g_c.numel() != c_raw.numel():
        raise RuntimeError("g_c and c_raw must have the same number of elements")
    lib = _lib.load()
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=g_c.device)
    if scratch is None:
        scratch = torch.empty(lib.cnl_dot_scratch_floats(), dtype=torch.float32, device=g_c.device)
    elif scratch.numel() < lib.cnl_dot_scratch_floats() or scratch.dtype != torch.float32 or not scratch.is_cuda:
        raise RuntimeError("scratch must be a CUDA float tensor of at least cnl_dot_scratch_floats() elements")
    with torch.cuda.device(g_c.device):
        rc = lib.cnl_tv_lambda_grad(g_c.data_ptr(), c_raw.data_ptr(), g_c.numel(), out.data_ptr(),
                                    scratch.data_ptr(), _stream_ptr(g_c.device))
    _lib.check(rc, "tvInpaint lambda_grad")
    return out


def read_history(id: int, like: torch.Tensor, its: int):
    """Stored iterates of the last forward(id): (hist [its_eff,N,C,H,W], ckpt_y [K,N,C,H,W]) as CUDA tensors."""
    lib = _lib.load()
    its_eff = 2 * (int(its) // 2)
    with torch.cuda.device(like.device):
        k = lib.cnl_tv_num_checkpoints(int(id))
        if k < 0:
            raise RuntimeError("slot holds no forward pass")
        hist = torch.empty((its_eff,) + tuple(like.shape), dtype=torch.float32, device=like.device)
        ck = torch.empty((k,) + tuple(like.shape), dtype=torch.float32, device=like.device)
        st = _stream_ptr(like.device)
        for g in range(its_eff):
            _lib.check(lib.cnl_tv_read_history(int(id), g, hist[g].data_ptr(), st), "read_history")
        for i in range(k):
            _lib.check(lib.cnl_tv_read_checkpoint(int(id), i, ck[i].data_ptr(), st), "read_checkpoint")
    return hist, ck


def get_timing(id: int) -> dict:
    """CUDA-event records made while option OPT_TIMING was on (see cnl_tv_get_timing); clears them."""
    import ctypes
    buf = (ctypes.c_double * 8)()
    _lib.check(_lib.load().cnl_tv_get_timing(int(id), ctypes.cast(buf, ctypes.c_void_p)), "get_timing")
    return {"fwd_ms": buf[0], "fwd_launches": int(buf[1]), "fwd_calls": int(buf[2]),
            "rev_ms": buf[3], "rev_launches": int(buf[4]), "rev_calls": int(buf[5]),
            "fwd_iters": int(buf[6]), "rev_iters": int(buf[7])}
