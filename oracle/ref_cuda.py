"""ctypes loader for oracle/_ref/libtvref.so: the reference's own cudaTV kernels, built unmodified by
oracle/build_ref.py.  TEST INFRASTRUCTURE ONLY (second checker on a GPU box, and the reference's own B200 timing).

The reference handles one image per call (batch 1), image height a multiple of 16 and width a multiple of 32."""
import ctypes
import os

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libtvref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(LIB_PATH)
        lib.ref_tv_forward.restype = ctypes.c_int
        lib.ref_tv_forward.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 5
        lib.ref_tv_backward.restype = ctypes.c_int
        lib.ref_tv_backward.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_int] * 5
        _lib = lib
    return _lib


def forward(wx, wy, c, b, init, its, pid):
    """Tensors are CUDA fp32, shapes [1,1,H,W] / [1,C,H,W]; returns the solution [1,C,H,W]."""
    import torch
    assert b.shape[0] == 1
    _, ch, h, w = b.shape
    out = torch.zeros_like(b)
    torch.cuda.synchronize()
    rc = load().ref_tv_forward(wx.data_ptr(), wy.data_ptr(), c.data_ptr(), b.data_ptr(), init.data_ptr(),
                               out.data_ptr(), ch, h, w, int(its), int(pid))
    if rc != 0:
        raise RuntimeError(f"reference forward returned {rc}")
    return out


def backward(grad, wx, wy, c, b, its, pid):
    import torch
    assert b.shape[0] == 1
    _, ch, h, w = b.shape
    g = [torch.zeros_like(t) for t in (wx, wy, c, b, b)]
    grad = grad.clone()          # the reference zeroes non-finite entries of the upstream gradient in place
    torch.cuda.synchronize()
    rc = load().ref_tv_backward(wx.data_ptr(), wy.data_ptr(), c.data_ptr(), b.data_ptr(), grad.data_ptr(),
                                g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), g[3].data_ptr(), g[4].data_ptr(),
                                ch, h, w, int(its), int(pid))
    if rc != 0:
        raise RuntimeError(f"reference backward returned {rc}")
    return g


# ---- cudaMedian -------------------------------------------------------------------------------------------------
MEDIAN_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libmedianref.so")
_median = None


def median_available() -> bool:
    return os.path.exists(MEDIAN_LIB_PATH)


def _load_median():
    global _median
    if _median is None:
        lib = ctypes.CDLL(MEDIAN_LIB_PATH)
        lib.ref_median_forward.restype = ctypes.c_int
        lib.ref_median_forward.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_int] * 4
        lib.ref_median_backward.restype = ctypes.c_int
        lib.ref_median_backward.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 4
        _median = lib
    return _median


def median_forward(vol):
    """vol: CUDA fp32 [1,H,W,K] -> [1,2,H,W] from the reference's kMedianScore."""
    import torch
    n, h, w, k = vol.shape
    out = torch.zeros((n, 2, h, w), device=vol.device)
    torch.cuda.synchronize()
    rc = _load_median().ref_median_forward(vol.data_ptr(), out.data_ptr(), n, h, w, k)
    if rc != 0:
        raise RuntimeError(f"reference median forward returned {rc}")
    return out


def median_backward(vol, grad):
    import torch
    n, h, w, k = vol.shape
    g = torch.zeros_like(vol)
    torch.cuda.synchronize()
    rc = _load_median().ref_median_backward(vol.data_ptr(), grad.data_ptr(), g.data_ptr(), n, h, w, k)
    if rc != 0:
        raise RuntimeError(f"reference median backward returned {rc}")
    return g


# ---- cudaQuadFit ------------------------------------------------------------------------------------------------
QUADFIT_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libquadfitref.so")
_quadfit = None


def quadfit_available() -> bool:
    return os.path.exists(QUADFIT_LIB_PATH)


def _load_quadfit():
    global _quadfit
    if _quadfit is None:
        lib = ctypes.CDLL(QUADFIT_LIB_PATH)
        lib.ref_quadfit_forward.restype = ctypes.c_int
        lib.ref_quadfit_forward.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4
        lib.ref_quadfit_backward.restype = ctypes.c_int
        lib.ref_quadfit_backward.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 4
        _quadfit = lib
    return _quadfit


def quadfit_forward(f0, f1, flow2):
    """CUDA fp32 tensors [N,C,H,W], flow2 [N,2,H,W] -> [N,3,H,W] from the reference's kQuadFitFlow."""
    import torch
    n, c, h, w = f0.shape
    out = torch.zeros((n, 3, h, w), device=f0.device)
    torch.cuda.synchronize()
    rc = _load_quadfit().ref_quadfit_forward(f0.data_ptr(), f1.data_ptr(), flow2.data_ptr(), out.data_ptr(), n, c, h, w)
    if rc != 0:
        raise RuntimeError(f"reference quadfit forward returned {rc}")
    return out


def quadfit_backward(f0, f1, flow2, grad):
    import torch
    n, c, h, w = f0.shape
    g0, g1 = torch.zeros_like(f0), torch.zeros_like(f1)
    torch.cuda.synchronize()
    rc = _load_quadfit().ref_quadfit_backward(f0.data_ptr(), f1.data_ptr(), flow2.data_ptr(), grad.data_ptr(),
                                              g0.data_ptr(), g1.data_ptr(), n, c, h, w)
    if rc != 0:
        raise RuntimeError(f"reference quadfit backward returned {rc}")
    return g0, g1


# ---- cudaTGV ----------------------------------------------------------------------------------------------------
TGV_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libtgvref.so")
_tgv = None


def tgv_available() -> bool:
    return os.path.exists(TGV_LIB_PATH)


def _load_tgv():
    global _tgv
    if _tgv is None:
        lib = ctypes.CDLL(TGV_LIB_PATH)
        lib.ref_tgv_forward.restype = ctypes.c_int
        lib.ref_tgv_forward.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 5
        lib.ref_tgv_backward.restype = ctypes.c_int
        lib.ref_tgv_backward.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_int] * 5
        _tgv = lib
    return _tgv


def tgv_forward(dx, dy, c, b, init, its, pid):
    """CUDA fp32: dx, dy [1,2,H,W]; c [1,1,H,W]; b [1,C,H,W]; init [1,3,C,H,W] -> solution [1,3,C,H,W]."""
    import torch
    assert b.shape[0] == 1
    _, ch, h, w = b.shape
    out = torch.zeros_like(init)
    torch.cuda.synchronize()
    rc = _load_tgv().ref_tgv_forward(dx.data_ptr(), dy.data_ptr(), c.data_ptr(), b.data_ptr(), init.data_ptr(),
                                     out.data_ptr(), ch, h, w, int(its), int(pid))
    if rc != 0:
        raise RuntimeError(f"reference TGV forward returned {rc}")
    return out


def tgv_backward(grad, dx, dy, c, b, its, pid):
    import torch
    assert b.shape[0] == 1
    _, ch, h, w = b.shape
    g = [torch.zeros_like(dx), torch.zeros_like(dy), torch.zeros_like(c), torch.zeros_like(b), torch.zeros_like(grad)]
    grad = grad.clone()
    torch.cuda.synchronize()
    rc = _load_tgv().ref_tgv_backward(dx.data_ptr(), dy.data_ptr(), c.data_ptr(), b.data_ptr(), grad.data_ptr(),
                                      g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), g[3].data_ptr(), g[4].data_ptr(),
                                      ch, h, w, int(its), int(pid))
    if rc != 0:
        raise RuntimeError(f"reference TGV backward returned {rc}")
    return g
