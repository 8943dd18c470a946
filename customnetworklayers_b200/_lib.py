"""ctypes binding of libcnl_b200.so (the C ABI declared in include/cnl_b200.h).

There is no CPU fallback: if the library is missing or a call fails, a RuntimeError is raised."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_longlong, c_ulonglong, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcnl_b200.so")

# every exported symbol with (restype, argtypes); tests check this table against the header
SIGNATURES = {
    "cnl_tv_forward": (c_int, [c_void_p] * 6 + [c_int] * 6 + [c_void_p]),
    "cnl_tv_backward": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_void_p]),
    "cnl_tv_release": (c_int, [c_int]),
    "cnl_tv_read_history": (c_int, [c_int, c_int, c_void_p, c_void_p]),
    "cnl_tv_read_checkpoint": (c_int, [c_int, c_int, c_void_p, c_void_p]),
    "cnl_tv_num_checkpoints": (c_int, [c_int]),
    "cnl_tv_set_option": (c_int, [c_int, c_int, c_int]),
    "cnl_tv_get_timing": (c_int, [c_int, c_void_p]),
    "cnl_tv_run_count": (c_int, [c_int]),
    "cnl_tv_forward_count": (c_int, [c_int]),
    "cnl_peer_allreduce_bytes": (c_longlong, []),
    "cnl_peer_allreduce_sum": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_ulonglong, c_void_p]),
    "cnl_peer_allreduce_status": (c_int, []),
    "cnl_tv_lambda_grad_allreduce": (c_int, [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_ulonglong, c_void_p]),
    "cnl_launch_count": (c_ulonglong, []),
    "cnl_tv_lambda_grad": (c_int, [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p]),
    "cnl_dot_scratch_floats": (c_int, []),
    "cnl_tv_lambda_grad_static": (c_int, [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p]),
    "cnl_tv_lambda_grad_static_max_count": (c_longlong, []),
    "cnl_median_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "cnl_median_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "cnl_quadfit_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 4 + [c_void_p]),
    "cnl_quadfit_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 4 + [c_void_p]),
    "cnl_quadfit_cost_forward": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "cnl_quadfit_cost_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "cnl_tgv_forward": (c_int, [c_void_p] * 6 + [c_int] * 6 + [c_void_p]),
    "cnl_tgv_backward": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_void_p]),
    "cnl_tgv_release": (c_int, [c_int]),
    "cnl_tgv_set_option": (c_int, [c_int, c_int, c_int]),
    "cnl_tgv_read_state": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p]),
    "cnl_tgv_num_checkpoints": (c_int, [c_int]),
    "cnl_wmedian_forward": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_void_p]),
    "cnl_wmedian_backward": (c_int, [c_void_p] * 8 + [c_int] * 5 + [c_void_p]),
    "cnl_wmedian_scratch_bytes": (c_longlong, [c_int]),
    "cnl_last_error": (c_char_p, []),
    "cnl_version": (c_char_p, []),
}

OPT_CONDITIONER = 1
OPT_FUSE = 2
OPT_TIMING = 3
OPT_RECOMPUTE = 4
OPT_FLOW = 5

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library (building nothing: run `python -m customnetworklayers_b200.build` first)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m customnetworklayers_b200.build`. "
            "This package has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().cnl_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}: {last_error()}")
