"""Forward + backward of the TV layer for callers whose tensors live in (pinned) HOST memory.

The batch is cut into chunks; the host->device copy of chunk k+1 and the device->host copy of chunk k-1 run on
their own CUDA streams while chunk k is being solved, so PCIe traffic in both directions overlaps the kernels.
One id slot is enough: forward(k) and backward(k) are consecutive on the compute stream."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import tvInpaint_cuda_ext as ext
from .dist import allreduce_scalar_grads

IN_KEYS = ("wx", "wy", "c", "b", "init", "grad")
OUT_KEYS = ("sol", "g_wx", "g_wy", "g_c", "g_b", "g_init")


class HostPipeline:
    """Reusable streams for tv_fwd_bwd_from_host on one device."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)


def tv_fwd_bwd_from_host(pipe: HostPipeline, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor],
                         its: int, pid: int, lam: Optional[torch.Tensor] = None, chunk: int = 2,
                         host_lam_grad: Optional[torch.Tensor] = None):
    """Solves c = lam * host_in["c"] problems from pinned host tensors and writes the solution and the five
    gradients into pinned host tensors (host_out), plus the all-reduced lambda gradient into host_lam_grad.

    host_in : wx, wy, c [N,1,H,W]; b, init, grad [N,C,H,W]  (grad = upstream gradient of the solution)
    host_out: sol, g_b, g_init [N,C,H,W]; g_wx, g_wy, g_c [N,1,H,W]
    Returns the lambda gradient as a 1-element CUDA tensor.  The caller synchronises (e.g. torch.cuda.synchronize())
    before reading host_out."""
    dev = pipe.device
    comp = torch.cuda.current_stream(dev)
    n = host_in["b"].shape[0]
    keep = []
    g_lam = torch.zeros(1, device=dev)
    start = torch.cuda.Event()
    start.record(comp)
    pipe.s_in.wait_event(start)           # do not run ahead of work already queued on the compute stream
    pipe.s_out.wait_event(start)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        with torch.cuda.stream(pipe.s_in):
            # what the forward pass needs first; the upstream gradient follows behind it
            d = {k: host_in[k][lo:hi].to(dev, non_blocking=True) for k in IN_KEYS if k != "grad"}
            ev_in = torch.cuda.Event()
            ev_in.record(pipe.s_in)
            d["grad"] = host_in["grad"][lo:hi].to(dev, non_blocking=True)
            ev_grad = torch.cuda.Event()
            ev_grad.record(pipe.s_in)
        comp.wait_event(ev_in)
        c = d["c"] * lam if lam is not None else d["c"]
        sol = ext.forward(d["wx"], d["wy"], c, d["b"], d["init"], its, pid)[0]
        ev_f = torch.cuda.Event()
        ev_f.record(comp)
        pipe.s_out.wait_event(ev_f)
        with torch.cuda.stream(pipe.s_out):          # the solution goes back while the backward pass runs
            host_out["sol"][lo:hi].copy_(sol, non_blocking=True)
        comp.wait_event(ev_grad)
        grads = ext.backward(d["grad"], d["wx"], d["wy"], c, d["b"], its, pid)
        g_lam += ext.lambda_grad(grads[2], d["c"])
        ev_c = torch.cuda.Event()
        ev_c.record(comp)
        pipe.s_out.wait_event(ev_c)
        with torch.cuda.stream(pipe.s_out):
            for key, t in zip(OUT_KEYS[1:], grads):
                host_out[key][lo:hi].copy_(t, non_blocking=True)
        keep.append((d, c, sol, grads))
    allreduce_scalar_grads(g_lam)
    done = torch.cuda.Event()
    done.record(pipe.s_out)
    comp.wait_event(done)                 # the compute stream now covers the copies too
    if host_lam_grad is not None:
        host_lam_grad.copy_(g_lam, non_blocking=True)
    pipe._keep = keep                     # keep device tensors alive until the next call / a synchronise
    return g_lam
