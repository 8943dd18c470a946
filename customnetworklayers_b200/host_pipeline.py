"""Forward + backward of the TV layer for callers whose tensors live in (pinned) HOST memory.

Three CUDA streams work side by side: host->device copies, kernels, device->host copies.  Within one call the batch
is cut into chunks, so that the kernels of chunk k run while chunk k+1 arrives and the results of chunk k-1 leave.
Across calls nothing waits for the previous call to drain: the inputs land in one of `depth` (default 2) sets of
device buffers owned by the pipeline, so the copies of the next call run under the kernels of the current one and
the gradients of the current call leave under the kernels of the next.  A call returns as soon as its work is
enqueued; `HostPipeline.join()` makes the current stream wait for every result copy issued so far (a host-side
`torch.cuda.synchronize()` does as well), after which the pinned output tensors are valid.

One id slot is enough: forward(k) and backward(k) are consecutive on the compute stream."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from . import tvInpaint_cuda_ext as ext
from .dist import allreduce_scalar_grads

IN_KEYS = ("wx", "wy", "c", "b", "init", "grad")
OUT_KEYS = ("sol", "g_wx", "g_wy", "g_c", "g_b", "g_init")


class _BufferSet:
    """One set of device buffers for a call -- the six inputs, the scaled confidence, the solution and the five
    gradients -- plus the events after which its inputs may be refilled and its outputs overwritten.  Owning these
    keeps the caching allocator (and its cross-stream bookkeeping) out of the steady state entirely."""

    def __init__(self):
        self.buf: Dict[str, torch.Tensor] = {}
        self.inputs_free: Optional[torch.cuda.Event] = None      # kernels that read the inputs are done
        self.outputs_free: Optional[torch.cuda.Event] = None     # result copies to the host are done

    def fit(self, host_in: Dict[str, torch.Tensor], device) -> None:
        shapes = {k: host_in[k].shape for k in IN_KEYS}
        shapes.update({"c_scaled": shapes["c"], "sol": shapes["b"], "g_wx": shapes["wx"], "g_wy": shapes["wy"],
                       "g_c": shapes["c"], "g_b": shapes["b"], "g_init": shapes["b"]})
        for k, shp in shapes.items():
            if k not in self.buf or self.buf[k].shape != shp:
                self.buf[k] = torch.empty(shp, dtype=torch.float32, device=device)
        if "lam" not in self.buf:
            self.buf["lam"] = torch.empty(1, dtype=torch.float32, device=device)
            self.buf["lam_part"] = torch.empty(1, dtype=torch.float32, device=device)
            from . import _lib
            self.buf["scratch"] = torch.empty(_lib.load().cnl_dot_scratch_floats(), dtype=torch.float32, device=device)


class HostPipeline:
    """Streams and device-side input buffers for tv_fwd_bwd_from_host on one device."""

    def __init__(self, device, depth: int = 2):
        self.device = torch.device(device)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.sets: List[_BufferSet] = [_BufferSet() for _ in range(max(1, depth))]
        self.turn = 0
        self.last_out: Optional[torch.cuda.Event] = None
        self.timeline = None            # set to a list to collect per-chunk CUDA events (see chunk_breakdown)

    def join(self) -> None:
        """The current stream waits for every device->host copy issued so far."""
        if self.last_out is not None:
            torch.cuda.current_stream(self.device).wait_event(self.last_out)

    def chunk_breakdown(self):
        """After a synchronise: per recorded chunk, milliseconds from the start of the call to (inputs landed, forward
        done, backward done, gradients back in host memory).  Needs `timeline = []` before the calls."""
        rows = []
        for t0, ev in self.timeline or []:
            rows.append({k: t0.elapsed_time(e) for k, e in ev.items()})
        return rows


def _chunks(n: int, chunk) -> List[tuple]:
    """[lo, hi) ranges: `chunk` is a size or a sequence of sizes (the last size repeats until the batch is covered)."""
    sizes = [int(chunk)] if isinstance(chunk, int) else [int(c) for c in chunk]
    if not sizes or min(sizes) < 1:
        raise ValueError("chunk sizes must be >= 1")
    out, lo, i = [], 0, 0
    while lo < n:
        hi = min(n, lo + sizes[min(i, len(sizes) - 1)])
        out.append((lo, hi))
        lo, i = hi, i + 1
    return out


def tv_fwd_bwd_from_host(pipe: HostPipeline, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor],
                         its: int, pid: int, lam: Optional[torch.Tensor] = None, chunk=2,
                         host_lam_grad: Optional[torch.Tensor] = None):
    """Solves c = lam * host_in["c"] problems from pinned host tensors and writes the solution and the five
    gradients into pinned host tensors (host_out), plus the all-reduced lambda gradient into host_lam_grad.

    host_in : wx, wy, c [N,1,H,W]; b, init, grad [N,C,H,W]  (grad = upstream gradient of the solution)
    host_out: sol, g_b, g_init [N,C,H,W]; g_wx, g_wy, g_c [N,1,H,W]
    Returns the lambda gradient as a 1-element CUDA tensor (a buffer of the pipeline: valid until the call after next).
    Nothing here blocks the host; the pinned outputs are
    valid after pipe.join() followed by a synchronise of the current stream, or after torch.cuda.synchronize().
    host_in must not be rewritten before its copies have run (an event on pipe.s_in or a synchronise tells)."""
    dev = pipe.device
    comp = torch.cuda.current_stream(dev)
    n = host_in["b"].shape[0]
    slot = pipe.sets[pipe.turn]
    pipe.turn = (pipe.turn + 1) % len(pipe.sets)
    slot.fit(host_in, dev)
    ranges = _chunks(n, chunk)
    record = pipe.timeline is not None
    t0 = None
    if record:
        t0 = torch.cuda.Event(enable_timing=True)
        t0.record(comp)
        pipe.s_in.wait_event(t0)          # measured from a common origin; costs the overlap with the previous call
    if slot.inputs_free is not None:
        pipe.s_in.wait_event(slot.inputs_free)    # the kernels that read this set two calls ago are done
    ev_in, ev_grad = [], []
    with torch.cuda.stream(pipe.s_in):
        for lo, hi in ranges:
            # what the forward pass needs first; the upstream gradient follows behind it
            for k in IN_KEYS[:-1]:
                slot.buf[k][lo:hi].copy_(host_in[k][lo:hi], non_blocking=True)
            e = torch.cuda.Event(enable_timing=record)
            e.record(pipe.s_in)
            ev_in.append(e)
            slot.buf["grad"][lo:hi].copy_(host_in["grad"][lo:hi], non_blocking=True)
            e = torch.cuda.Event()
            e.record(pipe.s_in)
            ev_grad.append(e)
    if slot.outputs_free is not None:
        comp.wait_event(slot.outputs_free)        # the results this set held two calls ago have reached the host
    g_lam = slot.buf["lam"]
    g_lam.zero_()
    B = slot.buf
    for i, (lo, hi) in enumerate(ranges):
        d = {k: B[k][lo:hi] for k in IN_KEYS}
        comp.wait_event(ev_in[i])
        if lam is not None:
            c = torch.mul(d["c"], lam, out=B["c_scaled"][lo:hi])
        else:
            c = d["c"]
        sol = ext.forward(d["wx"], d["wy"], c, d["b"], d["init"], its, pid, out=B["sol"][lo:hi])[0]
        ev_f = torch.cuda.Event(enable_timing=record)
        ev_f.record(comp)
        pipe.s_out.wait_event(ev_f)
        with torch.cuda.stream(pipe.s_out):          # the solution goes back while the backward pass runs
            host_out["sol"][lo:hi].copy_(sol, non_blocking=True)
        comp.wait_event(ev_grad[i])
        grads = ext.backward(d["grad"], d["wx"], d["wy"], c, d["b"], its, pid,
                             out=[B[k][lo:hi] for k in OUT_KEYS[1:]])
        g_lam += ext.lambda_grad(grads[2], d["c"], out=B["lam_part"], scratch=B["scratch"])
        ev_b = torch.cuda.Event(enable_timing=record)
        ev_b.record(comp)
        pipe.s_out.wait_event(ev_b)
        with torch.cuda.stream(pipe.s_out):
            for key, t in zip(OUT_KEYS[1:], grads):
                host_out[key][lo:hi].copy_(t, non_blocking=True)
            ev_o = torch.cuda.Event(enable_timing=record)
            ev_o.record(pipe.s_out)
        pipe.last_out = ev_o
        if record:
            pipe.timeline.append((t0, {"inputs_landed": ev_in[i], "forward_done": ev_f, "backward_done": ev_b,
                                       "gradients_in_host_memory": ev_o}))
    slot.inputs_free = torch.cuda.Event()
    slot.inputs_free.record(comp)
    allreduce_scalar_grads(g_lam)
    # On the copy stream: a device->host copy issued on the compute stream would queue behind the gradient copies in the
    # copy engine and hold the next call's kernels back for as long as those take.
    ev_l = torch.cuda.Event()
    ev_l.record(comp)
    pipe.s_out.wait_event(ev_l)
    with torch.cuda.stream(pipe.s_out):
        if host_lam_grad is not None:
            host_lam_grad.copy_(g_lam, non_blocking=True)
        slot.outputs_free = torch.cuda.Event()
        slot.outputs_free.record(pipe.s_out)
    pipe.last_out = slot.outputs_free
    return g_lam
