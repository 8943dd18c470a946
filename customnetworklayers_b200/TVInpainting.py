"""Drop-in for the reference's Python layer `cudaTV/TVInpainting.py`: same class names, argument order, HWC
convention and per-instance `id` slots 0..9.  A leading batch dimension is accepted as an extension."""
from __future__ import annotations

import torch
from torch import nn
from torch.autograd import Function

from . import tvInpaint_cuda_ext


class TVInpaintingFunction(Function):
    """Mirrors TVInpaintingFunction (cudaTV/TVInpainting.py:11-29).  Inputs are N x C x H x W; `its` and `pid`
    are plain ints kept on the context (the reference round-trips them through a CPU tensor, :18, :27)."""

    @staticmethod
    def forward(ctx, dx, dy, dc, db, di, its, pid):
        dx, dy, dc, db, di = (t.contiguous() for t in (dx, dy, dc, db, di))
        sol = tvInpaint_cuda_ext.forward(dx, dy, dc, db, di, its, pid)[0]
        ctx.save_for_backward(dx, dy, dc, db)
        ctx.its = int(its)
        ctx.pid = int(pid)
        ctx.generation = tvInpaint_cuda_ext.forward_count(pid, db.device)
        return sol

    @staticmethod
    def backward(ctx, grad_sol):
        dx, dy, dc, db = ctx.saved_tensors
        d_oGx, d_oGy, d_oGc, d_oGb, d_oGi = tvInpaint_cuda_ext.backward(grad_sol.contiguous(), dx, dy, dc, db,
                                                                       ctx.its, ctx.pid, generation=ctx.generation)
        return d_oGx, d_oGy, d_oGc, d_oGb, d_oGi, None, None


class TVInpaint(nn.Module):
    """Mirrors TVInpaint (cudaTV/TVInpainting.py:32-55).

    forward(t_dx, t_dy, t_dc, t_db, t_di): edge weights in x and y, confidence (each H x W x 1), right-hand side
    and initial solution (each H x W x C); returns the H x W x C solution.  With a leading batch dimension
    (N x H x W x *) the N problems are solved in one call and an N x H x W x C tensor is returned."""

    def __init__(self, device, its, pid=6):
        super().__init__()
        self.its = its
        self.id = pid
        self.device = device

    def forward(self, t_dx, t_dy, t_dc, t_db, t_di):
        batched = t_dx.dim() == 4
        assert t_dx.shape[-1] == 1, "diffusion tensors should have 1 channel\n"
        if batched:
            to_nchw = lambda t: t.permute(0, 3, 1, 2)
        else:
            to_nchw = lambda t: t.permute(2, 0, 1).unsqueeze(0)          # order is 1,Channel,Height,Width
        sol = TVInpaintingFunction.apply(to_nchw(t_dx), to_nchw(t_dy), to_nchw(t_dc), to_nchw(t_db), to_nchw(t_di),
                                         self.its, self.id)
        if batched:
            return sol.permute(0, 2, 3, 1).contiguous()
        return sol.squeeze(0).permute(1, 2, 0).contiguous()

    def init(self):
        pass
