"""Drop-in for the reference's Python layer `cudaTGV/TGVInpainting.py`: `TGVInpaintingFunction` and `TGVInpaint`
(H x W x 2 weight tensors [edge weight, beta], H x W x 1 confidence, H x W x C right-hand side, H x W x 3C initial
primary + auxiliary planes; returns H x W x 3C).  A leading batch dimension is accepted."""
from __future__ import annotations

from torch import nn
from torch.autograd import Function

from . import tgvInpaint_cuda_ext


class TGVInpaintingFunction(Function):
    """Mirrors TGVInpaintingFunction (cudaTGV/TGVInpainting.py:18-46)."""

    @staticmethod
    def forward(ctx, dx, dy, dc, db, di, its, pid):
        dx, dy, dc, db, di = (t.contiguous() for t in (dx, dy, dc, db, di))
        sol = tgvInpaint_cuda_ext.forward(dx, dy, dc, db, di, its, pid)[0]
        ctx.save_for_backward(dx, dy, dc, db)
        ctx.its, ctx.pid = int(its), int(pid)
        return sol

    @staticmethod
    def backward(ctx, grad_sol):
        dx, dy, dc, db = ctx.saved_tensors
        g = tgvInpaint_cuda_ext.backward(grad_sol.contiguous(), dx, dy, dc, db, ctx.its, ctx.pid)
        return g[0], g[1], g[2], g[3], g[4], None, None


class TGVInpaint(nn.Module):
    """Mirrors TGVInpaint (cudaTGV/TGVInpainting.py:49-74)."""

    def __init__(self, device, its, pid=3):
        super().__init__()
        self.its = its
        self.id = pid
        self.device = device

    def forward(self, t_dx, t_dy, t_dc, t_db, t_di):
        assert t_dx.shape[-1] == 2, "tensors should have 2 channels\n"
        assert t_di.shape[-1] == 3 * t_db.shape[-1], "input should have 3 planes per channel (primary and two auxilliary variables)\n"
        if t_dx.dim() == 4:
            f = lambda t: t.permute(0, 3, 1, 2)
            sol = TGVInpaintingFunction.apply(f(t_dx), f(t_dy), f(t_dc), f(t_db), f(t_di), self.its, self.id)
            return sol.permute(0, 2, 3, 1).contiguous()
        f = lambda t: t.permute(2, 0, 1).unsqueeze(0)
        sol = TGVInpaintingFunction.apply(f(t_dx), f(t_dy), f(t_dc), f(t_db), f(t_di), self.its, self.id)
        return sol.squeeze(0).permute(1, 2, 0).contiguous()

    def init(self):
        pass
