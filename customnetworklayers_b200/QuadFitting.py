"""Drop-in for the reference's Python layer `cudaQuadFit/QuadFitting.py`: `QuadFittingFromFlowFunction` and
`QuadFittingFromFlow` (H x W x C features, H x W x L flow with L >= 2; returns H x W x 3 = fx, fy, score), plus
`QuadFittingFromCost` for a given 5-point cost stencil."""
from __future__ import annotations

from torch import nn
from torch.autograd import Function

from . import QuadFit_cuda_ext


class QuadFittingFromFlowFunction(Function):
    """Mirrors QuadFittingFromFlowFunction (cudaQuadFit/QuadFitting.py:17-40); no gradient w.r.t. flow."""

    @staticmethod
    def forward(ctx, feat0, feat1, flow):
        feat0, feat1, flow = feat0.contiguous(), feat1.contiguous(), flow.contiguous()
        sol = QuadFit_cuda_ext.forward(feat0, feat1, flow)[0]
        ctx.save_for_backward(feat0, feat1, flow)
        return sol

    @staticmethod
    def backward(ctx, grad_sol):
        feat0, feat1, flow = ctx.saved_tensors
        g0, g1 = QuadFit_cuda_ext.backward(grad_sol.contiguous(), feat0, feat1, flow)
        return g0, g1, None


class QuadFittingFromFlow(nn.Module):
    """Mirrors QuadFittingFromFlow (cudaQuadFit/QuadFitting.py:43-64)."""

    def __init__(self, device):
        super().__init__()
        self.device = device

    def forward(self, t_feat0, t_feat1, t_flow):
        if t_feat0.dim() == 4:       # N x H x W x C extension
            nchw = lambda t: t.permute(0, 3, 1, 2)
            sol = QuadFittingFromFlowFunction.apply(nchw(t_feat0), nchw(t_feat1), nchw(t_flow))
            return sol.permute(0, 2, 3, 1).contiguous()
        assert t_flow.shape[-1] >= 2, "flow needs the displacement in X and Y direction\n"
        chw = lambda t: t.permute(2, 0, 1).unsqueeze(0)
        sol = QuadFittingFromFlowFunction.apply(chw(t_feat0), chw(t_feat1), chw(t_flow))
        return sol.squeeze(0).permute(1, 2, 0).contiguous()

    def init(self):
        pass


class QuadFittingFromCostFunction(Function):
    @staticmethod
    def forward(ctx, cost5):
        cost5 = cost5.contiguous()
        ctx.save_for_backward(cost5)
        return QuadFit_cuda_ext.cost_forward(cost5)

    @staticmethod
    def backward(ctx, grad):
        (cost5,) = ctx.saved_tensors
        return QuadFit_cuda_ext.cost_backward(grad.contiguous(), cost5)


class QuadFittingFromCost(nn.Module):
    """Sub-pixel refinement from a 5-point stencil cost5 [N,5,H,W] = (c00, c0+, c+0, c0-, c-0) of a score to maximise
    (negate a matching cost); returns [N,3,H,W] = (fx, fy, fitted score)."""

    def forward(self, cost5):
        return QuadFittingFromCostFunction.apply(cost5)
