"""Drop-in for the reference's Python layer `cudaMedian/median.py`: `MedianFunction` and `Median` with the same
names and conventions (H x W x K volume in, H x W median position out); a leading batch dimension is accepted."""
from __future__ import annotations

from torch import nn
from torch.autograd import Function

from . import median_cuda_ext


class MedianFunction(Function):
    """Mirrors MedianFunction (cudaMedian/median.py:15-58): in_vol is N x H x W x K."""

    @staticmethod
    def forward(ctx, in_vol):
        in_vol = in_vol.contiguous()
        sol = median_cuda_ext.forward(in_vol)[0]
        ctx.save_for_backward(in_vol)
        return sol

    @staticmethod
    def backward(ctx, grad_sol):
        (in_vol,) = ctx.saved_tensors
        return median_cuda_ext.backward(grad_sol.contiguous(), in_vol)[0]


class Median(nn.Module):
    """Mirrors Median (cudaMedian/median.py:61-87): forward(t_vol [H,W,K]) -> [H,W] sub-bin median position."""

    def __init__(self, device):
        super().__init__()
        self.device = device

    def forward(self, t_vol):
        if t_vol.dim() == 4:
            return MedianFunction.apply(t_vol)[:, 0]
        sol = MedianFunction.apply(t_vol.unsqueeze(0))
        return sol.squeeze(0).permute(1, 2, 0)[:, :, 0]

    def init(self):
        pass
