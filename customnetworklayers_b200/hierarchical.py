"""Coarse-to-fine stack of TV-inpainting layers, one id slot per level, as sketched in the reference's README
(README.md:64-71: "multiple of these layers ... to build a hierarchical scheme"; the reference ships no code for it).

Per level l (coarse to fine):
    refined_l = offsets_l + QuadFittingFromCost(cost5_l)[:, :2]        sub-pixel refinement of integer matches
    init_l    = refined_0                      (coarsest level)
              = 2 * bilinear_upsample_x2(sol_{l-1})                     (flow values scale with the resolution)
    sol_l     = TVInpaint(wx_l, wy_l, lambda_l * c_l, b = refined_l, init = init_l, its, id = l)
Everything is differentiable through the layers' own backward passes; the learned scalars are lambda_l."""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.nn.functional as F
from torch import nn

from .QuadFitting import QuadFittingFromCostFunction
from .TVInpainting import TVInpaintingFunction
from .dist import allreduce_scalar_grads


class HierarchicalTV(nn.Module):
    def __init__(self, levels: int = 3, its: int = 50, first_id: int = 0):
        super().__init__()
        if levels < 1 or not (0 <= first_id and first_id + levels <= 10):
            raise ValueError("levels need distinct ids within 0..9")
        self.levels, self.its, self.first_id = levels, its, first_id
        self.lam = nn.Parameter(torch.ones(levels))

    def forward(self, inputs: List[Dict[str, torch.Tensor]]) -> List[torch.Tensor]:
        """inputs[l] (coarse to fine): wx, wy, c [N,1,H_l,W_l]; offsets [N,2,H_l,W_l]; cost5 [N,5,H_l,W_l].
        Returns the solutions of all levels (the last one is the full-resolution flow)."""
        sols = []
        prev = None
        for l, I in enumerate(inputs):
            refined = I["offsets"] + QuadFittingFromCostFunction.apply(I["cost5"])[:, :2]
            if prev is None:
                init = refined
            else:
                init = 2.0 * F.interpolate(prev, size=refined.shape[-2:], mode="bilinear", align_corners=False)
            sol = TVInpaintingFunction.apply(I["wx"], I["wy"], self.lam[l] * I["c"], refined.contiguous(),
                                             init.contiguous(), self.its, self.first_id + l)
            sols.append(sol)
            prev = sol
        return sols

    def allreduce_parameter_grads(self) -> None:
        """Data-parallel step: sum the gradients of the learned scalars over all ranks (the only collective)."""
        if self.lam.grad is not None:
            allreduce_scalar_grads(self.lam.grad)
