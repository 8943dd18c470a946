"""Coarse-to-fine stack (three TV layers on ids 0..2 with a quadratic-fit refinement before each level).  The
reference has no code for the stack, so its composition is unpinned; what is checked is that the stack equals the
same composition of the CPU oracles, forward and (for the parameters of the finest level) backward."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from customnetworklayers_b200.synthetic import make_hierarchy_inputs
from oracle import quadfit_ref as Q
from oracle import tv_ref as R
from tests.parity import assert_close

pytestmark = pytest.mark.gpu


def test_stack_matches_oracle_composition():
    from customnetworklayers_b200 import tvInpaint_cuda_ext as tvext
    from customnetworklayers_b200.hierarchical import HierarchicalTV
    n, h, w, its = 2, 64, 96, 10
    levels, grad = make_hierarchy_inputs(n, h, w, seed=3)
    for pid in range(3):
        tvext.release(pid)
        tvext.set_option(pid, 1, 0)
    model = HierarchicalTV(levels=3, its=its).cuda()
    with torch.no_grad():
        model.lam.copy_(torch.tensor([0.8, 1.0, 1.3]))
    dev = [{k: v.cuda().requires_grad_(k == "cost5") for k, v in I.items()} for I in levels]
    sols = model(dev)
    assert [tuple(s.shape) for s in sols] == [(n, 2, 16, 24), (n, 2, 32, 48), (n, 2, 64, 96)]
    sols[-1].backward(grad.cuda())
    model.allreduce_parameter_grads()          # no process group: a no-op
    assert model.lam.grad is not None and torch.isfinite(model.lam.grad).all() and float(model.lam.grad.abs().sum()) > 0
    assert all(torch.isfinite(d["cost5"].grad).all() and float(d["cost5"].grad.abs().sum()) > 0 for d in dev)
    # oracle composition, forward
    prev = None
    lam = [0.8, 1.0, 1.3]
    for l, I in enumerate(levels):
        refined = I["offsets"].double() + torch.from_numpy(Q.quadfit_from_cost_forward(I["cost5"].numpy()))[:, :2].double()
        init = refined if prev is None else 2.0 * F.interpolate(prev, size=refined.shape[-2:], mode="bilinear", align_corners=False)
        sol, hist, cky = R.tv_forward_history(I["wx"], I["wy"], lam[l] * I["c"].double(), refined, init, its)
        assert_close(sols[l], sol, f"level {l} solution", tol=2e-4)
        prev = sol
    # finest level, backward: lambda gradient = sum g_c * c_raw with the oracle's reverse sweep on the device's history
    hist_d, cky_d = tvext.read_history(2, sols[-1], its)
    I = levels[-1]
    g = R.tv_backward_raw(I["wx"], I["wy"], lam[2] * I["c"].double(), refined, grad, its, None, hist=hist_d.cpu(), ckpt_y=cky_d.cpu())
    ref_lam2 = float((g[2] * I["c"].double()).sum())
    assert abs(float(model.lam.grad[2]) - ref_lam2) <= 2e-4 * max(1.0, abs(ref_lam2))
