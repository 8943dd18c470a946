"""Shared helpers of the parity tests: error norms and tolerances."""
import torch

# tolerance for fp32 forward and backward: 1e-4 relative, measured norm-wise per output tensor
REL_TOL = 1e-4


def rel_errors(a: torch.Tensor, ref: torch.Tensor):
    """(max|a-ref| / max|ref|, ||a-ref||_2 / ||ref||_2); both 0 when ref is identically zero and a too."""
    a = a.detach().double().cpu()
    ref = ref.detach().double().cpu()
    d = a - ref
    mx = float(ref.abs().max()) if ref.numel() else 0.0
    nr = float(ref.norm()) if ref.numel() else 0.0
    e_max = float(d.abs().max()) / mx if mx > 0 else float(d.abs().max()) if d.numel() else 0.0
    e_l2 = float(d.norm()) / nr if nr > 0 else float(d.norm())
    return e_max, e_l2


def assert_close(a, ref, name, tol=REL_TOL):
    e_max, e_l2 = rel_errors(a, ref)
    assert e_max <= tol and e_l2 <= tol, f"{name}: max-rel {e_max:.3e}, l2-rel {e_l2:.3e} exceed {tol:g}"
    return e_max, e_l2
