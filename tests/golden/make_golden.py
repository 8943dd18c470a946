"""Generates tests/golden/tv_reference_cuda.npz: inputs and outputs of the REFERENCE's own cudaTV kernels
(oracle/_ref/libtvref.so, built unmodified by oracle/build_ref.py) on a few small problems.  Needs a GPU:

    python tests/golden/make_golden.py <out_dir> [tv] [median] ...           # on a machine with a GPU
    cp <out_dir>/*_reference_cuda.npz tests/golden/                          # back in the working tree

The committed file pins the CPU oracle (tests/test_golden.py, no GPU needed) and the CUDA path."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

CASES = [  # channels, height, width, its, seed
    (2, 16, 32, 4, 101),
    (1, 32, 32, 7, 102),
    (2, 32, 64, 10, 103),
    (3, 16, 64, 20, 104),
]


def main(out_path):
    from customnetworklayers_b200.synthetic import make_inputs
    from oracle import ref_cuda
    data = {"n_cases": np.array(len(CASES))}
    for i, (ch, h, w, its, seed) in enumerate(CASES):
        I = make_inputs(1, ch, h, w, seed=seed)
        I["init"] = I["b"] + 0.25 * I["grad"].flip(-1)          # an init that differs from b
        D = {k: v.cuda() for k, v in I.items()}
        sol = ref_cuda.forward(D["wx"], D["wy"], D["c"], D["b"], D["init"], its, i % 10)
        grads = ref_cuda.backward(D["grad"], D["wx"], D["wy"], D["c"], D["b"], its, i % 10)
        data[f"case{i}_its"] = np.array(its)
        for k, v in I.items():
            data[f"case{i}_{k}"] = v.numpy()
        data[f"case{i}_sol"] = sol.cpu().numpy()
        for name, g in zip(("g_wx", "g_wy", "g_c", "g_b", "g_init"), grads):
            data[f"case{i}_{name}"] = g.cpu().numpy()
    np.savez_compressed(out_path, **data)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")




def median_main(out_path):
    """tests/golden/median_reference_cuda.npz: the reference's own cudaMedian kernels (oracle/_ref/libmedianref.so)."""
    from customnetworklayers_b200.synthetic import make_median_volume
    from oracle import ref_cuda
    cases = [(12, 16, 49, 201), (9, 7, 9, 202), (5, 6, 121, 203)]
    data = {"n_cases": np.array(len(cases))}
    for i, (h, w, k, seed) in enumerate(cases):
        vol, grad = make_median_volume(1, h, w, k, seed=seed)
        vol[0, 0, 0] = 0.1 / k                      # one pixel without a crossing
        v, g = vol.cuda(), grad.cuda()
        data[f"case{i}_vol"] = vol.numpy()
        data[f"case{i}_grad"] = grad.numpy()
        data[f"case{i}_out"] = ref_cuda.median_forward(v).cpu().numpy()
        data[f"case{i}_gvol"] = ref_cuda.median_backward(v, g).cpu().numpy()
    np.savez_compressed(out_path, **data)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


def quadfit_main(out_path):
    """tests/golden/quadfit_reference_cuda.npz: the reference's own cudaQuadFit kernels (oracle/_ref/libquadfitref.so)."""
    from customnetworklayers_b200.synthetic import make_quadfit_inputs
    from oracle import ref_cuda
    cases = [(1, 4, 12, 16, 301), (2, 7, 9, 11, 302), (1, 16, 20, 24, 303)]
    data = {"n_cases": np.array(len(cases))}
    for i, (n, c, h, w, seed) in enumerate(cases):
        f0, f1, flow, grad = make_quadfit_inputs(n, c, h, w, seed=seed)
        D = [t.cuda() for t in (f0, f1, flow, grad)]
        out = ref_cuda.quadfit_forward(D[0], D[1], D[2])
        g0, g1 = ref_cuda.quadfit_backward(D[0], D[1], D[2], D[3])
        for k, v in (("feat0", f0), ("feat1", f1), ("flow", flow), ("grad", grad), ("out", out), ("g0", g0), ("g1", g1)):
            data[f"case{i}_{k}"] = v.cpu().numpy()
    np.savez_compressed(out_path, **data)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


def tgv_main(out_path):
    """tests/golden/tgv_reference_cuda.npz: the reference's own cudaTGV kernels (oracle/_ref/libtgvref.so); one
    channel runs its generic kernels, two channels its two-channel kernels."""
    from customnetworklayers_b200.synthetic import make_tgv_inputs
    from oracle import ref_cuda
    cases = [(1, 16, 32, 4, 401), (2, 16, 32, 6, 402), (1, 32, 32, 10, 403), (2, 32, 64, 20, 404), (3, 16, 32, 8, 405)]
    data = {"n_cases": np.array(len(cases))}
    for i, (ch, h, w, its, seed) in enumerate(cases):
        I = make_tgv_inputs(1, ch, h, w, seed=seed)
        I["init"][:, 1:] = 0.1 * torch.randn(I["init"][:, 1:].shape, generator=torch.Generator().manual_seed(seed))
        D = {k: v.cuda() for k, v in I.items()}
        sol = ref_cuda.tgv_forward(D["dx"], D["dy"], D["c"], D["b"], D["init"], its, i % 10)
        grads = ref_cuda.tgv_backward(D["grad"], D["dx"], D["dy"], D["c"], D["b"], its, i % 10)
        data[f"case{i}_its"] = np.array(its)
        for k, v in I.items():
            data[f"case{i}_{k}"] = v.numpy()
        data[f"case{i}_sol"] = sol.cpu().numpy()
        for name, g in zip(("g_dx", "g_dy", "g_c", "g_b", "g_init"), grads):
            data[f"case{i}_{name}"] = g.cpu().numpy()
    np.savez_compressed(out_path, **data)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    which = sys.argv[2:] or ["tv", "median", "quadfit", "tgv"]
    if "tv" in which:
        main(os.path.join(out_dir, "tv_reference_cuda.npz"))
    if "median" in which:
        median_main(os.path.join(out_dir, "median_reference_cuda.npz"))
    if "tgv" in which:
        tgv_main(os.path.join(out_dir, "tgv_reference_cuda.npz"))
    if "quadfit" in which:
        quadfit_main(os.path.join(out_dir, "quadfit_reference_cuda.npz"))
