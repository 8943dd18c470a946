"""Recipe that compiles the reference's own CUDA kernels (unmodified, from where the reference checkout lies:
environment variable CNL_REFERENCE_ROOT, else the default location below) against the small ImageUtilities stand-in in oracle/iu_shim into shared libraries under oracle/_ref/ (libtvref.so, libmedianref.so, ...).  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py

The output is git-ignored; it travels with the working tree to machines that have a GPU.  Where the reference
checkout is absent nothing is built and the prebuilt file, if any, is used as is.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.environ.get("CNL_REFERENCE_ROOT", "/root/reference")
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libtvref.so")
# output library -> (wrapper source, reference source directory)
TARGETS = {
    "libtvref.so": ("ref_tv_wrapper.cu", "cudaTV/cudaCode"),
    "libmedianref.so": ("ref_median_wrapper.cu", "cudaMedian/cudaCode"),
    "libquadfitref.so": ("ref_quadfit_wrapper.cu", "cudaQuadFit/cudaCode"),
    "libtgvref.so": ("ref_tgv_wrapper.cu", "cudaTGV/cudaCode"),
}


def build() -> str:
    if not os.path.isdir(REF_ROOT):
        print("reference sources not present; keeping what is in", OUT_DIR)
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    # -maxrregcount=128: the reference launches 512-thread blocks without __launch_bounds__; built for sm_100a its TGV
    # reverse kernels otherwise need more than 128 registers per thread and every launch fails (out of resources)
    for lib, (wrapper, src_dir) in TARGETS.items():
        wrapper_path = os.path.join(HERE, wrapper)
        if not os.path.exists(wrapper_path):
            continue
        out = os.path.join(OUT_DIR, lib)
        cmd = ["/usr/local/cuda/bin/nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
               "--extended-lambda", "-maxrregcount=128", "-Xcompiler", "-fPIC", "-shared", "--cudart", "shared", "-w",
               "-I", os.path.join(HERE, "iu_shim"), "-I", os.path.join(REF_ROOT, src_dir), wrapper_path, "-o", out]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"building {lib} from the reference's {src_dir} failed")
        print("built", out)
    return OUT


if __name__ == "__main__":
    build()
