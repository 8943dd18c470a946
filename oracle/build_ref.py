"""Recipe that compiles the reference's own cudaTV kernels (unmodified, from /root/reference) against the small
ImageUtilities stand-in in oracle/iu_shim into oracle/_ref/libtvref.so.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py

The output is git-ignored; it travels to the GPU box with the working tree.  Without /root/reference (e.g. on the
GPU box) nothing is built and the prebuilt file, if any, is used as is.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_SRC = "/root/reference/cudaTV/cudaCode"
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libtvref.so")


def build() -> str:
    if not os.path.isdir(REF_SRC):
        print("reference sources not present; keeping", OUT if os.path.exists(OUT) else "(nothing)")
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["/usr/local/cuda/bin/nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
           "--extended-lambda", "-Xcompiler", "-fPIC", "-shared", "--cudart", "shared", "-w",
           "-I", os.path.join(HERE, "iu_shim"), "-I", REF_SRC,
           os.path.join(HERE, "ref_tv_wrapper.cu"), "-o", OUT]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("building the reference's cudaTV kernels failed")
    print("built", OUT)
    return OUT


if __name__ == "__main__":
    build()
