"""TEST INFRASTRUCTURE: builds oracle/_ref/libref_kernels.so = the reference's own CUDA kernels
(src/backend/cuda_kernels.cu, compiled for sm_100a from where the file lies in the reference tree) + the host launchers of
oracle/ref_kernels_launch.cu.  Nothing of the reference is copied: the launcher file includes it through an -I path.
Only the reference's one .cu file is compiled (no build system of the reference is run).  The output is git-ignored and
travels to GPU machines as a built file; where the reference tree is absent this script does nothing.

    python oracle/build_ref.py [reference root]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "libref_kernels.so")


def build(reference_root: str) -> str:
    """Returns the library path, or "" when the reference tree (or its kernel file) is not there."""
    src_dir = os.path.join(reference_root, "src", "backend")
    if not os.path.exists(os.path.join(src_dir, "cuda_kernels.cu")):
        return ""
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = [os.environ.get("NVCC", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-shared",
           "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", src_dir, "-o", OUT, os.path.join(HERE, "ref_kernels_launch.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return OUT


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("RG_REFERENCE_ROOT", "")
    print(build(root) or "reference tree not found: nothing built")
