"""Build step: compiles the CUDA sources under csrc/ into lib/librg_b200.so for
sm_100a with nvcc.  Run as `python -m rustygradients_b200.build` (add -v to see
ptxas resource usage)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "librg_b200.so")
SOURCES = ["rg_api.cu", "rg_gpt.cu", "rg_mega.cu", "rg_cloop.cu", "rg_gemm_tc.cu", "rg_attn_tc.cu", "rg_noalloc.cu", "rg_ingest.cu",
           "rg_tokenizer.cu"]


def _newest_source_mtime() -> float:
    latest = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for name in os.listdir(root):
            latest = max(latest, os.path.getmtime(os.path.join(root, name)))
    return latest


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile if the library is missing or older than any source; returns its path."""
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_source_mtime():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--use_fast_math" if False else "-DRG_NO_FAST_MATH",
           "-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
