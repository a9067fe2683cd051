"""Build libffmoe.so (sm_100a only) in-tree with nvcc.

Usage: python -m flashfusedmoe_b200.build [--force]
The shared library lands next to this file so that it travels with the source tree.
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libffmoe.so")
PTXAS_LOG = os.path.join(HERE, "libffmoe.ptxas.txt")
SOURCES = ["ffm_api.cu", "ffm_route.cu", "ffm_rows.cu", "ffm_route_bwd.cu", "ffm_gemm_sm100.cu", "ffm_p2p.cu", "ffm_fp8.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]


def _newest_source_mtime():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    paths.append(os.path.join(HERE, "..", "include", "ffmoe.h"))
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ into libffmoe.so. Returns the library path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source_mtime():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc] + NVCC_FLAGS + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for src, p in procs:
        out, _ = p.communicate()
        log.append(out)
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    # ptxas -v output (registers, spills, shared memory per kernel), kept beside the library: the GLU-epilogue GEMM
    # is sensitive to register allocation (tests/test_cabi_cpu.py checks it)
    with open(PTXAS_LOG, "w") as f:
        f.write("".join(log))
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-lcudart"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
