"""Builds libnmoe_b200.so (the C-ABI library) in-tree with nvcc for sm_100a."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnmoe_b200.so")
SOURCES = ["gemm.cu", "quant.cu", "router.cu", "router_fast.cu", "plan.cu", "ep.cu", "layer.cu",
           "route_noalloc.cu", "dense.cu"]
HEADERS = ["common.cuh", "kernels.h", os.path.join("..", "..", "include", "nmoe.h")]
NVCC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    deps = [os.path.join(CSRC, h) for h in HEADERS] + [__file__]
    objects = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        if force or _stale(obj, deps + [path]):
            cmd = [NVCC, *FLAGS, "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            subprocess.run(cmd, check=True)
        objects.append(obj)
    if force or _stale(LIB, objects):
        subprocess.run([NVCC, "-shared", "-o", LIB, *objects, "-gencode",
                        "arch=compute_100a,code=sm_100a"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
