"""Build recipe for the test oracle.  TEST INFRASTRUCTURE ONLY.

`build_port()` compiles oracle/nmoe_oracle.c (the CPU restatement) into
oracle/libnmoe_oracle.so.  `build_reference()` compiles the reference's own host
sources, from where they lie under the reference checkout, together with
oracle/ref_driver*.cpp into oracle/_ref/ref_driver; it is skipped when the
reference checkout is absent (the prebuilt binary travels with the tree).

Flags: -O2 -ffp-contract=off.  The reference's CMake sets neither an
optimisation level nor -march, so its x86-64 host build keeps FP32 multiplies
and adds separate; contraction to FMA would change the rounding of the
sequential K accumulation.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: NMOE_REFERENCE_ROOT, else a directory `reference` beside this
# repository; when neither exists the reference-built parts are skipped
REFERENCE_ROOT = os.environ.get("NMOE_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(HERE)), "reference")
CUDA_INCLUDE = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"
PORT_LIB = os.path.join(HERE, "libnmoe_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_BIN = os.path.join(REF_DIR, "ref_driver")
SHIM_BIN = os.path.join(REF_DIR, "shim_driver")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_port(force=False):
    src = os.path.join(HERE, "nmoe_oracle.c")
    if not force and _newer(PORT_LIB, [src]):
        return PORT_LIB
    cmd = ["gcc", "-std=c11", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
           "-fvisibility=hidden", "-Wall", "-o", PORT_LIB, src, "-lm"]
    subprocess.run(cmd, check=True)
    return PORT_LIB


def build_reference(force=False):
    """Returns the driver path, or None when it can be neither built nor found."""
    backend = os.path.join(REFERENCE_ROOT, "runtime", "src", "backend")
    if not os.path.isdir(backend):
        return REF_BIN if os.path.exists(REF_BIN) else None
    sources = [os.path.join(HERE, "ref_driver.cpp"), os.path.join(HERE, "ref_driver_linear.cpp"),
               os.path.join(backend, "nvfp4_packing.cpp"),
               os.path.join(backend, "nvfp4_scale_layout.cpp")]
    deps = sources + [os.path.join(backend, "expert_layer.cpp"), os.path.join(backend, "linear_op.cpp")]
    if not force and _newer(REF_BIN, deps):
        return REF_BIN
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-ffunction-sections",
           "-fdata-sections", "-I", REFERENCE_ROOT, "-I",
           os.path.join(REFERENCE_ROOT, "runtime", "include"), "-I", CUDA_INCLUDE,
           *sources, "-Wl,--gc-sections", "-o", REF_BIN]
    subprocess.run(cmd, check=True)
    return REF_BIN


def build_shim_driver(force=False):
    """The drop-in shim (nemotron-inference_b200/shim) linked with the reference's own
    device tensor and cuBLASLt handle classes and libnmoe_b200.so: proves that code written
    against the reference's headers runs on the new layer.  Returns the binary path, or
    None when it can be neither built nor found."""
    backend = os.path.join(REFERENCE_ROOT, "runtime", "src", "backend")
    package = os.path.join(os.path.dirname(HERE), "nemotron-inference_b200")
    library = os.path.join(package, "libnmoe_b200.so")
    if not os.path.isdir(backend) or not os.path.exists(library):
        return SHIM_BIN if os.path.exists(SHIM_BIN) else None
    sources = [os.path.join(HERE, "shim_driver.cpp"),
               os.path.join(package, "shim", "expert_layer_shim.cpp"),
               os.path.join(backend, "device_tensor.cpp"),
               os.path.join(backend, "cublaslt_handle.cpp")]
    if not force and _newer(SHIM_BIN, sources + [os.path.join(os.path.dirname(HERE), "include", "nmoe.h")]):
        return SHIM_BIN
    os.makedirs(REF_DIR, exist_ok=True)
    cuda_lib = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/lib64"
    cmd = ["g++", "-std=c++20", "-O2", "-I", os.path.join(REFERENCE_ROOT, "runtime", "include"),
           "-I", os.path.join(os.path.dirname(HERE), "include"), "-I", CUDA_INCLUDE, *sources,
           "-L", package, "-lnmoe_b200", "-L", cuda_lib, "-lcudart", "-lcublasLt",
           "-Wl,-rpath,$ORIGIN/../../nemotron-inference_b200", "-Wl,-rpath," + cuda_lib,
           "-o", SHIM_BIN]
    subprocess.run(cmd, check=True)
    return SHIM_BIN


if __name__ == "__main__":
    print(build_port(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
    print(build_shim_driver(force="--force" in sys.argv))
