"""CPU tests of the drop-in boundary: the C-ABI library loads without a GPU, exports every
symbol include/nmoe.h declares, and fails loudly (no CPU fallback) without a device."""
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "nmoe.h")).read()
    return sorted(set(re.findall(r"NMOE_API[^;(]*?\b(nmoe_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(package):
    lib = package.load_library()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(package.EXPORTED_SYMBOLS) == declared


def test_header_cites_reference_for_every_entry_point():
    text = open(os.path.join(ROOT, "include", "nmoe.h")).read()
    assert "expert_layer.h:84-105" in text and "nvfp4_packing.cpp:90-157" in text


def test_status_strings(package):
    lib = package.load_library()
    assert lib.nmoe_status_string(0) == b"ok"
    assert b"timed out" in lib.nmoe_status_string(4)


def test_swizzled_scale_bytes_matches_reference_layout(package, oracle):
    lib = package.load_library()
    for rows, cols in [(1, 16), (128, 64), (130, 112), (1856, 2688), (2688, 1856)]:
        assert lib.nmoe_swizzled_scale_bytes(rows, cols) == oracle.lib().nmo_swizzled_scale_bytes(rows, cols)
    assert lib.nmoe_swizzled_scale_bytes(1856, 2688) == 322560  # 1920 x 168
    assert lib.nmoe_swizzled_scale_bytes(4, 15) == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_no_cpu_fallback(package, synthetic):
    x = torch.zeros((2, 64))
    with pytest.raises(ValueError):
        package.quantize_nvfp4(x)
    cfg = synthetic.baseline_config(8, experts=32, hidden=64, routed=64, shared=64)
    with pytest.raises(RuntimeError):
        package.ExpertLayerSlice.create(cfg, None)


def test_invalid_arguments_are_rejected_without_a_device(package):
    lib = package.load_library()
    assert lib.nmoe_quantize_nvfp4(None, None, 0, 1, 16, 1, None, None, None, None) == 1
    assert lib.nmoe_layer_run(None, None, None, 0, 1, None, 0) == 1
    assert lib.nmoe_layer_create(None, None, None) == 1


def test_cpp_shim_compiles_against_the_reference_headers():
    """nemotron-inference_b200/shim/expert_layer_shim.cpp defines the members that the
    reference's expert_layer.h declares; it must compile against that very header."""
    import shutil
    import subprocess
    reference_root = os.environ.get("NMOE_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(ROOT), "reference")  # the checkout beside this repository
    reference_include = os.path.join(reference_root, "runtime", "include")
    if not os.path.isdir(reference_include) or shutil.which("g++") is None:
        pytest.skip("needs the reference checkout and g++")
    cuda_include = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    shim = os.path.join(ROOT, "nemotron-inference_b200", "shim", "expert_layer_shim.cpp")
    done = subprocess.run(["g++", "-std=c++20", "-fsyntax-only", "-Wall", "-I", reference_include,
                           "-I", os.path.join(ROOT, "include"), "-I", cuda_include, shim],
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
