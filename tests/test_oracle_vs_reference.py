"""CPU tests that execute the REFERENCE's own host code (oracle/_ref/ref_driver, built from
the reference sources) beside the oracle on fresh random inputs.  Skipped where the driver
was not built (no reference checkout)."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def ref(oracle):
    if not oracle.have_reference():
        pytest.skip("oracle/_ref/ref_driver is not built")
    return oracle


def _ref_pack(oracle, x):
    rows, cols = x.shape
    raw = oracle.ref_run("pack", [rows, cols, "0", "x", "out"], {"x": x}, {"out": np.uint8})["out"]
    return (raw[4:4 + rows * cols // 2].reshape(rows, cols // 2),
            raw[4 + rows * cols // 2:].reshape(rows, cols // 16), raw[:4].view(np.float32)[0])


def test_encoders_dense_sweep(ref):
    # every float whose low 12 mantissa bits are zero, both signs, finite
    bits = (np.arange(0, 1 << 20, dtype=np.uint32) << 12)
    values = bits.view(np.float32)
    values = values[np.isfinite(values)]
    fp4 = ref.ref_run("encode_fp4", ["x", "out"], {"x": values}, {"out": np.uint8})["out"]
    fp8 = ref.ref_run("encode_fp8", ["x", "out"], {"x": values}, {"out": np.uint8})["out"]
    step = 37  # the per-value ctypes call is slow; a stride still covers every binade densely
    assert np.array_equal(ref.encode_e2m1(values[::step]), fp4[::step])
    assert np.array_equal(ref.encode_e4m3(values[::step]), fp8[::step])


@pytest.mark.parametrize("seed,rows,cols,scale", [(0, 3, 2688, 1.0), (1, 2, 1856, 30.0),
                                                  (2, 1, 3712, 4000.0), (3, 5, 64, 1e-4)])
def test_packer_random(ref, seed, rows, cols, scale):
    rng = np.random.default_rng(seed)
    x = (rng.normal(0, 1, (rows, cols)) * scale).astype(np.float32)
    x[0, :16] = 0
    p, s, ts = ref.pack_nvfp4(x)
    rp, rs, rts = _ref_pack(ref, x)
    assert np.array_equal(p, rp) and np.array_equal(s, rs) and np.float32(ts) == rts
    deq = ref.ref_run("dequant", [rows, cols, "p", "s", repr(float(ts)), "out"], {"p": p, "s": s},
                      {"out": np.float32})["out"].reshape(rows, cols)
    assert np.array_equal(ref.dequant_nvfp4(p, s, ts), deq)


def test_topk_random(ref):
    rng = np.random.default_rng(7)
    T, E, k = 200, 128, 6
    logits = rng.normal(0, 1.04, (T, E)).astype(np.float32)
    bias = rng.uniform(-0.01, 0.01, E).astype(np.float32)
    raw = ref.ref_run("topk", [T, E, k, 1, 1, 1, "2.5", "l", "b", "out"], {"l": logits, "b": bias},
                      {"out": np.uint8})["out"].reshape(T, 2, k, 4)
    idx, w = ref.select_top_experts(logits, bias, k, 1, 1, True, 2.5)
    assert np.array_equal(idx, raw[:, 0].copy().view(np.int32).reshape(T, k))
    assert np.array_equal(w, raw[:, 1].copy().view(np.float32).reshape(T, k))


def test_linear_row_random(ref):
    rng = np.random.default_rng(9)
    N, K, rows = 80, 256, 3
    wp, ws, wts = ref.quantize_weight(rng.normal(0, 0.02, (N, K)).astype(np.float32))
    x = rng.normal(0, 1, (rows, K)).astype(np.float32)
    out = ref.ref_run("linear", [rows, N, K, "x", "p", "s", repr(wts), "out"],
                      {"x": x, "p": wp, "s": ws}, {"out": np.float32})["out"].reshape(rows, N)
    assert np.array_equal(ref.nvfp4_linear_literal(x, wp, ws, wts), out)


def test_golden_vectors_are_current(ref, tmp_path):
    """The committed fixture equals what the generator produces from the reference now."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    committed = np.load(os.path.join(here, "golden", "reference_vectors.npz"))
    tables = ref.ref_run("decode_tables", ["out"], {}, {"out": np.float32})["out"]
    assert np.array_equal(tables[:16], committed["decode_e2m1"])
    codes = ref.ref_run("encode_fp8", ["x", "out"], {"x": committed["e4m3_probe"]},
                        {"out": np.uint8})["out"]
    assert np.array_equal(codes, committed["e4m3_codes"])
