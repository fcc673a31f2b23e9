"""Generates tests/golden/reference_vectors.npz by running the REFERENCE's own host
functions (oracle/_ref/ref_driver, compiled from the reference sources) on small
seeded inputs.  Run it where the reference checkout is present:

    python tests/golden/make_golden.py

The vectors pin the CPU oracle (and through it the CUDA path) where the reference
checkout is absent.  Inputs follow the reference's own unit tests where it has
some (testing/backend/nvfp4_packing_test.cpp:31-106,
testing/backend/device_nvfp4_matrix_test.cpp:26-248).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

oracle = entry.load_oracle()


def ref_pack(x, fixed=0.0):
    rows, cols = x.shape
    raw = oracle.ref_run("pack", [rows, cols, repr(float(fixed)), "x", "out"],
                         {"x": x.astype(np.float32)}, {"out": np.uint8})["out"]
    if raw.size == 0:
        return None
    ts = raw[:4].view(np.float32)[0]
    packed = raw[4:4 + rows * cols // 2].reshape(rows, cols // 2)
    scales = raw[4 + rows * cols // 2:].reshape(rows, cols // 16)
    return packed, scales, ts


def main():
    rng = np.random.default_rng(20240611)
    out = {}
    tables = oracle.ref_run("decode_tables", ["out"], {}, {"out": np.float32})["out"]
    out["decode_e2m1"], out["decode_e4m3"] = tables[:16], tables[16:]

    # encoders: every boundary, its float neighbours, and random values
    e2m1_edges = np.array([0, 0.25, 0.5, 0.75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 7, 100],
                          dtype=np.float32)
    probes = np.concatenate([e2m1_edges, np.nextafter(e2m1_edges, np.float32(np.inf)),
                             np.nextafter(e2m1_edges, np.float32(-np.inf)),
                             rng.uniform(-7, 7, 2000).astype(np.float32)])
    probes = np.concatenate([probes, -probes]).astype(np.float32)
    out["e2m1_probe"] = probes
    out["e2m1_codes"] = oracle.ref_run("encode_fp4", ["x", "out"], {"x": probes}, {"out": np.uint8})["out"]
    e4m3_values = oracle.decode_e4m3_table()[:127].astype(np.float32)
    mids = ((e4m3_values[:-1].astype(np.float64) + e4m3_values[1:]) / 2).astype(np.float32)
    probes8 = np.concatenate([e4m3_values, mids, np.nextafter(mids, np.float32(np.inf)),
                              np.nextafter(mids, np.float32(-np.inf)),
                              np.array([448, 460, 464, 470, 480, 1e4, 1e-5, 2 ** -10, 2 ** -9], np.float32),
                              np.exp(rng.uniform(np.log(1e-4), np.log(600), 3000)).astype(np.float32)])
    out["e4m3_probe"] = probes8
    out["e4m3_codes"] = oracle.ref_run("encode_fp8", ["x", "out"], {"x": probes8}, {"out": np.uint8})["out"]

    sig = np.concatenate([np.linspace(-12, 12, 481), rng.normal(0, 2, 500)]).astype(np.float32)
    out["sigmoid_in"] = sig
    out["sigmoid_out"] = oracle.ref_run("sigmoid", ["x", "out"], {"x": sig}, {"out": np.float32})["out"]

    # packer cases
    cases = {
        "ramp9": (np.arange(32) % 9 - 4).astype(np.float32).reshape(2, 16) * 0.5,
        "ramp11": (np.arange(32) % 11 - 5).astype(np.float32).reshape(2, 16) * 0.25,
        "big": np.full((1, 16), 4096.0, np.float32),
        "zeros": np.zeros((2, 32), np.float32),
        "tiny": np.full((1, 16), 1e-5, np.float32),
        "normal": rng.normal(0, 1, (4, 64)).astype(np.float32),
        "relu2": np.square(np.maximum(rng.normal(0, 1.1, (3, 96)), 0)).astype(np.float32),
        "mixed_big": np.concatenate([rng.normal(0, 1, (1, 32)), rng.normal(0, 3000, (1, 32))]).astype(np.float32),
    }
    for name, x in cases.items():
        p, s, ts = ref_pack(x)
        out[f"pack_{name}_x"], out[f"pack_{name}_p"], out[f"pack_{name}_s"] = x, p, s
        out[f"pack_{name}_ts"] = np.float32(ts)
    x = cases["normal"]
    p, s, ts = ref_pack(x, fixed=0.002197265625)
    out["pack_fixed_p"], out["pack_fixed_s"], out["pack_fixed_ts"] = p, s, np.float32(ts)

    # swizzle: 16x64 as in the reference test plus a ragged multi-tile case
    for name, (rows, cols) in {"a": (16, 64), "b": (130, 112)}.items():
        sc = rng.integers(0, 127, (rows, cols // 16), dtype=np.uint8)
        out[f"swz_{name}_in"] = sc
        out[f"swz_{name}_out"] = oracle.ref_run("swizzle", [rows, cols, "x", "out"], {"x": sc},
                                                {"out": np.uint8})["out"]
        out[f"swz_{name}_cols"] = np.int32(cols)

    # top-k
    for name, (T, E, k, ng, tg) in {"e128": (24, 128, 6, 1, 1), "grouped": (12, 64, 4, 8, 3)}.items():
        logits = rng.normal(0, 1.0, (T, E)).astype(np.float32)
        bias = rng.uniform(-0.01, 0.01, E).astype(np.float32)
        raw = oracle.ref_run("topk", [T, E, k, ng, tg, 1, "2.5", "l", "b", "out"],
                             {"l": logits, "b": bias}, {"out": np.uint8})["out"]
        rec = raw.reshape(T, 2, k, 4)
        out[f"topk_{name}_logits"], out[f"topk_{name}_bias"] = logits, bias
        out[f"topk_{name}_idx"] = rec[:, 0].copy().view(np.int32).reshape(T, k)
        out[f"topk_{name}_w"] = rec[:, 1].copy().view(np.float32).reshape(T, k)
        out[f"topk_{name}_cfg"] = np.array([k, ng, tg], np.int32)

    # one expert FFN on a small shape (weights from the harness quantiser)
    H, I, rows = 128, 96, 5
    up = oracle.quantize_weight(rng.normal(0, 0.02, (I, H)).astype(np.float32))
    down = oracle.quantize_weight(rng.normal(0, 0.02, (H, I)).astype(np.float32))
    xs = rng.normal(0, 1, (rows, H)).astype(np.float32)
    res = oracle.ref_run("expert", [rows, H, I, "x", "up", "us", repr(up[2]), "dp", "ds", repr(down[2]),
                                    "hid", "out"],
                         {"x": xs, "up": up[0], "us": up[1], "dp": down[0], "ds": down[1]},
                         {"hid": np.float32, "out": np.float32})
    out["ffn_x"], out["ffn_hidden"], out["ffn_out"] = xs, res["hid"].reshape(rows, I), res["out"].reshape(rows, H)
    out["ffn_up_p"], out["ffn_up_s"], out["ffn_up_ts"] = up[0], up[1], np.float32(up[2])
    out["ffn_down_p"], out["ffn_down_s"], out["ffn_down_ts"] = down[0], down[1], np.float32(down[2])

    # double-accumulate dense matmul (router gate)
    a = rng.normal(0, 1, (3, 200)).astype(np.float32)
    w = rng.normal(0, 0.02, (8, 200)).astype(np.float32)
    out["dense_a"], out["dense_w"] = a, w
    out["dense_out"] = oracle.ref_run("dense", [3, 8, 200, "a", "w", "out"], {"a": a, "w": w},
                                      {"out": np.float32})["out"].reshape(3, 8)
    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
