"""GPU parity of one routed-expert NVFP4 FFN (configs[0]): y = W_down relu(W_up x)^2 with
dynamic per-16-block activation quantisation, against the reference's host FP32
dequantise-then-matmul path as restated by the oracle."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def _run_case(package, oracle, synthetic, rows, hidden, inter, variant, seed=0):
    up, down = synthetic.make_ffn_weights(hidden, inter, seed=seed, device="cuda")
    x = synthetic.make_tokens(rows, hidden, seed=seed + 100, device="cuda")
    ffn = package.ExpertFfn(up, down, max_rows=max(rows, 128))
    out = ffn.run(x, variant)
    gp, gs = ffn.hidden_codes(rows)
    ffn.close()
    x_np = x.to(torch.float32).cpu().numpy()
    # oracle through a layer-free composition: pack rows, dequantise, sequential FP32 matmul
    oup = oracle.Nvfp4Weight(up.packed.cpu().numpy(), up.block_scales.cpu().numpy(), up.tensor_scale)
    odn = oracle.Nvfp4Weight(down.packed.cpu().numpy(), down.block_scales.cpu().numpy(),
                             down.tensor_scale)
    hidden_ref, out_ref = oracle.expert_ffn(x_np, oup, odn)
    hp, hs, hts = oracle.pack_nvfp4_per_row(hidden_ref)
    code_mismatch = helpers.nibble_mismatches(gp.cpu().numpy(), hp)
    scale_mismatch = int(np.count_nonzero(gs.cpu().numpy() != hs))
    # second oracle pass on the device's own intermediate codes isolates the down projection
    h_dev = oracle.dequant_nvfp4(gp.cpu().numpy(), gs.cpu().numpy(), 1.0)
    out_forced = np.stack([oracle_row for oracle_row in _down_rows(oracle, h_dev, odn)])
    max_abs, cosine = helpers.max_abs_and_cosine(out.cpu().numpy(), out_ref)
    max_abs_forced, _ = helpers.max_abs_and_cosine(out.cpu().numpy(), out_forced)
    return dict(max_abs=max_abs, cosine=cosine, max_abs_forced=max_abs_forced,
                code_mismatch=code_mismatch, scale_mismatch=scale_mismatch,
                total_codes=int(hp.size * 2))


def _down_rows(oracle, h_deq, down):
    """Sequential FP32 dot products of already-dequantised rows with the dequantised weight."""
    w = oracle.dequant_nvfp4(down.packed, down.scales, down.tensor_scale)
    for row in h_deq:
        acc = np.zeros(w.shape[0], dtype=np.float32)
        for c in range(w.shape[1]):
            acc = (acc + row[c] * w[:, c]).astype(np.float32)
        yield acc


@pytest.mark.parametrize("rows,variant", [(64, 0), (64, 1), (64, 3), (20, 2), (130, 3), (300, 1), (300, 0)])
def test_single_expert_ffn_baseline_shape(package, oracle, synthetic, rows, variant):
    r = _run_case(package, oracle, synthetic, rows, 2688, 1856, variant)
    print(rows, variant, r)
    assert r["cosine"] >= helpers.COSINE_TOL
    assert r["max_abs_forced"] <= 1e-3          # down projection alone: accumulation-order noise
    assert r["code_mismatch"] <= max(2, r["total_codes"] // 20000)  # rounding ties only
    assert r["max_abs"] <= helpers.MAX_ABS_TOL or r["code_mismatch"] + r["scale_mismatch"] > 0


@pytest.mark.parametrize("hidden,inter", [(64, 64), (256, 128), (512, 1024)])
def test_single_expert_ffn_small_shapes(package, oracle, synthetic, hidden, inter):
    for rows, variant in [(3, 1), (3, 2), (40, 1), (40, 3)]:
        r = _run_case(package, oracle, synthetic, rows, hidden, inter, variant, seed=hidden)
        print(hidden, inter, rows, variant, r)
        assert r["cosine"] >= helpers.COSINE_TOL
        assert r["max_abs_forced"] <= 1e-3
