"""CPU tests: the oracle (oracle/nmoe_oracle.c) against the committed golden vectors
that the reference's own host functions produced, and its internal consistency."""
import os

import numpy as np
import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def test_decode_tables_match_reference(oracle, golden):
    assert np.array_equal(oracle.decode_e2m1_table(), golden["decode_e2m1"])
    ours, ref = oracle.decode_e4m3_table(), golden["decode_e4m3"]
    assert np.array_equal(np.isnan(ours), np.isnan(ref))
    assert np.array_equal(ours[~np.isnan(ours)], ref[~np.isnan(ref)])


def test_fp4_value_table(oracle):
    # the value set of nvfp4_pack_compare_test.cpp:28
    assert list(oracle.decode_e2m1_table()[:8]) == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert list(oracle.decode_e2m1_table()[8:]) == [-0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def test_encoders_match_reference(oracle, golden):
    assert np.array_equal(oracle.encode_e2m1(golden["e2m1_probe"]), golden["e2m1_codes"])
    assert np.array_equal(oracle.encode_e4m3(golden["e4m3_probe"]), golden["e4m3_codes"])


def test_sigmoid_matches_reference(oracle, golden):
    assert np.array_equal(oracle.sigmoid(golden["sigmoid_in"]), golden["sigmoid_out"])


@pytest.mark.parametrize("name", ["ramp9", "ramp11", "big", "zeros", "tiny", "normal", "relu2",
                                  "mixed_big"])
def test_packer_matches_reference(oracle, golden, name):
    packed, scales, ts = oracle.pack_nvfp4(golden[f"pack_{name}_x"])
    assert np.array_equal(packed, golden[f"pack_{name}_p"])
    assert np.array_equal(scales, golden[f"pack_{name}_s"])
    assert np.float32(ts) == golden[f"pack_{name}_ts"]


def test_packer_known_answers(oracle, golden):
    # nvfp4_packing_test.cpp: moderate inputs keep tensor scale >= 1, 4096.0 raises it,
    # a fixed scale of 0.002197265625 is preserved, bad shapes are rejected
    assert oracle.pack_nvfp4(golden["pack_ramp9_x"])[2] == 1.0
    assert oracle.pack_nvfp4(golden["pack_big_x"])[2] > 1.0
    p, s, ts = oracle.pack_nvfp4(golden["pack_normal_x"], fixed_tensor_scale=0.002197265625)
    assert np.float32(ts) == np.float32(0.002197265625) == golden["pack_fixed_ts"]
    assert np.array_equal(p, golden["pack_fixed_p"]) and np.array_equal(s, golden["pack_fixed_s"])
    assert oracle.pack_nvfp4(np.zeros((1, 15), np.float32)) is None
    assert oracle.pack_nvfp4(np.full((1, 16), np.inf, np.float32)) is None
    # all-zero input: zero codes and scale byte 0x38 (= 1.0), as nvfp4_gemm_runner_test.cpp:235-322 uses
    p, s, ts = oracle.pack_nvfp4(np.zeros((2, 32), np.float32))
    assert not p.any() and np.all(s == 0x38) and ts == 1.0


@pytest.mark.parametrize("name", ["a", "b"])
def test_swizzle_matches_reference(oracle, golden, name):
    out = oracle.swizzle_scales(golden[f"swz_{name}_in"], int(golden[f"swz_{name}_cols"]))
    assert np.array_equal(out, golden[f"swz_{name}_out"])


@pytest.mark.parametrize("name", ["e128", "grouped"])
def test_topk_matches_reference(oracle, golden, name):
    k, ng, tg = (int(v) for v in golden[f"topk_{name}_cfg"])
    idx, w = oracle.select_top_experts(golden[f"topk_{name}_logits"], golden[f"topk_{name}_bias"],
                                       k, ng, tg, True, 2.5)
    assert np.array_equal(idx, golden[f"topk_{name}_idx"])
    assert np.array_equal(w, golden[f"topk_{name}_w"])


def test_dense_double_matmul_matches_reference(oracle, golden):
    assert np.array_equal(oracle.router_logits(golden["dense_a"], golden["dense_w"]),
                          golden["dense_out"])


def test_expert_ffn_matches_reference(oracle, golden):
    up = oracle.Nvfp4Weight(golden["ffn_up_p"], golden["ffn_up_s"], float(golden["ffn_up_ts"]))
    down = oracle.Nvfp4Weight(golden["ffn_down_p"], golden["ffn_down_s"],
                              float(golden["ffn_down_ts"]))
    hidden, out = oracle.expert_ffn(golden["ffn_x"], up, down)
    assert np.array_equal(hidden, golden["ffn_hidden"])
    assert np.array_equal(out, golden["ffn_out"])
    # the weights-dequantised-once path is the same arithmetic
    fast = oracle.expert_ffn_forward(golden["ffn_x"], up, down)
    assert np.array_equal(fast.out, golden["ffn_out"])
    hp, hs, _ = oracle.pack_nvfp4_per_row(golden["ffn_hidden"])
    assert np.array_equal(fast.hid_packed, hp) and np.array_equal(fast.hid_scales, hs)


def _tiny_layer(synthetic, seed=5, experts=32, hidden=128, routed=64, shared=128, zipf=False):
    cfg = synthetic.baseline_config(64, experts=experts, hidden=hidden, routed=routed,
                                    shared=shared, top_k=4)
    return cfg, synthetic.make_layer(cfg, seed=seed, device="cpu", norm_weight_uniform=True,
                                     skewed=zipf)


def test_grouped_layer_is_bit_equal_to_literal_loop(oracle, synthetic):
    import helpers
    cfg, data = _tiny_layer(synthetic, zipf=True)
    x = synthetic.make_tokens(9, cfg.hidden_size, seed=3).to(torch.float32).numpy()
    ocfg, ow = helpers.oracle_config(cfg), helpers.oracle_weights(data)
    fast = oracle.layer_forward(ocfg, ow, x, want_routed_out=True)
    literal = oracle.layer_forward_literal(ocfg, ow, x)
    assert np.array_equal(fast.out, literal)
    # stage outputs are self-consistent
    assert np.array_equal(fast.normalized, oracle.rmsnorm(x, ow.norm_weight, cfg.rms_epsilon))
    p, s, ts = oracle.pack_nvfp4_per_row(fast.normalized)
    assert np.array_equal(p, fast.act_packed) and np.array_equal(s, fast.act_scales)
    assert fast.adopted_codes == 0 and fast.inadmissible_codes == 0


def test_override_adopts_only_admissible_codes(oracle, synthetic):
    import helpers
    cfg, data = _tiny_layer(synthetic)
    x = synthetic.make_tokens(4, cfg.hidden_size, seed=11).to(torch.float32).numpy()
    ocfg, ow = helpers.oracle_config(cfg), helpers.oracle_weights(data)
    base = oracle.layer_forward(ocfg, ow, x)
    cands = [base.hid_packed.copy(), base.hid_scales.copy(), base.shid_packed.copy(),
             base.shid_scales.copy()]
    same = oracle.layer_forward(ocfg, ow, x, candidates=cands)
    assert np.array_equal(same.out, base.out) and same.adopted_codes == 0
    cands[0][0, 0, 0] ^= 0x07  # a gross code error is not a rounding tie
    bad = oracle.layer_forward(ocfg, ow, x, candidates=cands)
    assert bad.inadmissible_codes >= 1 and np.array_equal(bad.out, base.out)
    assert not bad.adopted_token.any()


def test_override_distance_is_measured_in_accumulation_noise_units(oracle, golden):
    """A neighbouring code is adopted exactly when the limit reaches the distance that
    the oracle reports for it; the distance of a real near-tie is a few noise units,
    that of an arbitrary value thousands."""
    up = oracle.Nvfp4Weight(golden["ffn_up_p"], golden["ffn_up_s"], float(golden["ffn_up_ts"]))
    down = oracle.Nvfp4Weight(golden["ffn_down_p"], golden["ffn_down_s"],
                              float(golden["ffn_down_ts"]))
    x = golden["ffn_x"]
    base = oracle.expert_ffn_forward(x, up, down)
    distances = []
    for byte in range(0, base.hid_packed.shape[1], 3):
        cand = base.hid_packed.copy()
        low = int(cand[0, byte]) & 0x0f
        if low & 8 or (low & 7) == 7:
            continue
        cand[0, byte] = (cand[0, byte] & 0xf0) | (low + 1)  # the next larger magnitude
        wide = oracle.expert_ffn_forward(x, up, down, candidates=(cand, base.hid_scales),
                                         override_limit=1e9)
        assert wide.adopted_codes == 1 and wide.inadmissible_codes == 0 and wide.adopted_row[0]
        assert not wide.adopted_row[1:].any()
        d = wide.max_noise_units
        distances.append(d)
        below = oracle.expert_ffn_forward(x, up, down, candidates=(cand, base.hid_scales),
                                          override_limit=float(d) * 0.99)
        assert below.adopted_codes == 0 and below.inadmissible_codes == 1
        assert np.array_equal(below.out, base.out)
        above = oracle.expert_ffn_forward(x, up, down, candidates=(cand, base.hid_scales),
                                          override_limit=float(d) * 1.01)
        assert above.adopted_codes == 1
    assert len(distances) >= 4
    # arbitrary values are nowhere near a rounding boundary on this scale
    assert np.median(distances) > 1e3


def test_synthetic_weight_quantiser_matches_oracle(oracle, synthetic):
    g = torch.Generator().manual_seed(0)
    w = torch.randn((48, 160), generator=g) * 0.02
    w[3, 16:32] = 0.0
    packed, scales, ts = synthetic.quantize_weight(w)
    op, os_, ots = oracle.quantize_weight(w.numpy())
    assert np.array_equal(packed.numpy(), op)
    assert np.array_equal(scales.numpy(), os_)
    assert np.float32(ts.item()) == np.float32(ots)
    # configs[0]: global scale = amax / (6*448)
    assert np.float32(ots) == np.float32(w.abs().max().item()) / np.float32(2688.0)


def test_router_near_tie_margin_is_reported(oracle):
    logits = np.zeros((1, 32), np.float32)
    logits[0, :7] = [3, 2.5, 2, 1.5, 1, 0.5, 0.5]
    bias = np.zeros(32, np.float32)
    assert oracle.selection_margins(logits, bias, 6)[0] == 0.0
    idx, _ = oracle.select_top_experts(logits, bias, 6)
    assert list(idx[0]) == [0, 1, 2, 3, 4, 5]  # ties resolve to the lower index


def test_identity_latent_projections_change_nothing(oracle, synthetic):
    """fc1_latent = fc2_latent = identity: the double-accumulated dense linear returns its
    input bit for bit, so the layer equals the one without projections (how the literal
    reference, which insists on the projections, is driven at the benchmark shapes)."""
    import helpers
    cfg, data = _tiny_layer(synthetic)
    x = synthetic.make_tokens(5, cfg.hidden_size, seed=2).to(torch.float32).numpy()
    ocfg, ow = helpers.oracle_config(cfg), helpers.oracle_weights(data)
    base = oracle.layer_forward(ocfg, ow, x)
    ow.fc1 = np.eye(cfg.hidden_size, dtype=np.float32)
    ow.fc2 = np.eye(cfg.hidden_size, dtype=np.float32)
    same = oracle.layer_forward(ocfg, ow, x)
    assert np.array_equal(same.out, base.out)
    assert np.array_equal(same.latent, base.normalized)
    assert np.array_equal(same.projected, same.routed_latent)


def test_latent_layer_composes_the_documented_steps(oracle, synthetic):
    """The latent data flow restated with the oracle's own unit operators: fc1 (scaled FP8),
    routed sum, fc2, mixer, residual (expert_layer.cpp:809-813, :951-953, :1047-1069)."""
    import helpers
    cfg = synthetic.baseline_config(64, experts=32, hidden=128, routed=64, shared=128, top_k=4,
                                    latent=64)
    data = synthetic.make_layer(cfg, seed=8, device="cpu", norm_weight_uniform=True,
                                latent_family="fp8", shared_up_family="bf16",
                                shared_down_family="fp8")
    x = synthetic.make_tokens(6, cfg.hidden_size, seed=4).to(torch.float32).numpy()
    ocfg, ow = helpers.oracle_config(cfg), helpers.oracle_weights(data)
    r = oracle.layer_forward(ocfg, ow, x, want_routed_out=True)
    y = oracle.rmsnorm(x, ow.norm_weight, cfg.rms_epsilon)
    latent = oracle.router_logits(oracle.fp8_round_trip(y, ow.fc1_input_scale), ow.fc1)
    assert np.array_equal(r.latent, latent)
    p, s, ts = oracle.pack_nvfp4_per_row(latent)
    assert np.array_equal(p, r.act_packed) and np.array_equal(s, r.act_scales)
    routed = np.zeros_like(latent)
    for k in range(cfg.top_k):
        routed = (routed + r.routed_out[:, k, :] * r.top_weight[:, k:k + 1]).astype(np.float32)
    assert np.array_equal(routed, r.routed_latent)
    assert np.array_equal(r.projected, oracle.router_logits(routed, ow.fc2))
    su = oracle.router_logits(y, ow.shared_up_dense)
    su = np.where(su > 0, su * su, 0).astype(np.float32)
    assert np.array_equal(su, r.shid_values)
    shared = oracle.router_logits(oracle.fp8_round_trip(su, ow.shared_down_input_scale),
                                  ow.shared_down_dense)
    assert np.array_equal(shared, r.shared_out)
    assert np.array_equal(r.out, (x + (r.projected + shared)).astype(np.float32))


def test_fp8_round_trip_matches_torch_e4m3(oracle):
    g = torch.Generator().manual_seed(5)
    x = torch.randn((4, 64), generator=g) * 3.0
    scale = 8.0 / 448.0
    expect = ((x / scale).to(torch.float8_e4m3fn).to(torch.float32) * scale).numpy()
    inside = (x.abs() / scale <= 448.0).numpy()  # torch does not saturate; the reference does
    got = oracle.fp8_round_trip(x.numpy(), scale)
    assert np.array_equal(got[inside], expect[inside])
    assert np.all(np.abs(got[~inside]) == np.float32(448.0 * scale)) or inside.all()
