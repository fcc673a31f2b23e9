"""GPU parity of the latent-MoE form of the layer, the one the reference's checkpoint has
(runtime/src/api/single_token_forward_model.cpp:116-126): fc1_latent in front of the routed
experts and fc2_latent behind them (runtime/src/backend/expert_layer.cpp:809-813,
:1047-1053), the shared expert's projections in the dense, scaled-FP8 or NVFP4 family
(:534-617), and of the unfused activation path with its trace fields."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def _run(layer, x, out_dtype=torch.float32):
    out = torch.empty(x.shape, dtype=out_dtype, device="cuda")
    assert layer.run(x, out), layer.last_error
    return out


@pytest.mark.parametrize("latent_family,shared_up_family,shared_down_family", [
    ("bf16", "nvfp4", "nvfp4"), ("fp8", "fp8", "nvfp4"), ("fp32", "bf16", "fp8")])
def test_small_latent_layer_every_stage(package, synthetic, latent_family, shared_up_family,
                                        shared_down_family):
    cfg = synthetic.baseline_config(max_tokens=512, experts=32, hidden=512, routed=256, shared=512,
                                    latent=256)
    data = synthetic.make_layer(cfg, seed=41, device="cuda", norm_weight_uniform=True,
                                latent_family=latent_family, shared_up_family=shared_up_family,
                                shared_down_family=shared_down_family)
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None, package.ExpertLayerSlice.create_error
    for tokens in (1, 3, 33, 300):
        x = synthetic.make_tokens(tokens, cfg.hidden_size, seed=tokens + 50, device="cuda")
        out = _run(layer, x)
        rep = helpers.compare_layer_with_oracle(layer, data, x, out)
        print(latent_family, shared_up_family, shared_down_family, rep.summary())
        assert rep.ok(), rep.summary()
        assert rep.norm_max_diff == 0.0 and rep.latent_max_diff == 0.0
        out_bf16 = _run(layer, x, torch.bfloat16)
        rep16 = helpers.compare_layer_with_oracle(layer, data, x, out_bf16, raw_run=False)
        assert rep16.ok(), rep16.summary()
    layer.close()


def test_checkpoint_shape_latent_layer(package, synthetic):
    # hidden 4096, latent 1024, routed 2688, shared 5376, 512 experts, top-22, scaling 5:
    # fc1_latent and shared_up scaled FP8, shared_down NVFP4, as the checkpoint has them
    # (testing/oracle/expert_layer1_decode_block/metadata.json)
    cfg = synthetic.checkpoint_shape_config(max_tokens=64)
    data = synthetic.make_layer(cfg, seed=77, device="cuda", norm_weight_uniform=True,
                                latent_family="fp8", shared_up_family="fp8")
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None, package.ExpertLayerSlice.create_error
    for tokens in (1, 8):
        x = synthetic.make_tokens(tokens, cfg.hidden_size, seed=tokens + 9, device="cuda")
        out = _run(layer, x)
        rep = helpers.compare_layer_with_oracle(layer, data, x, out)
        print(rep.summary())
        assert rep.ok(), rep.summary()
    layer.close()


def test_unfused_activation_path_and_trace_fields(package, synthetic, oracle):
    cfg = synthetic.baseline_config(max_tokens=256, experts=32, hidden=512, routed=256, shared=512)
    data = synthetic.make_layer(cfg, seed=21, device="cuda", norm_weight_uniform=True)
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None
    ocfg, ow = helpers.oracle_config(cfg), helpers.oracle_weights(data)
    for tokens in (1, 40, 200):
        x = synthetic.make_tokens(tokens, cfg.hidden_size, seed=tokens + 3, device="cuda")
        fused = _run(layer, x)
        layer.set_unfused_activation(True)
        unfused = _run(layer, x)
        rep = helpers.compare_layer_with_oracle(layer, data, x, unfused)
        print("unfused", rep.summary())
        assert rep.ok(), rep.summary()
        # both paths quantise the same FP32 values by the same rule
        assert torch.equal(fused, unfused)
        if tokens <= 64:
            # what ExpertLayerRunTrace holds beyond the fused path's buffers
            # (expert_layer.h:63-76; gated at 1e-3 by expert_layer_oracle_test.cpp:1061-1077)
            activated, outputs, shared_activated = layer.unfused_trace(tokens)
            ref = oracle.layer_forward(ocfg, ow, x.to(torch.float32).cpu().numpy(),
                                       want_routed_out=True)
            scale = max(1.0, float(np.abs(ref.hid_values).max()))
            assert np.abs(activated.cpu().numpy() - ref.hid_values).max() <= 1e-3 * scale
            assert np.abs(shared_activated.cpu().numpy() - ref.shid_values).max() <= 1e-3 * scale
            if rep.adopted_codes + rep.adopted_scales == 0:
                assert np.abs(outputs.cpu().numpy() - ref.routed_out).max() <= 1e-3
        layer.set_unfused_activation(False)
    layer.close()


def test_activated_rows_beyond_the_fp4_range_need_the_unfused_path(package, synthetic):
    # relu^2 values above 6 * 448 give the row a tensor scale != 1
    # (nvfp4_packing.cpp:119-126): the fused epilogue reports it, the unfused path
    # reproduces the reference
    cfg = synthetic.baseline_config(max_tokens=64, experts=32, hidden=512, routed=256, shared=512)
    data = synthetic.make_layer(cfg, seed=23, device="cuda", norm_weight_uniform=True)
    for pair in data.bindings.routed_experts:
        pair.up_proj.tensor_scale *= 400.0
    data.up_ts = data.up_ts * 400.0
    data.bindings.shared_up.tensor_scale *= 400.0
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None
    x = synthetic.make_tokens(12, cfg.hidden_size, seed=5, device="cuda")
    out = torch.empty(x.shape, dtype=torch.float32, device="cuda")
    assert not layer.run(x, out)
    assert "ACTIVATION_RANGE" in layer.last_error
    layer.set_unfused_activation(True)
    assert layer.run(x, out), layer.last_error
    rep = helpers.compare_layer_with_oracle(layer, data, x, out)
    print("beyond range", rep.summary())
    # rows with a tensor scale != 1 are outside the tie analysis: exact bytes expected
    assert rep.hidden_code_mismatches == 0 and rep.hidden_scale_mismatches == 0
    assert rep.index_set_mismatches == 0 and rep.act_code_mismatches == 0
    # the outputs are 160,000 times their usual size here: the layer tolerance, which is
    # absolute, is taken relative to them (what is left is FP32 summation order)
    magnitude = float(out.abs().max().item())
    assert magnitude > 1e3
    assert rep.max_abs <= 1e-5 * magnitude and rep.cosine >= helpers.COSINE_TOL
    layer.close()


def test_scratch_grows_on_demand(package, synthetic):
    cfg = synthetic.baseline_config(max_tokens=16, experts=32, hidden=512, routed=256, shared=512)
    data = synthetic.make_layer(cfg, seed=21, device="cuda")
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    x = synthetic.make_tokens(300, cfg.hidden_size, seed=1, device="cuda")
    out = torch.empty(x.shape, dtype=torch.float32, device="cuda")
    assert not layer.run(x, out)  # NMOE_ERR_CAPACITY
    layer.reserve_tokens(300)
    assert layer.run(x, out), layer.last_error
    rep = helpers.compare_layer_with_oracle(layer, data, x, out)
    assert rep.ok(), rep.summary()
    layer.close()
