"""The layer's bindings from checkpoint tensors by the reference's tensor names
(BuildExpertLayerBindings, runtime/src/backend/expert_layer.cpp:427-492; NVFP4 triple of
tools/manifest/generate_forward_manifest.py:344-400)."""
import importlib

import pytest
import torch


@pytest.fixture(scope="module")
def checkpoint(package):
    return importlib.import_module("nemotron_inference_b200.checkpoint")


def _same_matrix(a, b):
    return (torch.equal(a.packed, b.packed) and torch.equal(a.block_scales, b.block_scales) and
            a.tensor_scale == b.tensor_scale)


@pytest.mark.parametrize("latent,shared_up,shared_down", [(0, "nvfp4", "nvfp4"),
                                                          (64, "fp8", "nvfp4"),
                                                          (64, "bf16", "fp8")])
def test_bindings_round_trip_through_checkpoint_names(checkpoint, synthetic, latent, shared_up,
                                                      shared_down):
    cfg = synthetic.baseline_config(8, experts=32, hidden=128, routed=64, shared=128, top_k=4,
                                    latent=latent)
    data = synthetic.make_layer(cfg, seed=3, device="cpu", latent_family="fp8",
                                shared_up_family=shared_up, shared_down_family=shared_down)
    tensors = checkpoint.tensors_from_bindings(data.bindings, layer_index=7)
    assert "backbone.layers.7.mixer.experts.31.down_proj.weight_scale_2" in tensors
    back = checkpoint.bindings_from_tensors(tensors, 7, cfg.n_routed_experts)
    assert back is not None and len(back.routed_experts) == 32
    for got, want in zip(back.routed_experts, data.bindings.routed_experts):
        assert _same_matrix(got.up_proj, want.up_proj)
        assert _same_matrix(got.down_proj, want.down_proj)
    for which in ("shared_up", "shared_down"):
        want, got = getattr(data.bindings, which), getattr(back, which)
        assert (want is None) == (got is None)
        if want is not None:
            assert _same_matrix(got, want)
        want_l, got_l = getattr(data.bindings, which + "_linear"), getattr(back, which + "_linear")
        assert (want_l is None) == (got_l is None)
        if want_l is not None:
            assert got_l.is_fp8 == want_l.is_fp8
            assert torch.equal(got_l.weight.view(torch.uint8) if got_l.is_fp8 else got_l.weight,
                               want_l.weight)
            if want_l.is_fp8:
                assert got_l.weight_scale == pytest.approx(want_l.weight_scale, rel=1e-7)
                assert got_l.input_scale == pytest.approx(want_l.input_scale, rel=1e-7)
    assert (back.fc1_latent is None) == (latent == 0)
    if latent:
        assert back.fc1_latent.is_fp8 and not back.fc2_latent.is_fp8
    # one rank's share for expert parallelism
    shard = checkpoint.bindings_from_tensors(tensors, 7, cfg.n_routed_experts, rank=3, world=4)
    assert shard.first_local_expert == 24 and len(shard.routed_experts) == 8
    assert _same_matrix(shard.routed_experts[0].up_proj, data.bindings.routed_experts[24].up_proj)


def test_missing_tensors_give_none(checkpoint, synthetic):
    cfg = synthetic.baseline_config(8, experts=32, hidden=128, routed=64, shared=128, top_k=4)
    data = synthetic.make_layer(cfg, seed=3, device="cpu")
    tensors = checkpoint.tensors_from_bindings(data.bindings, layer_index=0)
    for missing in ("backbone.layers.0.norm.weight",
                    "backbone.layers.0.mixer.experts.5.up_proj.weight_scale",
                    "backbone.layers.0.mixer.shared_experts.down_proj.weight"):
        broken = dict(tensors)
        del broken[missing]
        assert checkpoint.bindings_from_tensors(broken, 0, cfg.n_routed_experts) is None
    # the tensor scale may come as input_scale when weight_scale_2 is absent
    renamed = dict(tensors)
    key = "backbone.layers.0.mixer.experts.0.up_proj.weight_scale_2"
    renamed[key.replace("weight_scale_2", "input_scale")] = renamed.pop(key)
    assert checkpoint.bindings_from_tensors(renamed, 0, cfg.n_routed_experts) is not None
