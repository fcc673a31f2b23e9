"""The drop-in boundary exercised from C++: oracle/_ref/shim_driver is the reference's own
header types (ExpertLayerConfig, GemmDescriptor, DeviceTensorFp32, CublasLtHandle, ...) +
nemotron-inference_b200/shim/expert_layer_shim.cpp + libnmoe_b200.so.  It must return exactly
what the Python binding returns for the same bytes, and keep the reference's error behaviour."""
import os
import struct
import subprocess

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "oracle", "_ref", "shim_driver")


def _bytes(t: torch.Tensor) -> bytes:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()


def _nvfp4(m) -> bytes:
    return (_bytes(m.packed) + _bytes(m.block_scales) +
            struct.pack("<f", float(m.tensor_scale)))


@pytest.mark.parametrize("tokens", [1, 37])
def test_reference_typed_cpp_caller_gets_the_same_rows(package, synthetic, oracle, tmp_path,
                                                       tokens, monkeypatch):
    import helpers
    monkeypatch.setenv("NMOE_SHIM_MAX_TOKENS", "8")  # 37 tokens make the scratch grow
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/shim_driver was not built (needs the reference checkout)")
    experts, hidden, routed, shared = 32, 512, 256, 512
    cfg = synthetic.baseline_config(max_tokens=64, experts=experts, hidden=hidden, routed=routed,
                                    shared=shared)
    data = synthetic.make_layer(cfg, seed=55, device="cuda", norm_weight_uniform=True)
    b = data.bindings
    x = synthetic.make_tokens(tokens, hidden, seed=56, device="cuda").to(torch.float32)

    blob = struct.pack("<10q", hidden, routed, shared, experts, cfg.top_k, tokens,
                       1 if cfg.norm_topk_prob else 0, 0, 0, 0)
    blob += struct.pack("<ff", cfg.rms_epsilon, cfg.routed_scaling_factor)
    blob += _bytes(b.input_norm_weight.to(torch.float32))
    blob += _bytes(b.gate_weight.to(torch.bfloat16))
    blob += _bytes(b.gate_score_correction_bias.to(torch.float32))
    for pair in b.routed_experts:
        blob += _nvfp4(pair.up_proj) + _nvfp4(pair.down_proj)
    blob += _nvfp4(b.shared_up) + _nvfp4(b.shared_down)
    blob += _bytes(x)
    src, dst = tmp_path / "layer.bin", tmp_path / "rows.bin"
    src.write_bytes(blob)
    done = subprocess.run([DRIVER, str(src), str(dst)], capture_output=True, text=True,
                          timeout=300, env=dict(os.environ, NEMOTRON_FORWARD_DEBUG="1"))
    assert done.returncode == 0, done.stderr

    raw = dst.read_bytes()
    rows, cols, rejected, selected = struct.unpack("<4q", raw[:32])
    assert (rows, cols) == (tokens, hidden)
    assert rejected == 1  # Run with a mis-shaped output returns false, as the reference does
    got = np.frombuffer(raw, dtype=np.float32, count=rows * cols, offset=32).reshape(rows, cols)

    layer = package.ExpertLayerSlice.create(cfg, b)
    assert layer is not None, package.ExpertLayerSlice.create_error
    want = torch.empty((tokens, hidden), dtype=torch.float32, device="cuda")
    assert layer.run(x, want), layer.last_error
    assert np.array_equal(got, want.cpu().numpy())

    if tokens == 1:  # the trace the reference fills for one token
        assert selected == cfg.top_k
        trace = layer.trace(1)
        at = 32 + rows * cols * 4
        for slot in range(cfg.top_k):
            index, weight = struct.unpack("<qf", raw[at:at + 12])
            at += 12
            assert index == int(trace.selected_index[0, slot])
            assert weight == float(trace.selected_weight[0, slot])
        # every vector of the trace against the CPU oracle, at the tolerances of the
        # reference's own layer test (testing/backend/expert_layer_oracle_test.cpp:1061-1077)
        names = ("normalized_input", "router_logits", "latent_output", "routed_latent_output",
                 "routed_expert_activated_hidden", "routed_expert_outputs",
                 "routed_expert_weighted_contributions", "projected_routed_output",
                 "shared_output", "mixer_output")
        fields = {}
        for name in names:
            (n,) = struct.unpack("<q", raw[at:at + 8])
            fields[name] = np.frombuffer(raw, dtype=np.float32, count=n, offset=at + 8)
            at += 8 + 4 * n
        (n,) = struct.unpack("<q", raw[at:at + 8])
        order = np.frombuffer(raw, dtype=np.int64, count=n, offset=at + 8)
        ref = oracle.layer_forward(helpers.oracle_config(cfg), helpers.oracle_weights(data),
                                   x.cpu().numpy(), want_routed_out=True)
        K = cfg.top_k
        assert list(order) == list(ref.top_index[0])
        weighted = ref.routed_out[0] * ref.top_weight[0][:, None]
        expect = {
            "normalized_input": (ref.normalized[0], 1e-5), "router_logits": (ref.logits[0], 2e-5),
            "latent_output": (ref.normalized[0], 1e-5),
            "routed_latent_output": (ref.routed_latent[0], 1e-3),
            "routed_expert_activated_hidden": (ref.hid_values[0].ravel(), 1e-3),
            "routed_expert_outputs": (ref.routed_out[0].ravel(), 1e-3),
            "routed_expert_weighted_contributions": (weighted.ravel(), 1e-3),
            "projected_routed_output": (ref.projected[0], 1e-3),
            "shared_output": (ref.shared_out[0], 1e-3),
            "mixer_output": (ref.projected[0] + ref.shared_out[0], 1e-3)}
        for name, (want_values, tol) in expect.items():
            assert fields[name].shape == want_values.shape, name
            assert np.abs(fields[name] - want_values).max() <= tol, name
        assert K * hidden == fields["routed_expert_outputs"].size
    else:
        assert selected == 0
    layer.close()
