"""GPU parity of the whole MoE layer against the CPU oracle: configs[1] (decode sizes),
configs[2] (skewed prefill) and reduced-size variants, through ExpertLayerSlice."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def baseline_layer(package, synthetic):
    cfg = synthetic.baseline_config(max_tokens=8192)
    data = synthetic.make_layer(cfg, seed=1000, device="cuda")
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None and layer.valid(), package.ExpertLayerSlice.create_error
    yield layer, data
    layer.close()


def _run(layer, x, out_dtype=torch.float32):
    out = torch.empty(x.shape, dtype=out_dtype, device="cuda")
    assert layer.run(x, out), layer.last_error
    return out


def test_small_layer_every_stage(package, synthetic):
    cfg = synthetic.baseline_config(max_tokens=1024, experts=32, hidden=512, routed=256, shared=512)
    data = synthetic.make_layer(cfg, seed=21, device="cuda", norm_weight_uniform=True)
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None
    for tokens in (1, 3, 33, 200, 300, 1000):
        x = synthetic.make_tokens(tokens, cfg.hidden_size, seed=tokens, device="cuda")
        out = _run(layer, x)
        rep = helpers.compare_layer_with_oracle(layer, data, x, out)
        print(rep.summary())
        assert rep.ok(), rep.summary()
        # weights may differ in the last bit where glibc's expf is not the correctly rounded exp
        assert rep.norm_max_diff == 0.0 and rep.weight_max_diff <= 1.2e-7
        # below 256 tokens every logit is an FP64 sum; above, only the candidates' are
        assert rep.logits_max_diff == 0.0 or tokens >= 256
    layer.close()


def test_layer_input_rows_whose_tensor_scale_is_not_one(package, synthetic, oracle):
    """A norm weight of ~200 and rows dominated by one element put the largest normalised
    value (about sqrt(H) * 200) beyond 6 * 448: the quantiser's tensor scale leaves 1 for
    those rows (nvfp4_packing.cpp:119-126) and stays 1 for the ordinary rows beside them.
    Only the layer-input quantiser is checked (such activations overflow the experts)."""
    cfg = synthetic.baseline_config(max_tokens=64, experts=32, hidden=512, routed=256, shared=512)
    data = synthetic.make_layer(cfg, seed=77, device="cuda", norm_weight_uniform=True)
    data.bindings.input_norm_weight = (data.bindings.input_norm_weight.to(torch.float32) * 200.0)
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None, package.ExpertLayerSlice.create_error
    x = synthetic.make_tokens(16, cfg.hidden_size, seed=78, device="cuda").to(torch.float32)
    x[::2] *= 1e-3
    x[::2, 5] = 40.0  # every other row: one element carries the whole norm
    out = torch.empty_like(x)
    layer.run(x, out)  # the status may report the experts' activation range: not the subject
    trace = layer.trace(16)
    y = oracle.rmsnorm(x.cpu().numpy(), data.bindings.input_norm_weight.cpu().numpy(),
                       cfg.rms_epsilon)
    packed, scales, ts = oracle.pack_nvfp4_per_row(y)
    assert np.all(ts[::2] > 1.0) and np.all(ts[1::2] == 1.0)
    assert np.array_equal(trace.act_tensor_scale.cpu().numpy(), ts)
    assert np.array_equal(trace.act_packed.cpu().numpy(), packed)
    assert np.array_equal(trace.act_scales.cpu().numpy(), scales)
    layer.close()


@pytest.mark.parametrize("tokens", [1, 8, 32, 64])
def test_decode_sizes_config1(baseline_layer, synthetic, tokens):
    layer, data = baseline_layer
    x = synthetic.make_tokens(tokens, 2688, seed=2000 + tokens, device="cuda")
    out = _run(layer, x)
    rep = helpers.compare_layer_with_oracle(layer, data, x, out)
    print(rep.summary())
    assert rep.ok(), rep.summary()
    out_bf16 = _run(layer, x, torch.bfloat16)
    rep16 = helpers.compare_layer_with_oracle(layer, data, x, out_bf16, raw_run=False)
    print(rep16.summary())
    assert rep16.ok(), rep16.summary()


def test_results_do_not_depend_on_batching(baseline_layer, synthetic):
    # expert_layer_oracle_test.cpp:1086-1161: a 3-token batch equals three single-token runs
    layer, _ = baseline_layer
    x = synthetic.make_tokens(3, 2688, seed=77, device="cuda")
    batched = _run(layer, x)
    for t in range(3):
        single = _run(layer, x[t:t + 1].contiguous())
        assert torch.equal(single[0], batched[t])


def test_small_batches_replay_a_recorded_graph(baseline_layer, synthetic):
    # on a capturable stream a small batch is recorded once and replayed afterwards: same
    # result as the eager run, and a replay reads the CURRENT contents of its buffers
    layer, _ = baseline_layer
    x = synthetic.make_tokens(8, 2688, seed=91, device="cuda")
    eager = _run(layer, x)                       # legacy default stream: eager
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    out = torch.empty_like(eager)
    with torch.cuda.stream(stream):
        for _ in range(3):                       # record, replay, replay
            layer.run_async(x, out)
        stream.synchronize()
        assert layer.sync_status() == 0
        assert torch.equal(out, eager)
        other = synthetic.make_tokens(8, 2688, seed=92, device="cuda")
        x.copy_(other)
        layer.run_async(x, out)
        stream.synchronize()
    torch.cuda.synchronize()
    assert torch.equal(out, _run(layer, other))


def test_layer_from_checkpoint_tensor_names(package, synthetic):
    # weights named as the reference's checkpoint names them, on the HOST, straight into
    # the layer: same rows as the layer built from the synthetic bindings
    import importlib
    checkpoint = importlib.import_module("nemotron_inference_b200.checkpoint")
    cfg = synthetic.baseline_config(max_tokens=64, experts=32, hidden=512, routed=256, shared=512)
    data = synthetic.make_layer(cfg, seed=61, device="cuda", norm_weight_uniform=True)
    tensors = {name: t.cpu() for name, t in
               checkpoint.tensors_from_bindings(data.bindings, layer_index=3).items()}
    bindings = checkpoint.bindings_from_tensors(tensors, 3, cfg.n_routed_experts)
    direct = package.ExpertLayerSlice.create(cfg, data.bindings)
    named = package.ExpertLayerSlice.create(cfg, bindings)
    assert direct is not None and named is not None, package.ExpertLayerSlice.create_error
    x = synthetic.make_tokens(40, cfg.hidden_size, seed=62, device="cuda")
    assert torch.equal(_run(direct, x), _run(named, x))
    direct.close()
    named.close()


def test_run_rejects_bad_shapes(baseline_layer):
    layer, _ = baseline_layer
    x = torch.zeros((2, 100), device="cuda")
    assert not layer.run(x, torch.empty_like(x))
    big = torch.zeros((8193, 2688), device="cuda", dtype=torch.bfloat16)
    assert not layer.run(big, torch.empty((8193, 2688), device="cuda"))


def test_prefill_skewed_config2(package, synthetic):
    cfg = synthetic.baseline_config(max_tokens=8192)
    data = synthetic.make_layer(cfg, seed=3000, device="cuda", skewed=True)
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None
    x = synthetic.make_tokens(8192, 2688, seed=3001, device="cuda")
    out = _run(layer, x)
    trace_idx = layer.trace(8192).selected_index.cpu().numpy()
    counts = np.bincount(trace_idx.ravel(), minlength=128)
    print("expert load: max/mean = %.2f, empty experts = %d" % (counts.max() / counts.mean(),
                                                                 int((counts == 0).sum())))
    rep = helpers.compare_layer_with_oracle(layer, data, x, out)
    print(rep.summary())
    assert rep.ok(), rep.summary()
    assert counts.max() / counts.mean() > 3.0
    layer.close()


def test_layer_stack_matches_oracle_applied_layer_by_layer(package, synthetic, oracle):
    # configs[4] in miniature: independently seeded layers, RMSNorm weight ~U(0.9, 1.1),
    # the FP32 hidden state handed from layer to layer (the caller loop of
    # runtime/src/api/single_token_forward_model.cpp:588-656).  Every layer is gated on the
    # full parity report with the DEVICE output of the previous layer as its input, so a
    # rounding tie in one layer cannot hide an error in the next; the stack itself must
    # then return exactly what the layers return one by one.
    import importlib
    stack_mod = importlib.import_module("nemotron_inference_b200.stack")
    cfg = synthetic.baseline_config(max_tokens=512, experts=32, hidden=512, routed=256, shared=512)
    datas = [synthetic.make_layer(cfg, seed=700 + i, device="cuda", norm_weight_uniform=True)
             for i in range(3)]
    layers = [package.ExpertLayerSlice.create(cfg, d.bindings) for d in datas]
    stack = stack_mod.MoeLayerStack(layers, cfg.hidden_size, 512)
    for tokens in (5, 400):
        x = synthetic.make_tokens(tokens, cfg.hidden_size, seed=tokens + 1, device="cuda")
        current = x
        for index, (layer, data) in enumerate(zip(layers, datas)):
            out = _run(layer, current)
            rep = helpers.compare_layer_with_oracle(layer, data, current, out)
            print(f"stack T={tokens} layer {index}: {rep.summary()}")
            assert rep.ok(), rep.summary()
            current = out
        stacked = torch.empty((tokens, cfg.hidden_size), dtype=torch.float32, device="cuda")
        stack.run(x, stacked)
        torch.cuda.synchronize()
        assert stack.sync_status() == 0
        assert torch.equal(stacked, current)
    # another layer kind between two MoE layers, as in the model's loop: a callback
    mixed = stack_mod.MoeLayerStack(
        [layers[0], lambda a, b: b.copy_(a.to(torch.float32) * 0.5), layers[1]],
        cfg.hidden_size, 512)
    x = synthetic.make_tokens(7, cfg.hidden_size, seed=8, device="cuda")
    got = torch.empty((7, cfg.hidden_size), dtype=torch.float32, device="cuda")
    mixed.run(x, got)
    want = _run(layers[1], (_run(layers[0], x) * 0.5).contiguous())
    assert mixed.sync_status() == 0 and torch.equal(got, want)
    for layer in layers:
        layer.close()
