"""HostPipeline: batches in pinned host memory, transfers overlapped with the compute.  Every
batch must come back exactly as the one-batch-at-a-time call returns it, whatever the depth."""
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("depth", [1, 2, 3])
def test_pipelined_batches_equal_direct_runs(package, synthetic, depth):
    host_pipeline = importlib.import_module("nemotron_inference_b200.host_pipeline")
    cfg = synthetic.baseline_config(max_tokens=512, experts=32, hidden=512, routed=256, shared=512)
    data = synthetic.make_layer(cfg, seed=77, device="cuda", norm_weight_uniform=True)
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None, package.ExpertLayerSlice.create_error
    batches = [synthetic.make_tokens(rows, 512, seed=100 + i).pin_memory()
               for i, rows in enumerate((512, 300, 512, 7, 512, 256, 33))]
    expected = []
    for x_host in batches:
        out = torch.empty(x_host.shape, dtype=torch.bfloat16, device="cuda")
        assert layer.run(x_host.cuda(), out), layer.last_error
        expected.append(out.cpu())
    results = [torch.zeros(x.shape, dtype=torch.bfloat16).pin_memory() for x in batches]
    pipe = host_pipeline.HostPipeline(lambda x, out: layer.run_async(x, out), 512, 512,
                                      depth=depth)
    for x_host, out_host in zip(batches, results):
        pipe.submit(x_host, out_host)
    pipe.synchronize()
    assert layer.sync_status() == 0
    for got, want in zip(results, expected):
        assert torch.equal(got, want)
    layer.close()


def test_pageable_host_memory_is_rejected(package, synthetic):
    host_pipeline = importlib.import_module("nemotron_inference_b200.host_pipeline")
    pipe = host_pipeline.HostPipeline(lambda x, out: None, 8, 512)
    with pytest.raises(ValueError):
        pipe.submit(torch.zeros((8, 512), dtype=torch.bfloat16),
                    torch.zeros((8, 512), dtype=torch.bfloat16))
