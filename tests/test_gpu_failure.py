"""Failure detection on the device without faulting, trapping or hanging it: a kernel that
waits for another GPU gives up after a limit and leaves an error status the host reads."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

NMOE_ERR_DEVICE_TIMEOUT = 4


def test_bounded_flag_wait_runs_out_and_the_layer_stays_usable(package, synthetic):
    cfg = synthetic.baseline_config(max_tokens=64, experts=32, hidden=512, routed=256, shared=512)
    data = synthetic.make_layer(cfg, seed=11, device="cuda")
    layer = package.ExpertLayerSlice.create(cfg, data.bindings)
    assert layer is not None
    x = synthetic.make_tokens(16, cfg.hidden_size, seed=12, device="cuda")
    out = torch.empty((16, cfg.hidden_size), dtype=torch.float32, device="cuda")
    assert layer.run(x, out), layer.last_error
    before = out.clone()

    # a flag that nothing raises: the wait runs out after the (short) limit
    layer.set_wait_limit_ms(20.0)
    flag = torch.zeros((1,), dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    start = time.perf_counter()
    layer.wait_flag(flag, 1)
    status = layer.sync_status()
    elapsed = time.perf_counter() - start
    assert status == NMOE_ERR_DEVICE_TIMEOUT
    assert elapsed < 2.0, f"the bounded wait took {elapsed:.3f} s"

    # a raised flag passes at once, and the error slot was cleared by the read above
    flag.fill_(1)
    layer.wait_flag(flag, 1)
    assert layer.sync_status() == 0

    # the context and the layer are intact
    assert layer.run(x, out), layer.last_error
    assert torch.equal(out, before)
    layer.close()
