"""CPU tests of the layer stack's caller loop (runtime/src/api/single_token_forward_model.cpp:588-656:
each layer's FP32 output is the next layer's input, `current` / `next` swap): order of the layers,
buffer alternation, the three kinds of layer objects the loop accepts."""
import importlib

import numpy as np
import torch


def _stack_module(package):
    return importlib.import_module("nemotron_inference_b200.stack")


class _Engine:  # what the loop sees of an ExpertParallelEngine
    def __init__(self, log, scale):
        self.log, self.scale = log, scale

    def step(self, x, out):
        self.log.append(("step", x.data_ptr(), out.data_ptr()))
        out.copy_(x.to(out.dtype) * self.scale)


class _Slice:  # what the loop sees of an ExpertLayerSlice
    def __init__(self, log, bias):
        self.log, self.bias = log, bias

    def run_async(self, x, out):
        self.log.append(("run_async", x.data_ptr(), out.data_ptr()))
        out.copy_(x.to(out.dtype) + self.bias)


def test_layers_run_in_order_on_alternating_buffers(package):
    stack_module = _stack_module(package)
    log = []

    def callback(x, out):  # another layer kind, the caller's own code
        log.append(("call", x.data_ptr(), out.data_ptr()))
        out.copy_(x.to(out.dtype) * x.to(out.dtype))

    layers = [_Engine(log, 2.0), callback, _Slice(log, 1.0), _Engine(log, 0.5)]
    stack = stack_module.MoeLayerStack(layers, hidden_size=8, max_tokens=16, device=torch.device("cpu"))
    x = torch.arange(24, dtype=torch.float32).reshape(3, 8).to(torch.bfloat16)
    out = torch.empty((3, 8), dtype=torch.float32)
    stack.run(x, out)
    expect = ((x.to(torch.float32) * 2.0) ** 2 + 1.0) * 0.5
    assert torch.equal(out, expect)
    assert [kind for kind, _, _ in log] == ["step", "call", "run_async", "step"]
    # the input is read from the caller's tensor, the result lands in the caller's tensor,
    # every layer reads what the layer before wrote, and no layer writes the buffer it reads
    assert log[0][1] == x.data_ptr() and log[-1][2] == out.data_ptr()
    for before, after in zip(log, log[1:]):
        assert after[1] == before[2]
    assert all(src != dst for _, src, dst in log)
    assert len({dst for _, _, dst in log[:-1]}) == 2  # ping and pong


def test_fewer_tokens_than_the_buffers_hold(package):
    stack_module = _stack_module(package)
    log = []
    stack = stack_module.MoeLayerStack([_Slice(log, 1.0), _Slice(log, 1.0), _Slice(log, 1.0)],
                                       hidden_size=4, max_tokens=8, device=torch.device("cpu"))
    for tokens in (1, 8, 5):
        x = torch.zeros((tokens, 4), dtype=torch.float32)
        out = torch.empty_like(x)
        stack.run(x, out)
        assert np.array_equal(out.numpy(), np.full((tokens, 4), 3.0, np.float32))


def test_a_single_layer_writes_straight_to_the_output(package):
    stack_module = _stack_module(package)
    log = []
    stack = stack_module.MoeLayerStack([_Engine(log, 3.0)], hidden_size=4, max_tokens=2,
                                       device=torch.device("cpu"))
    x = torch.ones((2, 4), dtype=torch.float32)
    out = torch.empty_like(x)
    stack.run(x, out)
    assert log == [("step", x.data_ptr(), out.data_ptr())] and torch.equal(out, x * 3.0)
