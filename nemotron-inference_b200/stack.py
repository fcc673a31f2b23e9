"""A stack of MoE expert layers applied back to back (the MoE path of the model's layer
loop, runtime/src/api/single_token_forward_model.cpp:588-656: the caller hands each
layer's FP32 output to the next and swaps `current` / `next`).  Every layer carries its
own input RMSNorm and residual add, so the stack is layer(layer(...layer(x))).

Works over single-device layers (`ExpertLayerSlice`), over expert-parallel engines
(`ExpertParallelEngine`) and over plain callables `f(x, out)`: the model's layer loop
interleaves MoE layers with Mamba and attention layers (:603-636), which stay the caller's
own code and enter the stack as callbacks on the same device buffers.  The hidden state
stays on the device in FP32 between layers; nothing synchronises with the host except the
split-size exchange inside a compact expert-parallel step.
"""
from __future__ import annotations

from typing import List, Sequence

import torch


class MoeLayerStack:
    def __init__(self, layers: Sequence, hidden_size: int, max_tokens: int, device=None):
        self.layers = list(layers)
        device = device or torch.device("cuda", torch.cuda.current_device())
        self._ping = torch.empty((max_tokens, hidden_size), dtype=torch.float32, device=device)
        self._pong = torch.empty((max_tokens, hidden_size), dtype=torch.float32, device=device)

    @staticmethod
    def _run_one(layer, x: torch.Tensor, out: torch.Tensor) -> None:
        if hasattr(layer, "step"):         # ExpertParallelEngine
            layer.step(x, out)
        elif hasattr(layer, "run_async"):  # ExpertLayerSlice
            layer.run_async(x, out)
        else:                              # another layer kind, the caller's own code
            layer(x, out)

    def run(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """x: [tokens, hidden] bf16 or FP32; out: same shape, bf16 or FP32 (may not alias x)."""
        tokens = x.shape[0]
        current = x
        buffers = [self._ping[:tokens], self._pong[:tokens]]
        for index, layer in enumerate(self.layers):
            last = index == len(self.layers) - 1
            target = out if last else buffers[index % 2]
            self._run_one(layer, current, target)
            current = target

    def capture(self, x: torch.Tensor, out: torch.Tensor) -> bool:
        """Records the whole stack on (x, out) as ONE CUDA graph (possible when no layer
        synchronises with the host: single-device layers, expert-parallel engines on peer
        windows or fixed-capacity segments).  False, and eager execution, otherwise."""
        try:
            for _ in range(2):
                self.run(x, out)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self.run(x, out)
            self._graph = graph
            return True
        except Exception as error:  # noqa: BLE001 - any capture failure means "stay eager"
            self.capture_error = str(error)
            self._graph = None
            torch.cuda.synchronize()
            return False

    def replay(self) -> None:
        self._graph.replay()

    def release_graph(self) -> None:
        if getattr(self, "_graph", None) is not None:
            torch.cuda.synchronize()
            self._graph = None
            import gc
            gc.collect()

    def sync_status(self) -> int:
        status = 0
        for layer in self.layers:
            owner = layer.stages if hasattr(layer, "stages") else layer
            if hasattr(owner, "sync_status"):
                status = status or owner.sync_status()
        return status
