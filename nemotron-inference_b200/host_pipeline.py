"""Running the layer over batches that live in HOST memory.

A caller that keeps its activations in pinned host memory pays two PCIe transfers per
batch.  Issued one after the other (upload, compute, download) they cost more than the
layer itself at prefill sizes; `HostPipeline` overlaps them instead: while batch i is
computed, batch i+1 is uploaded on a second stream and batch i-1 is downloaded on a third.
Device buffers are double-buffered per direction; CUDA events order every reuse, the host
never blocks in `submit`.

    pipe = HostPipeline(lambda x, out: layer.run_async(x, out), tokens, hidden)
    for x_host, out_host in batches:        # pinned tensors
        pipe.submit(x_host, out_host)
    pipe.drain()                            # all results are in their host tensors
"""
from __future__ import annotations

from typing import Callable, List

import torch


class HostPipeline:
    def __init__(self, run: Callable[[torch.Tensor, torch.Tensor], None], tokens: int, hidden: int,
                 in_dtype: torch.dtype = torch.bfloat16, out_dtype: torch.dtype = torch.bfloat16,
                 depth: int = 2, device=None):
        """`run(x, out)` launches one layer pass on the current stream (it must not
        synchronise).  `depth` batches can be in flight."""
        if depth < 1:
            raise ValueError("depth must be at least 1")
        device = device or torch.device("cuda", torch.cuda.current_device())
        self._run = run
        self._depth = depth
        self._x: List[torch.Tensor] = [torch.empty((tokens, hidden), dtype=in_dtype, device=device)
                                       for _ in range(depth)]
        self._out: List[torch.Tensor] = [torch.empty((tokens, hidden), dtype=out_dtype,
                                                     device=device) for _ in range(depth)]
        self._upload_stream = torch.cuda.Stream(device=device)
        self._download_stream = torch.cuda.Stream(device=device)
        self._uploaded = [torch.cuda.Event() for _ in range(depth)]
        self._computed = [torch.cuda.Event() for _ in range(depth)]
        self._downloaded = [torch.cuda.Event() for _ in range(depth)]
        self._count = 0
        self.h2d_bytes_per_batch = self._x[0].numel() * self._x[0].element_size()
        self.d2h_bytes_per_batch = self._out[0].numel() * self._out[0].element_size()

    def start_after(self, event: torch.cuda.Event) -> None:
        """No upload starts before `event` (used to put a timing mark in front of the pipe)."""
        self._upload_stream.wait_event(event)

    def submit(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Queues one batch: upload x_host, run the layer, download into out_host."""
        if not (x_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("host tensors must be pinned: pageable copies would block the host")
        rows = x_host.shape[0]
        slot = self._count % self._depth
        compute = torch.cuda.current_stream()
        x, out = self._x[slot][:rows], self._out[slot][:rows]
        with torch.cuda.stream(self._upload_stream):
            if self._count >= self._depth:
                # the batch that used this slot before must have been computed
                self._upload_stream.wait_event(self._computed[slot])
            x.copy_(x_host, non_blocking=True)
            self._uploaded[slot].record()
        compute.wait_event(self._uploaded[slot])
        if self._count >= self._depth:
            compute.wait_event(self._downloaded[slot])  # its result has left the device
        self._run(x, out)
        self._computed[slot].record(compute)
        with torch.cuda.stream(self._download_stream):
            self._download_stream.wait_event(self._computed[slot])
            out_host.copy_(out, non_blocking=True)
            self._downloaded[slot].record()
        self._count += 1

    def drain(self) -> None:
        """Makes the current stream wait for every queued download (does not block the host)."""
        compute = torch.cuda.current_stream()
        for slot in range(min(self._count, self._depth)):
            compute.wait_event(self._downloaded[slot])

    def synchronize(self) -> None:
        self.drain()
        torch.cuda.current_stream().synchronize()
