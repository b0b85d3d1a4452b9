"""Run a device step on batches that live in pinned host memory, with the copies hidden behind compute.

A caller whose activations arrive from the host (a data-parallel trainer feeding one attention layer
per process, an offloaded KV/activation store) pays two PCIe transfers per step.  Issued on the
compute stream they serialise with the kernels.  ``HostPipeline`` keeps ``depth`` sets of device input
buffers and three streams: host-to-device copies of step i+1 and device-to-host copies of step i-1 run
while step i computes.  Every step still copies all of its inputs in and all of its results out.
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch


class HostPipeline:
    def __init__(self, step_fn: Callable[..., Sequence[torch.Tensor]], example_inputs: Sequence[torch.Tensor],
                 device: torch.device, depth: int = 2):
        """step_fn(*device_inputs) -> sequence of device tensors (the step's results).
        example_inputs: host tensors with the shapes and dtypes of one batch."""
        assert depth >= 1
        self.step_fn = step_fn
        self.device = device
        self.depth = depth
        self._in = [[torch.empty(t.shape, dtype=t.dtype, device=device) for t in example_inputs] for _ in range(depth)]
        self._h2d = torch.cuda.Stream(device)
        self._d2h = torch.cuda.Stream(device)
        self._copied_in = [torch.cuda.Event() for _ in range(depth)]     # slot's inputs are on the device
        self._computed = [torch.cuda.Event() for _ in range(depth)]      # slot's step finished (inputs free again)
        self._copied_out = [torch.cuda.Event() for _ in range(depth)]    # slot's results are on the host
        self._results: List[Sequence[torch.Tensor]] = [() for _ in range(depth)]
        self._n = 0

    def submit(self, host_inputs: Sequence[torch.Tensor], host_outputs: Sequence[torch.Tensor]) -> None:
        """Queue one step: host_inputs (pinned) -> device, step_fn, results -> host_outputs (pinned).
        Returns at once; call drain() before reading host_outputs."""
        s = self._n % self.depth
        main = torch.cuda.current_stream(self.device)
        if self._n >= self.depth:
            self._h2d.wait_event(self._computed[s])      # the slot's previous step no longer reads its inputs
        with torch.cuda.stream(self._h2d):
            for d, h in zip(self._in[s], host_inputs):
                d.copy_(h, non_blocking=True)
            self._copied_in[s].record(self._h2d)
        main.wait_event(self._copied_in[s])
        if self._n >= self.depth:
            # results of the slot's previous step are dropped below: their copy out must be done
            main.wait_event(self._copied_out[s])
        outs = self.step_fn(*self._in[s])
        self._computed[s].record(main)
        self._d2h.wait_event(self._computed[s])
        with torch.cuda.stream(self._d2h):
            for h, o in zip(host_outputs, outs):
                h.copy_(o, non_blocking=True)
            self._copied_out[s].record(self._d2h)
        self._results[s] = outs                           # keep the device results alive until copied out
        self._n += 1

    def drain(self) -> None:
        """Make the current stream wait for every queued copy, then wait for it on the host."""
        main = torch.cuda.current_stream(self.device)
        for s in range(min(self._n, self.depth)):
            main.wait_event(self._copied_out[s])
        main.synchronize()
        self._results = [() for _ in range(self.depth)]

    def join_stream(self) -> None:
        """Order the current stream after every queued copy without blocking the host (for event timing)."""
        main = torch.cuda.current_stream(self.device)
        for s in range(min(self._n, self.depth)):
            main.wait_event(self._copied_out[s])
