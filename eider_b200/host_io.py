"""Steps whose inputs come from and whose results go back to pinned host memory.

The reference's runtime hands the quantized-linear path host-resident activations only at the edges of a model (prompt
chunks in, logits out), but a caller that does drive single layers from the host pays PCIe for every step: at 512 tokens
the prefill GEMM reads 5 MB and returns 28 MB, 0.6 ms of copies around 0.04 ms of kernels.  `HostStreamer` keeps that
traffic off the critical path as far as PCIe allows: two sets of device buffers, the upload of step i + 1 and the download
of step i - 1 on their own streams (the two directions of the link are independent) while step i computes, events between
them, nothing blocking the host.  A step is then as long as its slowest leg instead of the sum of the three.
"""
from __future__ import annotations

from typing import Callable

import torch


class HostStreamer:
    """submit(x_host, compute, y_host) for step after step; drain() before the host reads the last results.

    `compute(x_dev) -> y_dev` runs on the current stream.  Its result is copied into a staging buffer of this object on
    the same stream before the download starts, so `compute` may return the same tensor (or memory that peers overwrite)
    every step.  `take(y_dev)` selects what is returned to the host (default: all of it); `y_host` must be pinned and
    have that shape.  Results of step i are complete in `y_host` once an event recorded after submit i + depth or after
    drain() has completed."""

    def __init__(self, in_shape, in_dtype, out_shape, out_dtype, depth: int = 2, device="cuda"):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.depth = depth
        self.copy_in = torch.cuda.Stream(device=device)
        self.copy_out = torch.cuda.Stream(device=device)
        self.x_dev = [torch.empty(in_shape, dtype=in_dtype, device=device) for _ in range(depth)]
        self.y_dev = [torch.empty(out_shape, dtype=out_dtype, device=device) for _ in range(depth)]
        mk = lambda: [torch.cuda.Event() for _ in range(depth)]
        self.uploaded, self.consumed, self.staged, self.downloaded = mk(), mk(), mk(), mk()
        self.step = 0
        self.h2d_bytes = self.x_dev[0].numel() * self.x_dev[0].element_size()
        self.d2h_bytes = self.y_dev[0].numel() * self.y_dev[0].element_size()

    def start_after(self, event: torch.cuda.Event) -> None:
        """Neither copy stream starts anything before `event` (e.g. the first event of a timed region)."""
        self.copy_in.wait_event(event)
        self.copy_out.wait_event(event)

    def submit(self, x_host: torch.Tensor, compute: Callable[[torch.Tensor], torch.Tensor], y_host: torch.Tensor,
               take: Callable[[torch.Tensor], torch.Tensor] = lambda y: y) -> None:
        if not (x_host.is_pinned() and y_host.is_pinned()):
            raise ValueError("host buffers must be pinned: pageable memory makes every copy synchronous")
        slot = self.step % self.depth
        recycled = self.step >= self.depth
        main = torch.cuda.current_stream()
        # upload: the slot's device input is free once the step that last used it has read it
        if recycled:
            self.copy_in.wait_event(self.consumed[slot])
        with torch.cuda.stream(self.copy_in):
            self.x_dev[slot].copy_(x_host, non_blocking=True)
            self.uploaded[slot].record()
        # compute, then stage the part that goes back (the staging buffer is free once its last download has finished)
        main.wait_event(self.uploaded[slot])
        y = compute(self.x_dev[slot])
        self.consumed[slot].record(main)
        if recycled:
            main.wait_event(self.downloaded[slot])
        self.y_dev[slot].copy_(take(y), non_blocking=True)
        self.staged[slot].record(main)
        # download
        self.copy_out.wait_event(self.staged[slot])
        with torch.cuda.stream(self.copy_out):
            y_host.copy_(self.y_dev[slot], non_blocking=True)
            self.downloaded[slot].record()
        self.step += 1

    def drain(self) -> None:
        """The current stream waits for every download issued so far (record an event after this to time the whole run)."""
        main = torch.cuda.current_stream()
        for slot in range(min(self.step, self.depth)):
            main.wait_event(self.downloaded[slot])
