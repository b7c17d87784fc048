"""Streaming steps between pinned host buffers and the device: every step's result comes back for that step's input,
whatever the overlap of uploads, kernels and downloads."""
import pytest

from tests.util import require_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("depth", [1, 2, 3])
def test_streamed_steps_return_their_own_results(depth):
    require_cuda()
    import torch
    from eider_b200 import host_io
    rows, cols, steps = 256, 4096, 9
    xs = [torch.full((rows, cols), float(i + 1), dtype=torch.bfloat16).pin_memory() for i in range(steps)]
    ys = [torch.zeros(rows // 2, cols, dtype=torch.float32).pin_memory() for _ in range(steps)]
    shared = torch.empty(rows, cols, dtype=torch.float32, device="cuda")  # one output buffer for every step, as a plan has

    def compute(x):
        torch.mul(x.float(), 3.0, out=shared)
        return shared

    streamer = host_io.HostStreamer((rows, cols), torch.bfloat16, (rows // 2, cols), torch.float32, depth=depth)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(steps):
            streamer.submit(xs[i], compute, ys[i], take=lambda y: y[rows // 2:])
        streamer.drain()
    stream.synchronize()
    for i in range(steps):
        assert torch.all(ys[i] == 3.0 * (i + 1)), i
    assert streamer.h2d_bytes == rows * cols * 2 and streamer.d2h_bytes == rows // 2 * cols * 4


def test_streamer_rejects_pageable_memory():
    require_cuda()
    import torch
    from eider_b200 import host_io
    streamer = host_io.HostStreamer((4, 4), torch.float32, (4, 4), torch.float32)
    with pytest.raises(ValueError):
        streamer.submit(torch.zeros(4, 4), lambda x: x, torch.zeros(4, 4).pin_memory())
