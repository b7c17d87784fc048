"""The allocation-free route sort (table inside the library image) against the ordinary entry point.

Runs last on purpose: if it fails under `-x`, every other test has already run.  It must pass on its own in a fresh
process and after the rest of the suite, and on two calls in a row (the shared table keeps the previous call's contents).
"""
import numpy as np
import pytest

from tests.util import require_cuda

pytestmark = pytest.mark.gpu


def _sort_both(lib, torch, ind, experts):
    routes = ind.numel()
    i32 = dict(dtype=torch.int32, device="cuda")

    def outputs():
        return [torch.full((experts,), -1, **i32), torch.full((experts + 1,), -1, **i32), torch.full((experts,), -1, **i32),
                torch.full((routes,), -1, **i32), torch.full((routes,), -1, **i32), torch.full((routes,), -1, **i32)]

    ref = outputs()
    scratch = torch.empty(max(1, lib.eider_b200_moe_sort_scratch_bytes(routes, experts)), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.eider_b200_moe_sort_routes_on_stream(ind.data_ptr(), *[t.data_ptr() for t in ref], routes, experts,
                                                  scratch.data_ptr(), scratch.numel(), stream)
    assert rc == 0
    got = outputs()
    rc = lib.eider_b200_moe_sort_routes_noalloc_on_stream(ind.data_ptr(), *[t.data_ptr() for t in got], routes, experts, stream)
    assert rc == 0
    torch.cuda.synchronize()
    return ref, got


def test_noalloc_sort_matches_scratch_sort_twice_in_a_row():
    torch = require_cuda()
    from eider_b200 import _lib
    lib = _lib.load()
    gen = torch.Generator(device="cuda").manual_seed(123)
    # two different problems back to back: the second must not see anything of the first in the shared table
    # (the last case fills the built-in table exactly: 256 chunks x 1024 experts = 262144 entries)
    for routes, experts in [(32768, 128), (5000, 60), (65536, 1024)]:
        ind = torch.randint(0, experts, (routes,), device="cuda", generator=gen, dtype=torch.int32)
        ref, got = _sort_both(lib, torch, ind, experts)
        for a, b in zip(ref, got):
            assert torch.equal(a, b)
        # and the result is a permutation grouped by expert
        sorted_experts = got[4].cpu().numpy()
        assert np.all(np.diff(sorted_experts) >= 0)


def test_noalloc_sort_rejects_what_does_not_fit():
    torch = require_cuda()
    from eider_b200 import _lib
    lib = _lib.load()
    limit = lib.eider_b200_moe_sort_noalloc_max_entries()
    experts = 1024
    routes = (limit // experts + 1) * 256  # one chunk too many for the built-in table
    t = torch.zeros(routes, dtype=torch.int32, device="cuda")
    small = torch.zeros(experts + 1, dtype=torch.int32, device="cuda")
    rc = lib.eider_b200_moe_sort_routes_noalloc_on_stream(t.data_ptr(), small.data_ptr(), small.data_ptr(), small.data_ptr(),
                                                          t.data_ptr(), t.data_ptr(), t.data_ptr(), routes, experts, None)
    assert rc == 1  # cudaErrorInvalidValue, before any launch
    assert lib.eider_b200_moe_sort_routes_noalloc_on_stream(None, None, None, None, None, None, None, 8, 4, None) == 1
