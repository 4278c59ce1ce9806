"""The workspace-free forward entry point, ht_forest_forward_static_f32.

It exists for callers that cannot allocate device memory where they call the library (and so
have no workspace to pass): its scratch is a fixed array inside the library.  The test calls it
through the C ABI twice in a row -- the second call finds the array as the first left it -- and
requires the output to equal that of ht_forest_forward_f32 bit for bit (the forward tests of
this suite compare exactly), on a shape the tile kernel takes and on one the any-shape kernel
takes.  It also checks that a problem too large for the array is refused, not truncated.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It does not depend on any other test having run.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import random_forest_inputs
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu


def dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


@pytest.mark.parametrize("kind,shape", [
    ("tree", (2048, 128, (), 64, 8, ())),      # shared-memory tile kernel
    ("fern", (1500, 300, (), 40, 6, ())),      # tile kernel, 16-bit compact feature indices
    ("tree", (37, 20, (3,), 9, 4, (2,))),      # any-shape kernel (image-shaped input, 2 outputs per leaf)
])
def test_static_scratch_forward_matches_workspace_forward(kind, shape):
    from hingetreefortorch_b200 import _cabi
    B, C, inner, T, depth, extra = shape
    memory_before = None
    results = []
    for call in range(2):
        x, thr, ord_, w = random_forest_inputs(100 + call, kind, B, C, inner, T, depth, extra)
        dx, dthr, dord, dw = dev(x, thr, ord_, w)
        forest = _cabi.Forest(kind, dx, dw)
        want = forest.forward(dx, dthr, dord, dw)
        out = torch.empty_like(want)
        torch.cuda.synchronize()
        if memory_before is None:
            forest.forward_static(dx, dthr, dord, dw, out=torch.empty_like(want))  # first call: address look-up
            torch.cuda.synchronize()
        # nothing allocated, neither through torch's caching allocator nor behind its back (free device
        # memory as the driver reports it stays where it was)
        memory_before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        got = forest.forward_static(dx, dthr, dord, dw, out=out)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == memory_before
        assert torch.cuda.mem_get_info()[0] == free_before
        assert np.array_equal(got.cpu().numpy(), ho.forward(kind, x, thr, ord_, w))
        assert forest.ordinal_flags() == 0
        assert torch.equal(got, want), "call %d differs from ht_forest_forward_f32" % call
        results.append(got)
    assert not torch.equal(results[0], results[1])  # the two calls really had different inputs


def test_problem_larger_than_the_static_scratch_is_refused():
    from hingetreefortorch_b200 import _cabi
    lib = _cabi.library()
    limit = lib.ht_forest_static_scratch_bytes()
    assert limit >= 1 << 20
    # 8192 trees of depth 10 need far more than the array holds
    problem = _cabi.ForestProblem(0, 10, 64, 128, 1, 8192, 1, 0, 0)
    assert lib.ht_forest_workspace_bytes(ctypes.byref(problem)) > limit
    x = torch.zeros(64, 128, device="cuda")
    rc = lib.ht_forest_forward_static_f32(ctypes.byref(problem), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()),
                                          ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()),
                                          ctypes.c_void_p(x.data_ptr()), None, None)
    assert rc == -4
    assert b"workspace" in lib.ht_status_string(rc)
