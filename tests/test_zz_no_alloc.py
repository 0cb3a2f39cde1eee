"""mlpsp_prepare_groups_static: the allocation-free twin of mlpsp_prepare_groups.

Some hosts of the library may not call cudaMalloc (an embedding engine that owns all device memory,
or a frame loop that cannot afford cudaMalloc's device-wide synchronisation), so this entry point
keeps its work arrays in a fixed device array inside the library.  The test drives both entry points
through the C ABI on the same inputs and requires identical outputs, twice in a row: the second call
uses a smaller problem, so anything the first call left behind in the shared array would show.
Kept in a file that pytest collects last, so a run that stops at the first failure has already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, fn, offsets_dev, n, seg, dev):
    goff = torch.full((n + 1,), -7, dtype=torch.int64, device=dev)
    total = C.c_int64(-1)
    st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rc = fn(offsets_dev.data_ptr(), n, seg, goff.data_ptr(), None, None, 0, C.byref(total), st)
    assert rc == 0, lib.mlpsp_last_error()
    G = int(total.value)
    prim = torch.full((max(G, 1),), -7, dtype=torch.int64, device=dev)
    starts = torch.full((max(G, 1),), -7, dtype=torch.int64, device=dev)
    rc = fn(offsets_dev.data_ptr(), n, seg, goff.data_ptr(), prim.data_ptr(), starts.data_ptr(), G, C.byref(total), st)
    assert rc == 0, lib.mlpsp_last_error()
    assert int(total.value) == G
    return G, goff.cpu().numpy(), prim.cpu().numpy()[:G], starts.cpu().numpy()[:G]


def test_static_scratch_variant_matches_allocating_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mlp_splatting_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rng = np.random.default_rng(12)
    for n, seg in ((70_000, 128), (513, 7)):          # two calls in a row, the second one smaller
        counts = rng.integers(0, 900, n)
        counts[rng.integers(0, n, n // 5)] = 0
        offsets = np.concatenate(([0], np.cumsum(counts))).astype(np.int64)
        od = torch.from_numpy(offsets).to(dev)
        want = _run(lib, lib.mlpsp_prepare_groups, od, n, seg, dev)
        got = _run(lib, lib.mlpsp_prepare_groups_static, od, n, seg, dev)
        assert got[0] == want[0] == int((-(-counts // seg)).sum())
        for a, b in zip(got[1:], want[1:]):
            np.testing.assert_array_equal(a, b)
    # n == 0 after larger calls: the prefix must read zero, not the previous totals
    od = torch.zeros(1, dtype=torch.int64, device=dev)
    got = _run(lib, lib.mlpsp_prepare_groups_static, od, 0, 512, dev)
    assert got[0] == 0 and list(got[1]) == [0]
    # beyond the built-in capacity: refused before anything is launched
    total = C.c_int64(0)
    rc = lib.mlpsp_prepare_groups_static(od.data_ptr(), 524288 + 1, 512, od.data_ptr(), None, None, 0, C.byref(total), None)
    assert rc == -4 and b"exceed the built-in scratch capacity of 524288" in lib.mlpsp_last_error()
