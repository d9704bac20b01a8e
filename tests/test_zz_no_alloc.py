"""The allocation-free scan entry point against the regular one.

k2j_exclusive_scan_u32_noalloc exists for hosts that cannot let a library allocate device memory
(profiler callbacks during context teardown, processes whose memory belongs to a caching allocator).
It keeps its scratch in a fixed array inside the library and all calls share that array, so the test
runs it twice in a row, on different inputs, and each time compares with k2j_exclusive_scan_u32, whose
scratch comes from the context's workspace.  Integer work: the results must be identical.  The file
name sorts last so a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _both(ctx, lib, sizes_np):
    import torch
    n = len(sizes_np)
    d_sizes = torch.from_numpy(sizes_np).cuda()
    ref_off = torch.empty(n, dtype=torch.int64, device="cuda")
    ref_total = ctx.exclusive_scan(d_sizes, ref_off)
    new_off = torch.full((n,), -1, dtype=torch.int64, device="cuda")
    new_total = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    st = lib.k2j_exclusive_scan_u32_noalloc(0, C.c_void_p(stream), d_sizes.data_ptr(), n, new_off.data_ptr(),
                                            new_total.data_ptr())
    assert st == 0
    torch.cuda.synchronize()
    assert int(new_total.item()) == ref_total
    assert torch.equal(new_off, ref_off)
    want = np.concatenate([[0], np.cumsum(sizes_np.astype(np.int64))])
    assert ref_total == want[-1] and (new_off.cpu().numpy() == want[:-1]).all()


def test_noalloc_scan_matches_regular_scan_twice_in_a_row():
    from kineto_b200 import api
    lib = api.load_library()
    ctx = api.K2J(0)
    try:
        rng = np.random.default_rng(7)
        first = rng.integers(0, 3000, 1_300_007).astype(np.int32)
        second = rng.integers(0, 90000, 4_099).astype(np.int32)   # shorter: leftovers of the first call stay in the scratch
        _both(ctx, lib, first)
        _both(ctx, lib, second)
    finally:
        ctx.close()


def test_noalloc_scan_rejects_oversized_input():
    import torch
    from kineto_b200 import api
    lib = api.load_library()
    dummy = torch.zeros(8, dtype=torch.int64, device="cuda")
    st = lib.k2j_exclusive_scan_u32_noalloc(0, None, dummy.data_ptr(), (1 << 24) + 1, dummy.data_ptr(), dummy.data_ptr())
    assert st == 1   # K2J_ERR_INVALID_ARGUMENT: larger than the fixed scratch allows
