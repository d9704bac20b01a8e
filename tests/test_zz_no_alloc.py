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
    torch.cuda.synchronize()  # the context scans on its own stream: its inputs must be complete first
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


@pytest.mark.parametrize("n", [0, 1, 2047, 2048, 2049, 5 * 2048, 1 << 24])
def test_noalloc_scan_at_the_edges_of_its_blocks_and_of_its_scratch(n):
    """Lengths around the 2048-element blocks the scratch holds one sum for, nothing at all, and the largest input
    the fixed scratch allows."""
    from kineto_b200 import api
    lib = api.load_library()
    ctx = api.K2J(0)
    try:
        _both(ctx, lib, np.random.default_rng(n).integers(0, 1000, n).astype(np.int32))
    finally:
        ctx.close()


def test_noalloc_scan_allocates_nothing_and_keeps_the_current_device():
    """After one warm-up call (the driver loads the kernels and the array on first use) further calls leave the
    amount of free device memory exactly where it was, and the caller's current device is untouched."""
    import torch
    from kineto_b200 import api
    lib = api.load_library()
    sizes = torch.randint(0, 1000, (300_000,), dtype=torch.int32, device="cuda")
    off = torch.empty(300_000, dtype=torch.int64, device="cuda")
    total = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call(n):
        assert lib.k2j_exclusive_scan_u32_noalloc(0, C.c_void_p(stream), sizes.data_ptr(), n, off.data_ptr(), total.data_ptr()) == 0
        torch.cuda.synchronize()

    call(1000)  # warm-up
    free0 = torch.cuda.mem_get_info()[0]
    dev0 = torch.cuda.current_device()
    call(300_000)
    call(0)
    call(77)
    assert torch.cuda.mem_get_info()[0] == free0
    assert torch.cuda.current_device() == dev0
    assert int(total.item()) == int(sizes[:77].sum().item())


def test_noalloc_scan_rejects_oversized_input():
    import torch
    from kineto_b200 import api
    lib = api.load_library()
    dummy = torch.zeros(8, dtype=torch.int64, device="cuda")
    st = lib.k2j_exclusive_scan_u32_noalloc(0, None, dummy.data_ptr(), (1 << 24) + 1, dummy.data_ptr(), dummy.data_ptr())
    assert st == 1   # K2J_ERR_INVALID_ARGUMENT: larger than the fixed scratch allows
