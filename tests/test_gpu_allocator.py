"""The RuntimeAllocator verbs on the device, through the C ABI (RuntimeAllocator.hpp:176-310).

The reference's allocator hands out zero-filled tensors and raw buffers that a MemoryGuard has agreed to, keeps a pool of
scratchpads by tag, and counts what it gave out.  The same verbs over HBM: what they hand out is usable by the
device-pointer entry points, the guard sees every byte, and a refusal is an error code, never an allocation.
"""
import numpy as np
import pytest

from mimir_framework_b200 import abi

pytestmark = pytest.mark.gpu


def _to_host(backend, ptr, n):
    """Copies n floats at device address ptr back with the library's own element-wise entry point (y = relu(x) leaves
    non-negative data unchanged) into a torch tensor."""
    import torch

    y = torch.full((n,), float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    backend.check(backend.lib().mimir_b200_dev_eltwise(abi.ELT_RELU, ptr, None, y.data_ptr(), 1, n, 0, stream))
    torch.cuda.synchronize()
    return y.cpu().numpy()


def test_tensor_alloc_is_zero_filled_counted_and_released(backend):
    before = backend.guard_stats()["current"]
    s0 = backend.allocator_stats()
    ptr, nbytes = backend.tensor_alloc([3, 5, 7], "t0")
    assert nbytes == 3 * 5 * 7 * 4 and ptr % 256 == 0
    assert backend.guard_stats()["current"] == before + nbytes
    s1 = backend.allocator_stats()
    assert s1["num_allocations"] == s0["num_allocations"] + 1 and s1["total_allocated"] == s0["total_allocated"] + nbytes
    np.testing.assert_array_equal(_to_host(backend, ptr, 105), np.zeros(105, np.float32))  # std::vector<float>(numel, 0.0f)
    backend.buffer_free(ptr)
    assert backend.guard_stats()["current"] == before
    with pytest.raises(backend.MimirB200Error) as e:
        backend.buffer_free(ptr)  # not handed out any more
    assert e.value.status == abi.E_INVALID
    for bad in ([4, 0], [-1], [1 << 30, 1 << 30, 1 << 30]):
        with pytest.raises(backend.MimirB200Error) as e:
            backend.tensor_alloc(bad, "bad")
        assert e.value.status == abi.E_INVALID


def test_allocated_tensor_feeds_a_device_entry_point(backend):
    """A LayerNorm between two tensors of the allocator, checked against the oracle."""
    import torch
    from oracle import port
    from conftest import assert_close

    rows, n = 6, 1024
    x = np.random.default_rng(2).standard_normal(rows * n).astype(np.float32)
    px, _ = backend.tensor_alloc([rows, n], "x")
    py, _ = backend.tensor_alloc([rows, n], "y")
    try:
        src = torch.from_numpy(x).cuda()
        stream = torch.cuda.current_stream().cuda_stream
        lib = backend.lib()
        # copy into the allocator's tensor with the element-wise entry point (x + 0 of the zero-filled tensor itself)
        backend.check(lib.mimir_b200_dev_eltwise(abi.ELT_ADD, src.data_ptr(), px, px, 1, rows * n, rows * n, stream))
        backend.check(lib.mimir_b200_dev_layernorm(px, None, None, py, rows, n, 1e-5, stream))
        out = torch.empty(rows * n, device="cuda")
        backend.check(lib.mimir_b200_dev_eltwise(abi.ELT_ADD, py, px, out.data_ptr(), 1, rows * n, rows * n, stream))
        torch.cuda.synchronize()
        want = port.layernorm(x, None, None, rows, n, 1e-5) + x
        assert_close(out.cpu().numpy(), want, "layernorm between allocator tensors")
    finally:
        backend.buffer_free(px)
        backend.buffer_free(py)


def test_scratchpad_pool_reuses_by_tag(backend):
    p1, b1 = backend.scratchpad_get(1 << 20, "im2col")
    backend.scratchpad_return(p1)
    held = backend.guard_stats()["current"]
    p2, b2 = backend.scratchpad_get(1 << 19, "im2col")  # the pooled one is large enough: reused, nothing new
    assert p2 == p1 and b2 == b1 == 1 << 20 and backend.guard_stats()["current"] == held
    backend.scratchpad_return(p2)
    p3, b3 = backend.scratchpad_get(1 << 21, "im2col")  # too small: a new buffer, the small one stays pooled
    assert p3 != p1 and b3 == 1 << 21 and backend.guard_stats()["current"] == held + (1 << 21)
    p4, _ = backend.scratchpad_get(1 << 10, "other")  # another tag has its own slot
    assert p4 not in (p1, p3)
    backend.scratchpad_return(p3)  # the tag's slot is taken by the small one: this one is freed
    assert backend.guard_stats()["current"] == held + (1 << 10)
    backend.scratchpad_return(p4)
    pa, _ = backend.scratchpad_get(16, "im2col")
    pb, _ = backend.scratchpad_get(16, "other")
    assert pa == p1 and pb == p4
    backend.buffer_free(pa)
    backend.buffer_free(pb)
    with pytest.raises(backend.MimirB200Error):
        backend.scratchpad_return(pa)


def test_refusals_by_cap_limit_and_freeze_allocate_nothing(backend):
    lib = backend.lib()
    base = backend.guard_stats()
    try:
        backend.check(lib.mimir_b200_allocator_set_local_cap(base["current"] + (1 << 20)))
        with pytest.raises(backend.MimirB200Error) as e:
            backend.buffer_alloc(2 << 20, "over the cap")
        assert e.value.status == abi.E_OOM_BUDGET and "local cap" in str(e.value)
        p = backend.buffer_alloc(1 << 19, "under the cap")
        backend.buffer_free(p)
    finally:
        backend.check(lib.mimir_b200_allocator_set_local_cap(0))
    try:
        lib.mimir_b200_guard_freeze(1)
        with pytest.raises(backend.MimirB200Error) as e:
            backend.tensor_alloc([16], "frozen")
        assert e.value.status == abi.E_OOM_BUDGET and "frozen" in str(e.value)
    finally:
        lib.mimir_b200_guard_freeze(0)
    try:
        backend.check(lib.mimir_b200_guard_set_limit(base["current"] + (1 << 20)))
        with pytest.raises(backend.MimirB200Error) as e:
            backend.buffer_alloc(4 << 20, "over the limit")
        assert e.value.status == abi.E_OOM_BUDGET
    finally:
        backend.check(lib.mimir_b200_guard_set_limit(base["limit"]))
    assert backend.guard_stats()["current"] == base["current"]


def test_check_no_leaks_follows_the_ten_megabyte_rule(backend):
    """check_no_leaks (RuntimeAllocator.hpp:299-304) is `current < 10 MB` at the guard."""
    cur = backend.guard_stats()["current"]
    assert backend.allocator_check_no_leaks() == (cur // (1 << 20) < 10)
    p = backend.buffer_alloc(12 << 20, "big")
    assert backend.allocator_check_no_leaks() is False
    backend.buffer_free(p)
    assert backend.allocator_check_no_leaks() == (cur // (1 << 20) < 10)
