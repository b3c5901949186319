"""Host-side logic of the C ABI that needs no GPU: the budget guard's verbs (the reference's own known-answer test
replayed), the batch slicing of the replica entry points, and the fan-out / join that reports a failed rank."""
import ctypes as C

import pytest

from mimir_framework_b200 import abi, runtime as rt


def _guard():
    a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert rt.lib().mimir_b200_guard_stats(C.byref(a), C.byref(b), C.byref(c)) == abi.OK
    return a.value, b.value, c.value


def test_memory_guard_known_answers_of_the_reference():
    """Tests/test_memory_guard.cpp:6-29, verb for verb: reset, setLimit(100), 50 granted, 60 refused with the
    usage unchanged, release, freeze refuses, block refuses."""
    lib = rt.lib()
    old_limit = _guard()[0]
    try:
        assert lib.mimir_b200_guard_reset() == abi.OK
        assert lib.mimir_b200_guard_set_limit(100) == abi.OK
        assert _guard()[1] == 0
        assert lib.mimir_b200_guard_request(50, b"a") == abi.OK
        assert _guard()[1] == 50
        assert lib.mimir_b200_guard_request(60, b"b") == abi.E_OOM_BUDGET
        assert b"over the limit" in lib.mimir_b200_last_error()
        assert _guard()[1] == 50
        assert lib.mimir_b200_guard_release(50) == abi.OK
        assert _guard()[1] == 0
        # freeze mode blocks allocations
        assert lib.mimir_b200_guard_freeze(1) == abi.OK
        assert lib.mimir_b200_guard_request(1, b"freeze") == abi.E_OOM_BUDGET
        assert b"frozen" in lib.mimir_b200_last_error()
        assert lib.mimir_b200_guard_freeze(0) == abi.OK
        # block mode blocks allocations
        assert lib.mimir_b200_guard_block(1) == abi.OK
        assert lib.mimir_b200_guard_request(1, b"block") == abi.E_OOM_BUDGET
        assert b"blocked" in lib.mimir_b200_last_error()
        assert lib.mimir_b200_guard_block(0) == abi.OK
        blocked, frozen, nb, nf = C.c_int(), C.c_int(), C.c_size_t(), C.c_size_t()
        assert lib.mimir_b200_guard_state(C.byref(blocked), C.byref(frozen), C.byref(nb), C.byref(nf)) == abi.OK
        assert (blocked.value, frozen.value) == (0, 0) and nb.value >= 1 and nf.value >= 1
        # both switches set: "blocked" is reported first, as in MemoryGuard::requestAllocation
        lib.mimir_b200_guard_block(1)
        lib.mimir_b200_guard_freeze(1)
        assert lib.mimir_b200_guard_request(1, b"both") == abi.E_OOM_BUDGET
        assert b"blocked" in lib.mimir_b200_last_error()
        lib.mimir_b200_guard_block(0)
        lib.mimir_b200_guard_freeze(0)
        assert lib.mimir_b200_guard_request(1, b"ok") == abi.OK
        assert _guard()[2] == 50  # the peak survived the release
        assert lib.mimir_b200_guard_reset() == abi.OK
        assert _guard()[1:] == (0, 0)
    finally:
        lib.mimir_b200_guard_block(0)
        lib.mimir_b200_guard_freeze(0)
        lib.mimir_b200_guard_reset()
        lib.mimir_b200_guard_set_limit(old_limit)


def _shard(total, world, rank):
    b, e = C.c_longlong(), C.c_longlong()
    rt.check(rt.lib().mimir_b200_shard_range(total, world, rank, C.byref(b), C.byref(e)))
    return b.value, e.value


def test_shard_ranges_are_disjoint_cover_everything_and_differ_by_at_most_one():
    for total in (0, 1, 7, 8, 64, 65537):
        for world in (1, 2, 3, 8):
            r = [_shard(total, world, k) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == total
            assert all(r[k][1] == r[k + 1][0] for k in range(world - 1))
            sizes = [e - b for b, e in r]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    b, e = C.c_longlong(), C.c_longlong()
    assert rt.lib().mimir_b200_shard_range(10, 2, 2, C.byref(b), C.byref(e)) == abi.E_INVALID
    assert rt.lib().mimir_b200_shard_range(-1, 2, 0, C.byref(b), C.byref(e)) == abi.E_INVALID


def test_python_sharding_helper_agrees_with_the_library():
    from mimir_framework_b200 import sharding

    for total, world in ((65536, 8), (13, 4), (3, 8)):
        for k in range(world):
            assert sharding.shard_range(total, world, k) == _shard(total, world, k)


@pytest.mark.parametrize("ranks,bad", [(1, -1), (4, -1), (4, 2), (8, 0), (8, 7)])
def test_join_reports_a_failed_rank_by_rank_and_lets_the_others_finish(ranks, bad):
    status = rt.lib().mimir_b200_replicas_selftest_join(ranks, bad)
    if bad < 0:
        assert status == abi.OK
    else:
        assert status == abi.E_INVALID
        msg = rt.lib().mimir_b200_last_error().decode()
        assert f"replica {bad} (device {bad})" in msg and "injected failure" in msg
        assert all(f"replica {r} " not in msg for r in range(ranks) if r != bad)


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.mark.skipif(_has_gpu(), reason="checks the no-GPU failure mode")
def test_replicas_without_a_gpu_fail_loudly_and_name_the_rank():
    descs = abi.desc_array([abi.make_desc("l", "ReLU")])
    devs = (C.c_int * 2)(0, 1)
    h = C.c_void_p()
    status = rt.lib().mimir_b200_replicas_create(devs, 2, 0, C.addressof(descs), 1, abi.PREC_BF16X2, C.byref(h))
    assert status == abi.E_CUDA and not h.value
    msg = rt.lib().mimir_b200_last_error().decode()
    assert "replica 0 (device 0)" in msg and "no CUDA device" in msg
    dup = (C.c_int * 2)(3, 3)
    assert rt.lib().mimir_b200_replicas_create(dup, 2, 0, C.addressof(descs), 1, abi.PREC_BF16X2, C.byref(h)) == abi.E_INVALID


def _selection():
    on, dev, budget = C.c_int(-1), C.c_int(-1), C.c_size_t(1)
    assert rt.lib().mimir_b200_env_selection(C.byref(on), C.byref(dev), C.byref(budget)) == abi.OK
    return on.value, dev.value, budget.value


def test_selection_by_environment_follows_the_reference_flag_conventions(monkeypatch):
    """Model.cpp:704-722: a flag is true for any non-empty value other than "0"; an integer that does not parse keeps
    its default.  Default off."""
    for k in ("MIMIR_B200", "MIMIR_B200_DEVICE", "MIMIR_B200_HBM_BUDGET_MB"):
        monkeypatch.delenv(k, raising=False)
    assert _selection() == (0, 0, 0)
    for v, want in (("1", 1), ("0", 0), ("", 0), ("yes", 1), ("00", 1)):
        monkeypatch.setenv("MIMIR_B200", v)
        assert _selection()[0] == want, v
    monkeypatch.setenv("MIMIR_B200_DEVICE", "3")
    monkeypatch.setenv("MIMIR_B200_HBM_BUDGET_MB", "2048")
    assert _selection() == (1, 3, 2048 << 20)
    monkeypatch.setenv("MIMIR_B200_DEVICE", "abc")
    monkeypatch.setenv("MIMIR_B200_HBM_BUDGET_MB", "-5")
    assert _selection() == (1, 0, 0)
    # not selected: init_from_env touches nothing and reports "off"
    monkeypatch.setenv("MIMIR_B200", "0")
    on = C.c_int(7)
    assert rt.lib().mimir_b200_init_from_env(C.byref(on)) == abi.OK and on.value == 0


@pytest.mark.skipif(_has_gpu(), reason="checks the no-GPU failure mode")
def test_selected_without_a_gpu_is_an_error_not_a_fallback(monkeypatch):
    monkeypatch.setenv("MIMIR_B200", "1")
    on = C.c_int(7)
    assert rt.lib().mimir_b200_init_from_env(C.byref(on)) == abi.E_CUDA and on.value == 0
