"""One process, several GPUs: a replica per device, the batch cut into per-device slices, one host thread each,
every slice copied into its place in ONE pinned host buffer.  Runs on however many devices are visible (one is
enough to exercise the path; with two or more the slices really run on different GPUs).  The failure test injects
the failure on the host, before anything is launched on that rank."""
import numpy as np
import pytest

from conftest import assert_close
from mimir_framework_b200 import abi, configs
from oracle import port

pytestmark = pytest.mark.gpu


def _graph():
    cfg = dict(seq_len=16, d_model=64, vocab_size=200, num_layers=1, num_heads=2, mlp_hidden=96, output_dim=48)
    descs = configs.transformer_encoder(**cfg)
    weights = configs.seeded_weights(descs, seed=4, std=0.05)
    return cfg, descs, weights


@pytest.mark.parametrize("batch", [12, 5])
def test_replicas_gather_into_one_host_buffer_equals_a_single_model(backend, batch):
    import torch

    cfg, descs, weights = _graph()
    n_dev = min(torch.cuda.device_count(), 4)
    r = np.random.default_rng(batch)
    ids = r.integers(1, 200, (batch, 16)).astype(np.float32)
    mag, mod = (r.standard_normal(64) * 0.02).astype(np.float32), (r.standard_normal(64) * 0.02).astype(np.float32)
    spec = {"x": (16, False), "mag": (64, True), "mod": (64, True)}
    single = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        single.upload_weights(i, w)
    single.plan(spec, batch)
    want = single.forward({"x": (ids.ravel(), False), "mag": (mag, True), "mod": (mod, True)}, batch, 48)
    single.close()
    reps = backend.Replicas(list(range(n_dev)), descs, pipeline=2)
    for i, w in enumerate(weights):
        reps.upload_weights(i, w)
    reps.plan(spec, batch)
    x_host = torch.from_numpy(ids).pin_memory()
    out = torch.full((batch, 48), float("nan")).pin_memory()
    hspec = {"x": (x_host.data_ptr(), 16, False), "mag": (mag, 64, True), "mod": (mod, 64, True)}
    for _ in range(3):
        n = reps.forward_host_ptrs(hspec, batch, out.data_ptr(), out.numel())
        assert n == 48
        assert np.array_equal(out.numpy(), want), "the gathered buffer differs from the single-device forward"
    one = {k: (a if bc else a.reshape(batch, -1)[batch - 1]) for k, (a, bc) in {"x": (ids, False), "mag": (mag, True), "mod": (mod, True)}.items()}
    assert_close(out.numpy()[batch - 1], port.run_graph(descs, weights, one), "last sample vs oracle")
    # a host-injected failure on the last rank: reported by rank, the others finish, the next call works again
    bad = n_dev - 1
    reps.inject_failure(bad)
    with pytest.raises(backend.MimirB200Error) as e:
        reps.forward_host_ptrs(hspec, batch, out.data_ptr(), out.numel())
    assert f"replica {bad} (device {bad})" in str(e.value) and "injected failure" in str(e.value)
    out.fill_(float("nan"))
    reps.forward_host_ptrs(hspec, batch, out.data_ptr(), out.numel())
    assert np.array_equal(out.numpy(), want)
    reps.close()
    backend.init(0, 0)  # the session's device is current again for the tests that follow


def test_guard_block_and_freeze_refuse_a_plan_and_release_still_works(backend):
    """The device arena obeys the guard's switches (MemoryGuard.hpp:37-72): a plan made while allocations are frozen or
    blocked is refused before anything is launched; destroying a model (a release) still works; afterwards plans pass."""
    cfg, descs, weights = _graph()
    m = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    spec = {"x": (16, False), "mag": (64, True), "mod": (64, True)}
    lib = backend.lib()
    try:
        for verb, word in ((lib.mimir_b200_guard_freeze, "frozen"), (lib.mimir_b200_guard_block, "blocked")):
            verb(1)
            with pytest.raises(backend.MimirB200Error) as e:
                m.plan(spec, 4)
            assert e.value.status == abi.E_OOM_BUDGET and word in str(e.value)
            verb(0)
        before = backend.guard_stats()["current"]
        lib.mimir_b200_guard_freeze(1)
        m.close()  # releases stay possible
        assert backend.guard_stats()["current"] < before
    finally:
        lib.mimir_b200_guard_freeze(0)
        lib.mimir_b200_guard_block(0)
    m2 = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        m2.upload_weights(i, w)
    assert m2.plan(spec, 4) > 0
    m2.close()
