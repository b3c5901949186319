"""The CUDA backend against the reference's golden vectors and known answers, through the graph
C ABI (so routing, aliases and fusion are on the path)."""
import numpy as np
import pytest

from conftest import assert_close
from golden_cases import layernorm_property_case, load_golden, reference_kats
from test_oracle_golden import BITEXACT

pytestmark = pytest.mark.gpu
GOLDEN = load_golden()
KATS = reference_kats()


def run(backend, descs, weights, inputs, out_n):
    m = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan({k: (v.size, False) for k, v in inputs.items()}, 1)
    y = m.forward({k: (v, False) for k, v in inputs.items()}, 1, out_n)
    m.close()
    return y.ravel()


@pytest.mark.parametrize("case", GOLDEN, ids=[g[0] for g in GOLDEN])
def test_backend_matches_golden_vectors(backend, case):
    name, descs, weights, inputs, want = case
    got = run(backend, descs, weights, inputs, want.size)
    if name in BITEXACT:
        assert np.array_equal(got, want), name
    else:
        assert_close(got, want, name)


@pytest.mark.parametrize("case", KATS, ids=[k[0] for k in KATS])
def test_backend_reproduces_reference_known_answers(backend, case):
    name, descs, weights, inputs, want, atol = case
    got = run(backend, descs, weights, inputs, want.size)
    np.testing.assert_allclose(got, want, atol=max(atol, 2e-6), rtol=0, err_msg=name)


def test_backend_layernorm_mean_variance_property(backend):
    descs, weights, inputs = layernorm_property_case()
    out = run(backend, descs, weights, inputs, 4)
    assert abs(out.mean()) < 1e-5 and abs(out.var() - 1.0) < 1e-4
