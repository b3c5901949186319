"""Every architecture of the reference's registry (ModelArchitectures.cpp), at a small width, through
the oracle's graph walk (CPU) and through the CUDA backend's graph path (GPU), against the output of
the compiled reference committed under tests/golden/registry_graphs.*."""
import json

import numpy as np
import pytest

import registry_cases as rc
from conftest import assert_close
from oracle import port, ref

GRAPHS = rc.load_registry_graphs()
IDS = [g[0] for g in GRAPHS]


def test_fixture_covers_the_whole_registry():
    assert sorted(IDS) == sorted(rc.CFG)
    types = {d.type.decode() for _, descs, _, _ in GRAPHS for d in descs}
    # the cases of the layer switch the registry graphs reach
    assert {"Linear", "Conv2d", "MultiHeadAttention", "CrossAttention", "Split", "DepthwiseConv2d", "LeakyReLU",
            "Reparameterize", "UpsampleNearest", "Concat", "Permute", "LayerNorm", "Embedding", "TokenMeanPool",
            "GlobalAvgPool2d"} <= types


@pytest.mark.parametrize("case", GRAPHS, ids=IDS)
def test_port_graph_walk_matches_reference_output(case):
    arch, descs, inputs, want = case
    got = port.run_graph(descs, rc.make_weights(descs), inputs)
    assert got.shape == want.shape
    scale = float(np.abs(want).max())
    np.testing.assert_allclose(got, want, atol=2e-5 * max(scale, 1.0), rtol=1e-4, err_msg=arch)


@pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not built here")
@pytest.mark.parametrize("arch", ["sd3_5", "mobilenet", "vae_conv", "ponyxl_ddpm"])
def test_compiled_reference_reproduces_registry_fixture(arch):
    _, descs, inputs, want = next(g for g in GRAPHS if g[0] == arch)
    m = ref.RefModel(registry=arch, cfg_json=json.dumps(rc.CFG[arch]))
    for i, w in enumerate(rc.make_weights(m.layer_descs())):
        if w is not None:
            m.set_weights(i, w)
    assert np.array_equal(m.forward(inputs), want)


@pytest.mark.gpu
@pytest.mark.parametrize("case", GRAPHS, ids=IDS)
def test_backend_runs_registry_graph(backend, case):
    arch, descs, inputs, want = case
    weights = rc.make_weights(descs)
    batch = 2
    second = rc.make_inputs(arch, seed=11)
    for k in inputs:  # inputs the reference derives itself (mag / mod) stay as they are
        if k not in second or second[k].shape != inputs[k].shape or k in ("mag", "mod"):
            second[k] = inputs[k]
    m = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan({k: (v.size, False) for k, v in inputs.items()}, batch)
    got = m.forward({k: (np.concatenate([inputs[k], second[k]]), False) for k in inputs}, batch, want.size).reshape(batch, -1)
    m.close()
    assert_close(got[0], want, arch)
    assert_close(got[1], port.run_graph(descs, weights, second), arch + " (second sample, against the oracle)")
