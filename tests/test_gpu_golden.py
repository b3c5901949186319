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


# The remaining switch cases with a batch: every sample is an independent reference forward.
BATCHED = ["cross_attention_causal0", "cross_attention_causal1", "split_concat", "chunk_concat", "depthwise_conv_s2_bias", "conv1d_s2_bias",
           "conv_transpose2d_relu", "maxpool_k3s2p1", "avgpool_k3s1p1", "zeropad2d", "reflectionpad2d", "replicationpad2d",
           "pixel_shuffle_r2", "upsamplebilinear", "upsamplebicubic", "matmul", "batch_matmul", "batchnorm_partial_weights",
           "instance_norm_affine", "leaky_relu_02", "mish", "divide_small_divisors", "transpose_2d",
           "embedding_bag_offsets", "embedding_bag_single_bag", "patch_embed", "bilinear_bias", "rnn_bias", "gru_bias", "lstm_bias",
           "maxpool1d_k3s2p1"]


@pytest.mark.parametrize("name", BATCHED)
def test_backend_batched_matches_port(backend, name):
    from oracle import port
    _, descs, weights, inputs, want = next(g for g in GOLDEN if g[0] == name)
    batch = 3
    rng = np.random.default_rng(7)
    samples = [{k: (v if s == 0 else rng.standard_normal(v.size).astype(np.float32)) for k, v in inputs.items()} for s in range(batch)]
    m = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan({k: (v.size, False) for k, v in inputs.items()}, batch)
    stacked = {k: (np.concatenate([s[k] for s in samples]), False) for k in inputs}
    got = m.forward(stacked, batch, want.size).reshape(batch, -1)
    m.close()
    for s in range(batch):
        ref_out = port.run_graph(descs, weights, samples[s])
        if name in BITEXACT:
            assert np.array_equal(got[s], ref_out), f"{name} sample {s}"
        else:
            assert_close(got[s], ref_out, f"{name} sample {s}")
