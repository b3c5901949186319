"""Incremental decoding with a key / value cache (mimir_b200_model_decode_*).

The reference has no cache: its answer for position t is row t of a full causal forward over tokens 0..t..S-1
(Model::forwardPass; for token-wise graphs that row depends on tokens 0..t only).  So the oracle for a decode
step is that row of the oracle's full forward, and the test walks a sequence token by token - from position 0,
and after a prefill of the first tokens through the model's ordinary forward.
"""
import numpy as np
import pytest

from mimir_framework_b200 import abi, configs
from mimir_framework_b200.abi import make_desc
from oracle import port

pytestmark = pytest.mark.gpu

V, E, H, F = 50, 64, 2, 96


def gpt(S, E=E, H=H):
    """Token-wise decoder: Embedding -> 2 x [LayerNorm -> causal attention -> Add -> LayerNorm -> Linear -> GELU ->
    Linear -> Add] -> LayerNorm -> Linear to the vocabulary."""
    d = [make_desc("emb", "Embedding", inputs=["x"], output="h", vocab_size=V, embed_dim=E, padding_idx=-1, seq_len=S, params_count=V * E)]
    for i in range(2):
        d += [
            make_desc(f"n1_{i}", "LayerNorm", inputs=["h"], output="a0", in_features=E, affine=1, use_bias=1, params_count=2 * E),
            make_desc(f"att_{i}", "MultiHeadAttention", inputs=["a0"], output="a1", seq_len=S, embed_dim=E, num_heads=H, causal=1, params_count=4 * E * E),
            make_desc(f"add1_{i}", "Add", inputs=["h", "a1"], output="r"),
            make_desc(f"n2_{i}", "LayerNorm", inputs=["r"], output="f0", in_features=E, affine=1, use_bias=1, params_count=2 * E),
            make_desc(f"fc1_{i}", "Linear", inputs=["f0"], output="f1", in_features=E, out_features=F, seq_len=S, params_count=E * F + F),
            make_desc(f"gelu_{i}", "GELU", inputs=["f1"], output="f2"),
            make_desc(f"fc2_{i}", "Linear", inputs=["f2"], output="f3", in_features=F, out_features=E, seq_len=S, params_count=F * E + E),
            make_desc(f"add2_{i}", "Add", inputs=["r", "f3"], output="h"),
        ]
    d += [make_desc("nf", "LayerNorm", inputs=["h"], output="hf", in_features=E, affine=1, use_bias=1, params_count=2 * E),
          make_desc("head", "Linear", inputs=["hf"], output="x", in_features=E, out_features=V, seq_len=S, params_count=E * V + V)]
    return d


def close(got, want, what):
    err = np.abs(got - want)
    assert np.all(err <= 1e-4 + 1e-3 * np.abs(want)), f"{what}: max abs error {err.max():.3e}"


# 20 rows per step leave the weight-streaming path for the tensor-core GEMM; 300 positions span three key chunks of
# the decode attention kernel
# head_dim 64 (E = 128) puts the prefill on the tensor-core attention core, whose cache-filling form lays fp32 QKV rows
# out per head instead of reading the projection's planes in place
@pytest.mark.parametrize("batch,S,P,E", [(2, 12, 7, 64), (20, 12, 7, 64), (3, 300, 292, 64), (2, 150, 140, 128)])
def test_decode_steps_reproduce_the_rows_of_the_full_causal_forward(backend, batch, S, P, E):
    full = gpt(S, E)
    weights = configs.seeded_weights(full, seed=3, std=0.08)
    ids = np.random.default_rng(batch).integers(0, V, (batch, S)).astype(np.float32)
    want = np.stack([port.run_graph(full, weights, {"x": ids[b]}).reshape(S, V) for b in range(batch)])  # [batch][S][V]

    # (1) from an empty cache, token by token; the model itself is planned for the full length
    m = backend.GraphModel(full)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan({"x": (S, False)}, batch)
    assert m.decode_begin({"x": (1, False)}, batch, S) == 2 * 2 * batch * S * E * 4
    for t in range(S):
        got = m.decode_step({"x": (ids[:, t].copy(), False)}, batch, t, V)
        if S <= 16 or t % 37 == 0 or t >= S - 3:
            close(got, want[:, t, :], f"decode from scratch, position {t}")
    m.decode_end()
    m.close()

    # (2) prefill of the first P tokens through the ordinary forward of a model built for P tokens, then steps
    pre = gpt(P, E)
    m = backend.GraphModel(pre)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan({"x": (P, False)}, batch)
    m.decode_begin({"x": (1, False)}, batch, S)
    first = m.forward({"x": (ids[:, :P].copy().ravel(), False)}, batch, P * V).reshape(batch, P, V)
    close(first, want[:, :P, :], "prefill rows")
    first_again = m.forward({"x": (ids[:, :P].copy().ravel(), False)}, batch, P * V).reshape(batch, P, V)  # replayed as a CUDA graph
    assert np.array_equal(first, first_again)
    for t in range(P, S):
        got = m.decode_step({"x": (ids[:, t].copy(), False)}, batch, t, V)
        close(got, want[:, t, :], f"decode after prefill, position {t}")
    with pytest.raises(backend.MimirB200Error, match="outside the cache"):
        m.decode_step({"x": (ids[:, 0].copy(), False)}, batch, S, V)
    m.plan({"x": (P, False)}, batch)  # a new plan invalidates the decode state
    with pytest.raises(backend.MimirB200Error, match="decode_begin again"):
        m.decode_step({"x": (ids[:, 0].copy(), False)}, batch, 0, V)
    m.close()


def test_decode_refuses_graphs_that_do_not_act_per_token(backend):
    S = 8
    cases = {
        "whole-sample RMSNorm": [make_desc("n", "RMSNorm", inputs=["x"], output="x", params_count=S * E)],
        "non-causal attention": [make_desc("a", "MultiHeadAttention", inputs=["x"], output="x", seq_len=S, embed_dim=E, num_heads=H, causal=0, params_count=4 * E * E)],
        "Linear over the flattened sequence": [make_desc("l", "Linear", inputs=["x"], output="x", in_features=S * E, out_features=E, params_count=S * E * E + E)],
    }
    for what, descs in cases.items():
        m = backend.GraphModel(descs)
        for i, w in enumerate(configs.seeded_weights(descs, seed=1)):
            m.upload_weights(i, w)
        m.plan({"x": (S * E, False)}, 2)
        with pytest.raises(backend.MimirB200Error, match="decode:"):
            m.decode_begin({"x": (E, False)}, 2, S)
        m.close()
