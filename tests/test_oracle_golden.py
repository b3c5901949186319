"""Pins the plain-C oracle (oracle/mimir_oracle.c through oracle/port.py) before it is trusted:
  1. against every known-answer test the reference's own test-suite holds for the path;
  2. against golden vectors produced by the compiled reference (tests/golden/make_golden.py);
  3. where the compiled reference is present, that it still reproduces the committed vectors.
CPU only."""
import numpy as np
import pytest

from golden_cases import layernorm_property_case, load_golden, reference_kats
from oracle import port, ref

GOLDEN = load_golden()
KATS = reference_kats()
# integer / index / pure data-movement cases must be bit-exact
BITEXACT = {"embedding_pad_oob_round", "upsample_nearest", "permute_201", "concat3", "relu", "add_broadcast", "add_scalar", "multiply",
            "split_concat", "chunk_concat", "maxpool_k3s2p1", "zeropad2d", "reflectionpad2d", "replicationpad2d", "pixel_shuffle_r2",
            "leaky_relu_02", "subtract", "transpose_2d", "reparameterize_inference", "squeeze_unsqueeze", "stack2",
            "embedding_bag_offsets", "embedding_bag_unsorted_offsets", "embedding_bag_single_bag", "maxpool1d_k3s2p1",
            "maxpool1d_default_stride", "maxpool1d_k4s1p3"}


@pytest.mark.parametrize("case", KATS, ids=[k[0] for k in KATS])
def test_port_reproduces_reference_known_answers(case):
    name, descs, weights, inputs, want, atol = case
    got = port.run_graph(descs, weights, inputs)
    assert got.shape == want.shape
    np.testing.assert_allclose(got, want, atol=atol, rtol=0)


def test_port_layernorm_mean_variance_property():
    descs, weights, inputs = layernorm_property_case()
    out = port.run_graph(descs, weights, inputs)
    assert abs(out.mean()) < 1e-5 and abs(out.var() - 1.0) < 1e-4


@pytest.mark.parametrize("case", GOLDEN, ids=[g[0] for g in GOLDEN])
def test_port_matches_golden_vectors(case):
    name, descs, weights, inputs, want = case
    got = port.run_graph(descs, weights, inputs)
    assert got.shape == want.shape
    if name in BITEXACT:
        assert np.array_equal(got, want), name
    else:
        # the restatement sums in a slightly different order than the AVX2/OpenMP build: a few ulp
        np.testing.assert_allclose(got, want, atol=5e-6, rtol=2e-5, err_msg=name)


def test_port_error_behaviour():
    from mimir_framework_b200.abi import make_desc
    x = np.ones(10, np.float32)
    with pytest.raises(RuntimeError, match="Missing input tensor"):
        port.run_graph([make_desc("a", "Add", inputs=["x", "nope"])], [None], {"x": x})
    with pytest.raises(RuntimeError):  # "Add: input sizes must match or be broadcastable"
        port.run_graph([make_desc("a", "Add", inputs=["x", "b"])], [None], {"x": x, "b": np.ones(3, np.float32)})


@pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not built here")
@pytest.mark.parametrize("case", GOLDEN[:12] + GOLDEN[-2:], ids=[g[0] for g in GOLDEN[:12] + GOLDEN[-2:]])
def test_compiled_reference_reproduces_committed_vectors(case):
    name, descs, weights, inputs, want = case
    m = ref.RefModel(descs)
    for i, w in enumerate(weights):
        if w is not None:
            m.set_weights(i, w)
    if descs[0].type == b"MaxPool1d":
        # the reference's layer switch has no case for it: the layer throws, its function is reached directly
        with pytest.raises(RuntimeError, match="UNKNOWN"):
            m.forward(inputs)
        d = descs[0]
        assert np.array_equal(ref.maxpool1d(inputs["x"], d.in_channels, d.raw_kernel_h, d.raw_stride_h, d.raw_pad_h), want), name
        return
    assert np.array_equal(m.forward(inputs), want), name


@pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not built here")
def test_compiled_reference_passes_its_own_known_answers():
    for name, descs, weights, inputs, want, atol in KATS:
        m = ref.RefModel(descs)
        for i, w in enumerate(weights):
            if w is not None:
                m.set_weights(i, w)
        np.testing.assert_allclose(m.forward(inputs), want, atol=max(atol, 1e-7), rtol=0, err_msg=name)


@pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not built here")
def test_port_of_the_legacy_static_ops_matches_the_compiled_reference():
    """Model::computeAttention and Model::computeBatchNorm (software branch) against their plain-C restatements."""
    r = np.random.default_rng(3)
    for seq, d_model, heads in [(5, 8, 2), (33, 48, 3), (64, 64, 1)]:
        q, k, v = (r.standard_normal(seq * d_model).astype(np.float32) for _ in range(3))
        np.testing.assert_allclose(port.attention_qkv(q, k, v, seq, d_model, heads), ref.compute_attention(q, k, v, seq, d_model, heads),
                                   atol=2e-6, rtol=1e-5)
    for batch, ch, spatial in [(1, 1, 1), (3, 5, 17), (2, 16, 64)]:
        x = (r.standard_normal(batch * ch * spatial) * 2).astype(np.float32)
        g, b, m = (r.standard_normal(ch).astype(np.float32) for _ in range(3))
        var = (r.random(ch) + 0.05).astype(np.float32)
        np.testing.assert_allclose(port.batchnorm_running(x, g, b, m, var, batch, ch, spatial, 1e-5),
                                   ref.compute_batchnorm(x, g, b, m, var, batch, ch, spatial, 1e-5), atol=1e-6, rtol=1e-6)


@pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not built here")
def test_port_of_the_static_conv_family_matches_the_compiled_reference():
    """Model::computeConv2D (bias, dilation), computeConvTranspose2D (scatter form), computeBatchNorm with training = true and
    computeActivation("elu") against their plain-C restatements."""
    r = np.random.default_rng(11)
    for ic, oc, h, wd, k, st, pad, dil, bias in [(3, 5, 9, 11, 3, 1, 1, 1, True), (2, 4, 12, 10, 3, 2, 2, 2, True), (4, 3, 7, 7, 1, 1, 0, 1, False),
                                                  (1, 2, 15, 13, 5, 3, 4, 3, True), (2, 2, 20, 20, 9, 1, 4, 1, False)]:
        x = r.standard_normal(ic * h * wd).astype(np.float32)
        w = (r.standard_normal(oc * ic * k * k) * 0.3).astype(np.float32)
        b = r.standard_normal(oc).astype(np.float32) if bias else None
        # the compiled reference is an AVX2 build: its Conv::conv2d counts every remainder tap eight times (Layers.hpp:658-666)
        want = ref.compute_conv2d(x, w, b, h, wd, ic, oc, k, st, pad, dil)
        got = port.conv2d_dilated(x, w, b, ic, oc, h, wd, k, st, pad, dil, avx2_lanes=True)
        assert got.shape == want.shape
        np.testing.assert_allclose(got, want, atol=5e-5, rtol=5e-5)
        if k < 8:  # then every tap is a remainder tap: 8 x the scalar branch's sum, plus the bias
            scalar = port.conv2d_dilated(x, w, b, ic, oc, h, wd, k, st, pad, dil)
            bb = np.repeat(b, scalar.size // oc) if b is not None else 0.0
            np.testing.assert_allclose(8.0 * (scalar - bb) + bb, want, atol=5e-5, rtol=5e-5)
    for ic, oc, h, wd, k, st, pad, bias in [(3, 4, 5, 6, 4, 2, 1, True), (2, 3, 7, 5, 3, 1, 0, False), (1, 2, 4, 4, 2, 3, 0, True), (4, 2, 6, 6, 3, 2, 2, True)]:
        x = r.standard_normal(ic * h * wd).astype(np.float32)
        w = (r.standard_normal(oc * ic * k * k) * 0.3).astype(np.float32)
        b = r.standard_normal(oc).astype(np.float32) if bias else None
        want = ref.compute_conv2d(x, w, b, h, wd, ic, oc, k, st, pad, transposed=True)
        got = port.conv_transpose2d_scatter(x, w, b, ic, oc, h, wd, k, st, pad)
        assert got.shape == want.shape
        np.testing.assert_allclose(got, want, atol=5e-6, rtol=2e-5)
    for batch, ch, spatial in [(1, 1, 2), (3, 5, 17), (4, 16, 64)]:
        x = (r.standard_normal(batch * ch * spatial) * 2 + 0.5).astype(np.float32)
        g, b = (r.standard_normal(ch).astype(np.float32) for _ in range(2))
        np.testing.assert_allclose(port.batchnorm_batchstats(x, g, b, batch, ch, spatial, 1e-5),
                                   ref.compute_batchnorm_training(x, g, b, batch, ch, spatial, 1e-5), atol=2e-6, rtol=2e-6)
    x = (r.standard_normal(300) * 3).astype(np.float32)
    np.testing.assert_allclose(port.elu(x, 1.3), ref.compute_activation("elu", x, 1.3), atol=1e-6, rtol=1e-6)
    assert np.array_equal(ref.compute_activation("no_such_activation", x), x)  # an unknown name leaves the data alone


def test_operand_rounding_restatement_on_cpu_values():
    """The rounding the checker applies: nearest-even to 8 (bf16) or 11 (half) significant bits; weights through the
    power-of-two scale."""
    x = np.array([1.0, 1.00390625, 1.01171875, 3.14159, -2.71828e-5, 0.0], np.float32)
    b = port.OperandRounding("bf16").act(x)
    assert np.array_equal(b, np.array([1.0, 1.0, 1.015625, 3.140625, -2.7179718e-05, 0.0], np.float32))
    h = port.OperandRounding("f16").act(x)
    assert np.array_equal(h[:3], x[:3]) and h[3] == np.float32(3.140625)
    w = port.OperandRounding("f16").weight(x * np.float32(1e-6))  # far below half's normal range without the scale
    np.testing.assert_allclose(w, x * np.float32(1e-6), rtol=2.0 ** -11)
