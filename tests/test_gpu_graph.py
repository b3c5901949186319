"""Whole-graph parity through the model C ABI (create / upload_weights / plan / forward) against the
CPU oracle walking the same descriptors, plus planner behaviour (budget refusal, name routing)."""
import json

import numpy as np
import pytest

from conftest import assert_close
from mimir_framework_b200 import abi, configs
from mimir_framework_b200.abi import make_desc
from oracle import port, ref

pytestmark = pytest.mark.gpu


def oracle_batch(descs, weights, inputs, batch):
    outs = []
    for s in range(batch):
        one = {k: (a if bc else a.reshape(batch, -1)[s]) for k, (a, bc) in inputs.items()}
        outs.append(port.run_graph(descs, weights, one))
    return np.stack(outs)


def gpu_batch(backend, descs, weights, inputs, batch, out_n, precision=abi.PREC_BF16X2):
    m = backend.GraphModel(descs, precision)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    spec = {k: ((a.size if bc else a.size // batch), bc) for k, (a, bc) in inputs.items()}
    m.plan(spec, batch)
    out = m.forward(inputs, batch, out_n)
    m.close()
    return out


@pytest.mark.parametrize("rows,k", [(300, 256), (1024, 512)])
def test_linear_gelu_stack(backend, rows, k):
    """Configuration 2 at reduced size: activation fused into the GEMM epilogue, hi/lo planes handed
    from one GEMM to the next."""
    descs = configs.linear_gelu_stack(rows, k)
    weights = configs.linear_gelu_stack_weights(k)
    x = configs.linear_gelu_stack_input(rows, k)
    want = port.run_graph(descs, weights, {"x": x.ravel()})
    got = gpu_batch(backend, descs, weights, {"x": (x.ravel(), False)}, 1, rows * k)
    assert_close(got, want, f"linear+gelu stack {rows}x{k}")
    if ref.available():
        m = ref.RefModel(descs)
        for i, w in enumerate(weights):
            if w is not None:
                m.set_weights(i, w)
        assert_close(got, m.forward({"x": x.ravel()}), "linear+gelu stack vs compiled reference")


def test_linear_gelu_stack_full_k_rows_subset(backend):
    """K = N = 4096 like the headline configuration, 2048 rows; the oracle is run on a seeded subset
    of rows (rows are independent)."""
    rows, k = 2048, 4096
    descs = configs.linear_gelu_stack(rows, k)
    weights = configs.linear_gelu_stack_weights(k)
    x = configs.linear_gelu_stack_input(rows, k)
    got = gpu_batch(backend, descs, weights, {"x": (x.ravel(), False)}, 1, rows * k).reshape(rows, k)
    pick = np.sort(np.random.default_rng(0).choice(rows, 48, replace=False))
    sub = configs.linear_gelu_stack(len(pick), k)
    want = port.run_graph(sub, weights, {"x": x[pick].ravel()}).reshape(len(pick), k)
    assert_close(got[pick], want, "linear+gelu stack K=4096")
    err = np.abs(got[pick] - want)
    bound = 1e-4 + 1e-3 * np.abs(want)
    assert float((err / bound).max()) < 0.8, f"margin to the tolerance too thin: {float((err / bound).max()):.2f}"


def test_transformer_encoder_registry_graph(backend):
    """Configuration 1: the registry transformer graph (small width so the oracle is quick), batch 3,
    ids with padding (id 0) and out-of-range entries, mag/mod broadcast inputs."""
    cfg = dict(seq_len=32, d_model=64, vocab_size=500, num_layers=2, num_heads=4, mlp_hidden=96, output_dim=40)
    descs = configs.transformer_encoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.05)
    r = np.random.default_rng(0)
    batch = 3
    ids = r.integers(0, 500, (batch, 32)).astype(np.float32)
    ids[0, 3] = 0
    ids[1, 5] = 777
    mag = (r.standard_normal(64) * 0.02).astype(np.float32)
    mod = (r.standard_normal(64) * 0.02).astype(np.float32)
    inputs = {"x": (ids.ravel(), False), "mag": (mag, True), "mod": (mod, True)}
    want = oracle_batch(descs, weights, inputs, batch)
    got = gpu_batch(backend, descs, weights, inputs, batch, 40)
    assert_close(got, want, "transformer encoder graph")
    if ref.available():
        # the same graph built by the reference's own registry must give the same descriptors
        m = ref.RefModel(registry="transformer", cfg_json=json.dumps(dict(cfg, causal=False)))
        rd = m.layer_descs()
        assert [d.type for d in rd] == [d.type for d in descs]
        assert [int(d.params_count) for d in rd] == [int(d.params_count) for d in descs]
        for i, w in enumerate(weights):
            if w is not None:
                m.set_weights(i, w)
        want_ref = np.stack([m.forward({"x": ids[s], "mag": mag, "mod": mod}) for s in range(batch)])
        assert_close(got, want_ref, "transformer encoder graph vs compiled reference")


def test_named_routing_and_missing_input(backend):
    # Tests/test_layers_named_routing.cpp:14-51: a+b -> sum, sum*c -> x; a missing input is an error
    descs = [make_desc("add", "Add", inputs=["a", "b"], output="sum"), make_desc("mul", "Multiply", inputs=["sum", "c"], output="x")]
    a, b, c = (np.array(v, np.float32) for v in ([1, 2, 3], [10, 20, 30], [2, 2, 2]))
    got = gpu_batch(backend, descs, [None, None], {"a": (a, False), "b": (b, False), "c": (c, False)}, 1, 3)
    assert np.array_equal(got.ravel(), (a + b) * c)
    m = backend.GraphModel(descs)
    with pytest.raises(backend.MimirB200Error, match="Missing input tensor"):
        m.plan({"a": (3, False), "b": (3, False)}, 1)
    m.close()


def test_unsupported_layer_type_is_an_error_not_a_fallback(backend):
    with pytest.raises(backend.MimirB200Error) as e:
        backend.GraphModel([make_desc("l", "Lambda")])  # throws in the reference's switch too (Model.cpp:5703-5709)
    assert e.value.status == abi.E_UNSUPPORTED


def test_budget_refusal_happens_at_plan_time(backend):
    # Tests/test_memory_guard.cpp:6-29 for the device arena: a plan above the limit is refused
    # before anything is launched, and the guard's counters are unchanged afterwards.
    descs = configs.linear_gelu_stack(4096, 256)
    m = backend.GraphModel(descs)
    for i, w in enumerate(configs.linear_gelu_stack_weights(256)):
        m.upload_weights(i, w)
    before = backend.guard_stats()
    launches = backend.stats()["kernels_launched"]
    backend.check(backend.lib().mimir_b200_guard_set_limit(before["current"] + (1 << 20)))
    try:
        with pytest.raises(backend.MimirB200Error) as e:
            m.plan({"x": (4096 * 256, False)}, 1)
        assert e.value.status == abi.E_OOM_BUDGET
        assert backend.stats()["kernels_launched"] == launches
        assert backend.guard_stats()["current"] == before["current"]
    finally:
        backend.check(backend.lib().mimir_b200_guard_set_limit(before["limit"]))
    m.plan({"x": (4096 * 256, False)}, 1)  # fits again
    m.close()


def test_arena_reuses_memory_after_last_consumer(backend):
    # a long chain of same-sized activations must not need one buffer per layer
    n, depth = 1 << 16, 24
    descs = []
    prev = "x"
    for i in range(depth):
        out = "x" if i == depth - 1 else f"t{i}"
        descs.append(make_desc(f"r{i}", "ReLU" if i % 2 else "Tanh", inputs=[prev], output=out))
        prev = out
    m = backend.GraphModel(descs)
    peak = m.plan({"x": (n, False)}, 4)
    assert peak <= 3 * 4 * n * 4 + 4096, peak
    x = np.random.default_rng(0).standard_normal((4, n)).astype(np.float32)
    got = m.forward({"x": (x.ravel(), False)}, 4, n)
    want = x.copy()
    for i in range(depth):
        want = np.maximum(want, 0) if i % 2 else np.tanh(want)
    assert_close(got, want, "relu/tanh chain", abs_tol=1e-6, rel_tol=1e-5)
    m.close()


def test_conv_groupnorm_silu_residual_block(backend):
    """One block of configuration 4: Conv3x3 -> GroupNorm(32) -> SiLU -> Add(skip 1x1 conv)."""
    ic, oc, hw, batch = 64, 128, 12, 2
    descs = [
        make_desc("conv", "Conv2d", inputs=["x"], output="c", in_channels=ic, out_channels=oc, input_height=hw, input_width=hw,
                  kernel=3, stride=1, padding=1, params_count=oc * ic * 9),
        make_desc("gn", "GroupNorm", inputs=["c"], output="g", in_channels=oc, input_height=hw, input_width=hw, num_groups=32,
                  params_count=2 * oc),
        make_desc("act", "SiLU", inputs=["g"], output="a"),
        make_desc("skip", "Conv2d", inputs=["__input__"], output="s", in_channels=ic, out_channels=oc, input_height=hw,
                  input_width=hw, kernel=1, stride=1, padding=0, params_count=oc * ic),
        make_desc("add", "Add", inputs=["a", "s"], output="x"),
    ]
    r = np.random.default_rng(2)
    weights = [(r.standard_normal(oc * ic * 9) * np.sqrt(2 / (ic * 9))).astype(np.float32),
               np.concatenate([np.ones(oc), np.zeros(oc)]).astype(np.float32), None,
               (r.standard_normal(oc * ic) * np.sqrt(2 / ic)).astype(np.float32), None]
    x = r.random((batch, ic * hw * hw)).astype(np.float32)
    inputs = {"x": (x.ravel(), False)}
    assert_close(gpu_batch(backend, descs, weights, inputs, batch, oc * hw * hw), oracle_batch(descs, weights, inputs, batch), "conv block")


@pytest.mark.parametrize("S,E,H,F", [(64, 128, 2, 256), (96, 512, 8, 320)])
def test_decoder_block_bf16_weights(backend, S, E, H, F):
    """One block of configuration 3 at reduced size: RMSNorm (whole-tensor) -> causal attention ->
    Add -> RMSNorm -> Linear -> GELU -> Linear -> Add, weights pre-rounded to bf16, BF16W precision.
    The second size has samples above 16384 elements: there the norms run as the single-pass kernel and hand
    operand planes straight to the attention block and to fc1."""
    descs = [
        make_desc("n1", "RMSNorm", inputs=["x"], output="h1", params_count=S * E),
        make_desc("attn", "MultiHeadAttention", inputs=["h1"], output="a", seq_len=S, embed_dim=E, num_heads=H, causal=1, params_count=4 * E * E),
        make_desc("add1", "Add", inputs=["__input__", "a"], output="r1"),
        make_desc("n2", "RMSNorm", inputs=["r1"], output="h2", params_count=S * E),
        make_desc("fc1", "Linear", inputs=["h2"], output="f1", in_features=E, out_features=F, seq_len=S, params_count=E * F + F),
        make_desc("gelu", "GELU", inputs=["f1"], output="f1a"),
        make_desc("fc2", "Linear", inputs=["f1a"], output="f2", in_features=F, out_features=E, seq_len=S, params_count=F * E + E),
        make_desc("add2", "Add", inputs=["r1", "f2"], output="x"),
    ]
    weights = configs.seeded_weights(descs, seed=1, std=0.05, bf16=True)
    x = np.random.default_rng(0).standard_normal((2, S * E)).astype(np.float32)
    inputs = {"x": (x.ravel(), False)}
    want = oracle_batch(descs, weights, inputs, 2)
    assert_close(gpu_batch(backend, descs, weights, inputs, 2, S * E, precision=abi.PREC_BF16W), want, "decoder block bf16 weights")
    assert_close(gpu_batch(backend, descs, weights, inputs, 2, S * E), want, "decoder block split weights")


def test_pipelined_forward_equals_single_pass(backend):
    """model_set_pipeline: micro-batches overlapped over three streams and two arena buffers must give
    exactly the bytes of the un-pipelined forward (broadcast inputs included), for the host-pointer and
    the device-pointer entry points."""
    import torch

    cfg = dict(seq_len=16, d_model=32, vocab_size=100, num_layers=1, num_heads=2, mlp_hidden=48, output_dim=24)
    descs = configs.transformer_encoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.05)
    r = np.random.default_rng(0)
    batch = 12
    ids = r.integers(0, 100, (batch, 16)).astype(np.float32)
    mag, mod = (r.standard_normal(32) * 0.02).astype(np.float32), (r.standard_normal(32) * 0.02).astype(np.float32)
    inputs = {"x": (ids.ravel(), False), "mag": (mag, True), "mod": (mod, True)}
    spec = {"x": (16, False), "mag": (32, True), "mod": (32, True)}
    outs = {}
    for pipe in (1, 3, 4, 12):
        m = backend.GraphModel(descs, pipeline=pipe)
        for i, w in enumerate(weights):
            m.upload_weights(i, w)
        m.plan(spec, batch)
        outs[pipe] = m.forward(inputs, batch, 24).copy()
        # device-pointer path on the same model
        d_ids, d_mag, d_mod = (torch.from_numpy(a).cuda() for a in (ids, mag, mod))
        d_out = torch.empty(batch, 24, device="cuda")
        m.forward_device({"x": (d_ids.data_ptr(), 16, False), "mag": (d_mag.data_ptr(), 32, True), "mod": (d_mod.data_ptr(), 32, True)},
                         batch, d_out.data_ptr(), batch * 24, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert np.array_equal(d_out.cpu().numpy(), outs[pipe]), f"device path differs at pipeline {pipe}"
        m.close()
    for pipe in (3, 4, 12):
        assert np.array_equal(outs[pipe], outs[1]), f"pipeline {pipe} differs from the single pass"
    m = backend.GraphModel(descs, pipeline=5)
    with pytest.raises(backend.MimirB200Error, match="multiple"):
        m.plan(spec, batch)
    m.close()


def test_pipelined_forward_keeps_copy_in_and_copy_out_apart(backend):
    """8 micro-batches of 8 MB over two arena buffers.  (1) A two-layer Linear graph: un-pipelined, the planner puts the
    output into the dead input slot; pipelined, input slots are never handed on, so that the copy-in of micro-batch c may
    overlap the copy-out of micro-batch c-2 from the same buffer - results must be bit-equal.  (2) A graph that returns
    its own input: there the output IS an input slot, the copy-in has to wait for the copy-out, and every micro-batch
    must come back unchanged."""
    rows, k = 4096, 512   # 8 MB per micro-batch in and out
    P = 8
    descs = [make_desc("l0", "Linear", inputs=["x"], output="h", in_features=k, out_features=k, seq_len=rows, use_bias=1, params_count=k * k + k),
             make_desc("l1", "Linear", inputs=["h"], output="x", in_features=k, out_features=k, seq_len=rows, use_bias=1, params_count=k * k + k)]
    r = np.random.default_rng(5)
    weights = [np.concatenate([r.uniform(-1, 1, k * k).astype(np.float32) / np.sqrt(k), r.uniform(-0.1, 0.1, k).astype(np.float32)]) for _ in range(2)]
    x = r.standard_normal((P, rows * k), dtype=np.float32)
    m1 = backend.GraphModel(descs)
    mp = backend.GraphModel(descs, pipeline=P)
    for m in (m1, mp):
        for i, w in enumerate(weights):
            m.upload_weights(i, w)
    m1.plan({"x": (rows * k, False)}, P)
    mp.plan({"x": (rows * k, False)}, P)

    def overlap(m):
        (i0, ib), (o0, ob) = m.tensor_slot("x"), m.tensor_slot(None)
        return i0 < o0 + ob and o0 < i0 + ib
    assert overlap(m1), "un-pipelined: the output was expected in the dead input slot"
    assert not overlap(mp), "pipelined: input slots must stay the inputs' own"
    want = m1.forward({"x": (x.ravel(), False)}, P, rows * k)
    for _ in range(3):
        got = mp.forward({"x": (x.ravel(), False)}, P, rows * k)
        assert np.array_equal(got, want)
    sub = np.sort(r.choice(rows, 16, replace=False))
    ref_rows = port.run_graph([make_desc("l0", "Linear", inputs=["x"], output="h", in_features=k, out_features=k, seq_len=16, use_bias=1, params_count=k * k + k),
                               make_desc("l1", "Linear", inputs=["h"], output="x", in_features=k, out_features=k, seq_len=16, use_bias=1, params_count=k * k + k)],
                              weights, {"x": x[P - 1].reshape(rows, k)[sub].ravel()})
    assert_close(got.reshape(P, rows, k)[P - 1][sub], ref_rows, "pipelined two-layer stack, last micro-batch")
    m1.close()
    mp.close()
    # (2) the output is the input
    ident = [make_desc("keep", "Identity", inputs=["x"], output="x")]
    mi = backend.GraphModel(ident, pipeline=P)
    mi.plan({"x": (rows * k, False)}, P)
    assert overlap(mi)
    for _ in range(3):
        assert np.array_equal(mi.forward({"x": (x.ravel(), False)}, P, rows * k).ravel(), x.ravel())
    mi.close()


def test_gpt_decoder_reduced(backend):
    """Configuration 3 at reduced size (2 layers, d 128, 4 heads of 32, seq 96, vocab 300), bf16-rounded
    weights, both precision modes; logits within tolerance and argmax ids equal wherever the CPU top-2
    margin exceeds the tolerance."""
    cfg = dict(layers=2, d_model=128, heads=4, ffn=256, vocab=300, seq=96)
    descs = configs.gpt_decoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.05, bf16=True)
    batch = 2
    ids = np.random.default_rng(0).integers(0, 300, (batch, 96)).astype(np.float32)
    inputs = {"x": (ids.ravel(), False)}
    want = oracle_batch(descs, weights, inputs, batch)
    for prec in (abi.PREC_BF16W, abi.PREC_BF16X2):
        got = gpu_batch(backend, descs, weights, inputs, batch, 96 * 300, precision=prec)
        assert_close(got, want, f"decoder logits precision {prec}")
        w = want.reshape(batch * 96, 300)
        g = got.reshape(batch * 96, 300)
        top2 = np.sort(w, axis=1)[:, -2:]
        decided = (top2[:, 1] - top2[:, 0]) > 2 * (1e-4 + 1e-3 * np.abs(top2[:, 1]))
        assert decided.sum() > 0.9 * decided.size
        assert np.array_equal(g.argmax(1)[decided], w.argmax(1)[decided])


def test_conv_stack_reduced(backend):
    """Configuration 4 at reduced size: stem 7x7 s2 + three residual blocks with GroupNorm + SiLU."""
    descs = configs.conv_stack(image=40, channels=(16, 32, 32, 64), groups=8)
    weights = configs.conv_stack_weights(descs)
    batch = 2
    x = np.random.default_rng(0).random((batch, 3 * 40 * 40)).astype(np.float32)
    inputs = {"x": (x.ravel(), False)}
    assert_close(gpu_batch(backend, descs, weights, inputs, batch, 64 * 20 * 20), oracle_batch(descs, weights, inputs, batch), "conv stack")


def test_unet_mid_up_reduced(backend):
    """Configuration 5 at reduced size: strided convs, ResBlocks, single-head attention over the tokens of
    the mid block (Permute in and out), nearest upsampling x4, bf16-rounded weights."""
    descs = configs.unet_mid_up(latent=16, base=64, groups=8)
    weights = configs.seeded_weights(descs, seed=1, std=0.05, bf16=True)
    batch = 2
    x = np.random.default_rng(0).standard_normal((batch, 4 * 16 * 16)).astype(np.float32)
    inputs = {"x": (x.ravel(), False)}
    want = oracle_batch(descs, weights, inputs, batch)
    assert_close(gpu_batch(backend, descs, weights, inputs, batch, 3 * 64 * 64, precision=abi.PREC_BF16W), want, "unet mid+up")


def test_repeated_forwards_replay_a_cuda_graph_with_identical_results(backend):
    """The third forward with the same buffers replays a captured CUDA graph of the layer loop: results stay
    bit-identical, the launch counter keeps counting the kernels inside, and a re-plan drops the graph."""
    cfg = dict(seq_len=16, d_model=32, vocab_size=64, num_layers=1, num_heads=2, mlp_hidden=48, output_dim=8, causal=False)
    descs = configs.transformer_encoder(**cfg)
    weights = configs.seeded_weights(descs, seed=3, std=0.1)
    r = np.random.default_rng(0)
    batch = 4
    ids = r.integers(1, 64, (batch, 16)).astype(np.float32)
    mag, mod = r.standard_normal(32).astype(np.float32), r.standard_normal(32).astype(np.float32)
    inputs = {"x": (ids, False), "mag": (mag, True), "mod": (mod, True)}
    m = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan({"x": (16, False), "mag": (32, True), "mod": (32, True)}, batch)
    outs, per_call = [], []
    for _ in range(5):
        before = backend.stats()["kernels_launched"]
        outs.append(m.forward(inputs, batch, 8).copy())
        per_call.append(backend.stats()["kernels_launched"] - before)
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    assert len(set(per_call)) == 1 and per_call[0] > 10, per_call
    assert_close(outs[0], oracle_batch(descs, weights, inputs, batch), "transformer, replayed")
    # other inputs through the same graph, then a new plan (different batch)
    ids2 = r.integers(1, 64, (batch, 16)).astype(np.float32)
    inputs2 = {"x": (ids2, False), "mag": (mag, True), "mod": (mod, True)}
    assert_close(m.forward(inputs2, batch, 8), oracle_batch(descs, weights, inputs2, batch), "transformer, replayed, new ids")
    m.plan({"x": (16, False), "mag": (32, True), "mod": (32, True)}, 2)
    half = {"x": (ids[:2], False), "mag": (mag, True), "mod": (mod, True)}
    for _ in range(3):
        got = m.forward(half, 2, 8)
    assert_close(got, oracle_batch(descs, weights, half, 2), "transformer, re-planned")
    m.close()


@pytest.mark.parametrize("shared_output,fuse", [(False, "0"), (False, "1"), (True, "1")])
def test_groupnorm_silu_applied_inside_the_convolution(backend, monkeypatch, shared_output, fuse):
    """UNet-style ResBlock: GroupNorm -> SiLU -> Conv3x3 -> GroupNorm -> SiLU -> Conv3x3 + skip.  Unless
    MIMIR_B200_FUSE_GN_CONV=0, a GroupNorm whose output feeds nothing but the convolution is folded into the
    convolution's layout kernel (statistics pass + normalise on the fly); with a second consumer of the normalised
    tensor it must stay a layer of its own."""
    monkeypatch.setenv("MIMIR_B200_FUSE_GN_CONV", fuse)
    ch, hw, batch, groups = 64, 10, 3, 8
    gn = dict(in_channels=ch, input_height=hw, input_width=hw, num_groups=groups, params_count=2 * ch)
    cv = dict(in_channels=ch, out_channels=ch, input_height=hw, input_width=hw, kernel=3, stride=1, padding=1, params_count=ch * ch * 9)
    descs = [
        make_desc("gn1", "GroupNorm", inputs=["x"], output="n1", **gn),
        make_desc("act1", "SiLU", inputs=["n1"], output="a1"),
        make_desc("conv1", "Conv2d", inputs=["a1"], output="c1", **cv),
        make_desc("gn2", "GroupNorm", inputs=["c1"], output="n2", **gn),
        make_desc("act2", "SiLU", inputs=["n2"], output="a2"),
        make_desc("conv2", "Conv2d", inputs=["a2"], output="c2", **cv),
        make_desc("add", "Add", inputs=["c2", "a1" if shared_output else "__input__"], output="x"),
    ]
    r = np.random.default_rng(12)
    gw = lambda: np.concatenate([1 + 0.2 * r.standard_normal(ch), 0.1 * r.standard_normal(ch)]).astype(np.float32)  # noqa: E731
    cw = lambda: (r.standard_normal(ch * ch * 9) * np.sqrt(2 / (ch * 9))).astype(np.float32)  # noqa: E731
    weights = [gw(), None, cw(), gw(), None, cw(), None]
    x = (r.standard_normal((batch, ch * hw * hw)) * 1.5 + 0.3).astype(np.float32)
    inputs = {"x": (x.ravel(), False)}
    assert_close(gpu_batch(backend, descs, weights, inputs, batch, ch * hw * hw), oracle_batch(descs, weights, inputs, batch),
                 f"resblock, shared={shared_output}")


@pytest.mark.parametrize("conv_skip,fuse", [(False, "1"), (True, "1"), (True, "0")])
def test_nearest_upsample_gathered_by_the_convolutions_that_read_it(backend, monkeypatch, conv_skip, fuse):
    """UNet up block: UpsampleNearest 2x -> [GroupNorm -> SiLU -> Conv3x3 -> GroupNorm -> SiLU -> Conv3x3] + skip.  The
    convolutions that read the upsampled tensor take it from the half-size source while their operand planes are laid out
    (the folded GroupNorm's statistics too); with a 1x1 convolution on the skip path the upsampled tensor is never
    produced, with an identity skip it is still produced for the residual add.  MIMIR_B200_FUSE_UPSAMPLE=0 keeps the
    upsample a layer of its own."""
    monkeypatch.setenv("MIMIR_B200_FUSE_UPSAMPLE", fuse)
    ic, hw, batch, groups = 64, 8, 3, 8
    oc = 32 if conv_skip else ic
    up = 2 * hw
    gn = lambda c: dict(in_channels=c, input_height=up, input_width=up, num_groups=groups, params_count=2 * c)  # noqa: E731
    cv = lambda i, o, k: dict(in_channels=i, out_channels=o, input_height=up, input_width=up, kernel=k, stride=1, padding=k // 2,  # noqa: E731
                              params_count=o * i * k * k)
    descs = [
        make_desc("up", "UpsampleNearest", inputs=["x"], output="u", in_channels=ic, out_h=hw, out_w=hw, scale_h=2, scale_w=2),
        make_desc("gn1", "GroupNorm", inputs=["u"], output="n1", **gn(ic)),
        make_desc("act1", "SiLU", inputs=["n1"], output="a1"),
        make_desc("conv1", "Conv2d", inputs=["a1"], output="c1", **cv(ic, oc, 3)),
        make_desc("gn2", "GroupNorm", inputs=["c1"], output="n2", **gn(oc)),
        make_desc("act2", "SiLU", inputs=["n2"], output="a2"),
        make_desc("conv2", "Conv2d", inputs=["a2"], output="c2", **cv(oc, oc, 3)),
    ]
    r = np.random.default_rng(31)
    gw = lambda c: np.concatenate([1 + 0.2 * r.standard_normal(c), 0.1 * r.standard_normal(c)]).astype(np.float32)  # noqa: E731
    cw = lambda i, o, k: (r.standard_normal(o * i * k * k) * np.sqrt(2 / (i * k * k))).astype(np.float32)  # noqa: E731
    weights = [None, gw(ic), None, cw(ic, oc, 3), gw(oc), None, cw(oc, oc, 3)]
    if conv_skip:
        descs.append(make_desc("skip", "Conv2d", inputs=["u"], output="s", **cv(ic, oc, 1)))
        weights.append(cw(ic, oc, 1))
        descs.append(make_desc("add", "Add", inputs=["c2", "s"], output="x"))
    else:
        descs.append(make_desc("add", "Add", inputs=["c2", "u"], output="x"))
    weights.append(None)
    x = (r.standard_normal((batch, ic * hw * hw)) * 1.5 + 0.3).astype(np.float32)
    inputs = {"x": (x.ravel(), False)}
    assert_close(gpu_batch(backend, descs, weights, inputs, batch, oc * up * up), oracle_batch(descs, weights, inputs, batch),
                 f"up block, conv_skip={conv_skip}, fuse={fuse}")


def test_replayed_graph_with_one_pass_rmsnorm_and_cluster_layernorm(backend):
    """The captured layer loop holds a memset node + the ticketed single-pass RMSNorm, and a cluster-launched
    LayerNorm: five forwards (run, capture, three replays) must agree bit for bit and with the oracle."""
    S, E = 96, 512
    descs = [
        make_desc("n1", "RMSNorm", inputs=["x"], output="h1", params_count=S * E),
        make_desc("fc", "Linear", inputs=["h1"], output="h2", in_features=E, out_features=E, seq_len=S, params_count=E * E + E),
        make_desc("ln", "LayerNorm", inputs=["h2"], output="h3", affine=1, use_bias=1, params_count=2 * S * E),  # whole sample: 49152 elements
        make_desc("add", "Add", inputs=["h3", "__input__"], output="x"),
    ]
    weights = configs.seeded_weights(descs, seed=2, std=0.05)
    batch = 3
    x = np.random.default_rng(1).standard_normal((batch, S * E)).astype(np.float32)
    inputs = {"x": (x.ravel(), False)}
    m = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan({"x": (S * E, False)}, batch)
    outs = [m.forward(inputs, batch, S * E).copy() for _ in range(5)]
    m.close()
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    assert_close(outs[0], oracle_batch(descs, weights, inputs, batch), "rmsnorm -> linear -> layernorm, replayed")
