"""The one-MMA precision mode (MIMIR_B200_PREC_BF16): every contraction takes ONE 16-bit plane per operand, so its results
differ from the reference's fp32 arithmetic by the rounding of those operands.  The checker for it is the oracle with the
same rounding applied (oracle.port.OperandRounding): against that the backend must sit inside the usual gate; against the
unrounded oracle the distance is measured and bounded loosely, which is why the strict modes stay the default."""
import numpy as np
import pytest

from conftest import ABS_TOL, REL_TOL, assert_close
from mimir_framework_b200 import abi, configs
from oracle import port
from test_gpu_graph import gpu_batch

pytestmark = pytest.mark.gpu


def outside(got, want):
    got, want = np.asarray(got, np.float32).ravel(), np.asarray(want, np.float32).ravel()
    return int((np.abs(got - want) > ABS_TOL + REL_TOL * np.abs(want)).sum())


def test_decoder_in_the_one_mma_mode_matches_the_rounding_matched_oracle(backend):
    """A small decoder of configuration 3's shape family (RMSNorm over the whole sample, causal attention with 64-wide heads,
    GELU FFN, LM head; bf16-exact weights)."""
    seq, vocab, batch = 128, 512, 3
    descs = configs.gpt_decoder(layers=2, d_model=128, heads=2, ffn=256, vocab=vocab, seq=seq)
    weights = configs.seeded_weights(descs, bf16=True)
    ids = np.random.default_rng(5).integers(0, vocab, size=(batch, seq)).astype(np.float32)
    inputs = {"x": (ids.ravel(), False)}
    got = gpu_batch(backend, descs, weights, inputs, batch, seq * vocab, precision=abi.PREC_BF16).reshape(batch, -1)
    strict = gpu_batch(backend, descs, weights, inputs, batch, seq * vocab, precision=abi.PREC_BF16W).reshape(batch, -1)
    import os
    fmt = "bf16" if os.environ.get("MIMIR_B200_PLANES") == "bf16" else "f16"
    hooked = np.stack([port.run_graph(descs, weights, {"x": ids[s]}, rounding=port.OperandRounding(fmt)) for s in range(batch)])
    plain = np.stack([port.run_graph(descs, weights, {"x": ids[s]}) for s in range(batch)])
    assert_close(strict, plain, "decoder, strict mode against the fp32 oracle")
    assert_close(got, hooked, "decoder, one-MMA mode against the oracle with the same operand rounding")
    # against the reference's own arithmetic the one-MMA mode is a few operand roundings away: measured, not gated
    err = np.abs(got - plain)
    assert float(err.max()) < 50 * (ABS_TOL + REL_TOL * float(np.abs(plain).max())), "one-MMA mode drifted far from fp32"
    print(f"one-MMA decoder vs fp32 oracle: max abs {err.max():.3e}, {outside(got, plain)} of {got.size} outside the gate; "
          f"vs rounding-matched oracle: max abs {np.abs(got - hooked).max():.3e}")


def test_conv_block_in_the_one_mma_mode_matches_the_rounding_matched_oracle(backend):
    """GroupNorm -> SiLU -> Conv3x3 -> GroupNorm -> SiLU -> Conv3x3 + skip (the UNet configuration's block) with bf16-exact
    weights; the image is small enough that every convolution takes the tensor-core path."""
    ch, hw, batch, groups = 64, 12, 2, 8
    gn = dict(in_channels=ch, input_height=hw, input_width=hw, num_groups=groups, params_count=2 * ch)
    cv = dict(in_channels=ch, out_channels=ch, input_height=hw, input_width=hw, kernel=3, stride=1, padding=1, params_count=ch * ch * 9)
    descs = [
        abi.make_desc("gn1", "GroupNorm", inputs=["x"], output="n1", **gn),
        abi.make_desc("act1", "SiLU", inputs=["n1"], output="a1"),
        abi.make_desc("conv1", "Conv2d", inputs=["a1"], output="c1", **cv),
        abi.make_desc("gn2", "GroupNorm", inputs=["c1"], output="n2", **gn),
        abi.make_desc("act2", "SiLU", inputs=["n2"], output="a2"),
        abi.make_desc("conv2", "Conv2d", inputs=["a2"], output="c2", **cv),
        abi.make_desc("add", "Add", inputs=["c2", "__input__"], output="x"),
    ]
    r = np.random.default_rng(21)
    gw = lambda: np.concatenate([1 + 0.2 * r.standard_normal(ch), 0.1 * r.standard_normal(ch)]).astype(np.float32)  # noqa: E731
    cw = lambda: configs.round_to_bf16((r.standard_normal(ch * ch * 9) * np.sqrt(2 / (ch * 9))).astype(np.float32))  # noqa: E731
    weights = [gw(), None, cw(), gw(), None, cw(), None]
    x = (r.standard_normal((batch, ch * hw * hw)) * 1.5 + 0.3).astype(np.float32)
    inputs = {"x": (x.ravel(), False)}
    import os
    fmt = "bf16" if os.environ.get("MIMIR_B200_PLANES") == "bf16" else "f16"
    got = gpu_batch(backend, descs, weights, inputs, batch, ch * hw * hw, precision=abi.PREC_BF16).reshape(batch, -1)
    hooked = np.stack([port.run_graph(descs, weights, {"x": x[s]}, rounding=port.OperandRounding(fmt)) for s in range(batch)])
    plain = np.stack([port.run_graph(descs, weights, {"x": x[s]}) for s in range(batch)])
    assert_close(got, hooked, "conv block, one-MMA mode against the oracle with the same operand rounding")
    print(f"one-MMA conv block vs fp32 oracle: max abs {np.abs(got - plain).max():.3e}, {outside(got, plain)} of {got.size} outside the gate")
