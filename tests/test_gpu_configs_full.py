"""The five benchmark configurations at their REAL sizes through the graph C ABI, against the reference's own
CPU code (the compiled reference behind ``oracle/ref.py``; the plain-C restatement when that library is absent)
on the same seeded bytes.  Small batches keep the CPU side to about a minute in total: samples are independent,
so a sample of a small batch is computed exactly like the same sample of the full batch.

Gate: |gpu - cpu| <= 1e-4 + 1e-3 |cpu| on every element (``conftest.assert_close``); token ids (argmax of the
decoder's logits) equal wherever the CPU's own top-2 margin exceeds twice that gate.
"""
import json
import os

import numpy as np
import pytest

from conftest import ABS_TOL, REL_TOL, assert_close
from mimir_framework_b200 import abi, configs
from oracle import port, ref

pytestmark = pytest.mark.gpu


def cpu_forward(descs, weights, inputs_per_sample, registry=None, cfg=None):
    """One sample through the reference's CPU path."""
    if ref.available():
        ref.set_threads(os.cpu_count() or 1)
        ref.set_guard_limit(64 << 30)
        m = ref.RefModel(registry=registry, cfg_json=json.dumps(cfg)) if registry else ref.RefModel(descs)
        for i, w in enumerate(weights):
            if w is not None:
                m.set_weights(i, w)
        y = m.forward(inputs_per_sample)
        m.close()
        return y
    return port.run_graph(descs, weights, inputs_per_sample)


def gpu_forward(backend, descs, weights, spec, inputs, batch, out_n, precision):
    m = backend.GraphModel(descs, precision)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan(spec, batch)
    out = m.forward(inputs, batch, out_n).reshape(batch, out_n)
    m.close()
    return out


def test_config1_registry_transformer_full_size(backend):
    """Configuration 1 as stated: 2 layers, d_model 256, 4 heads, FFN 1024, vocab 8192, seq 128, batch 8, fp32;
    ids from seed 0 (id 0 hits padding_idx 0 -> zero row, as in the reference), weights N(0, 0.02) seed 1."""
    cfg = configs.TRANSFORMER_CFG
    descs = configs.transformer_encoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.02)
    batch, S, D = 8, cfg["seq_len"], cfg["d_model"]
    ids = np.random.default_rng(0).integers(0, cfg["vocab_size"], (batch, S)).astype(np.float32)
    r = np.random.default_rng(2)
    mag, mod = (r.standard_normal(D) * 0.02).astype(np.float32), (r.standard_normal(D) * 0.02).astype(np.float32)
    if ref.available():
        m = ref.RefModel(registry="transformer", cfg_json=json.dumps(cfg))
        rd = m.layer_descs()
        assert [d.type for d in rd] == [d.type for d in descs]
        assert [int(d.params_count) for d in rd] == [int(d.params_count) for d in descs]
        mag, mod = m.mag_mod()  # the Encoder's own vectors (Encoder.cpp:97-116)
        m.close()
    want = np.stack([cpu_forward(descs, weights, {"x": ids[s], "mag": mag, "mod": mod}, registry="transformer" if ref.available() else None, cfg=cfg)
                     for s in range(batch)])
    got = gpu_forward(backend, descs, weights, {"x": (S, False), "mag": (D, True), "mod": (D, True)},
                      {"x": (ids.ravel(), False), "mag": (mag, True), "mod": (mod, True)}, batch, cfg["output_dim"], abi.PREC_BF16X2)
    assert_close(got, want, "config 1 (registry transformer, batch 8)")


def test_config3_gpt_decoder_full_size(backend):
    """Configuration 3 as stated: 12 layers, d_model 768, 12 heads, FFN 3072, whole-sample RMSNorm, causal attention,
    vocab 32000, seq 1024, bf16-rounded weights; two samples of the seed-0 id matrix.  All 2 x 32 768 000 logits
    inside the gate, and the token ids (first maximum per position) equal on every decided position."""
    import torch

    cfg = configs.DECODER_CFG
    S, V = cfg["seq"], cfg["vocab"]
    descs = configs.gpt_decoder(**cfg)
    weights = configs.seeded_weights(descs, seed=1, std=0.02, bf16=True)
    batch = 2
    ids = np.random.default_rng(0).integers(0, V, (32, S)).astype(np.float32)[:batch].copy()
    m = backend.GraphModel(descs, abi.PREC_BF16W)
    for i, w in enumerate(weights):
        m.upload_weights(i, w)
    m.plan({"x": (S, False)}, batch)
    d_ids = torch.from_numpy(ids).cuda()
    d_out = torch.empty(batch * S * V, device="cuda")
    d_tok = torch.empty(batch * S, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    m.forward_device({"x": (d_ids.data_ptr(), S, False)}, batch, d_out.data_ptr(), d_out.numel(), st)
    backend.check(backend.lib().mimir_b200_argmax_rows_device(d_out.data_ptr(), d_tok.data_ptr(), batch * S, V, st))
    torch.cuda.synchronize()
    backend.check(backend.lib().mimir_b200_check_device(None))
    got = d_out.cpu().numpy().reshape(batch, S, V)
    tok = d_tok.cpu().numpy().reshape(batch, S)
    m.close()
    undecided_total = 0
    for s in range(batch):
        want = cpu_forward(descs, weights, {"x": ids[s]}).reshape(S, V)
        assert_close(got[s], want, f"config 3 (decoder prefill) sample {s}")
        part = np.partition(want, V - 2, axis=1)[:, V - 2:]
        top1, top2 = part.max(axis=1), part.min(axis=1)
        decided = (top1 - top2) > 2 * (ABS_TOL + REL_TOL * np.abs(top1))
        undecided_total += int((~decided).sum())
        assert np.array_equal(tok[s][decided], want.argmax(axis=1)[decided].astype(np.int32)), f"sample {s}: token ids differ on decided positions"
    print(f"config 3: {undecided_total} of {batch * S} positions had a CPU top-2 margin inside the gate and were not compared")
    assert undecided_total <= 0.05 * batch * S


def test_config4_conv_stack_full_size(backend):
    """Configuration 4 as stated: 3 x 224 x 224 input, stem 7x7 s2, four residual blocks 64 -> 128 -> 128 -> 256 -> 256
    at 112^2 with GroupNorm(32) + SiLU; two samples."""
    descs = configs.conv_stack()
    weights = configs.conv_stack_weights(descs)
    batch = 2
    x = np.random.default_rng(0).random((64, 3 * 224 * 224), dtype=np.float32)[:batch].copy()
    out_n = 256 * 112 * 112
    got = gpu_forward(backend, descs, weights, {"x": (x.shape[1], False)}, {"x": (x.ravel(), False)}, batch, out_n, abi.PREC_BF16X2)
    for s in range(batch):
        assert_close(got[s], cpu_forward(descs, weights, {"x": x[s]}), f"config 4 (conv stack) sample {s}")


def test_config5_unet_mid_up_full_size(backend):
    """Configuration 5 as frozen in configs.unet_mid_up: latent 4 x 64 x 64 -> 3 x 256 x 256, channels 512/256/128,
    one attention head of 512 over 256 tokens, bf16-rounded weights; two samples."""
    descs = configs.unet_mid_up()
    weights = configs.seeded_weights(descs, seed=1, std=0.02, bf16=True)
    batch = 2
    x = np.random.default_rng(0).standard_normal((16, 4 * 64 * 64), dtype=np.float32)[:batch].copy()
    out_n = 3 * 256 * 256
    got = gpu_forward(backend, descs, weights, {"x": (x.shape[1], False)}, {"x": (x.ravel(), False)}, batch, out_n, abi.PREC_BF16W)
    for s in range(batch):
        assert_close(got[s], cpu_forward(descs, weights, {"x": x[s]}), f"config 5 (UNet mid+up) sample {s}")
