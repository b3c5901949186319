"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own CPU code.

    python tests/golden/make_golden.py          # needs oracle/_ref/libmimir_ref.so (make -C oracle ref)

Each case is a small layer graph (descriptors as JSON), seeded weights and inputs, and the output of
the compiled reference (`Model::forwardPassNamed`, training = false) on them.  The fixtures pin the
plain-C oracle (CPU test) and the CUDA backend (GPU test) to the reference's actual behaviour; the
tests never need the reference itself.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from mimir_framework_b200 import configs  # noqa: E402
from mimir_framework_b200.abi import desc_to_dict, make_desc  # noqa: E402
from oracle import ref  # noqa: E402


def cases():
    r = np.random.default_rng(2024)
    f = lambda *s, scale=1.0: (r.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    out = []

    def add(name, descs, weights, inputs):
        out.append((name, descs, weights, inputs))

    w = r.uniform(-0.2, 0.2, 50 * 29 + 29).astype(np.float32)
    add("linear_seq", [make_desc("l", "Linear", in_features=50, out_features=29, seq_len=37, params_count=w.size)], [w], {"x": f(37 * 50)})
    add("linear_vec", [make_desc("l", "Linear", in_features=50, out_features=29, params_count=w.size)], [w], {"x": f(50)})
    add("linear_implicit_in_nobias", [make_desc("l", "Linear", out_features=7, use_bias=0, params_count=7 * 33)], [f(7 * 33, scale=0.3)], {"x": f(33)})
    E, S = 32, 24
    wa = f(4 * E * E, scale=0.15)
    for causal in (0, 1):
        add(f"attention_causal{causal}", [make_desc("a", "MultiHeadAttention", embed_dim=E, seq_len=S, num_heads=4, causal=causal, params_count=wa.size)], [wa], {"x": f(S * E)})
    add("self_attention_1head", [make_desc("a", "SelfAttention", embed_dim=E, seq_len=S, num_heads=1, params_count=wa.size)], [wa], {"x": f(S * E)})
    ic, oc, h = 5, 13, 11
    add("conv3x3_p1", [make_desc("c", "Conv2d", in_channels=ic, out_channels=oc, input_height=h, input_width=h, kernel=3, stride=1, padding=1, params_count=oc * ic * 9)], [f(oc * ic * 9, scale=0.2)], {"x": r.random(ic * h * h).astype(np.float32)})
    add("conv7x7_s2_p3_relu", [make_desc("c", "Conv2d", in_channels=ic, out_channels=oc, input_height=h, input_width=h, kernel=7, stride=2, padding=3, activation=1, params_count=oc * ic * 49)], [f(oc * ic * 49, scale=0.1)], {"x": r.random(ic * h * h).astype(np.float32)})
    add("conv1x1_rect", [make_desc("c", "Conv2d", in_channels=4, out_channels=6, input_height=5, input_width=9, kernel=1, stride=1, padding=0, params_count=24)], [f(24)], {"x": f(4 * 5 * 9)})
    n = 96
    add("layernorm_groups", [make_desc("n", "LayerNorm", in_features=n, params_count=2 * n)], [f(2 * n)], {"x": f(5 * n, scale=2.0) + 0.5})
    add("layernorm_whole", [make_desc("n", "LayerNorm", params_count=2 * 5 * n)], [f(10 * n)], {"x": f(5 * n)})
    add("layernorm_no_affine", [make_desc("n", "LayerNorm", in_features=n, affine=0)], [None], {"x": f(3 * n)})
    add("rmsnorm_partial_gamma", [make_desc("n", "RMSNorm", params_count=100)], [f(100)], {"x": f(300)})
    C = 16
    add("groupnorm", [make_desc("n", "GroupNorm", in_channels=C, input_height=7, input_width=9, num_groups=4, params_count=2 * C)], [f(2 * C)], {"x": f(C * 63, scale=1.5) + 0.3})
    for t in ("Softmax", "LogSoftmax", "GELU", "SiLU", "ReLU", "Tanh", "Sigmoid"):
        add(t.lower(), [make_desc("n", t)], [None], {"x": f(257, scale=3.0)})
    add("add_broadcast", [make_desc("n", "Add", inputs=["x", "b"])], [None], {"x": f(6 * 40), "b": f(40)})
    add("add_scalar", [make_desc("n", "Add", inputs=["x", "b"])], [None], {"x": f(33), "b": f(1)})
    add("multiply", [make_desc("n", "Multiply", inputs=["x", "b"])], [None], {"x": f(33), "b": f(33)})
    add("embedding_pad_oob_round", [make_desc("e", "Embedding", vocab_size=50, embed_dim=8, padding_idx=0, params_count=400)], [f(400)], {"x": np.array([0, 3, 49, 50, -1, 7.4, 7.5, 8.5, 2.5], np.float32)})
    add("upsample_nearest", [make_desc("u", "UpsampleNearest", in_channels=3, out_h=4, out_w=5, scale_h=2, scale_w=3)], [None], {"x": f(60)})
    add("permute_201", [make_desc("p", "Permute", shape=[3, 4, 5], permute_dims=[2, 0, 1])], [None], {"x": f(60)})
    add("concat3", [make_desc("c", "Concat", inputs=["x", "y", "z"])], [None], {"x": f(2), "y": f(1), "z": f(2)})
    add("token_mean_pool", [make_desc("t", "TokenMeanPool", seq_len=7, embed_dim=12)], [None], {"x": f(84)})
    add("global_avgpool", [make_desc("g", "GlobalAvgPool2d", in_channels=3, input_height=4, input_width=7)], [None], {"x": f(84)})
    d = configs.linear_gelu_stack(16, 64)
    add("linear_gelu_stack_16x64", d, configs.linear_gelu_stack_weights(64), {"x": configs.linear_gelu_stack_input(16, 64).ravel()})
    # ---- the remaining switch cases (appended: the generator above must keep its random stream) ----
    E, ql, kl = 32, 10, 17
    wx = f(4 * E * E, scale=0.15)
    for causal in (0, 1):
        add(f"cross_attention_causal{causal}", [make_desc("a", "CrossAttention", inputs=["x", "ctx"], embed_dim=E, num_heads=4, causal=causal, params_count=wx.size)],
            [wx], {"x": f(ql * E), "ctx": f(kl * E)})
    add("cross_attention_head_dim", [make_desc("a", "CrossAttention", inputs=["x", "ctx"], embed_dim=0, head_dim=8, num_heads=4, params_count=wx.size)],
        [wx], {"x": f(kl * E), "ctx": f(ql * E)})
    add("split_concat", [make_desc("s", "Split", output="s", split_sizes=[20, 13, 7]), make_desc("c", "Concat", inputs=["s_2", "s", "s_1"])],
        [None, None], {"x": f(40)})
    add("chunk_concat", [make_desc("s", "Chunk", output="c", num_chunks=3), make_desc("c", "Concat", inputs=["c_1", "c_2", "c_0", "c"])],
        [None, None], {"x": f(10)})
    add("depthwise_conv_s2_bias", [make_desc("d", "DepthwiseConv2d", in_channels=6, input_height=9, input_width=11, raw_kernel_h=3, raw_stride_h=2, raw_pad_h=1,
                                             use_bias=1, params_count=6 * 9 + 6)], [f(60, scale=0.3)], {"x": f(6 * 99)})
    add("conv1d_s2_bias", [make_desc("c", "Conv1d", in_channels=3, out_channels=5, raw_kernel_h=3, raw_stride_h=2, raw_pad_h=1, use_bias=1, params_count=45 + 5)],
        [f(50, scale=0.3)], {"x": f(60)})
    add("conv_transpose2d_relu", [make_desc("c", "ConvTranspose2d", in_channels=3, out_channels=4, input_height=5, input_width=6, kernel=4, stride=2, padding=1,
                                            activation=1, params_count=4 * 3 * 16)], [f(192, scale=0.2)], {"x": f(90)})
    add("maxpool_k3s2p1", [make_desc("p", "MaxPool2d", in_channels=3, input_height=7, input_width=9, kernel=3, stride=2, padding=1)], [None], {"x": f(189)})
    add("avgpool_k3s1p1", [make_desc("p", "AvgPool2d", in_channels=3, input_height=7, input_width=9, kernel=3, stride=1, padding=1)], [None], {"x": f(189)})
    add("avgpool_k2s2", [make_desc("p", "AvgPool2d", in_channels=2, input_height=6, input_width=8, kernel=2, stride=2, padding=0)], [None], {"x": f(96)})
    for t, kw in (("ZeroPad2d", dict(raw_pad_h=1, raw_pad_w=2)), ("ReflectionPad2d", dict(raw_pad_h=2)), ("ReplicationPad2d", dict(raw_pad_h=2))):
        add(t.lower(), [make_desc("p", t, in_channels=2, input_height=4, input_width=5, **kw)], [None], {"x": f(40)})
    add("pixel_shuffle_r2", [make_desc("p", "PixelShuffle", in_channels=8, input_height=3, input_width=5, scale_h=2)], [None], {"x": f(120)})
    for t in ("UpsampleBilinear", "UpsampleBicubic"):
        add(t.lower(), [make_desc("u", t, in_channels=3, out_h=5, out_w=7)], [None], {"x": f(105)})
    add("matmul", [make_desc("m", "MatMul", inputs=["x", "b"], in_features=5, out_features=37, embed_dim=9)], [None], {"x": f(5 * 37), "b": f(37 * 9)})
    add("batch_matmul", [make_desc("m", "BatchMatMul", inputs=["x", "b"], seq_len=3, in_features=33, out_features=40, embed_dim=35)], [None],
        {"x": f(3 * 33 * 40), "b": f(3 * 40 * 35)})
    add("batchnorm_partial_weights", [make_desc("n", "BatchNorm2d", params_count=24)], [f(24) + 1.0], {"x": f(96, scale=2.0) + 0.7})
    add("instance_norm_affine", [make_desc("n", "InstanceNorm2d", in_channels=4, input_height=5, input_width=6, params_count=8)], [f(8) + 1.0], {"x": f(120, scale=1.5)})
    add("leaky_relu_02", [make_desc("n", "LeakyReLU", leaky_relu_alpha=0.2)], [None], {"x": f(257, scale=3.0)})
    for t in ("Softplus", "Mish", "HardSigmoid", "HardSwish"):
        add(t.lower(), [make_desc("n", t)], [None], {"x": f(257, scale=8.0)})
    add("subtract", [make_desc("n", "Subtract", inputs=["x", "b"])], [None], {"x": f(33), "b": f(33)})
    dv = f(33)
    dv[[0, 5, 9]] = [0.0, -0.0, 1e-9]
    add("divide_small_divisors", [make_desc("n", "Divide", inputs=["x", "b"])], [None], {"x": f(33), "b": dv})
    add("transpose_2d", [make_desc("t", "Transpose", in_features=6, out_features=11)], [None], {"x": f(66)})
    add("reparameterize_inference", [make_desc("r", "Reparameterize", inputs=["x", "lv"])], [None], {"x": f(20), "lv": f(20)})
    add("squeeze_unsqueeze", [make_desc("a", "Squeeze"), make_desc("b", "Unsqueeze")], [None, None], {"x": f(12)})
    add("stack2", [make_desc("s", "Stack", inputs=["x", "y"])], [None], {"x": f(7), "y": f(7)})
    # the layer types whose fields arrived with descriptor version 3, and the recurrent layers
    tb = f(30 * 6)
    add("embedding_bag_offsets", [make_desc("e", "EmbeddingBag", inputs=["ids", "offs"], vocab_size=30, embed_dim=6, padding_idx=4, params_count=180)], [tb],
        {"ids": np.array([1, 4, 29, 30, -2, 7.4, 7.5, 3, 3, 12, 0], np.float32), "offs": np.array([0, 3, 3, 8, 40], np.float32)})
    add("embedding_bag_unsorted_offsets", [make_desc("e", "EmbeddingBag", inputs=["ids", "offs"], vocab_size=30, embed_dim=6, params_count=180)], [tb],
        {"ids": np.array([5, 6, 7, 8, 9, 10], np.float32), "offs": np.array([-3, 4, 2, 6], np.float32)})
    add("embedding_bag_single_bag", [make_desc("e", "EmbeddingBag", inputs=["ids"], vocab_size=30, embed_dim=6, params_count=180)], [tb],
        {"ids": np.array([2, 2, 19, 11], np.float32)})
    dm, stx, npch, pdim = 12, 3, 5, 48
    add("patch_embed", [make_desc("p", "PatchEmbed", embed_dim=dm, seq_text=stx, num_patches=npch, patch_dim=pdim, params_count=pdim * dm + dm)],
        [f(pdim * dm + dm, scale=0.3)], {"x": f((stx + 1) * dm + npch * pdim)})
    add("patch_embed_out_features", [make_desc("p", "PatchEmbed", out_features=dm, seq_text=stx, num_patches=2, patch_dim=7, params_count=7 * dm + dm)],
        [f(7 * dm + dm, scale=0.3)], {"x": f((stx + 1) * dm + 2 * 7)})
    add("bilinear_bias", [make_desc("b", "Bilinear", inputs=["x", "z"], in_features=9, out_features=14, embed_dim=5, use_bias=1, params_count=5 * 9 * 14 + 5)],
        [f(5 * 9 * 14 + 5, scale=0.3)], {"x": f(4 * 9), "z": f(4 * 14)})
    add("bilinear_target_shape_nobias", [make_desc("b", "Bilinear", inputs=["x", "z"], in_features=6, out_features=3, target_dim0=7, use_bias=0, params_count=7 * 18)],
        [f(7 * 18, scale=0.3)], {"x": f(6), "z": f(3)})
    T, I, H = 6, 10, 13
    for kind, g in (("RNN", 1), ("GRU", 3), ("LSTM", 4)):
        nw = g * H * I + g * H * H
        add(f"{kind.lower()}_bias", [make_desc("r", kind, seq_len=T, in_features=I, out_features=H, use_bias=1, params_count=nw + 2 * g * H)],
            [f(nw + 2 * g * H, scale=0.35)], {"x": f(T * I)})
        add(f"{kind.lower()}_nobias", [make_desc("r", kind, seq_len=3, in_features=4, out_features=5, use_bias=0, params_count=g * 5 * 4 + g * 25)],
            [f(g * 5 * 4 + g * 25, scale=0.5)], {"x": f(12)})
    add("avgpool1d_k3s2p1", [make_desc("p", "AvgPool1d", in_channels=3, raw_kernel_h=3, raw_stride_h=2, raw_pad_h=1)], [None], {"x": f(3 * 17)})
    return out


def transformer_case():
    """The registry transformer at a small width, built by the reference's own ModelArchitectures::create;
    mag / mod are the Encoder's defaults as the reference computes them."""
    cfg = dict(seq_len=8, d_model=16, vocab_size=50, num_layers=1, num_heads=2, mlp_hidden=24, output_dim=8, causal=False)
    m = ref.RefModel(registry="transformer", cfg_json=json.dumps(cfg))
    descs = m.layer_descs()
    ours = configs.transformer_encoder(**cfg)
    assert [desc_to_dict(a) for a in descs] == [desc_to_dict(b) for b in ours], "registry graph differs from configs.transformer_encoder"
    weights = configs.seeded_weights(ours, seed=1, std=0.1)
    for i, w in enumerate(weights):
        if w is not None:
            m.set_weights(i, w)
    mag, mod = m.mag_mod()
    ids = np.array([5, 0, 49, 17, 3, 3, 21, 8], np.float32)
    y = m.forward({"x": ids, "mag": mag, "mod": mod})
    return "transformer_registry_tiny", ours, weights, {"x": ids, "mag": mag, "mod": mod}, y


def function_cases():
    """Layer functions of the reference that its layer switch never dispatches, called directly."""
    r = np.random.default_rng(77)
    out = []
    # LayerOpsExt::maxpool1d_forward (LayerOpsExt.hpp:504-538): a MaxPool1d layer throws in Model::forwardPassView
    for nm, ch, length, k, st, pad in (("maxpool1d_k3s2p1", 3, 17, 3, 2, 1), ("maxpool1d_default_stride", 2, 9, 2, 0, 0), ("maxpool1d_k4s1p3", 1, 6, 4, 1, 3)):
        x = r.standard_normal(ch * length).astype(np.float32)
        d = make_desc("p", "MaxPool1d", in_channels=ch, raw_kernel_h=k, raw_stride_h=st, raw_pad_h=pad)
        out.append((nm, [d], [None], {"x": x}, ref.maxpool1d(x, ch, k, st, pad)))
    return out


def _compact(j):
    """Drops descriptor fields that hold the Layer defaults (desc_from_dict restores them)."""
    from mimir_framework_b200.abi import LAYER_DEFAULTS
    out = {}
    for k, v in j.items():
        if k in LAYER_DEFAULTS and LAYER_DEFAULTS[k] is not None and (abs(v - LAYER_DEFAULTS[k]) < 1e-9):
            continue
        if k in ("kernel_w", "stride_w", "padding_w") and v == j[{"kernel_w": "kernel", "stride_w": "stride", "padding_w": "padding"}[k]]:
            continue
        if k in ("shape", "permute_dims", "split_sizes") and not v:
            continue
        out[k] = v
    return out


def registry_graphs():
    """Every architecture of the reference's registry at a small width: the layer list comes from the
    reference's own builder, the weights from a seeded generator, the expected output from the
    compiled reference's forward."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import registry_cases as rc
    graphs, arrays = {}, {}
    for arch, cfg in rc.CFG.items():
        m = ref.RefModel(registry=arch, cfg_json=json.dumps(cfg))
        descs = m.layer_descs()
        weights = rc.make_weights(descs)
        for i, w in enumerate(weights):
            if w is not None:
                m.set_weights(i, w)
        inputs = rc.make_inputs(arch)
        if arch == "transformer":
            inputs["mag"], inputs["mod"] = m.mag_mod()
        y = m.forward(inputs)
        assert np.all(np.isfinite(y)) and y.size > 0, arch
        graphs[arch] = [_compact(desc_to_dict(d)) for d in descs]
        for k, v in inputs.items():
            arrays[f"{arch}/in/{k}"] = v
        arrays[f"{arch}/out"] = y
        print(f"{arch:20s} layers {len(descs):3d} out {y.size:6d} |y| mean {np.abs(y).mean():.3e}")
        m.close()
    np.savez_compressed(os.path.join(HERE, "registry_graphs.npz"), **arrays)
    with open(os.path.join(HERE, "registry_graphs.json"), "w") as fh:
        json.dump({"generator": "tests/golden/make_golden.py", "source": "ModelArchitectures::create + forwardPassNamed(training=false) of the compiled reference",
                   "configs": rc.CFG, "graphs": graphs}, fh)


def main():
    registry_graphs()
    index = []
    arrays = {}
    for name, descs, weights, inputs in cases():
        m = ref.RefModel(descs)
        for i, w in enumerate(weights):
            if w is not None:
                m.set_weights(i, w)
        y = m.forward(inputs)
        m.close()
        index.append(_store(arrays, name, descs, weights, inputs, y))
    name, descs, weights, inputs, y = transformer_case()
    index.append(_store(arrays, name, descs, weights, inputs, y))
    for name, descs, weights, inputs, y in function_cases():
        index.append(_store(arrays, name, descs, weights, inputs, y))
    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **arrays)
    with open(os.path.join(HERE, "reference_vectors.json"), "w") as fh:
        json.dump({"generator": "tests/golden/make_golden.py", "source": "compiled reference (oracle/_ref), forwardPassNamed(training=false)",
                   "cases": index}, fh, indent=1)
    print(f"wrote {len(index)} cases, {sum(a.nbytes for a in arrays.values())} bytes of arrays")


def _store(arrays, name, descs, weights, inputs, y):
    for i, w in enumerate(weights):
        if w is not None:
            arrays[f"{name}/w{i}"] = np.asarray(w, np.float32)
    for k, v in inputs.items():
        arrays[f"{name}/in/{k}"] = np.asarray(v, np.float32)
    arrays[f"{name}/out"] = np.asarray(y, np.float32)
    return {"name": name, "layers": [desc_to_dict(d) for d in descs], "inputs": list(inputs.keys()),
            "weights": [w is not None for w in weights]}


if __name__ == "__main__":
    main()
