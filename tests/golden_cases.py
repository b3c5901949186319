"""Loads the committed golden vectors (tests/golden/reference_vectors.*) and the reference's own
known-answer tests for the path, restated as data."""
import json
import os

import numpy as np

from mimir_framework_b200.abi import desc_from_dict, make_desc

HERE = os.path.dirname(os.path.abspath(__file__))


def load_golden():
    with open(os.path.join(HERE, "golden", "reference_vectors.json")) as fh:
        index = json.load(fh)["cases"]
    arrays = np.load(os.path.join(HERE, "golden", "reference_vectors.npz"))
    cases = []
    for c in index:
        name = c["name"]
        descs = [desc_from_dict(j) for j in c["layers"]]
        weights = [arrays[f"{name}/w{i}"] if has else None for i, has in enumerate(c["weights"])]
        inputs = {k: arrays[f"{name}/in/{k}"] for k in c["inputs"]}
        cases.append((name, descs, weights, inputs, arrays[f"{name}/out"]))
    return cases


def reference_kats():
    """(name, descs, weights, inputs, expected, atol) from Tests/test_layers_all_types.cpp,
    Tests/test_runtime_embedding_int_inputs.cpp and Tests/test_layers_named_routing.cpp."""
    f = lambda *v: np.array(v, np.float32)  # noqa: E731
    sig = lambda x: 1.0 / (1.0 + np.exp(-np.float32(x)))  # noqa: E731
    k = []
    # Linear, test_layers_all_types.cpp:71-100
    k.append(("linear", [make_desc("t0", "Linear", inputs=["x"], in_features=2, out_features=3, use_bias=1, params_count=9)],
              [f(1, 2, 0, 1, -1, 0, 0, 1, 0)], {"x": f(1, 2)}, f(5, 3, -1), 1e-6))
    # Conv2d k=1, :105-133
    k.append(("conv2d_k1", [make_desc("t0", "Conv2d", inputs=["x"], in_channels=1, out_channels=1, input_height=2, input_width=2,
                                      kernel=1, stride=1, padding=0, params_count=1)], [f(2)], {"x": f(1, 2, 3, 4)}, f(2, 4, 6, 8), 1e-6))
    # activations, :205-239
    x3 = f(-1, 0, 1)
    k.append(("relu", [make_desc("t0", "ReLU", inputs=["x"])], [None], {"x": x3}, f(0, 0, 1), 1e-6))
    k.append(("tanh", [make_desc("t0", "Tanh", inputs=["x"])], [None], {"x": x3}, np.tanh(x3), 1e-6))
    k.append(("sigmoid", [make_desc("t0", "Sigmoid", inputs=["x"])], [None], {"x": x3}, f(sig(-1), 0.5, sig(1)), 1e-6))
    k.append(("silu", [make_desc("t0", "SiLU", inputs=["x"])], [None], {"x": x3}, f(-sig(-1), 0, sig(1)), 1e-6))
    k.append(("gelu", [make_desc("t0", "GELU", inputs=["x"])], [None], {"x": f(0, 1)}, f(0, 0.8413), 2e-3))
    # Softmax / LogSoftmax, :244-262
    k.append(("softmax", [make_desc("t0", "Softmax", inputs=["x"])], [None], {"x": f(0, 0)}, f(0.5, 0.5), 1e-6))
    k.append(("logsoftmax", [make_desc("t0", "LogSoftmax", inputs=["x"])], [None], {"x": f(0, 0)}, f(-np.log(2), -np.log(2)), 1e-5))
    # RMSNorm, :306-323
    rms = np.sqrt(np.float32(12.5) + np.float32(1e-6))
    k.append(("rmsnorm", [make_desc("t0", "RMSNorm", inputs=["x"], eps=1e-6, params_count=2)], [f(1, 1)], {"x": f(3, 4)}, f(3 / rms, 4 / rms), 1e-5))
    # Dropout at inference is the identity, :328-340
    k.append(("dropout_identity", [make_desc("t0", "Dropout", inputs=["x"])], [None], {"x": f(1, 2, 3)}, f(1, 2, 3), 0))
    # pools, :345-389
    k.append(("global_avgpool", [make_desc("t0", "GlobalAvgPool2d", inputs=["x"], in_channels=1, input_height=2, input_width=2)], [None],
              {"x": f(1, 2, 3, 4)}, f(2.5), 1e-5))
    k.append(("token_mean_pool", [make_desc("t0", "TokenMeanPool", inputs=["x"], seq_len=2, embed_dim=3)], [None], {"x": f(1, 2, 3, 4, 5, 6)},
              f(2.5, 3.5, 4.5), 1e-6))
    # Add / Multiply, :394-422
    k.append(("add", [make_desc("t0", "Add", inputs=["x", "y"])], [None], {"x": f(1, 2, 3), "y": f(4, 5, 6)}, f(5, 7, 9), 1e-6))
    k.append(("multiply", [make_desc("t0", "Multiply", inputs=["x", "y"])], [None], {"x": f(1, 2, 3), "y": f(4, 5, 6)}, f(4, 10, 18), 1e-6))
    # Concat, :427-440
    k.append(("concat", [make_desc("t0", "Concat", inputs=["x", "y", "z"])], [None], {"x": f(1, 2), "y": f(3), "z": f(4, 5)}, f(1, 2, 3, 4, 5), 1e-6))
    # Embedding (float ids), :511-535
    k.append(("embedding", [make_desc("t0", "Embedding", inputs=["x"], vocab_size=3, embed_dim=2, padding_idx=-1, params_count=6)],
              [f(0, 0, 1, 10, 2, 20)], {"x": f(1, 2)}, f(1, 10, 2, 20), 1e-6))
    # EmbeddingBag: ids [1, 2, 1], offsets [0, 2, 3] -> bag0 = tok1 + tok2, bag1 = tok1, :537-554
    k.append(("embedding_bag", [make_desc("t0", "EmbeddingBag", inputs=["ids", "offs"], vocab_size=3, embed_dim=2, padding_idx=-1, params_count=6)],
              [f(0, 0, 1, 10, 2, 20)], {"ids": f(1, 2, 1), "offs": f(0, 2, 3)}, f(3, 30, 1, 10), 1e-6))
    # recurrent layers with zero weights -> zero output, :598-648
    for kind, g in (("RNN", 1), ("GRU", 3), ("LSTM", 4)):
        nw = g * 4 * 3 + g * 4 * 4 + 2 * g * 4
        k.append((f"{kind.lower()}_zero_weights", [make_desc("r", kind, inputs=["x"], seq_len=2, in_features=3, out_features=4, use_bias=1, params_count=nw)],
                  [np.zeros(nw, np.float32)], {"x": f(1, 2, 3, 4, 5, 6)}, np.zeros(8, np.float32), 1e-6))
    # Embedding with padding_idx = 0 -> zero row, test_runtime_embedding_int_inputs.cpp:44-62 (ids 1, 0, 2)
    table = np.arange(12, dtype=np.float32)
    table[:] = [0, 1, 2, 3, 10, 11, 12, 13, 20, 21, 22, 23]
    k.append(("embedding_padding", [make_desc("t0", "Embedding", inputs=["x"], vocab_size=3, embed_dim=4, padding_idx=0, params_count=12)],
              [table], {"x": f(1, 0, 2)}, f(10, 11, 12, 13, 0, 0, 0, 0, 20, 21, 22, 23), 1e-6))
    # named routing a+b -> sum, sum*c -> x, test_layers_named_routing.cpp:14-40
    k.append(("routing", [make_desc("add", "Add", inputs=["a", "b"], output="sum"), make_desc("mul", "Multiply", inputs=["sum", "c"], output="x")],
              [None, None], {"a": f(1, 2, 3), "b": f(10, 20, 30), "c": f(2, 2, 2)}, f(22, 44, 66), 1e-6))
    # DepthwiseConv2d k=1 -> scale by 3, test_layers_all_types.cpp:135-169
    k.append(("depthwise_k1", [make_desc("t0", "DepthwiseConv2d", in_channels=1, input_height=2, input_width=2, raw_kernel_h=1, raw_stride_h=1,
                                         raw_pad_h=0, use_bias=0, params_count=1)], [f(3)], {"x": f(1, 2, 3, 4)}, f(3, 6, 9, 12), 1e-6))
    # Conv1d k=1 -> scale by 4, :171-200
    k.append(("conv1d_k1", [make_desc("t0", "Conv1d", in_channels=1, out_channels=1, raw_kernel_h=1, raw_stride_h=1, raw_pad_h=0, use_bias=0,
                                      params_count=1)], [f(4)], {"x": f(1, 2, 3)}, f(4, 8, 12), 1e-6))
    # MaxPool2d / AvgPool2d 2x2 stride 2 on [1,2,3,4], :345-363
    pool = dict(in_channels=1, input_height=2, input_width=2, kernel=2, stride=2, padding=0)
    k.append(("maxpool", [make_desc("t0", "MaxPool2d", **pool)], [None], {"x": f(1, 2, 3, 4)}, f(4), 1e-6))
    k.append(("avgpool", [make_desc("t0", "AvgPool2d", **pool)], [None], {"x": f(1, 2, 3, 4)}, f(2.5), 1e-5))
    # Subtract / Divide, :405-421
    k.append(("subtract", [make_desc("t0", "Subtract", inputs=["x", "y"])], [None], {"x": f(1, 2, 3), "y": f(4, 5, 6)}, f(-3, -3, -3), 1e-6))
    k.append(("divide", [make_desc("t0", "Divide", inputs=["x", "y"])], [None], {"x": f(1, 2, 3), "y": f(4, 5, 6)}, f(0.25, 0.4, 0.5), 1e-6))
    # Split [2,2] then Concat gives the input back, :442-466
    k.append(("split_concat", [make_desc("split", "Split", inputs=["x"], output="s", split_sizes=[2, 2]),
                               make_desc("cat", "Concat", inputs=["s_0", "s_1"], output="x")], [None, None], {"x": f(1, 2, 3, 4)}, f(1, 2, 3, 4), 1e-6))
    # MatMul 2x3 . 3x2, :470-506
    k.append(("matmul", [make_desc("mm", "MatMul", inputs=["a", "b"], in_features=2, out_features=3, embed_dim=2)], [None],
              {"a": f(1, 2, 3, 4, 5, 6), "b": f(7, 8, 9, 10, 11, 12)}, f(58, 64, 139, 154), 1e-6))
    # PixelShuffle r=2 of 4 channels 1x1, :560-577; ZeroPad2d 1x1 pad 1, :579-592
    k.append(("pixel_shuffle", [make_desc("t0", "PixelShuffle", in_channels=4, input_height=1, input_width=1, scale_h=2)], [None],
              {"x": f(10, 11, 12, 13)}, f(10, 11, 12, 13), 1e-6))
    k.append(("zero_pad", [make_desc("t0", "ZeroPad2d", in_channels=1, input_height=1, input_width=1, raw_pad_h=1, raw_pad_w=1)], [None],
              {"x": f(5)}, f(0, 0, 0, 0, 5, 0, 0, 0, 0), 1e-6))
    return k


def layernorm_property_case():
    # test_layers_all_types.cpp:267-301: output of LayerNorm over [1,2,3,4] has mean 0 and variance 1
    return [make_desc("t0", "LayerNorm", inputs=["x"], in_features=4, affine=1, use_bias=1, eps=1e-6, params_count=8)], \
        [np.array([1, 1, 1, 1, 0, 0, 0, 0], np.float32)], {"x": np.array([1, 2, 3, 4], np.float32)}
