"""Layer graphs and seeded synthetic tensors of the benchmark configurations.

Graphs are expressed as ``MimirLayerDesc`` lists, i.e. exactly what the Layer->descriptor shim
produces from a Mímir ``std::vector<Layer>``.  All data is synthetic: numpy ``default_rng(seed)``
with the distributions each configuration names.
"""
from __future__ import annotations

import numpy as np

from .abi import make_desc

# ---- configuration 2: stand-alone Linear + bias + GELU stack ------------------------------------
LINEAR_STACK_K = 4096
LINEAR_STACK_LAYERS = 3


def linear_gelu_stack(rows: int, k: int = LINEAR_STACK_K, layers: int = LINEAR_STACK_LAYERS):
    """`layers` x [Linear k->k (seq_len = rows, bias) -> GELU], GELU after the last Linear too."""
    descs = []
    prev = "x"
    for i in range(layers):
        lin_out = f"stack/l{i}"
        act_out = "x" if i == layers - 1 else f"stack/a{i}"
        descs.append(make_desc(f"stack/linear{i}", "Linear", inputs=[prev], output=lin_out, in_features=k,
                               out_features=k, seq_len=rows, use_bias=1, params_count=k * k + k))
        descs.append(make_desc(f"stack/gelu{i}", "GELU", inputs=[lin_out], output=act_out))
        prev = act_out
    return descs


def linear_gelu_stack_weights(k: int = LINEAR_STACK_K, layers: int = LINEAR_STACK_LAYERS):
    """W ~ U(-1/sqrt(k), 1/sqrt(k)), bias ~ U(-0.1, 0.1); seeds 10, 11, 12 per layer.  One flat block
    per Linear in the reference's layout (W[out][in] then bias); GELU layers have no block."""
    out = []
    for i in range(layers):
        r = np.random.default_rng(10 + i)
        bound = 1.0 / np.sqrt(k)
        w = r.uniform(-bound, bound, k * k).astype(np.float32)
        b = r.uniform(-0.1, 0.1, k).astype(np.float32)
        out.append(np.concatenate([w, b]))
        out.append(None)
    return out


def linear_gelu_stack_input(rows: int, k: int = LINEAR_STACK_K, seed: int = 9, row_offset: int = 0) -> np.ndarray:
    """x ~ N(0, 1), fp32 [rows, k]; `row_offset` lets ranks draw disjoint, reproducible slices."""
    r = np.random.default_rng([seed, row_offset])
    return r.standard_normal((rows, k), dtype=np.float32)


def linear_gelu_stack_flops(rows: int, k: int = LINEAR_STACK_K, layers: int = LINEAR_STACK_LAYERS) -> int:
    return 2 * rows * k * k * layers


# ---- configuration 1: registry transformer encoder -----------------------------------------------
TRANSFORMER_CFG = dict(seq_len=128, d_model=256, vocab_size=8192, num_layers=2, num_heads=4, mlp_hidden=1024,
                       output_dim=256, causal=False)


def transformer_encoder(seq_len=128, d_model=256, vocab_size=8192, num_layers=2, num_heads=4, mlp_hidden=1024,
                        output_dim=256, causal=False, padding_idx=0):
    """The graph TransformerModel::buildInto pushes (TransformerModel.cpp:22-173): Embedding ->
    +mag -> +mod -> N x [LayerNorm(whole vector) -> MultiHeadAttention -> Add -> LayerNorm -> Linear
    over the flattened sequence -> GELU -> Linear -> Add] -> Linear head."""
    in_dim = seq_len * d_model
    p = "transformer"
    d = [
        make_desc(f"{p}/tok_embed", "Embedding", inputs=["__input__"], output=f"{p}/in", vocab_size=vocab_size,
                  embed_dim=d_model, padding_idx=padding_idx, params_count=vocab_size * d_model),
        make_desc(f"{p}/mag_in", "Identity", inputs=["mag"], output=f"{p}/mag_vec"),
        make_desc(f"{p}/add_mag", "Add", inputs=[f"{p}/in", f"{p}/mag_vec"], output=f"{p}/in_plus_mag"),
        make_desc(f"{p}/mod_in", "Identity", inputs=["mod"], output=f"{p}/mod_vec"),
        make_desc(f"{p}/add_mod", "Add", inputs=[f"{p}/in_plus_mag", f"{p}/mod_vec"], output=f"{p}/in_plus_mag_mod"),
    ]
    x = f"{p}/in_plus_mag_mod"
    for i in range(num_layers):
        b = f"{p}/block{i + 1}"
        d += [
            make_desc(f"{b}/ln1", "LayerNorm", inputs=[x], output=f"{b}/ln1_out", affine=1, use_bias=1, eps=1e-5,
                      params_count=2 * in_dim),
            make_desc(f"{b}/attn", "MultiHeadAttention", inputs=[f"{b}/ln1_out"], output=f"{b}/attn_out", seq_len=seq_len,
                      embed_dim=d_model, num_heads=num_heads, causal=int(causal), params_count=4 * d_model * d_model),
            make_desc(f"{b}/add1", "Add", inputs=[x, f"{b}/attn_out"], output=f"{b}/res1"),
            make_desc(f"{b}/ln2", "LayerNorm", inputs=[f"{b}/res1"], output=f"{b}/ln2_out", affine=1, use_bias=1, eps=1e-5,
                      params_count=2 * in_dim),
            make_desc(f"{b}/mlp_fc1", "Linear", inputs=[f"{b}/ln2_out"], output=f"{b}/mlp_h", in_features=in_dim,
                      out_features=mlp_hidden, use_bias=1, params_count=in_dim * mlp_hidden + mlp_hidden),
            make_desc(f"{b}/mlp_act", "GELU", inputs=[f"{b}/mlp_h"], output=f"{b}/mlp_h_act"),
            make_desc(f"{b}/mlp_fc2", "Linear", inputs=[f"{b}/mlp_h_act"], output=f"{b}/mlp_out", in_features=mlp_hidden,
                      out_features=in_dim, use_bias=1, params_count=mlp_hidden * in_dim + in_dim),
            make_desc(f"{b}/add2", "Add", inputs=[f"{b}/res1", f"{b}/mlp_out"], output=f"{b}/res2"),
        ]
        x = f"{b}/res2"
    d.append(make_desc(f"{p}/head", "Linear", inputs=[x], output="x", in_features=in_dim, out_features=output_dim,
                       use_bias=1, params_count=in_dim * output_dim + output_dim))
    return d


def seeded_weights(descs, seed: int = 1, std: float = 0.02, bf16: bool = False):
    """All weights N(0, std) from one generator in layer order; Linear biases zero; norm layers
    gamma = 1, beta = 0 (an N(0, 0.02) gamma would zero the signal)."""
    r = np.random.default_rng(seed)
    out = []
    for d in descs:
        n = int(d.params_count)
        t = d.type.decode()
        if n == 0:
            out.append(None)
            continue
        if t in ("LayerNorm", "GroupNorm"):
            half = n // 2 if d.use_bias else n
            w = np.concatenate([np.ones(half, np.float32), np.zeros(n - half, np.float32)])
        elif t == "RMSNorm":
            w = np.ones(n, np.float32)
        else:
            w = (r.standard_normal(n, dtype=np.float32) * np.float32(std)).astype(np.float32)
            if t == "Linear" and d.use_bias:
                w[n - d.out_features:] = 0.0
            if bf16:
                w = round_to_bf16(w)
        out.append(w)
    return out


def round_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned as fp32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)
