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


# ---- configuration 3: GPT-style causal decoder, prefill only -------------------------------------
DECODER_CFG = dict(layers=12, d_model=768, heads=12, ffn=3072, vocab=32000, seq=1024)


def gpt_decoder(layers=12, d_model=768, heads=12, ffn=3072, vocab=32000, seq=1024, norm="rms"):
    """Embedding -> layers x [RMSNorm -> MultiHeadAttention(causal) -> Add -> RMSNorm -> Linear -> GELU ->
    Linear -> Add] -> RMSNorm -> Linear (LM head), token-wise layers (`seq_len` set) like the
    reference's ViT / SD3.5 builders.  RMSNorm is the reference's whole-tensor form with one gamma per
    element (`params_count = seq * d_model`)."""
    E, S = d_model, seq

    def norm_desc(name, src, dst):
        # "layer": token-wise LayerNorm (in_features = E), the form under which every row depends on its own past only
        if norm == "layer":
            return make_desc(name, "LayerNorm", inputs=[src], output=dst, in_features=E, affine=1, use_bias=1, params_count=2 * E)
        return make_desc(name, "RMSNorm", inputs=[src], output=dst, params_count=S * E)

    d = [make_desc("dec/tok_embed", "Embedding", inputs=["__input__"], output="dec/h0", vocab_size=vocab, embed_dim=E,
                   padding_idx=-1, params_count=vocab * E)]
    x = "dec/h0"
    for i in range(layers):
        b = f"dec/block{i}"
        d += [
            norm_desc(f"{b}/norm1", x, f"{b}/n1"),
            make_desc(f"{b}/attn", "MultiHeadAttention", inputs=[f"{b}/n1"], output=f"{b}/a", seq_len=S, embed_dim=E,
                      num_heads=heads, causal=1, params_count=4 * E * E),
            make_desc(f"{b}/add1", "Add", inputs=[x, f"{b}/a"], output=f"{b}/r1"),
            norm_desc(f"{b}/norm2", f"{b}/r1", f"{b}/n2"),
            make_desc(f"{b}/fc1", "Linear", inputs=[f"{b}/n2"], output=f"{b}/f1", in_features=E, out_features=ffn, seq_len=S,
                      use_bias=1, params_count=E * ffn + ffn),
            make_desc(f"{b}/gelu", "GELU", inputs=[f"{b}/f1"], output=f"{b}/f1a"),
            make_desc(f"{b}/fc2", "Linear", inputs=[f"{b}/f1a"], output=f"{b}/f2", in_features=ffn, out_features=E, seq_len=S,
                      use_bias=1, params_count=ffn * E + E),
            make_desc(f"{b}/add2", "Add", inputs=[f"{b}/r1", f"{b}/f2"], output=f"{b}/r2"),
        ]
        x = f"{b}/r2"
    d += [norm_desc("dec/norm_f", x, "dec/nf"),
          make_desc("dec/lm_head", "Linear", inputs=["dec/nf"], output="x", in_features=E, out_features=vocab, seq_len=S,
                    use_bias=0, params_count=E * vocab)]
    return d


def gpt_decoder_flops(layers=12, d_model=768, heads=12, ffn=3072, vocab=32000, seq=1024):
    """Algorithmic flops per sample; attention counted on the causal half."""
    E, S = d_model, seq
    per_layer = 2 * S * E * 3 * E + 2 * S * S * E + 2 * S * E * E + 2 * 2 * S * E * ffn
    return layers * per_layer + 2 * S * E * vocab


def gpt_decoder_gemm_flops(layers=12, d_model=768, heads=12, ffn=3072, vocab=32000, seq=1024):
    """The part of gpt_decoder_flops that runs in the projection GEMMs (everything but the attention core)."""
    return gpt_decoder_flops(layers, d_model, heads, ffn, vocab, seq) - layers * 2 * seq * seq * d_model


# ---- configuration 4: conv vision block stack ------------------------------------------------------
def conv_stack(image=224, channels=(64, 128, 128, 256, 256), groups=32):
    """Stem Conv 7x7 s2 p3 3->C0, then per block [Conv 3x3 s1 p1 -> GroupNorm -> SiLU -> Add residual]; where
    the channel count changes the skip is a 1x1 conv (no bias anywhere: the reference never adds conv bias)."""
    hw = (image + 2 * 3 - 7) // 2 + 1
    d = [make_desc("cv/stem", "Conv2d", inputs=["x"], output="cv/s", in_channels=3, out_channels=channels[0], input_height=image,
                   input_width=image, kernel=7, stride=2, padding=3, params_count=channels[0] * 3 * 49)]
    x, c_in = "cv/s", channels[0]
    for i, c_out in enumerate(channels[1:]):
        b = f"cv/b{i}"
        last = i == len(channels) - 2
        d += [
            make_desc(f"{b}/conv", "Conv2d", inputs=[x], output=f"{b}/c", in_channels=c_in, out_channels=c_out, input_height=hw,
                      input_width=hw, kernel=3, stride=1, padding=1, params_count=c_out * c_in * 9),
            make_desc(f"{b}/gn", "GroupNorm", inputs=[f"{b}/c"], output=f"{b}/g", in_channels=c_out, input_height=hw, input_width=hw,
                      num_groups=groups, params_count=2 * c_out),
            make_desc(f"{b}/act", "SiLU", inputs=[f"{b}/g"], output=f"{b}/a"),
        ]
        skip = x
        if c_in != c_out:
            d.append(make_desc(f"{b}/skip", "Conv2d", inputs=[x], output=f"{b}/s", in_channels=c_in, out_channels=c_out,
                               input_height=hw, input_width=hw, kernel=1, stride=1, padding=0, params_count=c_out * c_in))
            skip = f"{b}/s"
        d.append(make_desc(f"{b}/add", "Add", inputs=[f"{b}/a", skip], output="x" if last else f"{b}/o"))
        x, c_in = f"{b}/o", c_out
    return d


def conv_stack_weights(descs, seed=1):
    """Kaiming-normal conv weights N(0, sqrt(2 / (ic k^2))), GroupNorm gamma = 1, beta = 0."""
    r = np.random.default_rng(seed)
    out = []
    for d in descs:
        t, n = d.type.decode(), int(d.params_count)
        if t == "Conv2d":
            fan = d.in_channels * d.kernel * d.kernel
            out.append((r.standard_normal(n, dtype=np.float32) * np.float32(np.sqrt(2.0 / fan))).astype(np.float32))
        elif t == "GroupNorm":
            out.append(np.concatenate([np.ones(n // 2, np.float32), np.zeros(n - n // 2, np.float32)]))
        else:
            out.append(None)
    return out


def conv_flops(descs):
    """Sum of 2 * oc * ic * k^2 * H_out * W_out over the Conv2d layers (per sample)."""
    f = 0
    for d in descs:
        if d.type.decode() == "Conv2d":
            oh = (d.input_height + 2 * d.padding - d.kernel) // d.stride + 1
            ow = (d.input_width + 2 * d.padding - d.kernel) // d.stride + 1
            f += 2 * d.out_channels * d.in_channels * d.kernel * d.kernel * oh * ow
    return f


# ---- configuration 5: UNet / VAE-decoder style mid + up path ----------------------------------------
def unet_mid_up(latent=64, base=512, groups=32):
    """Frozen interpretation of the loosely specified configuration: conv_in 4->512 @latent^2; two stride-2
    3x3 convs down to (latent/4)^2; mid = ResBlock -> [GroupNorm -> Permute CHW->[tokens, C] ->
    SelfAttention(1 head) -> Permute back -> Add] -> ResBlock; up = 4 x [UpsampleNearest 2x -> ResBlock]
    with channels 512 -> 512 -> 256 -> 128 -> 128; GroupNorm -> SiLU -> conv_out 128 -> 3.
    ResBlock = GN -> SiLU -> Conv3x3 -> GN -> SiLU -> Conv3x3 + skip (1x1 conv when channels change)."""
    d = []
    n = [0]

    def conv(x, out, ic, oc, hw, k=3, s=1, p=1):
        n[0] += 1
        d.append(make_desc(f"u/conv{n[0]}", "Conv2d", inputs=[x], output=out, in_channels=ic, out_channels=oc, input_height=hw,
                           input_width=hw, kernel=k, stride=s, padding=p, params_count=oc * ic * k * k))

    def gn_silu(x, out, c, hw):
        n[0] += 1
        d.append(make_desc(f"u/gn{n[0]}", "GroupNorm", inputs=[x], output=out + "_g", in_channels=c, input_height=hw, input_width=hw,
                           num_groups=groups, params_count=2 * c))
        d.append(make_desc(f"u/silu{n[0]}", "SiLU", inputs=[out + "_g"], output=out))

    def resblock(x, out, ic, oc, hw):
        t = out + "_t"
        gn_silu(x, t + "1", ic, hw)
        conv(t + "1", t + "2", ic, oc, hw)
        gn_silu(t + "2", t + "3", oc, hw)
        conv(t + "3", t + "4", oc, oc, hw)
        skip = x
        if ic != oc:
            conv(x, t + "s", ic, oc, hw, k=1, s=1, p=0)
            skip = t + "s"
        n[0] += 1
        d.append(make_desc(f"u/add{n[0]}", "Add", inputs=[t + "4", skip], output=out))

    hw = latent
    conv("x", "u/in", 4, base, hw)
    conv("u/in", "u/d1", base, base, hw, s=2)
    hw //= 2
    conv("u/d1", "u/d2", base, base, hw, s=2)
    hw //= 2
    resblock("u/d2", "u/m1", base, base, hw)
    tokens = hw * hw
    n[0] += 1
    d.append(make_desc(f"u/gn{n[0]}", "GroupNorm", inputs=["u/m1"], output="u/an", in_channels=base, input_height=hw, input_width=hw,
                       num_groups=groups, params_count=2 * base))
    d.append(make_desc("u/to_tokens", "Permute", inputs=["u/an"], output="u/at", shape=[base, tokens], permute_dims=[1, 0]))
    d.append(make_desc("u/attn", "SelfAttention", inputs=["u/at"], output="u/ao", seq_len=tokens, embed_dim=base, num_heads=1,
                       params_count=4 * base * base))
    d.append(make_desc("u/to_chw", "Permute", inputs=["u/ao"], output="u/ac", shape=[tokens, base], permute_dims=[1, 0]))
    d.append(make_desc("u/attn_add", "Add", inputs=["u/m1", "u/ac"], output="u/m2"))
    resblock("u/m2", "u/m3", base, base, hw)
    x, c = "u/m3", base
    for i, oc in enumerate((base, base // 2, base // 4, base // 4)):
        d.append(make_desc(f"u/up{i}", "UpsampleNearest", inputs=[x], output=f"u/up{i}o", in_channels=c, out_h=hw, out_w=hw,
                           scale_h=2, scale_w=2))
        hw *= 2
        resblock(f"u/up{i}o", f"u/r{i}", c, oc, hw)
        x, c = f"u/r{i}", oc
    gn_silu(x, "u/fin", c, hw)
    n[0] += 1
    d.append(make_desc("u/conv_out", "Conv2d", inputs=["u/fin"], output="x", in_channels=c, out_channels=3, input_height=hw,
                       input_width=hw, kernel=3, stride=1, padding=1, params_count=3 * c * 9))
    return d
