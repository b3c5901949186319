"""Small configurations of every architecture in the reference's registry
(Models/Registry/ModelArchitectures.cpp) and the named inputs each graph reads.  The layer lists
themselves are produced by the reference's own builders (ModelArchitectures::create) and committed
as tests/golden/registry_graphs.json by tests/golden/make_golden.py."""
import json
import os

import numpy as np

from mimir_framework_b200 import configs
from mimir_framework_b200.abi import desc_from_dict

HERE = os.path.dirname(os.path.abspath(__file__))

CFG = {
    "basic_mlp": dict(input_dim=24, hidden_dim=32, output_dim=10, hidden_layers=2),
    "transformer": dict(seq_len=8, d_model=16, vocab_size=50, num_layers=1, num_heads=2, mlp_hidden=24, output_dim=8, causal=False),
    "vit": dict(num_tokens=9, d_model=16, num_layers=1, num_heads=2, mlp_hidden=24, output_dim=5),
    "vae": dict(image_w=8, image_h=8, image_c=1, latent_dim=6, hidden_dim=20),
    "vae_conv": dict(image_w=16, image_h=16, image_c=3, latent_h=4, latent_w=4, latent_c=4, base_channels=8),
    "vae_conv_decode": dict(image_w=16, image_h=16, image_c=3, latent_h=4, latent_w=4, latent_c=4, base_channels=8),
    "resnet": dict(image_w=16, image_h=16, image_c=3, base_channels=8, num_classes=5, blocks1=1, blocks2=1, blocks3=1, blocks4=1),
    "unet": dict(image_w=16, image_h=16, image_c=3, base_channels=8, depth=2),
    "mobilenet": dict(image_w=16, image_h=16, image_c=3, base_channels=8, num_classes=5),
    "vgg16": dict(image_w=32, image_h=32, image_c=3, base_channels=4, num_classes=5, fc_hidden=16),
    "vgg19": dict(image_w=32, image_h=32, image_c=3, base_channels=4, num_classes=5, fc_hidden=16),
    "vgg16_feat": dict(image_w=32, image_h=32, image_c=3, base_channels=4),
    "patch_discriminator": dict(image_w=16, image_h=16, image_c=3, base_channels=4, num_down=2),
    "diffusion": dict(image_w=4, image_h=4, image_c=1, time_dim=4, hidden_dim=16),
    "gan_latent": dict(prompt_dim=6, noise_dim=4, latent_dim=8, hidden_dim=12, num_hidden_layers=2),
    "cond_diffusion": dict(prompt_dim=6, latent_w=2, latent_h=2, latent_c=2, time_dim=4, hidden_dim=16),
    "sd3_5": dict(stub_only=False, q_len=6, kv_len=5, d_model=16, num_heads=2, num_layers=1, mlp_hidden=24, causal=False),
    "vae_text": dict(vocab_size=40, seq_len=6, d_model=16, num_layers=1, num_heads=2, mlp_hidden=24, latent_tokens=3, proj_dim=8),
    "vae_text_decode": dict(vocab_size=40, seq_len=6, d_model=16, num_layers=1, num_heads=2, mlp_hidden=24, latent_tokens=3, proj_dim=8),
    "ponyxl_ddpm": dict(d_model=16, max_vocab=40, text_ctx_len=5, latent_seq_len=4, latent_in_dim=8, num_heads=2, unet_layers=1,
                        text_layers=1, mlp_hidden=24, latent_h=4, latent_w=4, unet_depth=1, image_w=16, image_h=16, image_c=3,
                        vae_base_channels=4),
}


def external_inputs(descs):
    """Names a graph reads before any layer defines them (besides the main input "x")."""
    produced, ext = {"x", "__input__"}, []
    for d in descs:
        for i in ([d.inputs[j].decode() for j in range(d.n_inputs)] or ["x"]):
            if i not in produced and i not in ext:
                ext.append(i)
        out = (d.output or b"x").decode() or "x"
        produced.add(out)
        if d.type.decode() in ("Split", "Chunk"):
            produced.update(f"{out}_{k}" for k in range(16))
    return ext


def input_sizes(arch):
    c = CFG[arch]
    img = lambda: c["image_w"] * c["image_h"] * c["image_c"]  # noqa: E731
    table = {
        "basic_mlp": lambda: {"x": c["input_dim"]},
        "transformer": lambda: {"x": c["seq_len"], "mag": c["d_model"], "mod": c["d_model"]},
        "vit": lambda: {"x": c["num_tokens"] * c["d_model"]},
        "vae": lambda: {"x": img()},
        "vae_conv": lambda: {"x": img()},
        "vae_conv_decode": lambda: {"x": c["latent_h"] * c["latent_w"] * c["latent_c"]},
        "diffusion": lambda: {"x": img() + c["time_dim"]},
        "gan_latent": lambda: {"x": c["prompt_dim"] + c["noise_dim"]},
        "cond_diffusion": lambda: {"x": c["prompt_dim"] + c["latent_w"] * c["latent_h"] * c["latent_c"] + c["time_dim"]},
        "sd3_5": lambda: {"x": (c["q_len"] + c["kv_len"]) * c["d_model"]},
        "vae_text": lambda: {"x": c["seq_len"], "text_ids": c["seq_len"]},
        "vae_text_decode": lambda: {"x": c["latent_tokens"] * c["d_model"]},
        "ponyxl_ddpm": lambda: {"x": 1, "latent": c["latent_seq_len"] * c["latent_in_dim"], "text_ids": c["text_ctx_len"],
                                "mag": c["d_model"], "mod": c["d_model"], "timestep": 1},
    }
    return table.get(arch, lambda: {"x": img()})()


def make_inputs(arch, seed=0):
    r = np.random.default_rng(seed)
    out = {}
    for k, n in input_sizes(arch).items():
        if k == "text_ids" or (arch in ("transformer", "vae_text") and k == "x"):
            vocab = CFG[arch].get("vocab_size", CFG[arch].get("max_vocab", 40))
            out[k] = r.integers(0, vocab, n).astype(np.float32)
        elif k == "timestep":
            out[k] = np.array([0.37], np.float32)
        else:
            out[k] = r.standard_normal(n).astype(np.float32)
    return out


def make_weights(descs):
    """Seeded weights with a fan-in scaled spread (std = sqrt(2 / fan_in)) so that activations stay of
    order one through the deep convolution stacks; norm layers gamma = 1, beta = 0; biases zero."""
    r = np.random.default_rng(5)
    out = []
    for d in descs:
        n, t = int(d.params_count), d.type.decode()
        if n == 0:
            out.append(None)
            continue
        if t in ("LayerNorm", "GroupNorm", "InstanceNorm2d"):
            half = n // 2 if d.use_bias else n
            out.append(np.concatenate([np.ones(half, np.float32), np.zeros(n - half, np.float32)]))
            continue
        if t in ("RMSNorm", "BatchNorm2d", "BatchNorm1d"):
            out.append(np.ones(n, np.float32))
            continue
        k = d.kernel if t in ("Conv2d", "ConvTranspose2d") else (d.raw_kernel_h if d.raw_kernel_h > 0 else 3)
        fan = {"Linear": max(d.in_features, 1), "Conv2d": d.in_channels * k * k, "ConvTranspose2d": d.in_channels * k * k,
               "DepthwiseConv2d": k * k, "Conv1d": max(d.in_channels, 1) * k, "Embedding": 2}.get(t, max(d.embed_dim, 1))
        w = (r.standard_normal(n, dtype=np.float32) * np.float32(np.sqrt(2.0 / fan))).astype(np.float32)
        if t == "Linear" and d.use_bias:
            w[n - d.out_features:] = 0.0
        out.append(w)
    return out


def load_registry_graphs():
    """[(arch, descs, inputs, expected output of the compiled reference)] from the committed fixture."""
    with open(os.path.join(HERE, "golden", "registry_graphs.json")) as fh:
        j = json.load(fh)
    arrays = np.load(os.path.join(HERE, "golden", "registry_graphs.npz"))
    out = []
    for arch, layers in j["graphs"].items():
        descs = [desc_from_dict(d) for d in layers]
        inputs = {k[len(arch) + 4:]: arrays[k] for k in arrays.files if k.startswith(arch + "/in/")}
        out.append((arch, descs, inputs, arrays[arch + "/out"]))
    return out
