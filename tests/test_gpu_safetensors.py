"""The checkpoint -> device loader (mimir_b200_model_load_safetensors) against checkpoints written by
the reference's own SafeTensorsWriter and against hand-built files."""
import json
import struct

import numpy as np
import pytest

import registry_cases as rc
from conftest import assert_close
from oracle import ref

pytestmark = pytest.mark.gpu
GRAPHS = {g[0]: g for g in rc.load_registry_graphs()}


def write_safetensors(path, tensors):
    """tensors: name -> (dtype string, numpy array holding the raw payload)."""
    header, off, blobs = {}, 0, []
    for name, (dtype, arr, shape) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    header["__metadata__"] = {"format": "safetensors", "note": "nested \"quotes\" and [brackets] {braces}", "n": 3}
    h = json.dumps(header).encode()
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def forward(backend, m, inputs, out_n):
    m.plan({k: (v.size, False) for k, v in inputs.items()}, 1)
    return m.forward({k: (v, False) for k, v in inputs.items()}, 1, out_n).ravel()


@pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not built here")
@pytest.mark.parametrize("arch", ["sd3_5", "mobilenet", "vae_text"])
def test_loads_checkpoint_written_by_the_reference(backend, tmp_path, arch):
    _, descs, inputs, want = GRAPHS[arch]
    rm = ref.RefModel(registry=arch, cfg_json=json.dumps(rc.CFG[arch]))
    weights = rc.make_weights(rm.layer_descs())
    for i, w in enumerate(weights):
        if w is not None:
            rm.set_weights(i, w)
    path = str(tmp_path / f"{arch}.safetensors")
    rm.save_safetensors(path)
    m = backend.GraphModel(descs)
    n_layers, n_bytes = m.load_safetensors(path)
    assert n_layers == sum(w is not None for w in weights)
    assert n_bytes == 4 * sum(w.size for w in weights if w is not None)
    got = forward(backend, m, inputs, want.size)
    m.close()
    # same device weights as the upload path -> identical results
    m2 = backend.GraphModel(descs)
    for i, w in enumerate(weights):
        m2.upload_weights(i, w)
    assert np.array_equal(got, forward(backend, m2, inputs, want.size))
    m2.close()
    assert_close(got, want, arch)


def test_hand_built_file_bf16_and_large_tensor(backend, tmp_path):
    from mimir_framework_b200.abi import make_desc
    from mimir_framework_b200.configs import round_to_bf16
    k, n = 3000, 3500  # 42 MB of fp32: more than one 32 MB staging chunk
    descs = [make_desc("fc", "Linear", in_features=k, out_features=n, use_bias=1, params_count=k * n + n),
             make_desc("norm", "LayerNorm", in_features=n, params_count=2 * n)]
    r = np.random.default_rng(3)
    w0 = (r.standard_normal(k * n + n) * 0.02).astype(np.float32)
    w1 = round_to_bf16(np.concatenate([1 + 0.1 * r.standard_normal(n), 0.1 * r.standard_normal(n)]).astype(np.float32))
    bf = (w1.view(np.uint32) >> 16).astype(np.uint16)
    path = str(tmp_path / "hand.safetensors")
    write_safetensors(path, {"unrelated/blob": ("U8", np.arange(13, dtype=np.uint8), [13]),
                             "fc/weights": ("F32", w0, [k * n + n]),
                             "norm/weights": ("BF16", bf, [2, n])})
    x = r.standard_normal(k).astype(np.float32)
    m = backend.GraphModel(descs)
    assert m.load_safetensors(path)[0] == 2
    got = forward(backend, m, {"x": x}, n)
    m.close()
    m2 = backend.GraphModel(descs)
    m2.upload_weights(0, w0)
    m2.upload_weights(1, w1)
    assert np.array_equal(got, forward(backend, m2, {"x": x}, n))
    m2.close()


def test_error_behaviour_follows_the_reference_reader(backend, tmp_path):
    from mimir_framework_b200.abi import make_desc
    descs = [make_desc("a", "Linear", in_features=4, out_features=2, use_bias=0, params_count=8),
             make_desc("b", "Linear", in_features=2, out_features=2, use_bias=0, params_count=4)]
    path = str(tmp_path / "partial.safetensors")
    write_safetensors(path, {"a/weights": ("F32", np.ones(8, np.float32), [8])})
    m = backend.GraphModel(descs)
    with pytest.raises(backend.MimirB200Error, match="Missing tensor in strict mode: b/weights"):
        m.load_safetensors(path, strict=True)
    assert m.load_safetensors(path, strict=False)[0] == 1  # non-strict: the layer keeps whatever it had
    write_safetensors(path, {"a/weights": ("F32", np.ones(6, np.float32), [6]), "b/weights": ("F32", np.ones(4, np.float32), [4])})
    with pytest.raises(backend.MimirB200Error, match="Size mismatch for a/weights"):
        m.load_safetensors(path)
    write_safetensors(path, {"a/weights": ("F16", np.ones(8, np.float16), [8]), "b/weights": ("F32", np.ones(4, np.float32), [4])})
    with pytest.raises(backend.MimirB200Error, match="dtype F16"):
        m.load_safetensors(path)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", 20) + b"{not json at all....")
    with pytest.raises(backend.MimirB200Error, match="not valid JSON"):
        m.load_safetensors(path)
    with pytest.raises(backend.MimirB200Error, match="cannot open"):
        m.load_safetensors(str(tmp_path / "nope.safetensors"))
    m.close()


def test_untrusted_header_values_are_checked_before_any_weight_is_touched(backend, tmp_path):
    """Offsets that wrap around, a shape whose product overflows, and a second tensor that is bad: every one is refused,
    and the model still computes with the weights it had before the failed load (nothing is half-loaded)."""
    import json as js
    from mimir_framework_b200.abi import make_desc
    descs = [make_desc("a", "Linear", inputs=["x"], output="h", in_features=4, out_features=4, use_bias=0, params_count=16),
             make_desc("b", "Linear", inputs=["h"], output="x", in_features=4, out_features=2, use_bias=0, params_count=8)]
    r = np.random.default_rng(0)
    wa, wb = r.standard_normal(16).astype(np.float32), r.standard_normal(8).astype(np.float32)
    m = backend.GraphModel(descs)
    m.upload_weights(0, wa)
    m.upload_weights(1, wb)
    x = r.standard_normal(4).astype(np.float32)
    before = forward(backend, m, {"x": x}, 2)

    def write_raw(path, header: dict, payload: bytes):
        h = js.dumps(header).encode()
        with open(path, "wb") as fh:
            fh.write(struct.pack("<Q", len(h)) + h + payload)
    path = str(tmp_path / "bad.safetensors")
    big = 2 ** 64 - 128
    cases = [
        # begin / end close to 2^64 with the right difference: their sum with the data start wraps
        ({"a/weights": {"dtype": "F32", "shape": [16], "data_offsets": [big, big + 64]},
          "b/weights": {"dtype": "F32", "shape": [8], "data_offsets": [0, 32]}}, "data_offsets of a/weights"),
        # a shape whose element product overflows 64 bits
        ({"a/weights": {"dtype": "F32", "shape": [2 ** 40, 2 ** 40], "data_offsets": [0, 64]},
          "b/weights": {"dtype": "F32", "shape": [8], "data_offsets": [64, 96]}}, "Size mismatch for a/weights"),
        # the first tensor is fine, the second runs past the end of the file
        ({"a/weights": {"dtype": "F32", "shape": [16], "data_offsets": [0, 64]},
          "b/weights": {"dtype": "F32", "shape": [8], "data_offsets": [64, 96]}}, "data_offsets of b/weights"),
    ]
    for header, msg in cases:
        write_raw(path, header, np.full(16, 7.0, np.float32).tobytes())  # 64 bytes of payload only
        with pytest.raises(backend.MimirB200Error, match=msg):
            m.load_safetensors(path)
        assert np.array_equal(forward(backend, m, {"x": x}, 2), before), "a failed load changed the model"
    # "expected" is the layer's parameter count, "got" the tensor's element count
    write_safetensors(path, {"a/weights": ("F32", np.ones(6, np.float32), [6]), "b/weights": ("F32", np.ones(8, np.float32), [8])})
    with pytest.raises(backend.MimirB200Error, match="expected 16 got 6"):
        m.load_safetensors(path)
    m.close()
