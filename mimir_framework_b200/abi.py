"""ctypes view of ``include/mimir_b200.h``.

Only declarations live here: the structs (``MimirLayerDesc``, ``MimirNamedInput``,
``MimirB200Stats``), the status codes and the loader of ``libmimir_b200.so``.  The loader raises
if the library has not been built — there is no Python or CPU stand-in for any op.
"""
from __future__ import annotations

import ctypes as C
import os

MAX_INPUTS = 8
MAX_DIMS = 8
MAX_SPLITS = 16

OK, E_INVALID, E_UNSUPPORTED, E_OOM_BUDGET, E_CUDA, E_TIMEOUT, E_NOT_INIT = range(7)
STATUS_NAMES = ["OK", "E_INVALID", "E_UNSUPPORTED", "E_OOM_BUDGET", "E_CUDA", "E_TIMEOUT", "E_NOT_INIT"]

PREC_BF16X2, PREC_BF16W, PREC_BF16 = 0, 1, 2
ELT_ADD, ELT_MULTIPLY, ELT_GELU, ELT_SILU, ELT_RELU, ELT_TANH, ELT_SIGMOID = range(7)
ELT_LEAKY_RELU, ELT_SOFTPLUS, ELT_MISH, ELT_HARD_SIGMOID, ELT_HARD_SWISH, ELT_SUBTRACT, ELT_DIVIDE, ELT_ELU = range(7, 15)


class MimirLayerDesc(C.Structure):
    _fields_ = [
        ("name", C.c_char_p),
        ("type", C.c_char_p),
        ("inputs", C.c_char_p * MAX_INPUTS),
        ("n_inputs", C.c_int32),
        ("output", C.c_char_p),
        ("params_count", C.c_uint64),
        ("in_features", C.c_int32),
        ("out_features", C.c_int32),
        ("in_channels", C.c_int32),
        ("out_channels", C.c_int32),
        ("input_height", C.c_int32),
        ("input_width", C.c_int32),
        ("kernel", C.c_int32),
        ("stride", C.c_int32),
        ("padding", C.c_int32),
        ("eps", C.c_float),
        ("num_groups", C.c_int32),
        ("affine", C.c_int32),
        ("use_bias", C.c_int32),
        ("vocab_size", C.c_int32),
        ("embed_dim", C.c_int32),
        ("padding_idx", C.c_int32),
        ("num_heads", C.c_int32),
        ("seq_len", C.c_int32),
        ("causal", C.c_int32),
        ("out_h", C.c_int32),
        ("out_w", C.c_int32),
        ("scale_h", C.c_int32),
        ("scale_w", C.c_int32),
        ("activation", C.c_int32),
        ("n_dims", C.c_int32),
        ("shape", C.c_int32 * MAX_DIMS),
        ("permute_dims", C.c_int32 * MAX_DIMS),
        ("head_dim", C.c_int32),
        ("leaky_relu_alpha", C.c_float),
        ("kernel_w", C.c_int32),
        ("stride_w", C.c_int32),
        ("padding_w", C.c_int32),
        ("raw_kernel_h", C.c_int32),
        ("raw_stride_h", C.c_int32),
        ("raw_pad_h", C.c_int32),
        ("raw_pad_w", C.c_int32),
        ("n_splits", C.c_int32),
        ("split_sizes", C.c_int32 * MAX_SPLITS),
        ("num_chunks", C.c_int32),
        ("seq_text", C.c_int32),
        ("num_patches", C.c_int32),
        ("patch_dim", C.c_int32),
        ("target_dim0", C.c_int32),
    ]


class MimirNamedInput(C.Structure):
    _fields_ = [
        ("name", C.c_char_p),
        ("data", C.c_void_p),
        ("per_sample", C.c_uint64),
        ("broadcast", C.c_int32),
    ]


class MimirB200Stats(C.Structure):
    _fields_ = [
        ("arena_peak_bytes", C.c_uint64),
        ("weight_bytes", C.c_uint64),
        ("kernels_launched", C.c_uint64),
        ("flops_last_forward", C.c_uint64),
        ("bytes_last_forward", C.c_uint64),
        ("ms_last_forward", C.c_float),
    ]


# Defaults of the reference's `struct Layer` (Layers.hpp:86-219) for the fields the descriptor
# carries, after the accessor resolution the shim performs (kernel 3, stride 1, padding 0).
LAYER_DEFAULTS = dict(
    params_count=0, in_features=0, out_features=0, in_channels=0, out_channels=0,
    input_height=0, input_width=0, kernel=3, stride=1, padding=0, eps=1e-5, num_groups=1,
    affine=1, use_bias=1, vocab_size=0, embed_dim=0, padding_idx=-1, num_heads=8, seq_len=0,
    causal=0, out_h=0, out_w=0, scale_h=2, scale_w=2, activation=0,
    head_dim=64, leaky_relu_alpha=0.01, kernel_w=None, stride_w=None, padding_w=None,
    raw_kernel_h=0, raw_stride_h=1, raw_pad_h=0, raw_pad_w=0, num_chunks=2,
    seq_text=0, num_patches=0, patch_dim=0, target_dim0=0,
)
_FLOAT_FIELDS = ("eps", "leaky_relu_alpha")


def make_desc(name: str, type: str, inputs=(), output: str = "x", shape=(), permute_dims=(), split_sizes=(), **kw) -> MimirLayerDesc:
    """Builds one descriptor with the reference's Layer defaults for everything not given."""
    d = MimirLayerDesc()
    d.name = name.encode()
    d.type = type.encode()
    ins = list(inputs)
    if len(ins) > MAX_INPUTS:
        raise ValueError("too many inputs")
    for i, s in enumerate(ins):
        d.inputs[i] = s.encode()
    d.n_inputs = len(ins)
    d.output = output.encode()
    vals = dict(LAYER_DEFAULTS)
    for k, v in kw.items():
        if k not in vals:
            raise KeyError(f"unknown layer field {k!r}")
        vals[k] = v
    # the *_w accessors fall back to the square setting (Layers.hpp:251-257)
    for wk, hk in (("kernel_w", "kernel"), ("stride_w", "stride"), ("padding_w", "padding")):
        if vals[wk] is None:
            vals[wk] = vals[hk]
    for k, v in vals.items():
        setattr(d, k, v)
    if len(split_sizes) > MAX_SPLITS:
        raise ValueError("too many split sizes")
    d.n_splits = len(split_sizes)
    for i, v in enumerate(split_sizes):
        d.split_sizes[i] = int(v)
    if len(shape) != len(permute_dims) or len(shape) > MAX_DIMS:
        raise ValueError("shape / permute_dims mismatch")
    d.n_dims = len(shape)
    for i, (s, p) in enumerate(zip(shape, permute_dims)):
        d.shape[i] = s
        d.permute_dims[i] = p
    return d


def desc_array(descs) -> C.Array:
    arr = (MimirLayerDesc * len(descs))()
    for i, d in enumerate(descs):
        C.memmove(C.byref(arr, i * C.sizeof(MimirLayerDesc)), C.byref(d), C.sizeof(MimirLayerDesc))
    arr._keep = list(descs)  # keeps the byte strings alive
    return arr


def library_path() -> str:
    """The in-tree build; MIMIR_B200_LIB points at another build of the same library (A/B measurements)."""
    return os.environ.get("MIMIR_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libmimir_b200.so")


_lib = None


def load() -> C.CDLL:
    """Loads libmimir_b200.so (built by ``mimir_framework_b200.build``).  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m mimir_framework_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback."
        )
    _lib = C.CDLL(path)
    _lib.mimir_b200_last_error.restype = C.c_char_p
    return _lib


_SCALAR_FIELDS = [n for n, _ in MimirLayerDesc._fields_ if n not in ("name", "type", "inputs", "n_inputs", "output", "n_dims", "shape", "permute_dims", "n_splits", "split_sizes")]


def desc_to_dict(d: MimirLayerDesc) -> dict:
    """JSON-friendly form of a descriptor (used by the golden fixtures)."""
    out = {"name": (d.name or b"").decode(), "type": (d.type or b"").decode(),
           "inputs": [d.inputs[i].decode() for i in range(d.n_inputs)], "output": (d.output or b"x").decode() or "x",
           "shape": [int(d.shape[i]) for i in range(d.n_dims)], "permute_dims": [int(d.permute_dims[i]) for i in range(d.n_dims)],
           "split_sizes": [int(d.split_sizes[i]) for i in range(d.n_splits)]}
    for f in _SCALAR_FIELDS:
        v = getattr(d, f)
        out[f] = float(v) if f in _FLOAT_FIELDS else int(v)
    return out


def desc_from_dict(j: dict) -> MimirLayerDesc:
    kw = {f: j[f] for f in _SCALAR_FIELDS if f in j}
    return make_desc(j["name"], j["type"], inputs=j.get("inputs", []), output=j.get("output", "x"), shape=j.get("shape", []),
                     permute_dims=j.get("permute_dims", []), split_sizes=j.get("split_sizes", []), **kw)
