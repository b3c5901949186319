"""TEST INFRASTRUCTURE — ctypes binding of ``oracle/_ref/libmimir_ref.so``.

That library is the reference's own CPU implementation (compiled from its sources by
``oracle/Makefile``) behind ``oracle/ref_shim.cpp``.  Only tests, the fixture generator, the smoke
check and the benchmark's CPU arm import this module; the product never does.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from mimir_framework_b200.abi import MimirLayerDesc, MimirNamedInput, desc_array

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libmimir_ref.so")

_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(f"{LIB_PATH} not built: run `make -C oracle ref` where the reference is mounted")
        _lib = C.CDLL(LIB_PATH)
        _lib.mimir_ref_last_error.restype = C.c_char_p
    return _lib


def _check(rc: int):
    if rc != 0:
        raise RuntimeError("reference: " + lib().mimir_ref_last_error().decode(errors="replace"))


def set_threads(n: int) -> int:
    return lib().mimir_ref_set_threads(C.c_int(n))


def set_guard_limit(nbytes: int):
    lib().mimir_ref_set_guard_limit(C.c_ulonglong(nbytes))


class RefModel:
    """A reference ``Model`` built from descriptors or through the reference's registry."""

    def __init__(self, descs=None, registry=None, cfg_json: str = ""):
        self._h = C.c_void_p()
        if descs is not None:
            self._arr = desc_array(descs)
            _check(lib().mimir_ref_model_create(self._arr, C.c_int(len(descs)), C.byref(self._h)))
        else:
            _check(lib().mimir_ref_model_create_registry(registry.encode(), cfg_json.encode(), C.byref(self._h)))

    def close(self):
        if self._h:
            lib().mimir_ref_model_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def num_layers(self) -> int:
        return lib().mimir_ref_model_num_layers(self._h)

    def layer_desc(self, i: int) -> MimirLayerDesc:
        d = MimirLayerDesc()
        _check(lib().mimir_ref_model_layer_desc(self._h, C.c_int(i), C.byref(d)))
        return d

    def layer_descs(self):
        return [self.layer_desc(i) for i in range(self.num_layers)]

    def set_weights(self, i: int, w: np.ndarray):
        w = np.ascontiguousarray(w, dtype=np.float32)
        _check(lib().mimir_ref_model_set_weights(self._h, C.c_int(i), w.ctypes.data_as(C.c_void_p), C.c_ulonglong(w.size)))

    def get_weights(self, i: int) -> np.ndarray:
        n = int(self.layer_desc(i).params_count)
        w = np.empty(n, dtype=np.float32)
        _check(lib().mimir_ref_model_get_weights(self._h, C.c_int(i), w.ctypes.data_as(C.c_void_p), C.c_ulonglong(n)))
        return w

    def save_safetensors(self, path: str):
        """Checkpoint written by the reference's own SafeTensorsWriter."""
        _check(lib().mimir_ref_model_save_safetensors(self._h, os.fsencode(path)))

    def mag_mod(self, cap: int = 65536):
        mag = np.zeros(cap, dtype=np.float32)
        mod = np.zeros(cap, dtype=np.float32)
        n = C.c_int(0)
        _check(lib().mimir_ref_model_get_mag_mod(self._h, mag.ctypes.data_as(C.c_void_p), mod.ctypes.data_as(C.c_void_p), C.c_int(cap), C.byref(n)))
        return mag[: n.value].copy(), mod[: n.value].copy()

    def forward(self, inputs: dict, out_cap: int | None = None, return_seconds: bool = False):
        """One sample.  ``inputs`` maps tensor name -> 1-D float32 array ("x" is the main input)."""
        keep = []
        arr = (MimirNamedInput * len(inputs))()
        for i, (k, v) in enumerate(inputs.items()):
            v = np.ascontiguousarray(v, dtype=np.float32).ravel()
            keep.append(v)
            arr[i].name = k.encode()
            arr[i].data = v.ctypes.data
            arr[i].per_sample = v.size
            arr[i].broadcast = 0
        n = C.c_ulonglong(0)
        secs = C.c_double(0)
        if out_cap is None:
            # first call sizes the output
            _check(lib().mimir_ref_model_forward(self._h, arr, C.c_int(len(inputs)), None, C.c_ulonglong(0), C.byref(n), C.byref(secs)))
            out_cap = n.value
        out = np.empty(out_cap, dtype=np.float32)
        _check(lib().mimir_ref_model_forward(self._h, arr, C.c_int(len(inputs)), out.ctypes.data_as(C.c_void_p), C.c_ulonglong(out_cap), C.byref(n), C.byref(secs)))
        out = out[: n.value]
        return (out, secs.value) if return_seconds else out


def compute_attention(q, k, v, seq: int, d_model: int, heads: int) -> np.ndarray:
    """Model::computeAttention, software branch, one sample."""
    q, k, v = (np.ascontiguousarray(a, np.float32).ravel() for a in (q, k, v))
    out = np.empty(seq * d_model, np.float32)
    fp = C.POINTER(C.c_float)
    _check(lib().mimir_ref_compute_attention(q.ctypes.data_as(fp), k.ctypes.data_as(fp), v.ctypes.data_as(fp), out.ctypes.data_as(fp),
                                             C.c_int(seq), C.c_int(d_model), C.c_int(heads)))
    return out


def compute_batchnorm(x, gamma, beta, mean, var, batch: int, channels: int, spatial: int, eps: float = 1e-5) -> np.ndarray:
    """Model::computeBatchNorm, software branch, training = false."""
    d = np.array(x, np.float32).ravel().copy()
    g, b, m, v = (np.ascontiguousarray(a, np.float32).ravel() for a in (gamma, beta, mean, var))
    fp = C.POINTER(C.c_float)
    _check(lib().mimir_ref_compute_batchnorm(d.ctypes.data_as(fp), g.ctypes.data_as(fp), b.ctypes.data_as(fp), m.ctypes.data_as(fp),
                                             v.ctypes.data_as(fp), C.c_int(batch), C.c_int(channels), C.c_int(spatial), C.c_float(eps)))
    return d


def maxpool1d(x, in_channels: int, kernel_h: int, stride_h: int, pad_h: int) -> np.ndarray:
    """LayerOpsExt::maxpool1d_forward (LayerOpsExt.hpp:504-538), which the layer switch never dispatches."""
    x = np.ascontiguousarray(x, np.float32).ravel()
    out = np.empty(x.size + 16, np.float32)
    n = C.c_ulonglong(0)
    fp = C.POINTER(C.c_float)
    _check(lib().mimir_ref_maxpool1d(x.ctypes.data_as(fp), C.c_ulonglong(x.size), C.c_int(in_channels), C.c_int(kernel_h), C.c_int(stride_h),
                                     C.c_int(pad_h), out.ctypes.data_as(fp), C.c_ulonglong(out.size), C.byref(n)))
    return out[: n.value].copy()


def compute_conv2d(x, w, bias, in_h: int, in_w: int, in_c: int, out_c: int, k: int, stride: int, pad: int, dil: int = 1, transposed: bool = False) -> np.ndarray:
    """Model::computeConv2D (Conv::conv2d) or, with transposed, Model::computeConvTranspose2D (Conv::conv_transpose2d)."""
    x, w = (np.ascontiguousarray(a, np.float32).ravel() for a in (x, w))
    b = np.ascontiguousarray(bias, np.float32).ravel() if bias is not None else None
    cap = out_c * ((in_h + 2) * max(stride, 1) + k + 2 * pad) * ((in_w + 2) * max(stride, 1) + k + 2 * pad)
    out = np.empty(cap, np.float32)
    n = C.c_ulonglong(0)
    fp = C.POINTER(C.c_float)
    _check(lib().mimir_ref_compute_conv2d(C.c_int(1 if transposed else 0), x.ctypes.data_as(fp), w.ctypes.data_as(fp),
                                          b.ctypes.data_as(fp) if b is not None else None, out.ctypes.data_as(fp), C.c_ulonglong(cap), C.byref(n),
                                          C.c_int(in_h), C.c_int(in_w), C.c_int(in_c), C.c_int(out_c), C.c_int(k), C.c_int(stride), C.c_int(pad), C.c_int(dil)))
    return out[: n.value].copy()


def compute_batchnorm_training(x, gamma, beta, batch: int, channels: int, spatial: int, eps: float = 1e-5) -> np.ndarray:
    """Model::computeBatchNorm, software branch, training = true."""
    d = np.array(x, np.float32).ravel().copy()
    g, b = (np.ascontiguousarray(a, np.float32).ravel() for a in (gamma, beta))
    fp = C.POINTER(C.c_float)
    _check(lib().mimir_ref_compute_batchnorm_training(d.ctypes.data_as(fp), g.ctypes.data_as(fp), b.ctypes.data_as(fp), C.c_int(batch),
                                                      C.c_int(channels), C.c_int(spatial), C.c_float(eps)))
    return d


def compute_activation(name: str, x, param: float = 0.0) -> np.ndarray:
    """Model::computeActivation, software branch."""
    d = np.array(x, np.float32).ravel().copy()
    _check(lib().mimir_ref_compute_activation(name.encode(), d.ctypes.data_as(C.POINTER(C.c_float)), C.c_ulonglong(d.size), C.c_float(param)))
    return d
