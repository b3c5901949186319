"""Thin Python driver over the C ABI (``include/mimir_b200.h``), used by the tests and the benchmark.

Everything here calls ``libmimir_b200.so``; nothing computes in Python.  Host-pointer calls take
numpy arrays, device-pointer calls take raw addresses (e.g. ``torch.Tensor.data_ptr()``).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import abi
from .abi import MimirB200Stats, MimirLayerDesc, MimirNamedInput, desc_array


class MimirB200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        self.status = status
        name = abi.STATUS_NAMES[status] if 0 <= status < len(abi.STATUS_NAMES) else str(status)
        super().__init__(f"{name}: {message}")


_P = C.c_void_p
_SIGS = {
    "mimir_b200_init": [C.c_int, C.c_size_t],
    "mimir_b200_shutdown": [],
    "mimir_b200_abi_version": [],
    "mimir_b200_guard_set_limit": [C.c_size_t],
    "mimir_b200_guard_request": [C.c_size_t, C.c_char_p],
    "mimir_b200_guard_release": [C.c_size_t],
    "mimir_b200_guard_stats": [_P, _P, _P],
    "mimir_b200_guard_block": [C.c_int],
    "mimir_b200_guard_freeze": [C.c_int],
    "mimir_b200_guard_reset": [],
    "mimir_b200_guard_state": [_P, _P, _P, _P],
    "mimir_b200_tensor_alloc": [_P, C.c_int, C.c_char_p, _P, _P],
    "mimir_b200_buffer_alloc": [C.c_size_t, C.c_char_p, _P],
    "mimir_b200_buffer_free": [_P],
    "mimir_b200_scratchpad_get": [C.c_size_t, C.c_char_p, _P, _P],
    "mimir_b200_scratchpad_return": [_P],
    "mimir_b200_allocator_set_local_cap": [C.c_size_t],
    "mimir_b200_allocator_stats": [_P, _P, _P, _P],
    "mimir_b200_allocator_reset_stats": [],
    "mimir_b200_allocator_check_no_leaks": [_P],
    "mimir_b200_current_device": [_P],
    "mimir_b200_env_selection": [_P, _P, _P],
    "mimir_b200_init_from_env": [_P],
    "mimir_b200_shard_range": [C.c_longlong, C.c_int, C.c_int, _P, _P],
    "mimir_b200_replicas_create": [_P, C.c_int, C.c_size_t, _P, C.c_int, C.c_int, _P],
    "mimir_b200_replicas_destroy": [_P],
    "mimir_b200_replicas_count": [_P, _P],
    "mimir_b200_replicas_upload_weights": [_P, C.c_int, _P, C.c_uint64],
    "mimir_b200_replicas_set_pipeline": [_P, C.c_int],
    "mimir_b200_replicas_plan": [_P, _P, C.c_int, C.c_int, _P],
    "mimir_b200_replicas_forward": [_P, _P, C.c_int, C.c_int, _P, C.c_uint64, _P],
    "mimir_b200_replicas_inject_failure": [_P, C.c_int],
    "mimir_b200_replicas_selftest_join": [C.c_int, C.c_int],
    "mimir_b200_model_output_len": [_P, _P],
    "mimir_b200_linear_forward": [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int],
    "mimir_b200_linear_forward_ex": [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int],
    "mimir_b200_matmul": [_P, _P, _P, C.c_int, C.c_int, C.c_int],
    "mimir_b200_attention": [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int],
    "mimir_b200_conv2d": [_P, _P, _P] + [C.c_int] * 9,
    "mimir_b200_layernorm": [_P, _P, _P, _P, C.c_longlong, C.c_int, C.c_float],
    "mimir_b200_rmsnorm": [_P, _P, C.c_longlong, _P, C.c_int, C.c_longlong, C.c_float],
    "mimir_b200_groupnorm": [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int],
    "mimir_b200_softmax": [_P, _P, C.c_int, C.c_longlong, C.c_int],
    "mimir_b200_eltwise": [C.c_int, _P, _P, _P, C.c_int, C.c_longlong, C.c_longlong],
    "mimir_b200_embedding": [_P, _P, _P, _P, C.c_longlong, C.c_int, C.c_int, C.c_int],
    "mimir_b200_upsample_nearest": [_P, _P] + [C.c_int] * 6,
    "mimir_b200_permute": [_P, _P, C.c_int, C.c_int, _P, _P],
    "mimir_b200_token_mean_pool": [_P, _P, C.c_int, C.c_int, C.c_int],
    "mimir_b200_global_avgpool": [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int],
    "mimir_b200_eltwise_alpha": [C.c_int, _P, _P, _P, C.c_int, C.c_longlong, C.c_longlong, C.c_float],
    "mimir_b200_cross_attention": [_P, _P, _P, _P] + [C.c_int] * 6,
    "mimir_b200_depthwise_conv2d": [_P, _P, _P, _P] + [C.c_int] * 7,
    "mimir_b200_conv1d": [_P, _P, _P, _P] + [C.c_int] * 7,
    "mimir_b200_conv_transpose2d": [_P, _P, _P] + [C.c_int] * 9,
    "mimir_b200_pool2d": [C.c_int, _P, _P] + [C.c_int] * 10,
    "mimir_b200_pad2d": [C.c_int, _P, _P] + [C.c_int] * 6,
    "mimir_b200_pixel_shuffle": [_P, _P] + [C.c_int] * 5,
    "mimir_b200_upsample_bilinear": [_P, _P] + [C.c_int] * 7,
    "mimir_b200_batch_matmul": [_P, _P, _P, C.c_longlong, C.c_int, C.c_int, C.c_int],
    "mimir_b200_batchnorm_inference": [_P, _P, C.c_longlong, _P, C.c_int, C.c_longlong, C.c_float],
    "mimir_b200_batchnorm_running": [_P, _P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_longlong, C.c_float],
    "mimir_b200_batchnorm_batchstats": [_P, _P, _P, _P, C.c_int, C.c_int, C.c_longlong, C.c_float],
    "mimir_b200_conv2d_dilated": [_P, _P, _P, _P] + [C.c_int] * 9,
    "mimir_b200_conv_transpose2d_scatter": [_P, _P, _P, _P] + [C.c_int] * 8,
    "mimir_b200_attention_qkv": [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int],
    "mimir_b200_model_create": [_P, C.c_int, _P],
    "mimir_b200_model_destroy": [_P],
    "mimir_b200_model_set_precision": [_P, C.c_int],
    "mimir_b200_model_set_pipeline": [_P, C.c_int],
    "mimir_b200_model_upload_weights": [_P, C.c_int, _P, C.c_uint64],
    "mimir_b200_model_weights_device": [_P, C.c_int, C.c_uint64, _P],
    "mimir_b200_model_num_layers": [_P, _P],
    "mimir_b200_model_layer_info": [_P, C.c_int, _P, _P],
    "mimir_b200_model_tensor_slot": [_P, C.c_char_p, _P, _P],
    "mimir_b200_model_load_safetensors": [_P, C.c_char_p, C.c_int, _P, _P],
    "mimir_b200_model_plan": [_P, _P, C.c_int, C.c_int, _P],
    "mimir_b200_model_forward": [_P, _P, C.c_int, C.c_int, _P, C.c_uint64, _P],
    "mimir_b200_model_forward_device": [_P, _P, C.c_int, C.c_int, _P, C.c_uint64, _P, _P],
    "mimir_b200_model_decode_begin": [_P, _P, C.c_int, C.c_int, C.c_int, _P],
    "mimir_b200_model_decode_step": [_P, _P, C.c_int, C.c_int, C.c_int, _P, C.c_uint64, _P],
    "mimir_b200_model_decode_end": [_P],
    "mimir_b200_argmax_rows_device": [_P, _P, C.c_longlong, C.c_int, _P],
    "mimir_b200_get_stats": [_P],
    "mimir_b200_check_device": [_P],
    "mimir_b200_selftest_wait_timeout": [C.c_ulonglong, _P],
    "mimir_b200_profile_gemm": [C.c_int],
    "mimir_b200_profile_read": [_P, _P],
    "mimir_b200_dev_layernorm": [_P, _P, _P, _P, C.c_longlong, C.c_int, C.c_float, _P],
    "mimir_b200_dev_rmsnorm": [_P, _P, C.c_longlong, _P, C.c_int, C.c_longlong, C.c_float, _P],
    "mimir_b200_dev_rmsnorm_noalloc": [_P, _P, C.c_longlong, _P, C.c_int, C.c_longlong, C.c_float, _P],
    "mimir_b200_dev_groupnorm": [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, _P],
    "mimir_b200_dev_softmax": [_P, _P, C.c_int, C.c_longlong, C.c_int, _P],
    "mimir_b200_dev_eltwise": [C.c_int, _P, _P, _P, C.c_int, C.c_longlong, C.c_longlong, _P],
}

EXPORTED_SYMBOLS = sorted(list(_SIGS) + ["mimir_b200_last_error"])

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        l = abi.load()
        for name, args in _SIGS.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = C.c_int
        _lib = l
    return _lib


def check(status: int):
    if status != abi.OK:
        raise MimirB200Error(status, lib().mimir_b200_last_error().decode(errors="replace"))


def init(device: int = 0, hbm_budget_bytes: int = 0):
    check(lib().mimir_b200_init(device, hbm_budget_bytes))


def shutdown():
    check(lib().mimir_b200_shutdown())


def guard_stats():
    a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
    check(lib().mimir_b200_guard_stats(C.byref(a), C.byref(b), C.byref(c)))
    return dict(limit=a.value, current=b.value, peak=c.value)


# ---- RuntimeAllocator verbs (device pointers as integers) ------------------------------------------
def tensor_alloc(shape, name=None):
    arr = (C.c_int * len(shape))(*shape)
    ptr, nbytes = C.c_void_p(), C.c_size_t()
    check(lib().mimir_b200_tensor_alloc(arr, len(shape), name.encode() if name else None, C.byref(ptr), C.byref(nbytes)))
    return ptr.value, nbytes.value


def buffer_alloc(nbytes, tag=None):
    ptr = C.c_void_p()
    check(lib().mimir_b200_buffer_alloc(nbytes, tag.encode() if tag else None, C.byref(ptr)))
    return ptr.value


def buffer_free(ptr):
    check(lib().mimir_b200_buffer_free(C.c_void_p(ptr)))


def scratchpad_get(min_bytes, tag=None):
    ptr, nbytes = C.c_void_p(), C.c_size_t()
    check(lib().mimir_b200_scratchpad_get(min_bytes, tag.encode() if tag else None, C.byref(ptr), C.byref(nbytes)))
    return ptr.value, nbytes.value


def scratchpad_return(ptr):
    check(lib().mimir_b200_scratchpad_return(C.c_void_p(ptr)))


def allocator_stats():
    a, b, c, d = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
    check(lib().mimir_b200_allocator_stats(C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
    return dict(total_allocated=a.value, num_allocations=b.value, peak=c.value, current=d.value)


def allocator_check_no_leaks():
    ok = C.c_int()
    check(lib().mimir_b200_allocator_check_no_leaks(C.byref(ok)))
    return bool(ok.value)


def stats() -> dict:
    s = MimirB200Stats()
    check(lib().mimir_b200_get_stats(C.byref(s)))
    return {k: getattr(s, k) for k, _ in MimirB200Stats._fields_}


def profile_gemm(enable: bool):
    check(lib().mimir_b200_profile_gemm(int(enable)))


def profile_read():
    ms, n = C.c_float(0), C.c_int(0)
    check(lib().mimir_b200_profile_read(C.byref(ms), C.byref(n)))
    return ms.value, n.value


def _f(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data


# ---- per-op calls, host arrays -------------------------------------------------------------------
def linear_forward(x, w, bias, batch, in_f, out_f, precision=None, activation=-1):
    x, w, bias = _f(x), _f(w), _f(bias)
    y = np.empty(batch * out_f, np.float32)
    if precision is None and activation == -1:
        check(lib().mimir_b200_linear_forward(_p(x), _p(w), _p(bias), _p(y), batch, in_f, out_f))
    else:
        check(lib().mimir_b200_linear_forward_ex(_p(x), _p(w), _p(bias), _p(y), batch, in_f, out_f,
                                                 abi.PREC_BF16X2 if precision is None else precision, activation))
    return y


def matmul(a, b, M, K, N):
    a, b = _f(a), _f(b)
    y = np.empty(M * N, np.float32)
    check(lib().mimir_b200_matmul(_p(a), _p(b), _p(y), M, K, N))
    return y


def attention(x, w, batch, seq, embed, heads, causal):
    x, w = _f(x), _f(w)
    y = np.empty(batch * seq * embed, np.float32)
    check(lib().mimir_b200_attention(_p(x), _p(w), _p(y), batch, seq, embed, heads, int(causal)))
    return y


def conv2d(x, w, batch, ic, oc, h, wd, k, stride, pad, relu=False):
    x, w = _f(x), _f(w)
    oh = (h + 2 * pad - k) // stride + 1
    ow = (wd + 2 * pad - k) // stride + 1
    y = np.empty(batch * oc * max(oh, 0) * max(ow, 0), np.float32)
    check(lib().mimir_b200_conv2d(_p(x), _p(w), _p(y), batch, ic, oc, h, wd, k, stride, pad, int(relu)))
    return y


def layernorm(x, gamma, beta, rows, n, eps=1e-5):
    x, gamma, beta = _f(x), _f(gamma), _f(beta)
    y = np.empty(rows * n, np.float32)
    check(lib().mimir_b200_layernorm(_p(x), _p(gamma), _p(beta), _p(y), rows, n, eps))
    return y


def rmsnorm(x, gamma, batch, n, eps=1e-5):
    x, gamma = _f(x), _f(gamma)
    y = np.empty(batch * n, np.float32)
    check(lib().mimir_b200_rmsnorm(_p(x), _p(gamma), 0 if gamma is None else gamma.size, _p(y), batch, n, eps))
    return y


def groupnorm(x, gamma, beta, batch, ch, h, w, groups, eps=1e-5, act=-1):
    x, gamma, beta = _f(x), _f(gamma), _f(beta)
    y = np.empty(batch * ch * h * w, np.float32)
    check(lib().mimir_b200_groupnorm(_p(x), _p(gamma), _p(beta), _p(y), batch, ch, h, w, groups, eps, act))
    return y


def softmax(x, batch, n, log=False):
    x = _f(x)
    y = np.empty(batch * n, np.float32)
    check(lib().mimir_b200_softmax(_p(x), _p(y), batch, n, int(log)))
    return y


def eltwise(op, a, b=None, batch=1):
    a, b = _f(a), _f(b)
    n = a.size // batch
    nb = 0 if b is None else b.size // batch
    y = np.empty(a.size, np.float32)
    check(lib().mimir_b200_eltwise(op, _p(a), _p(b), _p(y), batch, n, nb))
    return y


def embedding(ids, table, vocab, dim, padding_idx=-1):
    table = _f(table)
    ids = np.ascontiguousarray(ids)
    y = np.empty(ids.size * dim, np.float32)
    if ids.dtype == np.int32:
        check(lib().mimir_b200_embedding(None, _p(ids), _p(table), _p(y), ids.size, vocab, dim, padding_idx))
    else:
        ids = _f(ids)
        check(lib().mimir_b200_embedding(_p(ids), None, _p(table), _p(y), ids.size, vocab, dim, padding_idx))
    return y


def upsample_nearest(x, batch, ch, in_h, in_w, sh, sw):
    x = _f(x)
    y = np.empty(x.size * sh * sw, np.float32)
    check(lib().mimir_b200_upsample_nearest(_p(x), _p(y), batch, ch, in_h, in_w, sh, sw))
    return y


def permute(x, shape, dims, batch=1):
    x = _f(x)
    y = np.empty_like(x)
    sh = (C.c_int * len(shape))(*shape)
    dm = (C.c_int * len(dims))(*dims)
    check(lib().mimir_b200_permute(_p(x), _p(y), batch, len(shape), C.addressof(sh), C.addressof(dm)))
    return y


def token_mean_pool(x, batch, seq, dim):
    x = _f(x)
    y = np.empty(batch * dim, np.float32)
    check(lib().mimir_b200_token_mean_pool(_p(x), _p(y), batch, seq, dim))
    return y


def global_avgpool(x, batch, ch, h, w):
    x = _f(x)
    y = np.empty(batch * ch, np.float32)
    check(lib().mimir_b200_global_avgpool(_p(x), _p(y), batch, ch, h, w))
    return y


def eltwise_alpha(op, a, alpha, b=None, batch=1):
    a, b = _f(a), _f(b)
    n = a.size // batch
    nb = 0 if b is None else b.size // batch
    y = np.empty(a.size, np.float32)
    check(lib().mimir_b200_eltwise_alpha(op, _p(a), _p(b), _p(y), batch, n, nb, alpha))
    return y


def cross_attention(q, kv, w, batch, q_len, kv_len, embed, heads, causal):
    q, kv, w = _f(q), _f(kv), _f(w)
    y = np.empty(batch * q_len * embed, np.float32)
    check(lib().mimir_b200_cross_attention(_p(q), _p(kv), _p(w), _p(y), batch, q_len, kv_len, embed, heads, int(causal)))
    return y


def depthwise_conv2d(x, w, bias, batch, ch, h, wd, k, stride, pad):
    x, w, bias = _f(x), _f(w), _f(bias)
    oh, ow = (h + 2 * pad - k) // stride + 1, (wd + 2 * pad - k) // stride + 1
    y = np.empty(batch * ch * oh * ow, np.float32)
    check(lib().mimir_b200_depthwise_conv2d(_p(x), _p(w), _p(bias), _p(y), batch, ch, h, wd, k, stride, pad))
    return y


def conv1d(x, w, bias, batch, ic, oc, length, k, stride, pad):
    x, w, bias = _f(x), _f(w), _f(bias)
    y = np.empty(batch * oc * ((length + 2 * pad - k) // stride + 1), np.float32)
    check(lib().mimir_b200_conv1d(_p(x), _p(w), _p(bias), _p(y), batch, ic, oc, length, k, stride, pad))
    return y


def conv_transpose2d(x, w, batch, ic, oc, h, wd, k, stride, pad, relu=False):
    x, w = _f(x), _f(w)
    oh, ow = (h - 1) * stride - 2 * pad + k, (wd - 1) * stride - 2 * pad + k
    y = np.empty(batch * oc * oh * ow, np.float32)
    check(lib().mimir_b200_conv_transpose2d(_p(x), _p(w), _p(y), batch, ic, oc, h, wd, k, stride, pad, int(relu)))
    return y


def pool2d(is_max, x, batch, ch, h, wd, kh, kw, sh, sw, ph, pw):
    x = _f(x)
    oh, ow = (h + 2 * ph - kh) // sh + 1, (wd + 2 * pw - kw) // sw + 1
    y = np.empty(batch * ch * oh * ow, np.float32)
    check(lib().mimir_b200_pool2d(int(is_max), _p(x), _p(y), batch, ch, h, wd, kh, kw, sh, sw, ph, pw))
    return y


def pad2d(mode, x, batch, ch, h, wd, ph, pw):
    x = _f(x)
    y = np.empty(batch * ch * (h + 2 * ph) * (wd + 2 * pw), np.float32)
    check(lib().mimir_b200_pad2d(mode, _p(x), _p(y), batch, ch, h, wd, ph, pw))
    return y


def pixel_shuffle(x, batch, ic, h, wd, r):
    x = _f(x)
    y = np.empty_like(x)
    check(lib().mimir_b200_pixel_shuffle(_p(x), _p(y), batch, ic, h, wd, r))
    return y


def upsample_bilinear(x, batch, ch, h, wd, oh, ow, half_pixel=False):
    x = _f(x)
    y = np.empty(batch * ch * oh * ow, np.float32)
    check(lib().mimir_b200_upsample_bilinear(_p(x), _p(y), batch, ch, h, wd, oh, ow, int(half_pixel)))
    return y


def batch_matmul(a, b, nb, M, K, N):
    a, b = _f(a), _f(b)
    y = np.empty(nb * M * N, np.float32)
    check(lib().mimir_b200_batch_matmul(_p(a), _p(b), _p(y), nb, M, K, N))
    return y


def batchnorm_inference(x, w, batch, n, eps=1e-5):
    x, w = _f(x), _f(w)
    y = np.empty(batch * n, np.float32)
    check(lib().mimir_b200_batchnorm_inference(_p(x), _p(w), 0 if w is None else w.size, _p(y), batch, n, eps))
    return y


def batchnorm_running(x, gamma, beta, mean, var, batch, channels, spatial, eps=1e-5):
    x, gamma, beta, mean, var = (_f(a) for a in (x, gamma, beta, mean, var))
    y = np.empty(batch * channels * spatial, np.float32)
    check(lib().mimir_b200_batchnorm_running(_p(x), _p(gamma), _p(beta), _p(mean), _p(var), _p(y), batch, channels, spatial, eps))
    return y


def batchnorm_batchstats(x, gamma, beta, batch, channels, spatial, eps=1e-5):
    """Model::computeBatchNorm with training = true: statistics of each channel over the batch and the spatial positions."""
    x, gamma, beta = (_f(a) for a in (x, gamma, beta))
    y = np.empty(batch * channels * spatial, np.float32)
    check(lib().mimir_b200_batchnorm_batchstats(_p(x), _p(gamma), _p(beta), _p(y), batch, channels, spatial, eps))
    return y


def conv2d_dilated(x, w, bias, batch, in_c, out_c, in_h, in_w, k, stride, pad, dil=1):
    """Model::computeConv2D (Conv::conv2d, scalar branch): bias and dilation."""
    x, w, bias = _f(x), _f(w), _f(bias)
    oh = (in_h + 2 * pad - dil * (k - 1) - 1) // stride + 1
    ow = (in_w + 2 * pad - dil * (k - 1) - 1) // stride + 1
    y = np.empty(batch * out_c * oh * ow, np.float32)
    check(lib().mimir_b200_conv2d_dilated(_p(x), _p(w), _p(bias), _p(y), batch, in_c, out_c, in_h, in_w, k, stride, pad, dil))
    return y


def conv_transpose2d_scatter(x, w, bias, batch, in_c, out_c, in_h, in_w, k, stride, pad):
    """Model::computeConvTranspose2D (Conv::conv_transpose2d): the scatter form on top of the bias."""
    x, w, bias = _f(x), _f(w), _f(bias)
    oh, ow = (in_h - 1) * stride - 2 * pad + k, (in_w - 1) * stride - 2 * pad + k
    y = np.empty(batch * out_c * oh * ow, np.float32)
    check(lib().mimir_b200_conv_transpose2d_scatter(_p(x), _p(w), _p(bias), _p(y), batch, in_c, out_c, in_h, in_w, k, stride, pad))
    return y


def attention_qkv(q, k, v, batch, seq, d_model, heads):
    q, k, v = _f(q), _f(k), _f(v)
    y = np.empty(batch * seq * d_model, np.float32)
    check(lib().mimir_b200_attention_qkv(_p(q), _p(k), _p(v), _p(y), batch, seq, d_model, heads))
    return y


# ---- whole graph -----------------------------------------------------------------------------------
class GraphModel:
    """A layer graph on the device: ``mimir_b200_model_*``."""

    def __init__(self, descs, precision: int = abi.PREC_BF16X2, pipeline: int = 1):
        self._descs = list(descs)
        self._arr = desc_array(self._descs)
        self._h = C.c_void_p()
        check(lib().mimir_b200_model_create(C.addressof(self._arr), len(self._descs), C.byref(self._h)))
        check(lib().mimir_b200_model_set_precision(self._h, precision))
        if pipeline != 1:
            check(lib().mimir_b200_model_set_pipeline(self._h, pipeline))
        self.batch = 0
        self.arena_bytes = 0

    def close(self):
        if self._h:
            lib().mimir_b200_model_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def upload_weights(self, i: int, w):
        if w is None:
            return
        w = _f(w)
        check(lib().mimir_b200_model_upload_weights(self._h, i, _p(w), w.size))

    def load_safetensors(self, path: str, strict: bool = True):
        """Streams "<layer>/weights" tensors of a safetensors checkpoint into the device blocks."""
        n, b = C.c_int(0), C.c_ulonglong(0)
        check(lib().mimir_b200_model_load_safetensors(self._h, os.fsencode(path), int(strict), C.byref(n), C.byref(b)))
        return n.value, b.value

    @staticmethod
    def _inputs(spec):
        """spec: name -> (address_or_array, per_sample, broadcast)"""
        arr = (MimirNamedInput * len(spec))()
        keep = []
        for i, (name, (data, per, bc)) in enumerate(spec.items()):
            arr[i].name = name.encode()
            if isinstance(data, np.ndarray):
                data = _f(data)
                keep.append(data)
                arr[i].data = data.ctypes.data
            else:
                arr[i].data = data
            arr[i].per_sample = per
            arr[i].broadcast = int(bc)
        arr._keep = keep
        return arr

    def plan(self, spec: dict, batch: int) -> int:
        arr = self._inputs({k: (0, per, bc) for k, (per, bc) in spec.items()})
        peak = C.c_uint64(0)
        check(lib().mimir_b200_model_plan(self._h, C.addressof(arr), len(spec), batch, C.byref(peak)))
        self.batch = batch
        self.arena_bytes = peak.value
        return peak.value

    def tensor_slot(self, input_name=None):
        """(byte offset, byte size) of a graph input's slot, or of the output's (None), in one arena buffer."""
        off, nb = C.c_uint64(0), C.c_uint64(0)
        check(lib().mimir_b200_model_tensor_slot(self._h, None if input_name is None else input_name.encode(), C.byref(off), C.byref(nb)))
        return off.value, nb.value

    def forward(self, inputs: dict, batch: int, out_per_sample: int) -> np.ndarray:
        """inputs: name -> (numpy array, broadcast flag).  Host in, host out."""
        spec = {}
        for k, (a, bc) in inputs.items():
            a = _f(a)
            spec[k] = (a, a.size if bc else a.size // batch, bc)
        arr = self._inputs(spec)
        out = np.empty(batch * out_per_sample, np.float32)
        n = C.c_uint64(0)
        check(lib().mimir_b200_model_forward(self._h, C.addressof(arr), len(spec), batch, _p(out), out.size, C.byref(n)))
        return out.reshape(batch, n.value) if n.value * batch == out.size else out

    def decode_begin(self, spec: dict, batch: int, max_seq: int) -> int:
        """spec: name -> (per-TOKEN size, broadcast).  Returns the bytes of the key / value caches."""
        arr = self._inputs({k: (0, per, bc) for k, (per, bc) in spec.items()})
        nbytes = C.c_uint64(0)
        check(lib().mimir_b200_model_decode_begin(self._h, C.addressof(arr), len(spec), batch, max_seq, C.byref(nbytes)))
        return nbytes.value

    def decode_step(self, inputs: dict, batch: int, pos: int, out_per_sample: int) -> np.ndarray:
        """inputs: name -> (numpy array holding ONE token per sample, broadcast flag)."""
        spec = {}
        for k, (a, bc) in inputs.items():
            a = _f(a)
            spec[k] = (a, a.size if bc else a.size // batch, bc)
        arr = self._inputs(spec)
        out = np.empty(batch * out_per_sample, np.float32)
        n = C.c_uint64(0)
        check(lib().mimir_b200_model_decode_step(self._h, C.addressof(arr), len(spec), batch, pos, _p(out), out.size, C.byref(n)))
        return out.reshape(batch, n.value) if n.value * batch == out.size else out

    def decode_end(self):
        check(lib().mimir_b200_model_decode_end(self._h))

    def forward_host_ptrs(self, spec: dict, batch: int, out_ptr: int, out_capacity: int) -> int:
        """spec: name -> (host address, per_sample, broadcast).  For pinned buffers."""
        arr = self._inputs(spec)
        n = C.c_uint64(0)
        check(lib().mimir_b200_model_forward(self._h, C.addressof(arr), len(spec), batch, out_ptr, out_capacity, C.byref(n)))
        return n.value

    def forward_device(self, spec: dict, batch: int, out_ptr: int, out_capacity: int, stream: int = 0) -> int:
        """spec: name -> (device address, per_sample, broadcast).  Asynchronous on ``stream``."""
        arr = self._inputs(spec)
        n = C.c_uint64(0)
        check(lib().mimir_b200_model_forward_device(self._h, C.addressof(arr), len(spec), batch, out_ptr, out_capacity,
                                                    C.byref(n), stream))
        return n.value


class Replicas:
    """One replica of a layer graph per listed device, one host thread per device: ``mimir_b200_replicas_*``."""

    def __init__(self, devices, descs, precision: int = abi.PREC_BF16X2, hbm_budget_bytes: int = 0, pipeline: int = 1):
        self._descs = list(descs)
        self._arr = desc_array(self._descs)
        self._h = C.c_void_p()
        devs = (C.c_int * len(devices))(*devices)
        check(lib().mimir_b200_replicas_create(devs, len(devices), hbm_budget_bytes, C.addressof(self._arr), len(self._descs), precision,
                                               C.byref(self._h)))
        if pipeline != 1:
            check(lib().mimir_b200_replicas_set_pipeline(self._h, pipeline))

    def close(self):
        if self._h:
            lib().mimir_b200_replicas_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def upload_weights(self, i: int, w):
        if w is None:
            return
        w = _f(w)
        check(lib().mimir_b200_replicas_upload_weights(self._h, i, _p(w), w.size))

    def plan(self, spec: dict, batch_total: int) -> int:
        arr = GraphModel._inputs({k: (0, per, bc) for k, (per, bc) in spec.items()})
        peak = C.c_uint64(0)
        check(lib().mimir_b200_replicas_plan(self._h, C.addressof(arr), len(spec), batch_total, C.byref(peak)))
        return peak.value

    def inject_failure(self, rank: int):
        check(lib().mimir_b200_replicas_inject_failure(self._h, rank))

    def forward_host_ptrs(self, spec: dict, batch_total: int, out_ptr: int, out_capacity: int) -> int:
        """spec: name -> (host address or array, per_sample, broadcast); the output lands in one host buffer."""
        arr = GraphModel._inputs(spec)
        n = C.c_uint64(0)
        check(lib().mimir_b200_replicas_forward(self._h, C.addressof(arr), len(spec), batch_total, out_ptr, out_capacity, C.byref(n)))
        return n.value
