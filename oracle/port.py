"""TEST INFRASTRUCTURE — ctypes binding of the plain-C restatement (``libmimir_oracle.so``) and a
restatement of the reference's graph walk.

``run_graph`` follows ``Model::forwardPassView`` (Model.cpp:4621-6824): a tensor store keyed by
name, initialised with the main input under ``"x"`` and ``"__input__"`` (:4640-4642) plus the extra
named inputs (:4663-4667); each layer reads ``inputs`` (empty => ``{"x"}``, :4802), runs its op,
and stores under ``output`` (empty => ``"x"``, :6655); the result is ``store["x"]`` (:6823).
One sample per call, like the reference.  Never imported by the product.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmimir_oracle.so")
_lib = None

ELT = {"Add": 0, "Multiply": 1, "GELU": 2, "SiLU": 3, "ReLU": 4, "Tanh": 5, "Sigmoid": 6, "Softplus": 8, "Mish": 9,
       "HardSigmoid": 10, "HardSwish": 11, "Subtract": 12, "Divide": 13}


def build():
    subprocess.run(["make", "-C", _HERE, "port"], check=True, capture_output=True)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = C.CDLL(LIB_PATH)
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def linear(x, w, bias, rows, in_f, out_f):
    x, w = _f(x), _f(w)
    bias = _f(bias) if bias is not None else None
    y = np.empty(rows * out_f, np.float32)
    lib().mo_linear(_p(x), _p(w), _p(bias), _p(y), C.c_long(rows), C.c_int(in_f), C.c_int(out_f))
    return y


def matmul(a, b, M, K, N):
    a, b = _f(a), _f(b)
    y = np.empty(M * N, np.float32)
    lib().mo_matmul(_p(a), _p(b), _p(y), C.c_long(M), C.c_long(K), C.c_long(N))
    return y


def attention(x, wblock, seq, E, heads, causal):
    x, wblock = _f(x), _f(wblock)
    wqkv, wout = wblock[: 3 * E * E], np.ascontiguousarray(wblock[3 * E * E : 4 * E * E])
    y = np.empty(seq * E, np.float32)
    lib().mo_attention(_p(x), _p(wqkv), _p(wout), _p(y), C.c_int(seq), C.c_int(E), C.c_int(heads), C.c_int(int(causal)))
    return y


def conv2d(x, w, ic, oc, h, wd, k, stride, pad, relu):
    x, w = _f(x), _f(w)
    oh = (h + 2 * pad - k) // stride + 1
    ow = (wd + 2 * pad - k) // stride + 1
    y = np.empty(oc * oh * ow, np.float32)
    lib().mo_conv2d(_p(x), _p(w), _p(y), *(C.c_int(v) for v in (ic, oc, h, wd, k, stride, pad, int(relu))))
    return y


def layernorm(x, gamma, beta, rows, n, eps):
    x = _f(x)
    gamma = _f(gamma) if gamma is not None else None
    beta = _f(beta) if beta is not None else None
    y = np.empty_like(x)
    lib().mo_layernorm(_p(x), _p(gamma), _p(beta), _p(y), C.c_long(rows), C.c_int(n), C.c_float(eps))
    return y


def rmsnorm(x, gamma, eps):
    x = _f(x)
    gamma = _f(gamma) if gamma is not None and len(gamma) else None
    y = np.empty_like(x)
    lib().mo_rmsnorm(_p(x), _p(gamma), C.c_long(0 if gamma is None else gamma.size), _p(y), C.c_long(x.size), C.c_float(eps))
    return y


def groupnorm(x, gamma, beta, ch, h, w, groups, eps):
    x = _f(x)
    gamma = _f(gamma) if gamma is not None else None
    beta = _f(beta) if beta is not None else None
    y = np.empty_like(x)
    lib().mo_groupnorm(_p(x), _p(gamma), _p(beta), _p(y), C.c_int(ch), C.c_int(h), C.c_int(w), C.c_int(groups), C.c_float(eps))
    return y


def softmax(x, log=False):
    x = _f(x)
    y = np.empty_like(x)
    lib().mo_softmax(_p(x), _p(y), C.c_long(x.size), C.c_int(int(log)))
    return y


def eltwise(op, a, b=None):
    a = _f(a)
    b = _f(b) if b is not None else None
    if b is not None and b.size > a.size:
        a, b = b, a  # add_forward swaps so that `big` is first (LayerOps.hpp:171-176)
    y = np.empty_like(a)
    rc = lib().mo_eltwise(C.c_int(op), _p(a), _p(b), _p(y), C.c_long(a.size), C.c_long(0 if b is None else b.size))
    if rc:
        raise RuntimeError("eltwise: sizes not broadcastable")
    return y


def embedding(ids, table, vocab, dim, padding_idx):
    ids, table = _f(ids), _f(table)
    y = np.empty(ids.size * dim, np.float32)
    lib().mo_embedding(_p(ids), _p(table), _p(y), C.c_long(ids.size), C.c_int(vocab), C.c_int(dim), C.c_int(padding_idx))
    return y


def upsample_nearest(x, ch, in_h, in_w, sh, sw):
    x = _f(x)
    y = np.empty(ch * in_h * sh * in_w * sw, np.float32)
    lib().mo_upsample_nearest(_p(x), _p(y), *(C.c_int(v) for v in (ch, in_h, in_w, sh, sw)))
    return y


def permute(x, shape, dims):
    x = _f(x)
    y = np.empty_like(x)
    sh = (C.c_int * len(shape))(*shape)
    dm = (C.c_int * len(dims))(*dims)
    lib().mo_permute(_p(x), _p(y), C.c_int(len(shape)), sh, dm)
    return y


def token_mean_pool(x, seq, dim):
    x = _f(x)
    y = np.empty(dim, np.float32)
    lib().mo_token_mean_pool(_p(x), _p(y), C.c_int(seq), C.c_int(dim))
    return y


def global_avgpool(x, ch, h, w):
    x = _f(x)
    y = np.empty(ch, np.float32)
    lib().mo_global_avgpool(_p(x), _p(y), C.c_int(ch), C.c_int(h), C.c_int(w))
    return y


def _ci(*v):
    return [C.c_int(int(i)) for i in v]


def leaky_relu(x, alpha):
    x = _f(x)
    y = np.empty_like(x)
    lib().mo_leaky_relu(_p(x), _p(y), C.c_long(x.size), C.c_float(alpha))
    return y


def cross_attention(q_in, kv_in, w, q_len, kv_len, E, heads, causal):
    q_in, kv_in, w = _f(q_in), _f(kv_in), _f(w)
    wq, wkv, wout = w[: E * E], w[E * E : 3 * E * E], w[3 * E * E : 4 * E * E]
    y = np.empty(q_len * E, np.float32)
    lib().mo_cross_attention(_p(q_in), _p(kv_in), _p(_f(wq)), _p(_f(wkv)), _p(_f(wout)), _p(y), *_ci(q_len, kv_len, E, heads, causal))
    return y


def depthwise_conv2d(x, w, bias, ch, h, wd, k, stride, pad):
    x, w = _f(x), _f(w)
    bias = _f(bias) if bias is not None else None
    oh, ow = (h + 2 * pad - k) // stride + 1, (wd + 2 * pad - k) // stride + 1
    y = np.empty(ch * oh * ow, np.float32)
    lib().mo_depthwise_conv2d(_p(x), _p(w), _p(bias), _p(y), *_ci(ch, h, wd, k, stride, pad))
    return y


def conv1d(x, w, bias, ic, oc, length, k, stride, pad):
    x, w = _f(x), _f(w)
    bias = _f(bias) if bias is not None else None
    y = np.empty(oc * ((length + 2 * pad - k) // stride + 1), np.float32)
    lib().mo_conv1d(_p(x), _p(w), _p(bias), _p(y), *_ci(ic, oc, length, k, stride, pad))
    return y


def conv_transpose2d(x, w, ic, oc, h, wd, k, stride, pad, relu):
    x, w = _f(x), _f(w)
    oh, ow = (h - 1) * stride - 2 * pad + k, (wd - 1) * stride - 2 * pad + k
    y = np.empty(oc * oh * ow, np.float32)
    lib().mo_conv_transpose2d(_p(x), _p(w), _p(y), *_ci(ic, oc, h, wd, k, stride, pad, relu))
    return y


def pool2d(is_max, x, ch, h, wd, kh, kw, sh, sw, ph, pw):
    x = _f(x)
    oh, ow = (h + 2 * ph - kh) // sh + 1, (wd + 2 * pw - kw) // sw + 1
    y = np.empty(ch * oh * ow, np.float32)
    lib().mo_pool2d(C.c_int(int(is_max)), _p(x), _p(y), *_ci(ch, h, wd, kh, kw, sh, sw, ph, pw))
    return y


def pad2d(mode, x, ch, h, wd, ph, pw):
    x = _f(x)
    y = np.empty(ch * (h + 2 * ph) * (wd + 2 * pw), np.float32)
    lib().mo_pad2d(C.c_int(mode), _p(x), _p(y), *_ci(ch, h, wd, ph, pw))
    return y


def pixel_shuffle(x, ic, h, wd, r):
    x = _f(x)
    y = np.empty_like(x)
    lib().mo_pixel_shuffle(_p(x), _p(y), *_ci(ic, h, wd, r))
    return y


def upsample_bilinear(x, ch, h, wd, oh, ow, half_pixel):
    x = _f(x)
    y = np.empty(ch * oh * ow, np.float32)
    lib().mo_upsample_bilinear(_p(x), _p(y), *_ci(ch, h, wd, oh, ow, half_pixel))
    return y


def batch_matmul(a, b, nb, M, K, N):
    a, b = _f(a), _f(b)
    y = np.empty(nb * M * N, np.float32)
    lib().mo_batch_matmul(_p(a), _p(b), _p(y), C.c_long(nb), *_ci(M, K, N))
    return y


def batchnorm_inference(x, w, eps):
    x = _f(x)
    w = _f(w) if w is not None else None
    y = np.empty_like(x)
    lib().mo_batchnorm_inference(_p(x), _p(w), C.c_long(0 if w is None else w.size), _p(y), C.c_long(x.size), C.c_float(eps))
    return y


def batchnorm_running(x, gamma, beta, mean, var, batch, channels, spatial, eps=1e-5):
    x, gamma, beta, mean, var = (_f(a) for a in (x, gamma, beta, mean, var))
    y = np.empty_like(x)
    lib().mo_batchnorm_running(_p(x), _p(gamma), _p(beta), _p(mean), _p(var), _p(y), *_ci(batch, channels), C.c_long(spatial), C.c_float(eps))
    return y


def attention_qkv(q, k, v, seq, d_model, heads):
    q, k, v = _f(q), _f(k), _f(v)
    y = np.empty_like(q)
    lib().mo_attention_qkv(_p(q), _p(k), _p(v), _p(y), *_ci(seq, d_model, heads))
    return y


def instance_norm2d(x, w, ch, h, wd, eps):
    x = _f(x)
    w = _f(w) if w is not None else None
    y = np.empty_like(x)
    lib().mo_instance_norm2d(_p(x), _p(w), _p(y), *_ci(ch, h, wd), C.c_float(eps))
    return y


def embedding_bag(ids, offsets, table, vocab, dim, padding_idx):
    ids, table = _f(ids), _f(table)
    off = _f(offsets) if offsets is not None else None
    n_off = off.size if off is not None else 0
    bags = max(1, n_off - 1) if n_off else 1
    y = np.empty(bags * dim, np.float32)
    fn = lib().mo_embedding_bag
    fn.restype = C.c_long
    got = fn(_p(ids), C.c_long(ids.size), _p(off) if n_off else None, C.c_long(n_off), _p(table), _p(y), C.c_int(vocab), C.c_int(dim),
             C.c_int(padding_idx))
    if got < 0:
        raise RuntimeError("EmbeddingBag: offsets must have at least 2 entries")
    return y


def patch_embed(x, w, d_model, seq_text, num_patches, patch_dim):
    x, w = _f(x), _f(w)
    y = np.empty((seq_text + 1 + num_patches) * d_model, np.float32)
    lib().mo_patch_embed(_p(x), _p(w), _p(y), C.c_int(d_model), C.c_int(seq_text), C.c_int(num_patches), C.c_int(patch_dim))
    return y


def bilinear(x1, x2, w, bias, in1, in2, out_f):
    x1, x2, w = _f(x1), _f(x2), _f(w)
    rows = x1.size // in1
    y = np.empty(rows * out_f, np.float32)
    lib().mo_bilinear(_p(x1), _p(x2), _p(w), _p(_f(bias)) if bias is not None else None, _p(y), C.c_long(rows), C.c_int(in1), C.c_int(in2),
                      C.c_int(out_f))
    return y


def maxpool1d(x, ch, k, stride, pad):
    x = _f(x)
    length = x.size // ch
    ol = (length + 2 * pad - k) // stride + 1
    y = np.empty(ch * max(ol, 0), np.float32)
    lib().mo_maxpool1d(_p(x), _p(y), C.c_int(ch), C.c_long(length), C.c_int(k), C.c_int(stride), C.c_int(pad))
    return y


def recurrent(kind, x, w, T, I, H, use_bias):  # noqa: E741
    x, w = _f(x), _f(w)
    y = np.empty(T * H, np.float32)
    lib().mo_recurrent(C.c_int(kind), _p(x), _p(w), _p(y), C.c_int(T), C.c_int(I), C.c_int(H), C.c_int(1 if use_bias else 0))
    return y


def conv2d_dilated(x, w, bias, ic, oc, h, wd, k, stride, pad, dil, avx2_lanes=False):
    """Conv::conv2d: the scalar branch, or (avx2_lanes) what an AVX2 build of the reference computes: remainder taps count eight times."""
    x, w = _f(x), _f(w)
    oh = (h + 2 * pad - dil * (k - 1) - 1) // stride + 1
    ow = (wd + 2 * pad - dil * (k - 1) - 1) // stride + 1
    y = np.empty(oc * oh * ow, np.float32)
    lib().mo_conv2d_dilated(_p(x), _p(w), _p(_f(bias)) if bias is not None else None, _p(y), *_ci(ic, oc, h, wd, k, stride, pad, dil, 1 if avx2_lanes else 0))
    return y


def conv_transpose2d_scatter(x, w, bias, ic, oc, h, wd, k, stride, pad):
    x, w = _f(x), _f(w)
    oh, ow = (h - 1) * stride - 2 * pad + k, (wd - 1) * stride - 2 * pad + k
    y = np.empty(oc * oh * ow, np.float32)
    lib().mo_conv_transpose2d_scatter(_p(x), _p(w), _p(_f(bias)) if bias is not None else None, _p(y), *_ci(ic, oc, h, wd, k, stride, pad))
    return y


def batchnorm_batchstats(x, gamma, beta, batch, channels, spatial, eps=1e-5):
    x, g, b = _f(x), _f(gamma), _f(beta)
    y = np.empty_like(x)
    lib().mo_batchnorm_batchstats(_p(x), _p(g), _p(b), _p(y), C.c_int(batch), C.c_int(channels), C.c_long(spatial), C.c_float(eps))
    return y


def elu(x, alpha):
    x = _f(x)
    y = np.empty_like(x)
    lib().mo_elu(_p(x), _p(y), C.c_long(x.size), C.c_float(alpha))
    return y


def split_pieces(d, n):
    """Sizes of the tensors a Split / Chunk layer stores (Model.cpp:5802-5832)."""
    if d.type.decode() == "Split":
        sizes = [int(d.split_sizes[i]) for i in range(d.n_splits)]
        if not sizes:
            raise RuntimeError("Split: split_sizes must be configured")
        if sum(sizes) != n:
            raise RuntimeError("Split: sum of split_sizes != input size")
        return sizes
    base, rem = divmod(n, d.num_chunks)
    return [base + (1 if i < rem else 0) for i in range(d.num_chunks)]


def _dflt(v, default):
    return v if v > 0 else default


class OperandRounding:
    """What a single 16-bit operand plane does to the contractions of the CUDA backend's one-MMA precision mode: the
    activation operand of every Linear, Conv2d and attention projection is rounded to nearest-even in the plane format
    ("f16": 11 significant bits, "bf16": 8), the weights to the same format after a per-layer power-of-two scale that
    brings the largest magnitude of the block into [2^13, 2^14).  Everything else (the attention core, norms,
    accumulation) stays the reference's fp32 arithmetic.  Used only to check that mode of the backend; the reference
    itself has no reduced-precision path."""

    def __init__(self, fmt="f16"):
        if fmt not in ("f16", "bf16"):
            raise ValueError(fmt)
        self.fmt = fmt

    def act(self, x):
        x = _f(x)
        if self.fmt == "f16":
            with np.errstate(over="ignore"):
                return x.astype(np.float16).astype(np.float32)
        u = x.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000  # round to nearest even on the upper 16 bits
        return u.astype(np.uint32).view(np.float32)

    def weight(self, w):
        w = _f(w)
        amax = float(np.max(np.abs(w))) if w.size else 0.0
        if self.fmt != "f16" or not amax > 0.0:
            return self.act(w)
        e = int(np.frexp(np.float32(amax))[1])  # amax = f * 2^e, f in [0.5, 1)
        s = float(np.ldexp(1.0, min(60, max(-60, 14 - e))))
        return (self.act(w * np.float32(s)) / np.float32(s)).astype(np.float32)


def attention_core(qkv, seq, E, heads, causal):
    qkv = _f(qkv)
    att = np.empty(seq * E, np.float32)
    lib().mo_attention_core(_p(qkv), _p(att), C.c_int(seq), C.c_int(E), C.c_int(heads), C.c_int(int(causal)))
    return att


def run_layer(d, ins, w, rounding=None):
    """One layer of the switch in Model::forwardPassView (Model.cpp:4891-6291) on one sample.  `rounding`
    (an OperandRounding) restates the backend's one-MMA mode instead of the reference's fp32 contractions."""
    t = d.type.decode()
    x = ins[0]
    if rounding is not None:
        if t == "Linear":
            in_f = d.in_features if d.in_features > 0 else x.size
            nw = in_f * d.out_features
            w = np.concatenate([rounding.weight(w[:nw]), w[nw:]])
            ins = [rounding.act(x)] + list(ins[1:])
            x = ins[0]
        elif t in ("SelfAttention", "MultiHeadAttention"):
            seq = d.seq_len if d.seq_len > 0 else 1
            E = d.embed_dim if d.embed_dim > 0 else x.size
            heads = d.num_heads if d.num_heads > 0 else 1
            wr = rounding.weight(w[: 4 * E * E])  # one scale for the whole block, as the backend takes it
            qkv = matmul(rounding.act(x), wr[: 3 * E * E], seq, E, 3 * E)
            att = attention_core(qkv, seq, E, heads, d.causal)
            return matmul(rounding.act(att), np.ascontiguousarray(wr[3 * E * E :]), seq, E, E)
        elif t == "Conv2d":
            nw = d.out_channels * d.in_channels * d.kernel * d.kernel
            w = rounding.weight(w[:nw])
            ins = [rounding.act(x)] + list(ins[1:])
            x = ins[0]
        elif t in ("CrossAttention",):
            raise NotImplementedError("operand rounding is not restated for " + t)
    if t == "Linear":
        in_f = d.in_features if d.in_features > 0 else x.size
        rows = d.seq_len if (d.seq_len > 0 and x.size == d.seq_len * in_f) else 1
        if rows == 1 and x.size != in_f:
            raise RuntimeError("Linear: input size mismatch")
        bias = w[in_f * d.out_features : in_f * d.out_features + d.out_features] if d.use_bias else None
        return linear(x, w[: in_f * d.out_features], bias, rows, in_f, d.out_features)
    if t in ("SelfAttention", "MultiHeadAttention"):
        seq = d.seq_len if d.seq_len > 0 else 1
        E = d.embed_dim if d.embed_dim > 0 else x.size
        heads = d.num_heads if d.num_heads > 0 else 1
        return attention(x, w, seq, E, heads, d.causal)
    if t == "Conv2d":
        ic = d.in_channels
        h = d.input_height if d.input_height > 0 else 64
        wd = d.input_width if d.input_width > 0 else 64
        if h * wd * ic != x.size:  # Model.cpp:4916-4944
            hw = x.size // ic
            if d.input_height > 0 and hw % d.input_height == 0:
                h, wd = d.input_height, hw // d.input_height
            elif d.input_width > 0 and hw % d.input_width == 0:
                wd, h = d.input_width, hw // d.input_width
            else:
                s = int(round(hw ** 0.5))
                if s * s == hw:
                    h = wd = s
        return conv2d(x, w, ic, d.out_channels, h, wd, d.kernel, d.stride, d.padding, d.activation != 0)
    if t == "LayerNorm":
        n = d.in_features if d.in_features > 0 else x.size
        gamma = w[:n] if d.affine else None
        beta = w[n : 2 * n] if (d.affine and d.use_bias) else None
        return layernorm(x, gamma, beta, x.size // n, n, d.eps)
    if t == "RMSNorm":
        return rmsnorm(x, w if (d.affine and w is not None) else None, d.eps)
    if t == "GroupNorm":
        ch = d.in_channels if d.in_channels > 0 else 64
        h = d.input_height if d.input_height > 0 else 32
        wd = d.input_width if d.input_width > 0 else 32
        gamma = w[:ch] if d.affine else None
        beta = w[ch : 2 * ch] if (d.affine and d.use_bias) else None
        return groupnorm(x, gamma, beta, ch, h, wd, d.num_groups, d.eps)
    if t in ("Softmax", "LogSoftmax"):
        return softmax(x, t == "LogSoftmax")
    if t in ("GELU", "SiLU", "ReLU", "Tanh", "Sigmoid", "Softplus", "Mish", "HardSigmoid", "HardSwish"):
        return eltwise(ELT[t], x)
    if t == "LeakyReLU":
        return leaky_relu(x, d.leaky_relu_alpha if d.leaky_relu_alpha > 0 else 0.01)
    if t in ("Add", "Multiply", "Subtract", "Divide"):
        if len(ins) < 2:
            raise RuntimeError(f"{t} layer requires 2 inputs")
        return eltwise(ELT[t], ins[0], ins[1])
    if t == "Embedding":
        return embedding(x, w, max(1, d.vocab_size), max(1, d.embed_dim), d.padding_idx)
    if t == "UpsampleNearest":
        sh = d.scale_h if d.scale_h > 0 else 2
        sw = d.scale_w if d.scale_w > 0 else 2
        return upsample_nearest(x, d.in_channels, d.out_h, d.out_w, sh, sw)
    if t == "Permute":
        return permute(x, list(d.shape[: d.n_dims]), list(d.permute_dims[: d.n_dims]))
    if t in ("Concat", "Stack"):
        return np.concatenate([_f(i) for i in ins])
    if t in ("Identity", "Reshape", "Flatten", "View", "Dropout", "Dropout2d", "AlphaDropout", "Squeeze", "Unsqueeze", "Reparameterize"):
        return _f(x).copy()  # Reparameterize at inference returns mu, its first input (Model.cpp:5767-5770)
    if t == "CrossAttention":
        heads = _dflt(d.num_heads, 1)
        E = d.embed_dim if d.embed_dim > 0 else d.head_dim * heads
        return cross_attention(ins[0], ins[1], w, ins[0].size // E, ins[1].size // E, E, heads, d.causal)
    if t == "DepthwiseConv2d":
        ch, h, wd = _dflt(d.in_channels, 3), _dflt(d.input_height, 32), _dflt(d.input_width, 32)
        k, st = _dflt(d.raw_kernel_h, 3), _dflt(d.raw_stride_h, 1)
        pad = d.raw_pad_h if d.raw_pad_h >= 0 else 0
        return depthwise_conv2d(x, w[: ch * k * k], w[ch * k * k : ch * k * k + ch] if d.use_bias else None, ch, h, wd, k, st, pad)
    if t == "Conv1d":
        ic, oc = _dflt(d.in_channels, 1), _dflt(d.out_channels, 1)
        k, st = _dflt(d.raw_kernel_h, 3), _dflt(d.raw_stride_h, 1)
        pad = d.raw_pad_h if d.raw_pad_h >= 0 else 0
        nw = oc * ic * k
        return conv1d(x, w[:nw], w[nw : nw + oc] if d.use_bias else None, ic, oc, x.size // ic, k, st, pad)
    if t == "ConvTranspose2d":
        return conv_transpose2d(x, w, d.in_channels, d.out_channels, _dflt(d.input_height, 64), _dflt(d.input_width, 64), d.kernel,
                                d.stride, d.padding, d.activation != 0)
    if t == "MaxPool2d":
        return pool2d(1, x, _dflt(d.in_channels, 64), _dflt(d.input_height, 64), _dflt(d.input_width, 64), d.kernel, d.kernel,
                      d.stride, d.stride, d.padding, d.padding)
    if t == "AvgPool2d":
        return pool2d(0, x, _dflt(d.in_channels, 64), _dflt(d.input_height, 32), _dflt(d.input_width, 32), d.kernel,
                      _dflt(d.kernel_w, d.kernel), d.stride, _dflt(d.stride_w, d.stride), d.padding, d.padding_w)
    if t == "AvgPool1d":  # LayerOpsExt.hpp:540-575: per channel over the length, mean of the in-bounds taps
        ch = _dflt(d.in_channels, 1)
        k = _dflt(d.raw_kernel_h, 2)
        st = d.raw_stride_h if d.raw_stride_h > 0 else k
        pad = d.raw_pad_h if d.raw_pad_h >= 0 else 0
        return pool2d(0, x, ch, 1, x.size // ch, 1, k, 1, st, 0, pad)
    if t in ("ZeroPad2d", "ReflectionPad2d", "ReplicationPad2d"):
        mode = ("ZeroPad2d", "ReflectionPad2d", "ReplicationPad2d").index(t)
        ph = d.raw_pad_h if d.raw_pad_h >= 0 else 1
        pw = (d.raw_pad_w if d.raw_pad_w >= 0 else 1) if mode == 0 else ph
        return pad2d(mode, x, _dflt(d.in_channels, 3), _dflt(d.input_height, 32), _dflt(d.input_width, 32), ph, pw)
    if t == "PixelShuffle":
        return pixel_shuffle(x, _dflt(d.in_channels, 12), _dflt(d.input_height, 32), _dflt(d.input_width, 32), _dflt(d.scale_h, 2))
    if t in ("UpsampleBilinear", "UpsampleBicubic"):
        return upsample_bilinear(x, _dflt(d.in_channels, 3), d.out_h, d.out_w, 2 * d.out_h, 2 * d.out_w, t == "UpsampleBicubic")
    if t == "MatMul":
        return batch_matmul(ins[0], ins[1], 1, d.in_features, d.out_features, d.embed_dim)
    if t == "BatchMatMul":
        return batch_matmul(ins[0], ins[1], d.seq_len, d.in_features, d.out_features, d.embed_dim)
    if t in ("BatchNorm2d", "BatchNorm1d"):
        return batchnorm_inference(x, w if (d.affine and w is not None and w.size) else None, d.eps)
    if t == "InstanceNorm2d":
        ch = _dflt(d.in_channels, 3)
        return instance_norm2d(x, w if (d.affine and w is not None and w.size >= 2 * ch) else None, ch, _dflt(d.input_height, 32),
                               _dflt(d.input_width, 32), d.eps)
    if t == "Transpose":
        return permute(x, [d.in_features, d.out_features], [1, 0])
    if t == "EmbeddingBag":
        return embedding_bag(ins[0], ins[1] if len(ins) >= 2 else None, w, max(1, d.vocab_size), max(1, d.embed_dim), d.padding_idx)
    if t == "PatchEmbed":
        dm = d.embed_dim if d.embed_dim > 0 else d.out_features
        st, npch, pd = max(1, d.seq_text), max(1, d.num_patches), max(1, d.patch_dim)
        if x.size != (st + 1) * dm + npch * pd:
            raise RuntimeError("PatchEmbed: input size mismatch")
        if w is None or w.size != pd * dm + dm:
            raise RuntimeError("PatchEmbed: weights not initialized or invalid size")
        return patch_embed(x, w, dm, st, npch, pd)
    if t == "Bilinear":
        if len(ins) < 2:
            raise RuntimeError("Bilinear requires 2 inputs")
        in1, in2 = max(1, d.in_features), max(1, d.out_features)
        out_f = d.embed_dim if d.embed_dim > 0 else d.target_dim0
        if out_f <= 0:
            raise RuntimeError("Bilinear: set embed_dim (output dim) or target_shape[0]")
        if ins[0].size % in1 or ins[1].size % in2 or ins[0].size // in1 != ins[1].size // in2:
            raise RuntimeError("Bilinear: batch mismatch between inputs")
        nw = out_f * in1 * in2
        return bilinear(ins[0], ins[1], w[:nw], w[nw : nw + out_f] if d.use_bias else None, in1, in2, out_f)
    if t == "MaxPool1d":  # LayerOpsExt.hpp:504-538 (the reference's layer switch has no case that calls it)
        ch = _dflt(d.in_channels, 1)
        k = _dflt(d.raw_kernel_h, 2)
        st = d.raw_stride_h if d.raw_stride_h > 0 else k
        return maxpool1d(x, ch, k, st, d.raw_pad_h if d.raw_pad_h >= 0 else 0)
    if t in ("RNN", "GRU", "LSTM"):
        if d.seq_len <= 0 or d.in_features <= 0 or d.out_features <= 0:
            raise RuntimeError("Recurrent: seq_len / in_features / out_features must be set")
        if x.size != d.seq_len * d.in_features:
            raise RuntimeError("Recurrent: input size mismatch (expected seq_len*in_features)")
        return recurrent(("RNN", "GRU", "LSTM").index(t), x, w, d.seq_len, d.in_features, d.out_features, d.use_bias)
    if t == "TokenMeanPool":
        return token_mean_pool(x, d.seq_len, d.embed_dim)
    if t in ("GlobalAvgPool2d", "AdaptiveAvgPool2d"):
        ch = d.in_channels if d.in_channels > 0 else 64
        h = d.input_height if d.input_height > 0 else 32
        wd = d.input_width if d.input_width > 0 else 32
        return global_avgpool(x, ch, h, wd)
    raise NotImplementedError(t)


def run_graph(descs, weights, inputs, rounding=None):
    """descs: list of MimirLayerDesc; weights: list of arrays (or None); inputs: name -> array."""
    store = {}
    main = inputs.get("x", inputs.get("__input__"))
    store["x"] = _f(main)
    store["__input__"] = _f(main)
    for k, v in inputs.items():
        store[k] = _f(v)
    for d, w in zip(descs, weights):
        names = [d.inputs[i].decode() for i in range(d.n_inputs)] or ["x"]
        for n in names:
            if n not in store:
                raise RuntimeError("Missing input tensor: " + n)
        out_name = (d.output or b"x").decode() or "x"
        if d.type.decode() in ("Split", "Chunk"):
            src = store[names[0]]
            off = 0
            for i, sz in enumerate(split_pieces(d, src.size)):
                store[f"{out_name}_{i}"] = src[off : off + sz].copy()
                off += sz
            out = store[out_name + "_0"].copy()
        else:
            out = run_layer(d, [store[n] for n in names], None if w is None else _f(w), rounding)
        store[out_name] = out
    return store["x"]
