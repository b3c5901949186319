"""Parity of every per-op C-ABI entry point against the CPU oracle, on seeded inputs.

The checker is ``oracle/port.py`` (plain-C restatement) and, where it is built, the reference's own
compiled CPU code (``oracle/_ref``).  Integer/index work (embedding, argmax, data movement) must be
bit-exact; floating point must satisfy |gpu - cpu| <= 1e-4 + 1e-3 |cpu|.
"""
import numpy as np
import pytest

from conftest import assert_close
from mimir_framework_b200 import abi
from oracle import port

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("rows,in_f,out_f,bias", [
    (1, 2, 3, True),          # the reference's own Linear test shape (test_layers_all_types.cpp:71-100)
    (37, 50, 29, True),       # ragged everything, skinny path excluded (rows > 16)
    (8, 300, 70, True),       # skinny (weight-streaming) path
    (16, 4096, 130, False),   # skinny path, several K slices
    (3, 77, 5, True),         # skinny path, K not a multiple of 4 (scalar loads), fewer outputs than a row group
    (8, 33000, 24, True),     # skinny path, one row group spread over many warps
    (5, 130, 1000, False),    # skinny path, warps that span several row groups
    (8, 8192, 1000, True),    # skinny path, 256 items on 148 CTAs: ranges of one and two items, some across a tile border
    (16, 3000, 2000, False),  # skinny path, 378 items (ranges of 2 and 3), ragged K slice and ragged last tile
    (3, 20000, 300, True),    # skinny path, 40 K slices per tile: a tile's partials come from many CTAs
    (128, 64, 256, True),     # exactly one tile
    (129, 65, 257, True),     # one past a tile in every dimension
    (300, 1000, 515, True),
    (1024, 4096, 512, True),  # K of the headline config
])
def test_linear(backend, rows, in_f, out_f, bias):
    r = rng(rows * 7 + in_f)
    x = r.standard_normal(rows * in_f).astype(np.float32)
    w = r.uniform(-1, 1, out_f * in_f).astype(np.float32) / np.float32(np.sqrt(in_f))
    b = r.uniform(-0.1, 0.1, out_f).astype(np.float32) if bias else None
    want = port.linear(x, w, b, rows, in_f, out_f)
    got = backend.linear_forward(x, w, b, rows, in_f, out_f)
    assert_close(got, want, f"linear {rows}x{in_f}x{out_f}")


def test_linear_reference_known_answer(backend):
    # Tests/test_layers_all_types.cpp:71-100
    w = np.array([1, 2, 0, 1, -1, 0], np.float32)
    b = np.array([0, 1, 0], np.float32)
    got = backend.linear_forward(np.array([1, 2], np.float32), w, b, 1, 2, 3)
    np.testing.assert_allclose(got, [5, 3, -1], atol=1e-6)


@pytest.mark.parametrize("act", [abi.ELT_GELU, abi.ELT_SILU, abi.ELT_RELU])
@pytest.mark.parametrize("rows", [8, 200])
def test_linear_fused_activation(backend, act, rows):
    r = rng(act + rows)
    in_f, out_f = 192, 320
    x = r.standard_normal(rows * in_f).astype(np.float32)
    w = (r.standard_normal(out_f * in_f) / np.sqrt(in_f)).astype(np.float32)
    b = r.uniform(-0.1, 0.1, out_f).astype(np.float32)
    want = port.eltwise(act, port.linear(x, w, b, rows, in_f, out_f))
    got = backend.linear_forward(x, w, b, rows, in_f, out_f, activation=act)
    assert_close(got, want, f"linear+act{act}")


def test_linear_bf16_weight_mode(backend):
    # weights already representable in bf16: the two-MMA mode must meet the same tolerance
    r = rng(5)
    rows, in_f, out_f = 260, 768, 384
    x = r.standard_normal(rows * in_f).astype(np.float32)
    w = (r.standard_normal(out_f * in_f) * 0.02).astype(np.float32)
    w = (w.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)  # truncate to bf16
    want = port.linear(x, w, None, rows, in_f, out_f)
    got = backend.linear_forward(x, w, None, rows, in_f, out_f, precision=abi.PREC_BF16W)
    assert_close(got, want, "linear bf16-weight mode")


@pytest.mark.parametrize("M,K,N", [(2, 3, 2), (40, 64, 192), (130, 70, 33), (256, 256, 768)])
def test_matmul(backend, M, K, N):
    r = rng(M + K + N)
    a = r.standard_normal(M * K).astype(np.float32)
    b = (r.standard_normal(K * N) / np.sqrt(K)).astype(np.float32)
    assert_close(backend.matmul(a, b, M, K, N), port.matmul(a, b, M, K, N), f"matmul {M}x{K}x{N}")


def test_matmul_reference_known_answer(backend):
    # Tests/test_layers_all_types.cpp:473-506: [[1,2,3],[4,5,6]] x [[7,8],[9,10],[11,12]]
    got = backend.matmul(np.arange(1, 7, dtype=np.float32), np.arange(7, 13, dtype=np.float32), 2, 3, 2)
    np.testing.assert_allclose(got, [58, 64, 139, 154], rtol=1e-6)


@pytest.mark.parametrize("batch,seq,E,heads,causal", [
    (1, 40, 64, 4, 0), (1, 40, 64, 4, 1),     # head_dim 16 -> row kernel
    (2, 128, 256, 4, 0),                      # config-1 attention shape (head_dim 64)
    (2, 200, 128, 2, 1),                      # ragged seq, causal, head_dim 64
    (1, 96, 128, 4, 1),                       # head_dim 32
    (1, 70, 256, 2, 0),                       # head_dim 128
    (1, 64, 512, 1, 0),                       # single head, head_dim 512 (UNet mid-block shape class), row kernel (seq % 128 != 0)
    (3, 256, 512, 1, 0),                      # the UNet mid block itself: one wide head as two block-diagonal GEMMs
    (2, 128, 128, 1, 1),                      # the same form, causal, one 128-row tile per sample
    (2, 384, 192, 1, 1),                      # three row tiles per sample, score rows of 384 (K of the second GEMM a multiple of 128 only)
    (3, 129, 192, 3, 1),                      # tensor-core core (head_dim 64): one row past a query tile
    (1, 1, 64, 1, 0),                         # tensor-core core: a single token
    (2, 63, 128, 2, 0),                       # tensor-core core: ragged key tile
    (1, 1024, 128, 2, 1),                     # tensor-core core: decoder sequence length, causal
])
def test_attention(backend, batch, seq, E, heads, causal):
    r = rng(seq + E + heads + causal)
    x = r.standard_normal(batch * seq * E).astype(np.float32)
    w = (r.standard_normal(4 * E * E) / np.sqrt(E)).astype(np.float32)
    want = np.concatenate([port.attention(x[i * seq * E:(i + 1) * seq * E], w, seq, E, heads, causal) for i in range(batch)])
    got = backend.attention(x, w, batch, seq, E, heads, causal)
    assert_close(got, want, f"attention b{batch} s{seq} E{E} h{heads} c{causal}")


@pytest.mark.parametrize("causal", [0, 1])
def test_attention_running_maximum_grows_across_key_tiles(backend, causal):
    """Scores whose row maximum grows by 2^8 .. 2^16 from one 64-key tile to the next (later keys are
    "louder"): the tensor-core kernel keeps a stale maximum below 2^8 of growth and rescales the output
    it holds in TMEM above it, so both branches run.  Scores reach |s| = 24 here, which amplifies the
    rounding differences of the QKV projection by e^(24 * 1e-5): the gate is widened accordingly (the
    fp32 CUDA-core attention shows the same spread); a wrong rescale would be off by factors."""
    batch, seq, E, heads = 2, 320, 128, 2
    r = rng(77)
    x = r.standard_normal((batch, seq, E)).astype(np.float32)
    x *= (1.0 + 5.0 * np.arange(seq, dtype=np.float32) / seq)[None, :, None]
    w = (r.standard_normal(4 * E * E) / np.sqrt(E)).astype(np.float32)
    w[: 3 * E * E].reshape(E, 3 * E)[:, : 2 * E] *= 0.45
    x = x.ravel()
    want = np.concatenate([port.attention(x[i * seq * E:(i + 1) * seq * E], w, seq, E, heads, causal) for i in range(batch)])
    got = backend.attention(x, w, batch, seq, E, heads, causal)
    assert_close(got, want, f"attention with growing maximum, causal={causal}", abs_tol=1e-3, rel_tol=5e-3)


def test_attention_identity_weights(backend):
    # hand-checkable: Wq=Wk=0 makes every score 0 -> uniform attention -> each output row is the mean
    # of V rows (all rows for non-causal); Wv = Wout = I.
    seq, E = 5, 8
    w = np.zeros(4 * E * E, np.float32)
    wqkv = w[:3 * E * E].reshape(E, 3 * E)
    wqkv[:, 2 * E:] = np.eye(E)
    w[3 * E * E:] = np.eye(E).ravel()
    x = rng(1).standard_normal(seq * E).astype(np.float32)
    got = backend.attention(x, w, 1, seq, E, 2, 0).reshape(seq, E)
    want = np.tile(x.reshape(seq, E).mean(0), (seq, 1))
    assert_close(got, want, "attention identity")


@pytest.mark.parametrize("batch,ic,oc,h,w,k,s,p,relu", [
    (1, 1, 1, 2, 2, 1, 1, 0, 0),      # the reference's Conv2d test (test_layers_all_types.cpp:105-133)
    (2, 5, 13, 11, 9, 3, 1, 1, 0),
    (1, 3, 64, 32, 32, 7, 2, 3, 0),   # stem shape class
    (2, 16, 24, 14, 14, 3, 1, 1, 1),
    (1, 64, 128, 28, 28, 3, 1, 1, 0),
    (1, 32, 48, 10, 10, 1, 1, 0, 0),  # 1x1 skip conv (shifted-GEMM path, one tap)
    (3, 32, 40, 13, 9, 3, 1, 1, 1),   # shifted-GEMM path: several samples, odd sizes, ReLU
    (2, 64, 24, 7, 11, 5, 1, 2, 0),   # shifted-GEMM path, 5x5 taps
    (1, 256, 300, 20, 20, 3, 1, 1, 0),  # shifted-GEMM path, two column tiles
    (2, 32, 16, 12, 12, 3, 2, 1, 0),  # stride 2 stays on the im2col path
    (2, 64, 3, 40, 40, 3, 1, 1, 0),   # few output channels: operands swapped (channels on the TMEM lanes)
    (2, 256, 128, 24, 24, 3, 1, 1, 1),  # 128 channels with a long K: swapped too, ReLU
    (3, 32, 20, 30, 26, 5, 1, 2, 0),  # swapped, 5x5 taps, ragged pixel tiles
    (2, 40, 3, 70, 66, 3, 1, 1, 0),   # an RGB head on a large image: direct fp32 kernel, ragged tiles, channel tail (40 = 5 x 8)
    (1, 19, 8, 64, 64, 5, 1, 2, 1),   # direct kernel: eight output channels, 5x5, channel count not a multiple of 8, ReLU
    (2, 12, 1, 96, 50, 1, 1, 0, 0),   # direct kernel: one output channel, 1x1
    (2, 40, 3, 72, 68, 3, 1, 1, 0),   # direct kernel, rows of whole 16-byte chunks: the vector form, one ragged tile
    (1, 16, 3, 66, 260, 3, 1, 1, 1),  # vector form: three tiles across (128 + 128 + 4), halo values cross tile and lane borders
    (1, 6, 2, 65, 132, 7, 1, 3, 0),   # vector form, 7x7: three halo values either side
    (2, 40, 24, 10, 12, 3, 1, 1, 0),  # streamed layout pass: 40 channels (a partial channel block), one short pixel tile
    (1, 72, 32, 9, 68, 3, 1, 1, 1),   # streamed layout pass: two channel blocks (64 + 8), two pixel tiles (64 + 4), 11 padded rows
    (2, 16, 32, 6, 8, 1, 1, 0, 0),    # streamed layout pass without a padding ring (1x1)
])
def test_conv2d(backend, batch, ic, oc, h, w, k, s, p, relu):
    r = rng(ic * oc + h)
    x = r.random(batch * ic * h * w).astype(np.float32)
    wt = (r.standard_normal(oc * ic * k * k) * np.sqrt(2.0 / (ic * k * k))).astype(np.float32)
    if (ic, oc, k) == (1, 1, 1):
        x = np.array([1, 2, 3, 4], np.float32)
        wt = np.array([2.0], np.float32)
    per = ic * h * w
    want = np.concatenate([port.conv2d(x[i * per:(i + 1) * per], wt, ic, oc, h, w, k, s, p, relu) for i in range(batch)])
    got = backend.conv2d(x, wt, batch, ic, oc, h, w, k, s, p, relu)
    assert_close(got, want, f"conv {ic}->{oc} k{k} s{s}")
    if (ic, oc, k) == (1, 1, 1):
        np.testing.assert_allclose(got, [2, 4, 6, 8], atol=1e-6)


@pytest.mark.parametrize("rows,n", [(4, 300), (3, 768), (2, 32768), (1, 40000), (9, 5), (3, 98304), (5, 98301), (2, 200000), (150, 5000),
                                    (150, 40000), (149, 40002)])  # a row shared by the CTAs of a cluster; ragged slices
def test_layernorm(backend, rows, n):
    r = rng(n)
    x = (r.standard_normal(rows * n) * 2 + 0.5).astype(np.float32)
    g, b = r.standard_normal(n).astype(np.float32), r.standard_normal(n).astype(np.float32)
    assert_close(backend.layernorm(x, g, b, rows, n), port.layernorm(x, g, b, rows, n, 1e-5), f"layernorm {rows}x{n}")
    assert_close(backend.layernorm(x, None, None, rows, n), port.layernorm(x, None, None, rows, n, 1e-5), "layernorm no affine")


@pytest.mark.parametrize("batch,n,ng", [(2, 1200, 700), (1, 16384, 16384), (3, 50000, 50000), (2, 786432, 786432),
                                        (3, 33333, 20001), (5, 16385, 0)])
def test_rmsnorm(backend, batch, n, ng):
    r = rng(n)
    x = r.standard_normal(batch * n).astype(np.float32)
    g = r.standard_normal(ng).astype(np.float32) if ng else None
    want = np.concatenate([port.rmsnorm(x[i * n:(i + 1) * n], g, 1e-5) for i in range(batch)])
    assert_close(backend.rmsnorm(x, g, batch, n), want, f"rmsnorm {batch}x{n}")


def test_rmsnorm_long_sample_follows_the_sequential_sum(backend):
    """The reference adds the squares of a whole sample in one fp32 chain (LayerOpsExt.hpp:353-356); over 786 432
    elements that chain loses ~4e-4 of the sum.  The single-pass kernel replays the chain's rounding, so it must sit
    far closer to the reference than that loss (half of which would show in every output)."""
    n = 786432
    x = rng(5).standard_normal(2 * n).astype(np.float32)
    want = np.concatenate([port.rmsnorm(x[i * n:(i + 1) * n], None, 1e-5) for i in range(2)])
    got = backend.rmsnorm(x, None, 2, n)
    rel = np.abs(got - want) / np.maximum(np.abs(want), 1e-3)
    assert rel.max() < 5e-6, f"max relative deviation {rel.max():.3e}"
    exact = x.reshape(2, n) / np.sqrt((x.reshape(2, n).astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5)
    assert np.abs(want - exact.ravel()).max() > 2e-5, "the case no longer exercises the chain's rounding loss"


def test_rmsnorm_reference_known_answer(backend):
    # Tests/test_layers_all_types.cpp:306-323: x = [3, 4], gamma = 1 -> x / sqrt(12.5 + eps)
    got = backend.rmsnorm(np.array([3, 4], np.float32), np.ones(2, np.float32), 1, 2, 1e-5)
    rms = np.sqrt(np.float32(12.5) + np.float32(1e-5))
    np.testing.assert_allclose(got, [3 / rms, 4 / rms], rtol=1e-6)


@pytest.mark.parametrize("batch,ch,h,w,groups,act", [
    (1, 4, 2, 2, 2, -1), (2, 16, 9, 9, 4, -1), (2, 64, 28, 28, 32, abi.ELT_SILU), (1, 256, 56, 56, 32, abi.ELT_SILU),
    (5, 64, 160, 120, 32, abi.ELT_SILU), (10, 32, 180, 110, 16, -1),  # >= one row per SM, rows of 150 KB: the cluster sweep
])
def test_groupnorm(backend, batch, ch, h, w, groups, act):
    r = rng(ch + h)
    per = ch * h * w
    x = (r.standard_normal(batch * per) * 1.5 + 0.3).astype(np.float32)
    g, b = r.standard_normal(ch).astype(np.float32), r.standard_normal(ch).astype(np.float32)
    want = np.concatenate([port.groupnorm(x[i * per:(i + 1) * per], g, b, ch, h, w, groups, 1e-5) for i in range(batch)])
    if act >= 0:
        want = port.eltwise(act, want)
    assert_close(backend.groupnorm(x, g, b, batch, ch, h, w, groups, 1e-5, act), want, f"groupnorm C{ch} {h}x{w}")


def test_layernorm_long_rows_far_from_zero(backend):
    """Rows whose first element (the shift of the one-sweep statistics) lies five standard deviations from the mean: the
    shifted sums give way to a second, centred sweep (LayerOps.hpp:287-300 takes the variance around the mean), and every
    CTA that shares a row must take that decision alike."""
    rows, n = 150, 40000
    x = (rng(3).standard_normal(rows * n) + 5.0).astype(np.float32)
    x[::n] = 0.0
    assert_close(backend.layernorm(x, None, None, rows, n), port.layernorm(x, None, None, rows, n, 1e-5), "layernorm, poor shift")


@pytest.mark.parametrize("batch,n,log", [(3, 7, False), (2, 1200, True), (2, 32000, False), (1, 70000, False), (1, 70000, True)])
def test_softmax(backend, batch, n, log):
    x = (rng(n).standard_normal(batch * n) * 3).astype(np.float32)
    want = np.concatenate([port.softmax(x[i * n:(i + 1) * n], log) for i in range(batch)])
    assert_close(backend.softmax(x, batch, n, log), want, f"softmax {batch}x{n} log={log}")


@pytest.mark.parametrize("op", [abi.ELT_GELU, abi.ELT_SILU, abi.ELT_RELU, abi.ELT_TANH, abi.ELT_SIGMOID])
def test_activations(backend, op):
    x = np.concatenate([(rng(op).standard_normal(4099) * 4).astype(np.float32), np.array([0, -0.0, 1, -1, 20, -20, 88, -88], np.float32)])
    assert_close(backend.eltwise(op, x), port.eltwise(op, x), f"activation {op}", abs_tol=1e-6, rel_tol=1e-5)


def test_add_multiply_bitexact(backend):
    r = rng(9)
    a, b = r.standard_normal(3 * 1000).astype(np.float32), r.standard_normal(3 * 1000).astype(np.float32)
    assert np.array_equal(backend.eltwise(abi.ELT_ADD, a, b, batch=3), a + b)
    assert np.array_equal(backend.eltwise(abi.ELT_MULTIPLY, a, b, batch=3), a * b)
    # `i % small_n` broadcast per sample (LayerOps.hpp:190-197) and scalar broadcast
    small = r.standard_normal(3 * 250).astype(np.float32)
    want = (a.reshape(3, 4, 250) + small.reshape(3, 1, 250)).ravel()
    assert np.array_equal(backend.eltwise(abi.ELT_ADD, a, small, batch=3), want)
    assert np.array_equal(backend.eltwise(abi.ELT_ADD, a[:1000], np.array([2.5], np.float32)), a[:1000] + np.float32(2.5))
    with pytest.raises(backend.MimirB200Error):
        backend.eltwise(abi.ELT_ADD, a[:1000], a[:333])  # "Add: input sizes must match or be broadcastable"
    with pytest.raises(backend.MimirB200Error):
        backend.eltwise(abi.ELT_MULTIPLY, a[:1000], a[:500])


def test_embedding_bitexact(backend):
    r = rng(3)
    vocab, dim = 50, 24
    table = r.standard_normal(vocab * dim).astype(np.float32)
    ids = np.array([0, 3, 49, 50, -1, 7.4, 7.5, 8.5, 2.5, -0.4], np.float32)  # padding, out of range, llround ties
    want = port.embedding(ids, table, vocab, dim, 0)
    assert np.array_equal(backend.embedding(ids, table, vocab, dim, 0), want)
    # int ids, padding_idx -> zero row (Tests/test_runtime_embedding_int_inputs.cpp:44-74)
    iids = np.array([1, 0, 2, 49, 77], np.int32)
    got = backend.embedding(iids, table, vocab, dim, 0).reshape(5, dim)
    assert np.array_equal(got[0], table.reshape(vocab, dim)[1]) and not got[1].any() and not got[4].any()
    # odd dim (scalar path), no padding index
    table3 = r.standard_normal(10 * 3).astype(np.float32)
    assert np.array_equal(backend.embedding(np.array([9, 0], np.float32), table3, 10, 3, -1), port.embedding([9, 0], table3, 10, 3, -1))


def test_data_movement_bitexact(backend):
    r = rng(4)
    x = r.standard_normal(2 * 3 * 4 * 5).astype(np.float32)
    want = np.concatenate([port.upsample_nearest(x[i * 60:(i + 1) * 60], 3, 4, 5, 2, 3) for i in range(2)])
    assert np.array_equal(backend.upsample_nearest(x, 2, 3, 4, 5, 2, 3), want)
    x2 = r.standard_normal(2 * 3 * 5 * 6).astype(np.float32)  # 2 x 2 with an even width: the vectorised kernel
    want = np.concatenate([port.upsample_nearest(x2[i * 90:(i + 1) * 90], 3, 5, 6, 2, 2) for i in range(2)])
    assert np.array_equal(backend.upsample_nearest(x2, 2, 3, 5, 6, 2, 2), want)
    for dims in ([2, 0, 1], [0, 2, 1], [1, 0, 2]):
        want = np.concatenate([port.permute(x[i * 60:(i + 1) * 60], [3, 4, 5], dims) for i in range(2)])
        assert np.array_equal(backend.permute(x, [3, 4, 5], dims, batch=2), want)
    with pytest.raises(backend.MimirB200Error):
        backend.permute(x[:60], [3, 4, 5], [0, 0, 1])


def test_pools(backend):
    r = rng(6)
    x = r.standard_normal(2 * 7 * 12).astype(np.float32)
    want = np.concatenate([port.token_mean_pool(x[i * 84:(i + 1) * 84], 7, 12) for i in range(2)])
    assert_close(backend.token_mean_pool(x, 2, 7, 12), want, "token mean pool", abs_tol=1e-6, rel_tol=1e-6)
    want = np.concatenate([port.global_avgpool(x[i * 84:(i + 1) * 84], 3, 4, 7) for i in range(2)])
    assert_close(backend.global_avgpool(x, 2, 3, 4, 7), want, "global avgpool", abs_tol=1e-6, rel_tol=1e-5)


def test_norm_statistics_are_robust_to_offsets_and_outliers(backend):
    """The streaming norm kernels take mean and variance from one sweep of sums shifted by the row's first
    element; rows with a large common offset and rows whose first element is an outlier (worst case for
    the shift) must still match the two-pass reference."""
    r = rng(77)
    rows, n = 200, 5000  # >= one row per SM: the CTA-per-row sweep path
    x = (300.0 + r.standard_normal((rows, n))).astype(np.float32)
    x[::2, 0] = 1e4
    x[1::4, 0] = -3e3
    g, b = r.standard_normal(n).astype(np.float32), r.standard_normal(n).astype(np.float32)
    assert_close(backend.layernorm(x.ravel(), g, b, rows, n), port.layernorm(x.ravel(), g, b, rows, n, 1e-5), "layernorm offset/outlier rows")
    # GroupNorm slabs with the same treatment
    batch, ch, h, w, groups = 8, 64, 20, 20, 32
    per = ch * h * w
    xg = (50.0 + r.standard_normal(batch * per) * 0.5).astype(np.float32)
    xg[::per // groups] = 7e3  # first element of every group slab
    gg, bg = r.standard_normal(ch).astype(np.float32), r.standard_normal(ch).astype(np.float32)
    want = np.concatenate([port.groupnorm(xg[i * per:(i + 1) * per], gg, bg, ch, h, w, groups, 1e-5) for i in range(batch)])
    assert_close(backend.groupnorm(xg, gg, bg, batch, ch, h, w, groups, 1e-5, -1), want, "groupnorm offset/outlier slabs")


@pytest.mark.parametrize("batch,seq,d_model,heads", [(1, 5, 8, 2), (2, 77, 128, 2), (3, 130, 96, 3), (1, 300, 40, 1)])
def test_attention_on_separate_qkv(backend, batch, seq, d_model, heads):
    """Model::computeAttention (Model.cpp:4223-4289): projected Q / K / V in, no mask, heads side by side."""
    r = rng(seq * d_model)
    q, k, v = (r.standard_normal(batch * seq * d_model).astype(np.float32) for _ in range(3))
    n = seq * d_model
    want = np.concatenate([port.attention_qkv(q[b * n:(b + 1) * n], k[b * n:(b + 1) * n], v[b * n:(b + 1) * n], seq, d_model, heads)
                           for b in range(batch)])
    assert_close(backend.attention_qkv(q, k, v, batch, seq, d_model, heads), want, f"attention_qkv {batch}x{seq}x{d_model}/{heads}")


@pytest.mark.parametrize("batch,ch,spatial", [(1, 1, 1), (2, 3, 50), (4, 64, 49), (1, 7, 1000)])
def test_batchnorm_with_running_statistics(backend, batch, ch, spatial):
    """Model::computeBatchNorm at inference (Layers.hpp:932-970)."""
    r = rng(ch * spatial)
    x = (r.standard_normal(batch * ch * spatial) * 3 + 1).astype(np.float32)
    g, b, m = (r.standard_normal(ch).astype(np.float32) for _ in range(3))
    var = (r.random(ch) + 0.1).astype(np.float32)
    want = port.batchnorm_running(x, g, b, m, var, batch, ch, spatial, 1e-5)
    assert_close(backend.batchnorm_running(x, g, b, m, var, batch, ch, spatial), want, f"batchnorm_running {batch}x{ch}x{spatial}")


@pytest.mark.parametrize("batch,ch,spatial", [(1, 1, 2), (3, 5, 17), (4, 64, 49), (2, 7, 3000)])
def test_batchnorm_with_batch_statistics(backend, batch, ch, spatial):
    """Model::computeBatchNorm with training = true (Layers.hpp:940-959): statistics from the batch itself."""
    r = rng(ch * spatial + 1)
    x = (r.standard_normal(batch * ch * spatial) * 3 + 1).astype(np.float32)
    g, b = (r.standard_normal(ch).astype(np.float32) for _ in range(2))
    want = port.batchnorm_batchstats(x, g, b, batch, ch, spatial, 1e-5)
    np.testing.assert_allclose(backend.batchnorm_batchstats(x, g, b, batch, ch, spatial), want, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("ic,oc,h,wd,k,st,pad,dil,bias", [(3, 5, 9, 11, 3, 1, 1, 1, True), (2, 4, 12, 10, 3, 2, 2, 2, True), (4, 3, 7, 7, 1, 1, 0, 1, False),
                                                           (1, 2, 15, 13, 5, 3, 4, 3, True), (2, 2, 20, 20, 9, 1, 4, 1, False), (16, 8, 32, 32, 3, 1, 2, 2, True)])
def test_static_conv2d_with_bias_and_dilation(backend, ic, oc, h, wd, k, st, pad, dil, bias):
    """Model::computeConv2D -> Conv::conv2d, scalar branch (Layers.hpp:690-721); two samples at once."""
    r = rng(ic * h * wd + k)
    x = r.standard_normal(2 * ic * h * wd).astype(np.float32)
    w = (r.standard_normal(oc * ic * k * k) * 0.3).astype(np.float32)
    b = r.standard_normal(oc).astype(np.float32) if bias else None
    n = ic * h * wd
    want = np.concatenate([port.conv2d_dilated(x[s * n:(s + 1) * n], w, b, ic, oc, h, wd, k, st, pad, dil) for s in range(2)])
    np.testing.assert_allclose(backend.conv2d_dilated(x, w, b, 2, ic, oc, h, wd, k, st, pad, dil), want, atol=1e-5, rtol=2e-5)


@pytest.mark.parametrize("ic,oc,h,wd,k,st,pad,bias", [(3, 4, 5, 6, 4, 2, 1, True), (2, 3, 7, 5, 3, 1, 0, False), (1, 2, 4, 4, 2, 3, 0, True), (4, 2, 6, 6, 3, 2, 2, True),
                                                       (8, 8, 16, 16, 5, 3, 1, True)])
def test_static_conv_transpose2d_scatter_form(backend, ic, oc, h, wd, k, st, pad, bias):
    """Model::computeConvTranspose2D -> Conv::conv_transpose2d (Layers.hpp:775-818); two samples at once."""
    r = rng(ic * h * wd + k + 5)
    x = r.standard_normal(2 * ic * h * wd).astype(np.float32)
    w = (r.standard_normal(oc * ic * k * k) * 0.3).astype(np.float32)
    b = r.standard_normal(oc).astype(np.float32) if bias else None
    n = ic * h * wd
    want = np.concatenate([port.conv_transpose2d_scatter(x[s * n:(s + 1) * n], w, b, ic, oc, h, wd, k, st, pad) for s in range(2)])
    np.testing.assert_allclose(backend.conv_transpose2d_scatter(x, w, b, 2, ic, oc, h, wd, k, st, pad), want, atol=1e-5, rtol=2e-5)


def test_elu_of_the_static_family(backend):
    """Model::elu_inplace (Model.hpp:505-509) behind computeActivation("elu")."""
    x = (rng(3).standard_normal(5000) * 3).astype(np.float32)
    got = backend.eltwise_alpha(abi.ELT_ELU, x, 1.3)
    np.testing.assert_allclose(got, port.elu(x, 1.3), atol=1e-6, rtol=1e-6)


def test_gemm_output_through_tma_stores():
    """MIMIR_B200_GEMM_TMA_STORE=1 routes row-major fp32 GEMM outputs through shared-memory staging and TMA stores
    (off by default: measured neutral).  The switch is read once per process, so the Linear, MatMul and attention
    cases - ragged row and column counts included - run again in a child interpreter with it set."""
    import os
    import subprocess
    import sys

    env = dict(os.environ, MIMIR_B200_GEMM_TMA_STORE="1")
    here = os.path.abspath(__file__)
    r = subprocess.run([sys.executable, "-m", "pytest", here, "-q", "-m", "gpu", "-x", "-k",
                        "test_linear or test_matmul or test_attention and not tma_stores"], env=env, capture_output=True, text=True,
                       cwd=os.path.dirname(os.path.dirname(here)))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert " passed" in r.stdout


def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_device_usable(backend):
    """The tensor-core kernels bound every mbarrier wait; when one runs out they set a device word, drain, free their
    tensor memory and return.  Here that path runs on purpose: a one-block kernel waits 1 ms on a barrier that nothing
    arrives on.  The host then reads E_TIMEOUT with the site of the wait, the word is cleared, and a GEMM straight
    afterwards is correct - nothing faulted, nothing spun past its limit."""
    lib = backend.lib()
    backend.check(lib.mimir_b200_check_device(None))  # clean to start with
    backend.check(lib.mimir_b200_selftest_wait_timeout(1_000_000, None))
    status = lib.mimir_b200_check_device(None)
    assert status == abi.E_TIMEOUT
    assert "site 90" in lib.mimir_b200_last_error().decode()
    assert lib.mimir_b200_check_device(None) == abi.OK  # reading it cleared it
    r = np.random.default_rng(0)
    x, w = r.standard_normal((200, 96)).astype(np.float32), r.standard_normal((64, 96)).astype(np.float32)
    assert_close(backend.linear_forward(x.ravel(), w.ravel(), None, 200, 96, 64), port.linear(x.ravel(), w.ravel(), None, 200, 96, 64), "GEMM after a timed-out wait")
    assert lib.mimir_b200_selftest_wait_timeout(0, None) == abi.E_INVALID
    assert lib.mimir_b200_selftest_wait_timeout(10**12, None) == abi.E_INVALID
