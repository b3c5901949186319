"""The CTA-pair form of the GEMM kernel (tcgen05 cta_group::2) is taken by default only for launches of a full wave of
tiles; MIMIR_B200_GEMM_PAIR=1 (read once per process, hence the child process) forces it wherever the form allows, so that
ragged shapes reach it: an odd number of row tiles (the last pair's second CTA has no rows), row and column counts that
are not multiples of the tile, K-block counts of 1 and more, every precision mode, bias / GELU / residual epilogues, the
operand-plane hand-off between two layers, and a convolution in the shifted-GEMM form."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, os
import numpy as np
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, ROOT)
from conftest import assert_close
from mimir_framework_b200 import abi, configs, runtime as rt
from oracle import port
rt.init(0, 0)
r = np.random.default_rng(3)
def run(descs, weights, x, out_n, prec):
    m = rt.GraphModel(descs, prec)
    for i, w in enumerate(weights): m.upload_weights(i, w)
    m.plan({"x": (x.size, False)}, 1)
    y = m.forward({"x": (x, False)}, 1, out_n); m.close(); return y.ravel()
n = 0
for rows, k, nout in [(300, 64, 70), (129, 512, 256), (640, 96, 520), (1000, 768, 300), (257, 32, 33)]:
    for prec in (abi.PREC_BF16X2, abi.PREC_BF16W):
        w = (r.standard_normal(k * nout + nout) * 0.05).astype(np.float32)
        if prec == abi.PREC_BF16W: w = configs.round_to_bf16(w)
        x = r.standard_normal(rows * k).astype(np.float32)
        d = [abi.make_desc("l", "Linear", in_features=k, out_features=nout, seq_len=rows, params_count=w.size)]
        assert_close(run(d, [w], x, rows * nout, prec), port.run_graph(d, [w], {"x": x}), f"linear {rows}x{k}x{nout} prec {prec}")
        n += 1
# Linear + GELU -> Linear + residual: planes handed from one pair launch to the next
rows, k = 700, 128
w1 = (r.standard_normal(k * 320 + 320) * 0.05).astype(np.float32); w2 = (r.standard_normal(320 * k + k) * 0.05).astype(np.float32)
d = [abi.make_desc("f1", "Linear", output="h", in_features=k, out_features=320, seq_len=rows, params_count=w1.size),
     abi.make_desc("g", "GELU", inputs=["h"], output="g"),
     abi.make_desc("f2", "Linear", inputs=["g"], output="o", in_features=320, out_features=k, seq_len=rows, params_count=w2.size),
     abi.make_desc("a", "Add", inputs=["o", "__input__"], output="x")]
x = r.standard_normal(rows * k).astype(np.float32)
assert_close(run(d, [w1, None, w2, None], x, rows * k, abi.PREC_BF16X2), port.run_graph(d, [w1, None, w2, None], {"x": x}), "ffn with residual"); n += 1
# convolution, 256 output channels (the unswapped channel-major form), 3 x 3 and 1 x 1
for ks in (3, 1):
    ic, oc, hw = 64, 256, 20
    cw = (r.standard_normal(oc * ic * ks * ks) * np.sqrt(2 / (ic * ks * ks))).astype(np.float32)
    d = [abi.make_desc("c", "Conv2d", in_channels=ic, out_channels=oc, input_height=hw, input_width=hw, kernel=ks, stride=1, padding=ks // 2, params_count=cw.size)]
    x = r.standard_normal(ic * hw * hw).astype(np.float32)
    assert_close(run(d, [cw], x, oc * hw * hw, abi.PREC_BF16X2), port.run_graph(d, [cw], {"x": x}), f"conv {ks}x{ks}"); n += 1
rt.check(rt.lib().mimir_b200_check_device(None))
print("PAIR_CASES_OK", n)
"""


def test_forced_cta_pairs_on_ragged_shapes():
    env = dict(os.environ, MIMIR_B200_GEMM_PAIR="1")
    out = subprocess.run([sys.executable, "-c", "ROOT = %r\n" % ROOT + CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "PAIR_CASES_OK 13" in out.stdout, out.stdout[-2000:]
