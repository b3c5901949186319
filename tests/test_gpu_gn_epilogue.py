"""GroupNorm statistics out of the producing convolution's GEMM epilogue (MIMIR_B200_GN_EPILOGUE=1, read once per process,
hence the child process; off by default because it measured slower than the statistics sweep it replaces).

The convolution's epilogue leaves per-(32-pixel block, 32-channel chunk) sums behind, a small kernel merges them into
(mean, 1 / std) per (sample, group), and the GroupNorm that follows - on its own, or folded into the next convolution's
layout pass - reads them instead of sweeping the tensor.  Cases: 4, 8, 16 and 32 channels per group; 128 output channels
(operands swapped) and 256 (unswapped, CTA pairs where a full wave forms); several samples whose padded grids are not a
multiple of 32 rows, so that pixel blocks straddle two samples; enough (sample, group) rows for the stand-alone GroupNorm to
take the statistics it is handed (the row sweeps want one row per SM); a residual Add folded into the convolution; GroupNorm + SiLU
followed by a convolution (the folded form) and by an Add (the stand-alone form)."""
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
from mimir_framework_b200 import abi, runtime as rt
from oracle import port
rt.init(0, 0)
r = np.random.default_rng(11)
def conv(name, x, out, ic, oc, hw, ks=3):
    return abi.make_desc(name, "Conv2d", inputs=[x], output=out, in_channels=ic, out_channels=oc, input_height=hw[0], input_width=hw[1],
                         kernel=ks, stride=1, padding=ks // 2, params_count=oc * ic * ks * ks)
def gn(name, x, out, c, hw, groups):
    return abi.make_desc(name, "GroupNorm", inputs=[x], output=out, in_channels=c, input_height=hw[0], input_width=hw[1], num_groups=groups,
                         affine=1, use_bias=1, eps=1e-5, params_count=2 * c)
def weights(descs):
    out = []
    for d in descs:
        t, n = d.type.decode(), int(d.params_count)
        if t == "Conv2d":
            fan = d.in_channels * d.kernel * d.kernel
            out.append((r.standard_normal(n) * np.sqrt(2.0 / fan)).astype(np.float32))
        elif t == "GroupNorm":
            out.append(np.concatenate([1 + 0.2 * r.standard_normal(n // 2), 0.1 * r.standard_normal(n // 2)]).astype(np.float32))
        else:
            out.append(None)
    return out
n = 0
for batch, ic, oc, hw, groups in [(3, 32, 128, (13, 12), 32), (2, 64, 256, (20, 20), 32), (5, 32, 128, (9, 11), 8), (2, 32, 256, (12, 16), 8),
                                 (3, 64, 128, (10, 10), 4), (10, 32, 128, (8, 8), 16), (5, 32, 128, (12, 12), 32)]:
    # conv -> GN -> SiLU -> conv (folded into the second convolution's layout pass) -> GN -> SiLU -> Add(skip) (stand-alone)
    d = [conv("c1", "x", "a", ic, oc, hw), gn("g1", "a", "b", oc, hw, groups), abi.make_desc("s1", "SiLU", inputs=["b"], output="c"),
         conv("c2", "c", "d", oc, oc, hw), gn("g2", "d", "e", oc, hw, groups), abi.make_desc("s2", "SiLU", inputs=["e"], output="f"),
         abi.make_desc("add", "Add", inputs=["f", "a"], output="x")]
    w = weights(d)
    x = r.standard_normal(batch * ic * hw[0] * hw[1]).astype(np.float32)
    m = rt.GraphModel(d)
    for i, wi in enumerate(w):
        if wi is not None: m.upload_weights(i, wi)
    per = ic * hw[0] * hw[1]
    m.plan({"x": (per, False)}, batch)
    got = m.forward({"x": (x, False)}, batch, oc * hw[0] * hw[1]).ravel(); m.close()
    want = np.concatenate([port.run_graph(d, w, {"x": x[i * per:(i + 1) * per]}) for i in range(batch)])
    assert_close(got, want, f"conv-gn chain b{batch} {ic}->{oc} {hw} groups {groups}")
    n += 1
rt.check(rt.lib().mimir_b200_check_device(None))
print("GN_EPILOGUE_CASES_OK", n)
"""


def test_groupnorm_statistics_from_the_convolution_epilogue():
    env = dict(os.environ, MIMIR_B200_GN_EPILOGUE="1")
    out = subprocess.run([sys.executable, "-c", "ROOT = %r\n" % ROOT + CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "GN_EPILOGUE_CASES_OK 7" in out.stdout, out.stdout[-2000:]
