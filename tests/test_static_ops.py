"""The legacy static dispatch family (Model::computeLinear / computeMaxPool2D / ... , Model.hpp:388-429) as C++
wrappers over the C ABI (include/mimir_b200_static_ops.hpp): a small C++ program is compiled against the header
and the shared library; on a GPU box it runs and its outputs are checked against the oracle."""
import os
import subprocess

import numpy as np
import pytest

from mimir_framework_b200 import abi
from oracle import port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DRIVER = r"""
#include <cstdio>
#include <vector>
#include "mimir_b200_static_ops.hpp"
using namespace mimir_b200::static_ops;
static void dump(const char* name, const std::vector<float>& v) {
  std::printf("%s", name);
  for (float f : v) std::printf(" %.9g", f);
  std::printf("\n");
}
int main() {
  if (mimir_b200_init(0, 0) != MIMIR_B200_OK) { std::printf("init failed: %s\n", mimir_b200_last_error()); return 2; }
  std::vector<float> x(40), y;
  for (int i = 0; i < 40; ++i) x[i] = 0.25f * static_cast<float>((i * 7) % 11) - 1.0f;
  LayerParams lp;
  lp.in_features = 40; lp.out_features = 6;
  lp.weights.resize(240); lp.bias.resize(6);
  for (int i = 0; i < 240; ++i) lp.weights[i] = 0.01f * static_cast<float>((i * 13) % 17) - 0.05f;
  for (int i = 0; i < 6; ++i) lp.bias[i] = 0.1f * static_cast<float>(i);
  computeLinear(x, y, lp);
  dump("linear", y);
  std::vector<float> img(2 * 6 * 6), p;
  for (size_t i = 0; i < img.size(); ++i) img[i] = static_cast<float>((i * 5) % 13) - 6.0f;
  computeMaxPool2D(img, p, 6, 6, 2, 2, -1);
  dump("maxpool", p);
  computeAvgPool2D(img, p, 6, 6, 2, 3, 1);
  dump("avgpool", p);
  std::vector<float> a = x;
  computeActivation(a, "leaky_relu", 0.2f);
  dump("leaky", a);
  a = x;
  computeActivation(a, "gelu");
  dump("gelu", a);
  a = x;
  computeActivation(a, "softmax");
  dump("softmax", a);
  std::vector<float> g(8), b(8);
  for (int i = 0; i < 8; ++i) { g[i] = 1.0f + 0.1f * i; b[i] = -0.05f * i; }
  a = x;
  computeLayerNorm(a, g, b, 8, 1e-5f);
  dump("layernorm", a);
  a = x;
  computeActivation(a, "elu", 1.3f);
  dump("elu", a);
  a = x;
  computeActivation(a, "no_such_activation");
  dump("unknown_activation", a);
  { std::vector<float> o, kk(x.rbegin(), x.rend()); computeAttention(x, kk, x, o, 5, 8, 2); dump("attention", o); }
  {
    std::vector<float> d = x, gm{1.5f, -0.5f}, bt{0.1f, 0.2f}, mu{0.25f, -0.75f}, vr{0.5f, 2.0f};
    computeBatchNorm(d, gm, bt, mu, vr, 4, 2, 5, 1e-5f);
    dump("batchnorm", d);
    d = x;
    computeBatchNorm(d, gm, bt, mu, vr, 4, 2, 5, 1e-5f, true);
    dump("bn_training", d);
  }
  {
    // 2 x 5 x 4 input, 3 output channels, 3 x 3 kernel, stride 2, padding 2, dilation 2, with bias
    LayerParams cp;
    cp.kernel_size = 3; cp.stride = 2; cp.padding = 2; cp.dilation = 2;
    cp.weights.resize(3 * 2 * 9); cp.bias = {0.5f, -0.25f, 0.125f};
    for (size_t i = 0; i < cp.weights.size(); ++i) cp.weights[i] = 0.05f * static_cast<float>((i * 11) % 19) - 0.4f;
    std::vector<float> o;
    computeConv2D(x, o, cp, 5, 4, 2, 3);
    dump("conv2d", o);
    cp.dilation = 1; cp.padding = 1;
    computeConvTranspose2D(x, o, cp, 5, 4, 2, 3);
    dump("conv_transpose2d", o);
  }
  mimir_b200_shutdown();
  return 0;
}
"""


def _build(tmp_path):
    src = tmp_path / "static_ops_driver.cpp"
    src.write_text(DRIVER)
    exe = tmp_path / "static_ops_driver"
    libdir = os.path.dirname(abi.library_path())
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", libdir,
                    "-lmimir_b200", f"-Wl,-rpath,{libdir}"], check=True)
    return exe


def test_static_ops_header_compiles_and_links(tmp_path):
    assert os.path.exists(_build(tmp_path))


@pytest.mark.gpu
def test_static_ops_against_the_oracle(tmp_path):
    exe = _build(tmp_path)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    got = {}
    for line in out.splitlines():
        name, *vals = line.split()
        got[name] = np.array([float(v) for v in vals], np.float32)
    x = np.array([0.25 * ((i * 7) % 11) - 1.0 for i in range(40)], np.float32)
    w = np.array([0.01 * ((i * 13) % 17) - 0.05 for i in range(240)], np.float32)
    b = np.array([0.1 * i for i in range(6)], np.float32)
    np.testing.assert_allclose(got["linear"], port.linear(x, w, b, 1, 40, 6), atol=1e-4, rtol=1e-3)
    img = np.array([(i * 5) % 13 - 6.0 for i in range(72)], np.float32)
    assert np.array_equal(got["maxpool"], port.pool2d(1, img, 2, 6, 6, 2, 2, 2, 2, 0, 0))
    np.testing.assert_allclose(got["avgpool"], port.pool2d(0, img, 2, 6, 6, 3, 3, 1, 1, 0, 0), atol=1e-6)
    assert np.array_equal(got["leaky"], port.leaky_relu(x, 0.2))
    np.testing.assert_allclose(got["gelu"], port.eltwise(port.ELT["GELU"], x), atol=1e-6)
    np.testing.assert_allclose(got["softmax"], port.softmax(x, False), atol=1e-7, rtol=1e-5)
    g = np.array([1.0 + 0.1 * i for i in range(8)], np.float32)
    be = np.array([-0.05 * i for i in range(8)], np.float32)
    np.testing.assert_allclose(got["layernorm"], port.layernorm(x, g, be, 5, 8, 1e-5), atol=1e-5, rtol=1e-4)
    np.testing.assert_allclose(got["attention"], port.attention_qkv(x, x[::-1].copy(), x, 5, 8, 2), atol=1e-5, rtol=1e-4)
    np.testing.assert_allclose(got["batchnorm"], port.batchnorm_running(x, [1.5, -0.5], [0.1, 0.2], [0.25, -0.75], [0.5, 2.0], 4, 2, 5, 1e-5),
                               atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(got["elu"], port.elu(x, 1.3), atol=1e-6, rtol=1e-6)
    assert np.array_equal(got["unknown_activation"], x)
    np.testing.assert_allclose(got["bn_training"], port.batchnorm_batchstats(x, [1.5, -0.5], [0.1, 0.2], 4, 2, 5, 1e-5), atol=2e-6, rtol=2e-6)
    cw = np.array([0.05 * ((i * 11) % 19) - 0.4 for i in range(54)], np.float32)
    cb = np.array([0.5, -0.25, 0.125], np.float32)
    np.testing.assert_allclose(got["conv2d"], port.conv2d_dilated(x, cw, cb, 2, 3, 5, 4, 3, 2, 2, 2), atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(got["conv_transpose2d"], port.conv_transpose2d_scatter(x, cw, cb, 2, 3, 5, 4, 3, 2, 1), atol=2e-6, rtol=1e-5)
