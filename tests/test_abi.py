"""The C-ABI library loads and exports every entry point that include/mimir_b200.h declares, and the
product path fails loudly (no CPU fallback) when there is no CUDA device.  CPU only: no compute call."""
import ctypes
import os
import re

import pytest

from mimir_framework_b200 import abi, runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mimir_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mimir_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = abi.load()
    names = declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_python_driver_binds_exactly_the_declared_symbols():
    assert sorted(runtime.EXPORTED_SYMBOLS) == declared_symbols()


def test_struct_layout_matches_header(tmp_path):
    """Compiles the header with the C compiler and compares sizeof / offsetof with the ctypes view."""
    import subprocess
    src = tmp_path / "layout.c"
    src.write_text("""
#include <stdio.h>
#include <stddef.h>
#include "mimir_b200.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(MimirLayerDesc), sizeof(MimirNamedInput), sizeof(MimirB200Stats),
         offsetof(MimirLayerDesc, params_count), offsetof(MimirLayerDesc, eps), offsetof(MimirLayerDesc, shape),
         offsetof(MimirNamedInput, broadcast), offsetof(MimirLayerDesc, head_dim), offsetof(MimirLayerDesc, raw_pad_w),
         offsetof(MimirLayerDesc, split_sizes), offsetof(MimirLayerDesc, num_chunks));
  return 0;
}
""")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [ctypes.sizeof(abi.MimirLayerDesc), ctypes.sizeof(abi.MimirNamedInput), ctypes.sizeof(abi.MimirB200Stats),
            abi.MimirLayerDesc.params_count.offset, abi.MimirLayerDesc.eps.offset, abi.MimirLayerDesc.shape.offset,
            abi.MimirNamedInput.broadcast.offset, abi.MimirLayerDesc.head_dim.offset, abi.MimirLayerDesc.raw_pad_w.offset,
            abi.MimirLayerDesc.split_sizes.offset, abi.MimirLayerDesc.num_chunks.offset]
    assert got == want


def test_abi_version():
    assert runtime.lib().mimir_b200_abi_version() == 3


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.mark.skipif(_has_gpu(), reason="checks the no-GPU failure mode")
def test_no_gpu_is_an_error_not_a_fallback():
    with pytest.raises(runtime.MimirB200Error) as e:
        runtime.init(0, 0)
    assert e.value.status == abi.E_CUDA
    # nothing works before init, and nothing silently computes on the CPU
    import numpy as np
    with pytest.raises(runtime.MimirB200Error) as e:
        runtime.linear_forward(np.ones(2, np.float32), np.ones(6, np.float32), None, 1, 2, 3)
    assert e.value.status == abi.E_NOT_INIT


def test_missing_library_raises(monkeypatch, tmp_path):
    monkeypatch.setattr(abi, "_lib", None)
    monkeypatch.setattr(abi, "library_path", lambda: str(tmp_path / "libmimir_b200.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        abi.load()
