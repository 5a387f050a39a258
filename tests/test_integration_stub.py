"""The binding a maintainer of the reference would write over the C ABI (the C++ block of INTEGRATION.md) is valid C++
against include/qlka.h and the torch headers: compiled with -fsyntax-only, nothing is run."""

import os
import re
import shutil
import subprocess
import sysconfig

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_binding_stub_compiles(tmp_path):
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    try:
        from torch.utils import cpp_extension
        includes = cpp_extension.include_paths()
    except Exception as e:                                  # pragma: no cover
        pytest.skip(f"torch headers unavailable: {e}")
    cuda_inc = "/usr/local/cuda/include"
    if not os.path.exists(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("no CUDA headers (ATen/cuda/CUDAContext.h needs them)")
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```cpp\n(.*?)```", text, re.S)
    assert blocks, "INTEGRATION.md has no C++ block"
    src = tmp_path / "binding_stub.cpp"
    src.write_text(blocks[0])
    cmd = [gxx, "-std=c++17", "-fsyntax-only", "-DTORCH_EXTENSION_NAME=qlka_stub", f"-I{os.path.join(ROOT, 'include')}",
           f"-I{cuda_inc}", f"-I{sysconfig.get_paths()['include']}", *[f"-I{p}" for p in includes], str(src)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
