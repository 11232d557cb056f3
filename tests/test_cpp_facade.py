"""The C++ face (include/flashmoe/flashmoe.hpp: the reference's namespace and function names over
the C ABI) compiles with a plain host compiler, links the shared library and reports argument
errors as exceptions.  No GPU is touched."""
import os
import shutil
import subprocess

import pytest

from flashmoe_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_facade_compiles_links_and_validates(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    N.lib()
    exe = tmp_path / "facade_check"
    libdir = str(N.LIB_PATH.parent)
    cmd = [gxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "facade_check.cpp"), "-L", libdir, "-lflashmoe_b200",
           f"-Wl,-rpath,{libdir}", "-o", str(exe)]
    p = subprocess.run(cmd, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "FACADE_OK" in r.stdout, r.stdout + r.stderr
