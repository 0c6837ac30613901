"""The header-only C++ host layer (ginn_b200/include/ginn): it must compile with a plain host
compiler against the C ABI, and its GPU test program (tests/cpp/test_host_api.cpp, modelled on
the reference's node and autobatch tests) must pass on a B200."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")
BIN = os.path.join(CPP, "test_host_api")


def build():
    from oracle import oracle as orc
    orc.build_cpu_path()
    res = subprocess.run(["make", "-C", CPP], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr


def test_host_layer_compiles_with_a_host_compiler():
    build()
    assert os.path.exists(BIN)


@pytest.mark.gpu
def test_host_layer_on_gpu():
    build()
    res = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(res.stdout, res.stderr)
    assert res.returncode == 0, res.stdout + res.stderr
