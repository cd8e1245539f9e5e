"""The C++ host mirror (alice-train_b200/cpp/alice_train.hpp) compiled with g++ against the shared
library.  On CPU: it compiles, links, and reports "no device" the way GpuContext::new_blocking does in
the reference.  On a GPU: tests/cpp/host_mirror_test.cpp replays the reference's unit-test vectors."""
import os
import subprocess

import pytest

from helpers import PKG, ROOT

EXE = os.path.join(ROOT, "tests", "cpp", "_build", "host_mirror_test")


@pytest.fixture(scope="module")
def exe():
    import importlib.util
    spec = importlib.util.spec_from_file_location("ab_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    return mod.build_cpp_test()


def test_cpp_mirror_compiles_and_links(exe):
    assert os.path.exists(exe)
    out = subprocess.run(["ldd", exe], capture_output=True, text=True).stdout
    assert "libalice_b200.so" in out and "not found" not in out.split("libalice_b200.so")[1].splitlines()[0]


def test_cpp_mirror_without_device(exe):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    r = subprocess.run([exe, "--no-device"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "no-device ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_mirror_replays_reference_vectors(exe):
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and " 0 failed" in r.stdout, r.stdout + r.stderr
