"""The C++ host mirror of device.Backend (puter_b200/host/backend.hpp): builds everywhere, runs the reference's literal
fixtures on a GPU, and fails loudly (code -1, no fallback) without one."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "host_backend_test.bin")


def _build():
    from puter_b200.csrc import build as b

    lib = b.build()
    src = os.path.join(ROOT, "tests", "host_backend_test.cpp")
    if not os.path.exists(EXE) or os.path.getmtime(EXE) < max(os.path.getmtime(src), os.path.getmtime(lib)):
        subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O1", src, "-o", EXE, "-L" + os.path.dirname(lib), "-lputer_b200",
                               "-Wl,-rpath," + os.path.dirname(lib)])
    return EXE


def test_host_mirror_builds_and_refuses_to_run_without_a_device():
    import torch

    exe = _build()
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    res = subprocess.run([exe], capture_output=True, text=True)
    assert res.returncode == 77 and "no CPU fallback" in res.stdout


@pytest.mark.gpu
def test_host_mirror_reference_fixtures_on_gpu():
    res = subprocess.run([_build()], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "all checks passed" in res.stdout
