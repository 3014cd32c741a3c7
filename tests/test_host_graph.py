"""The C++ host mirror of Marian's operator surface (marian-dev_b200/host): build check on CPU, and on
a GPU the operator-level test program tests/cpp/host_graph_test.cpp (affine / dot / affineWithReluDropout
on an expression graph with an intgemm8 parameter, bit-exact against the CPU checker, reference error texts)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "host_graph_test")


def _build():
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    if not os.path.exists(os.path.join(ROOT, "marian-dev_b200", "libmarian_i8.so")):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "marian-dev_b200", "csrc")])
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "marian-dev_b200", "host")])
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "tests", "cpp")])


def test_host_library_and_test_program_build():
    _build()
    assert os.path.exists(os.path.join(ROOT, "marian-dev_b200", "libmarian_host.so"))
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_host_graph_operator_tests(cuda_device):
    if not os.path.exists(EXE):
        _build()
    out = subprocess.run([EXE], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "host graph tests passed" in out.stdout
