"""The C++ GPU harnesses (examples/gpu): each links the C-ABI library, calls the
compiler-derived entry symbol with host buffers, checks every output against its own scalar
computation and prints `<capability> proof ok` (the reference's tier-3 convention,
docs/build-and-test.md:23-61)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "tianchen-rv_b200")
HARNESSES = ["add_f32", "add_i32", "q4_0_q8_0_block_dot", "q8_0_q8_0_block_dot", "q4_0_q8_0_gemm", "quantize_row_q8_0",
             "forward_f32", "repack_q4_0_q8_0"]


@pytest.fixture(scope="module")
def built(cuda):
    subprocess.run(["make", "-s", "-C", PKG, "harnesses"], check=True)


@pytest.mark.parametrize("name", HARNESSES)
def test_harness_proof(built, name):
    r = subprocess.run([os.path.join(PKG, "build", "bin", f"harness_{name}")], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "proof ok" in r.stdout
