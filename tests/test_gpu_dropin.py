"""GPU: the reference's OWN test programs (tests/test_lut_gemm.cpp, tests/test_tmac_correctness.cpp,
tests/test_quantization.cpp of the reference, CMakeLists.txt:106-119) and its micro-benchmark
(tools/lutmac-bench.cpp), compiled UNCHANGED from the reference checkout against the drop-in
(shim/lutmac_b200_dropin.cpp) and liblutmac_b200.so in place of the reference's CPU kernels, plus
shim/test_dropin_linear (every branch of lut_linear).  The programs are built by shim/Makefile where
the reference checkout is present and travel as binaries; here they only run."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "shim", "_build")


def run(name, *args):
    exe = os.path.join(BUILD, name)
    if not os.path.exists(exe):
        pytest.skip(f"{exe} not built (make -C shim REF=<reference checkout>)")
    r = subprocess.run([exe, *args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (name, r.stdout[-1500:], r.stderr[-1500:])
    return r.stdout


# the counts are the number of tests each of the reference's programs registers
@pytest.mark.parametrize("name,passed", [("test_quantization", 4), ("test_lut_gemm", 8)])
def test_reference_test_programs_pass_on_the_gpu(name, passed):
    out = run(name)
    m = re.search(r"(\d+) passed, (\d+) failed", out)
    assert m, out[-800:]
    assert (int(m.group(1)), int(m.group(2))) == (passed, 0), out[-800:]


def test_reference_correctness_program_passes_on_the_gpu():
    """tests/test_tmac_correctness.cpp: ternary, 2-bit and 3-bit GEMV against Block::get dequantisation;
    it throws on a mismatch and prints its three maximum errors otherwise."""
    out = run("test_tmac_correctness")
    assert "All Correctness Tests Passed!" in out, out[-800:]
    assert len(re.findall(r"Max Error \(\w+\): ", out)) == 3, out[-800:]


def test_reference_micro_benchmark_runs_on_the_gpu():
    out = run("lutmac-bench", "--hidden-size", "1024", "--iterations", "3", "--warmup", "1")
    assert "GFLOP" in out or "GB/s" in out or "us" in out, out[-800:]


def test_lut_linear_branches_through_the_drop_in():
    out = run("test_dropin_linear")
    assert "all lut_linear branches ok" in out, out[-1500:]
    for branch in ("ternary", "int2 (RRQ)", "int4", "int8", "raw fp32"):
        assert re.search(re.escape(branch) + r".*ok", out), (branch, out[-1500:])
