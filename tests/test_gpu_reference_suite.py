"""brotensor's own parity tests (tests/test_q4k_parity.cpp, test_q6k_parity.cpp, test_q8_0_parity.cpp,
test_quant_prefill_parity.cpp), compiled unmodified against brotensor's headers and core, with the nine
quant slots of its CUDA table filled by this repository's backend
(brotensor_b200/integration/brotensor_backend.cpp over libb200q.so). The executables are built on the
development machine by `make -C oracle gpu` into oracle/_ref/ and travel prebuilt; the control build
(`ref_*`, brotensor's own kernels in the same harness) must pass too, so a failure of `b200_*` alone
points at this repository."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
TESTS = ["test_q4k_parity", "test_q6k_parity", "test_q8_0_parity", "test_quant_prefill_parity"]


def _run(exe):
    path = os.path.join(REF, exe)
    if not os.path.exists(path):
        pytest.skip(f"oracle/_ref/{exe} not built (make -C oracle gpu, needs the brotensor source tree)")
    p = subprocess.run([path], capture_output=True, text=True, timeout=600)
    out = p.stdout + p.stderr
    assert p.returncode == 0, out[-3000:]
    assert "skipping" not in out, out[-1000:]  # the test must have found the CUDA backend
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("name", TESTS)
def test_brotensor_own_test_passes_on_this_backend(name):
    out = _run("b200_" + name)
    assert "FAIL" not in out, out[-3000:]


@pytest.mark.gpu
@pytest.mark.parametrize("name", TESTS)
def test_control_brotensor_own_kernels(name):
    _run("ref_" + name)
