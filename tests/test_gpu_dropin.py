"""The drop-in C++ kernel_manager_t (einsummable_b200/host/) driven with the
reference's own einsummable_t / touch_t / fill_t types and compared with the
reference's own interpreter, as exps/gpuexec_kernelmanager.cc does.  The driver
(oracle/ref_km_parity.cc) is built where the reference tree exists and travels
as a binary."""
import os
import subprocess

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu
BIN = os.path.join(ROOT, "oracle", "_ref", "km_parity")


@pytest.mark.skipif(not os.path.exists(BIN), reason="oracle/_ref/km_parity not built (needs the reference tree)")
def test_dropin_kernel_manager_matches_reference_interpreter():
    res = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(res.stdout[-4000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "ALL OK" in res.stdout
    assert res.stdout.count("ok   ") >= 35
