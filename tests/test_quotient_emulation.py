"""CPU check of the arithmetic identities behind the quantizer kernels (tests/emul/emul_quotient.c): the correctly
rounded quotient from a reciprocal and one exact residual (float and double), rint through the subnormal grid, and
the shifted packing constant — evaluated with the host's IEEE operations on 80 M samples."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("gcc") is None, reason="gcc not available")
def test_quotient_and_rint_identities(tmp_path):
    exe = str(tmp_path / "emul_quotient")
    src = os.path.join(ROOT, "tests", "emul", "emul_quotient.c")
    # -ffp-contract=off: only the explicit fmaf/fma calls fuse; -mfma where the host has it (else libm's exact fma)
    flags = ["-O1", "-std=c11", "-ffp-contract=off"]
    cpu = open("/proc/cpuinfo").read() if os.path.exists("/proc/cpuinfo") else ""
    if " fma " in cpu or " fma\n" in cpu:
        flags.append("-mfma")
    subprocess.check_call(["gcc", *flags, "-o", exe, src, "-lm"])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.count(": ok") == 5
