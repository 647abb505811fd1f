"""CPU check of the register dequantizer and MMA fragment mapping used by the
mat-vec kernel: tests/emul/emul_fragments.cu includes the kernel's own header
and emulates one warp on the host."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"),
                    reason="nvcc not available")
def test_fragment_mapping_by_emulation(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = str(tmp_path / "emul_fragments")
    src = os.path.join(ROOT, "tests", "emul", "emul_fragments.cu")
    subprocess.check_call([nvcc, "-std=c++17", "-O1", "-Wno-deprecated-gpu-targets", "-I",
                           os.path.join(ROOT, "include"), "-o", exe, src])
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.count(": ok") == 12
