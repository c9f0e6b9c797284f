"""The half-wise (two fp16 per register) mask / encoder arithmetic of the pack kernel, checked on the host against the
element-wise rules it restates (csrc/mask24.h, csrc/formats.h). No GPU: the header is plain integer C++."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_pack16_agrees_with_elementwise_rules(tmp_path):
    exe = str(tmp_path / "pack16_check")
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "onebitsparsemul_b200", "csrc"),
                           os.path.join(ROOT, "tests", "host", "pack16_check.cpp"), "-o", exe])
    out = subprocess.run([exe, "1000000"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.split() == ["0", "0", "0"]
