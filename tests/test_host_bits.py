"""The pure bit manipulation behind the compression kernels (bit-plane transposes, bitmap reordering,
bit-sliced radix select) is plain integer code; this builds it for the host with g++ and checks it
against straightforward loops.  No GPU, no CUDA toolkit needed."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_compress_bit_helpers_on_host(tmp_path):
    exe = tmp_path / "compress_bits_check"
    src = os.path.join(HERE, "host", "compress_bits_check.cpp")
    inc = os.path.join(ROOT, "mustafar_b200", "csrc")
    subprocess.run(["g++", "-O2", "-std=c++17", "-I", inc, "-o", str(exe), src], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True, timeout=300)
    assert out.stdout.strip().endswith("ok")
