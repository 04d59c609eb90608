"""CPU check of the host-side layout arithmetic of the single-session decode kernel (which CTA owns which rows, chunk sizes, the
shared-memory ring, every fixed capacity of the kernel's tables): a small program built with nvcc and run on the host - it makes
no CUDA call.  It covers the shapes and weight formats the GPU tests run (tiny, 3B, 7B; fp16, int8 per row, int8 per group) and a
few the GPU tests do not, and checks that unsupported shapes are refused with a reason instead of reaching the kernel."""
import os
import shutil
import subprocess

import pytest

from conftest import ROOT


def test_layout_of_the_streaming_decode_kernel(tmp_path):
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None)
    if not nvcc:
        pytest.skip("no nvcc")
    exe = tmp_path / "stream_layout_check"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++17", "--expt-relaxed-constexpr", "-I", os.path.join(ROOT, "include"), "-I",
           os.path.join(ROOT, "rwkv-rsv_b200", "csrc"), os.path.join(ROOT, "tests", "native", "stream_layout_check.cu"), "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0 and "all layout checks passed" in run.stdout, run.stdout[-3000:]
    assert run.stdout.count("\nok ") + run.stdout.startswith("ok ") >= 25
