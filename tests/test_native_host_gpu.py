"""The flat C ABI driven by a native host with no Python and no torch in the process (what a Rust caller does):
tests/cpp/capture_replay_host.cpp follows the reference's graph test
(crates/baracuda-kernels/tests/capture_replay_gather_gemv.rs): zeroed output, eager warm launch, capture, replays
without re-zeroing, inputs rewritten between replays; expectations are computed on the host inside the program."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def test_capture_replay_from_a_native_host(qlib, tmp_path):
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    assert shutil.which("g++") and (cuda / "include" / "cuda_runtime.h").exists()
    exe = tmp_path / "capture_replay_host"
    libdir = ROOT / "baracuda_b200"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), "-I", str(cuda / "include"),
                    str(ROOT / "tests" / "cpp" / "capture_replay_host.cpp"), "-L", str(libdir), "-lbaracuda_kernels_q",
                    "-L", str(cuda / "lib64"), "-lcudart", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{cuda / 'lib64'}",
                    "-o", str(exe)], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "capture_replay_host ok" in res.stdout, res.stdout + res.stderr
