"""The C++ host mirror (vibe_compiler_b200/host/B200TargetModelBackend.h): it must compile and link against libwb200
with the system compiler (CPU), and drive GEMM / elementwise requests with the reference's evidence rules (GPU)."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SOURCE = ROOT / "tests" / "host_cpp" / "host_mirror_check.cpp"


def build_program(tmp_path) -> Path:
    from vibe_compiler_b200 import build
    library = build.build()
    out = tmp_path / "host_mirror_check"
    cuda_lib = "/usr/local/cuda/lib64"
    command = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", str(SOURCE), "-o", str(out), f"-L{library.parent}", "-lwb200",
               f"-Wl,-rpath,{library.parent}", f"-Wl,-rpath-link,{cuda_lib}", f"-Wl,-rpath,{cuda_lib}"]
    subprocess.run(command, check=True, capture_output=True, text=True, timeout=300)
    return out


def test_cpp_host_mirror_compiles_and_reports_a_missing_device(tmp_path):
    import torch
    program = build_program(tmp_path)
    result = subprocess.run([str(program)], capture_output=True, text=True, timeout=120)
    if not torch.cuda.is_available():
        assert result.returncode == 3, result.stdout + result.stderr      # WB200_ERR_NO_DEVICE, no CPU fallback


@pytest.mark.gpu
def test_cpp_host_mirror_runs_requests(tmp_path):
    program = build_program(tmp_path)
    result = subprocess.run([str(program)], capture_output=True, text=True, timeout=120)
    assert result.returncode == 0 and "PASS" in result.stdout, result.stdout + result.stderr
