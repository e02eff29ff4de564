"""The C ABI from a C host: tests/c_host/list_host.c (gcc, the CUDA runtime, libbas - no Python, no torch in the
program) builds a list with two selection entries and two contractions, runs it and checks masks and outputs for
equality against its own plain-C restatement of the reference's rule.  The CPU test compiles and links it (the
header is valid C, every symbol it uses is exported); the GPU test runs it."""

import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "towards-batched-activation-sparsity_b200"
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))


def _build(tmp_path) -> Path:
    gcc = shutil.which("gcc")
    if gcc is None or not (CUDA / "include" / "cuda_runtime.h").exists():
        pytest.skip("needs gcc and the CUDA toolkit's headers")
    from bas import abi  # noqa: F401  (builds libbas.so if it is missing)
    exe = tmp_path / "list_host"
    subprocess.check_call([gcc, "-std=c11", "-O1", "-Wall", "-I", str(ROOT / "include"), "-I", str(CUDA / "include"),
                           str(ROOT / "tests" / "c_host" / "list_host.c"), "-o", str(exe),
                           "-L", str(PKG), "-lbas", "-L", str(CUDA / "lib64"), "-lcudart", "-lm",
                           f"-Wl,-rpath,{PKG}", f"-Wl,-rpath,{CUDA / 'lib64'}"])
    return exe


def test_c_host_compiles_and_links(tmp_path):
    assert _build(tmp_path).exists()


@pytest.mark.gpu
def test_c_host_runs(tmp_path):
    exe = _build(tmp_path)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "C_HOST_LIST OK" in res.stdout
