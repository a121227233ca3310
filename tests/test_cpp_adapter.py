"""Builds the C++20 adapter test against the C-ABI library; runs it on a GPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SOURCE = ROOT / "tests" / "cpp" / "adapter_test.cpp"
WIRE_SOURCE = ROOT / "tests" / "cpp" / "wire_test.cpp"


def build(pkg, target: Path, source: Path = SOURCE) -> None:
    pkg.library()  # the shared library must exist
    library_dir = pkg.LIBRARY_PATH.parent
    compiler = shutil.which("g++")
    if compiler is None:
        pytest.skip("no g++ on this machine")
    cuda_lib = Path("/usr/local/cuda/lib64")
    if not (cuda_lib / "libcudart.so").exists():
        pytest.skip("no CUDA runtime library to link the test's device allocations against")
    subprocess.run([compiler, "-std=c++20", "-O1", "-Wall", "-Wextra", str(source), "-o", str(target), f"-L{library_dir}",
                    "-lmoe_b200_sampler", f"-L{cuda_lib}", "-lcudart", f"-Wl,-rpath,{library_dir}", f"-Wl,-rpath,{cuda_lib}"], check=True)


def test_adapter_compiles_and_links(pkg, tmp_path):
    build(pkg, tmp_path / "adapter_test")


@pytest.mark.gpu
def test_adapter_runs_like_the_reference_tests(pkg, torch_cuda, tmp_path):
    target = tmp_path / "adapter_test"
    build(pkg, target)
    result = subprocess.run([str(target)], capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "all adapter tests passed" in result.stdout


def test_wire_router_compiles_and_links(pkg, tmp_path):
    build(pkg, tmp_path / "wire_test", WIRE_SOURCE)


@pytest.mark.gpu
def test_wire_router_batches_concurrent_generations(pkg, torch_cuda, tmp_path):
    """JSONL requests of several Sessions (the reference worker's `generate` fields) sampled in one call per step."""
    target = tmp_path / "wire_test"
    build(pkg, target, WIRE_SOURCE)
    result = subprocess.run([str(target)], capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "all wire tests passed" in result.stdout
