"""The CMake build a C++ consumer uses (CMakeLists.txt at the repository root, the counterpart
of the reference's one-executable-per-bench-file build, its CMakeLists.txt:14,24-41):
it configures for sm_100a only, declares the library with every kernel translation unit and one
executable per bench main, and builds a bench main against an already built libgemmzoo.so."""
import shutil
import subprocess
from pathlib import Path

import pytest

from gemm_zoo_b200 import build as b

ROOT = Path(__file__).resolve().parent.parent


def _cmake():
    exe = shutil.which("cmake")
    if exe is None:
        pytest.skip("cmake not installed")
    return exe


def _configure(build_dir, *extra):
    cmd = [_cmake(), "-S", str(ROOT), "-B", str(build_dir), "-G", "Ninja", f"-DCMAKE_CUDA_COMPILER={b.nvcc_path()}", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def _targets(build_dir):
    r = subprocess.run([shutil.which("ninja"), "-C", str(build_dir), "-t", "targets", "all"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return r.stdout


def test_configure_declares_library_and_every_bench_main(tmp_path):
    _configure(tmp_path / "full")
    targets = _targets(tmp_path / "full")
    assert "libgemmzoo.so" in targets
    for unit in b.lib_sources():  # the host layer and every kernel translation unit
        assert f"{unit.name}.o" in targets, unit.name
    for src in (b.PKG / "nvidia" / "bench").glob("*.cu"):
        assert f"{src.stem}:" in targets, src.stem
    cache = (tmp_path / "full" / "CMakeCache.txt").read_text()
    assert "CMAKE_CUDA_ARCHITECTURES:STRING=100a" in cache


def test_one_bench_main_builds_against_the_built_library(tmp_path):
    lib = b.build_lib()
    _configure(tmp_path / "pre", f"-DGEMMZOO_PREBUILT_LIB={lib}")
    r = subprocess.run([_cmake(), "--build", str(tmp_path / "pre"), "--target", "bench_sm100_bf16"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert (tmp_path / "pre" / "bench_sm100_bf16").exists()
