"""The host layer of the library (descriptor validation, configuration choice, plan geometry,
partition and tile-order helpers, argument checks of every entry point) built with
AddressSanitizer and UndefinedBehaviorSanitizer and driven by tests/host_fuzz.c with tens of
thousands of seeded descriptors.  The kernels' objects are linked as they are; only
csrc/gemm_api.cu is recompiled with the sanitizers.  No GPU is needed."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

from gemm_zoo_b200 import build as b

ROOT = Path(__file__).resolve().parent.parent


def test_host_layer_is_clean_under_asan_and_ubsan(tmp_path):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("gcc not installed")
    b.build_lib()  # makes sure the kernel objects exist
    kernel_objs = sorted((b.CSRC / "build").glob("k_*.o"))
    assert kernel_objs
    obj = tmp_path / "gemm_api_san.o"
    san = "-fsanitize=address,-fsanitize=undefined,-fno-omit-frame-pointer"
    r = subprocess.run([b.nvcc_path(), *b.ARCH, "-O1", "-g", "-std=c++17", "-Xcompiler", f"-fPIC,{san}", "-c",
                        f"-I{b.INCLUDE}", f"-I{b.CSRC}", "-o", str(obj), str(b.CSRC / "gemm_api.cu")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    lib = tmp_path / "libgemmzoo_san.so"
    r = subprocess.run([b.nvcc_path(), *b.ARCH, "-shared", "-Xcompiler", "-fPIC", "-Xlinker", "-lasan", "-Xlinker", "-lubsan",
                        "-o", str(lib), str(obj), *map(str, kernel_objs)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    exe = tmp_path / "host_fuzz"
    r = subprocess.run([gcc, "-O1", "-g", "-fsanitize=address,undefined", f"-I{b.INCLUDE}", "-o", str(exe),
                        str(ROOT / "tests" / "host_fuzz.c"), f"-L{tmp_path}", "-lgemmzoo_san", f"-Wl,-rpath,{tmp_path}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="protect_shadow_gap=0:detect_leaks=0:abort_on_error=0",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([str(exe)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    assert "HOST FUZZ OK" in r.stdout
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr, r.stderr[-3000:]
