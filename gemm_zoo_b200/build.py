"""In-tree build of the native pieces (no JIT cache, no pip install).

    python -m gemm_zoo_b200.build            # everything
    python -m gemm_zoo_b200.build lib        # libgemmzoo.so only

Targets
  lib        gemm_zoo_b200/libgemmzoo.so        the C ABI + sm_100a kernels (one object per
                                                 translation unit, compiled in parallel)
  debug      gemm_zoo_b200/libgemmzoo_dbg.so    the same with bounds-checked epilogue stores
  cublaslt   gemm_zoo_b200/libgz_cublaslt.so    cuBLASLt comparator (bench/tests only)
  bench      gemm_zoo_b200/nvidia/bench/build/* bench mains built against the C++ functor

The CPU oracle and the reference-kernel wrapper are test infrastructure and build from
oracle/build.py, not from here.  The same library can be built with the CMakeLists.txt at the
repository root.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_COMMON = ["-lineinfo", "-O3", "-std=c++17", "-Xfatbin", "-compress-all"]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC")
    return cand


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print("+", " ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(str(c) for c in cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def lib_sources():
    """Translation units of libgemmzoo.so: the host layer and one kernel table per pair of types."""
    return [CSRC / "gemm_api.cu"] + sorted((CSRC / "inst").glob("*.cu"))


def build_lib(force=False, verbose=False, ptxas_info=False, jobs=None, debug=False) -> Path:
    """debug=True: libgemmzoo_dbg.so, the same sources with -DGZ_BOUNDS_CHECK (every plain global
    store of the epilogue checks its coordinates first); used by tests/test_debug_bounds.py."""
    out = PKG / ("libgemmzoo_dbg.so" if debug else "libgemmzoo.so")
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((INCLUDE / "gemmzoo").glob("*.h"))
    objdir = CSRC / ("build_dbg" if debug else "build")
    objdir.mkdir(exist_ok=True)
    todo, objs = [], []
    for src in lib_sources():
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [nvcc_path(), *ARCH, *NVCC_COMMON, "-Xcompiler", "-fPIC,-fvisibility=hidden", "-c",
                   f"-I{INCLUDE}", f"-I{CSRC}", "-o", obj, src]
            if debug:
                cmd += ["-DGZ_BOUNDS_CHECK"]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            todo.append(cmd)
    if todo:
        with ThreadPoolExecutor(max_workers=jobs or min(len(todo), os.cpu_count() or 1)) as pool:
            logs = list(pool.map(lambda c: _run(c, verbose), todo))
        if ptxas_info:
            print("\n".join(logs))
    if todo or force or _newer(out, objs):
        # link beside the target and rename: a reader never sees a half-written library
        tmp = out.with_suffix(".so.tmp")
        _run([nvcc_path(), *ARCH, "-shared", "-Xcompiler", "-fPIC", "-o", tmp, *objs], verbose)
        os.replace(tmp, out)
    return out


def build_cublaslt(force=False, verbose=False) -> Path:
    out = PKG / "libgz_cublaslt.so"
    src = PKG / "cmp" / "cublaslt_cmp.cu"
    if force or _newer(out, [src, PKG / "nvidia" / "kernel_functors" / "cublaslt_gemm.cuh"]):
        cmd = [nvcc_path(), *ARCH, *NVCC_COMMON, "-Xcompiler", "-fPIC", "-shared", f"-I{INCLUDE}",
               f"-I{PKG / 'nvidia'}", "-o", out, src, "-lcublasLt"]
        _run(cmd, verbose)
    return out


def build_bench(force=False, verbose=False):
    outs = []
    bench_dir = PKG / "nvidia" / "bench"
    lib = build_lib(verbose=verbose)
    (bench_dir / "build").mkdir(exist_ok=True)
    for src in sorted(bench_dir.glob("*.cu")):
        out = bench_dir / "build" / src.stem
        deps = [src, lib] + list((PKG / "nvidia").rglob("*.cuh")) + list((PKG / "nvidia").rglob("*.hpp"))
        if force or _newer(out, deps):
            cmd = [nvcc_path(), *ARCH, *NVCC_COMMON, f"-I{INCLUDE}", f"-I{PKG / 'nvidia'}", "-o", out, src,
                   f"-L{PKG}", "-lgemmzoo", f"-Xlinker=-rpath={PKG}", "-lcublasLt"]
            _run(cmd, verbose)
        outs.append(out)
    return outs


def build_all(force=False, verbose=False):
    res = {"lib": build_lib(force, verbose), "lib_debug": build_lib(force, verbose, debug=True)}
    if (PKG / "cmp" / "cublaslt_cmp.cu").exists():
        res["cublaslt"] = build_cublaslt(force, verbose)
    if list((PKG / "nvidia" / "bench").glob("*.cu")):
        res["bench"] = build_bench(force, verbose)
    return res


if __name__ == "__main__":
    what = sys.argv[1:] or ["all"]
    force = "--force" in what
    what = [w for w in what if not w.startswith("--")] or ["all"]
    for w in what:
        if w == "all":
            print(build_all(force, True))
        elif w == "lib":
            print(build_lib(force, True, ptxas_info=True))
        elif w == "debug":
            print(build_lib(force, True, debug=True))
        elif w == "cublaslt":
            print(build_cublaslt(force, True))
        elif w == "bench":
            print(build_bench(force, True))
        else:
            raise SystemExit(f"unknown target {w}")
