"""In-tree build of the native pieces (no JIT cache, no pip install).

    python -m gemm_zoo_b200.build            # everything
    python -m gemm_zoo_b200.build lib        # libgemmzoo.so only

Targets
  lib        gemm_zoo_b200/libgemmzoo.so        the C ABI + sm_100a kernels
  cublaslt   gemm_zoo_b200/libgz_cublaslt.so    cuBLASLt comparator (bench/tests only)
  oracle     oracle/liboracle.so                CPU restatement of the reference GEMM (checker)
  ref        oracle/_ref/libref_kernels.so      the reference project's own kernels, compiled
                                                 from its sources where they lie (only when
                                                 those sources are present on this machine)
  bench      gemm_zoo_b200/nvidia/bench/build/* bench mains built against the C++ functor
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
ORACLE = ROOT / "oracle"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_COMMON = ["-lineinfo", "-O3", "-std=c++17"]


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


def build_lib(force=False, verbose=False, ptxas_info=False) -> Path:
    out = PKG / "libgemmzoo.so"
    srcs = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(
        (INCLUDE / "gemmzoo").glob("*.h"))
    if force or _newer(out, srcs):
        cmd = [nvcc_path(), *ARCH, *NVCC_COMMON, "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
               f"-I{INCLUDE}", f"-I{CSRC}", "-o", out, CSRC / "gemm_api.cu"]
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        log = _run(cmd, verbose)
        if ptxas_info:
            print(log)
    return out


def build_cublaslt(force=False, verbose=False) -> Path:
    out = PKG / "libgz_cublaslt.so"
    src = PKG / "cmp" / "cublaslt_cmp.cu"
    if force or _newer(out, [src, PKG / "nvidia" / "kernel_functors" / "cublaslt_gemm.cuh"]):
        cmd = [nvcc_path(), *ARCH, *NVCC_COMMON, "-Xcompiler", "-fPIC", "-shared", f"-I{INCLUDE}",
               f"-I{PKG / 'nvidia'}", "-o", out, src, "-lcublasLt"]
        _run(cmd, verbose)
    return out


def build_oracle(force=False, verbose=False) -> Path:
    out = ORACLE / "liboracle.so"
    src = ORACLE / "ref_gemm.cpp"
    if force or _newer(out, [src]):
        cmd = [os.environ.get("GXX", "/usr/bin/g++"), "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-std=c++17",
               "-ffp-contract=off", "-o", out, src]
        _run(cmd, verbose)
    return out


def reference_root() -> Path | None:
    p = Path(os.environ.get("GEMMZOO_REFERENCE", "/root/reference"))
    return p if (p / "nvidia" / "kernels" / "generic_gemm.cuh").exists() else None


def build_ref(force=False, verbose=False) -> Path | None:
    """Compile the reference project's kernels from its own sources (never copied)."""
    ref = reference_root()
    out = ORACLE / "_ref" / "libref_kernels.so"
    if ref is None:
        return out if out.exists() else None
    src = ORACLE / "ref_kernels_wrap.cu"
    if force or _newer(out, [src]):
        out.parent.mkdir(parents=True, exist_ok=True)
        cmd = [nvcc_path(), *ARCH, *NVCC_COMMON, "-Xcompiler", "-fPIC", "-shared",
               f"-I{ref / 'nvidia'}", "-o", out, src]
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
    res = {"lib": build_lib(force, verbose)}
    if (PKG / "cmp" / "cublaslt_cmp.cu").exists():
        res["cublaslt"] = build_cublaslt(force, verbose)
    if (ORACLE / "ref_gemm.cpp").exists():
        res["oracle"] = build_oracle(force, verbose)
    if (ORACLE / "ref_kernels_wrap.cu").exists():
        res["ref"] = build_ref(force, verbose)
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
        elif w == "cublaslt":
            print(build_cublaslt(force, True))
        elif w == "oracle":
            print(build_oracle(force, True))
        elif w == "ref":
            print(build_ref(force, True))
        elif w == "bench":
            print(build_bench(force, True))
        else:
            raise SystemExit(f"unknown target {w}")
