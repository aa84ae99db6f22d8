"""TEST INFRASTRUCTURE: builds the checkers, never anything the product path loads.

    python -m oracle.build            # both
    python -m oracle.build oracle     # oracle/liboracle.so: the CPU restatement of the reference GEMM
    python -m oracle.build ref        # oracle/_ref/libref_kernels.so: the reference project's own
                                      # kernels, compiled from its sources where they lie (nothing
                                      # is copied); only where those sources are present

The reference tree is looked for in $GEMMZOO_REFERENCE, else in a directory named `reference`
beside this repository.  Without it a prebuilt oracle/_ref/libref_kernels.so is kept as it is.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ORACLE = Path(__file__).resolve().parent
ROOT = ORACLE.parent


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd):
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(str(c) for c in cmd) + "\n" + r.stdout + r.stderr)


def build_oracle(force=False) -> Path:
    out = ORACLE / "liboracle.so"
    src = ORACLE / "ref_gemm.cpp"
    if force or _newer(out, [src]):
        _run([os.environ.get("GXX", "/usr/bin/g++"), "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared",
              "-std=c++17", "-ffp-contract=off", "-o", out, src])
    return out


def reference_root() -> Path | None:
    env = os.environ.get("GEMMZOO_REFERENCE")
    p = Path(env) if env else ROOT.parent / "reference"
    return p if (p / "nvidia" / "kernels" / "generic_gemm.cuh").exists() else None


def build_ref(force=False) -> Path | None:
    ref = reference_root()
    out = ORACLE / "_ref" / "libref_kernels.so"
    if ref is None:
        return out if out.exists() else None
    src = ORACLE / "ref_kernels_wrap.cu"
    if force or _newer(out, [src]):
        nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        out.parent.mkdir(parents=True, exist_ok=True)
        _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", f"-I{ref / 'nvidia'}", "-o", out, src])
    return out


def build_all(force=False):
    return {"oracle": build_oracle(force), "ref": build_ref(force)}


if __name__ == "__main__":
    what = [w for w in sys.argv[1:] if not w.startswith("--")] or ["all"]
    force = "--force" in sys.argv
    for w in what:
        if w == "all":
            print(build_all(force))
        elif w == "oracle":
            print(build_oracle(force))
        elif w == "ref":
            print(build_ref(force))
        else:
            raise SystemExit(f"unknown target {w}")
