"""The debug build of the library (libgemmzoo_dbg.so: the same sources compiled with
-DGZ_BOUNDS_CHECK).  In it every plain global store of the epilogue first checks its coordinates
against the output matrix; a store that fails is skipped and reported as GZ_ERR_DEBUG_CHECK with
the row and column it aimed at.  (TMA stores need no check: the hardware clips them to the tensor
map.)

CPU: the debug library exports every symbol the header declares.
GPU: a child process loads the debug library in place of the release one and runs the cases whose
epilogues store with plain instructions - ragged edges, the direct-store epilogue, D rows that TMA
cannot describe, the swapped (skinny) tiles, split-K, tail strips - through the same parity checker
as the release build: results correct, guard bands intact, and no store refused."""
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api, build as b

ROOT = Path(__file__).resolve().parent.parent


def test_debug_library_exports_the_same_symbols():
    import ctypes
    lib = b.build_lib(debug=True)
    assert lib == api.debug_lib_path() and lib.exists()
    L = ctypes.CDLL(str(lib))
    for name in gz.EXPORTED_SYMBOLS:
        getattr(L, name)


CHILD = textwrap.dedent('''
    import sys
    sys.path.insert(0, {root!r})
    import gemm_zoo_b200.api as api
    api.lib_path = api.debug_lib_path          # before the first lib() call: this process runs the debug build
    import gemm_zoo_b200 as gz
    from tests.helpers import Case, check
    F16, BF16, F32, S8, S32 = gz.DT_F16, gz.DT_BF16, gz.DT_F32, gz.DT_S8, gz.DT_S32
    cases = [
        # ragged edges, direct-store epilogue (plain stores from registers)
        Case(BF16, BF16, 300, 520, 256, b_col=True, flags=gz.FLAG_EPILOGUE_DIRECT, alpha=2, beta=-1),
        Case(BF16, F32, 333, 777, 192, b_col=True, flags=gz.FLAG_EPILOGUE_DIRECT, config=gz.CFG_2CTA_N256),
        Case(BF16, BF16, 700, 520, 256, b_col=True, flags=gz.FLAG_EPILOGUE_DIRECT, config=gz.CFG_2CTA_M512_N256, beta=1),
        Case(S8, S32, 130, 264, 400, b_col=True, flags=gz.FLAG_EPILOGUE_DIRECT, dist="full", alpha=3, beta=-2),
        # D whose rows TMA cannot describe: staged boxes leave by plain stores
        Case(BF16, BF16, 260, 520, 128, b_col=True, pad_d=4, pad_c=4, beta=1),
        Case(F32, F32, 200, 264, 192, pad_d=2, beta=0),
        # swapped (skinny) tiles, with and without split-K
        Case(BF16, BF16, 16, 1000, 512, b_col=True, beta=1),
        Case(BF16, BF16, 5, 520, 2048, b_col=True, flags=gz.FLAG_SPLIT_K),
        Case(S8, S32, 33, 2048, 4096, b_col=True, dist="full", flags=gz.FLAG_SPLIT_K, config=gz.CFG_SWAP_M64),
        Case(F16, F32, 128, 384, 256, b_col=True, config=gz.CFG_SWAP_M128),
        # tail strips of the last wave
        Case(BF16, BF16, 2304, 2048 + 256, 128, b_col=True, config=gz.CFG_2CTA_N256, flags=gz.FLAG_EPILOGUE_DIRECT),
    ]
    bad = 0
    for c in cases:
        r = check(c)
        if not r["ok"]:
            bad += 1
            print("MISMATCH", r)
    print("DEBUG BUILD", "FAILED" if bad else "OK", len(cases), api.lib_path().name)
    sys.exit(1 if bad else 0)
''')


@pytest.mark.gpu
def test_plain_store_epilogues_pass_the_bounds_checks(tmp_path):
    b.build_lib(debug=True)
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=str(ROOT)))
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert "DEBUG BUILD OK" in r.stdout and "libgemmzoo_dbg.so" in r.stdout
