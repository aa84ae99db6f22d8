"""CPU-only tests of the C ABI: the library loads and exports every symbol the
header declares, descriptor validation reaches every argument error without a
GPU, the tile order visits every tile exactly once, and the column partition
covers N exactly."""
import ctypes as C
import re
from pathlib import Path

import pytest

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "gemmzoo" / "gemm.h").read_text()
    declared = re.findall(r"GZ_API\s+[\w\s\*]+?\b(gz_\w+)\s*\(", header)
    assert len(declared) >= 12
    L = gz.lib()
    for name in declared:
        assert hasattr(L, name), name
    assert sorted(declared) == sorted(gz.EXPORTED_SYMBOLS)
    assert L.gz_version() >= 100


def test_library_exports_every_k_sharded_symbol():
    from gemm_zoo_b200 import ksharded
    header = (ROOT / "include" / "gemmzoo" / "ksharded.h").read_text()
    declared = re.findall(r"GZ_API\s+[\w\s\*]+?\b(gz_\w+)\s*\(", header)
    L = gz.lib()
    for name in declared:
        assert hasattr(L, name), name
    assert sorted(declared) == sorted(ksharded.EXPORTED_SYMBOLS)
    # argument errors that need no GPU
    d = ksharded.make_desc(gz.DT_BF16, gz.DT_BF16, 16, 1024, 512, world=2, rank=0)
    assert ksharded.workspace_bytes(d) >= 2 * 2 * 16 * 512 * 4
    bad = ksharded.make_desc(gz.DT_BF16, gz.DT_BF16, 16, 1000, 512, world=2, rank=0)  # 1000 % 64 != 0
    with pytest.raises(gz.GzError) as e:
        ksharded.workspace_bytes(bad)
    assert e.value.status == api.GZ_ERR_UNSUPPORTED
    for kw in (dict(world=9, rank=0), dict(world=2, rank=2), dict(world=0, rank=0)):
        with pytest.raises(gz.GzError) as e:
            ksharded.workspace_bytes(ksharded.make_desc(gz.DT_BF16, gz.DT_BF16, 16, 1024, 512, **kw))
        assert e.value.status == api.GZ_ERR_INVALID_ARG
    # K slices: aligned boundaries that cover K exactly
    bounds = [ksharded.k_slice(4096 + 64, 8, r) for r in range(8)]
    assert bounds[0][0] == 0 and bounds[-1][1] == 4096 + 64
    assert all(bounds[i][1] == bounds[i + 1][0] and bounds[i][1] % 64 == 0 for i in range(7))


def test_status_strings():
    for s in range(0, 9):
        assert len(gz.status_string(s)) > 1
    assert "unknown" in gz.status_string(99)


def _desc(**kw):
    base = dict(in_type=gz.DT_BF16, out_type=gz.DT_BF16, m=256, n=256, k=256)
    base.update(kw)
    return gz.GemmDesc.make(**base)


def test_validate_ok_and_defaults():
    st, info = gz.validate(_desc())
    assert st == api.GZ_OK
    assert (info.lda, info.ldb, info.ldc, info.ldd) == (256, 256, 256, 256)
    st, info = gz.validate(_desc(layout_a=gz.COL_MAJOR, layout_b=gz.COL_MAJOR, m=128, n=512, k=64))
    assert st == api.GZ_OK and (info.lda, info.ldb) == (128, 64)


@pytest.mark.parametrize("kw,expect", [
    (dict(m=0), api.GZ_ERR_INVALID_ARG),
    (dict(n=-5), api.GZ_ERR_INVALID_ARG),
    (dict(k=0), api.GZ_ERR_INVALID_ARG),
    (dict(lda=100), api.GZ_ERR_INVALID_ARG),            # lda < k for row-major A
    (dict(ldb=10), api.GZ_ERR_INVALID_ARG),
    (dict(ldc=255), api.GZ_ERR_INVALID_ARG),
    (dict(ldd=1), api.GZ_ERR_INVALID_ARG),
    (dict(layout_a=7), api.GZ_ERR_INVALID_ARG),
    (dict(in_type=9), api.GZ_ERR_INVALID_ARG),
    (dict(device=-1), api.GZ_ERR_INVALID_ARG),
    (dict(config=11), api.GZ_ERR_INVALID_ARG),
    (dict(flags=gz.FLAG_EPILOGUE_DIRECT | gz.FLAG_EPILOGUE_TMA), api.GZ_ERR_INVALID_ARG),
    (dict(flags=0x100), api.GZ_ERR_INVALID_ARG),
    (dict(in_type=gz.DT_BF16, out_type=gz.DT_F16), api.GZ_ERR_UNSUPPORTED),
    (dict(in_type=gz.DT_F32, out_type=gz.DT_BF16), api.GZ_ERR_UNSUPPORTED),
    (dict(in_type=gz.DT_S32, out_type=gz.DT_S32), api.GZ_ERR_UNSUPPORTED),
    (dict(m=2 ** 31), api.GZ_ERR_TOO_LARGE),
    (dict(k=2 ** 33), api.GZ_ERR_TOO_LARGE),
    # 100 bf16 = 200 bytes per row, not a multiple of 16: an explicit tensor-core config is refused
    (dict(k=100, lda=100, config=gz.CFG_1CTA_N128), api.GZ_ERR_MISALIGNED),
])
def test_validate_errors(kw, expect):
    st, _ = gz.validate(_desc(**kw))
    assert st == expect


def test_struct_size_is_checked():
    d = _desc()
    d.struct_size = 8
    assert gz.validate(d)[0] == api.GZ_ERR_INVALID_ARG
    assert gz.lib().gz_gemm_desc_validate(None, 0, None) == api.GZ_ERR_INVALID_ARG


def test_misaligned_leading_dimension_selects_simt_kernel():
    st, info = gz.validate(_desc(m=33, n=77, k=45))
    assert st == api.GZ_OK and info.config == gz.CFG_SIMT
    st, info = gz.validate(_desc(in_type=gz.DT_F32, out_type=gz.DT_F32, m=50, n=70, k=90, lda=93))
    assert st == api.GZ_OK and info.config == gz.CFG_SIMT


def test_auto_configuration_choices():
    st, info = gz.validate(_desc(m=8192, n=8192, k=8192, layout_b=gz.COL_MAJOR), 148)
    # large 16-bit problem: 512x256 tiles (two row blocks per CTA), 7 waves of 74 CTA pairs
    assert st == 0 and info.config == gz.CFG_2CTA_M512_N256 and info.grid == 148 and info.tiles == 512
    assert info.tile_m == 512 and info.tile_n == 256 and 200 * 1024 < info.smem_bytes <= 227 * 1024
    # aligned D rows leave through shared memory and TMA stores unless the caller asks otherwise
    assert info.epilogue_tma == 1
    st, info = gz.validate(_desc(m=8192, n=8192, k=8192, layout_b=gz.COL_MAJOR, flags=gz.FLAG_EPILOGUE_DIRECT), 148)
    assert st == 0 and info.epilogue_tma == 0
    st, info = gz.validate(_desc(m=256, n=250, k=64, layout_b=gz.COL_MAJOR), 148)  # 500-byte rows of D
    assert st == 0 and info.epilogue_tma == 0
    # 4-byte outputs cannot park both accumulators in registers: 256-row tiles
    st, info = gz.validate(_desc(in_type=gz.DT_S8, out_type=gz.DT_S32, m=8192, n=8192, k=8192, layout_b=gz.COL_MAJOR), 148)
    assert st == 0 and info.config == gz.CFG_2CTA_N256 and info.tiles == 1024
    # too few tiles for the larger tile to pay
    st, info = gz.validate(_desc(m=4096, n=4096, k=4096, layout_b=gz.COL_MAJOR), 148)
    assert st == 0 and info.config == gz.CFG_2CTA_N256
    st, info = gz.validate(_desc(m=16, n=14336, k=4096, layout_b=gz.COL_MAJOR), 148)
    assert st == 0 and info.ctas_per_tile == 1 and info.grid <= 148
    # s8 with N-contiguous B needs a 128-column chunk per CTA: the 2-CTA 128-wide tile is refused
    st, _ = gz.validate(_desc(in_type=gz.DT_S8, out_type=gz.DT_S32, config=gz.CFG_2CTA_N128))
    assert st == api.GZ_ERR_UNSUPPORTED
    st, info = gz.validate(_desc(in_type=gz.DT_S8, out_type=gz.DT_S32, m=4096, n=4096, k=4096))
    assert st == 0 and info.config in (gz.CFG_2CTA_N256, gz.CFG_1CTA_N256, gz.CFG_1CTA_N128)


@pytest.mark.parametrize("tm,tn,g", [(1, 1, 8), (1, 112, 16), (7, 3, 8), (32, 32, 8), (33, 17, 16),
                                     (128, 64, 8), (5, 1, 3), (64, 113, 16), (3, 200, 1)])
def test_tile_order_visits_every_tile_once(tm, tn, g):
    seen = set()
    for t in range(tm * tn):
        m, n = gz.tile_coords(tm, tn, g, t)
        assert 0 <= m < tm and 0 <= n < tn
        seen.add((m, n))
    assert len(seen) == tm * tn


def test_tile_order_groups_rows():
    # inside a group the row index runs fastest
    assert [gz.tile_coords(32, 32, 8, t) for t in range(10)] == [(t % 8, t // 8) for t in range(10)]
    assert gz.tile_coords(32, 32, 8, 8 * 32) == (8, 0)
    # short last group: 10 tile rows, groups of 8 -> last group has 2 rows
    assert [gz.tile_coords(10, 4, 8, 32 + t) for t in range(4)] == [(8, 0), (9, 0), (8, 1), (9, 1)]


@pytest.mark.parametrize("n,parts,align", [(8192, 8, 8), (14336, 8, 8), (14336, 3, 64), (1000, 7, 8),
                                           (5, 8, 8), (16384, 2, 256), (8192 * 8, 8, 256)])
def test_partition_columns_covers_n(n, parts, align):
    prev = 0
    sizes = []
    for p in range(parts):
        b, e = gz.partition_columns(n, parts, p, align)
        assert b == prev and e >= b
        if e < n:
            assert e % align == 0
        sizes.append(e - b)
        prev = e
    assert prev == n
    nonzero = [s for s in sizes if s]
    assert max(nonzero) - min(nonzero) <= 2 * align or len(nonzero) < parts


def test_partition_columns_rejects_bad_arguments():
    with pytest.raises(gz.GzError):
        gz.partition_columns(0, 2, 0)
    with pytest.raises(gz.GzError):
        gz.partition_columns(10, 2, 2)


def test_plan_creation_without_gpu_reports_no_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(gz.GzError) as ei:
        gz.Plan(_desc())
    assert ei.value.status == api.GZ_ERR_NO_DEVICE


def test_null_arguments():
    L = gz.lib()
    assert L.gz_gemm_plan_create(None, None) == api.GZ_ERR_INVALID_ARG
    assert L.gz_gemm_plan_destroy(None) == api.GZ_ERR_INVALID_ARG
    assert L.gz_gemm_run(None, None, None, None, None, None, None, None) == api.GZ_ERR_INVALID_ARG
    assert L.gz_fill(None, 0, 10, 0, 0, 0, 1.0, None) == api.GZ_ERR_INVALID_ARG
