"""CPU checks of the boundary: the C-ABI library loads and exports every symbol that
include/*.h declares, and its argument checks answer without touching a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    for h in ("mixedgemm_c.h", "fp4.h", "fp6.h", "fp8.h", "mxdtype.h"):
        txt = open(os.path.join(ROOT, "include", h)).read()
        txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
        for m in re.finditer(r"^\s*(?:const\s+)?(?:int|size_t|char\s*\*|const char\s*\*)\s*\*?\s*(mg_\w+)\s*\(", txt, re.M):
            if "static inline" not in txt[max(0, m.start() - 20):m.start() + 20]:
                names.add(m.group(1))
    return names


@pytest.fixture(scope="module")
def lib():
    from mixedgemm_b200 import build, _capi
    build.build_lib()
    return _capi.load()


def test_exports_every_declared_symbol(lib):
    from mixedgemm_b200 import _capi
    declared = _declared_symbols()
    assert {"mg_reorder_quantize_x", "mg_reorder_quantize_w", "mg_matmul", "mg_matmul_f32", "mg_matmul_fp4",
            "mg_matmul_fp6", "mg_matmul_fp8", "mg_sf_bytes", "mg_matmul_workspace_bytes", "mg_strerror",
            "mg_device_status", "mg_version", "mg_last_cuda_error"} <= declared
    for name in declared:
        assert hasattr(lib, name), name
    assert declared <= set(_capi.PROTOTYPES), declared - set(_capi.PROTOTYPES)


def test_pure_host_entry_points(lib):
    assert lib.mg_version() >= 1
    assert lib.mg_sf_bytes(300, 448) == 3 * 4 * 512
    assert lib.mg_sf_bytes(128, 128) == 512
    assert lib.mg_sf_bytes(0, 128) == 0
    assert lib.mg_strerror(0) == b"ok"
    assert b"shape" in lib.mg_strerror(1)
    assert lib.mg_matmul_workspace_bytes(2048, 4096, 2560, 1408, 128) == 0
    # K=14336: 4928 and 448 are padded to 4992 and 512
    want = 0
    for n in (2048 * (4992 // 4 * 3), 4096 * (4992 // 2), 2048 * 512, 4096 * 256):
        want += (n + 1023) // 1024 * 1024
    assert lib.mg_matmul_workspace_bytes(2048, 4096, 8960, 4928, 448) == want


def test_argument_checks_need_no_gpu(lib):
    null = None
    # shape errors are detected before any CUDA call
    assert lib.mg_reorder_quantize_x(null, 4, 128, null, 64, 32, 16, *[null] * 6, null) == 1
    assert lib.mg_reorder_quantize_x(null, 4, 128, null, 80, 32, 16, *[null] * 6, null) == 1
    assert lib.mg_reorder_quantize_x(null, 0, 128, null, 64, 32, 32, *[null] * 6, null) == 0
    assert lib.mg_reorder_quantize_x(null, 4, 128, null, 64, 32, 32, *[null] * 6, null) == 2
    assert lib.mg_matmul(*[null] * 6, 128, 100, 256, 128, 128, null, null, 100, *[null] * 6, null, 0, null) == 1
    assert lib.mg_matmul(*[null] * 6, 128, 128, 256, 128, 128, null, null, 128, *[null] * 6, null, 0, null) == 2


def test_python_mirror_has_reference_entry_points():
    import inspect
    import mixedgemm_b200 as mg
    assert mg.test_function() == "Hello from test_function!"
    assert list(inspect.signature(mg.reorder_quantize_x).parameters)[:7] == [
        "X", "reorder_index", "KN", "KS", "KO", "seqlen", "outfeatures"]
    assert list(inspect.signature(mg.reorder_quantize_w).parameters)[:7] == [
        "W", "reorder_index", "KN", "KS", "KO", "seqlen", "outfeatures"]
    assert list(inspect.signature(mg.matmul).parameters)[:12] == [
        "AN", "BN", "AS", "BS", "AO", "BO", "SFAN", "SFBN", "SFAS", "SFBS", "SFAO", "SFBO"]


def _schedule(lib, tiles, cost, clusters):
    n = len(tiles)
    total = sum(tiles)
    use = ctypes.c_int(-1)
    off = (ctypes.c_uint16 * (clusters + 1))()
    tile = (ctypes.c_uint16 * max(total, 1))()
    st = lib.mg_pair_schedule(n, (ctypes.c_int * n)(*tiles), (ctypes.c_int * n)(*cost), clusters, ctypes.byref(use),
                              off, tile)
    assert st == 0
    return use.value, list(off), list(tile)[:total]


def test_tile_schedule_of_a_multi_problem_launch(lib):
    """The order the CTA-pair GEMM computes a list of problems in (mg_pair_schedule, host only): every
    tile exactly once, every SM pair's tiles in list order, the busiest pair within one tile of the
    mean, and round-robin where a table would change nothing."""
    # the Llama-3-8B step: gate, up (448 tiles of 22 + 1), down (128 of 78 + 1), q, k, v, o
    tiles, cost, clusters = [448, 448, 128, 128, 32, 32, 128], [23, 23, 79, 23, 23, 23, 23], 74
    use, off, tile = _schedule(lib, tiles, cost, clusters)
    assert use == 1 and off[0] == 0 and off[clusters] == sum(tiles)
    assert sorted(tile) == list(range(sum(tiles)))
    per_tile = [c for n, c in zip(tiles, cost) for _ in range(n)]
    loads = []
    for c in range(clusters):
        mine = tile[off[c]:off[c + 1]]
        assert mine == sorted(mine) and len(mine) >= 1
        loads.append(sum(per_tile[t] for t in mine))
    mean = sum(per_tile) / clusters
    assert max(loads) <= mean + max(cost)
    rr = [sum(per_tile[t] for t in range(c, sum(tiles), clusters)) for c in range(clusters)]
    assert max(loads) < max(rr)                      # better than dealing the list out round-robin
    # equal costs, one problem, or no more tiles than pairs: round-robin
    assert _schedule(lib, [448, 128], [23, 23], 74)[0] == 0
    assert _schedule(lib, [500], [23], 74)[0] == 0
    assert _schedule(lib, [40, 20], [23, 79], 74)[0] == 0
    assert _schedule(lib, [6000, 3000], [23, 79], 74)[0] == 0      # more tiles than the table holds
    # the same list again comes from the cache and is the same
    assert _schedule(lib, tiles, cost, clusters) == (use, off, tile)
    # five different lists push it out of the four-entry cache and back in
    for k in range(5):
        _schedule(lib, [100 + k, 50], [10, 30], 60)
    assert _schedule(lib, tiles, cost, clusters) == (use, off, tile)
    assert lib.mg_pair_schedule(0, None, None, 74, None, None, None) == 2
    n2 = (ctypes.c_int * 2)(10, 10)
    u = ctypes.c_int()
    buf = (ctypes.c_uint16 * 200)()
    assert lib.mg_pair_schedule(2, n2, n2, 97, ctypes.byref(u), buf, buf) == 1
    assert lib.mg_pair_schedule(9, n2, n2, 74, ctypes.byref(u), buf, buf) == 1
