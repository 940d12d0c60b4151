"""The C-ABI library: it loads, exports every symbol the public header declares,
rejects bad arguments before touching the GPU, and the planner covers the
reference's domain and beyond.  Runs without a GPU (no compute calls)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from accelerated_scan import _native


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ascan_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ascan_[a-z_]+)\s*\(", text)))


def test_header_symbols_exported():
    names = declared_symbols()
    assert set(names) >= set(_native.EXPORTS)
    for name in names:
        assert hasattr(_native.lib, name), name


def test_version_and_strerror():
    assert _native.lib.ascan_version() >= 100
    assert _native.strerror(0) == "success"
    assert "invalid" in _native.strerror(1)
    assert "unknown" in _native.strerror(12345)


def test_bad_arguments_rejected_without_gpu():
    lib = _native.lib
    null = ctypes.c_void_p(None)
    fake = ctypes.c_void_p(256)   # never dereferenced: validation fails first
    assert lib.ascan_forward(fake, fake, fake, -1, 8, 0, 0, null, null, 0, null) == 1
    assert lib.ascan_forward(fake, fake, fake, 4, 0, 0, 0, null, null, 0, null) == 1
    assert lib.ascan_forward(fake, fake, fake, 4, 8, 99, 0, null, null, 0, null) == 1
    assert lib.ascan_forward(null, fake, fake, 4, 8, 0, 0, null, null, 0, null) == 1
    assert lib.ascan_forward(fake, fake, fake, 0, 8, 0, 0, null, null, 0, null) == 0   # empty: nothing to do
    assert lib.ascan_backward(fake, fake, fake, fake, null, 4, 8, 0, null, null, null, null, 0, null) == 1
    assert lib.ascan_backward(fake, fake, fake, fake, fake, 4, 8, 0, fake, null, null, null, 0, null) == 1
    assert lib.ascan_reduce_forward(fake, fake, null, 4, 8, 0, null, 0, null) == 1
    assert lib.ascan_reduce_backward(fake, null, null, fake, 4, 8, 0, null, 0, null) == 1
    assert lib.ascan_check(null, null) == 1


@pytest.mark.parametrize("T", [1, 7, 32, 64, 128, 256, 512, 1024, 4096, 65536, 16323, 8000, 33753, 127323, 1 << 20])
@pytest.mark.parametrize("dtype", [_native.F32, _native.BF16, _native.F16, _native.C64])
@pytest.mark.parametrize("kind", [0, 1, 2, 3])
def test_planner_invariants(T, dtype, kind):
    esize = {0: 4, 1: 2, 2: 2, 3: 8}[dtype]
    for rows in (1, 16, 512, 2500, 5000, 12288):
        pl = _native.plan(rows, T, dtype, kind, aligned=True, sm_count=148)
        assert pl["grid"] >= 1 and pl["warps_per_cta"] >= 1
        assert pl["warps_per_cta"] * 32 <= (448 if kind == 1 else 512)
        assert pl["smem_bytes"] <= 227 * 1024
        assert pl["tile_elems"] == 32 * pl["chunks_per_lane"] * (16 // esize)
        assert pl["items"] == pl["row_groups"] * pl["segs_per_row"]
        assert pl["row_groups"] * pl["rows_per_item"] >= rows
        assert pl["segs_per_row"] == pl["coarse_segs"] + pl["fine_segs"]
        assert pl["coarse_segs"] * pl["seg_elems"] + pl["fine_segs"] * pl["fine_elems"] >= T
        if pl["dynamic"] == 0:
            # unsplit rows at a few items per warp (at most eight) are dealt round-robin: no tickets, no scratch
            assert pl["segs_per_row"] == 1 and pl["kernel"] == 0 and pl["workspace_bytes"] == 0
            assert pl["items"] <= 8 * pl["grid"] * pl["warps_per_cta"]
        elif pl["kernel"] == 1:
            # look-back plan: fewer rows than 3/4 of the SMs; a CTA is a team of workers plus a bookkeeper, a
            # segment is one part of `stages` tiles per worker; 32-byte records per segment, block of 32
            # segments and super-block of 32 blocks
            assert rows < (222 if kind == 0 else 111) and kind in (0, 1)
            workers = pl["warps_per_cta"] - 1
            assert 1 <= workers <= 15 and pl["grid"] == min(148, pl["items"])
            segs = pl["segs_per_row"]
            blocks = (segs + 31) // 32
            assert pl["workspace_bytes"] == 256 + 32 * rows * (segs + blocks + (blocks + 31) // 32)
            assert pl["seg_elems"] == pl["fine_elems"] == workers * pl["stages"] * pl["tile_elems"]
            assert (segs - 1) * pl["seg_elems"] < T
            assert pl["stages"] == 2 and pl["chunks_per_lane"] == 3
            chained = _native.plan(rows, T, dtype, kind, sm_count=148, lookback=False, team=False)
            assert chained["kernel"] == 0 and chained["workspace_bytes"] in (0, 256, 256 + 32 * rows)
        else:
            assert pl["workspace_bytes"] == (256 + 32 * rows if pl["segs_per_row"] > 1 else 256)
        if pl["kernel"] == 2:
            # team plan: fewer rows than warps, whole teams per CTA, rows never grouped
            assert rows < 4 * 148 * 12 and (kind in (0, 1) or dtype != _native.C64) and pl["loader"] == 0
            # 16 warps per CTA for the forward kinds, 12 for the backward kinds
            wide = pl["warps_per_cta"] == 16
            assert kind in (0, 2) or not wide
            assert pl["team_size"] in ((2, 4, 8, 16) if wide else (2, 3, 4, 6, 12))
            assert pl["warps_per_cta"] % pl["team_size"] == 0
            assert pl["rows_per_item"] == 1 and pl["grid"] == 148
            per_cta = pl["warps_per_cta"]
            assert (148 * per_cta) // pl["team_size"] <= max(rows, 148) or pl["team_size"] == per_cta
        else:
            assert pl["team_size"] == 1
        if pl["row_grid"]:
            # short rows on the tile grid: unseeded scan kinds, two chunks per lane, rows divide the tile, whole
            # tiles per item, never split, bulk loader
            assert kind in (0, 1) and pl["chunks_per_lane"] == 2 and pl["loader"] == 0 and pl["kernel"] == 0
            assert pl["tile_elems"] % T == 0 and T % (pl["tile_elems"] // 32) == 0
            assert (pl["rows_per_item"] * T) % pl["tile_elems"] == 0 and pl["segs_per_row"] == 1
            assert _native.plan(rows, T, dtype, kind, sm_count=148, seeded=True)["row_grid"] == 0
        if pl["segs_per_row"] > 1:
            # split rows: one row per item, segments are whole tiles
            assert pl["rows_per_item"] == 1 and pl["seg_elems"] % pl["tile_elems"] == 0
            assert pl["fine_elems"] % pl["tile_elems"] == 0
            assert pl["segs_per_row"] < 32768 or pl["kernel"] == 1      # chained carries tag segments in 15 bits
            # only the last piece of a row (in memory order) may be short, none is empty
            if kind in (1, 3):
                assert pl["fine_segs"] * pl["fine_elems"] + (pl["coarse_segs"] - 1) * pl["seg_elems"] < T or pl["coarse_segs"] == 0
                assert pl["coarse_segs"] > 0 or (pl["fine_segs"] - 1) * pl["fine_elems"] < T
            else:
                assert pl["coarse_segs"] * pl["seg_elems"] + (pl["fine_segs"] - 1) * pl["fine_elems"] < T
                assert pl["coarse_segs"] * pl["seg_elems"] <= T
        if pl["loader"] == 0:
            # bulk copies: every item starts on a 16-byte boundary and the matrix ends on one
            assert (pl["rows_per_item"] * T * esize) % 16 == 0
            assert (pl["seg_elems"] * esize) % 16 == 0 or pl["segs_per_row"] == 1
            assert (rows * T * esize) % 16 == 0
        # no more warps than items, spread over the SMs
        assert pl["grid"] * pl["warps_per_cta"] <= max(pl["items"], 1) + pl["warps_per_cta"] * 148
        unaligned = _native.plan(rows, T, dtype, kind, aligned=False, sm_count=148)
        assert unaligned["loader"] == 1
        static = _native.plan(rows, T, dtype, kind, workspace=False, sm_count=148)
        assert static["dynamic"] == 0 and static["segs_per_row"] == 1 and static["workspace_bytes"] == 0


@pytest.mark.parametrize("dtype", [0, 1, 3])
@pytest.mark.parametrize("kind", [0, 1])
def test_lookback_plan_decomposition(dtype, kind):
    """The look-back plan over row counts and lengths: rows are cut into segments of equal size, one part of `stages`
    tiles per worker warp, no more workers than a row has parts and than shared memory holds, one CTA per segment
    in flight at most, and the scratch that the plan asks for matches its records."""
    esize = {0: 4, 1: 2, 3: 8}[dtype]
    tile = 32 * 3 * (16 // esize)
    # bytes per worker: its tiles of two resident segments (inputs, and 128 bytes of halo per stage in the backward),
    # a staging tile (forward), mbarriers, prefix maps of two compute-type values per stage and lane
    nin = 3 if kind == 1 else 2
    stage = nin * 32 * 3 * 16 + (128 if kind == 1 else 0)
    prefix = 16 if dtype == 3 else 8
    per_worker = 2 * 2 * stage + (0 if kind == 1 else 32 * 3 * 16) + 128 + 2 * 2 * 32 * prefix
    max_workers = min(15, (227 * 1024 - 3072) // per_worker)
    for rows in (1, 2, 7, 64, 110):
        for tiles in (4, 5, 29, 30, 31, 60, 61, 342, 1366, 2731, 43691):
            for ragged in (0, 16 // esize):
                T = tiles * tile - ragged
                pl = _native.plan(rows, T, dtype, kind, aligned=True, sm_count=148)
                assert pl["kernel"] == 1, (rows, T, pl)
                workers = pl["warps_per_cta"] - 1
                segs = pl["segs_per_row"]
                parts = (tiles + 1) // 2
                assert 1 <= workers <= max_workers
                assert segs == -(-parts // max_workers) and workers == -(-parts // segs)
                assert pl["seg_elems"] == workers * 2 * tile and (segs - 1) * pl["seg_elems"] < T <= segs * pl["seg_elems"]
                assert pl["smem_bytes"] == workers * per_worker + 3072 <= 227 * 1024
                assert pl["items"] == rows * segs and pl["grid"] == min(148, pl["items"])
                blocks = (segs + 31) // 32
                assert pl["workspace_bytes"] == 256 + 32 * rows * (segs + blocks + (blocks + 31) // 32)


def test_planner_rejects_bad_input():
    pl = _native.Plan()
    assert _native.lib.ascan_plan_describe(4, 0, 0, 0, 1, 148, ctypes.byref(pl)) == 1
    assert _native.lib.ascan_plan_describe(4, 8, 7, 0, 1, 148, ctypes.byref(pl)) == 1
    assert _native.lib.ascan_plan_describe(4, 8, 0, 9, 1, 148, ctypes.byref(pl)) == 1
    assert _native.lib.ascan_plan_describe(4, 8, 0, 0, 1, 148, None) == 1


def test_python_api_mirrors_reference_names():
    import accelerated_scan.warp as warp
    import accelerated_scan.complex as cplx

    for name in ("scan", "Scan", "scan_forward", "warpscan_forward", "warpscan_backward"):
        assert hasattr(warp, name)
    for name in ("scan", "Scan", "forward_scan", "backward_scan"):
        assert hasattr(cplx, name)


def test_cpu_tensors_fail_loudly():
    import torch
    import accelerated_scan.warp as warp
    import accelerated_scan.complex as cplx

    g = torch.rand(1, 2, 32)
    with pytest.raises(RuntimeError):
        warp.scan(g, g.clone())
    with pytest.raises(TypeError):
        cplx.scan(g, g.clone())
    with pytest.raises(AssertionError):
        warp.Scan.apply(g, torch.rand(1, 2, 16))


def test_extensions_fail_loudly_on_cpu_tensors():
    """The modules beyond the reference's surface have no CPU path either."""
    import torch
    from accelerated_scan import gated, stateful

    g = torch.rand(1, 2, 64)
    with pytest.raises(RuntimeError):
        gated.scan(g, g.clone())
    with pytest.raises(RuntimeError):
        stateful.scan(g, g.clone(), torch.zeros(1, 2))
    with pytest.raises(RuntimeError):
        stateful.final_state(g, g.clone())
    c = torch.complex(g, g)
    with pytest.raises(RuntimeError):
        gated.scan(c, c)
