"""Static work decomposition of the native path (host code only; needs the built library, no GPU):
tile lists must cover every gradient matrix exactly once, orthonormalisation chunks every factor
row exactly once, and the tensor-core tile extent must respect its alignment rules."""
import numpy as np
import pytest

from powersgd_b200.plan import CompressionPlan

native = pytest.importorskip("powersgd_b200.ops.native")


def _lib():
    try:
        return native.lib()
    except Exception as exc:  # library not built on this machine
        pytest.skip(f"native library unavailable: {exc}")


SHAPES = [(64, 27), (128, 576), (512, 4608), (1000, 650), (10, 512), (4096, 4096), (333, 129)]


@pytest.mark.parametrize("rank", [1, 2, 4, 16])
@pytest.mark.parametrize("tc", [False, True])
def test_tiles_cover_every_matrix_exactly_once(rank, tc):
    from powersgd_b200.cuda_path import TilePlan

    plan = CompressionPlan.build(SHAPES, rank=rank)
    tiles = TilePlan(plan, _lib())
    tiles.fin_rows = 96
    nmat = len(tiles.mats)
    tc_flags = [tc and plan.groups[gi].m % 4 == 0 for gi, _p, _i in tiles.mats]
    widths = [4 if plan.groups[gi].m % 4 == 0 else 2 if plan.groups[gi].m % 2 == 0 else 1 for gi, _p, _i in tiles.mats]
    arrays = tiles.build(widths, tc_flags)
    for name in ("nt", "nn", "fin"):
        cover = [np.zeros((plan.groups[gi].n, plan.groups[gi].m), dtype=np.int32) for gi, _p, _i in tiles.mats]
        for key in ("f", "tc"):
            for t in arrays[name][key]:
                assert int(t["vec"]) == widths[int(t["mat"])]
                cover[t["mat"]][t["row0"] : t["row0"] + t["rows"], t["col0"] : t["col0"] + t["cols"]] += 1
        for c in cover:
            assert (c == 1).all(), name
    # split tiles of one output block share a ticket and occupy consecutive partial-sum slots
    for name in ("nt", "nn"):
        for key in ("f", "tc"):
            by_ticket = {}
            for t in arrays[name][key]:
                by_ticket.setdefault(int(t["ticket"]), []).append(t)
            for group in by_ticket.values():
                assert sorted(int(t["split"]) for t in group) == list(range(len(group)))
                assert all(int(t["nsplit"]) == len(group) for t in group)
                assert len({int(t["slot0"]) for t in group}) == 1


@pytest.mark.parametrize("rank", [1, 3, 16])
def test_orth_chunks_cover_every_factor_row_once(rank):
    from powersgd_b200.cuda_path import TilePlan

    shapes = SHAPES + [(64, 27)] * 3  # a shape group of four: one joint unit at rank 1
    plan = CompressionPlan.build(shapes, rank=rank)
    tiles = TilePlan(plan, _lib())
    for side in ("p", "q"):
        for chunk_rows in (64, 1000):
            units, chunks = tiles.orth_units(side, chunk_rows)
            assert sum(int(u["nchunks"]) for u in units) == len(chunks)
            for ui, u in enumerate(units):
                mine = chunks[u["chunk0"] : u["chunk0"] + u["nchunks"]]
                assert (mine["unit"] == ui).all()
                seen = np.zeros(int(u["sub_len"]) * int(u["nsub"]), dtype=np.int32)
                for c in mine:
                    assert 0 < c["rows"] <= chunk_rows
                    lo, hi = int(c["row0"]), int(c["row0"]) + int(c["rows"])
                    assert lo // u["sub_len"] == (hi - 1) // u["sub_len"] == c["sub"]  # inside one sub-matrix
                    seen[lo:hi] += 1
                assert (seen == 1).all()
                if rank > 1 and u["r"] > 1:
                    assert u["nsub"] == 1


def test_tensor_core_tile_extent_is_aligned_and_fills_one_wave_when_it_can(monkeypatch):
    from powersgd_b200.cuda_path import TilePlan, _split_even

    monkeypatch.delenv("PSGD_B200_TC_K", raising=False)
    plan = CompressionPlan.build([(4096, 4096)] * 4, rank=4)
    tiles = TilePlan(plan, _lib())
    groups = [plan.groups[gi] for gi, _p, _i in tiles.mats]
    for transposed in (True, False):
        k = tiles._pick_tc_k(groups, transposed)
        assert k % 32 == 0 and 256 <= k <= 8192
        blocks = _split_even(4096, k, 32)
        assert all(start % 32 == 0 for start, _ in blocks)  # TMA coordinates stay 16-byte aligned
        ntiles = 4 * 32 * len(blocks)
        assert ntiles <= 148 * TilePlan.TC_CTAS_PER_SM  # one round of resident CTAs
    monkeypatch.setenv("PSGD_B200_TC_K", "512")
    assert tiles._pick_tc_k(groups, True) == 512


def test_bulk_allreduce_layout_helpers():
    lib = _lib()
    chunk = int(lib.psgd_bulk_chunk_floats())
    assert chunk % 4 == 0
    for world in (2, 4, 8):
        n_pad = 3 * world * chunk
        need = int(lib.psgd_bulk_arena_bytes(n_pad, world))
        assert need == 8 * n_pad + 2 * world * 3 * 4  # data + landing area + two flag tables
    for k, same in ((8, 1), (8, 0), (32, 0), (64, 1)):
        rows = int(lib.psgd_finalize_strip_rows(k, same))
        assert rows % 32 == 0 and 32 <= rows <= 256


def test_multicast_runtime_degrades_without_a_driver():
    """csrc/mcast.cpp looks its driver entry points up at run time: on a machine without a GPU the
    library still loads, reports no multicast support and refuses politely (error code + message)."""
    import ctypes

    import torch

    from powersgd_b200.parallel.nvls import _McBuffer

    lib = _lib()
    assert ctypes.sizeof(_McBuffer) == int(lib.psgd_mc_buffer_bytes())
    if torch.cuda.is_available():
        pytest.skip("this check is for driver-less machines")
    assert int(lib.psgd_mc_supported()) == 0
    out = ctypes.c_ulonglong(0)
    assert int(lib.psgd_mc_round_up(2, ctypes.c_ulonglong(1 << 20), ctypes.byref(out))) != 0
    assert lib.psgd_last_error()
    state = _McBuffer()
    assert int(lib.psgd_mc_release(ctypes.byref(state))) == 0   # nothing set up: nothing to undo



def test_in_switch_path_policy(monkeypatch):
    """`auto` takes the in-switch all-reduce from four workers on unless NCCL_NVLS_ENABLE=0 (how the
    failure tests run); `nvls` forces it, `bulk` never takes it."""
    from powersgd_b200.cuda_path import NativeFlatAllReduce

    wants = NativeFlatAllReduce._wants_nvls
    monkeypatch.delenv("NCCL_NVLS_ENABLE", raising=False)
    assert not wants("auto", 2) and not wants("auto", 3) and wants("auto", 4) and wants("auto", 8)
    assert wants("nvls", 2) and not wants("bulk", 8)
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    assert not wants("auto", 8) and wants("nvls", 8)
