"""The allocation-free factor product, called through its exported C symbol.

Some users of the native library cannot allocate device memory when they need a product
(allocator frozen or being recorded, fixed memory budgets inside communication hooks,
embedders without PyTorch). `psgd_matmul_tn_noalloc` serves them from a scratch array built
into the library. This test loads the symbol with ctypes, runs it twice in a row (the second
call sees the first call's leftovers in the shared scratch) and compares each result with
the regular grouped entry point, which gets caller-allocated scratch.

Collected last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular_entry_point(lib, M, P, r):
    """Q = M^T P through psgd_gemm_ffma_launch with descriptor tables and scratch from torch."""
    from powersgd_b200.cuda_path import TilePlan, _to_device
    from powersgd_b200.ops import layout
    from powersgd_b200.plan import CompressionPlan

    n, m = M.shape
    plan = CompressionPlan.build([(n, m)], rank=r)
    tiles = TilePlan(plan, lib)
    vec = 4 if (m % 4 == 0 and M.data_ptr() % 16 == 0) else 2 if (m % 2 == 0 and M.data_ptr() % 8 == 0) else 1
    arrays = tiles.build([vec])
    desc = np.zeros(1, dtype=layout.MAT_DTYPE)
    desc["grad"] = M.data_ptr()
    desc["n"], desc["m"], desc["r"] = n, m, r
    desc_dev = _to_device(desc, M.device)
    tile_arr = arrays["nt"]["f"]
    tile_dev = _to_device(tile_arr, M.device)
    partial = torch.empty(tiles.partial_floats, device=M.device)
    tickets = torch.zeros(tiles.n_tickets, dtype=torch.int32, device=M.device)
    Q = torch.full((m, r), float("nan"), device=M.device)
    null = ctypes.c_void_p(0)
    empty = (ctypes.c_void_p * 1)()
    code = lib.psgd_gemm_ffma_launch(
        1, r, ctypes.c_void_p(desc_dev.data_ptr()), ctypes.c_void_p(tile_dev.data_ptr()), len(tile_arr),
        ctypes.c_void_p(P.data_ptr()), ctypes.c_void_p(Q.data_ptr()), null, 0, ctypes.cast(empty, ctypes.c_void_p),
        ctypes.cast(empty, ctypes.c_void_p), ctypes.c_void_p(partial.data_ptr()), ctypes.c_void_p(tickets.data_ptr()),
        null, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    assert code == 0, lib.psgd_last_error()
    torch.cuda.synchronize()
    return Q


def test_noalloc_product_matches_regular_entry_point_twice_in_a_row():
    from powersgd_b200.ops import native

    lib = native.lib()
    entry = lib.psgd_matmul_tn_noalloc  # the exported C symbol
    entry.restype = ctypes.c_int
    entry.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    gen = torch.Generator(device="cpu").manual_seed(7)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # different problems back to back: split over several row blocks, odd pitch, rank 3 -> padded;
    # 16-byte rows with one row block (no scratch needed), ranks 1 / 2 / 8, and a shape that fills
    # the built-in scratch exactly (2^20 floats: 4 column blocks x 256 row blocks x 128 x 8)
    for n, m, r in [(1000, 650, 4), (777, 1301, 3), (200, 512, 8), (1000, 512, 1), (300, 130, 2), (65536, 512, 8)]:
        M = torch.randn(n, m, generator=gen).to(dev)
        P = torch.randn(n, r, generator=gen).to(dev)
        Q = torch.full((m, r), float("nan"), device=dev)
        before = torch.cuda.memory_allocated(dev)
        code = entry(M.data_ptr(), n, m, P.data_ptr(), r, Q.data_ptr(), stream)
        assert code == 0, lib.psgd_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        expect = _regular_entry_point(lib, M, P, r)
        oracle = (M.double().T @ P.double()).float()
        rel = ((Q - expect).norm() / expect.norm()).item()
        assert rel < 2e-5, (n, m, r, rel)
        assert ((Q - oracle).norm() / oracle.norm()).item() < 2e-5

    # sizes beyond the built-in scratch are refused with a message, and nothing is launched
    assert entry(M.data_ptr(), 10, 10, P.data_ptr(), 9, Q.data_ptr(), stream) != 0
    assert b"rank" in lib.psgd_last_error()
    assert entry(M.data_ptr(), 1 << 20, 1 << 14, P.data_ptr(), 8, Q.data_ptr(), stream) != 0
    assert b"scratch" in lib.psgd_last_error()
    torch.cuda.synchronize()
