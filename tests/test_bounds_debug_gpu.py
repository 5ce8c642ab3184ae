"""The bounds-checked build of the native library (csrc/psgd_bounds.cuh): the same kernels compiled
with -DPSGD_BOUNDS_CHECK validate every tile against its matrix, its access width and the scratch
capacities, record the first violation in a status block and SKIP the access (no trap, no fault).

Two checks, each in a child process that loads the debug library through PSGD_B200_LIB:
  * the ragged small-shape suite (row pitches 27 and 650, rank above a dimension, rank-1 groups,
    several half-iterations, fused SGD) runs without a single violation and matches the PyTorch path;
  * a tile list that lies about its matrix (rows beyond the end, a 16-byte access width on a pitch of
    27 floats, a scratch slot beyond the arena) is caught: violations are recorded, nothing is written.
"""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEBUG_LIB = os.path.join(ROOT, "powersgd_b200", "csrc", "libpsgd_b200_debug.so")


def _run(code: str) -> subprocess.CompletedProcess:
    if not os.path.exists(DEBUG_LIB):
        pytest.skip("debug library not built (python -m powersgd_b200.csrc.build --debug)")
    env = dict(os.environ, PSGD_B200_LIB=DEBUG_LIB, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable, "-c", textwrap.dedent(code)], capture_output=True, text=True, timeout=600, env=env)


def test_small_shape_suite_has_no_violations_on_the_checked_build():
    res = _run(
        """
        import ctypes, torch
        from powersgd_b200 import BasicConfig, BasicPowerSGD, Config, PowerSGD, optimizer_step
        from powersgd_b200.ops import native
        lib = native.lib()
        assert hasattr(lib, "psgd_bounds_status"), "not the checked build"
        lib.psgd_bounds_status.restype = ctypes.c_int
        status = (ctypes.c_int * 24)()
        dev = torch.device("cuda:0")
        shapes = [(64, 3, 3, 3), (64, 64, 3, 3), (64, 64, 3, 3), (128, 64, 1, 1), (10, 512), (130, 650), (300, 1200), (33, 2100), (5, 9)]
        g = torch.Generator().manual_seed(0)
        for rank, iters in [(1, 2), (2, 2), (4, 3), (8, 1), (16, 2)]:
            params = [torch.zeros(s, device=dev) for s in shapes]
            ours = BasicPowerSGD(params, BasicConfig(rank=rank, num_iters_per_step=iters), backend="native")
            oracle = BasicPowerSGD(params, BasicConfig(rank=rank, num_iters_per_step=iters), backend="torch")
            ga = [torch.randn(s, generator=g).to(dev) for s in shapes]
            gb = [x.clone() for x in ga]
            for step in range(2):
                nat = ours._native
                if nat is not None and nat._key is not None:
                    # capacities of THIS object's scratch and factor buffers
                    limits = (nat._partial.numel(), nat._tickets.numel(), nat.h_in[0].numel(), nat.h_in[0].numel())
                else:
                    limits = (0, 0, 0, 0)   # not allocated yet: unchecked on the first call
                lib.psgd_debug_limits_products(*[ctypes.c_longlong(v) for v in limits])
                oa, ob = ours.aggregate(ga), oracle.aggregate(gb)
                torch.cuda.synchronize()
                for x, y, shp in zip(oa, ob, shapes):
                    n_, m_ = shp[0], int(torch.Size(shp).numel() // shp[0])
                    if min(n_, m_) <= rank * iters + 2:
                        continue   # residual exhausted: the factors are rounding noise, only the checks matter
                    rel = ((x.double() - y.double()).norm() / y.double().norm().clamp_min(1e-30)).item()
                    assert rel < 1e-3, (rank, iters, step, tuple(x.shape), rel)
        lib.psgd_debug_limits_products(*[ctypes.c_longlong(0)] * 4)
        # fused optimizer step through the checked kernels
        model = torch.nn.Sequential(torch.nn.Linear(200, 300), torch.nn.ReLU(), torch.nn.Linear(300, 129), torch.nn.ReLU(), torch.nn.Linear(129, 10)).to(dev)
        opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9, nesterov=True, weight_decay=1e-4)
        agg = PowerSGD(list(model.parameters()), Config(rank=4, num_iters_per_step=2, start_compressing_after_num_steps=1), backend="native")
        x, y = torch.randn(64, 200, device=dev), torch.randint(0, 10, (64,), device=dev)
        for _ in range(4):
            torch.nn.functional.cross_entropy(model(x), y).backward()
            optimizer_step(opt, agg)
        torch.cuda.synchronize()
        total = lib.psgd_bounds_status(status, 0)
        assert total == 0, list(status)
        print("CHECKED-OK")
        """
    )
    assert "CHECKED-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_inconsistent_tiles_are_recorded_and_skipped():
    res = _run(
        """
        import ctypes, numpy as np, torch
        from powersgd_b200.cuda_path import TilePlan, _to_device
        from powersgd_b200.ops import layout, native
        from powersgd_b200.plan import CompressionPlan
        lib = native.lib()
        lib.psgd_bounds_status.restype = ctypes.c_int
        status = (ctypes.c_int * 24)()
        dev = torch.device("cuda:0")
        n, m, r = 64, 27, 2
        M = torch.randn(n, m, device=dev)
        P = torch.randn(n, r, device=dev)
        plan = CompressionPlan.build([(n, m)], rank=r)
        tiles = TilePlan(plan, lib)
        arr = tiles.build([1])["nt"]["f"].copy()
        desc = np.zeros(1, dtype=layout.MAT_DTYPE)
        desc["grad"], desc["n"], desc["m"], desc["r"] = M.data_ptr(), n, m, r
        desc_dev = _to_device(desc, dev)
        partial = torch.empty(tiles.partial_floats, device=dev)
        tickets = torch.zeros(tiles.n_tickets, dtype=torch.int32, device=dev)
        null, empty = ctypes.c_void_p(0), (ctypes.c_void_p * 1)()

        def launch(tile_arr):
            Q = torch.full((m, r), 7.0, device=dev)
            tile_dev = _to_device(tile_arr, dev)
            code = lib.psgd_gemm_ffma_launch(1, r, ctypes.c_void_p(desc_dev.data_ptr()), ctypes.c_void_p(tile_dev.data_ptr()), len(tile_arr),
                ctypes.c_void_p(P.data_ptr()), ctypes.c_void_p(Q.data_ptr()), null, 0, ctypes.cast(empty, ctypes.c_void_p),
                ctypes.cast(empty, ctypes.c_void_p), ctypes.c_void_p(partial.data_ptr()), ctypes.c_void_p(tickets.data_ptr()), null,
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert code == 0
            torch.cuda.synchronize()
            return Q

        good = launch(arr)
        assert lib.psgd_bounds_status(status, 1) == 0
        assert torch.allclose(good, M.T @ P, atol=1e-4)
        for what, edit in [(1, lambda a: a.__setitem__("rows", a["rows"] + 5)),          # rows beyond the matrix
                           (3, lambda a: a.__setitem__("vec", 4)),                        # 16-byte accesses on a pitch of 27 floats
                           (2, lambda a: a.__setitem__("cols", 40))]:                     # columns beyond the matrix
            bad = arr.copy()
            edit(bad)
            out = launch(bad)
            total = lib.psgd_bounds_status(status, 1)
            assert total >= 1 and status[2] == what, (what, total, list(status)[:8])
            assert bool((out == 7.0).all()), "a rejected tile must not write"
        print("CAUGHT-OK")
        """
    )
    assert "CAUGHT-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
