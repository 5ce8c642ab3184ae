"""The power-iteration reducers of the research harness on the native sm_100a kernels.

`RankKReducer` (paper-code/gradient_reducers.py:665-788) and `HalfRankKReducer` (:794-936) issue,
per matrix-shaped tensor, library matrix products, a TorchScript Gram-Schmidt and three library
all-reduces. Their dataflow is the one the grouped kernels of this package already implement:

    RankK      p = M q  ->  sum over workers  ->  orthonormalise p  ->  q = M^T p  ->  mean over
               workers  ->  out = p q^T,  memory = M - out        (error against the GLOBAL product)
    HalfRankK  one half power-iteration per call, alternating sides, memory = M - (LOCAL product)

so on CUDA tensors they run as a handful of launches over ALL tensors at once: the grouped product
kernels (whose epilogues push the fresh factor to every peer), the orthonormalisation launch
(which gathers the pushed factor), and the strip kernel that writes `out` and `memory` in one
pass (and gathers the last factor itself). No shape batching: every tensor is its own group, as
in the original, which also keeps its per-matrix normalisation at rank 1.

The PyTorch formulation in `reducers.py` stays the oracle and the CPU path.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cuda_path import NativeCompressor, NativeFlatAllReduce, _ptr, _ptr_array, _stream_ptr
from ..ops import native
from ..plan import CompressionPlan
from ..utils import is_dense, world_size


class _Core:
    """What `NativeCompressor` needs to know about its owner: plan, factor buffers, counters."""

    class _Cfg:
        def __init__(self, rank: int, iters: int):
            self.rank, self.num_iters_per_step = rank, iters

    def __init__(self, shapes: Sequence[Sequence[int]], rank: int, iters: int, device: torch.device):
        self.device = device
        self.config = self._Cfg(rank, iters)
        self.plan = CompressionPlan.build(shapes, rank, batch_same_shapes=False)
        self.step_counter = 0
        self._ps_buffer = torch.zeros(max(self.plan.p_total, 1), device=device)
        self._qs_buffer = torch.zeros(max(self.plan.q_total, 1), device=device)

    def p_view(self, i: int) -> torch.Tensor:
        g = self.plan.groups[i]
        return self._ps_buffer[g.p_offset : g.p_offset + g.p_numel].view(g.n, g.r)

    def q_view(self, i: int) -> torch.Tensor:
        g = self.plan.groups[i]
        return self._qs_buffer[g.q_offset : g.q_offset + g.q_numel].view(g.m, g.r)


def usable(tensors: Sequence[torch.Tensor]) -> bool:
    """Native path: CUDA, float32, dense tensors, and the library present (its absence on a CUDA
    machine is an error unless PSGD_B200_ALLOW_FALLBACK=1)."""
    if not tensors or not all(t.is_cuda and t.dtype == torch.float32 and is_dense(t) for t in tensors):
        return False
    return native.use_for_cuda()


class NativeLowRank:
    """Shared driver: descriptors over (input, output, memory) triples, the flat all-reduce of the
    1-D tensors, and the launch sequences of the two reducers."""

    def __init__(self, matrices, rank: int, iters: int, device: torch.device):
        shapes = [tuple(t.shape) for t, _o, _m in matrices]
        self.core = _Core(shapes, rank, iters, device)
        self.comp = NativeCompressor(self.core)
        self.flat = NativeFlatAllReduce()
        self.launches = 0

    # factor memories in the layout of the original (`p_memory`, `q_memory`: tensor after tensor)
    @property
    def p_memory(self) -> torch.Tensor:
        return self.core._ps_buffer[: self.core.plan.p_total]

    @property
    def q_memory(self) -> torch.Tensor:
        return self.core._qs_buffer[: self.core.plan.q_total]

    def _bind(self, matrices) -> None:
        self.comp._bind(
            [t for t, _o, _m in matrices],
            params=[m for _t, _o, m in matrices],   # `param` slot of the descriptor: where the residual goes
            need_out=True,
            outs=[o for _t, o, _m in matrices],
        )

    def reduce_vectors(self, vectors) -> None:
        """Mean over workers of the 1-D tensors, written into the caller's outputs (inputs kept)."""
        if vectors:
            self.flat.aggregate([t for t, _o, _m in vectors], outs=[o for _t, o, _m in vectors], keep_inputs=True)
            self.launches += self.flat.launches

    # ------------------------------------------------------------------------------------------
    def rank_k(self, matrices) -> None:
        """p = M q (q as it is), sum, orthonormalise, q = M^T p, mean, out = p q^T, memory = M - out."""
        comp, core = self.comp, self.core
        comp.check()
        comp.launches = 0
        self._bind(matrices)
        workers = world_size()
        p2p = workers > 1 and comp.comm is not None
        P, Q = core._ps_buffer, core._qs_buffer
        p_loc, q_loc, p_hat = comp.h_loc[0], comp.h_loc[1], comp.h_in[1]
        # p = M q; one worker: straight into the factor memory
        comp._gemm(False, Q, p_loc, [], [], P if workers == 1 else None)
        if workers > 1 and not p2p:
            P.copy_(p_loc[: P.numel()])
            comp._allreduce_sum(P)
        # orthonormalise p in place (multi-GPU: the launch first gathers the pushed p's)
        comp._orth("p", P, p_hat, [], [], comp.h_sum[0] if p2p else None)
        # q = M^T p
        comp._gemm(True, p_hat, q_loc, [], [], Q if workers == 1 else None)
        gather = p2p and comp._gathers_in_finalize()
        if p2p and not gather:
            code = comp.lib.psgd_factor_reduce_launch(
                comp.comm.ptr, ctypes.c_longlong(Q.numel()), _ptr(comp.h_sum[1]), _ptr(Q), _stream_ptr()
            )
            native.check(code, "psgd_factor_reduce_launch")
            comp.launches += 1
        elif workers > 1 and not p2p:
            Q.copy_(q_loc[: Q.numel()])
            comp._allreduce_sum(Q)
        if workers > 1 and not gather:
            comp.h_sum[1][: Q.numel()].copy_(Q)
            Q.div_(workers)  # the factor memory keeps the MEAN, which the next step starts from
        # out = p (sum q / W)^T, memory = M - out
        self._finalize_global(p_hat, q_loc, q_loc if workers == 1 else comp.h_sum[1], workers, Q if gather else None)
        self.launches += comp.launches

    def _finalize_global(self, left: torch.Tensor, right_loc: torch.Tensor, right_sum: torch.Tensor, workers: int,
                         gather_state: Optional[torch.Tensor]) -> None:
        """One worker: local and summed factors coincide (single-accumulator kernel). Several: the
        kernel reads (or gathers) the summed right factor; the local one is staged but, with the
        global-residual option, not used."""
        comp = self.comp
        tiles, count = comp._tiles_dev["fin"]["f"]
        one = [left]
        code = comp.lib.psgd_finalize_launch(
            _ptr(comp._mats_dev), _ptr(tiles), count, comp.tiles.fin_rows, comp.tiles.max_r, _ptr(comp._hyper_dev), 1,
            ctypes.cast(_ptr_array(one), ctypes.c_void_p), ctypes.cast(_ptr_array([right_loc]), ctypes.c_void_p),
            ctypes.cast(_ptr_array(one), ctypes.c_void_p), ctypes.cast(_ptr_array([right_sum]), ctypes.c_void_p),
            1.0 / workers, 0,
            comp.comm.ptr if gather_state is not None else ctypes.c_void_p(0), 0,
            _ptr(comp.h_sum[1]) if gather_state is not None else ctypes.c_void_p(0),
            _ptr(gather_state) if gather_state is not None else ctypes.c_void_p(0),
            3,  # residual = M - update, written to the `param` slot (the caller's memory tensor)
            1.0 / workers,
            _stream_ptr(),
        )
        native.check(code, "psgd_finalize_launch")
        comp.launches += 1

    # ------------------------------------------------------------------------------------------
    def half_rank_k(self, matrices, compute_p: bool) -> None:
        """One half power-iteration: orthonormalise the warm-start factor of the other side,
        multiply, memory = M - (local product), out = product with the mean fresh factor."""
        comp, core = self.comp, self.core
        comp.check()
        comp.launches = 0
        self._bind(matrices)
        # the library core multiplies with P as the basis on even parity
        core.step_counter = 1 if compute_p else 0
        workers = world_size()
        if workers == 1:
            saved, comp.h_sum = comp.h_sum, comp.h_loc
        try:
            sides, pending = comp._half_iterations()
            comp._finalize(sides, fused_sgd=False, workers=workers, gather_state=pending, flags=2)
        finally:
            if workers == 1:
                comp.h_sum = saved
        self.launches += comp.launches
