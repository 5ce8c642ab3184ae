"""Drives the native sm_100a kernels for the compressor core and the flat all-reduce.

Per optimizer step the reference issues several hundred small PyTorch ops
(powersgd/powersgd.py:146-235). Here a step is, for T half-iterations:

    T x [ orthonormalise (2 launches; multi-GPU: the first one also gathers the factor the previous
          product pushed, i.e. it is the consumer of the in-kernel all-reduce)
          -> grouped product (1 launch; multi-GPU: its epilogue pushes the fresh factor to every peer) ]
      ->  decompress + error feedback (+ SGD) (1 launch; multi-GPU: gathers the last factor itself)

over ALL shape groups at once. The gradient matrices are addressed in place through a
pointer table (no `torch.stack`, no un-batching copies), the deflation between half-iterations
is algebraic (small r x r corrections), and the residual is written exactly once.

Factor bookkeeping for half-iteration t of a step (left = the P side is the input):

    left :  Lloc = Lsum = orth(P)      Rloc = local M^T P      Rsum = sum over workers
    right:  Rloc = Rsum = orth(Q)      Lloc = local M Q        Lsum = sum over workers

    residual = M - sum_t Lloc_t Rloc_t^T        update = (1/W) sum_t Lsum_t Rsum_t^T
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from .ops import layout, native
from .utils import is_dense, like_strided, same_layout, world_size


class _Range:
    """A named phase of `aggregate()`: an NVTX range when PSGD_B200_NVTX=1 (phase names show up
    in profiler timelines), a CUDA-event pair appended to `_Range.events` when a benchmark set
    that list (per-phase device times), free otherwise."""

    enabled = os.environ.get("PSGD_B200_NVTX", "0") == "1"
    events: Optional[list] = None

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if self.enabled:
            torch.cuda.nvtx.range_push(self.name)
        if _Range.events is not None:
            self._start = torch.cuda.Event(enable_timing=True)
            self._start.record()

    def __exit__(self, *exc):
        if _Range.events is not None:
            stop = torch.cuda.Event(enable_timing=True)
            stop.record()
            _Range.events.append((self.name, self._start, stop))
        if self.enabled:
            torch.cuda.nvtx.range_pop()


def _stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _ptr_array(tensors: Sequence[torch.Tensor]):
    arr = (ctypes.c_void_p * max(len(tensors), 1))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


def _to_device(array: np.ndarray, device: torch.device) -> torch.Tensor:
    """Upload a descriptor table. Staged through pinned memory with an async copy on the current
    stream, so that it is legal during CUDA-graph capture (where it becomes a copy node that
    re-reads the pinned buffer on every replay; the buffer is kept alive with the result)."""
    raw = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
    pinned = torch.empty(max(raw.size, 1), dtype=torch.uint8).pin_memory()
    pinned.numpy()[: raw.size] = raw
    out = torch.empty(max(raw.size, 1), dtype=torch.uint8, device=device)
    out.copy_(pinned, non_blocking=True)
    out._psgd_pinned_src = pinned
    if torch.cuda.is_current_stream_capturing():
        # the recorded copy node reads `pinned` and writes `out` on every replay: both must
        # outlive whatever later rebinding drops them from their owner, i.e. live as long as the
        # graph does. Inside a `capture_scope` the graph's owner keeps them; a capture made
        # without one parks them here for the life of the process.
        (_capture_keep if _capture_keep is not None else _CAPTURED_TABLES).append((out, pinned))
    return out


_CAPTURED_TABLES: list = []
_capture_keep: Optional[list] = None


class capture_scope:
    """`with capture_scope() as keep:` around a CUDA-graph capture collects the descriptor tables
    uploaded during it in `keep`; store `keep` next to the graph and drop both together."""

    def __enter__(self) -> list:
        global _capture_keep
        self._outer = _capture_keep
        _capture_keep = []
        return _capture_keep

    def __exit__(self, *exc):
        global _capture_keep
        _capture_keep = self._outer


def _split_even(total: int, max_chunk: int, multiple: int) -> List[Tuple[int, int]]:
    """Cut [0, total) into near-equal chunks of at most `max_chunk`, starts on `multiple`."""
    if total <= max_chunk:
        return [(0, total)]
    parts = -(-total // max_chunk)
    size = -(-total // parts)
    size = -(-size // multiple) * multiple
    out, start = [], 0
    while start < total:
        out.append((start, min(size, total - start)))
        start += size
    return out


class TilePlan:
    """Static tile lists (independent of tensor addresses) for one CompressionPlan."""

    def __init__(self, plan, lib):
        self.plan = plan
        mats = []  # (group index, position, compressed-list index)
        for gi, g in enumerate(plan.groups):
            for pos, idx in enumerate(g.members):
                mats.append((gi, pos, idx))
        self.mats = mats
        self.max_r = max((g.r for g in plan.groups), default=1)
        if self.max_r > layout.MAX_RANK:
            raise ValueError(f"rank {self.max_r} exceeds the compiled maximum {layout.MAX_RANK}")
        self.rt = lib.psgd_gemm_template_rank(self.max_r)
        self.total_elems = sum(g.n * g.m * g.batch for g in plan.groups)
        nt_rows_cap = lib.psgd_gemm_nt_max_rows(self.max_r)
        self.nt_rows = min(nt_rows_cap, 128 if self.total_elems < (64 << 20) else 256)
        self.nn_rows = lib.psgd_gemm_nn_tile_rows(self.max_r)
        self.nn_cols_cap = 1024
        self.rp_tc = lib.psgd_gemm_tc_rank_pad(self.max_r)
        self.fin_tc_ok = False  # set by the compressor: (half-iterations x rank) fits the tensor-core finalize
        self.fin_rows = 32      # set by the compressor: height of a finalize strip (multiple of 32)

    def build(self, vec_widths: Sequence[int], tc_flags: Optional[Sequence[bool]] = None):
        """Tile arrays for the CUDA-core kernels (key "f"; every tile carries the access width of
        its matrix: 4, 2 or 1 floats) and, for the matrices flagged in `tc_flags`, tensor-core
        tiles (key "tc")."""
        nt = {"f": [], "tc": []}
        nn = {"f": [], "tc": []}
        fin = {"f": [], "tc": []}
        ticket = 0
        nt_slots = nn_slots = tc_slots = 0
        tc_flags = tc_flags or [False] * len(self.mats)
        # K extent of one tensor-core tile: long enough to amortise the pipeline ramp and the
        # epilogue, short enough that a small model still fills the GPU, and such that the last
        # wave of CTAs is nearly full (the block scheduler runs TC_CTAS_PER_SM per SM at a time)
        tc_mats = [self.plan.groups[gi] for (gi, _p, _i), f in zip(self.mats, tc_flags) if f]
        tc_k_nt = self._pick_tc_k(tc_mats, transposed=True)
        tc_k_nn = self._pick_tc_k(tc_mats, transposed=False)
        for mi, (gi, _pos, _idx) in enumerate(self.mats):
            g = self.plan.groups[gi]
            v = int(vec_widths[mi])
            if tc_flags[mi] and self.fin_tc_ok:
                for r0 in range(0, g.n, 128):
                    for c0 in range(0, g.m, 64):
                        fin["tc"].append((mi, r0, min(128, g.n - r0), c0, min(64, g.m - c0), 0, 1, 0, 0, v, (0, 0)))
            else:
                for r0 in range(0, g.n, self.fin_rows):
                    for c0 in range(0, g.m, 128):
                        fin["f"].append((mi, r0, min(self.fin_rows, g.n - r0), c0, min(128, g.m - c0), 0, 1, 0, 0, v, (0, 0)))
            if tc_flags[mi]:
                row_blocks = _split_even(g.n, tc_k_nt, 32)
                for c0 in range(0, g.m, 128):
                    for si, (r0, rows) in enumerate(row_blocks):
                        nt["tc"].append((mi, r0, rows, c0, min(128, g.m - c0), si, len(row_blocks), ticket, tc_slots, v, (0, 0)))
                    ticket += 1
                    tc_slots += len(row_blocks)
                col_blocks = _split_even(g.m, tc_k_nn, 32)
                for r0 in range(0, g.n, 128):
                    for si, (c0, cols) in enumerate(col_blocks):
                        nn["tc"].append((mi, r0, min(128, g.n - r0), c0, cols, si, len(col_blocks), ticket, tc_slots, v, (0, 0)))
                    ticket += 1
                    tc_slots += len(col_blocks)
                continue
            # tall matrices: tiles of 256 rows (128 KiB: small enough that every SM holds several at
            # any time, which is what hides the load latency) but never more than 160 partial tiles
            # per column block (the kernel walks a taller tile in chunks of its staging buffer)
            rows_per_tile = max(self.nt_rows if g.n <= 4096 else 256, -(-(-(-g.n // 160)) // 128) * 128)
            row_blocks = _split_even(g.n, rows_per_tile, 1)
            for c0 in range(0, g.m, 128):
                cols = min(128, g.m - c0)
                for si, (r0, rows) in enumerate(row_blocks):
                    nt["f"].append((mi, r0, rows, c0, cols, si, len(row_blocks), ticket, nt_slots, v, (0, 0)))
                ticket += 1
                nt_slots += len(row_blocks)
            col_blocks = _split_even(g.m, self.nn_cols_cap, 128)
            for r0 in range(0, g.n, self.nn_rows):
                rows = min(self.nn_rows, g.n - r0)
                for si, (c0, cols) in enumerate(col_blocks):
                    nn["f"].append((mi, r0, rows, c0, cols, si, len(col_blocks), ticket, nn_slots, v, (0, 0)))
                ticket += 1
                nn_slots += len(col_blocks)
        self.n_tickets = max(ticket, 1)
        self.partial_floats = max(nt_slots * 128 * self.rt, nn_slots * self.nn_rows * self.rt, 1)
        self.partial_tc_floats = max(tc_slots * 128 * self.rp_tc, 1)

        def arr(items):
            return np.array(items, dtype=layout.TILE_DTYPE) if items else np.zeros(0, dtype=layout.TILE_DTYPE)

        return {
            "nt": {k: arr(v) for k, v in nt.items()},
            "nn": {k: arr(v) for k, v in nn.items()},
            "fin": {k: arr(v) for k, v in fin.items()},
        }

    TC_CTAS_PER_SM = 2
    # prologue + epilogue of a tile (~4 us), in units of streamed K rows (~0.03 us each): measured
    # as rounds x (overhead + rows) over tile extents 512 ... 4096 on 4 x 4096^2
    TC_TILE_OVERHEAD_ROWS = 136

    def _pick_tc_k(self, groups, transposed: bool) -> int:
        if not groups:
            return 512
        if os.environ.get("PSGD_B200_TC_K"):
            return int(os.environ["PSGD_B200_TC_K"])  # tuning knob: fixed K extent (a multiple of 32)
        slots = 148 * self.TC_CTAS_PER_SM
        best, best_score = 512, -1.0
        longest = max((g.n if transposed else g.m) for g in groups)
        for k in range(256, max(256, min(8192, -(-longest // 32) * 32)) + 1, 32):
            tiles = 0
            for g in groups:
                k_len, out_len = (g.n, g.m) if transposed else (g.m, g.n)
                tiles += -(-out_len // 128) * len(_split_even(k_len, k, 32))
            waves = -(-tiles // slots)
            score = tiles / (waves * slots) * k / (k + self.TC_TILE_OVERHEAD_ROWS)
            if score > best_score + 1e-9:
                best, best_score = k, score
        return best

    def orth_units(self, side: str, chunk_rows: int) -> Tuple[np.ndarray, np.ndarray]:
        """Units (one per matrix; one per shape group at rank 1) and their row chunks of at most
        `chunk_rows` rows, which never straddle the sub-matrices of a rank-1 unit."""
        units, chunks = [], []
        mi = 0

        def add(base, length, nsub, r, first_mat):
            chunk0 = len(chunks)
            for sub in range(nsub):
                for r0 in range(0, length, chunk_rows):
                    chunks.append((len(units), sub, sub * length + r0, min(chunk_rows, length - r0)))
            units.append((base, length, nsub, r, first_mat, chunk0, len(chunks) - chunk0, 0))

        for g in self.plan.groups:
            length = g.n if side == "p" else g.m
            base = g.p_offset if side == "p" else g.q_offset
            if g.r == 1:
                add(base, length, g.batch, 1, mi)
            else:
                for b in range(g.batch):
                    add(base + b * length * g.r, length, 1, g.r, mi + b)
            mi += g.batch
        return np.array(units, dtype=layout.ORTH_UNIT_DTYPE), np.array(chunks, dtype=layout.ORTH_CHUNK_DTYPE)


class NativeCompressor:
    """Runs `BasicPowerSGD.aggregate` on the GPU with the in-tree kernels."""

    def __init__(self, core):
        self.core = core
        self.lib = native.lib()
        self.device = core.device
        self.plan = core.plan
        self.tiles = TilePlan(core.plan, self.lib)
        self.T = core.config.num_iters_per_step
        self.tiles.fin_tc_ok = (
            self.T * self.tiles.max_r <= self.lib.psgd_finalize_tc_max_k()
            and os.environ.get("PSGD_B200_FINALIZE", "ffma") == "tc"
        )
        if self.T > layout.MAX_HIST:
            raise ValueError(f"num_iters_per_step {self.T} exceeds the compiled maximum {layout.MAX_HIST}")
        # finalize strips: as tall as the factor panels allow in shared memory, but short enough
        # that a small model still spreads over ~6 strips per SM
        strip_cap = int(self.lib.psgd_finalize_strip_rows(self.T * self.tiles.max_r, 1 if world_size() == 1 else 0))
        want = self.tiles.total_elems // (128 * 148 * 6)
        self.tiles.fin_rows = max(32, min(strip_cap, want // 32 * 32))
        nm = len(self.tiles.mats)
        cap = max(self.plan.p_total, self.plan.q_total, 1)
        f32 = dict(device=self.device, dtype=torch.float32)
        self.h_in = [torch.zeros(cap, **f32) for _ in range(self.T)]
        self.h_loc = [torch.zeros(cap, **f32) for _ in range(self.T)]
        self.h_sum = [torch.zeros(cap, **f32) for _ in range(self.T)]
        self.cmat = [[torch.zeros(nm * layout.CMAT_STRIDE, **f32) for _ in range(t)] for t in range(self.T)]
        chunk_rows = int(self.lib.psgd_orth_chunk_rows(self.tiles.max_r))
        rt = int(self.lib.psgd_orth_template_rank(self.tiles.max_r))
        self.units, self.chunks, self.n_units, self.n_chunks = {}, {}, {}, {}
        for s in ("p", "q"):
            units, chunks = self.tiles.orth_units(s, chunk_rows)
            self.units[s], self.chunks[s] = _to_device(units, self.device), _to_device(chunks, self.device)
            self.n_units[s], self.n_chunks[s] = len(units), len(chunks)
        # scratch of the orthonormalisation: partial sums per chunk, R^-1 / column status / ticket per unit
        part_doubles = int(self.lib.psgd_orth_part_doubles(self.tiles.max_r, max(self.T - 1, 0)))
        max_units = max(max(self.n_units.values()), 1)
        self._orth_part = torch.zeros(max(max(self.n_chunks.values()), 1) * part_doubles, device=self.device, dtype=torch.float64)
        self._orth_rinv = torch.zeros(max_units * rt * rt, device=self.device, dtype=torch.float64)
        self._orth_dead = torch.zeros(max_units * rt, device=self.device, dtype=torch.int32)
        self._orth_tickets = torch.zeros(max_units, device=self.device, dtype=torch.int32)
        self._key = None
        self._out_arena: Optional[torch.Tensor] = None
        self._hyper_dev = _to_device(self._default_hyper(), self.device)
        self.launches = 0  # kernels launched by the last aggregate()
        self._side_stream = torch.cuda.Stream(device=self.device)
        self._early = None  # (side, event) of an orthonormalisation issued by begin_step()
        self._early_launches = 0
        self._early_bucket: frozenset = frozenset()
        self._early_product_done = None  # event of a first product launched ahead for the early bucket
        # multi-GPU: factors are all-reduced by the product kernels themselves (peer pushes) plus
        # a small consumer kernel; PSGD_B200_COMM=nccl selects the library all-reduce instead
        self.comm = None
        if world_size() > 1 and os.environ.get("PSGD_B200_COMM", "p2p") == "p2p":
            from .parallel.symm import Channel, assert_same_on_all_ranks

            # a rank with another model, rank or iteration count would push factors of another
            # layout: find out now, with a message, instead of through a timeout later
            assert_same_on_all_ranks(
                (self.plan.signature(), int(core.config.rank), int(self.T)), "PowerSGD compression plan"
            )
            self.comm = Channel(cap)
        # status word of the tensor-core kernels' bounded waits: mapped pinned host memory, so the
        # host can look at it every step without touching the GPU
        from .parallel.symm import StatusWord

        self._status = StatusWord()

    @staticmethod
    def _default_hyper() -> np.ndarray:
        h = np.zeros(1, dtype=layout.HYPER_DTYPE)
        h["grad_scale"] = 1.0
        h["one_minus_dampening"] = 1.0
        return h

    # -- descriptors -----------------------------------------------------------------------
    def _bind(
        self,
        grads: Sequence[torch.Tensor],
        params: Optional[Sequence[torch.Tensor]] = None,
        moms: Optional[Sequence[Optional[torch.Tensor]]] = None,
        hyper_index: Optional[Sequence[int]] = None,
        need_out: bool = True,
        outs: Optional[Sequence[torch.Tensor]] = None,
    ) -> None:
        """`outs`: caller-owned tensors (laid out like the gradients) that receive the averaged
        update instead of this object's own arena."""
        key = (
            tuple(g.data_ptr() for g in grads),
            None if params is None else tuple(p.data_ptr() for p in params),
            None if moms is None else tuple(0 if m is None else m.data_ptr() for m in moms),
            need_out,
            None if outs is None else tuple(o.data_ptr() for o in outs),
        )
        if key == self._key:
            return
        for g in grads:
            if not is_dense(g) or g.dtype != torch.float32 or g.device != self.device:
                raise ValueError("native PowerSGD needs dense float32 gradients on its device")
        for name, others in (("parameters", params), ("momentum buffers", moms), ("outputs", outs)):
            for g, o in zip(grads, others or []):
                if o is not None and not same_layout(o, g):
                    raise ValueError(f"native PowerSGD needs {name} laid out like their gradients")
        if need_out and outs is None and self._out_arena is None:
            self._out_arena = torch.empty(self.tiles.total_elems, device=self.device, dtype=torch.float32)
        where = self.plan.locate()
        descs = np.zeros(len(self.tiles.mats), dtype=layout.MAT_DTYPE)
        vec = []
        out_views: List[Optional[torch.Tensor]] = [None] * len(grads)
        cursor = 0
        # output arena is laid out in compressed-list order so that views are plain slices
        out_offsets = []
        for g in grads:
            out_offsets.append(cursor)
            cursor += g.numel()
        for mi, (gi, pos, idx) in enumerate(self.tiles.mats):
            g = self.plan.groups[gi]
            d = descs[mi]
            d["grad"] = grads[idx].data_ptr()
            d["param"] = 0 if params is None else params[idx].data_ptr()
            d["mom"] = 0 if (moms is None or moms[idx] is None) else moms[idx].data_ptr()
            if need_out and outs is not None:
                out_views[idx] = outs[idx]
                d["out"] = outs[idx].data_ptr()
            elif need_out:
                view = self._out_arena[out_offsets[idx] : out_offsets[idx] + grads[idx].numel()]
                out_views[idx] = like_strided(view, grads[idx])
                d["out"] = view.data_ptr()
            d["n"], d["m"], d["r"] = g.n, g.m, g.r
            d["p_off"] = g.p_offset + pos * g.n * g.r
            d["q_off"] = g.q_offset + pos * g.m * g.r
            d["grp_p_off"], d["grp_p_len"] = g.p_offset, g.p_numel
            d["grp_q_off"], d["grp_q_len"] = g.q_offset, g.q_numel
            d["hyper"] = 0 if hyper_index is None else hyper_index[idx]
            d["index"] = mi
            ptrs = [int(d["grad"]), int(d["param"]), int(d["mom"]), int(d["out"])]
            # widest global access every row of the matrix (and of its companions) allows
            if g.m % 4 == 0 and all(p % 16 == 0 for p in ptrs):
                vec.append(4)
            elif g.m % 2 == 0 and all(p % 8 == 0 for p in ptrs):
                vec.append(2)
            else:
                vec.append(1)
        assert where is not None
        self._mats_dev = _to_device(descs, self.device)
        # tensor-core (TMA + tcgen05) path: matrices TMA can address and that are worth it
        mode = os.environ.get("PSGD_B200_GEMM", "auto")
        hbm_bound = self.tiles.total_elems * 4 > (96 << 20)
        tc = []
        maps = np.zeros((len(self.tiles.mats), 256), dtype=np.uint8)
        for mi, (gi, _pos, idx) in enumerate(self.tiles.mats):
            g = self.plan.groups[gi]
            ok = vec[mi] == 4 and g.n >= 128 and g.m >= 128 and mode != "ffma"
            ok = ok and (mode == "tc" or hbm_bound or self.tiles.max_r >= 8)
            if ok:
                buf = (ctypes.c_ubyte * 256)()
                code = self.lib.psgd_tma_encode_matrix(buf, ctypes.c_void_p(grads[idx].data_ptr()), g.n, g.m)
                native.check(code, "psgd_tma_encode_matrix")
                maps[mi] = np.frombuffer(buf, dtype=np.uint8)
            tc.append(bool(ok))
        self._maps_dev = _to_device(maps, self.device)
        self._tc_split = os.environ.get("PSGD_B200_TC_PRECISION", "split") != "tf32"
        self.uses_tensor_cores = any(tc)
        # compressed-list positions whose products run on the tensor-core kernels (one launch per
        # half-iteration for all of them; they are not split into an early and a late bucket)
        self.tensor_core_positions = frozenset(idx for (_gi, _pos, idx), flag in zip(self.tiles.mats, tc) if flag)
        tile_arrays = self.tiles.build(vec, tc)
        self._tile_arrays = tile_arrays
        self._tiles_dev: Dict[str, Dict[int, Tuple[torch.Tensor, int]]] = {}
        for name, by_vec in tile_arrays.items():
            self._tiles_dev[name] = {
                v: (_to_device(a, self.device) if len(a) else None, len(a)) for v, a in by_vec.items()
            }
        self._split_tile_lists()
        self._partial = torch.empty(self.tiles.partial_floats, device=self.device, dtype=torch.float32)
        self._partial_tc = torch.empty(self.tiles.partial_tc_floats, device=self.device, dtype=torch.float32)
        self._tickets = torch.zeros(self.tiles.n_tickets, device=self.device, dtype=torch.int32)
        self._out_views = out_views
        self._key = key

    # -- early bucket ---------------------------------------------------------------------
    def set_early_bucket(self, compressed_indices: Sequence[int]) -> None:
        """Compressed tensors (positions in the compressed list) whose gradients are complete
        early in backward: the first product of a step can be launched for them from a
        post-accumulate hook, on a side stream, while backward is still running for the rest."""
        self._early_bucket = frozenset(int(i) for i in compressed_indices)
        if self._key is not None:
            self._split_tile_lists()

    def _split_tile_lists(self) -> None:
        """Product tile lists of the early bucket ("fA") and of everything else ("fB")."""
        early_mats = [mi for mi, (_gi, _pos, idx) in enumerate(self.tiles.mats) if idx in self._early_bucket]
        for name in ("nt", "nn"):
            arr = self._tile_arrays[name]["f"]
            mask = np.isin(arr["mat"], early_mats) if len(arr) else np.zeros(0, dtype=bool)
            for key, sub in (("fA", arr[mask]), ("fB", arr[~mask])):
                self._tiles_dev[name][key] = (_to_device(np.ascontiguousarray(sub), self.device) if len(sub) else None, len(sub))

    def early_product(self) -> bool:
        """Launch the first product of the coming step for the early bucket NOW, on the side
        stream (after the orthonormalisation `begin_step` issued there). Returns False when there
        is nothing to launch early. `_half_iterations` then only launches the rest and joins."""
        if not self._early_bucket or self._early is None or self._key is None:
            return False
        core = self.core
        left = (core.step_counter * self.T) % 2 == 0
        if self._early[0] != ("p" if left else "q"):
            return False
        name = "nt" if left else "nn"
        if self._tiles_dev[name]["fA"][1] == 0:
            return False
        state_out = core._qs_buffer if left else core._ps_buffer
        fork = torch.cuda.Event()
        fork.record(torch.cuda.current_stream())
        self._side_stream.wait_event(fork)
        with torch.cuda.stream(self._side_stream):
            before = self.launches
            self._gemm(left, self.h_in[0], self.h_loc[0], [], self.cmat[0], state_out if world_size() == 1 else None, part="early")
            self._early_launches += self.launches - before
            done = torch.cuda.Event()
            done.record(self._side_stream)
        self._early_product_done = done
        return True

    # -- phases ----------------------------------------------------------------------------
    def _orth(self, side: str, x: torch.Tensor, copy_to: torch.Tensor, prev: List[torch.Tensor], cm: List[torch.Tensor],
              gather_to: Optional[torch.Tensor] = None):
        """Orthonormalise `x` in place (mirrored into `copy_to`). With `gather_to`, `x` is first
        filled with the sum over workers of the factor the previous product pushed (the sum is
        also written to `gather_to`): the launch is the consumer of the in-kernel all-reduce."""
        code = self.lib.psgd_orth_launch(
            _ptr(self.units[side]),
            self.n_units[side],
            _ptr(self.chunks[side]),
            self.n_chunks[side],
            self.tiles.max_r,
            _ptr(x),
            _ptr(copy_to),
            len(prev),
            ctypes.cast(_ptr_array(prev), ctypes.c_void_p),
            ctypes.cast(_ptr_array(cm), ctypes.c_void_p),
            _ptr(self._orth_part),
            _ptr(self._orth_rinv),
            _ptr(self._orth_dead),
            _ptr(self._orth_tickets),
            self.comm.ptr if gather_to is not None else ctypes.c_void_p(0),
            _ptr(gather_to),
            _stream_ptr(),
        )
        native.check(code, "psgd_orth_launch")
        self.launches += 2  # Gram + factorisation, then the application of R^-1

    def _gemm(self, transposed: bool, fin: torch.Tensor, fout: torch.Tensor, corr_fac, corr_c,
              fout2: Optional[torch.Tensor] = None, part: str = "all"):
        """`part`: "all", or one half of a split launch - "early" (the CUDA-core tiles of the
        matrices in the early bucket) / "late" (everything else); see `set_early_bucket`."""
        name = "nt" if transposed else "nn"
        tiles, count = self._tiles_dev[name]["tc"]
        if count and part != "early":
            code = self.lib.psgd_gemm_tc_launch(
                1 if transposed else 0,
                1 if self._tc_split else 0,
                self.tiles.max_r,
                _ptr(self._mats_dev),
                _ptr(tiles),
                count,
                _ptr(self._maps_dev),
                _ptr(fin),
                _ptr(fout),
                _ptr(fout2),
                len(corr_fac),
                ctypes.cast(_ptr_array(corr_fac), ctypes.c_void_p),
                ctypes.cast(_ptr_array(corr_c), ctypes.c_void_p),
                _ptr(self._partial_tc),
                _ptr(self._tickets),
                self.comm.ptr if self.comm is not None else ctypes.c_void_p(0),
                self._status.dev_ptr,
                _stream_ptr(),
            )
            native.check(code, "psgd_gemm_tc_launch")
            self.launches += 1
        tiles, count = self._tiles_dev[name]["f" if part == "all" else ("fA" if part == "early" else "fB")]
        if count:
            code = self.lib.psgd_gemm_ffma_launch(
                1 if transposed else 0,
                self.tiles.max_r,
                _ptr(self._mats_dev),
                _ptr(tiles),
                count,
                _ptr(fin),
                _ptr(fout),
                _ptr(fout2),
                len(corr_fac),
                ctypes.cast(_ptr_array(corr_fac), ctypes.c_void_p),
                ctypes.cast(_ptr_array(corr_c), ctypes.c_void_p),
                _ptr(self._partial),
                _ptr(self._tickets),
                self.comm.ptr if self.comm is not None else ctypes.c_void_p(0),
                _stream_ptr(),
            )
            native.check(code, "psgd_gemm_ffma_launch")
            self.launches += 1

    def _gathers_in_finalize(self) -> bool:
        """Multi-GPU: can the decompression launch gather the last factor from the channel itself?
        Only the strip kernel does, and only when it is the sole decompression launch."""
        if self.comm is None or world_size() == 1:
            return False
        if self._tiles_dev["fin"]["tc"][1]:
            return False
        return bool(self.lib.psgd_finalize_uses_strip(self.T, self.tiles.max_r, self.tiles.fin_rows, 0))

    def _finalize(self, sides: List[bool], fused_sgd: bool, workers: int, gather_state: Optional[torch.Tensor] = None,
                  flags: int = 0):
        """`gather_state`: the warm-start buffer that receives the summed factor of the last
        half-iteration when this launch is also its consumer (see `_gathers_in_finalize`).
        `flags`: residual options of the strip / general kernels (csrc/finalize.cu, FinalizeArgs)."""
        if flags and self._tiles_dev["fin"]["tc"][1]:
            raise ValueError("residual options are not available with the tensor-core decompression kernel")
        lloc, rloc, lsum, rsum = [], [], [], []
        for t, left in enumerate(sides):
            if left:
                lloc.append(self.h_in[t]); lsum.append(self.h_in[t])
                rloc.append(self.h_loc[t]); rsum.append(self.h_sum[t])
            else:
                rloc.append(self.h_in[t]); rsum.append(self.h_in[t])
                lloc.append(self.h_loc[t]); lsum.append(self.h_sum[t])
        tiles, count = self._tiles_dev["fin"]["tc"]
        if count:
            code = self.lib.psgd_finalize_tc_launch(
                _ptr(self._mats_dev),
                _ptr(tiles),
                count,
                _ptr(self._maps_dev),
                _ptr(self._hyper_dev),
                len(sides),
                self.tiles.max_r,
                ctypes.cast(_ptr_array(lloc), ctypes.c_void_p),
                ctypes.cast(_ptr_array(rloc), ctypes.c_void_p),
                ctypes.cast(_ptr_array(lsum), ctypes.c_void_p),
                ctypes.cast(_ptr_array(rsum), ctypes.c_void_p),
                1.0 / workers,
                1 if fused_sgd else 0,
                self._status.dev_ptr,
                _stream_ptr(),
            )
            native.check(code, "psgd_finalize_tc_launch")
            self.launches += 1
        tiles, count = self._tiles_dev["fin"]["f"]
        if count:
            gather = gather_state is not None
            code = self.lib.psgd_finalize_launch(
                _ptr(self._mats_dev),
                _ptr(tiles),
                count,
                self.tiles.fin_rows,
                self.tiles.max_r,
                _ptr(self._hyper_dev),
                len(sides),
                ctypes.cast(_ptr_array(lloc), ctypes.c_void_p),
                ctypes.cast(_ptr_array(rloc), ctypes.c_void_p),
                ctypes.cast(_ptr_array(lsum), ctypes.c_void_p),
                ctypes.cast(_ptr_array(rsum), ctypes.c_void_p),
                1.0 / workers,
                1 if fused_sgd else 0,
                self.comm.ptr if gather else ctypes.c_void_p(0),
                0 if sides[-1] else 1,  # last half-iteration left: the fresh (summed) factor is the right one
                _ptr(self.h_sum[len(sides) - 1]) if gather else ctypes.c_void_p(0),
                _ptr(gather_state) if gather else ctypes.c_void_p(0),
                int(flags),
                1.0,
                _stream_ptr(),
            )
            native.check(code, "psgd_finalize_launch")
            self.launches += 1

    def _half_iterations(self):
        """Runs the T half-iterations. Returns (sides, pending): `pending` is the warm-start buffer
        whose summed factor the decompression launch still has to gather, or None."""
        core = self.core
        workers = world_size()
        p2p = workers > 1 and self.comm is not None
        defer_last = p2p and self._gathers_in_finalize()
        sides: List[bool] = []
        pending: Optional[torch.Tensor] = None   # state buffer whose sum is still in the channel's slots
        for t in range(self.T):
            left = (core.step_counter * self.T + t) % 2 == 0
            sides.append(left)
            side = "p" if left else "q"
            state_in = core._ps_buffer if left else core._qs_buffer
            state_out = core._qs_buffer if left else core._ps_buffer
            # earlier LOCAL factors on the input side (cross products) and on the output side (corrections)
            same, other = [], []
            for i in range(t):
                in_side_i = self.h_in[i] if sides[i] == left else self.h_loc[i]
                out_side_i = self.h_loc[i] if sides[i] == left else self.h_in[i]
                same.append(in_side_i)
                other.append(out_side_i)
            with _Range(f"psgd.iter{t}.orth"):
                gather_to = None
                if pending is not None:
                    # the basis of this half-iteration IS the factor the previous product pushed
                    assert pending is state_in
                    gather_to, pending = self.h_sum[t - 1], None
                if t == 0 and self._early is not None:
                    # the first basis was orthonormalised on the side stream while forward / backward ran
                    early_side, event = self._early
                    self._early = None
                    torch.cuda.current_stream().wait_event(event)
                    if early_side != side:  # state changed under us (e.g. a checkpoint was loaded): redo
                        self._orth(side, state_in, self.h_in[t], same, self.cmat[t])
                else:
                    self._orth(side, state_in, self.h_in[t], same, self.cmat[t], gather_to)
            with _Range(f"psgd.iter{t}.product"):
                # one worker: the product is final, so the kernel also writes the warm-start buffer
                part = "all"
                if t == 0 and self._early_product_done is not None:
                    part = "late"  # the early bucket's tiles were launched during backward
                self._gemm(left, self.h_in[t], self.h_loc[t], other, self.cmat[t], state_out if workers == 1 else None, part=part)
                if part == "late":
                    torch.cuda.current_stream().wait_event(self._early_product_done)
                    self._early_product_done = None
            total = state_out.numel()
            with _Range(f"psgd.iter{t}.reduce"):
                if p2p and (t < self.T - 1 or defer_last):
                    pending = state_out  # gathered by the next consumer of that factor
                elif p2p:
                    code = self.lib.psgd_factor_reduce_launch(
                        self.comm.ptr, ctypes.c_longlong(total), _ptr(self.h_sum[t]), _ptr(state_out), _stream_ptr()
                    )
                    native.check(code, "psgd_factor_reduce_launch")
                    self.launches += 1
                elif workers > 1:
                    self.h_sum[t][:total].copy_(self.h_loc[t][:total])
                    self._allreduce_sum(self.h_sum[t][:total])
                    state_out.copy_(self.h_sum[t][:total])
        return sides, pending

    def _allreduce_sum(self, flat: torch.Tensor) -> None:
        dist.all_reduce(flat)

    def begin_step(self) -> None:
        """Orthonormalise the basis of the first half-iteration NOW, on a side stream.

        That basis only depends on the factors left by the previous step, not on the gradients
        about to be computed, so the launch overlaps with forward / backward; `aggregate` then
        waits on an event instead of launching it. Captured in a CUDA graph this is a parallel
        branch of the step."""
        if self._early is not None:
            return
        core = self.core
        left = (core.step_counter * self.T) % 2 == 0
        side = "p" if left else "q"
        state_in = core._ps_buffer if left else core._qs_buffer
        main = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(main)
        self._side_stream.wait_event(fork)
        with torch.cuda.stream(self._side_stream):
            before = self.launches
            self._orth(side, state_in, self.h_in[0], [], self.cmat[0])
            self._early_launches = self.launches - before  # counted with the step that uses them
            done = torch.cuda.Event()
            done.record(self._side_stream)
        self._early = (side, done)

    def close(self) -> None:
        """Release the peer mappings and the symmetric arena (collective across ranks)."""
        if self.comm is not None:
            self.comm.close()
            self.comm = None

    def check(self) -> None:
        """Raise `PowerSGDCommTimeout` if a bounded device-side wait of an EARLIER launch gave up
        (a peer that never pushed, a tensor-core pipeline that stalled). Plain host reads of
        mapped pinned words: no synchronisation, cheap enough for every step."""
        if self.comm is not None:
            self.comm.check()
        self._status.check("a tensor-core pipeline wait")

    # -- public ----------------------------------------------------------------------------
    def aggregate(self, gradients: List[torch.Tensor]) -> List[torch.Tensor]:
        self.check()
        self.launches = self._early_launches if self._early is not None else 0
        self._bind(gradients)
        workers = world_size()
        if workers == 1:
            saved = self.h_sum
            self.h_sum = self.h_loc
        try:
            sides, pending = self._half_iterations()
            with _Range("psgd.finalize"):
                self._finalize(sides, fused_sgd=False, workers=workers, gather_state=pending)
        finally:
            if workers == 1:
                self.h_sum = saved
        return list(self._out_views)

    def aggregate_and_step(
        self,
        gradients: List[torch.Tensor],
        params: List[torch.Tensor],
        moms: List[Optional[torch.Tensor]],
        hyper_index: List[int],
        hyper_dev: torch.Tensor,
    ) -> None:
        """Same as `aggregate`, but applies SGD to `params` inside the last kernel instead of
        materialising the averaged gradients."""
        self.check()
        self.launches = self._early_launches if self._early is not None else 0
        self._bind(gradients, params, moms, hyper_index, need_out=False)
        workers = world_size()
        keep = self._hyper_dev
        self._hyper_dev = hyper_dev
        if workers == 1:
            saved = self.h_sum
            self.h_sum = self.h_loc
        try:
            sides, pending = self._half_iterations()
            with _Range("psgd.finalize+sgd"):
                self._finalize(sides, fused_sgd=True, workers=workers, gather_state=pending)
        finally:
            self._hyper_dev = keep
            if workers == 1:
                self.h_sum = saved


class NativeFlatAllReduce:
    """Mean of a list of float32 tensors through one flat buffer, with the packing, the 1/W
    scale, the zeroing of the inputs and (optionally) the SGD update done by one multi-tensor
    kernel on each side of the collective."""

    # one-shot pushes send (W-1) copies of the buffer: right for the small per-step buffers
    # (latency of one hop). Larger ones (whole models: the plain all-reduce aggregator, the
    # un-compressed warm-up phase) go two-shot: reduce-scatter + all-gather through peer stores,
    # 2 (W-1)/W copies. Beyond the arena limit the library ring takes over (eager only).
    ONE_SHOT_LIMIT_FLOATS = 1 << 18
    P2P_ARENA_LIMIT_BYTES = 8 << 30

    def __init__(self):
        self.lib = native.lib()
        self._key = None
        self.launches = 0
        self.comm = None
        self.path = "local"
        self.n_pad = 0
        self._bulk_layout = None
        self._pushed = False  # one-shot path: this step's pack + push already left with another launch
        self._keep_inputs = False
        self._nvls = None     # in-switch all-reduce object (parallel/nvls.py)
        self._nvls_failed = False

    def check(self) -> None:
        """Raise `PowerSGDCommTimeout` if a bounded wait of an earlier launch gave up."""
        if self.comm is not None:
            self.comm.check()
        if self._nvls is not None:
            self._nvls.check()

    def _bind(self, grads, params=None, moms=None, hyper_index=None, need_out=True, outs=None):
        key = (
            tuple(g.data_ptr() for g in grads),
            None if params is None else tuple(p.data_ptr() for p in params),
            None if moms is None else tuple(0 if m is None else m.data_ptr() for m in moms),
            need_out,
            None if outs is None else tuple(o.data_ptr() for o in outs),
        )
        if key == self._key:
            return
        device = grads[0].device
        # every tensor starts at a multiple of four floats in the flat buffer (16-byte accesses)
        total = sum(-(-g.numel() // 4) * 4 for g in grads)
        self._flat = torch.zeros(total, device=device, dtype=torch.float32)
        self._out = torch.empty(total, device=device, dtype=torch.float32) if (need_out and outs is None) else None
        items = np.zeros(len(grads), dtype=layout.FLAT_DTYPE)
        per_block = self.lib.psgd_flat_block_elems()
        block_item, block_first = [], []
        views, cursor = [], 0
        for i, g in enumerate(grads):
            if not is_dense(g) or g.dtype != torch.float32:
                raise ValueError("native flat all-reduce needs dense float32 tensors")
            for o in ((params[i] if params is not None else None), (moms[i] if moms is not None else None),
                      (outs[i] if outs is not None else None)):
                if o is not None and not same_layout(o, g):
                    raise ValueError("native flat all-reduce needs parameters, momentum buffers and outputs laid out like the gradients")
            it = items[i]
            it["grad"] = g.data_ptr()
            it["param"] = 0 if params is None else params[i].data_ptr()
            it["mom"] = 0 if (moms is None or moms[i] is None) else moms[i].data_ptr()
            if need_out and outs is not None:
                views.append(outs[i])
                it["out"] = outs[i].data_ptr()
            elif need_out:
                v = self._out[cursor : cursor + g.numel()]
                views.append(like_strided(v, g))
                it["out"] = v.data_ptr()
            it["numel"] = g.numel()
            it["flat_off"] = cursor
            it["hyper"] = 0 if hyper_index is None else hyper_index[i]
            for first in range(0, g.numel(), per_block):
                block_item.append(i)
                block_first.append(first)
            cursor += -(-g.numel() // 4) * 4
        pointers = [int(items[name][i]) for name in ("grad", "param", "mom", "out") for i in range(len(grads))]
        self._vec = 1 if all(ptr % 16 == 0 for ptr in pointers) else 0
        self._items_dev = _to_device(items, device)
        self._items_host = items
        self._block_item = _to_device(np.asarray(block_item, dtype=np.int32), device)
        self._block_first = _to_device(np.asarray(block_first, dtype=np.int32), device)
        self._nblocks = len(block_item)
        self._views = views
        self._hyper_dev = _to_device(NativeCompressor._default_hyper(), device)
        self._key = key
        self._choose_path(total, world_size())

    def _choose_path(self, total: int, workers: int) -> None:
        """local | oneshot (flag-in-data words to every peer) | bulk (two-shot, plain floats +
        chunk flags; the flat buffer lives in the symmetric arena; PSGD_B200_FLAT=bulk forces it
        for small buffers too) | nvls (PSGD_B200_FLAT=nvls: in-switch reduction of a buffer bound to
        an NVLink multicast object, for buffers above the one-shot limit) | nccl
        (PSGD_B200_COMM=nccl, or arena too large)."""
        want = os.environ.get("PSGD_B200_FLAT", "auto")
        p2p = workers > 1 and os.environ.get("PSGD_B200_COMM", "p2p") == "p2p"
        self.n_pad = total
        if workers == 1:
            path, cap = "local", 0
        elif not p2p:
            path, cap = "nccl", 0
        elif total <= self.ONE_SHOT_LIMIT_FLOATS and want != "bulk":
            path, cap = "oneshot", total
        elif self._wants_nvls(want, workers) and self._nvls_buffer(total) is not None:
            path, cap = "nvls", 0
            self.n_pad = self._nvls.n_pad
        else:
            unit = workers * int(self.lib.psgd_bulk_chunk_floats())
            self.n_pad = -(-total // unit) * unit
            nbytes = int(self.lib.psgd_bulk_arena_bytes(ctypes.c_longlong(self.n_pad), workers))
            path, cap = "bulk", -(-nbytes // (16 * workers))
        if cap and 2 * workers * cap * 8 > self.P2P_ARENA_LIMIT_BYTES:
            path, cap = "nccl", 0
        # An arena is reused only under the discipline it was written with: flag-in-data words of
        # old epochs never match a new one, but the bulk layout puts its flag tables where another
        # layout had data, so a change of protocol or of the bulk size starts from a zeroed arena.
        bulk_layout = self.n_pad if path == "bulk" else None
        if self.comm is not None and (self.comm.cap < cap or cap == 0 or bulk_layout != self._bulk_layout):
            self.comm.close()
            self.comm = None
        self._bulk_layout = bulk_layout
        if cap and self.comm is None:
            from .parallel.symm import Channel

            self.comm = Channel(cap)
        if path == "bulk":
            # pack writes and unpack reads the arena's data region directly
            self._flat = self.comm.slots.tensor(0, self.n_pad)
        elif path == "nvls":
            self._flat = self._nvls.buffer  # this rank's replica of the multicast-bound buffer
        if path != "nvls" and self._nvls is not None:
            self._nvls.close()
            self._nvls = None
        self.path = path

    @staticmethod
    def _wants_nvls(want: str, workers: int) -> bool:
        """In-switch reduction for buffers above the one-shot limit: always with
        PSGD_B200_FLAT=nvls; by default from four workers on (measured at four GPUs: 10-27 % faster
        than the library all-reduce from 1 MiB to 268 MB, where the two-shot peer-store kernels are
        12-35 % behind it; at two GPUs the peer-store kernels are as fast as either). Setting
        NCCL_NVLS_ENABLE=0 - the switch that keeps the communication library off NVLink multicast -
        keeps this path off too, which is how the failure tests run."""
        if want == "nvls":
            return True
        return want == "auto" and workers >= 4 and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"

    def _nvls_buffer(self, total: int):
        """The in-switch all-reduce object for `total` floats, or None when the machine offers no
        NVLink multicast (every rank decides alike; a warning is printed once)."""
        if self._nvls is not None and self._nvls.n_pad >= total:
            return self._nvls
        if self._nvls_failed:
            return None
        from .parallel.nvls import NvlsAllReduce, NvlsUnavailable

        if self._nvls is not None:
            self._nvls.close()
            self._nvls = None
        try:
            self._nvls = NvlsAllReduce(total)
        except NvlsUnavailable as exc:
            import warnings

            warnings.warn(f"in-switch all-reduce not available ({exc}); using the peer-store kernels")
            self._nvls, self._nvls_failed = None, True
        return self._nvls

    def _launch(self, mode: int, hyper_dev: torch.Tensor, divisor: float) -> None:
        code = self.lib.psgd_flat_launch(
            mode,
            self._vec,
            _ptr(self._items_dev),
            _ptr(self._block_item),
            _ptr(self._block_first),
            self._nblocks,
            _ptr(hyper_dev),
            _ptr(self._flat),
            float(divisor),
            self.comm.ptr if self.comm is not None else ctypes.c_void_p(0),
            ctypes.c_longlong(self.n_pad),
            1 if self._keep_inputs else 0,
            _stream_ptr(),
        )
        native.check(code, "psgd_flat_launch")
        self.launches += 1

    def _run(self, hyper_dev: torch.Tensor, workers: int, sgd: bool) -> None:
        if self.path == "local":
            self._launch(4 if sgd else 3, hyper_dev, 1.0)
        elif self.path == "bulk":
            self._launch(0, hyper_dev, float(workers))
            code = self.lib.psgd_bulk_allreduce_launch(self.comm.ptr, ctypes.c_longlong(self.n_pad), workers, _stream_ptr())
            native.check(code, "psgd_bulk_allreduce_launch")
            self.launches += 2
            self._launch(13 if sgd else 12, hyper_dev, 1.0)
        elif self.path == "nvls":
            self._launch(0, hyper_dev, float(workers))
            self._nvls.all_reduce_()
            self.launches += self._nvls.launches
            self._launch(2 if sgd else 1, hyper_dev, 1.0)
        elif self.path == "oneshot":
            if self._pushed:
                self._pushed = False
            else:
                self._launch(5, hyper_dev, float(workers))
            self._launch(7 if sgd else 6, hyper_dev, 1.0)
        else:
            self._launch(0, hyper_dev, float(workers))
            dist.all_reduce(self._flat)
            self._launch(2 if sgd else 1, hyper_dev, 1.0)

    def aggregate(self, gradients: List[torch.Tensor], outs: Optional[Sequence[torch.Tensor]] = None,
                  keep_inputs: bool = False) -> List[torch.Tensor]:
        """Mean over workers. `outs`: caller-owned destination tensors (default: views of this
        object's buffer, valid until the next call). `keep_inputs`: do not zero the inputs."""
        self.check()
        self.launches = 0
        self._bind(gradients, outs=outs)
        self._keep_inputs = bool(keep_inputs)
        try:
            self._run(self._hyper_dev, world_size(), sgd=False)
        finally:
            self._keep_inputs = False
        return list(self._views)

    def aggregate_and_step(self, gradients, params, moms, hyper_index, hyper_dev) -> None:
        self.check()
        self.launches = 0
        self._bind(gradients, params, moms, hyper_index, need_out=False)
        self._run(hyper_dev, world_size(), sgd=True)

    def close(self) -> None:
        """Release the symmetric arena (collective across ranks)."""
        if self.comm is not None:
            self.comm.close()
            self.comm = None
        if self._nvls is not None:
            self._nvls.close()
            self._nvls = None
        self._key = None
        self._bulk_layout = None


class MultiTensorAccumulate:
    """`dst[i] += src[i]` for two lists of float32 tensors in ONE launch.

    Error feedback keeps the compression residual in `p.grad` and lets autograd accumulate the
    next gradient onto it (powersgd/__init__.py:17-25), which costs one small add kernel per
    parameter. A training step that owns the loop detaches the residuals before backward, lets
    autograd adopt the fresh gradients without arithmetic, and folds them in with this kernel.

    Multi-GPU: the same launch can carry the first half of the flat all-reduce of the uncompressed
    tensors (`push=`): their gradients are scaled, zeroed and pushed into every peer's slots while
    the residuals are folded, so that the data is on its way before the low-rank kernels start."""

    def __init__(self):
        self.lib = native.lib()
        self._key = None

    def __call__(self, dst: Sequence[torch.Tensor], src: Sequence[torch.Tensor], push: "Optional[NativeFlatAllReduce]" = None) -> None:
        key = (tuple(t.data_ptr() for t in dst), tuple(t.data_ptr() for t in src), None if push is None else push._key)
        if key != self._key:
            device = dst[0].device
            per_block = self.lib.psgd_flat_block_elems()
            pushed = [] if push is None else list(np.frombuffer(push._items_host.tobytes(), dtype=layout.FLAT_DTYPE))
            items = np.zeros(len(dst) + len(pushed), dtype=layout.FLAT_DTYPE)
            block_item, block_first = [], []
            for i, (d, s_) in enumerate(zip(dst, src)):
                if not same_layout(d, s_) or d.dtype != torch.float32 or s_.dtype != torch.float32:
                    raise ValueError("accumulate needs float32 tensors of equal shape and layout")
                if not is_dense(d):
                    raise ValueError("accumulate needs dense tensors")
                items[i]["grad"], items[i]["out"], items[i]["numel"] = s_.data_ptr(), d.data_ptr(), d.numel()
                items[i]["op"] = 8
            for j, it in enumerate(pushed):
                items[len(dst) + j] = it
                items[len(dst) + j]["op"] = 5
            for i in range(len(items)):
                for first in range(0, int(items[i]["numel"]), per_block):
                    block_item.append(i)
                    block_first.append(first)
            self._vec = 1 if all(ptr % 16 == 0 for ptr in key[0] + key[1]) else 0
            self._items = _to_device(items, device)
            self._block_item = _to_device(np.asarray(block_item, dtype=np.int32), device)
            self._block_first = _to_device(np.asarray(block_first, dtype=np.int32), device)
            self._nblocks = len(block_item)
            self._hyper = _to_device(NativeCompressor._default_hyper(), device)
            self._key = key
        code = self.lib.psgd_flat_launch(
            8 if push is None else 9, self._vec, _ptr(self._items), _ptr(self._block_item), _ptr(self._block_first),
            self._nblocks, _ptr(self._hyper), ctypes.c_void_p(0), 1.0 if push is None else float(world_size()),
            ctypes.c_void_p(0) if push is None else push.comm.ptr, ctypes.c_longlong(0), 0, _stream_ptr(),
        )
        native.check(code, "psgd_flat_launch")
        if push is not None:
            push._pushed = True


class FusedSGDDriver:
    """Glue between `torch.optim.SGD` and the fused kernels.

    Keeps `optimizer.state[p]["momentum_buffer"]` as the live momentum tensors (so optimizer
    checkpoints stay valid), refreshes a small device table of per-group hyper-parameters
    every step (learning-rate schedules keep working), and follows torch's first-step rule
    that a fresh momentum buffer is the gradient itself.

    The table travels through a ring of pinned host slots, one eager async copy per step, so
    that a step recorded in a CUDA graph reads its hyper-parameters from device memory and
    the host never overwrites a slot that a copy in flight still reads.
    """

    RING = 4

    def __init__(self, agg):
        self.agg = agg
        self.device = agg.device
        self._slots: List[torch.Tensor] = []
        self._slot_events: List[Optional[torch.cuda.Event]] = []
        self._cursor = 0
        self._hyper_dev: Optional[torch.Tensor] = None
        self._cache_key = None
        self._flat_all = NativeFlatAllReduce()
        self._flat_plain = NativeFlatAllReduce()
        self.launches = 0

    def _collect(self, optimizer):
        groups = optimizer.param_groups
        key = (id(optimizer), tuple(len(g["params"]) for g in groups), tuple(float(g["momentum"]) != 0.0 for g in groups))
        fresh_groups = set()
        if key != self._cache_key or any(
            float(g["momentum"]) != 0.0 and optimizer.state[p].get("momentum_buffer") is None
            for g in groups
            for p in g["params"][:1]
        ):
            params, moms, index = [], [], []
            for gi, group in enumerate(groups):
                mu = float(group["momentum"])
                for p in group["params"]:
                    params.append(p)
                    index.append(gi)
                    if mu != 0.0:
                        st = optimizer.state[p]
                        if st.get("momentum_buffer") is None:
                            st["momentum_buffer"] = torch.zeros_like(p)  # preserve_format: laid out like the parameter
                            fresh_groups.add(gi)
                        moms.append(st["momentum_buffer"])
                    else:
                        moms.append(None)
            self._params, self._moms, self._index = params, moms, index
            self._grads = [p.grad.data for p in params]
            self._cache_key = key
        return fresh_groups

    def prepare(self, optimizer) -> None:
        """Host side of a step: momentum buffers, hyper-parameter table, async upload."""
        fresh = self._collect(optimizer)
        groups = optimizer.param_groups
        table = np.zeros(len(groups), dtype=layout.HYPER_DTYPE)
        for gi, group in enumerate(groups):
            mu = float(group["momentum"])
            row = table[gi]
            row["lr"] = group["lr"]
            row["momentum"] = mu
            row["one_minus_dampening"] = 1.0 if gi in fresh else 1.0 - float(group["dampening"])
            row["weight_decay"] = group["weight_decay"]
            row["nesterov"] = 1 if group["nesterov"] else 0
            row["has_momentum"] = 1 if mu != 0.0 else 0
            row["grad_scale"] = 1.0
        nbytes = table.nbytes
        if self._hyper_dev is None or self._hyper_dev.numel() != nbytes:
            self._slots = [torch.empty(nbytes, dtype=torch.uint8).pin_memory() for _ in range(self.RING)]
            self._slot_events = [None] * self.RING
            self._hyper_dev = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        blob = table.tobytes()
        if not fresh and blob == getattr(self, "_last_blob", None):
            return  # nothing changed since the last upload: the device table is already right
        self._last_blob = blob
        i = self._cursor
        self._cursor = (i + 1) % self.RING
        if self._slot_events[i] is not None:
            self._slot_events[i].synchronize()
        self._slots[i].numpy()[:] = table.view(np.uint8).reshape(-1)
        self._hyper_dev.copy_(self._slots[i], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._slot_events[i] = ev

    def check(self) -> None:
        """Raise `PowerSGDCommTimeout` if any bounded device-side wait of an earlier step gave up:
        a peer that stayed away leaves zeros in place of its contribution, so the step that
        follows must not run. Host reads of mapped pinned words only; called every step."""
        core = self.agg._powersgd
        if core._native is not None:
            core._native.check()
        self._flat_all.check()
        self._flat_plain.check()

    def fold(self, accumulate: "MultiTensorAccumulate", dst: Sequence[torch.Tensor], src: Sequence[torch.Tensor]) -> None:
        """`dst[i] += src[i]` (residual + fresh gradient) in one launch which, on several GPUs in
        the compression phase, also packs and pushes the uncompressed tensors' gradients."""
        agg = self.agg
        push = None
        if world_size() > 1 and agg.step_counter >= agg.config.start_compressing_after_num_steps and getattr(self, "_params", None):
            mask = agg.is_compressed_mask
            pick = lambda xs: [x for x, k in zip(xs, mask) if not k]  # noqa: E731
            plain = [p.grad for p in pick(self._params)]
            if plain and all(g is not None for g in plain):
                flat = self._flat_plain
                flat._bind([g.data for g in plain], pick(self._params), pick(self._moms), pick(self._index), need_out=False)
                if flat.path == "oneshot":
                    push = flat
        accumulate(dst, src, push=push)

    def step(self, optimizer, prepared: bool = False) -> None:
        self.check()
        if not prepared:
            self.prepare(optimizer)
        # the gradient tensors may have been replaced since the last step (dropped zero gradients
        # re-created by autograd, a loaded checkpoint): always bind what the parameters hold now
        if any(p.grad.data_ptr() != g.data_ptr() for p, g in zip(self._params, self._grads)):
            self._grads = [p.grad.data for p in self._params]
        agg = self.agg
        hyper_dev, index, params, moms, grads = self._hyper_dev, self._index, self._params, self._moms, self._grads
        if len(grads) != len(agg.is_compressed_mask):
            raise ValueError("optimizer parameters do not match the aggregator's parameter list")
        agg.step_counter += 1
        if agg.step_counter <= agg.config.start_compressing_after_num_steps:
            self._flat_all.aggregate_and_step(grads, params, moms, index, hyper_dev)
            self.launches = self._flat_all.launches
            return
        mask = agg.is_compressed_mask
        pick = lambda xs, keep: [x for x, k in zip(xs, mask) if k == keep]  # noqa: E731
        core = agg._powersgd
        self.launches = 0
        if core.params:
            if core._native is None:
                core._native = NativeCompressor(core)
            core._native.aggregate_and_step(
                pick(grads, True), pick(params, True), pick(moms, True), pick(index, True), hyper_dev
            )
            core.step_counter += 1
            self.launches += core._native.launches
        plain = pick(grads, False)
        if plain:
            # after the low-rank path: a consumer that spins on its peers next to the product
            # kernels (tried as a parallel side-stream branch) cost more than it hid
            self._flat_plain.aggregate_and_step(
                plain, pick(params, False), pick(moms, False), pick(index, False), hyper_dev
            )
            self.launches += self._flat_plain.launches
