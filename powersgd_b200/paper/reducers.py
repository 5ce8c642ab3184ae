"""Gradient reducers of the research harness.

Every reducer has the contract of paper-code/gradient_reducers.py:16-34:

    reducer = SomeReducer(random_seed, device, timer, **options)
    bits = reducer.reduce(grad_in, grad_out, memory_out)

`grad_in` holds each worker's (gradient + carried error), `grad_out` receives the aggregate
that every worker applies, `memory_out` receives what this worker failed to communicate
(error feedback), and the return value is the number of bits this worker sent.

All randomness that must agree between workers comes from a `numpy.random.RandomState`
seeded identically everywhere. Unlike the original base class no 512 MB table of random
numbers is allocated (it was never read).

Reducers, with the reference lines they restate:
  ExactReducer (:959-978), RankKReducer (:665-788), HalfRankKReducer (:794-936),
  SVDReducer (:584-661), AtomoReducer (:981-1093), TopKReducer (:209-279),
  GlobalTopKReducer (:282-349), UniformRandomSparseBlockReducer (:352-410),
  UniformRandomSparseReducer (:413-456), RandomSparseBlockReducer (:459-526),
  RandomSparseReducer (:529-581), SignAndNormReducer (:37-105), SignReducer (:108-157),
  SignSGDwithMajorityVoteReducer (:160-207).
"""
from __future__ import annotations

import os
from typing import List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..orthogonalization import gram_schmidt_
from ..ops import signpack
from ..ops.svd import svd_many
from ..ops.topk import sparse_combine, topk_abs, topk_abs_many
from ..utils import TensorBuffer, n_bits
from ..utils.timer import Timer


def _world() -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def all_reduce(tensor: torch.Tensor, async_op: bool = False):
    """SUM all-reduce that is a no-op with one worker."""
    if _world()[0] > 1:
        return dist.all_reduce(tensor, async_op=async_op)
    return None


def all_gather(out_list: List[torch.Tensor], tensor: torch.Tensor, async_op: bool = False):
    if _world()[0] > 1:
        return dist.all_gather(out_list, tensor, async_op=async_op)
    assert len(out_list) == 1
    out_list[0].copy_(tensor)
    return None


def _wait(handle) -> None:
    if handle is not None and hasattr(handle, "wait"):
        handle.wait()


def _gather_all(tensor: torch.Tensor, workers: int) -> List[torch.Tensor]:
    """Every worker's `tensor` (same shape everywhere). CUDA tensors of 4-byte elements travel
    through this package's in-kernel all-gather (peer stores, one launch); PSGD_B200_COMM=nccl or
    anything else goes through the library collective."""
    if workers == 1:
        return [tensor]
    if tensor.is_cuda and tensor.element_size() == 4 and os.environ.get("PSGD_B200_COMM", "p2p") == "p2p":
        from ..ops import native

        if native.use_for_cuda():
            from ..parallel.symm import native_all_gather

            return native_all_gather(tensor)
    outs = [torch.empty_like(tensor) for _ in range(workers)]
    dist.all_gather(outs, tensor)
    return outs


def _rows(gathered: List[torch.Tensor]) -> torch.Tensor:
    """[workers, K] tensor over the per-worker results of `_gather_all` (no copy when they already
    are the rows of one gathered buffer, as the in-kernel all-gather returns them)."""
    first = gathered[0]
    base = first._base if first._base is not None else None
    if base is not None and base.dim() == 2 and base.shape == (len(gathered), first.numel()) and all(
        g._base is base and g.data_ptr() == base.data_ptr() + r * first.numel() * first.element_size() for r, g in enumerate(gathered)
    ):
        return base
    return torch.stack([g.reshape(-1) for g in gathered])


def _sum_all(tensor: torch.Tensor, workers: int) -> None:
    """In-place SUM over workers. Small float32 CUDA messages (up to 2^18 floats) go through this
    package's one-launch in-kernel all-reduce; PSGD_B200_COMM=nccl, larger or other messages go
    through the library collective."""
    if workers == 1:
        return
    if (tensor.is_cuda and tensor.dtype == torch.float32 and tensor.is_contiguous() and tensor.nelement() <= (1 << 18)
            and os.environ.get("PSGD_B200_COMM", "p2p") == "p2p"):
        from ..ops import native

        if native.use_for_cuda():
            from ..parallel.symm import native_all_reduce_

            native_all_reduce_(tensor)
            return
    dist.all_reduce(tensor)


def reduce_mean_list(device, list_in: Sequence[torch.Tensor], list_out: Sequence[torch.Tensor], timer) -> int:
    """Mean over workers of a list of tensors through one flat buffer. Returns bits sent
    (0 with a single worker, where the inputs are simply copied)."""
    workers, _ = _world()
    if workers == 1:
        for src, dst in zip(list_in, list_out):
            dst.copy_(src)
        return 0
    with timer("reduce.mean.pack"):
        flat = TensorBuffer(list_in)
    with timer("reduce.mean.allreduce"):
        flat.all_reduce()
        flat.buffer /= workers
    with timer("reduce.mean.unpack", verbosity=2):
        flat.unpack(list_out)
    return flat.bits()


def l2norm(x: torch.Tensor) -> torch.Tensor:
    return torch.sqrt(torch.sum(x * x))


orthogonalize = gram_schmidt_  # the harness' name for its Gram-Schmidt


def _as_matrix(t: torch.Tensor) -> torch.Tensor:
    return t.view(t.shape[0], -1)


def _split_by_dim(grad_in, grad_out, memory_out):
    vectors, matrices = [], []
    for trio in zip(grad_in, grad_out, memory_out):
        (vectors if trio[0].ndimension() <= 1 else matrices).append(trio)
    return vectors, matrices


class Reducer:
    def __init__(self, random_seed, device, timer=None):
        self.rng = np.random.RandomState(random_seed)
        self.n_workers, self.rank = _world()
        self.device = device
        self.timer = timer if timer is not None else Timer(verbosity_level=0)

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        raise NotImplementedError


def _native_ok(grad_in, grad_out, memory_out) -> bool:
    """CUDA float32 dense tensors throughout: the reducers below then run on the native kernels."""
    from . import native_lowrank

    return native_lowrank.usable(list(grad_in) + list(grad_out) + list(memory_out))


class ExactReducer(Reducer):
    """Plain averaging; nothing is lost, so the memories are cleared. On CUDA tensors the mean
    runs through this package's peer-store all-reduce kernels (pack with 1/W, one-shot or
    two-shot exchange, unpack straight into `grad_out`)."""

    _native = None

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        with self.timer("reduce.zero_mem", verbosity=2):
            if memory_out and memory_out[0].is_cuda:
                torch._foreach_zero_(list(memory_out))
            else:
                for mem in memory_out:
                    mem.zero_()
        with self.timer("reduce.reduce", verbosity=2):
            if _native_ok(grad_in, grad_out, memory_out):
                from ..cuda_path import NativeFlatAllReduce

                if self._native is None:
                    self._native = NativeFlatAllReduce()
                self._native.aggregate(list(grad_in), outs=list(grad_out), keep_inputs=True)
                return 0 if self.n_workers == 1 else 8 * sum(t.nelement() * t.element_size() for t in grad_in)
            return reduce_mean_list(self.device, grad_in, grad_out, self.timer)


class _LowRankBase(Reducer):
    """Shared storage logic of the two power-iteration reducers: flat p / q memories with one
    [n, r] / [m, r] view per matrix-shaped tensor, r = min(n, m, rank), no shape batching."""

    def __init__(self, random_seed, device, timer=None, rank=1):
        super().__init__(random_seed, device, timer)
        self.rank = rank  # note: shadows the worker rank, as the original does
        self.p_memory = None
        self.q_memory = None
        self._native = None              # native_lowrank.NativeLowRank once CUDA tensors were seen
        self._native_launches_last = 0   # kernels launched by the last native reduce()

    def _native_driver(self, matrices, iters: int):
        """Driver of the native path; its factor memories become `p_memory` / `q_memory` (same
        layout as the original: tensor after tensor)."""
        from .native_lowrank import NativeLowRank

        fresh = self._native is None
        if fresh:
            self._native = NativeLowRank(matrices, self.rank, iters, self.device)
            self.p_memory, self.q_memory = self._native.p_memory, self._native.q_memory
        self._native.launches = 0
        return self._native, fresh

    def _rank1_bits(self, vectors) -> int:
        return 8 * sum(t.nelement() * t.element_size() for t, _, _ in vectors)

    def _views(self, matrices):
        sizes = []
        for tensor, _, _ in matrices:
            n, m = _as_matrix(tensor).shape
            sizes.append((n, m, min(n, m, self.rank)))
        fresh = self.p_memory is None
        if fresh:
            self.p_memory = torch.empty(sum(n * r for n, _, r in sizes), device=self.device)
            self.q_memory = torch.empty(sum(m * r for _, m, r in sizes), device=self.device)
        ps, qs, pc, qc = [], [], 0, 0
        for n, m, r in sizes:
            ps.append(self.p_memory[pc : pc + n * r].view(n, r))
            qs.append(self.q_memory[qc : qc + m * r].view(m, r))
            pc += n * r
            qc += m * r
        return ps, qs, fresh

    def _shared_randn_(self, target: torch.Tensor) -> None:
        # every worker seeds torch from the shared numpy stream, so all draw the same matrix
        torch.manual_seed(int(self.rng.randint(1_000_000_000)))
        target.copy_(torch.randn(*target.shape, device=self.device))


class RankKReducer(_LowRankBase):
    """Algorithm 1 of the paper: p = M q, all-reduce, orthogonalise p, q = M^T p, all-reduce
    (mean), output p q^T. The memory is the error against the GLOBAL approximation."""

    def __init__(self, random_seed, device, timer=None, n_power_iterations=0, reuse_query=False, rank=1):
        super().__init__(random_seed, device, timer, rank)
        assert n_power_iterations == 0
        self.reuse_query = reuse_query

    def set_random(self, vector: torch.Tensor) -> None:
        self._shared_randn_(vector)

    def _reduce_native(self, vectors, matrices) -> int:
        drv, fresh = self._native_driver(matrices, iters=2)
        with self.timer("reduce.prepare.q", verbosity=2):
            if fresh or not self.reuse_query:
                for i in range(len(matrices)):
                    self.set_random(drv.core.q_view(i))
        with self.timer("reduce.rank1", verbosity=2):
            drv.reduce_vectors(vectors)
        with self.timer("reduce.lowrank", verbosity=2):
            drv.rank_k(matrices)
        self._native_launches_last = drv.launches
        return n_bits(self.p_memory) + n_bits(self.q_memory) + self._rank1_bits(vectors)

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        bits = 0
        vectors, matrices = _split_by_dim(grad_in, grad_out, memory_out)
        if matrices and _native_ok(grad_in, grad_out, memory_out):
            return self._reduce_native(vectors, matrices)
        with self.timer("reduce.allocate_memory", verbosity=2):
            ps, qs, fresh = self._views(matrices)
        with self.timer("reduce.prepare.q", verbosity=2):
            if fresh or not self.reuse_query:
                for q in qs:
                    self.set_random(q)  # warm start otherwise: previous q, NOT re-orthogonalised
        with self.timer("reduce.compute.p", verbosity=2):
            for (tensor, _, _), q, p in zip(matrices, qs, ps):
                torch.matmul(_as_matrix(tensor), q, out=p)
        with self.timer("reduce.p", verbosity=2):
            all_reduce(self.p_memory)
            bits += n_bits(self.p_memory)
        with self.timer("reduce.rank1.pack", verbosity=2):
            flat = TensorBuffer([t for t, _, _ in vectors])
        with self.timer("reduce.rank1.all_reduce", verbosity=2):
            handle = flat.all_reduce(async_op=True)  # overlaps with the work below
            bits += flat.bits()
        with self.timer("reduce.normalize.p", verbosity=2):
            for p in ps:
                orthogonalize(p)
        with self.timer("reduce.compute.q", verbosity=2):
            for (tensor, _, _), q, p in zip(matrices, qs, ps):
                torch.matmul(_as_matrix(tensor).t(), p, out=q)
        with self.timer("reduce.q", verbosity=2):
            all_reduce(self.q_memory)
            bits += n_bits(self.q_memory)
            self.q_memory /= self.n_workers
        with self.timer("reduce.outerprod", verbosity=2):
            for (tensor, out, mem), q, p in zip(matrices, qs, ps):
                torch.matmul(p, q.t(), out=_as_matrix(out))
                mem.copy_(tensor - out)
        with self.timer("reduce.rank1.unpack", verbosity=2):
            _wait(handle)
            flat.buffer /= self.n_workers
            flat.unpack([out for _, out, _ in vectors])
        return bits


class HalfRankKReducer(_LowRankBase):
    """One matrix product per step, alternating sides; the warm-start factor is
    orthogonalised each step and the memory is the error against the LOCAL product."""

    def __init__(self, random_seed, device, timer=None, rank=1):
        super().__init__(random_seed, device, timer, rank)
        self.next_operation = "p"

    def set_random(self, vector: torch.Tensor) -> None:
        self._shared_randn_(vector)
        orthogonalize(vector)

    def _reduce_native(self, vectors, matrices) -> int:
        drv, fresh = self._native_driver(matrices, iters=1)
        compute_p = self.next_operation == "p"
        self.next_operation = "q" if compute_p else "p"
        if fresh:
            for i in range(len(matrices)):
                self.set_random(drv.core.q_view(i))
        with self.timer("reduce.rank1", verbosity=2):
            drv.reduce_vectors(vectors)
        with self.timer("reduce.lowrank", verbosity=2):
            drv.half_rank_k(matrices, compute_p)
        self._native_launches_last = drv.launches
        return n_bits(self.p_memory if compute_p else self.q_memory) + self._rank1_bits(vectors)

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        bits = 0
        vectors, matrices = _split_by_dim(grad_in, grad_out, memory_out)
        if matrices and _native_ok(grad_in, grad_out, memory_out):
            return self._reduce_native(vectors, matrices)
        with self.timer("reduce.rank1.pack", verbosity=2):
            flat = TensorBuffer([t for t, _, _ in vectors])
        with self.timer("reduce.rank1.all_reduce", verbosity=2):
            handle = flat.all_reduce(async_op=True)
            bits += flat.bits()
        ps, qs, fresh = self._views(matrices)

        compute_p = self.next_operation == "p"
        self.next_operation = "q" if compute_p else "p"
        side = "p" if compute_p else "q"
        with self.timer(f"reduce.normalize.{'q' if compute_p else 'p'}", verbosity=2):
            for basis in (qs if compute_p else ps):
                if compute_p and fresh:
                    self.set_random(basis)
                else:
                    orthogonalize(basis)
        with self.timer(f"reduce.compute.{side}", verbosity=2):
            for (tensor, _, _), q, p in zip(matrices, qs, ps):
                if compute_p:
                    torch.matmul(_as_matrix(tensor), q, out=p)
                else:
                    torch.matmul(_as_matrix(tensor).t(), p, out=q)
        with self.timer("reduce.fill_memory", verbosity=2):
            for (tensor, _, mem), q, p in zip(matrices, qs, ps):
                mem.copy_((_as_matrix(tensor) - p @ q.t()).view(tensor.shape))
        with self.timer(f"reduce.{side}", verbosity=2):
            fresh_memory = self.p_memory if compute_p else self.q_memory
            all_reduce(fresh_memory)
            bits += n_bits(fresh_memory)
            fresh_memory /= self.n_workers
        with self.timer("reduce.outerprod", verbosity=2):
            for (tensor, out, _), q, p in zip(matrices, qs, ps):
                out.copy_((p @ q.t()).view(tensor.shape))
        with self.timer("reduce.rank1.unpack", verbosity=2):
            _wait(handle)
            flat.buffer /= self.n_workers
            flat.unpack([out for _, out, _ in vectors])
        return bits


class SVDReducer(Reducer):
    """Best rank-r approximation per worker by a full SVD; factors are all-gathered and every
    worker averages all reconstructions."""

    def __init__(self, random_seed, device, timer=None, rank=1):
        super().__init__(random_seed, device, timer)
        self.rank = rank

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        bits = 0
        vectors, matrices = _split_by_dim(grad_in, grad_out, memory_out)
        with self.timer("reduce.rank1.zero_memory", verbosity=2):
            for _, _, mem in vectors:
                mem.zero_()
        with self.timer("reduce.rank1.reduce", verbosity=2):
            bits += reduce_mean_list(self.device, [t for t, _, _ in vectors], [o for _, o, _ in vectors], self.timer)
        for tensor, out, mem in matrices:
            matrix = _as_matrix(tensor)
            r = min(self.rank, *matrix.shape)
            u, s, vh = torch.linalg.svd(matrix, full_matrices=False)
            u, s, v = u[:, :r].contiguous(), s[:r].contiguous(), vh[:r].t().contiguous()
            mem.copy_(tensor)
            _as_matrix(mem).sub_((u * s) @ v.t())
            us, vs, ss = (_gather_all(x, self.n_workers) for x in (u, v, s))
            out.zero_()
            for uu, sv, vv in zip(us, ss, vs):
                _as_matrix(out).add_((uu * sv) @ vv.t(), alpha=1.0 / self.n_workers)
            bits += n_bits(u) + n_bits(s) + n_bits(v)
        return bits


class AtomoReducer(Reducer):
    """ATOMO: unbiased sampling of `rank` singular triplets with probabilities proportional
    to the singular values; no error feedback (memories are poisoned)."""

    POISON = -10_000_000.0

    def __init__(self, random_seed, device, timer=None, rank=1, svd_on_cpu=None):
        super().__init__(random_seed, device, timer)
        self.rank = rank
        # the original always factorised on the CPU; on a CUDA device the batched native kernel
        # is the default here (pass svd_on_cpu=True for the original behaviour)
        self.svd_on_cpu = (torch.device(device).type != "cuda") if svd_on_cpu is None else svd_on_cpu

    @staticmethod
    def reshape_to_2d(tensor: torch.Tensor) -> torch.Tensor:
        if tensor.ndimension() == 1:
            return tensor.view(tensor.shape[0] // 2, -1)
        if all(s == 1 for s in tensor.shape[2:]):
            return tensor.squeeze()
        return tensor.view((tensor.shape[0] * tensor.shape[1]) // 2, -1)

    def probabilities(self, singular_values: torch.Tensor, s=None) -> torch.Tensor:
        budget = self.rank if s is None else s
        mag = singular_values.abs()
        return torch.clamp(budget * mag / mag.sum(), max=1.0)

    def sample_singular_values(self, probabilities: torch.Tensor):
        with self.timer("atomo.sample_singular_values", verbosity=3):
            index = torch.arange(len(probabilities), device=probabilities.device)
            for _ in range(1001):
                keep = probabilities > torch.rand(len(probabilities), device=probabilities.device)
                if int(keep.sum()) == self.rank:
                    return index[keep], probabilities[keep]
            raise Exception("Ran out of attempts")

    def svd(self, matrix: torch.Tensor):
        # the original measured a CPU SVD as fastest for these small matrices and kept it
        src = matrix.cpu() if self.svd_on_cpu else matrix
        u, s, vh = torch.linalg.svd(src, full_matrices=False)
        return u.to(self.device), s.to(self.device), vh.t().to(self.device)

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        us, ss, vs = [], [], []
        with self.timer("reduce.encode", verbosity=2):
            views = [self.reshape_to_2d(tensor) for tensor in grad_in]
            if grad_in and grad_in[0].is_cuda and not self.svd_on_cpu:
                factors = svd_many(views)  # narrow matrices: one native launch for all of them
            else:
                factors = [self.svd(m) for m in views]
            for u, s, v in factors:
                pick, probs = self.sample_singular_values(self.probabilities(s))
                us.append(u[:, pick].contiguous())
                vs.append(v[:, pick].contiguous())
                ss.append(s[pick] / probs)
        with self.timer("reduce.pack", verbosity=2):
            packed = TensorBuffer(us + ss + vs)
        with self.timer("reduce.allgather", verbosity=2):
            payloads = packed.all_gather()
            bits = packed.bits()
        with self.timer("reduce.average", verbosity=2):
            for out in grad_out:
                out.zero_()
            k = len(us)
            for payload in payloads:
                packed.buffer = payload
                for i, out in enumerate(grad_out):
                    u, s, v = packed[i], packed[k + i], packed[2 * k + i]
                    out.add_(((u * s) @ v.t()).view(out.shape), alpha=1.0 / self.n_workers)
        with self.timer("reduce.memory", verbosity=2):
            for mem in memory_out:
                mem.fill_(self.POISON)
        return bits


def _top_size(compression: float, numel: int) -> int:
    # half the budget goes to the indices
    return max(1, int(0.5 * compression * numel))


class TopKReducer(Reducer):
    """Per-tensor magnitude top-k; values and int32 positions are all-gathered."""

    def __init__(self, random_seed, device, timer=None, compression=1 / 244):
        super().__init__(random_seed, device, timer)
        self.compression = compression

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        with self.timer("reduce.flatpack", verbosity=2):
            sizes = [_top_size(self.compression, t.nelement()) for t in grad_in]
            ends = np.cumsum(sizes).tolist()
        with self.timer("reduce.topk", verbosity=2):
            # selection, gather and the error-feedback write (memory = x with the taken entries
            # zeroed) are one fused operation over the whole list: four launches on CUDA
            values, positions = topk_abs_many(list(grad_in), sizes, list(memory_out))
        with self.timer("reduce.gather", verbosity=2):
            all_values = _gather_all(values, self.n_workers)
            all_positions = _gather_all(positions, self.n_workers)
            bits = n_bits(values) + n_bits(positions)
        with self.timer("reduce.combine", verbosity=2):
            # zero fill + the scatter of every worker's pairs, in rank order: one launch on CUDA
            sparse_combine(_rows(all_values), _rows(all_positions), grad_out, ends, float(self.n_workers))
        return bits


class GlobalTopKReducer(Reducer):
    """One magnitude top-k over the whole flattened gradient."""

    def __init__(self, random_seed, device, timer=None, compression=1 / 244):
        super().__init__(random_seed, device, timer)
        self.compression = compression

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        with self.timer("reduce.flatpack"):
            packed = TensorBuffer(grad_in)
            flat = packed.buffer
            k = _top_size(self.compression, flat.nelement())
        with self.timer("reduce.topk", verbosity=2):
            residual = torch.empty_like(flat)
            values, positions = topk_abs(flat, k, memory=residual)
        with self.timer("reduce.set_memory", verbosity=2):
            packed.buffer = residual
            packed.unpack(memory_out)
        with self.timer("reduce.reduce", verbosity=2):
            all_values = _gather_all(values, self.n_workers)
            all_positions = _gather_all(positions, self.n_workers)
            # positions travel as int32 here; the count keeps the original's int64 convention
            # (gradient_reducers.py:326-331) so that reported volumes stay comparable
            bits = n_bits(values) + 64 * positions.nelement()
        with self.timer("reduce.combine", verbosity=2):
            total = torch.empty_like(flat)
            sparse_combine(_rows(all_values), _rows(all_positions), [total], [k], float(self.n_workers))
            packed.buffer = total
            packed.unpack(grad_out)
        return bits


class _SparseBase(Reducer):
    """Shared machinery of the four random-sparsification reducers: pick positions with the
    shared RNG, all-reduce the picked values, scatter the mean back."""

    def _budget(self, tensor: torch.Tensor) -> int:
        raise NotImplementedError

    def _pick(self, tensor: torch.Tensor, budget: int):
        raise NotImplementedError

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        """The original works tensor by tensor (a gather, a copy, an indexed store, a zero fill and a
        scatter per tensor, gradient_reducers.py:350-581). Here the per-tensor picks - drawn in the
        same order from the shared stream - become ONE index into the flat gradient, so a step is a
        gather, an indexed zero, an all-reduce, a scatter and two multi-tensor unpacks."""
        grad_in = list(grad_in)
        with self.timer("reduce.block", verbosity=2):
            index = self._pick_all(grad_in)
        with self.timer("reduce.flatpack", verbosity=2):
            packed = TensorBuffer(grad_in)
            flat = packed.buffer
            values = flat[index]
        with self.timer("reduce.memory", verbosity=2):
            flat[index] = 0.0   # `flat` is a copy of the gradients: what is left is the memory
            packed.unpack(memory_out)
        with self.timer("reduce.reduce", verbosity=2):
            _sum_all(values, self.n_workers)
            values /= self.n_workers
            bits = n_bits(values)
        with self.timer("reduce.combine", verbosity=2):
            flat.zero_()
            flat[index] = values
            packed.unpack(grad_out)
        return bits


    def _pick_all(self, grad_in) -> torch.Tensor:
        """Positions of every tensor's picks in the flat gradient (tensor after tensor)."""
        picks, offset = [], 0
        for t in grad_in:
            picks.append(self._pick(t, self._budget(t)) + offset)
            offset += t.nelement()
        return torch.cat(picks)


class _BlockPick:
    def _pick(self, tensor: torch.Tensor, budget: int):
        numel = tensor.nelement()
        start = 0 if budget == numel and self._full_block_starts_at_zero else int(self.rng.choice(numel))
        return (torch.arange(budget, device=tensor.device) + start) % numel  # wraps around the end

    _layout_key = None

    def _pick_all(self, grad_in) -> torch.Tensor:
        """All blocks at once: the start of every block is drawn on the host in tensor order (the
        same draws as `_pick`), everything else is a handful of element-wise kernels over cached
        per-pick tables instead of three small kernels per tensor."""
        numels = [t.nelement() for t in grad_in]
        budgets = [self._budget(t) for t in grad_in]
        device = grad_in[0].device
        key = (tuple(numels), tuple(budgets), device)
        if key != self._layout_key:
            count = torch.tensor(budgets, device=device)
            owner = torch.repeat_interleave(torch.arange(len(grad_in), device=device), count)
            first = torch.cumsum(count, 0) - count
            self._within = torch.arange(int(sum(budgets)), device=device) - first[owner]
            numel_t = torch.tensor(numels, device=device)
            self._numel_of = numel_t[owner]
            self._offset_of = (torch.cumsum(numel_t, 0) - numel_t)[owner]
            self._owner = owner
            self._layout_key = key
        starts = [0 if (b == n and self._full_block_starts_at_zero) else int(self.rng.choice(n)) for n, b in zip(numels, budgets)]
        start_of = torch.tensor(starts, device=device)[self._owner]
        return (self._within + start_of) % self._numel_of + self._offset_of


class _ScatterPick:
    def _pick(self, tensor: torch.Tensor, budget: int):
        numel = tensor.nelement()
        if budget == numel and self._full_block_starts_at_zero:
            idx = np.arange(numel)
        else:
            idx = self.rng.choice(numel, budget, replace=False)
        return torch.from_numpy(np.asarray(idx)).long().to(tensor.device)


class _CompressionBudget(_SparseBase):
    _full_block_starts_at_zero = False

    def __init__(self, random_seed, device, timer=None, compression=1 / 244):
        super().__init__(random_seed, device, timer)
        self.compression = compression

    def _budget(self, tensor):
        return max(1, int(self.compression * tensor.nelement()))


class _RankBudget(_SparseBase):
    _full_block_starts_at_zero = True

    def __init__(self, random_seed, device, timer=None, rank=1):
        super().__init__(random_seed, device, timer)
        self.rank = rank

    def block_size(self, tensor):
        n, m = _as_matrix(tensor).shape
        return min(self.rank * (n + m), tensor.nelement())

    _budget = block_size


class UniformRandomSparseBlockReducer(_BlockPick, _CompressionBudget):
    """A contiguous (wrapping) block of `compression * numel` entries at a shared random start."""


class UniformRandomSparseReducer(_ScatterPick, _CompressionBudget):
    """`compression * numel` entries at shared random positions."""


class RandomSparseBlockReducer(_BlockPick, _RankBudget):
    """A contiguous block with the same float budget as a rank-`rank` factorisation."""


class RandomSparseReducer(_ScatterPick, _RankBudget):
    """Random positions with the same float budget as a rank-`rank` factorisation."""


class SignCompressor:
    """One bit per entry: sign -> 32 signs per int32 word (row i of the [32, L] sign matrix
    goes to bit 31 - i), and back. The packing kernels are native (ops/signpack)."""

    def compress(self, src: torch.Tensor):
        return signpack.pack_signs(src), src.size()

    def uncompress(self, words: torch.Tensor, size) -> torch.Tensor:
        return signpack.unpack_signs(words, torch.Size(size).numel()).view(size)

    packing = compress
    unpacking = uncompress

    def majority_vote(self, words_list: Sequence[torch.Tensor]) -> torch.Tensor:
        return signpack.majority_vote(torch.stack(list(words_list)))


class _SignBase(Reducer):
    def _exchange(self, grad_in):
        with self.timer("reduce.flatpack"):
            packed = TensorBuffer(grad_in)
        with self.timer("reduce.compress", verbosity=2):
            words, size = SignCompressor().compress(packed.buffer)
        with self.timer("reduce.gather", verbosity=2):
            gathered = _gather_all(words, self.n_workers)
        return packed, words, size, gathered


class SignAndNormReducer(_SignBase):
    """Signs scaled by each tensor's mean absolute value; memory = x - mean|x| sign(x).

    Same arithmetic as gradient_reducers.py:37-106, arranged on the flat buffer: the per-tensor
    scales stay on the device and are spread over their tensors' elements with one gather through a
    cached element-to-tensor index, so a step has no host synchronisation and no per-tensor kernels (the
    original reads every norm back with `.item()` and issues three kernels per tensor and worker)."""

    _owner_key = None

    def _element_owner(self, grad_in, device):
        """(index of the tensor every element of the flat buffer belongs to, 1 / numel per tensor);
        built once per tensor list."""
        key = (tuple(t.nelement() for t in grad_in), device)
        if key != self._owner_key:
            numels = torch.tensor(key[0], device=device)
            self._owner = torch.repeat_interleave(torch.arange(len(grad_in), device=device, dtype=torch.int32), numels)
            self._per_element = 1.0 / numels.to(torch.float32)
            self._owner_key = key
        return self._owner, self._per_element

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        grad_in = list(grad_in)
        with self.timer("reduce.norms", verbosity=2):
            norms = torch.stack(torch._foreach_norm(grad_in, 1))
        packed, words, size, gathered = self._exchange(grad_in)
        all_norms = _gather_all(norms, self.n_workers)
        bits = n_bits(words) + n_bits(norms)
        owner, per_element = self._element_owner(grad_in, norms.device)
        with self.timer("reduce.average", verbosity=2):
            comp = SignCompressor()
            mean = torch.zeros_like(packed.buffer)
            for their_words, their_norms in zip(gathered, all_norms):
                scale = torch.index_select(their_norms * per_element / self.n_workers, 0, owner)
                mean.addcmul_(comp.uncompress(their_words, size).view(-1), scale)
        with self.timer("reduce.memory", verbosity=2):
            own = torch.index_select(norms * per_element, 0, owner)
            residual = torch.addcmul(packed.buffer, packed.buffer.sign(), own, value=-1.0)
            packed.buffer = residual
            packed.unpack(memory_out)
        with self.timer("reduce.set_out", verbosity=2):
            packed.buffer = mean
            packed.unpack(grad_out)
        return bits


class SignReducer(_SignBase):
    """Mean of the workers' sign vectors. The memory follows the original, including its
    sign convention (`mem = x + sign(x)`, gradient_reducers.py:153-155)."""

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        packed, words, size, gathered = self._exchange(grad_in)
        bits = n_bits(words)
        with self.timer("reduce.memory", verbosity=2):
            flat = packed.buffer
            packed.buffer = flat + flat.sign()
            packed.unpack(memory_out)
        with self.timer("reduce.average", verbosity=2):
            comp = SignCompressor()
            mean = sum(comp.uncompress(w, size) for w in gathered) / self.n_workers
            packed.buffer = mean
            packed.unpack(grad_out)
        return bits


class SignSGDwithMajorityVoteReducer(_SignBase):
    """signSGD with majority vote: output = sign(sum of sign vectors); no error feedback."""

    def reduce(self, grad_in, grad_out, memory_out) -> int:
        packed, words, size, gathered = self._exchange(grad_in)
        bits = n_bits(words)
        with self.timer("reduce.majorityvote", verbosity=2):
            packed.buffer = signpack.vote_signs(torch.stack(gathered), torch.Size(size).numel())
        with self.timer("reduce.set_out", verbosity=2):
            packed.unpack(grad_out)
        with self.timer("reduce.memory", verbosity=2):
            for mem in memory_out:
                mem.fill_(AtomoReducer.POISON)
        return bits


REDUCERS = {
    cls.__name__: cls
    for cls in (
        ExactReducer, RankKReducer, HalfRankKReducer, SVDReducer, AtomoReducer, TopKReducer, GlobalTopKReducer,
        UniformRandomSparseBlockReducer, UniformRandomSparseReducer, RandomSparseBlockReducer, RandomSparseReducer,
        SignAndNormReducer, SignReducer, SignSGDwithMajorityVoteReducer,
    )
}
