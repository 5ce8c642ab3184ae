"""Gradient aggregators: the public contract of the library.

`Aggregator.aggregate(gradients)` returns the (approximate) mean gradient over all workers
and MUTATES its inputs: they are zeroed when nothing was lost, or left holding the local
compression residual, which the next backward pass accumulates onto (error feedback).
Reference behaviour: powersgd/powersgd.py:11-31 (contract, AllReduce), :34-105 (policy
wrapper), :108-275 (compressor core).

Two back ends implement the compressor core:

* "torch"  — device-agnostic batched PyTorch ops; used on CPU (gloo) and as the oracle.
* "native" — the sm_100a kernels driven by `cuda_path.NativeCompressor`; selected
  automatically for CUDA tensors. On a CUDA device a missing native library is an error,
  not a silent fallback (set PSGD_B200_ALLOW_FALLBACK=1 to opt into the torch path).
"""
from __future__ import annotations

import os
from abc import ABC, abstractmethod
from typing import Dict, List, NamedTuple, Optional, Sequence

import torch
import torch.distributed as dist

from .orthogonalization import orthogonalize
from .plan import CompressionPlan, avg_compressed_size, matrix_shape, should_compress
from .utils import allreduce_average, is_dense, is_distributed, pack, same_layout, unpack, world_size


class Aggregator(ABC):
    @abstractmethod
    def aggregate(self, gradients: List[torch.Tensor]) -> List[torch.Tensor]:
        """Return averaged gradients; overwrite the inputs with what was NOT communicated.

        With the native back end the returned tensors are views into an arena that the NEXT call
        overwrites (the reference returns fresh tensors): clone what must outlive a step."""


class Config(NamedTuple):
    rank: int  # width of the low-rank factors
    min_compression_rate: float = 2  # tensors that compress less than this go uncompressed
    num_iters_per_step: int = 1  # half power-iterations per optimizer step
    start_compressing_after_num_steps: int = 100


class BasicConfig(NamedTuple):
    rank: int
    num_iters_per_step: int = 1


def _pick_backend(requested: str, device: torch.device) -> str:
    if requested not in ("auto", "torch", "native"):
        raise ValueError(f"unknown backend {requested!r}")
    if requested == "torch":
        return "torch"
    if device.type != "cuda":
        if requested == "native":
            raise RuntimeError("the native back end needs CUDA tensors")
        return "torch"
    from .ops import native

    if native.available():
        return "native"
    if requested == "native" or os.environ.get("PSGD_B200_ALLOW_FALLBACK", "0") != "1":
        raise RuntimeError(
            "powersgd_b200: CUDA tensors were given but the native sm_100a library is not "
            f"loadable ({native.load_error()}); build it with `python -m powersgd_b200.csrc.build` "
            "or set PSGD_B200_ALLOW_FALLBACK=1 to run the slow PyTorch path"
        )
    return "torch"


class AllReduce(Aggregator):
    """Uncompressed mean of a list of tensors through one flat buffer.

    Outputs are views into the flat buffer; inputs are zeroed (powersgd/powersgd.py:22-31).
    """

    def __init__(self, backend: str = "auto"):
        self._backend_request = backend
        self._native = None

    def aggregate(self, gradients: List[torch.Tensor]) -> List[torch.Tensor]:
        if len(gradients) == 0:
            return []
        device = gradients[0].device
        plain = all(g.dtype == torch.float32 and is_dense(g) for g in gradients)
        if _pick_backend(self._backend_request, device) == "native" and plain:
            from .cuda_path import NativeFlatAllReduce

            if self._native is None:
                self._native = NativeFlatAllReduce()
            return self._native.aggregate(gradients)
        flat, shapes = pack(gradients)
        allreduce_average(flat)
        outputs = unpack(flat, shapes)
        for g in gradients:
            g.zero_()
        return outputs


class PowerSGD(Aggregator):
    """Policy wrapper: plain all-reduce during warm-up, then low-rank compression for the
    tensors that compress well enough and a flat all-reduce for the rest."""

    def __init__(self, params: Sequence[torch.Tensor], config: Config, backend: str = "auto"):
        params = list(params)
        self.config = config
        self.device = params[0].device
        self.is_compressed_mask = [should_compress(p.shape, config) for p in params]
        self.step_counter = 0
        self._backend_request = backend
        self._all_numels = [p.numel() for p in params]

        chosen = [p for p, keep in zip(params, self.is_compressed_mask) if keep]
        self._powersgd = BasicPowerSGD(
            chosen,
            config=BasicConfig(rank=config.rank, num_iters_per_step=config.num_iters_per_step),
            backend=backend,
            device=self.device,
            dtype=params[0].dtype,
        )
        self._allreduce = AllReduce(backend=backend)

    # -- reference-compatible internals -------------------------------------------------
    def _should_compress(self, shape) -> bool:
        return should_compress(shape, self.config)

    def _split(self, items: Sequence):
        picked, rest = [], []
        for item, keep in zip(items, self.is_compressed_mask):
            (picked if keep else rest).append(item)
        return picked, rest

    def _merge(self, compressed: List[torch.Tensor], uncompressed: List[torch.Tensor]) -> List[torch.Tensor]:
        if len(compressed) + len(uncompressed) != len(self.is_compressed_mask):
            raise ValueError("gradient list does not match the parameter list given at construction")
        a, b = iter(compressed), iter(uncompressed)
        return [next(a) if keep else next(b) for keep in self.is_compressed_mask]

    # -- public ---------------------------------------------------------------------------
    @property
    def compressing(self) -> bool:
        """Whether the NEXT call to `aggregate` will compress."""
        return self.step_counter >= self.config.start_compressing_after_num_steps

    def aggregate(self, gradients: List[torch.Tensor]) -> List[torch.Tensor]:
        if len(gradients) != len(self.is_compressed_mask):
            raise ValueError("gradient list does not match the parameter list given at construction")
        self.step_counter += 1
        if self.step_counter <= self.config.start_compressing_after_num_steps:
            return self._allreduce.aggregate(gradients)
        lowrank, plain = self._split(gradients)
        return self._merge(self._powersgd.aggregate(lowrank), self._allreduce.aggregate(plain))

    @property
    def compression_rate(self) -> float:
        """Floats in all tensors / floats sent per compressed step (factors + plain tensors)."""
        plain = sum(n for n, keep in zip(self._all_numels, self.is_compressed_mask) if not keep)
        sent = (self._powersgd.compressed_num_floats if self._powersgd.params else 0.0) + plain
        return sum(self._all_numels) / max(sent, 1e-30)

    # -- fused optimizer step (native back end + torch.optim.SGD) ------------------------
    def supports_fused_step(self, optimizer: torch.optim.Optimizer) -> bool:
        if type(optimizer) is not torch.optim.SGD:
            return False
        if _pick_backend(self._backend_request, self.device) != "native":
            return False
        # the fused path never calls optimizer.step(): registered step hooks would not fire
        if getattr(optimizer, "_optimizer_step_pre_hooks", None) or getattr(optimizer, "_optimizer_step_post_hooks", None):
            return False
        for group in optimizer.param_groups:
            if group.get("maximize", False) or group.get("differentiable", False):
                return False
            seen = [("momentum_buffer" in optimizer.state.get(p, {})) and optimizer.state[p]["momentum_buffer"] is not None
                    for p in group["params"]]
            if any(seen) and not all(seen):
                return False
            for p in group["params"]:
                if p.dtype != torch.float32 or p.grad is None or not is_dense(p) or not same_layout(p.grad, p):
                    return False
                buf = optimizer.state.get(p, {}).get("momentum_buffer")
                if buf is not None and not same_layout(buf, p):
                    return False
        return True

    def close(self) -> None:
        """Free multi-GPU resources (peer mappings, symmetric arenas). Call on every rank."""
        native = self._powersgd._native
        if native is not None:
            native.close()
        for flat in (getattr(self._allreduce, "_native", None), getattr(getattr(self, "_fused", None), "_flat_all", None),
                     getattr(getattr(self, "_fused", None), "_flat_plain", None)):
            if flat is not None and flat.comm is not None:
                flat.comm.close()
                flat.comm = None

    def begin_step(self) -> None:
        """Optional hint, called before forward: lets the native back end start the work of the
        coming aggregation that does not depend on the gradients (the first orthonormalisation)
        on a side stream, overlapped with forward and backward. A no-op otherwise."""
        if self.step_counter < self.config.start_compressing_after_num_steps:
            return
        native = self._powersgd._native
        if native is not None and native._key is not None:
            native.begin_step()

    def fused_step(self, optimizer: torch.optim.Optimizer, prepared: bool = False) -> None:
        """Aggregate and apply SGD inside the native kernels: the averaged gradient is never
        written to memory. Numerically the same update as `optimizer_step` with
        `torch.optim.SGD` (weight decay, momentum, dampening, nesterov)."""
        from .cuda_path import FusedSGDDriver

        if getattr(self, "_fused", None) is None:
            self._fused = FusedSGDDriver(self)
        self._fused.step(optimizer, prepared=prepared)
        # what a learning-rate scheduler looks at to tell that the optimizer has stepped
        optimizer._opt_called = True

    def state_dict(self, gradients: Optional[Sequence[torch.Tensor]] = None) -> Dict:
        from .state import aggregator_state_dict

        return aggregator_state_dict(self, gradients)

    def load_state_dict(self, state: Dict, gradients: Optional[Sequence[torch.Tensor]] = None) -> None:
        from .state import load_aggregator_state_dict

        load_aggregator_state_dict(self, state, gradients)


class BasicPowerSGD(Aggregator):
    """Rank-r power-iteration compressor with warm start and error feedback.

    Per call, `num_iters_per_step` half-iterations run; global parity
    `k = step_counter * num_iters_per_step + it` picks the side:

        k even:  P <- orth(P);  Q = M^T P;  M -= P Q^T (local Q);  Q <- sum over workers
        k odd :  Q <- orth(Q);  P = M Q;    M -= P Q^T (local P);  P <- sum over workers

    and every half-iteration adds `P Q^T / W` (with the summed factor) to the output.
    What is left in M is written back into the caller's tensors.
    (powersgd/powersgd.py:146-235.)
    """

    def __init__(
        self,
        params: Sequence[torch.Tensor],
        config: BasicConfig,
        backend: str = "auto",
        device: Optional[torch.device] = None,
        dtype: Optional[torch.dtype] = None,
    ):
        self.config = config
        self.params = list(params)
        self.device = self.params[0].device if self.params else (device or torch.device("cpu"))
        self.dtype = self.params[0].dtype if self.params else (dtype or torch.get_default_dtype())
        self.plan = CompressionPlan.build([p.shape for p in self.params], config.rank)
        self.step_counter = 0
        self._backend_request = backend
        self._native = None

        # Warm-start memory. One seeded generator draws every P group and then every Q group,
        # so replicas that build the object the same way start from identical factors.
        self.generator = torch.Generator(device=self.device).manual_seed(0)
        self._ps_buffer = torch.empty(self.plan.p_total, device=self.device, dtype=self.dtype)
        self._qs_buffer = torch.empty(self.plan.q_total, device=self.device, dtype=self.dtype)
        self._ps = [
            self._ps_buffer[g.p_offset : g.p_offset + g.p_numel].view(g.batch, g.n, g.r) for g in self.plan.groups
        ]
        self._qs = [
            self._qs_buffer[g.q_offset : g.q_offset + g.q_numel].view(g.batch, g.m, g.r) for g in self.plan.groups
        ]
        for view in self._ps + self._qs:
            view.copy_(torch.randn(view.shape, generator=self.generator, device=self.device, dtype=self.dtype))

    # dict keyed by 2-D shape -> list of matrix views, as the reference exposes it
    @property
    def params_per_shape(self) -> Dict[torch.Size, List[torch.Tensor]]:
        return self._matrices_per_shape(self.params)

    @staticmethod
    def _matrices_per_shape(tensors: Sequence[torch.Tensor]) -> Dict[torch.Size, List[torch.Tensor]]:
        out: Dict[torch.Size, List[torch.Tensor]] = {}
        for t in tensors:
            mat = view_as_matrix(t)
            out.setdefault(mat.shape, []).append(mat)
        return out

    @property
    def backend(self) -> str:
        return _pick_backend(self._backend_request, self.device)

    def aggregate(self, gradients: List[torch.Tensor]) -> List[torch.Tensor]:
        if len(gradients) != len(self.params):
            raise ValueError("gradient list does not match the compressed parameter list")
        if len(gradients) == 0:
            self.step_counter += 1
            return []
        native_ok = self.dtype == torch.float32 and all(is_dense(g) and g.dtype == torch.float32 for g in gradients)
        if self.backend == "native" and native_ok:
            from .cuda_path import NativeCompressor

            if self._native is None:
                self._native = NativeCompressor(self)
            outputs = self._native.aggregate(gradients)
        else:
            outputs = self._aggregate_torch(gradients)
        self.step_counter += 1
        return outputs

    def close(self) -> None:
        """Free multi-GPU resources of the native back end (symmetric arenas). Call on every rank."""
        if self._native is not None:
            self._native.close()
            self._native = None

    def _aggregate_torch(self, gradients: List[torch.Tensor]) -> List[torch.Tensor]:
        plan, iters = self.plan, self.config.num_iters_per_step
        mats = [view_as_matrix(g) for g in gradients]
        residual = [torch.stack([mats[i] for i in g.members]) for g in plan.groups]
        approx = [torch.zeros_like(r) for r in residual]
        workers = world_size()

        for it in range(iters):
            left_side = (self.step_counter * iters + it) % 2 == 0
            basis, fresh = (self._ps, self._qs) if left_side else (self._qs, self._ps)
            fresh_flat = self._qs_buffer if left_side else self._ps_buffer
            for M, b, f in zip(residual, basis, fresh):
                orthogonalize(b)
                torch.bmm(M.transpose(1, 2) if left_side else M, b, out=f)
            for M, b, f in zip(residual, basis, fresh):
                # deflate with the LOCAL fresh factor (before it is summed over workers)
                if left_side:
                    M.baddbmm_(b, f.transpose(1, 2), alpha=-1.0)
                else:
                    M.baddbmm_(f, b.transpose(1, 2), alpha=-1.0)
            if is_distributed():
                dist.all_reduce(fresh_flat)
            for A, b, f in zip(approx, basis, fresh):
                if left_side:
                    A.baddbmm_(b, f.transpose(1, 2), alpha=1.0 / workers)
                else:
                    A.baddbmm_(f, b.transpose(1, 2), alpha=1.0 / workers)

        outputs = [torch.empty_like(g) for g in gradients]
        for g, A, M in zip(plan.groups, approx, residual):
            for pos, idx in enumerate(g.members):
                view_as_matrix(outputs[idx]).copy_(A[pos])
                mats[idx].copy_(M[pos])
        return outputs

    # -- statistics (powersgd/powersgd.py:265-275) ----------------------------------------
    @property
    def uncompressed_num_floats(self) -> int:
        return sum(p.shape.numel() for p in self.params)

    @property
    def compressed_num_floats(self) -> float:
        return sum(avg_compressed_size(p.shape, self.config) for p in self.params)

    @property
    def compression_rate(self) -> float:
        return self.uncompressed_num_floats / self.compressed_num_floats


def batch_transpose(batch_of_matrices: torch.Tensor) -> torch.Tensor:
    return batch_of_matrices.transpose(1, 2)


def view_as_matrix(tensor: torch.Tensor) -> torch.Tensor:
    """[out features, everything else]; convolution kernels fold into the input features."""
    n, m = matrix_shape(tensor.shape)
    if not tensor.is_contiguous() and is_dense(tensor):
        # channels_last convolution weight: the same memory as a row-major matrix (its columns
        # are a fixed permutation of the contiguous layout's, which the algorithm does not care about)
        return tensor.as_strided((n, m), (m, 1))
    return tensor.view(n, m)
