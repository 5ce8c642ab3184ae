"""Small helpers shared by the aggregators, the reducers and the training loops.

Covers the helper surface of the reference library (powersgd/utils.py:6-49): flat packing
of tensor lists, optimizer parameter listing, the "is a process group up" probe and the
divide-then-sum averaging all-reduce.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Iterable, List, Sequence, Tuple

import torch
import torch.distributed as dist

from .mean_accumulator import MeanAccumulator
from .tensor_buffer import TensorBuffer, n_bits
from .timer import DeviceTimer, Timer

__all__ = [
    "pack",
    "unpack",
    "params_in_optimizer",
    "is_distributed",
    "flatten",
    "allreduce_average",
    "world_size",
    "rank",
    "TensorBuffer",
    "n_bits",
    "Timer",
    "DeviceTimer",
    "MeanAccumulator",
    "is_dense",
    "like_strided",
    "same_layout",
]


def is_distributed() -> bool:
    """True when torch.distributed has an initialised default process group."""
    return dist.is_available() and dist.is_initialized()


def world_size() -> int:
    return dist.get_world_size() if is_distributed() else 1


def rank() -> int:
    return dist.get_rank() if is_distributed() else 0


def pack(tensors: Sequence[torch.Tensor]) -> Tuple[torch.Tensor, List[torch.Size]]:
    """Copy `tensors` back to back into one new 1-D buffer; also return their shapes."""
    shapes = [t.shape for t in tensors]
    total = sum(s.numel() for s in shapes)
    first = tensors[0]
    flat = torch.empty(total, dtype=first.dtype, device=first.device)
    cursor = 0
    for t in tensors:
        n = t.numel()
        flat[cursor : cursor + n].copy_(t.reshape(-1))
        cursor += n
    return flat, shapes


def unpack(buffer: torch.Tensor, shapes: Sequence[torch.Size]) -> List[torch.Tensor]:
    """Views into `buffer`, one per entry of `shapes`, laid out back to back."""
    views, cursor = [], 0
    for shape in shapes:
        n = torch.Size(shape).numel()
        views.append(buffer[cursor : cursor + n].view(shape))
        cursor += n
    return views


def params_in_optimizer(optimizer: torch.optim.Optimizer) -> List[torch.Tensor]:
    """All parameters of all parameter groups, in group order."""
    return [p for group in optimizer.param_groups for p in group["params"]]


def flatten(nested: Iterable[Iterable[torch.Tensor]]) -> List[torch.Tensor]:
    """Concatenate a list of lists into one list."""
    return [t for inner in nested for t in inner]


def allreduce_average(data: torch.Tensor, *args, **kwargs):
    """In-place mean over workers: scale by 1/W first, then SUM all-reduce.

    The scale-before-sum order is the reference's (powersgd/utils.py:43-49) and is kept so
    that results are bit-compatible. Without a process group this is a no-op that returns
    an object with a `wait()` method, like an async work handle.
    """
    if not is_distributed():
        return SimpleNamespace(wait=lambda: None)
    data.div_(dist.get_world_size())
    return dist.all_reduce(data, *args, **kwargs)


def is_dense(t: torch.Tensor) -> bool:
    """The tensor's memory is one gap-free block whose first dimension is outermost: contiguous, or
    a 4-D channels_last tensor (convolution weights stored [out, kh, kw, in]). Such a tensor is a
    row-major [shape[0], numel / shape[0]] matrix in memory, which is all the kernels need; for
    channels_last the matrix columns are a fixed permutation of the contiguous ones, which
    PowerSGD is indifferent to."""
    return t.is_contiguous() or (t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last))


def same_layout(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Same shape and the same element order in memory (strides of size-1 dimensions are
    arbitrary, e.g. a 1x1 convolution weight reports different strides per memory format)."""
    if a.shape != b.shape:
        return False
    return all(n == 1 or sa == sb for n, sa, sb in zip(a.shape, a.stride(), b.stride()))


def like_strided(flat_view: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """View a flat run of `like.numel()` elements with the shape and strides of the dense `like`."""
    return flat_view.as_strided(like.shape, like.stride())

