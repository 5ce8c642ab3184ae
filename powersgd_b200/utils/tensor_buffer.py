"""Flat staging buffer for lists of tensors (paper-code/gradient_reducers.py:1123-1180)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def n_bits(tensor: torch.Tensor) -> int:
    """Bits occupied by a tensor's payload."""
    return 8 * tensor.nelement() * tensor.element_size()


def _dist_world() -> int:
    return dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1


class TensorBuffer:
    """Concatenates tensors into one 1-D `buffer`; indexing gives shaped views into it.

    `buffer` is a plain attribute and may be swapped for another flat tensor of the same
    length (the sign/Atomo reducers decode other workers' payloads that way).
    """

    def __init__(self, tensors: Sequence[torch.Tensor]):
        self._tensors = list(tensors)
        sizes = [t.nelement() for t in self._tensors]
        ends, acc = [], 0
        for s in sizes:
            acc += s
            ends.append(acc)
        self._end_idx = ends
        self._start_idx = [e - s for e, s in zip(ends, sizes)]
        if self._tensors:
            self.buffer = torch.cat([t.reshape(-1) for t in self._tensors])
        else:
            self.buffer = torch.empty(0)

    def __len__(self) -> int:
        return len(self._tensors)

    def __getitem__(self, index: int) -> torch.Tensor:
        lo, hi = self._start_idx[index], self._end_idx[index]
        return self.buffer[lo:hi].view(self._tensors[index].shape)

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]

    def pack(self, tensors: Optional[Sequence[torch.Tensor]] = None) -> None:
        source = list(self._tensors if tensors is None else tensors)
        if source:
            # one multi-tensor copy instead of a copy kernel per tensor (62 for ResNet-18)
            torch._foreach_copy_([self[i] for i in range(len(source))], source)

    def unpack(self, tensors: Sequence[torch.Tensor]) -> None:
        tensors = list(tensors)
        if tensors:
            torch._foreach_copy_(tensors, [self[i] for i in range(len(tensors))])

    def nelement(self) -> int:
        return self.buffer.nelement()

    def element_size(self) -> int:
        return self.buffer.element_size()

    def bits(self) -> int:
        return 8 * self.nelement() * self.element_size()

    def all_reduce(self, async_op: bool = False):
        """SUM all-reduce of the flat buffer; no-op handle when there is one worker."""
        if _dist_world() == 1:
            return _Done()
        handle = dist.all_reduce(self.buffer, async_op=async_op)
        return handle if async_op else _Done()

    def all_gather(self, async_op: bool = False):
        world = _dist_world()
        if world > 1 and not async_op and self.buffer.is_cuda and self.buffer.element_size() == 4:
            import os

            if os.environ.get("PSGD_B200_COMM", "p2p") == "p2p":
                from ..ops import native

                if native.use_for_cuda():   # one launch over peer stores instead of the library collective
                    from ..parallel.symm import native_all_gather

                    return native_all_gather(self.buffer)
        outs: List[torch.Tensor] = [torch.empty_like(self.buffer) for _ in range(world)]
        if world == 1:
            outs[0].copy_(self.buffer)
            return (outs, _Done()) if async_op else outs
        handle = dist.all_gather(outs, self.buffer, async_op=async_op)
        return (outs, handle) if async_op else outs


class _Done:
    def wait(self) -> None:
        return None
