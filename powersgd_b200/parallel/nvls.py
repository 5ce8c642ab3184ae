"""In-switch (NVLink SHARP) all-reduce of a flat float32 buffer: the flat aggregator's path for
buffers above the one-shot limit from four workers on (PSGD_B200_FLAT=nvls forces it, NCCL_NVLS_ENABLE=0
or PSGD_B200_FLAT=bulk keeps it off).

The buffer is allocated and bound to an NVLink multicast object by PyTorch's symmetric-memory
runtime (plumbing: allocation, handle exchange over the process group's store, binding); the
reduction itself is this package's kernel (csrc/nvls.cu: `multimem.ld_reduce` + `multimem.st`,
each rank reducing the slice it owns) with the two cross-rank barriers it needs carried inside the
same launch as bounded token exchanges on an in-kernel channel. The reference all-reduces whole models with NCCL (powersgd/powersgd.py:22-31);
on NVSwitch machines NCCL takes the same in-switch route.

A rank must not disappear while its memory is bound to the multicast object: keep this path out of
failure tests, and call `close()` (collective) before the process group is destroyed.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native


class NvlsUnavailable(RuntimeError):
    """No NVLink multicast on this machine / build (raised on every rank alike)."""


class NvlsAllReduce:
    """In-place SUM all-reduce of `buffer` (float32, this rank's replica of the symmetric buffer).

    Fill `buffer`, call `all_reduce_()` on every rank (one launch on the current stream: barrier,
    in-switch reduction, barrier; recordable in a CUDA graph), read `buffer`."""

    def __init__(self, n_floats: int, group=None):
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) < 2:
            raise NvlsUnavailable("needs an initialised process group of at least two ranks")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.lib = native.lib()
        device = torch.device("cuda", torch.cuda.current_device())
        unit = 4 * self.world
        self.n_pad = -(-int(n_floats) // unit) * unit
        try:
            import torch.distributed._symmetric_memory as symm_mem
            from torch._C._distributed_c10d import _SymmetricMemory

            from torch._C._autograd import DeviceType

            supported = bool(_SymmetricMemory.has_multicast_support(DeviceType.CUDA, device.index))
        except Exception as exc:  # API not in this PyTorch build
            supported, symm_mem = False, None
            reason = f"symmetric-memory runtime not usable: {exc}"
        else:
            reason = "the device reports no NVLink multicast support"
        # every rank takes the same decision
        flags = [None] * self.world
        dist.all_gather_object(flags, bool(supported), group=self.group)
        if not all(flags):
            raise NvlsUnavailable(reason if not supported else "a peer reports no NVLink multicast support")
        self._tensor = symm_mem.empty(self.n_pad, dtype=torch.float32, device=device)
        self._handle = symm_mem.rendezvous(self._tensor, self.group)
        self.mc_ptr = int(self._handle.multicast_ptr)
        ok = [None] * self.world
        dist.all_gather_object(ok, self.mc_ptr != 0 and self.mc_ptr % 16 == 0, group=self.group)
        if not all(ok):
            self._handle = self._tensor = None
            raise NvlsUnavailable("the symmetric-memory runtime returned no multicast address")
        self.buffer = self._tensor[: self.n_pad]
        from .symm import Channel

        self._channel = Channel(1 << 12, self.group)
        self._token = torch.zeros(4, dtype=torch.float32, device=device)
        self._fused = os.environ.get("PSGD_B200_NVLS_FUSED", "1") != "0"

    def all_reduce_(self, max_blocks: int = 0) -> torch.Tensor:
        """`max_blocks`: CTAs of the reduction kernel (0: PSGD_B200_NVLS_BLOCKS, else the library default).
        One launch (barriers inside the kernel); PSGD_B200_NVLS_FUSED=0 selects the three-launch form."""
        if max_blocks <= 0:
            max_blocks = int(os.environ.get("PSGD_B200_NVLS_BLOCKS", "0"))
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        if self._fused:
            native.check(
                self.lib.psgd_nvls_allreduce_fused_launch(self._channel.ptr, ctypes.c_void_p(self.mc_ptr), ctypes.c_longlong(self.n_pad), self.world, int(max_blocks), stream),
                "psgd_nvls_allreduce_fused_launch",
            )
            return self.buffer
        self._channel.all_reduce_(self._token)      # every replica is complete
        native.check(
            self.lib.psgd_nvls_allreduce_launch(ctypes.c_void_p(self.mc_ptr), ctypes.c_longlong(self.n_pad), self.rank, self.world, int(max_blocks), stream),
            "psgd_nvls_allreduce_launch",
        )
        self._channel.all_reduce_(self._token)      # every slice has been written back
        return self.buffer

    @property
    def launches(self) -> int:
        return 1 if self._fused else 3

    def check(self) -> None:
        self._channel.check()

    def close(self) -> None:
        """Collective: waits for the device, lets every rank arrive, then unbinds and frees."""
        if self._tensor is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._channel.close()
        self.buffer = None
        self._handle = None
        self._tensor = None
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
