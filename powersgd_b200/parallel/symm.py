"""Symmetric memory and in-kernel collective channels over NVLink peer mappings.

`Channel` is the host-side handle of one stream of collectives (csrc/psgd_comm.cuh): it
allocates this rank's slot arena (8-byte {value, epoch} words), exchanges CUDA-IPC handles with
the other ranks once (through the existing torch.distributed group — the only use of a library
collective), maps every peer's arena, and uploads the device descriptor that kernels take.

Failure handling: device-side waits are bounded (`timeout_ms`, default from
PSGD_B200_COMM_TIMEOUT_MS or 20 s). A wait that runs out writes a status word in mapped
pinned memory; `check()` turns it into `PowerSGDCommTimeout` on the host without touching
the GPU. The reference has no equivalent (its NCCL all-reduce simply blocks,
powersgd/powersgd.py:205-209).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native

MAX_WORLD = 8


class PowerSGDCommTimeout(RuntimeError):
    """A bounded device-side wait on a peer ran out."""


class PowerSGDConfigMismatch(RuntimeError):
    """The ranks of a job were set up differently (model shapes, rank, iterations per step)."""


def _vp(x: int) -> ctypes.c_void_p:
    return ctypes.c_void_p(int(x))


def assert_same_on_all_ranks(obj, what: str, group=None) -> None:
    """Collective: every rank contributes `obj` (anything picklable and comparable); raises
    `PowerSGDConfigMismatch` on EVERY rank when they differ. Called once when multi-rank state is
    set up, so that a rank with another model or configuration is reported by name instead of
    showing up later as a peer whose data never arrives. Works on any backend (host objects)."""
    if not (dist.is_available() and dist.is_initialized()):
        return
    world = dist.get_world_size(group)
    gathered: List[Optional[object]] = [None] * world
    dist.all_gather_object(gathered, obj, group=group)
    odd = [r for r, other in enumerate(gathered) if other != gathered[0]]
    if odd:
        raise PowerSGDConfigMismatch(
            f"{what} differs between ranks: ranks {odd} disagree with rank 0 "
            f"(this is rank {dist.get_rank(group)})"
        )


class StatusWord:
    """One int in mapped pinned host memory that kernels write (through `dev_ptr`) when a bounded
    wait gives up; the host reads it without touching the GPU."""

    def __init__(self):
        self.lib = native.lib()
        host_ptr, dev_ptr = ctypes.POINTER(ctypes.c_int)(), ctypes.POINTER(ctypes.c_int)()
        native.check(self.lib.psgd_status_alloc(ctypes.byref(host_ptr), ctypes.byref(dev_ptr)), "psgd_status_alloc")
        self._host = host_ptr
        self._dev = ctypes.cast(dev_ptr, ctypes.c_void_p).value

    @property
    def dev_ptr(self) -> ctypes.c_void_p:
        return _vp(self._dev)

    @property
    def value(self) -> int:
        return int(self._host[0]) if self._host else 0

    def set(self, code: int) -> None:
        """Host-side write (tests inject a failure this way; `set(0)` clears)."""
        self._host[0] = int(code)

    def check(self, what: str) -> None:
        code = self.value
        if code != 0:
            raise PowerSGDCommTimeout(f"{what} gave up on the device (status {code})")

    def close(self) -> None:
        if self._host:
            self.lib.psgd_status_free(self._host)
            self._host = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def default_timeout_ms() -> float:
    return float(os.environ.get("PSGD_B200_COMM_TIMEOUT_MS", "20000"))


class SymmetricBuffer:
    """`nbytes` of zeroed device memory on every rank, each rank's copy mapped on all others."""

    def __init__(self, nbytes: int, group=None):
        self.lib = native.lib()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nbytes = int(nbytes)
        local = ctypes.c_void_p()
        native.check(self.lib.psgd_symm_alloc(ctypes.c_size_t(self.nbytes), ctypes.byref(local)), "psgd_symm_alloc")
        self.local = int(local.value)
        hb = self.lib.psgd_symm_handle_bytes()
        handle = (ctypes.c_ubyte * hb)()
        native.check(self.lib.psgd_symm_export(_vp(self.local), handle), "psgd_symm_export")
        gathered: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle), group=group)
        self.ptrs: List[int] = []
        self._imported: List[int] = []
        for r, blob in enumerate(gathered):
            if r == self.rank:
                self.ptrs.append(self.local)
                continue
            buf = (ctypes.c_ubyte * hb).from_buffer_copy(blob)
            mapped = ctypes.c_void_p()
            native.check(self.lib.psgd_symm_import(buf, ctypes.byref(mapped)), "psgd_symm_import")
            self.ptrs.append(int(mapped.value))
            self._imported.append(int(mapped.value))
        dist.barrier(group=group)

    def tensor(self, offset_bytes: int, numel: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """A torch view of this rank's copy (no ownership: it must not outlive `close()`)."""
        itemsize = torch.empty((), dtype=dtype).element_size()
        if offset_bytes % itemsize or offset_bytes + numel * itemsize > self.nbytes:
            raise ValueError("view outside the symmetric buffer")
        typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1"}[dtype]

        class _View:
            __cuda_array_interface__ = {
                "shape": (int(numel),), "typestr": typestr, "data": (self.local + int(offset_bytes), False),
                "version": 2, "strides": None,
            }

        return torch.as_tensor(_View(), device=torch.device("cuda", torch.cuda.current_device()))

    def close(self) -> None:
        if self.local == 0:
            return
        torch.cuda.synchronize()
        for p in self._imported:
            self.lib.psgd_symm_unmap(_vp(p))
        self._imported = []
        if dist.is_initialized():
            try:
                dist.barrier(group=self.group)
            except Exception:
                pass
        self.lib.psgd_symm_free(_vp(self.local))
        self.local = 0


class Channel:
    """One ordered stream of in-kernel collectives with `cap` floats per rank per message."""

    def __init__(self, cap_floats: int, group=None, timeout_ms: Optional[float] = None):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("Channel needs an initialised torch.distributed process group")
        self.lib = native.lib()
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > MAX_WORLD:
            raise ValueError(f"in-kernel collectives support up to {MAX_WORLD} ranks on one NVSwitch domain")
        self.cap = max(int(cap_floats), 1)
        self.timeout_ms = default_timeout_ms() if timeout_ms is None else float(timeout_ms)
        device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.slots = SymmetricBuffer(2 * self.world * self.cap * 8, group)
        # local bookkeeping words: epoch, arrival counters
        self._words = torch.zeros(16, dtype=torch.int32, device=device)
        self._status = StatusWord()
        self._status_dev = self._status._dev
        nbytes = self.lib.psgd_comm_desc_bytes()
        host_desc = (ctypes.c_ubyte * nbytes)()
        slots = (ctypes.c_void_p * self.world)(*self.slots.ptrs)
        base = self._words.data_ptr()
        native.check(
            self.lib.psgd_comm_fill(
                host_desc, self.world, self.rank, slots, _vp(base), _vp(self._status_dev),
                ctypes.c_longlong(self.cap), ctypes.c_double(self.timeout_ms),
            ),
            "psgd_comm_fill",
        )
        self.desc = torch.frombuffer(bytearray(bytes(host_desc)), dtype=torch.uint8).to(device)
        torch.cuda.synchronize()

    @property
    def ptr(self) -> ctypes.c_void_p:
        return _vp(self.desc.data_ptr())

    @property
    def status(self) -> int:
        return self._status.value

    def check(self) -> None:
        code = self.status
        if code != 0:
            raise PowerSGDCommTimeout(
                f"rank {self.rank}: a device-side wait on a peer gave up after {self.timeout_ms:.0f} ms (status {code})"
            )

    def reset_status(self) -> None:
        self._status.set(0)
        self._words[8] = 0

    def all_reduce_(self, tensor: torch.Tensor, scale: float = 1.0, max_blocks: int = 296) -> torch.Tensor:
        """In-place one-launch SUM all-reduce (times `scale`) of a contiguous float32 tensor."""
        if tensor.numel() > self.cap:
            raise ValueError(f"message of {tensor.numel()} floats exceeds the channel capacity {self.cap}")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        native.check(
            self.lib.psgd_allreduce_oneshot_launch(
                self.ptr, _vp(tensor.data_ptr()), _vp(tensor.data_ptr()), ctypes.c_longlong(tensor.numel()),
                ctypes.c_float(scale), max_blocks, stream,
            ),
            "psgd_allreduce_oneshot_launch",
        )
        return tensor

    def all_gather(self, tensor: torch.Tensor, max_blocks: int = 296) -> torch.Tensor:
        """One-launch all-gather of a contiguous tensor of 4-byte elements (same length on every
        rank): returns a [world, numel] tensor of the same dtype, rank r's data in row r."""
        n = tensor.numel()
        if tensor.element_size() != 4 or not tensor.is_contiguous():
            raise ValueError("in-kernel all-gather moves contiguous tensors of 4-byte elements")
        if n > self.cap:
            raise ValueError(f"message of {n} words exceeds the channel capacity {self.cap}")
        out = torch.empty((self.world, n), dtype=tensor.dtype, device=tensor.device)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        native.check(
            self.lib.psgd_allgather_oneshot_launch(self.ptr, _vp(tensor.data_ptr()), _vp(out.data_ptr()), ctypes.c_longlong(n), max_blocks, stream),
            "psgd_allgather_oneshot_launch",
        )
        return out

    def close(self) -> None:
        self.slots.close()
        self._status.close()


class BulkAllReduce:
    """In-place SUM all-reduce of a large float32 buffer that lives in symmetric memory.

    Two-shot over peer stores with plain floats and one epoch flag per 16 KiB chunk
    (csrc/comm_kernels.cu): every rank pushes the slices it does not own to their owners, owners
    add the W contributions in rank order and store the sum into everybody's buffer. Three
    launches, no library collective, recordable in a CUDA graph. Fill `buffer` (a view of this
    rank's arena), call `all_reduce_()`, read `buffer`. The reference uses NCCL's all-reduce for
    this (powersgd/powersgd.py:22-31, paper-code/gradient_reducers.py ExactReducer).
    """

    def __init__(self, numel: int, group=None, timeout_ms: Optional[float] = None):
        lib = native.lib()
        world = dist.get_world_size(group)
        unit = world * int(lib.psgd_bulk_chunk_floats())
        self.numel = int(numel)
        self.n_pad = -(-self.numel // unit) * unit
        nbytes = int(lib.psgd_bulk_arena_bytes(ctypes.c_longlong(self.n_pad), world))
        self.channel = Channel(-(-nbytes // (16 * world)), group, timeout_ms)
        self.world = world
        self.buffer = self.channel.slots.tensor(0, self.n_pad)[: self.numel]

    def all_reduce_(self) -> torch.Tensor:
        ch = self.channel
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        native.check(ch.lib.psgd_bulk_allreduce_launch(ch.ptr, ctypes.c_longlong(self.n_pad), self.world, stream), "psgd_bulk_allreduce_launch")
        native.check(ch.lib.psgd_bulk_finish_launch(ch.ptr, ctypes.c_longlong(self.n_pad), self.world, stream), "psgd_bulk_finish_launch")
        return self.buffer

    def check(self) -> None:
        self.channel.check()

    def close(self) -> None:
        self.buffer = None
        self.channel.close()



_gather_channels: dict = {}


def native_all_gather(tensor: torch.Tensor, group=None) -> List[torch.Tensor]:
    """All-gather through the in-kernel collectives: list of per-rank tensors shaped like `tensor`.
    Collective: every rank calls it with a tensor of the same size. The channel behind it is cached
    per device and grows (a new, larger one is built by all ranks together) when a message does not fit."""
    device = tensor.device
    n = tensor.numel()
    ch = _gather_channels.get(device)
    if ch is None or ch.cap < n:
        if ch is not None:
            ch.close()
        ch = Channel(max(n, 1 << 16), group)
        _gather_channels[device] = ch
    ch.check()
    out = ch.all_gather(tensor.contiguous().view(-1))
    return [out[r].view(tensor.shape) for r in range(ch.world)]


def native_all_reduce_(tensor: torch.Tensor, group=None) -> torch.Tensor:
    """In-place SUM all-reduce of a small contiguous float32 CUDA tensor through the one-launch
    in-kernel collective (the channel is shared with `native_all_gather`). Collective."""
    device = tensor.device
    n = tensor.numel()
    ch = _gather_channels.get(device)
    if ch is None or ch.cap < n:
        if ch is not None:
            ch.close()
        ch = Channel(max(n, 1 << 16), group)
        _gather_channels[device] = ch
    ch.check()
    return ch.all_reduce_(tensor)


def close_gather_channels() -> None:
    """Release the cached all-gather channels (collective across ranks)."""
    for ch in list(_gather_channels.values()):
        ch.close()
    _gather_channels.clear()
