"""In-switch (NVLink SHARP) all-reduce of a flat float32 buffer: the flat aggregator's path for
buffers above the one-shot limit from four workers on (PSGD_B200_FLAT=nvls forces it, NCCL_NVLS_ENABLE=0
or PSGD_B200_FLAT=bulk keeps it off).

The buffer is bound to an NVLink multicast object by this package's own runtime (csrc/mcast.cpp:
virtual-memory allocation, `cuMulticast*` binding; the object's file descriptor travels from rank 0
to the peers over a Unix-domain socket whose name goes through the process group), or, with
PSGD_B200_NVLS_RUNTIME=torch or when the native set-up is refused, by PyTorch's symmetric-memory
runtime. The reduction is this package's kernel (csrc/nvls.cu: `multimem.ld_reduce` +
`multimem.st`, each rank reducing the slice it owns) with the two cross-rank barriers it needs
carried inside the same launch as bounded token exchanges on an in-kernel channel. The reference
all-reduces whole models with NCCL (powersgd/powersgd.py:22-31); on NVSwitch machines NCCL takes
the same in-switch route.

A rank must not disappear while its memory is bound to the multicast object: keep this path out of
failure tests, and call `close()` (collective) before the process group is destroyed.
"""
from __future__ import annotations

import ctypes
import os
import socket
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native


class NvlsUnavailable(RuntimeError):
    """No NVLink multicast on this machine / build (raised on every rank alike)."""


class _McBuffer(ctypes.Structure):
    # mirrors PsgdMcBuffer (csrc/mcast.cpp)
    _fields_ = [("mc_handle", ctypes.c_ulonglong), ("mem_handle", ctypes.c_ulonglong), ("local_ptr", ctypes.c_ulonglong),
                ("mc_ptr", ctypes.c_ulonglong), ("bytes", ctypes.c_ulonglong), ("device", ctypes.c_int), ("bound", ctypes.c_int)]


_socket_serial = [0]


def _last_error() -> str:
    msg = native.lib().psgd_last_error()
    return msg.decode() if msg else ""


def _all_true(flag: bool, group) -> bool:
    flags = [None] * dist.get_world_size(group)
    dist.all_gather_object(flags, bool(flag), group=group)
    return all(flags)


class MulticastBuffer:
    """`nbytes` (rounded up to the driver's granularity) on every rank, bound to one NVLink multicast
    object: `local_ptr` addresses this rank's replica, `mc_ptr` all replicas at once. Collective."""

    def __init__(self, nbytes: int, group=None):
        self.lib = native.lib()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self._state: Optional[_McBuffer] = None
        if ctypes.sizeof(_McBuffer) != int(self.lib.psgd_mc_buffer_bytes()):
            raise RuntimeError("multicast buffer record out of sync with the native library")
        if not _all_true(int(self.lib.psgd_mc_supported()) == 1, self.group):
            raise NvlsUnavailable("a device of the job reports no NVLink multicast support")
        rounded = ctypes.c_ulonglong()
        ok = self.lib.psgd_mc_round_up(self.world, ctypes.c_ulonglong(int(nbytes)), ctypes.byref(rounded)) == 0
        if not _all_true(ok, self.group):
            raise NvlsUnavailable(f"multicast granularity query failed: {_last_error() if not ok else 'on a peer'}")
        self.nbytes = int(rounded.value)
        state = _McBuffer()
        ok, why = self._share_object(state)
        if not _all_true(ok, self.group):
            self._release(state)
            raise NvlsUnavailable(f"multicast object not shared: {why or 'failure on a peer'}")
        ok = self.lib.psgd_mc_add_device(ctypes.byref(state)) == 0
        why = "" if ok else _last_error()
        if not _all_true(ok, self.group):   # doubles as the barrier between "all added" and "any bind"
            self._release(state)
            raise NvlsUnavailable(f"cuMulticastAddDevice refused: {why or 'on a peer'}")
        ok = self.lib.psgd_mc_bind(ctypes.byref(state)) == 0
        why = "" if ok else _last_error()
        if not _all_true(ok, self.group):
            self._release(state)
            raise NvlsUnavailable(f"binding memory to the multicast object failed: {why or 'on a peer'}")
        self._state = state
        self.local_ptr, self.mc_ptr = int(state.local_ptr), int(state.mc_ptr)

    def _share_object(self, state: _McBuffer):
        """Rank 0 creates the object and serves its file descriptor to every peer."""
        src = dist.get_global_rank(self.group, 0) if self.group is not dist.group.WORLD else 0
        if self.rank == 0:
            fd = ctypes.c_int(-1)
            ok = self.lib.psgd_mc_create(self.world, ctypes.c_ulonglong(self.nbytes), ctypes.byref(state), ctypes.byref(fd)) == 0
            why = "" if ok else _last_error()
            server, name = None, None
            if ok:
                _socket_serial[0] += 1
                name = f"\0psgd_b200_mc_{os.getpid()}_{_socket_serial[0]}"   # abstract namespace: nothing to unlink
                server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
                server.bind(name)
                server.listen(self.world)
                server.settimeout(60.0)
            dist.broadcast_object_list([name, why], src=src, group=self.group)
            if not ok:
                return False, why
            try:
                for _ in range(self.world - 1):
                    conn, _addr = server.accept()
                    with conn:
                        socket.send_fds(conn, [b"m"], [fd.value])
                        conn.recv(1)   # the peer has the descriptor
            except OSError as exc:
                ok, why = False, f"descriptor hand-over failed: {exc}"
            finally:
                server.close()
                os.close(fd.value)
            return ok, why
        box = [None, None]
        dist.broadcast_object_list(box, src=src, group=self.group)
        name, why = box
        if name is None:
            return False, why
        try:
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as conn:
                conn.settimeout(60.0)
                conn.connect(name)
                _msg, fds, _flags, _addr = socket.recv_fds(conn, 16, 1)
                conn.send(b"k")
        except OSError as exc:
            return False, f"descriptor hand-over failed: {exc}"
        if not fds:
            return False, "no descriptor received"
        ok = self.lib.psgd_mc_import(int(fds[0]), ctypes.c_ulonglong(self.nbytes), ctypes.byref(state)) == 0
        return ok, ("" if ok else _last_error())

    def _release(self, state: _McBuffer) -> None:
        self.lib.psgd_mc_release(ctypes.byref(state))

    def tensor(self, numel: int) -> torch.Tensor:
        """float32 view of this rank's replica (no ownership: it must not outlive `close()`)."""
        if numel * 4 > self.nbytes:
            raise ValueError("view outside the multicast buffer")

        class _View:
            __cuda_array_interface__ = {"shape": (int(numel),), "typestr": "<f4", "data": (self.local_ptr, False), "version": 2, "strides": None}

        return torch.as_tensor(_View(), device=torch.device("cuda", torch.cuda.current_device()))

    def close(self) -> None:
        """Collective: nothing may still address the buffer on any rank."""
        if self._state is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._release(self._state)
        self._state = None
        dist.barrier(group=self.group)


class _TorchRuntimeBuffer:
    """The same two addresses from PyTorch's symmetric-memory runtime."""

    def __init__(self, nbytes: int, group):
        device = torch.device("cuda", torch.cuda.current_device())
        world = dist.get_world_size(group)
        try:
            import torch.distributed._symmetric_memory as symm_mem
            from torch._C._autograd import DeviceType
            from torch._C._distributed_c10d import _SymmetricMemory

            supported = bool(_SymmetricMemory.has_multicast_support(DeviceType.CUDA, device.index))
            reason = "the device reports no NVLink multicast support"
        except Exception as exc:  # API not in this PyTorch build
            supported, symm_mem, reason = False, None, f"symmetric-memory runtime not usable: {exc}"
        if not _all_true(supported, group):
            raise NvlsUnavailable(reason if not supported else "a peer reports no NVLink multicast support")
        self.group = group
        self.nbytes = -(-int(nbytes) // 16) * 16
        self._tensor = symm_mem.empty(self.nbytes // 4, dtype=torch.float32, device=device)
        self._handle = symm_mem.rendezvous(self._tensor, group)
        self.mc_ptr = int(self._handle.multicast_ptr)
        self.local_ptr = int(self._tensor.data_ptr())
        if not _all_true(self.mc_ptr != 0 and self.mc_ptr % 16 == 0, group):
            self._handle = self._tensor = None
            raise NvlsUnavailable("the symmetric-memory runtime returned no multicast address")
        del world

    def tensor(self, numel: int) -> torch.Tensor:
        return self._tensor[:numel]

    def close(self) -> None:
        if self._tensor is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._handle = None
        self._tensor = None
        torch.cuda.synchronize()
        dist.barrier(group=self.group)


class NvlsAllReduce:
    """In-place SUM all-reduce of `buffer` (float32, this rank's replica of the multicast-bound buffer).

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
        runtime = os.environ.get("PSGD_B200_NVLS_RUNTIME", "native")
        self._memory = None
        if runtime != "torch":
            try:
                self._memory = MulticastBuffer(self.n_pad * 4, self.group)
                self.runtime = "native"
            except NvlsUnavailable as exc:
                native_reason = str(exc)
        if self._memory is None:
            try:
                self._memory = _TorchRuntimeBuffer(self.n_pad * 4, self.group)
                self.runtime = "torch"
            except NvlsUnavailable as exc:
                raise NvlsUnavailable(str(exc) if runtime == "torch" else f"{native_reason}; PyTorch runtime: {exc}")
        self.mc_ptr = int(self._memory.mc_ptr)
        self.buffer = self._memory.tensor(self.n_pad)
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
        if self._memory is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._channel.close()
        self.buffer = None
        self._memory.close()
        self._memory = None
