"""Magnitude top-k selection with the error-feedback write fused in (csrc/topk.cu).

`topk_abs(x, k, memory=None)` returns `(values, positions)` of the k entries of the flattened
tensor with the largest |x| (order unspecified, positions int32) and, when `memory` is given,
fills it with x where the taken entries are zeroed. On CPU (or on CUDA without the native
library when PSGD_B200_ALLOW_FALLBACK=1 allows it; otherwise that is an error) the same result
comes from `torch.topk` (gradient_reducers.py:240-253 is the reference sequence).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import native

_workspaces = {}


def topk_abs(x: torch.Tensor, k: int, memory: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    flat = x.reshape(-1)
    n = flat.numel()
    k = int(k)
    if flat.is_cuda and native.use_for_cuda() and flat.dtype == torch.float32 and flat.is_contiguous() and (
        memory is None or (memory.is_contiguous() and memory.dtype == torch.float32)
    ):
        lib = native.lib()
        ws = _workspaces.get(flat.device)
        if ws is None:
            ws = torch.zeros(lib.psgd_topk_workspace_ints(), dtype=torch.int32, device=flat.device)
            _workspaces[flat.device] = ws
        values = torch.empty(k, dtype=torch.float32, device=flat.device)
        positions = torch.empty(k, dtype=torch.int32, device=flat.device)
        code = lib.psgd_topk_abs(
            ctypes.c_void_p(flat.data_ptr()), ctypes.c_longlong(n), ctypes.c_longlong(k), ctypes.c_void_p(ws.data_ptr()),
            ctypes.c_void_p(values.data_ptr()), ctypes.c_void_p(positions.data_ptr()),
            ctypes.c_void_p(0 if memory is None else memory.data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
        )
        native.check(code, "psgd_topk_abs")
        return values, positions
    _, idx = torch.topk(flat.abs(), k, sorted=False)
    values = flat[idx].contiguous()
    if memory is not None:
        memory.copy_(x)
        memory.view(-1)[idx] = 0.0
    return values, idx.to(torch.int32)


_many_cache: dict = {}


def topk_abs_many(tensors, ks, memories=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """`topk_abs` for a list of tensors in four launches (csrc/topk.cu, psgd_topk_abs_many).

    Returns flat `(values, positions)`: tensor i's `ks[i]` pairs start at `sum(ks[:i])`; positions
    are int32 indices into the flattened tensor i. `memories[i]`, when given, receives tensor i with
    the taken entries zeroed. Falls back to one `topk_abs` per tensor off the GPU."""
    ks = [int(k) for k in ks]
    total = sum(ks)
    flats = [t.reshape(-1) for t in tensors]
    mems = list(memories) if memories is not None else [None] * len(flats)
    device = flats[0].device
    native_ok = (
        device.type == "cuda" and native.use_for_cuda()
        and all(t.dtype == torch.float32 and t.is_contiguous() for t in tensors)   # flats are then views
        and all(m is None or (m.is_contiguous() and m.dtype == torch.float32) for m in mems)
    )
    if not native_ok:
        values = torch.empty(total, dtype=torch.float32, device=device)
        positions = torch.empty(total, dtype=torch.int32, device=device)
        at = 0
        for t, k, m in zip(tensors, ks, mems):
            v, p = topk_abs(t, k, memory=m)
            values[at : at + k], positions[at : at + k] = v, p
            at += k
        return values, positions
    import numpy as np

    lib = native.lib()
    key = (device, tuple(f.data_ptr() for f in flats), tuple(0 if m is None else m.data_ptr() for m in mems), tuple(f.numel() for f in flats), tuple(ks))
    entry = _many_cache.get(key)
    if entry is None:
        dtype = np.dtype([("x", np.uint64), ("memory", np.uint64), ("n", np.int64), ("k", np.int64), ("out_off", np.int64)])
        if dtype.itemsize != int(lib.psgd_topk_item_bytes()):
            raise RuntimeError("top-k item record out of sync with the native library")
        items = np.zeros(len(flats), dtype=dtype)
        block_item, block_part, parts = [], [], []
        at = 0
        for i, (f, k, m) in enumerate(zip(flats, ks, mems)):
            n = f.numel()
            if not (0 < k <= n < (1 << 31)):
                raise ValueError(f"topk_abs_many: need 0 < k <= n < 2^31 (k = {k}, n = {n})")
            items[i] = (f.data_ptr(), 0 if m is None else m.data_ptr(), n, k, at)
            at += k
            nparts = max(1, min(256, -(-n // (512 * 8))))   # <= 8 elements per thread and pass up to 1 Mi entries, then longer loops
            parts.append(nparts)
            block_item += [i] * nparts
            block_part += list(range(nparts))
        to_dev = lambda a: torch.from_numpy(a.view(np.uint8) if a.dtype.names else a).to(device)  # noqa: E731
        entry = {
            "items": to_dev(items), "block_item": to_dev(np.asarray(block_item, dtype=np.int32)),
            "block_part": to_dev(np.asarray(block_part, dtype=np.int32)), "parts": to_dev(np.asarray(parts, dtype=np.int32)),
            "nblocks": len(block_item),
            "ws": torch.zeros(len(flats) * int(lib.psgd_topk_workspace_ints()), dtype=torch.int32, device=device),
        }
        # the tables hold addresses and lengths only, and the key is exactly those: an entry stays
        # valid for whatever tensors present the same addresses again, so no tensor is kept alive
        if len(_many_cache) >= 4:
            _many_cache.clear()
        _many_cache[key] = entry
    values = torch.empty(total, dtype=torch.float32, device=device)
    positions = torch.empty(total, dtype=torch.int32, device=device)
    vp = ctypes.c_void_p
    code = lib.psgd_topk_abs_many(
        vp(entry["items"].data_ptr()), len(flats), vp(entry["block_item"].data_ptr()), vp(entry["block_part"].data_ptr()),
        vp(entry["parts"].data_ptr()), entry["nblocks"], vp(entry["ws"].data_ptr()), vp(values.data_ptr()), vp(positions.data_ptr()),
        vp(torch.cuda.current_stream().cuda_stream),
    )
    native.check(code, "psgd_topk_abs_many")
    return values, positions


_SEG_DTYPE = None
_combine_scratch = {}


def sparse_combine(all_values: torch.Tensor, all_positions: torch.Tensor, outs, ends, divisor: float) -> None:
    """outs[s] <- sum over workers of value / divisor of the (value, position) pairs of segment s, scattered.

    `all_values` / `all_positions`: [workers, K] float32 / int32 (rows as all-gathered); segment s
    owns columns [ends[s-1], ends[s]) of every row, its positions index into the flattened
    `outs[s]`. Positions are unique within a row's segment. On CUDA one cooperative launch zeroes
    the outputs and applies the workers in rank order (csrc/topk.cu), so replicas stay
    bit-identical; elsewhere the same sum runs as one `index_add_` per worker
    (gradient_reducers.py:262-271)."""
    global _SEG_DTYPE
    workers, per_worker = all_values.shape
    use_native = (
        all_values.is_cuda and native.use_for_cuda() and all_values.dtype == torch.float32 and all_positions.dtype == torch.int32
        and all_values.is_contiguous() and all_positions.is_contiguous()
        and all(o.is_contiguous() and o.dtype == torch.float32 for o in outs)
    )
    if use_native:
        import numpy as np

        lib = native.lib()
        cap = int(lib.psgd_sparse_combine_max_segments())
        if _SEG_DTYPE is None:
            _SEG_DTYPE = np.dtype([("out", np.uint64), ("numel", np.int64), ("end", np.int64)])
        device = all_values.device
        scratch = _combine_scratch.get(device)
        if scratch is None:
            scratch = torch.zeros(2, dtype=torch.int32, device=device)  # [grid barrier, status]
            _combine_scratch[device] = scratch
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for first in range(0, len(outs), cap):
            chunk = list(range(first, min(first + cap, len(outs))))
            segs = np.zeros(len(chunk), dtype=_SEG_DTYPE)
            base = ends[first - 1] if first else 0
            for j, s in enumerate(chunk):
                segs[j] = (outs[s].data_ptr(), outs[s].numel(), ends[s] - base)
            segs_dev = torch.from_numpy(segs.view(np.uint8)).to(device, non_blocking=False)
            width = ends[chunk[-1]] - base
            vals = all_values if (base == 0 and width == per_worker) else all_values[:, base : base + width].contiguous()
            poss = all_positions if (base == 0 and width == per_worker) else all_positions[:, base : base + width].contiguous()
            code = lib.psgd_sparse_combine_launch(
                ctypes.c_void_p(vals.data_ptr()), ctypes.c_void_p(poss.data_ptr()), int(workers), ctypes.c_longlong(width),
                ctypes.c_void_p(segs_dev.data_ptr()), len(chunk), ctypes.c_float(divisor),
                ctypes.c_void_p(scratch.data_ptr()), ctypes.c_void_p(scratch.data_ptr() + 4), stream,
            )
            native.check(code, "psgd_sparse_combine_launch")
            segs_dev.record_stream(torch.cuda.current_stream())
        return
    start = 0
    for out, end in zip(outs, ends):
        out.zero_()
        flat = out.view(-1)
        for w in range(workers):
            flat.index_add_(0, all_positions[w, start:end].long(), all_values[w, start:end] / divisor)
        start = end


def sparse_combine_status(device) -> int:
    """0 unless a grid barrier of `sparse_combine` gave up on `device` (reads the device word: synchronises)."""
    scratch = _combine_scratch.get(torch.device(device))
    return 0 if scratch is None else int(scratch[1].item())
