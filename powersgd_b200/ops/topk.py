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
