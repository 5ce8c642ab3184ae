"""Thin SVD of many matrices at once.

`svd_many(matrices)` returns `[(U, S, V), ...]` with `M = U diag(S) V^T`, singular values in
descending order. Matrices whose narrow side has at most 32 entries — the shape class the ATOMO
reducer produces (e.g. 2048 x 18 for a 3x3 convolution) — are factorised by one launch of the
native Gram/Jacobi kernel (csrc/svd_tall.cu), wide ones through their transpose; everything
else, and every matrix on a CPU tensor, goes to `torch.linalg.svd` (the reference moves all of
them to the CPU, paper-code/gradient_reducers.py:1019-1029).
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

import numpy as np
import torch

from . import native

_ITEM = np.dtype([("x_off", "<i8"), ("u_off", "<i8"), ("s_off", "<i4"), ("v_off", "<i4"), ("n", "<i4"), ("c", "<i4")])
assert _ITEM.itemsize == 32


def _torch_svd(m: torch.Tensor):
    u, s, vh = torch.linalg.svd(m, full_matrices=False)
    return u, s, vh.transpose(-2, -1)


def svd_many(matrices: Sequence[torch.Tensor]) -> List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
    results: List = [None] * len(matrices)
    batch = []  # (index, tall matrix [n, c], transposed?)
    use_native = bool(matrices) and matrices[0].is_cuda and native.use_for_cuda()
    max_c = native.lib().psgd_svd_tall_max_cols() if use_native else 0
    for i, m in enumerate(matrices):
        n, c = m.shape
        if use_native and m.dtype == torch.float32 and min(n, c) <= max_c and min(n, c) >= 1:
            batch.append((i, m if n >= c else m.t(), n < c))
        else:
            results[i] = _torch_svd(m)
    if batch:
        device = matrices[0].device
        items = np.zeros(len(batch), dtype=_ITEM)
        x_cursor = s_cursor = v_cursor = 0
        for row, (_, tall, _) in zip(items, batch):
            n, c = tall.shape
            row["x_off"], row["u_off"], row["s_off"], row["v_off"], row["n"], row["c"] = x_cursor, x_cursor, s_cursor, v_cursor, n, c
            x_cursor += n * c
            s_cursor += c
            v_cursor += c * c
        x = torch.cat([tall.reshape(-1) if tall.is_contiguous() else tall.contiguous().reshape(-1) for _, tall, _ in batch])
        u = torch.empty_like(x)
        s = torch.empty(s_cursor, dtype=torch.float32, device=device)
        v = torch.empty(v_cursor, dtype=torch.float32, device=device)
        items_dev = torch.from_numpy(items.view(np.uint8).reshape(-1).copy()).to(device)
        code = native.lib().psgd_svd_tall_launch(
            ctypes.c_void_p(items_dev.data_ptr()), len(batch), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(u.data_ptr()),
            ctypes.c_void_p(s.data_ptr()), ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
        )
        native.check(code, "psgd_svd_tall_launch")
        for row, (i, tall, transposed) in zip(items, batch):
            n, c = tall.shape
            uu = u[int(row["u_off"]) : int(row["u_off"]) + n * c].view(n, c)
            ss = s[int(row["s_off"]) : int(row["s_off"]) + c]
            vv = v[int(row["v_off"]) : int(row["v_off"]) + c * c].view(c, c)
            results[i] = (vv, ss, uu) if transposed else (uu, ss, vv)
    return results
