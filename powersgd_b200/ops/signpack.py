"""One-bit sign compression (pack / unpack / majority vote).

Bit layout (shared by the CUDA kernels in csrc/signpack.cu and the PyTorch fallback): the flat
vector is zero padded to a multiple of 32 entries and viewed as [32, L]; bit i of word l is 1
iff entry i*L + l is negative. Zero and the padding decode as +1, like the `bit2byte`
extension used by paper-code/gradient_reducers.py:1209-1241.
"""
from __future__ import annotations

import ctypes

import torch

from . import native


def _words(numel: int) -> int:
    return (numel + 31) // 32


def _use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and native.use_for_cuda()


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _bit_weights(device) -> torch.Tensor:
    # int64 arithmetic, then reinterpret the low 32 bits as int32
    return (torch.ones(32, dtype=torch.int64, device=device) << torch.arange(32, device=device)).view(32, 1)


def _to_int32(x64: torch.Tensor) -> torch.Tensor:
    x64 = torch.where(x64 >= 2**31, x64 - 2**32, x64)
    return x64.to(torch.int32)


def pack_signs(src: torch.Tensor) -> torch.Tensor:
    flat = src.reshape(-1)
    numel, words = flat.numel(), _words(flat.numel())
    if _use_native(flat) and flat.dtype == torch.float32:
        flat = flat.contiguous()
        out = torch.empty(words, dtype=torch.int32, device=flat.device)
        native.check(
            native.lib().psgd_sign_pack(ctypes.c_void_p(flat.data_ptr()), numel, ctypes.c_void_p(out.data_ptr()), _stream()),
            "psgd_sign_pack",
        )
        return out
    padded = torch.zeros(words * 32, dtype=flat.dtype, device=flat.device)
    padded[:numel] = flat
    bits = (padded.view(32, words) < 0).to(torch.int64)
    return _to_int32((bits * _bit_weights(flat.device)).sum(dim=0))


def unpack_signs(words: torch.Tensor, numel: int, scale: float = 1.0, out: torch.Tensor = None, accumulate: bool = False) -> torch.Tensor:
    """+-`scale` per entry; with `accumulate` the values are added to `out`."""
    n_words = _words(numel)
    assert words.numel() == n_words
    if out is None:
        out = torch.zeros(numel, dtype=torch.float32, device=words.device) if accumulate else torch.empty(
            numel, dtype=torch.float32, device=words.device
        )
    if _use_native(words):
        words = words.contiguous()
        native.check(
            native.lib().psgd_sign_unpack(
                ctypes.c_void_p(words.data_ptr()), numel, float(scale), ctypes.c_void_p(out.data_ptr()), 1 if accumulate else 0, _stream()
            ),
            "psgd_sign_unpack",
        )
        return out
    w64 = words.to(torch.int64) & 0xFFFFFFFF
    bits = (w64.view(1, n_words) >> torch.arange(32, device=words.device).view(32, 1)) & 1
    vals = (1.0 - 2.0 * bits.to(torch.float32)).reshape(-1)[:numel] * scale
    if accumulate:
        out.add_(vals)
    else:
        out.copy_(vals)
    return out


def _vote(words: torch.Tensor, numel: int, mode: int):
    voters, n_words = words.shape
    if _use_native(words):
        words = words.contiguous()
        dst_w = torch.empty(n_words, dtype=torch.int32, device=words.device) if mode == 0 else None
        dst_f = torch.empty(numel, dtype=torch.float32, device=words.device) if mode == 1 else None
        native.check(
            native.lib().psgd_sign_vote(
                ctypes.c_void_p(words.data_ptr()), voters, numel, mode,
                ctypes.c_void_p(0 if dst_w is None else dst_w.data_ptr()),
                ctypes.c_void_p(0 if dst_f is None else dst_f.data_ptr()), _stream(),
            ),
            "psgd_sign_vote",
        )
        return dst_w if mode == 0 else dst_f
    w64 = words.to(torch.int64) & 0xFFFFFFFF
    bits = (w64.view(voters, 1, n_words) >> torch.arange(32, device=words.device).view(1, 32, 1)) & 1
    total = voters - 2 * bits.sum(dim=0)  # [32, L]
    if mode == 0:
        return _to_int32(((total < 0).to(torch.int64) * _bit_weights(words.device)).sum(dim=0))
    return torch.sign(total.to(torch.float32)).reshape(-1)[:numel]


def majority_vote(words: torch.Tensor) -> torch.Tensor:
    """Packed element-wise majority of [voters, L] packed sign vectors (ties decode as +1)."""
    return _vote(words, words.shape[1] * 32, 0)


def vote_signs(words: torch.Tensor, numel: int) -> torch.Tensor:
    """float sign(sum of the voters' +-1) per entry, in {-1, 0, +1}."""
    return _vote(words, numel, 1)
