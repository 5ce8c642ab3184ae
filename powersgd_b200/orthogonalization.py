"""In-place orthonormalisation of (batches of) tall factor matrices.

Two flavours exist in the reference and both are kept:

* `orthogonalize` — library semantics (powersgd/orthogonalization.py:4-8). For a trailing
  dimension of 1 the WHOLE tensor is divided by its joint Frobenius norm (one norm for all
  matrices of the batch, floored at `eps`); otherwise every matrix is replaced by the Q of
  its reduced QR factorisation.
* `gram_schmidt_` — research-harness semantics (paper-code/gradient_reducers.py:945-956):
  column-serial modified Gram-Schmidt with `eps` added to every column norm.

`cholesky_qr2_` is the formulation the CUDA kernels use (Gram matrix in float64, Cholesky,
triangular solve, twice); it spans the same subspace as the other two, which is all that
the compressor's outputs depend on.
"""
from __future__ import annotations

import torch

_EPS_LIB = 1e-16
_EPS_PAPER = 1e-8


def orthogonalize(matrix: torch.Tensor, eps: float = _EPS_LIB) -> torch.Tensor:
    if matrix.shape[-1] == 1:
        norm = torch.linalg.vector_norm(matrix)
        matrix.div_(torch.clamp(norm, min=eps))
    else:
        q, _ = torch.linalg.qr(matrix, mode="reduced")
        matrix.copy_(q)
    return matrix


def gram_schmidt_(matrix: torch.Tensor, eps: float = _EPS_PAPER) -> torch.Tensor:
    """Modified Gram-Schmidt on the columns of one [n, r] matrix, in place."""
    r = matrix.shape[1]
    for j in range(r):
        col = matrix[:, j : j + 1]
        col.div_(torch.sqrt((col * col).sum()) + eps)
        if j + 1 < r:
            tail = matrix[:, j + 1 :]
            tail.sub_(col * (col * tail).sum(dim=0, keepdim=True))
    return matrix


def cholesky_qr2_(batch: torch.Tensor, passes: int = 2) -> torch.Tensor:
    """Orthonormalise every [n, r] matrix of a [..., n, r] tensor via its r×r Gram matrix.

    A pivot that vanishes relative to its column's squared norm marks a rank-deficient
    column: it is replaced by a canonical basis vector and picked up by the next pass
    (this mirrors what Householder QR does on a zero column, which yields an identity
    column). Matches `psgd_orth_kernel` in csrc.
    """
    x = batch.reshape(-1, batch.shape[-2], batch.shape[-1])
    n, r = x.shape[-2], x.shape[-1]
    for _ in range(passes):
        xd = x.double()
        gram = xd.transpose(1, 2) @ xd
        for b in range(x.shape[0]):
            g = gram[b]
            rmat = torch.zeros_like(g)
            dead = []
            for j in range(r):
                s = g[j, j] - (rmat[:j, j] ** 2).sum()
                if not (s > 1e-12 * g[j, j]) or g[j, j] <= 0:
                    dead.append(j)
                    rmat[j, j] = 1.0
                    rmat[j, j + 1 :] = 0.0
                    rmat[:j, j] = 0.0
                    continue
                rmat[j, j] = torch.sqrt(s)
                for k in range(j + 1, r):
                    rmat[j, k] = (g[j, k] - (rmat[:j, j] * rmat[:j, k]).sum()) / rmat[j, j]
            sol = torch.linalg.solve_triangular(rmat, xd[b], upper=True, left=False)
            for j in dead:
                sol[:, j] = 0.0
                sol[j % n, j] = 1.0
            x[b].copy_(sol.to(x.dtype))
    return batch
