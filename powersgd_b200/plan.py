"""Shape-bucket planner.

Turns a parameter list into the static description that every back end shares: which
tensors are compressed, how the compressed ones fold into 2-D matrices, which matrices
share a shape group, the factor rank of each group and where each group's factors live
in the flat P and Q buffers.

Rules kept from the reference:
  * the compress / don't-compress decision looks at the RAW N-D shape
    (powersgd/powersgd.py:101-105, 292-294);
  * the factor rank is min(rank, n, m) of the 2-D view (powersgd.py:237-251);
  * a tensor folds to [shape[0], prod(shape[1:])] (powersgd.py:283-289);
  * groups are ordered by first appearance, matrices inside a group by parameter order,
    and a group's factors are stored as one contiguous [B, n, r] / [B, m, r] block.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import torch


def avg_compressed_size(shape: Sequence[int], config) -> float:
    """Average number of floats sent per step for a tensor of this raw shape."""
    dims = [int(d) for d in shape]
    r = min(int(config.rank), min(dims))
    return 0.5 * config.num_iters_per_step * r * sum(dims)


def should_compress(shape: Sequence[int], config) -> bool:
    numel = 1
    for d in shape:
        numel *= int(d)
    if len(shape) == 0:
        return False
    size = avg_compressed_size(shape, config)
    if size <= 0:
        return False
    return numel / size > config.min_compression_rate


def matrix_shape(shape: Sequence[int]) -> Tuple[int, int]:
    n = int(shape[0])
    m = 1
    for d in shape[1:]:
        m *= int(d)
    return n, m


@dataclass
class ShapeGroup:
    n: int
    m: int
    r: int
    members: List[int] = field(default_factory=list)  # indices into the compressed list
    p_offset: int = 0  # float offset of this group's [B, n, r] block in the P buffer
    q_offset: int = 0  # float offset of this group's [B, m, r] block in the Q buffer

    @property
    def batch(self) -> int:
        return len(self.members)

    @property
    def p_numel(self) -> int:
        return self.batch * self.n * self.r

    @property
    def q_numel(self) -> int:
        return self.batch * self.m * self.r


@dataclass
class CompressionPlan:
    shapes: List[torch.Size]  # raw shapes of the compressed tensors, in order
    groups: List[ShapeGroup]
    p_total: int
    q_total: int

    @classmethod
    def build(cls, shapes: Sequence[Sequence[int]], rank: int, batch_same_shapes: bool = True) -> "CompressionPlan":
        """`batch_same_shapes=False` gives every tensor its own group (the research harness' reducers
        keep one factor pair per tensor; at rank 1 this also means one norm per matrix)."""
        by_shape: Dict[Tuple, ShapeGroup] = {}
        for idx, shape in enumerate(shapes):
            n, m = matrix_shape(shape)
            key = (n, m) if batch_same_shapes else (n, m, idx)
            if key not in by_shape:
                by_shape[key] = ShapeGroup(n=n, m=m, r=min(int(rank), n, m))
            by_shape[key].members.append(idx)
        groups = list(by_shape.values())
        p_cursor = q_cursor = 0
        for g in groups:
            g.p_offset, g.q_offset = p_cursor, q_cursor
            p_cursor += g.p_numel
            q_cursor += g.q_numel
        return cls([torch.Size(s) for s in shapes], groups, p_cursor, q_cursor)

    def locate(self) -> List[Tuple[int, int]]:
        """For every compressed tensor: (group index, position inside the group)."""
        where = [(-1, -1)] * len(self.shapes)
        for gi, g in enumerate(self.groups):
            for pos, idx in enumerate(g.members):
                where[idx] = (gi, pos)
        return where

    def signature(self) -> Tuple:
        return tuple((g.n, g.m, g.r, tuple(g.members)) for g in self.groups)
