"""numpy mirrors of the C descriptors in csrc/psgd_types.h (same field order and sizes)."""
from __future__ import annotations

import numpy as np

MAX_RANK = 32
MAX_HIST = 8
CMAT_STRIDE = MAX_RANK * MAX_RANK

MAT_DTYPE = np.dtype(
    [
        ("grad", "<u8"),
        ("param", "<u8"),
        ("mom", "<u8"),
        ("out", "<u8"),
        ("n", "<i4"),
        ("m", "<i4"),
        ("r", "<i4"),
        ("p_off", "<i4"),
        ("q_off", "<i4"),
        ("grp_p_off", "<i4"),
        ("grp_p_len", "<i4"),
        ("grp_q_off", "<i4"),
        ("grp_q_len", "<i4"),
        ("hyper", "<i4"),
        ("index", "<i4"),
        ("pad0", "<i4"),
    ]
)
assert MAT_DTYPE.itemsize == 80

TILE_DTYPE = np.dtype(
    [
        ("mat", "<i4"),
        ("row0", "<i4"),
        ("rows", "<i4"),
        ("col0", "<i4"),
        ("cols", "<i4"),
        ("split", "<i4"),
        ("nsplit", "<i4"),
        ("ticket", "<i4"),
        ("slot0", "<i4"),
        ("vec", "<i4"),
        ("pad", "<i4", (2,)),
    ]
)
assert TILE_DTYPE.itemsize == 48

HYPER_DTYPE = np.dtype(
    [
        ("lr", "<f4"),
        ("momentum", "<f4"),
        ("one_minus_dampening", "<f4"),
        ("weight_decay", "<f4"),
        ("nesterov", "<i4"),
        ("has_momentum", "<i4"),
        ("grad_scale", "<f4"),
        ("pad", "<i4"),
    ]
)
assert HYPER_DTYPE.itemsize == 32

FLAT_DTYPE = np.dtype(
    [
        ("grad", "<u8"),
        ("param", "<u8"),
        ("mom", "<u8"),
        ("out", "<u8"),
        ("numel", "<i8"),
        ("flat_off", "<i8"),
        ("hyper", "<i4"),
        ("op", "<i4"),
        ("pad", "<i4", (2,)),
    ]
)
assert FLAT_DTYPE.itemsize == 64

ORTH_UNIT_DTYPE = np.dtype(
    [
        ("x_off", "<i4"),
        ("sub_len", "<i4"),
        ("nsub", "<i4"),
        ("r", "<i4"),
        ("first_mat", "<i4"),
        ("chunk0", "<i4"),
        ("nchunks", "<i4"),
        ("pad", "<i4"),
    ]
)
assert ORTH_UNIT_DTYPE.itemsize == 32

ORTH_CHUNK_DTYPE = np.dtype([("unit", "<i4"), ("sub", "<i4"), ("row0", "<i4"), ("rows", "<i4")])
assert ORTH_CHUNK_DTYPE.itemsize == 16
