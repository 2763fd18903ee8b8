"""Enumerations shared with the operator arguments.

Values are those of the reference adapter
(int_nbit_split_embedding_codegen_lookup_function.cpp:18-33).
"""
from __future__ import annotations

import enum


class PoolingMode(enum.IntEnum):
    SUM = 0
    MEAN = 1
    NONE = 2


class SparseType(enum.IntEnum):
    FP32 = 0
    FP16 = 1
    INT8 = 2
    INT4 = 3
    INT2 = 4
    BF16 = 5
    FP8 = 6

    def bit_rate(self) -> int:
        return {0: 32, 1: 16, 2: 8, 3: 4, 4: 2, 5: 16, 6: 8}[int(self)]

    def has_header(self) -> bool:
        """INT8 / INT4 / INT2 rows start with an fp16 scale and an fp16 bias."""
        return self in (SparseType.INT8, SparseType.INT4, SparseType.INT2)

    def align_size(self) -> int:
        """Elements a row's D must be a multiple of (same rule the reference test applies,
        test_int_nbit_split_embedding_codegen_lookup_function.py:318)."""
        return {0: 1, 1: 2, 2: 4, 3: 8, 4: 16, 5: 2, 6: 4}[int(self)]


def row_bytes(ty: int, D: int, row_alignment: int = 16) -> int:
    """Bytes of one table row: optional 4-byte header + payload, padded to row_alignment."""
    ty = SparseType(int(ty))
    payload = (D * ty.bit_rate() + 7) // 8
    b = payload + (4 if ty.has_header() else 0)
    if row_alignment > 1:
        b = (b + row_alignment - 1) // row_alignment * row_alignment
    return b
