"""Host-side shape logic of the GEMM router, in Python (the C++ mirror is ``host/stream_executor.cpp``).

``gemm_broadcast`` pads two operand shapes to rank 4 and ``get_gemm_type`` classifies them as VV / VM / MV / MM,
the decision the reference takes in ``gemmBroadcast`` / ``getGemmType``
(runtime/source/executor/utils/utils.cpp:293-396) before routing a matmul/addmm to its vector kernels.
This module holds no device code and can be imported without a GPU.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

VV, VM, MV, MM = "VV", "VM", "MV", "MM"


def gemm_broadcast(shape1: Sequence[int], shape2: Sequence[int]) -> Tuple[List[int], List[int]]:
    """Rank-4 views of the two matmul operands.

    matmul semantics decide where the 1s go: a 1-D left operand is a row vector, a 1-D right operand a column
    vector; missing batch dimensions are leading 1s."""
    a, b = list(shape1), list(shape2)
    if len(a) > 4 or len(b) > 4 or not a or not b:
        raise ValueError("operands of rank 1..4 expected")
    if len(a) == 1:
        a = [1, a[0]]
    if len(b) == 1:
        b = [b[0], 1]
    a = [1] * (4 - len(a)) + a
    b = [1] * (4 - len(b)) + b
    return a, b


def get_gemm_type(self_shape: Sequence[int], other_shape: Sequence[int]) -> str:
    """Class of two rank-4 shapes: vector classes need both leading dims 1 on both operands."""
    a, b = list(self_shape), list(other_shape)
    if len(a) != 4 or len(b) != 4:
        raise ValueError("rank-4 shapes expected (see gemm_broadcast)")
    if not (a[0] == 1 and a[1] == 1 and b[0] == 1 and b[1] == 1):
        return MM
    na = int(a[2] != 1) + int(a[3] != 1)
    nb = int(b[2] != 1) + int(b[3] != 1)
    if na == 1 and nb == 1:
        return VV
    if na == 1 and nb == 2:
        return VM
    if na == 2 and nb == 1:
        return MV
    return MM


def classify(shape1: Sequence[int], shape2: Sequence[int]) -> str:
    return get_gemm_type(*gemm_broadcast(shape1, shape2))
