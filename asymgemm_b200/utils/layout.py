"""Layout helpers callers of the operators use (reference: asym_gemm/utils/layout.py:5-15)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


def get_mk_alignment_for_contiguous_layout() -> int:
    """Row alignment of every contiguous-layout segment (csrc/utils/layout.hpp:108-110)."""
    return 128


def get_tma_aligned_size(x: int, element_size: int) -> int:
    """Smallest count >= x whose byte size is a multiple of 16 (csrc/utils/math.hpp:24-28)."""
    per = 16 // element_size
    return -(-x // per) * per


def build_contiguous_layout(rows_per_expert: Sequence[int], device="cuda", alignment: int = 128) -> Tuple[torch.Tensor, torch.Tensor, int, int, List[Tuple[int, int, int]]]:
    """Segment table for the contiguous layout from per-expert row counts.

    Experts with zero rows get no segment. Returns (offsets int32 [2*S], experts int32 [S+1] ending in -1,
    list_size = S+1, padded total rows, [(expert, start, valid_rows)]): the form the reference's tests build
    with build_offsets_experts_from_m_indices (tests/generators.py:388-427).
    """
    offsets: List[int] = []
    experts: List[int] = []
    segs: List[Tuple[int, int, int]] = []
    start = 0
    for e, rows in enumerate(rows_per_expert):
        rows = int(rows)
        if rows <= 0:
            continue
        padded = -(-rows // alignment) * alignment
        offsets += [start, start + padded]
        experts.append(e)
        segs.append((e, start, rows))
        start += padded
    experts.append(-1)
    return (torch.tensor(offsets, dtype=torch.int32, device=device),
            torch.tensor(experts, dtype=torch.int32, device=device), len(experts), start, segs)

