"""Error metrics used by the parity tests (reference: asym_gemm/testing/numeric.py:9-23)."""
from __future__ import annotations

import torch


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y>/(|x|^2+|y|^2): 0 for identical tensors, the metric the reference's tests threshold."""
    x, y = x.double(), y.double()
    denom = (x * x + y * y).sum()
    if denom == 0:
        return 0.0
    return float(1 - 2 * (x * y).sum() / denom)


def max_rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max |x - ref| / max |ref|: the 'max-rel' figure the tolerances are stated in."""
    x, ref = x.double(), ref.double()
    scale = ref.abs().max().clamp_min(1e-30)
    return float((x - ref).abs().max() / scale)


def count_bytes(*tensors) -> int:
    total = 0
    for t in tensors:
        if isinstance(t, (tuple, list)):
            total += count_bytes(*t)
        elif t is not None:
            total += t.numel() * t.element_size()
    return total
