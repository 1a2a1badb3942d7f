"""Dense fp32 restatement of the FP8 MoE layer (gate+up GEMM, SiLU*mul, 1x128 requantisation, down GEMM, router-weighted
sum) in plain torch, and seeded per-expert weights, for checking the expert-parallel layer's output.

A checker, not a code path of the layer: fp32 matmuls on dequantised operands, token by expert. The activation follows
the reference's CPU bucket, bf16(silu(gate) * up) with silu(g) = g / (1 + exp(-g)) (csrc/cpu/module.cpp:337-347); both
GEMM results are rounded to bf16 as the operators write them.
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch


def expert_generator(device, seed: int, expert: int, stream: int = 0) -> torch.Generator:
    """Generator for one expert's data: the same numbers whichever rank owns the expert."""
    return torch.Generator(device=device).manual_seed(int(seed) * 1000003 + 7919 * int(expert) + int(stream))


def expert_weights(seed: int, expert: int, hidden: int, inter: int, device, use_ue8m0: bool = False, std: float = 0.02):
    """(w13 e4m3 [2*inter, hidden], s13 fp32 [2*inter/128, hidden/128], w2 e4m3 [hidden, inter], s2) of expert `expert`:
    N(0, std) weights quantised with 128x128 block scales."""
    from ..utils import per_block_cast_to_fp8
    gen = expert_generator(device, seed, expert)
    q13, s13 = per_block_cast_to_fp8(torch.randn((2 * inter, hidden), device=device, generator=gen) * std, use_ue8m0=use_ue8m0)
    q2, s2 = per_block_cast_to_fp8(torch.randn((hidden, inter), device=device, generator=gen) * std, use_ue8m0=use_ue8m0)
    return q13, s13, q2, s2


def dequant_blocks(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    n, k = q.shape
    return q.float() * s.repeat_interleave(128, 0).repeat_interleave(128, 1)[:n, :k]


def dense_moe_reference(x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, weights_of: Callable[[int], Tuple], inter: int,
                        use_ue8m0: bool = False) -> torch.Tensor:
    """y fp32 [T, hidden] for tokens x bf16 [T, hidden] routed by ids [T, k] with weights wts [T, k];
    `weights_of(e)` returns (w13, s13, w2, s2) of global expert e on x's device."""
    from ..utils import per_token_cast_to_fp8
    xq, sx = per_token_cast_to_fp8(x.float(), use_ue8m0=use_ue8m0)
    xd = xq.float() * sx.repeat_interleave(128, 1)[:, : x.shape[1]]
    y = torch.zeros_like(xd)
    for e in ids.unique().tolist():
        w13, s13, w2, s2 = weights_of(int(e))
        tok, slot = (ids == e).nonzero(as_tuple=True)
        h = (xd[tok] @ dequant_blocks(w13, s13).t()).to(torch.bfloat16).float()
        g, u = h[:, :inter], h[:, inter:]
        act = ((g / (1.0 + torch.exp(-g))) * u).to(torch.bfloat16).float()
        aq, sa = per_token_cast_to_fp8(act, use_ue8m0=use_ue8m0)
        ad = aq.float() * sa.repeat_interleave(128, 1)[:, :inter]
        out = (ad @ dequant_blocks(w2, s2).t()).to(torch.bfloat16).float()
        y.index_add_(0, tok, out * wts[tok, slot].unsqueeze(1).float())
    return y
