"""Quantisers that define the scale formats the operators accept.

Same formats as the reference's ``asym_gemm/utils/math.py`` (per_token_cast_to_fp8 :24-34,
per_block_cast_to_fp8 :47-57, per_token_cast_to_int8 :60-74, per_token_cast_to_nvfp4_e4m3 :122-139), written
independently: a tensor quantised by either implementation is accepted by the operators.
"""
from __future__ import annotations

from typing import Tuple

import torch

FP8_MAX = 448.0
INT8_MAX = 127.0
FP4_MAX = 6.0


def ceil_div(x: int, y: int) -> int:
    return -(-x // y)


def align(x: int, y: int) -> int:
    return ceil_div(x, y) * y


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """Round positive scales up to the next power of two (the values an 8-bit exponent-only scale can hold)."""
    if x.numel() == 0:
        return x
    return torch.exp2(torch.ceil(torch.log2(x.abs().clamp_min(1e-12))))


def _pad_cols(x: torch.Tensor, multiple: int) -> torch.Tensor:
    rows, cols = x.shape
    padded = align(cols, multiple)
    if padded == cols:
        return x
    out = x.new_zeros((rows, padded))
    out[:, :cols] = x
    return out


def per_token_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (e4m3 [M, K], fp32 scales [M, ceil(K/gran_k)]); scale = amax/448 per row per K block."""
    assert x.dim() == 2
    rows, cols = x.shape
    blocks = _pad_cols(x, gran_k).view(rows, -1, gran_k)
    amax = blocks.abs().float().amax(dim=2).clamp(1e-4)
    sf = amax / FP8_MAX
    if use_ue8m0:
        sf = ceil_to_ue8m0(sf)
    q = (blocks * (1.0 / sf.unsqueeze(2))).to(torch.float8_e4m3fn).view(rows, -1)[:, :cols].contiguous()
    return q, sf


def per_block_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """[N, K] -> (e4m3 [N, K], fp32 scales [ceil(N/g), ceil(K/g)]); one scale per g x g block."""
    assert x.dim() == 2
    rows, cols = x.shape
    pr, pc = align(rows, gran_k), align(cols, gran_k)
    padded = x.new_zeros((pr, pc))
    padded[:rows, :cols] = x
    view = padded.view(pr // gran_k, gran_k, pc // gran_k, gran_k)
    amax = view.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    sf = amax / FP8_MAX
    if use_ue8m0:
        sf = ceil_to_ue8m0(sf)
    q = (view * (1.0 / sf)).to(torch.float8_e4m3fn).view(pr, pc)[:rows, :cols].contiguous()
    return q, sf.view(pr // gran_k, pc // gran_k)


def per_token_cast_to_int8(x: torch.Tensor, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (int8 [M, K], fp32 scales [M, ceil(K/gran_k)]); scale = amax/127, round to nearest, clamp."""
    assert x.dim() == 2
    rows, cols = x.shape
    blocks = _pad_cols(x, gran_k).view(rows, -1, gran_k)
    amax = blocks.abs().float().amax(dim=2).clamp(1e-4)
    sf = amax / INT8_MAX
    q = (blocks / sf.unsqueeze(2)).round().clamp(-INT8_MAX, INT8_MAX).to(torch.int8)
    return q.view(rows, -1)[:, :cols].contiguous(), sf


def per_channel_cast_to_int8(x: torch.Tensor, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Weights [N, K]: one scale per output channel per K block (same arithmetic as the per-token form)."""
    return per_token_cast_to_int8(x, gran_k)


_E2M1_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def encode_e2m1(x: torch.Tensor) -> torch.Tensor:
    """fp -> 4-bit E2M1 codes (uint8 0..15): magnitudes {0,.5,1,1.5,2,3,4,6}, ties go up, -0 is stored as +0."""
    mag = x.abs().clamp_max(FP4_MAX)
    bounds = torch.tensor(_E2M1_MIDPOINTS, dtype=mag.dtype, device=x.device)
    idx = torch.bucketize(mag, bounds)  # idx = number of bounds <= mag ... with right=False: bounds[i-1] < v <= bounds[i]
    code = idx.to(torch.uint8)
    neg = (x < 0) & (idx != 0)
    return code | (neg.to(torch.uint8) << 3)


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """[.., K] codes -> [.., K/2] bytes, even index in the low nibble."""
    pairs = codes.view(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return ((pairs[..., 0] & 0xF) | ((pairs[..., 1] & 0xF) << 4)).contiguous()


def per_token_cast_to_nvfp4_e4m3(x: torch.Tensor, gran_k: int = 16) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (packed E2M1 uint8 [M, K/2], e4m3 scales [M, ceil(K/gran_k)]); scale = e4m3(amax/6), 0 -> 1."""
    assert x.dim() == 2 and x.shape[1] % 2 == 0
    rows, cols = x.shape
    blocks = _pad_cols(x, gran_k).view(rows, -1, gran_k)
    amax = blocks.abs().float().amax(dim=2).clamp_min(1e-4)
    sf = (amax / FP4_MAX).to(torch.float8_e4m3fn)
    dec = sf.float()
    dec = torch.where(dec == 0, torch.ones_like(dec), dec)
    scaled = blocks * (1.0 / dec.unsqueeze(2))
    codes = encode_e2m1(scaled).view(rows, -1)
    return pack_e2m1(codes)[:, : cols // 2].contiguous(), sf
