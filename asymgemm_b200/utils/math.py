"""Quantisers that define the scale formats the operators accept.

Same formats as the reference's ``asym_gemm/utils/math.py`` (per_token_cast_to_fp8 :24-34, per_channel_cast_to_fp8 :37-45,
per_block_cast_to_fp8 :47-57, per_token_cast_to_int8 :60-74, per_custom_dims_cast_to_fp8 :82-88, per_token_cast_to_fp4
:103-119, per_token_cast_to_nvfp4_e4m3 :122-139, transpose_packed_fp4 :142-155), written independently: a tensor quantised
by either implementation is accepted by the operators.
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


def per_channel_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M, N] with M % gran_k == 0 -> (e4m3 [M, N], fp32 scales [M/gran_k, N]): one scale per column per block of gran_k rows."""
    assert x.dim() == 2 and x.shape[0] % gran_k == 0
    rows, cols = x.shape
    view = x.view(rows // gran_k, gran_k, cols)
    sf = view.abs().float().amax(dim=1).clamp(1e-4) / FP8_MAX
    if use_ue8m0:
        sf = ceil_to_ue8m0(sf)
    return (view * (1.0 / sf.unsqueeze(1))).to(torch.float8_e4m3fn).view(rows, cols), sf


def per_custom_dims_cast_to_fp8(x: torch.Tensor, dims: Tuple[int, ...], use_ue8m0: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scale per index along `dims` (amax over all other dimensions): (e4m3 like x, fp32 scales of the kept dims)."""
    reduce_over = tuple(i for i in range(x.dim()) if i not in set(dims))
    sf = x.abs().float().amax(dim=reduce_over, keepdim=True).clamp(1e-4) / FP8_MAX
    if use_ue8m0:
        sf = ceil_to_ue8m0(sf)
    return (x * (1.0 / sf)).to(torch.float8_e4m3fn), sf.squeeze()


def per_token_cast_to_fp4(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (packed E2M1 uint8 [M, K/2], fp32 scales [M, ceil(K/gran_k)]); scale = amax/6 per row per K block,
    optionally rounded up to a power of two."""
    assert x.dim() == 2 and x.shape[1] % 2 == 0
    rows, cols = x.shape
    blocks = _pad_cols(x, gran_k).view(rows, -1, gran_k)
    sf = blocks.abs().float().amax(dim=2).clamp_min(1e-4) / FP4_MAX
    if use_ue8m0:
        sf = ceil_to_ue8m0(sf)
    codes = encode_e2m1(blocks * (1.0 / sf.unsqueeze(2))).view(rows, -1)
    return pack_e2m1(codes)[:, : cols // 2].contiguous(), sf


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """[.., K/2] bytes -> [.., K] codes (low nibble = even index)."""
    out = torch.empty((*packed.shape[:-1], packed.shape[-1] * 2), dtype=torch.uint8, device=packed.device)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = (packed >> 4) & 0xF
    return out


def transpose_packed_fp4(a: torch.Tensor) -> torch.Tensor:
    """Packed E2M1 [M, N/2] -> packed [N, M/2]: the transpose of the 4-bit matrix, re-packed along its new rows."""
    assert a.dtype == torch.uint8 and a.dim() == 2 and a.shape[0] % 2 == 0
    return pack_e2m1(unpack_e2m1(a).t().contiguous())
