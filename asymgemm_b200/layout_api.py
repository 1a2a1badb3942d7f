"""Scale-factor layout helpers and runtime setters that callers of the reference package use next to the GEMMs
(registered by csrc/apis/layout.hpp:117-128 and csrc/apis/runtime.hpp:15-48 of the reference).

The kernels of this library read the fp32 / e4m3 scale tensors in the layout callers already hold, so none of these is
on the hot path; they exist so that code written against the reference keeps importing and gets tensors of the same
shape, strides and contents. All of them are plain torch tensor arithmetic on the tensor's own device.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from .utils.layout import get_tma_aligned_size as _tma_aligned_size

_state = {"tc_util": 100, "compile_mode": 0}


def get_tma_aligned_size(x: int, element_size: int) -> int:
    """Smallest count >= x whose byte size is a multiple of 16 (csrc/utils/math.hpp:24-28)."""
    assert 16 % element_size == 0
    return _tma_aligned_size(x, element_size)


def get_mn_major_tma_aligned_tensor(sf: torch.Tensor) -> torch.Tensor:
    """fp32 scales [.., mn, k] -> same shape, MN-major (stride 1 along mn) with the leading dimension padded so that
    every k column starts on a 16-byte boundary (impls/smxx_layout.hpp `get_mn_major_tma_aligned_tensor`)."""
    assert sf.dtype == torch.float32 and sf.dim() in (2, 3)
    batched = sf.dim() == 3
    x = sf if batched else sf.unsqueeze(0)
    g, mn, k = x.shape
    aligned = get_tma_aligned_size(mn, 4)
    buf = torch.zeros((g, k, aligned), dtype=sf.dtype, device=sf.device)
    buf[:, :, :mn] = x.transpose(1, 2)
    out = buf[:, :, :mn].transpose(1, 2)        # shape [g, mn, k], strides (k*aligned, 1, aligned)
    return out if batched else out[0]


def pack_ue8m0(sf: torch.Tensor) -> torch.Tensor:
    """Exponent byte of every fp32 scale (bits 23..30): exact for powers of two, truncating otherwise
    (impls/smxx_layout.cuh:96-100)."""
    return ((sf.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)


def get_mn_major_tma_aligned_packed_ue8m0_tensor(sf: torch.Tensor) -> torch.Tensor:
    """fp32 scales [.., mn, k] -> int32 [.., mn, ceil(k/4)]: four UE8M0 exponent bytes per word (lowest byte = lowest k),
    MN-major with a 16-byte aligned leading dimension (impls/smxx_layout.hpp:178-229)."""
    assert sf.dtype == torch.float32 and sf.dim() in (2, 3)
    batched = sf.dim() == 3
    x = sf if batched else sf.unsqueeze(0)
    g, mn, k = x.shape
    k4 = -(-k // 4)
    exps = torch.zeros((g, mn, k4 * 4), dtype=torch.int32, device=sf.device)
    exps[:, :, :k] = pack_ue8m0(x).to(torch.int32)
    words = exps.view(g, mn, k4, 4)
    packed = words[..., 0] | (words[..., 1] << 8) | (words[..., 2] << 16) | (words[..., 3] << 24)
    aligned = get_tma_aligned_size(mn, 4)
    buf = torch.zeros((g, k4, aligned), dtype=torch.int32, device=sf.device)
    buf[:, :, :mn] = packed.transpose(1, 2)
    out = buf[:, :, :mn].transpose(1, 2)
    return out if batched else out[0]


def transform_sf_into_required_layout(sf: torch.Tensor, mn: int, k: int, recipe: Tuple[int, int, int],
                                      num_groups: Optional[int] = None, is_sfa: bool = False,
                                      disable_ue8m0_cast: bool = False) -> torch.Tensor:
    """The SM100 branch of csrc/apis/layout.hpp:37-92: fp32 scales become packed UE8M0 words, MN-major; B's 128-row blocks
    are first broadcast to one scale per row. e4m3 (NVFP4) scales are returned as their bytes in MN-major order."""
    gran_mn, gran_k = (recipe[0], recipe[2]) if is_sfa else (recipe[1], recipe[2])
    if sf.dtype == torch.float32:
        if gran_mn == 1 and gran_k == 128:
            return get_mn_major_tma_aligned_packed_ue8m0_tensor(sf)
        if gran_mn == 128 and gran_k == 128:
            if disable_ue8m0_cast:
                return sf
            rows = torch.arange(mn, device=sf.device) // 128
            return get_mn_major_tma_aligned_packed_ue8m0_tensor(sf.index_select(-2, rows))
    if sf.dtype in (torch.float8_e4m3fn, torch.uint8) and gran_mn == 1 and gran_k in (16, 32):
        x = sf.view(torch.uint8)
        return x.transpose(-1, -2).contiguous().transpose(-1, -2)
    raise RuntimeError(f"Unknown SF transformation (dtype {sf.dtype}, recipe {tuple(recipe)}, is_sfa={is_sfa})")


def set_tc_util(value: int) -> None:
    """Accepted for compatibility (csrc/apis/runtime.hpp:22-27); the kernels here have no tensor-core throttle."""
    _state["tc_util"] = int(value)


def get_tc_util() -> int:
    return _state["tc_util"]


def set_compile_mode(mode: int) -> None:
    """Accepted for compatibility (csrc/apis/runtime.hpp:28-33); there is nothing to compile at run time."""
    _state["compile_mode"] = int(mode)


def get_compile_mode() -> int:
    return _state["compile_mode"]


def get_arch_pair() -> Tuple[int, int]:
    """(major, minor) compute capability of the current device (csrc/apis/runtime.hpp:37-42)."""
    return tuple(torch.cuda.get_device_capability())


def get_arch_major() -> int:
    return get_arch_pair()[0]
