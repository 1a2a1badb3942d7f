from .math import (  # noqa: F401
    align,
    ceil_div,
    ceil_to_ue8m0,
    per_block_cast_to_fp8,
    per_channel_cast_to_fp8,
    per_custom_dims_cast_to_fp8,
    per_token_cast_to_fp4,
    transpose_packed_fp4,
    per_channel_cast_to_int8,
    per_token_cast_to_fp8,
    per_token_cast_to_int8,
    per_token_cast_to_nvfp4_e4m3,
)
from .layout import build_contiguous_layout, get_mk_alignment_for_contiguous_layout, get_tma_aligned_size  # noqa: F401
