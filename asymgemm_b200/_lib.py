"""ctypes binding of the C ABI declared in ``include/asymgemm_b200.h``.

There is no CPU or eager fallback: if the shared library is missing, loading fails loudly.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int32, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libasymgemm_b200.so"
TORCH_OPS_PATH = LIB_PATH.with_name("libasymgemm_b200_torch.so")

AG_OK = 0
AG_E_INVALID = -1
AG_E_UNSUPPORTED = -2
AG_E_CUDA = -3
AG_E_NOT_MAPPED = -4
AG_E_DEVICE = -5

LAYOUT_CONTIGUOUS = 0
LAYOUT_MASKED = 1
D_BF16 = 0
D_FP32 = 1
EPILOGUE_NONE, EPILOGUE_SILU_MUL = 0, 1

KIND_BF16, KIND_FP8, KIND_INT8, KIND_NVFP4, KIND_FP8_UE8M0 = 0, 1, 2, 3, 4


class GemmDesc(Structure):
    """Mirror of ``ag_gemm_desc_t``."""

    _fields_ = [
        ("layout", c_int32),
        ("d_dtype", c_int32),
        ("a", c_void_p),
        ("sfa", c_void_p),
        ("b", c_void_p),
        ("sfb", c_void_p),
        ("d", c_void_p),
        ("offsets", c_void_p),
        ("experts", c_void_p),
        ("max_segments", c_int32),
        ("masked_m", c_void_p),
        ("m", c_int64),
        ("n", c_int64),
        ("k", c_int64),
        ("num_groups", c_int32),
        ("scratch", c_void_p),
        ("scratch_bytes", c_uint64),
        ("status", c_void_p),
        ("stream", c_void_p),
        ("num_sms", c_int32),
        ("timeout_ms", c_uint32),
        ("raw_dump", c_void_p),
        ("alpha", c_float),
        ("tile_config", c_int32),
        ("no_split", c_int32),
        ("stage", c_void_p),
        ("stage_bytes", c_uint64),
        ("stage_chunk_bytes", c_uint64),
        ("epilogue", c_int32), ("scatter_meta", c_void_p), ("scatter_bases", c_void_p),
    ]


EP_MAX_RANKS = 16
EP_BAD_EXPERT, EP_OVERFLOW = 64, 65


class EpPeers(Structure):
    """Mirror of ``ag_ep_peers_t``: every rank's four exchange buffers as this process can address them."""

    _fields_ = [("a", c_void_p * EP_MAX_RANKS), ("sfa", c_void_p * EP_MAX_RANKS), ("meta", c_void_p * EP_MAX_RANKS),
                ("ret", c_void_p * EP_MAX_RANKS)]


EXPORTS = [
    "ag_m_grouped_bf16_gemm_nt",
    "ag_m_grouped_fp8_gemm_nt",
    "ag_m_grouped_int8_gemm_nt",
    "ag_m_grouped_fp4_gemm_nt",
    "ag_m_grouped_fp8_gemm_nt_static_scratch",
    "ag_m_grouped_fp8_ue8m0_gemm_nt",
    "ag_fp8_sf_blocked_bytes",
    "ag_fp8_sf_to_blocked_ue8m0",
    "ag_static_scratch_bytes",
    "ag_scratch_bytes",
    "ag_scratch_bytes_for",
    "ag_read_status",
    "ag_set_num_sms",
    "ag_get_num_sms",
    "ag_get_mk_alignment_for_contiguous_layout",
    "ag_fp4_sf_blocked_bytes",
    "ag_fp4_sf_to_blocked",
    "ag_prefetch_staged_weights",
    "ag_prepare_weights",
    "ag_release_weights",
    "ag_measure_host_link",
    "ag_measure_host_stream",
    "ag_link_probe_create",
    "ag_link_probe_run",
    "ag_link_probe_destroy",
    "ag_selftest_wait_limit",
    "ag_probe_mma_issue",
    "ag_probe_operand_feed",
    "ag_quant_rows_fp8",
    "ag_silu_mul_quant_fp8",
    "ag_silu_mul_quant_fp8_upto",
    "ag_quant_rows_fp8_upto",
    "ag_peer_alloc",
    "ag_peer_open",
    "ag_peer_close",
    "ag_peer_free",
    "ag_ep_histogram",
    "ag_ep_plan",
    "ag_ep_dispatch",
    "ag_ep_return",
    "ag_move_rows",
    "ag_combine_topk",
    "ag_quant_rows_int8",
    "ag_silu_mul_quant_int8",
    "ag_combine_topk_f32",
    "ag_gemm_desc_size",
    "ag_last_error",
    "ag_version",
]

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m asymgemm_b200.build`. "
            "asymgemm_b200 has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name in ("ag_m_grouped_bf16_gemm_nt", "ag_m_grouped_fp8_gemm_nt", "ag_m_grouped_int8_gemm_nt",
                 "ag_m_grouped_fp4_gemm_nt", "ag_m_grouped_fp8_gemm_nt_static_scratch", "ag_m_grouped_fp8_ue8m0_gemm_nt"):
        fn = getattr(lib, name)
        fn.argtypes = [POINTER(GemmDesc)]
        fn.restype = c_int32
    lib.ag_static_scratch_bytes.argtypes = []
    lib.ag_static_scratch_bytes.restype = c_uint64
    lib.ag_scratch_bytes.argtypes = [c_int32, c_int64, c_int64, c_int32]
    lib.ag_scratch_bytes.restype = c_uint64
    lib.ag_scratch_bytes_for.argtypes = [c_int32, POINTER(GemmDesc), POINTER(c_uint64)]
    lib.ag_scratch_bytes_for.restype = c_int32
    lib.ag_read_status.argtypes = [c_void_p, c_void_p, POINTER(c_int32)]
    lib.ag_read_status.restype = c_int32
    lib.ag_set_num_sms.argtypes = [c_int32]
    lib.ag_set_num_sms.restype = None
    lib.ag_get_num_sms.argtypes = []
    lib.ag_get_num_sms.restype = c_int32
    lib.ag_get_mk_alignment_for_contiguous_layout.argtypes = []
    lib.ag_get_mk_alignment_for_contiguous_layout.restype = c_int32
    lib.ag_fp8_sf_blocked_bytes.argtypes = [c_int64, c_int64, c_int64]
    lib.ag_fp8_sf_blocked_bytes.restype = c_uint64
    lib.ag_fp8_sf_to_blocked_ue8m0.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p]
    lib.ag_fp8_sf_to_blocked_ue8m0.restype = c_int32
    lib.ag_fp4_sf_blocked_bytes.argtypes = [c_int64, c_int64, c_int64]
    lib.ag_fp4_sf_blocked_bytes.restype = c_uint64
    lib.ag_fp4_sf_to_blocked.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]
    lib.ag_fp4_sf_to_blocked.restype = c_int32
    lib.ag_quant_rows_fp8.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p]
    lib.ag_quant_rows_fp8.restype = c_int32
    lib.ag_silu_mul_quant_fp8.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p]
    lib.ag_silu_mul_quant_fp8.restype = c_int32
    lib.ag_quant_rows_fp8_upto.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p, c_void_p]
    lib.ag_quant_rows_fp8_upto.restype = c_int32
    lib.ag_silu_mul_quant_fp8_upto.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p, c_void_p]
    lib.ag_silu_mul_quant_fp8_upto.restype = c_int32
    lib.ag_peer_alloc.argtypes = [c_uint64, POINTER(c_void_p), c_void_p]
    lib.ag_peer_alloc.restype = c_int32
    lib.ag_peer_open.argtypes = [c_void_p, POINTER(c_void_p)]
    lib.ag_peer_open.restype = c_int32
    lib.ag_peer_close.argtypes = [c_void_p]
    lib.ag_peer_close.restype = c_int32
    lib.ag_peer_free.argtypes = [c_void_p]
    lib.ag_peer_free.restype = c_int32
    lib.ag_ep_histogram.argtypes = [c_void_p, c_int64, c_int32, c_void_p, c_void_p, c_void_p]
    lib.ag_ep_histogram.restype = c_int32
    lib.ag_ep_plan.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                               c_void_p, c_void_p, c_void_p, c_void_p]
    lib.ag_ep_plan.restype = c_int32
    lib.ag_ep_dispatch.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_int32, c_void_p, c_int32, c_int32, c_void_p,
                                   c_void_p, c_int64, c_void_p, POINTER(EpPeers), c_void_p]
    lib.ag_ep_dispatch.restype = c_int32
    lib.ag_ep_return.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, POINTER(EpPeers), c_void_p]
    lib.ag_ep_return.restype = c_int32
    lib.ag_move_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]
    lib.ag_move_rows.restype = c_int32
    lib.ag_combine_topk.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_void_p]
    lib.ag_combine_topk.restype = c_int32
    lib.ag_measure_host_stream.argtypes = [c_uint64, c_int64, c_int32, c_int32, c_int32, c_int32, POINTER(c_double)]
    lib.ag_measure_host_stream.restype = c_int32
    lib.ag_quant_rows_int8.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]
    lib.ag_quant_rows_int8.restype = c_int32
    lib.ag_silu_mul_quant_int8.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]
    lib.ag_silu_mul_quant_int8.restype = c_int32
    lib.ag_combine_topk_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_void_p]
    lib.ag_combine_topk_f32.restype = c_int32
    lib.ag_selftest_wait_limit.argtypes = [c_uint32, c_void_p, c_void_p]
    lib.ag_selftest_wait_limit.restype = c_int32
    lib.ag_probe_mma_issue.argtypes = [c_int32, c_int32, c_int32, ctypes.POINTER(ctypes.c_double)]
    lib.ag_probe_mma_issue.restype = c_int32
    lib.ag_probe_operand_feed.argtypes = [c_int32, c_int32, ctypes.POINTER(ctypes.c_double)]
    lib.ag_probe_operand_feed.restype = c_int32
    lib.ag_prefetch_staged_weights.argtypes = [c_void_p, c_uint64, c_int32, c_void_p, c_uint64, c_uint64, c_void_p, c_int32]
    lib.ag_prefetch_staged_weights.restype = c_int32
    lib.ag_prepare_weights.argtypes = [c_void_p, c_uint64, c_int32]
    lib.ag_prepare_weights.restype = c_int32
    lib.ag_release_weights.argtypes = [c_void_p]
    lib.ag_release_weights.restype = c_int32
    lib.ag_measure_host_link.argtypes = [c_uint64, c_int32, POINTER(c_double)]
    lib.ag_measure_host_link.restype = c_int32
    lib.ag_link_probe_create.argtypes = [c_int32, c_uint64, c_int32, c_int64, POINTER(c_void_p)]
    lib.ag_link_probe_create.restype = c_int32
    lib.ag_link_probe_run.argtypes = [c_void_p, c_double, POINTER(c_double)]
    lib.ag_link_probe_run.restype = c_int32
    lib.ag_link_probe_destroy.argtypes = [c_void_p]
    lib.ag_link_probe_destroy.restype = c_int32
    lib.ag_gemm_desc_size.argtypes = []
    lib.ag_gemm_desc_size.restype = c_uint64
    if int(lib.ag_gemm_desc_size()) != ctypes.sizeof(GemmDesc):
        raise RuntimeError(f"{LIB_PATH} was built from another version of include/asymgemm_b200.h "
                           f"(descriptor of {int(lib.ag_gemm_desc_size())} bytes, this package expects {ctypes.sizeof(GemmDesc)}): rebuild it")
    lib.ag_last_error.argtypes = []
    lib.ag_last_error.restype = c_char_p
    lib.ag_version.argtypes = []
    lib.ag_version.restype = c_char_p
    _lib = lib
    return lib


_torch_ops = None


def torch_ops():
    """`torch.ops.asymgemm_b200` (csrc/torch_ops.cpp, built beside the C library); raises if it has not been built."""
    global _torch_ops
    if _torch_ops is None:
        import torch
        load()                      # the extension links against the C library: load that first, from the same folder
        if not TORCH_OPS_PATH.exists():
            raise RuntimeError(
                f"{TORCH_OPS_PATH} is missing: build it with `python -m asymgemm_b200.build`. "
                "asymgemm_b200 has no CPU or PyTorch fallback."
            )
        torch.ops.load_library(str(TORCH_OPS_PATH))
        _torch_ops = torch.ops.asymgemm_b200
    return _torch_ops


def last_error() -> str:
    return load().ag_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Turn a negative status into the RuntimeError the reference API raises."""
    if rc != AG_OK:
        raise RuntimeError(f"asymgemm_b200: {last_error()} (code {rc})")
