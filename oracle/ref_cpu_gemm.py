"""ctypes binding of the reference's own CPU GEMM library, built into ``oracle/_ref`` by ``oracle/Makefile`` --
TEST INFRASTRUCTURE ONLY (oracle pin, golden-vector generation, timed CPU baseline).

The C ABI bound here is csrc/cpu/cpu_gemm/include/cpu_gemm/cpu_gemm.h:29-63 (``cg_gemm_desc_t``, ``cg_gemm``) and
runtime.h:19-52 of bytedance-iaas/AsymGEMM. The only dtype tuple used is the reference's INT8 weight path:
bf16 activations x int8 ``[N, K]`` weights with per-channel fp32 scales -> fp32 (src/dispatch/gemm.cpp:43-50,255-299).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_size_t, c_void_p
from pathlib import Path

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libcpu_gemm_ref.so"

CG_ROW_MAJOR, CG_NO_TRANS, CG_TRANS = 101, 111, 112
CG_F32, CG_BF16, CG_INT8 = 0, 2, 30


class QuantBlock(Structure):
    _fields_ = [("group_size", c_size_t), ("scale_dtype", c_int), ("has_zero", c_int)]


class GemmDesc(Structure):
    _fields_ = [
        ("order", c_int), ("trans_a", c_int), ("trans_b", c_int), ("offset_c_mode", c_int),
        ("m", c_size_t), ("n", c_size_t), ("k", c_size_t),
        ("alpha", c_float), ("beta", c_float),
        ("a", c_void_p), ("lda", c_size_t), ("dtype_a", c_int), ("block_a", QuantBlock),
        ("b", c_void_p), ("ldb", c_size_t), ("dtype_b", c_int), ("block_b", QuantBlock),
        ("c", c_void_p), ("ldc", c_size_t), ("dtype_c", c_int),
        ("a_scales", c_void_p), ("a_zeros", c_void_p), ("b_scales", c_void_p), ("b_zeros", c_void_p),
        ("output_offsets", c_void_p),
    ]


_lib = None
_rt = {}


def available() -> bool:
    return LIB_PATH.exists()


def load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(LIB_PATH))
        lib.cg_runtime_create.argtypes = [c_int]
        lib.cg_runtime_create.restype = c_void_p
        lib.cg_runtime_threads.argtypes = [c_void_p]
        lib.cg_runtime_threads.restype = c_int
        lib.cg_gemm.argtypes = [c_void_p, POINTER(GemmDesc)]
        lib.cg_gemm.restype = c_int
        lib.cg_int8_rm_backend_name.restype = c_char_p
        lib.cg_int8_rm_backend_ok.restype = c_int
        _lib = lib
    return _lib


def runtime(threads: int = 0):
    """One worker pool per requested size, kept for the life of the process (0 = all hardware threads)."""
    lib = load()
    if threads not in _rt:
        _rt[threads] = lib.cg_runtime_create(threads)
    return _rt[threads]


def backend_name() -> str:
    return load().cg_int8_rm_backend_name().decode()


def threads(rt) -> int:
    return int(load().cg_runtime_threads(rt))


def gemm_bf16_int8_f32(a_bf16_bits: np.ndarray, b_int8: np.ndarray, b_scales: np.ndarray, rt=None) -> np.ndarray:
    """C[m, n] = A[m, k] (bf16 bit patterns) x B[n, k]^T (int8, per-channel fp32 scales) through ``cg_gemm``.

    The library quantises every row of A to int8 with scale amax/127 before multiplying
    (src/kernels/amx/int8_buffers.h:60-123) and returns a_scale[m] * b_scale[n] * int32 sum in fp32.
    """
    lib = load()
    rt = rt if rt is not None else runtime(0)
    a = np.ascontiguousarray(a_bf16_bits, dtype=np.uint16)
    b = np.ascontiguousarray(b_int8, dtype=np.int8)
    s = np.ascontiguousarray(b_scales, dtype=np.float32)
    m, k = a.shape
    n = b.shape[0]
    c = np.zeros((m, n), dtype=np.float32)
    d = GemmDesc()
    d.order, d.trans_a, d.trans_b, d.offset_c_mode = CG_ROW_MAJOR, CG_NO_TRANS, CG_TRANS, 0
    d.m, d.n, d.k = m, n, k
    d.alpha, d.beta = 1.0, 0.0
    d.a, d.lda, d.dtype_a = a.ctypes.data, k, CG_BF16
    d.b, d.ldb, d.dtype_b = b.ctypes.data, k, CG_INT8
    d.c, d.ldc, d.dtype_c = c.ctypes.data, n, CG_F32
    d.b_scales = s.ctypes.data
    rc = lib.cg_gemm(rt, ctypes.byref(d))
    if rc != 0:
        raise RuntimeError(f"cg_gemm returned {rc}")
    return c


def exact_int32_block_sums(a_q: np.ndarray, b_q: np.ndarray, rt=None) -> np.ndarray:
    """int32 [K/128, M, N] computed by the reference library itself.

    Every row of ``a_q`` must contain a +-127 so that the library's per-row quantiser recovers the int8 values with
    scale exactly 1; with unit weight scales and K sliced per 128 the fp32 result is the exact integer block sum.
    """
    from .oracle import f32_to_bf16_bits
    m, k = a_q.shape
    n = b_q.shape[0]
    assert k % 128 == 0
    assert (np.abs(a_q.astype(np.int32)).max(axis=1) == 127).all(), "each row needs a +-127"
    ones = np.ones(n, dtype=np.float32)
    out = np.empty((k // 128, m, n), dtype=np.int32)
    for i in range(k // 128):
        a_blk = a_q[:, i * 128:(i + 1) * 128]
        # rows whose +-127 lies in another block still need amax == 127 inside this block: handled by the caller
        bits = f32_to_bf16_bits(a_blk.astype(np.float32))
        c = gemm_bf16_int8_f32(bits, b_q[:, i * 128:(i + 1) * 128], ones, rt)
        out[i] = np.rint(c).astype(np.int32)
    return out
