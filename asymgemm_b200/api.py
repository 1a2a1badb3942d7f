"""Operator API of the m-grouped asymmetric GEMM, with the reference's names, argument order and meaning.

Mirrors ``asym_gemm.m_grouped_{bf16,fp8,fp4,int8}_asym_gemm_nt_{contiguous,masked}`` (pybind signatures in
csrc/apis/gemm.hpp:1034-1115 of the reference): tensors are caller-owned, ``d`` is written in place, the
launch is asynchronous on torch's current CUDA stream, failures raise ``RuntimeError``. Every call goes
through the C ABI of ``libasymgemm_b200.so``; there is no PyTorch or CPU fallback.

Differences from the reference, all on the permissive side:
  * ``compiled_dims`` is accepted and ignored (kernels are compiled ahead of time).
  * ``list_size`` may be an int or a one-element tensor; passing ``None`` avoids the device sync that
    reading a CUDA tensor costs (the kernel stops at the -1 terminator of ``experts`` by itself).
  * fp32 FP8 scales are applied exactly in fp32; ``disable_ue8m0_cast`` therefore changes nothing.
  * INT8 runs on sm_100a (the reference raises there) and ``d`` may be bf16 or fp32.
  * B that is neither CUDA nor pinned raises instead of faulting.
"""
from __future__ import annotations

import contextlib
import threading
import weakref
from typing import Optional, Tuple, Union

import torch

from . import _lib

_MK_ALIGNMENT = 128
_state = {"timeout_ms": 0, "use_scratch": True, "tile_config": 0, "no_split": 0, "fp8_ue8m0": False,
          "weight_path": "stream", "stage_bytes": 128 << 20, "stage_slots": 2}
_call_caps = threading.local()
_scratch_cache: dict = {}
_stager_cache: dict = {}
_status_cache: dict = {}
_dev_copy_cache: dict = {}


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(f"Assertion error (asymgemm_b200): {msg}")


def get_mk_alignment_for_contiguous_layout() -> int:
    """Rows every contiguous-layout segment must be padded to (csrc/utils/layout.hpp:108-110)."""
    return _MK_ALIGNMENT


def set_num_sms(num_sms: int) -> None:
    """Cap the CTAs each launch may use (csrc/apis/runtime.hpp:15-21)."""
    _lib.load().ag_set_num_sms(int(num_sms))


def get_num_sms() -> int:
    return int(_lib.load().ag_get_num_sms())


@contextlib.contextmanager
def launch_sm_cap(num_sms: int):
    """Within the block, every operator call of this thread launches at most `num_sms` CTAs (`num_sms` of the C
    descriptor). Unlike `set_num_sms` this touches no process-wide state: other threads, other devices and calls after
    the block are unaffected. 0 or None leaves the calls alone."""
    prev = getattr(_call_caps, "num_sms", 0)
    _call_caps.num_sms = int(num_sms) if num_sms else 0
    try:
        yield
    finally:
        _call_caps.num_sms = prev


def set_wait_limit_ms(ms: int) -> None:
    """Bound (milliseconds) on every in-kernel barrier wait; 0 restores the default."""
    _state["timeout_ms"] = int(ms)


def set_tile_config(tile: int) -> None:
    """Force a tile configuration (see ``ag_gemm_desc_t.tile_config``); 0 = choose from where B lives."""
    _state["tile_config"] = int(tile)


def set_fp8_scale_mode(mode: str) -> None:
    """How the FP8 entry points apply their fp32 block scales when the call does not say (`ue8m0_scales=None`):
    "fp32" (default) multiplies by the exact fp32 scales in the TMEM drain; "ue8m0" lets the tensor core apply them as
    power-of-two factors like the reference's SM100 kernel (mantissas are dropped: use it with scales produced by
    `use_ue8m0=True` quantisers). The hardware path needs 128-row aligned segments / M_max."""
    if mode not in ("fp32", "ue8m0"):
        raise RuntimeError("mode must be 'fp32' or 'ue8m0'")
    _state["fp8_ue8m0"] = mode == "ue8m0"


def set_split_segments(flag: bool) -> None:
    """Device-resident B only: whether long segments are split into row chunks across CTAs (default) or kept whole."""
    _state["no_split"] = 0 if flag else 1


def set_weight_path(path: str, chunk_bytes: Optional[int] = None, slots: Optional[int] = None) -> None:
    """How host-resident weights reach the GPU (extension; weights already in HBM are unaffected).

    "stream" (default): the GEMM kernel reads pinned memory itself and fetches only the experts that received rows.
    "staged": the copy engine moves every expert, about `chunk_bytes` (default 128 MiB) of whole experts at a time, into
    a double buffer in HBM while the grouped GEMM of the previous chunk runs from there (`stage` of the C descriptor; this
    module owns one such buffer per device; `slots` > 2 makes it a ring of that many chunks, which lets
    `prefetch_weights` bank more of the next call's weights while the link would otherwise idle); same results, a few percent
    more of the link, for calls in which (nearly) all experts are active.
    "auto": staged for calls that can have rows for every expert (contiguous: at least 128 rows of `a` per expert, the
    padded size of one active expert; masked: `expected_m` >= 8) over at least 256 MiB of weights, the in-kernel stream
    otherwise (decode-sized batches, where most experts get no rows: 8 tokens x top-8 over 256 experts take 33 ms
    streamed and 135 ms staged). The reference's unified runtime stages its
    streamed partition the same way, by default (`_StageRing`, asym_gemm/unified_moe/runtime.py:110-200; its in-kernel
    reads reach 21.5 of the copy engine's 50 GB/s); here the in-kernel stream reaches 0.92 of the copy engine's rate, so
    staging is the option and the stream the default."""
    _require(path in ("stream", "staged", "auto"), "weight path must be 'stream', 'staged' or 'auto'")
    _state["weight_path"] = path
    if chunk_bytes is not None:
        _require(int(chunk_bytes) > 0, "chunk_bytes must be positive")
        _state["stage_bytes"] = int(chunk_bytes)
    if slots is not None:
        _require(2 <= int(slots) <= 8, "slots must be 2 .. 8")
        _state["stage_slots"] = int(slots)


def get_weight_path() -> str:
    return _state["weight_path"]


def prefetch_weights(b: torch.Tensor, device: Union[torch.device, int, None] = None) -> None:
    """With the "staged" weight path: start copying the first chunks (as many as the staging ring has slots, see
    `set_weight_path`) of the host-resident weights `b` into HBM now, ahead of the operator call that will use them -- the
    next layer's weights while this layer's results are still being exchanged and combined, when the host link would idle
    otherwise. The next staged call on the same `b` does not copy them again. The copies begin once the work already
    queued on the current stream has finished. Does nothing on the other weight paths (measured: handing the prefetched
    experts to the in-kernel stream as a separate launch gains nothing) and for weights on the GPU. The weights must not
    change between this call and that one."""
    if _state["weight_path"] != "staged" or b.is_cuda:
        return
    _require(b.dim() == 3 and b.is_contiguous() and b.is_pinned(), "weights must be a contiguous pinned [G, N, K] tensor")
    dev = torch.device("cuda", torch.cuda.current_device() if device is None else (device if isinstance(device, int) else device.index))
    g = int(b.shape[0])
    stage, slot_bytes = _stage_buffer(b, g, dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().ag_prefetch_staged_weights(b.data_ptr(), b.numel() * b.element_size() // g, g,
                                                          stage.data_ptr(), stage.numel(), slot_bytes,
                                                          torch.cuda.current_stream(dev).cuda_stream, 1))


def prepare_weights(b: torch.Tensor, read_only: bool = False) -> torch.Tensor:
    """Page-lock and map an ordinary (pageable) CPU tensor in place so that it can be passed as `b` (extension; the
    reference registers its weight slabs the same way, asym_gemm/unified_moe/runtime.py:236-279). A tensor that is
    already pinned or on the GPU is returned untouched. Keep the tensor alive, and call `release_weights` before its
    memory is freed."""
    _require(b.is_contiguous(), "weights must be contiguous")
    if b.is_cuda or b.is_pinned():
        return b
    _lib.check(_lib.load().ag_prepare_weights(b.data_ptr(), b.numel() * b.element_size(), 1 if read_only else 0))
    return b


def release_weights(b: torch.Tensor) -> None:
    """Undo `prepare_weights` for this tensor's memory (raises for memory it did not register)."""
    _lib.check(_lib.load().ag_release_weights(b.data_ptr()))


def set_use_scratch(flag: bool) -> None:
    """Whether long segments replay their weight column from device scratch (default) or re-read B."""
    _state["use_scratch"] = bool(flag)


def _status_word(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_cache.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_cache[key] = t
    return t


def check_status(device: Union[torch.device, int, None] = None, reset: bool = True) -> None:
    """Synchronise and raise ``RuntimeError`` if any kernel since the last check reported a status word."""
    dev = torch.device("cuda", torch.cuda.current_device() if device is None else (device if isinstance(device, int) else device.index))
    word = _status_word(dev)
    torch.cuda.synchronize(dev)
    v = int(word.item())
    if v != 0:
        lib = _lib.load()
        out = _lib.c_int32(0)
        lib.ag_read_status(word.data_ptr(), torch.cuda.current_stream(dev).cuda_stream, out)
        msg = _lib.last_error()
        if reset:
            word.zero_()
        raise RuntimeError(f"asymgemm_b200: {msg}")


def _scratch(kind: int, n: int, k: int, device: torch.device) -> Optional[torch.Tensor]:
    """Replay scratch for the launch about to be made: one buffer per (device, stream), because launches on different
    streams may overlap on the GPU and each CTA keeps its current weight column there."""
    if not _state["use_scratch"]:
        return None
    lib = _lib.load()
    need = int(lib.ag_scratch_bytes(kind, n, k, 0))
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    t = _scratch_cache.get(key)
    if t is None or t.numel() < need + 1024:
        if len(_scratch_cache) >= 8:
            _scratch_cache.clear()
        t = torch.empty(need + 1024, dtype=torch.uint8, device=device)
        _scratch_cache[key] = t
    off = (-t.data_ptr()) % 1024
    return t[off:off + need]


def _cache_get(cache: dict, t: torch.Tensor, device: torch.device):
    """Entries are tied to the identity of the source tensor object (a weak reference), its in-place version counter
    and its address: a new tensor that happens to reuse a freed tensor's memory never hits."""
    hit = cache.get((id(t), device.index))
    if hit is not None and hit[0]() is t and hit[1] == t._version and hit[2] == t.data_ptr():
        return hit[3]
    return None


def _cache_put(cache: dict, t: torch.Tensor, device: torch.device, value) -> None:
    key = (id(t), device.index)
    if len(cache) > 512:
        for k in [k for k, v in cache.items() if v[0]() is None]:
            del cache[k]
        if len(cache) > 512:
            cache.clear()
    cache[key] = (weakref.ref(t), t._version, t.data_ptr(), value)


def _device_copy(t: torch.Tensor, device: torch.device) -> torch.Tensor:
    """Device-resident copy of a small host tensor (weight scales), cached while the same tensor object is passed
    again unmodified."""
    if t.is_cuda:
        return t
    hit = _cache_get(_dev_copy_cache, t, device)
    if hit is not None:
        return hit
    dev = t.to(device)   # blocking, once per weight tensor: the cached copy may be used from any stream afterwards
    _cache_put(_dev_copy_cache, t, device, dev)
    return dev


def _list_size_to_segments(list_size, offsets: torch.Tensor, experts: torch.Tensor) -> int:
    cap = min(offsets.numel() // 2, experts.numel())
    if list_size is None:
        return cap
    if isinstance(list_size, torch.Tensor):
        _require(list_size.numel() == 1, "list_size tensor must have one element")
        list_size = int(list_size.item())
    # list_size counts the -1 terminator (tests/m_grouped/...:47-51 of the reference)
    return max(0, min(int(list_size), cap))


def _check_b_residency(b: torch.Tensor) -> None:
    _require(b.is_cuda or b.is_pinned(), "b must be a CUDA tensor or pinned host memory (b.is_cuda() or b.is_pinned())")


def _common_checks(a, b, d, masked: bool, k_div: int = 1, d_col_div: int = 1):
    """`d_col_div` = 2: d has half the columns of the product (fused SiLU*mul epilogue)."""
    if masked:
        _require(a.dim() == 3 and b.dim() == 3 and d.dim() == 3, "masked layout wants a [G,M,K], b [G,N,K], d [G,M,N]")
        g, m, k = a.shape
        g_, n, k_ = b.shape
        g__, m_, n_ = d.shape
        _require(g == g_ == g__ and m == m_ and n == n_ * d_col_div and k == k_, "shape mismatch between a, b and d")
    else:
        _require(a.dim() == 2 and b.dim() == 3 and d.dim() == 2, "contiguous layout wants a [M,K], b [G,N,K], d [M,N]")
        m, k = a.shape
        g, n, k_ = b.shape
        m_, n_ = d.shape
        _require(m == m_ and n == n_ * d_col_div and k == k_, "shape mismatch between a, b and d")
    _require(n > 0 and k > 0 and g > 0, "n, k and num_groups must be positive")
    _require(a.is_cuda, "a must be a CUDA tensor")
    _require(d.is_cuda or d.is_pinned(), "d must be a CUDA tensor (or, as an extension, pinned host memory the kernel writes directly)")
    _require(a.is_contiguous(), "a must be K-major (contiguous)")
    _require(b.is_contiguous(), "b must be K-major [G, N, K] (contiguous)")
    _require(d.is_contiguous(), "d must be row-major (contiguous)")
    _require(d.dtype in (torch.bfloat16, torch.float32), "d must be bfloat16 or float32")
    _check_b_residency(b)
    return int(g), int(m), int(n), int(k * k_div)


# "auto" weight path: stage when the call can have rows for (nearly) every expert and the weights are large enough for
# the per-chunk launches to disappear behind the copies. Only the device knows which experts are active, so the rule
# reads what the host has: a contiguous layout pads every active expert to 128 rows, so fewer than 128 rows of `a` per
# expert prove that some experts are idle; a masked call states its expected rows per group. (256 experts, Zipf(0.8)
# routing, K=7168, N=4096: the two paths tie near 4 valid rows per expert; 8 tokens x top-8 take 33 ms streamed and
# 135 ms staged, 512 tokens 150 and 136.)
_AUTO_ROWS_PER_EXPERT = {_lib.LAYOUT_CONTIGUOUS: 128, _lib.LAYOUT_MASKED: 8}
_AUTO_MIN_WEIGHT_BYTES = 256 << 20


def _use_staging(b: torch.Tensor, g: int, rows: int, layout: int, raw_dump) -> bool:
    mode = _state["weight_path"]
    if mode == "stream" or b.is_cuda or raw_dump is not None:
        return False
    if mode == "staged":
        return True
    return rows >= _AUTO_ROWS_PER_EXPERT[layout] * g and b.numel() * b.element_size() >= _AUTO_MIN_WEIGHT_BYTES


def _stage_buffer(b: torch.Tensor, g: int, device: torch.device) -> Tuple[torch.Tensor, int]:
    """(ring buffer in HBM for the staged weight path, bytes of one slot): one buffer per device, `stage_slots` slots of
    one chunk of whole experts of `b` each. The library orders the copies into it after the GEMMs of earlier calls that
    read it, on whichever stream they ran."""
    group_bytes = b.numel() * b.element_size() // g
    chunk = max(1, min(g, _state["stage_bytes"] // max(1, group_bytes)))
    slot = (chunk * group_bytes + 1023) // 1024 * 1024
    need = _state["stage_slots"] * slot
    t = _stager_cache.get(device.index)
    if t is None or t.numel() < need + 1024:
        # a buffer that is replaced goes back to the allocator only after the GEMMs that read it: wait for them here
        if t is not None:
            torch.cuda.synchronize(device)
        t = torch.empty(need + 1024, dtype=torch.uint8, device=device)
        _stager_cache[device.index] = t
    off = (-t.data_ptr()) % 1024
    return t[off:off + need], slot


def _launch(kind: int, fn_name: str, *, layout: int, a, sfa, b, sfb, d, offsets=None, experts=None, max_segments=0,
            masked_m=None, m: int, n: int, k: int, g: int, raw_dump=None, alpha: float = 1.0,
            rows_hint: Optional[int] = None, epilogue: int = 0, scatter=None) -> None:
    """Every operator ends here: one call of the torch extension's op, which fills the C descriptor from the tensors and
    launches on the current stream of a's device (csrc/torch_ops.cpp). `rows_hint`: rows the call is expected to
    multiply (masked layout: expected_m * groups; contiguous: m), for the "auto" weight path."""
    dev = a.device
    stage, slot_bytes = (_stage_buffer(b, g, dev) if _use_staging(b, g, m if rows_hint is None else rows_hint, layout, raw_dump)
                         else (None, 0))
    op = _lib.torch_ops().m_grouped_gemm_nt
    with torch.cuda.device(dev):
        op(kind, layout, a, sfa, b, sfb, d, offsets, experts, max_segments, masked_m, m, n, k, g, _scratch(kind, n, k, dev),
           _status_word(dev), _state["timeout_ms"], raw_dump, alpha, _state["tile_config"], _state["no_split"], stage, slot_bytes,
           getattr(_call_caps, "num_sms", 0), epilogue, None if scatter is None else scatter[0], None if scatter is None else scatter[1])


def _check_index_tensors(offsets, experts, g):
    _require(offsets.is_cuda and experts.is_cuda, "offsets and experts must be CUDA tensors")
    _require(offsets.is_contiguous() and experts.is_contiguous(), "offsets and experts must be contiguous")
    _require(offsets.dtype == torch.int32 and experts.dtype == torch.int32, "offsets and experts must be int32")


# --------------------------------------------------------------------------------------------- BF16
def m_grouped_bf16_asym_gemm_nt_contiguous(a, b, d, offsets, experts, list_size=None, compiled_dims: str = "nk",
                                           transpose_b: bool = False) -> None:
    """``d[rows of segment i] = a[rows] @ b[experts[i]].T`` in bf16 (csrc/apis/gemm.hpp:370-418, 679-732)."""
    _require(not transpose_b, "transpose_b=True (MN-major B) is not supported")
    g, m, n, k = _common_checks(a, b, d, masked=False)
    _require(a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "a and b must be bfloat16")
    _check_index_tensors(offsets, experts, g)
    if m == 0:
        return
    segs = _list_size_to_segments(list_size, offsets, experts)
    _launch(_lib.KIND_BF16, "ag_m_grouped_bf16_gemm_nt", layout=_lib.LAYOUT_CONTIGUOUS, a=a, sfa=None, b=b, sfb=None, d=d,
            offsets=offsets, experts=experts, max_segments=segs, m=m, n=n, k=k, g=g)


def m_grouped_bf16_asym_gemm_nt_masked(a, b, d, masked_m, expected_m: int, compiled_dims: str = "nk") -> None:
    """Masked layout: group ``g`` multiplies its first ``masked_m[g]`` rows (csrc/apis/gemm.hpp:420-486)."""
    g, m, n, k = _common_checks(a, b, d, masked=True)
    _require(a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "a and b must be bfloat16")
    _require(masked_m.is_cuda and masked_m.dtype == torch.int32 and masked_m.is_contiguous() and masked_m.numel() == g,
             "masked_m must be a contiguous int32 CUDA tensor with one entry per group")
    if m == 0 or expected_m == 0:
        return
    _launch(_lib.KIND_BF16, "ag_m_grouped_bf16_gemm_nt", layout=_lib.LAYOUT_MASKED, a=a, sfa=None, b=b, sfb=None, d=d,
            masked_m=masked_m, m=m, n=n, k=k, g=g, rows_hint=int(expected_m) * g)


# --------------------------------------------------------------------------------------------- FP8
def _fp8_scales(a, b, g, rows_shape, n, k, recipe):
    a_q, sfa = a
    b_q, sfb = b
    _require(a_q.dtype == torch.float8_e4m3fn and b_q.dtype == torch.float8_e4m3fn, "a and b must be float8_e4m3fn")
    if recipe is not None:
        _require(tuple(recipe) == (1, 128, 128), f"Unknown SF transformation for recipe {tuple(recipe)}")
    kb = (k + 127) // 128
    _require(sfa.dtype == torch.float32 and sfb.dtype == torch.float32, "scales must be float32")
    _require(tuple(sfa.shape) == (*rows_shape, kb), f"sfa must be {(*rows_shape, kb)}, got {tuple(sfa.shape)}")
    _require(tuple(sfb.shape) == (g, (n + 127) // 128, kb), f"sfb must be {(g, (n + 127) // 128, kb)}, got {tuple(sfb.shape)}")
    _require(sfa.is_cuda, "sfa must be a CUDA tensor")
    return sfa.contiguous(), _device_copy(sfb.contiguous(), a_q.device)


def _fp8_blocked_ue8m0(sf: torch.Tensor, groups: int, rows: int, kb: int, rows_per_scale: int, device, cache: bool) -> torch.Tensor:
    """fp32 scales -> blocked UE8M0 device buffer for the hardware-scaled FP8 kernel (weights: once, cached)."""
    lib = _lib.load()
    if cache:
        hit = _cache_get(_blocked_cache, sf, device)
        if hit is not None:
            return hit
    out = torch.empty(int(lib.ag_fp8_sf_blocked_bytes(groups, rows, kb)), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _lib.check(lib.ag_fp8_sf_to_blocked_ue8m0(sf.data_ptr(), out.data_ptr(), groups, rows, kb, rows_per_scale,
                                                  torch.cuda.current_stream(device).cuda_stream))
    if cache:
        torch.cuda.current_stream(device).synchronize()
        _cache_put(_blocked_cache, sf, device, out)
    return out


def _fp8_use_hw(ue8m0_scales: Optional[bool]) -> bool:
    return _state["fp8_ue8m0"] if ue8m0_scales is None else bool(ue8m0_scales)


def m_grouped_fp8_asym_gemm_nt_contiguous(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor], d,
                                          offsets, experts, list_size=None,
                                          recipe: Optional[Tuple[int, int, int]] = None, compiled_dims: str = "nk",
                                          disable_ue8m0_cast: bool = False, *, ue8m0_scales: Optional[bool] = None,
                                          epilogue: Optional[str] = None,
                                          scatter: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> None:
    """FP8 E4M3 with 1x128 (A) and 128x128 (B) fp32 scales, bf16 out (csrc/apis/gemm.hpp:81-157).

    ``ue8m0_scales`` (extension): True = apply the scales in the tensor core as power-of-two factors (the reference's
    SM100 numerics; segments must be 128-row aligned), False = exact fp32 in the drain, None = `set_fp8_scale_mode`.
    ``epilogue="silu_mul"`` (extension, exact-scale mode only): the gate+up GEMM of an MoE layer with its activation fused
    into the drain: `b` holds gate and up rows interleaved in groups of 16 (`ep.interleave_gate_up`), `d` is bf16
    [M, N/2] = bf16(silu(gate) * up) -- the bits the unfused GEMM plus the activation kernel produce.
    ``scatter=(meta, bases)`` (extension): result row r goes to row ``meta[r] & 0xffffffff`` of the buffer at address
    ``bases[meta[r] >> 32]`` instead of ``d[r]`` (int64 CUDA tensors; negative entries drop the row); the buffers may be
    peer memory -- the expert-parallel layer's down GEMM sends its results home this way (`scatter_meta` of the C descriptor).
    """
    _require(epilogue in (None, "silu_mul"), "epilogue must be None or 'silu_mul'")
    fused = epilogue == "silu_mul"
    g, m, n, k = _common_checks(a[0], b[0], d, masked=False, d_col_div=2 if fused else 1)
    _check_index_tensors(offsets, experts, g)
    sfa, sfb = _fp8_scales(a, b, g, (m,), n, k, recipe)
    if m == 0:
        return
    segs = _list_size_to_segments(list_size, offsets, experts)
    if scatter is not None:
        _require(len(scatter) == 2 and all(t.is_cuda and t.dtype == torch.int64 and t.is_contiguous() for t in scatter),
                 "scatter must be (meta, bases): contiguous int64 CUDA tensors")
        _require(scatter[0].numel() >= m, "scatter meta needs one entry per row of a")
    if fused:
        _require(not _fp8_use_hw(ue8m0_scales), "the fused SiLU*mul epilogue exists for the exact fp32-scale mode only")
        _require(n % 256 == 0 and d.dtype == torch.bfloat16, "the fused SiLU*mul epilogue needs n % 256 == 0 and a bf16 d")
        _launch(_lib.KIND_FP8, "ag_m_grouped_fp8_gemm_nt", layout=_lib.LAYOUT_CONTIGUOUS, a=a[0], sfa=sfa, b=b[0], sfb=sfb, d=d,
                offsets=offsets, experts=experts, max_segments=segs, m=m, n=n, k=k, g=g, epilogue=_lib.EPILOGUE_SILU_MUL, scatter=scatter)
        return
    if _fp8_use_hw(ue8m0_scales):
        kb, dev = (k + 127) // 128, a[0].device
        sfa_b = _fp8_blocked_ue8m0(sfa, 1, m, kb, 1, dev, cache=False)
        cacheable = b[1].is_contiguous() and (b[1].is_cuda or b[1].is_pinned())
        sfb_b = _fp8_blocked_ue8m0(b[1] if cacheable else sfb, g, n, kb, 128, dev, cache=cacheable)
        _launch(_lib.KIND_FP8_UE8M0, "ag_m_grouped_fp8_ue8m0_gemm_nt", layout=_lib.LAYOUT_CONTIGUOUS, a=a[0], sfa=sfa_b, b=b[0], sfb=sfb_b,
                d=d, offsets=offsets, experts=experts, max_segments=segs, m=m, n=n, k=k, g=g, scatter=scatter)
        return
    _launch(_lib.KIND_FP8, "ag_m_grouped_fp8_gemm_nt", layout=_lib.LAYOUT_CONTIGUOUS, a=a[0], sfa=sfa, b=b[0], sfb=sfb, d=d,
            offsets=offsets, experts=experts, max_segments=segs, m=m, n=n, k=k, g=g, scatter=scatter)


def m_grouped_fp8_asym_gemm_nt_masked(a, b, d, masked_m, expected_m: int, recipe=None, compiled_dims: str = "nk",
                                      disable_ue8m0_cast: bool = False, *, ue8m0_scales: Optional[bool] = None) -> None:
    """Masked FP8 (csrc/apis/gemm.hpp:159-235). ``ue8m0_scales``: see the contiguous entry point (needs M_max % 128 == 0)."""
    g, m, n, k = _common_checks(a[0], b[0], d, masked=True)
    sfa, sfb = _fp8_scales(a, b, g, (g, m), n, k, recipe)
    _require(masked_m.is_cuda and masked_m.dtype == torch.int32 and masked_m.is_contiguous() and masked_m.numel() == g,
             "masked_m must be a contiguous int32 CUDA tensor with one entry per group")
    if m == 0 or expected_m == 0:
        return
    if _fp8_use_hw(ue8m0_scales):
        _require(m % 128 == 0, "the hardware-scaled FP8 path needs M_max to be a multiple of 128")
        kb, dev = (k + 127) // 128, a[0].device
        sfa_b = _fp8_blocked_ue8m0(sfa, 1, g * m, kb, 1, dev, cache=False)
        cacheable = b[1].is_contiguous() and (b[1].is_cuda or b[1].is_pinned())
        sfb_b = _fp8_blocked_ue8m0(b[1] if cacheable else sfb, g, n, kb, 128, dev, cache=cacheable)
        _launch(_lib.KIND_FP8_UE8M0, "ag_m_grouped_fp8_ue8m0_gemm_nt", layout=_lib.LAYOUT_MASKED, a=a[0], sfa=sfa_b, b=b[0], sfb=sfb_b, d=d,
                masked_m=masked_m, m=m, n=n, k=k, g=g, rows_hint=int(expected_m) * g)
        return
    _launch(_lib.KIND_FP8, "ag_m_grouped_fp8_gemm_nt", layout=_lib.LAYOUT_MASKED, a=a[0], sfa=sfa, b=b[0], sfb=sfb, d=d,
            masked_m=masked_m, m=m, n=n, k=k, g=g, rows_hint=int(expected_m) * g)


# --------------------------------------------------------------------------------------------- INT8
def _int8_scales(a, b, g, rows_shape, n, k):
    a_q, sfa = a
    b_q, sfb = b
    _require(a_q.dtype == torch.int8 and b_q.dtype == torch.int8, "a and b must be int8")
    _require(k % 128 == 0, "k must be a multiple of 128")  # sm90_int8_asym_gemm_1d1d.hpp:226-227
    kb = k // 128
    _require(sfa.dtype == torch.float32 and sfb.dtype == torch.float32, "scales must be float32")
    _require(tuple(sfa.shape) == (*rows_shape, kb), f"sfa must be {(*rows_shape, kb)}, got {tuple(sfa.shape)}")
    _require(tuple(sfb.shape) == (g, n, kb), f"sfb must be {(g, n, kb)}, got {tuple(sfb.shape)}")
    _require(sfa.is_cuda, "sfa must be a CUDA tensor")
    return sfa.contiguous(), _device_copy(sfb.contiguous(), a_q.device)


def m_grouped_int8_asym_gemm_nt_contiguous(a, b, d, offsets, experts, list_size=None, recipe=None,
                                           compiled_dims: str = "nk", *, raw_accumulators: Optional[torch.Tensor] = None) -> None:
    """INT8 with per-token (A) and per-channel (B) fp32 scales per 128-wide K block (csrc/apis/gemm.hpp:569-600).

    ``raw_accumulators`` (extension): int32 CUDA tensor ``[K/128, M, N]`` that receives the exact block sums.
    """
    g, m, n, k = _common_checks(a[0], b[0], d, masked=False)
    _check_index_tensors(offsets, experts, g)
    sfa, sfb = _int8_scales(a, b, g, (m,), n, k)
    if raw_accumulators is not None:
        _require(raw_accumulators.is_cuda and raw_accumulators.dtype == torch.int32 and raw_accumulators.is_contiguous()
                 and tuple(raw_accumulators.shape) == (k // 128, m, n), "raw_accumulators must be int32 [K/128, M, N] on CUDA")
    if m == 0:
        return
    segs = _list_size_to_segments(list_size, offsets, experts)
    _launch(_lib.KIND_INT8, "ag_m_grouped_int8_gemm_nt", layout=_lib.LAYOUT_CONTIGUOUS, a=a[0], sfa=sfa, b=b[0], sfb=sfb, d=d,
            offsets=offsets, experts=experts, max_segments=segs, m=m, n=n, k=k, g=g, raw_dump=raw_accumulators)


def m_grouped_int8_asym_gemm_nt_masked(a, b, d, masked_m, expected_m: int, recipe=None, compiled_dims: str = "nk", *,
                                       raw_accumulators: Optional[torch.Tensor] = None) -> None:
    """Masked INT8 (csrc/apis/gemm.hpp:602-630)."""
    g, m, n, k = _common_checks(a[0], b[0], d, masked=True)
    sfa, sfb = _int8_scales(a, b, g, (g, m), n, k)
    _require(masked_m.is_cuda and masked_m.dtype == torch.int32 and masked_m.is_contiguous() and masked_m.numel() == g,
             "masked_m must be a contiguous int32 CUDA tensor with one entry per group")
    if raw_accumulators is not None:
        _require(raw_accumulators.is_cuda and raw_accumulators.dtype == torch.int32 and raw_accumulators.is_contiguous()
                 and tuple(raw_accumulators.shape) == (k // 128, g * m, n), "raw_accumulators must be int32 [K/128, G*M, N] on CUDA")
    if m == 0 or expected_m == 0:
        return
    _launch(_lib.KIND_INT8, "ag_m_grouped_int8_gemm_nt", layout=_lib.LAYOUT_MASKED, a=a[0], sfa=sfa, b=b[0], sfb=sfb, d=d,
            masked_m=masked_m, m=m, n=n, k=k, g=g, rows_hint=int(expected_m) * g, raw_dump=raw_accumulators)


# --------------------------------------------------------------------------------------------- NVFP4
_blocked_cache: dict = {}


def _fp4_blocked(sf: torch.Tensor, groups: int, rows: int, k16: int, device: torch.device, cache: bool) -> torch.Tensor:
    """Scales [groups, rows, k16] (e4m3 / uint8 bytes, CUDA or pinned host) -> blocked device buffer for the kernel.

    Weight scales are converted once and cached until the source tensor changes; activation scales every call
    (the reference re-lays both on every call, csrc/apis/gemm.hpp:271-290).
    """
    lib = _lib.load()
    if cache:
        hit = _cache_get(_blocked_cache, sf, device)
        if hit is not None:
            return hit
    nbytes = int(lib.ag_fp4_sf_blocked_bytes(groups, rows, k16))
    out = torch.empty(nbytes, dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _lib.check(lib.ag_fp4_sf_to_blocked(sf.data_ptr(), out.data_ptr(), groups, rows, k16,
                                            torch.cuda.current_stream(device).cuda_stream))
    if cache:
        torch.cuda.current_stream(device).synchronize()   # once per weight tensor: safe to reuse from any stream
        _cache_put(_blocked_cache, sf, device, out)
    return out


def _fp4_expand_scales(sf: torch.Tensor, rows: int, k16: int, gran_mn: int, gran_k: int, device: torch.device, what: str) -> torch.Tensor:
    """Scales given at a coarser granularity than one per row and 16 elements are replicated to that granularity, as the
    reference does before its kernel (csrc/apis/gemm.hpp:271-297): [.., rows/gran_mn, k/gran_k] -> [.., rows, k/16]."""
    rep_k = gran_k // 16
    want = (-(-rows // gran_mn), -(-(k16 * 16) // gran_k))
    _require(tuple(sf.shape[-2:]) == want, f"{what} must end in {want} for this recipe, got {tuple(sf.shape[-2:])}")
    out = (sf if sf.is_cuda else sf.to(device)).view(torch.uint8)
    if rep_k > 1:
        out = out.repeat_interleave(rep_k, dim=-1)[..., :k16]
    if gran_mn > 1:
        out = out.repeat_interleave(gran_mn, dim=-2)[..., :rows, :]
    return out.contiguous().view(torch.float8_e4m3fn)


def _fp4_prepare(a, b, d, masked: bool, recipe):
    """Checks of the NVFP4 operators. Returns (g, m, n, k, k16, sfa, sfb) with both scale tensors at one scale per row and
    16 elements: recipe (1, 1, 16) passes them through, a coarser recipe (gran_mn_a, gran_mn_b, gran_k), gran_k a multiple
    of 16, replicates them first."""
    a_q, sfa = a
    b_q, sfb = b
    g, m, n, k = _common_checks(a_q, b_q, d, masked=masked, k_div=2)
    _require(a_q.dtype == torch.uint8 and b_q.dtype == torch.uint8, "a and b must be packed E2M1 in uint8 (two values per byte)")
    for t in (sfa, sfb):
        _require(t.dtype in (torch.float8_e4m3fn, torch.uint8), "NVFP4 scales must be float8_e4m3fn (or their uint8 bytes)")
    _require(k % 32 == 0, "k must be a multiple of 32")
    k16 = k // 16
    gm_a, gm_b, gk = (1, 1, 16) if recipe is None else tuple(int(v) for v in recipe)
    _require(gm_a >= 1 and gm_b >= 1 and gk >= 16 and gk % 16 == 0, f"Unknown SF transformation for recipe {tuple(recipe) if recipe else None}")
    if (gm_a, gm_b, gk) != (1, 1, 16):
        sfa = _fp4_expand_scales(sfa, m, k16, gm_a, gk, a_q.device, "sfa")
        sfb = _fp4_expand_scales(sfb, n, k16, gm_b, gk, a_q.device, "sfb")
    rows_shape = (g, m) if masked else (m,)
    _require(tuple(sfa.shape) == (*rows_shape, k16), f"sfa must be {(*rows_shape, k16)}, got {tuple(sfa.shape)}")
    _require(tuple(sfb.shape) == (g, n, k16), f"sfb must be {(g, n, k16)}, got {tuple(sfb.shape)}")
    _require(sfa.is_cuda and sfa.is_contiguous(), "sfa must be a contiguous CUDA tensor")
    _require(sfb.is_contiguous() and (sfb.is_cuda or sfb.is_pinned()), "sfb must be contiguous and on CUDA or pinned")
    if masked:
        _require(m % 128 == 0, "masked NVFP4 needs M_max to be a multiple of 128")
    return g, m, n, k, k16, sfa, sfb


def m_grouped_fp4_asym_gemm_nt_contiguous(a, b, d, offsets, experts, list_size=None, recipe=None, compiled_dims: str = "nk",
                                          disable_ue8m0_cast: bool = True, *, alpha: float = 1.0) -> None:
    """NVFP4 (packed E2M1 + one E4M3 scale per 16 elements), bf16 out (csrc/apis/gemm.hpp:237-300).

    ``alpha`` (extension): product of the tensor-level fp32 scales, applied to the fp32 accumulator before rounding.
    Every segment must start on a multiple of 128 rows (the contiguous layout's alignment).
    """
    g, m, n, k, k16, sfa, sfb = _fp4_prepare(a, b, d, False, recipe)
    _check_index_tensors(offsets, experts, g)
    if m == 0:
        return
    dev = a[0].device
    sfa_b = _fp4_blocked(sfa, 1, m, k16, dev, cache=False)
    sfb_b = _fp4_blocked(sfb, g, n, k16, dev, cache=sfb is b[1])
    segs = _list_size_to_segments(list_size, offsets, experts)
    _launch(_lib.KIND_NVFP4, "ag_m_grouped_fp4_gemm_nt", layout=_lib.LAYOUT_CONTIGUOUS, a=a[0], sfa=sfa_b, b=b[0], sfb=sfb_b, d=d,
            offsets=offsets, experts=experts, max_segments=segs, m=m, n=n, k=k, g=g, alpha=alpha)


def m_grouped_fp4_asym_gemm_nt_masked(a, b, d, masked_m, expected_m: int, recipe=None, compiled_dims: str = "nk",
                                      disable_ue8m0_cast: bool = True, *, alpha: float = 1.0) -> None:
    """Masked NVFP4 (csrc/apis/gemm.hpp:302-365)."""
    g, m, n, k, k16, sfa, sfb = _fp4_prepare(a, b, d, True, recipe)
    _require(masked_m.is_cuda and masked_m.dtype == torch.int32 and masked_m.is_contiguous() and masked_m.numel() == g,
             "masked_m must be a contiguous int32 CUDA tensor with one entry per group")
    if m == 0 or expected_m == 0:
        return
    dev = a[0].device
    sfa_b = _fp4_blocked(sfa, 1, g * m, k16, dev, cache=False)
    sfb_b = _fp4_blocked(sfb, g, n, k16, dev, cache=sfb is b[1])
    _launch(_lib.KIND_NVFP4, "ag_m_grouped_fp4_gemm_nt", layout=_lib.LAYOUT_MASKED, a=a[0], sfa=sfa_b, b=b[0], sfb=sfb_b, d=d,
            masked_m=masked_m, m=m, n=n, k=k, g=g, rows_hint=int(expected_m) * g, alpha=alpha)
