"""Python wrappers of the MoE helper kernels (csrc/moe_glue.cu) declared in include/asymgemm_b200.h.

CUDA tensors go through the C ABI (and fail loudly if the library is missing). The row-movement helpers also accept
CPU tensors, where they are plain torch indexing: that branch exists only so that the expert-parallel routing logic can
be exercised by gloo ranks without a GPU; the quantisers and the GEMMs have no CPU branch.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def quant_rows_fp8(x: torch.Tensor, pow2_scales: bool = False, rows_used: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, cols] -> (e4m3 [rows, cols], fp32 scales [rows, ceil(cols/128)]), one kernel.
    `pow2_scales` rounds the scales up to powers of two (the quantisers' use_ue8m0=True). `rows_used`: device int32 tensor;
    rows from that count on are neither read nor written."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()):
        raise RuntimeError("quant_rows_fp8 wants a contiguous 2-D bf16 CUDA tensor")
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    sf = torch.empty((rows, (cols + 127) // 128), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().ag_quant_rows_fp8_upto(x.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, cols, int(pow2_scales),
                                                      rows_used.data_ptr() if rows_used is not None else None, _stream(x)))
    return q, sf


def silu_mul_quant_fp8(gate_up: torch.Tensor, inter: int, pow2_scales: bool = False,
                       rows_used: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, 2*inter] -> bf16(silu(gate) * up) quantised to (e4m3 [rows, inter], fp32 [rows, ceil(inter/128)]).
    `rows_used`: device int32 tensor; rows from that count on are neither read nor written."""
    if not (gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and gate_up.dim() == 2 and gate_up.is_contiguous()
            and gate_up.shape[1] == 2 * inter):
        raise RuntimeError("silu_mul_quant_fp8 wants a contiguous bf16 CUDA tensor [rows, 2*inter]")
    rows = gate_up.shape[0]
    q = torch.empty((rows, inter), dtype=torch.float8_e4m3fn, device=gate_up.device)
    sf = torch.empty((rows, (inter + 127) // 128), dtype=torch.float32, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        _lib.check(_lib.load().ag_silu_mul_quant_fp8_upto(gate_up.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, inter, int(pow2_scales),
                                                          rows_used.data_ptr() if rows_used is not None else None, _stream(gate_up)))
    return q, sf


def quant_rows_int8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, cols] -> (int8 [rows, cols], fp32 [rows, ceil(cols/128)] holding the row's scale in every K-block slot)."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()):
        raise RuntimeError("quant_rows_int8 wants a contiguous 2-D bf16 CUDA tensor")
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
    sf = torch.empty((rows, (cols + 127) // 128), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().ag_quant_rows_int8(x.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, cols, _stream(x)))
    return q, sf


def silu_mul_quant_int8(gate_up: torch.Tensor, inter: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 [rows, 2*inter] -> bf16(silu(gate) * up) quantised per row to (int8 [rows, inter], fp32 [rows, ceil(inter/128)])."""
    if not (gate_up.is_cuda and gate_up.dtype == torch.float32 and gate_up.dim() == 2 and gate_up.is_contiguous()
            and gate_up.shape[1] == 2 * inter):
        raise RuntimeError("silu_mul_quant_int8 wants a contiguous fp32 CUDA tensor [rows, 2*inter]")
    rows = gate_up.shape[0]
    q = torch.empty((rows, inter), dtype=torch.int8, device=gate_up.device)
    sf = torch.empty((rows, (inter + 127) // 128), dtype=torch.float32, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        _lib.check(_lib.load().ag_silu_mul_quant_int8(gate_up.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, inter, _stream(gate_up)))
    return q, sf


def _row_bytes(t: torch.Tensor) -> int:
    n = t.element_size()
    for s in t.shape[1:]:
        n *= int(s)
    return n


def move_rows(src: torch.Tensor, out_rows: int, src_rows: Optional[torch.Tensor] = None, dst_rows: Optional[torch.Tensor] = None,
              count: Optional[int] = None, zero: bool = False) -> torch.Tensor:
    """out[dst_rows[i] or i] = src[src_rows[i] or i] for i < count. `out` has `out_rows` rows of src's row shape and dtype."""
    count = int(count if count is not None else (src_rows.numel() if src_rows is not None else
                                                 (dst_rows.numel() if dst_rows is not None else src.shape[0])))
    out = (torch.zeros if zero else torch.empty)((out_rows,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
    if count == 0:
        return out
    rb = _row_bytes(src)
    if src.is_cuda and rb % 16 == 0 and src.is_contiguous():
        with torch.cuda.device(src.device):
            _lib.check(_lib.load().ag_move_rows(src.data_ptr(), out.data_ptr(),
                                                src_rows.data_ptr() if src_rows is not None else None,
                                                dst_rows.data_ptr() if dst_rows is not None else None, count, rb, _stream(src)))
        return out
    s = src.view(torch.uint8) if src.dtype == torch.float8_e4m3fn else src
    o = out.view(torch.uint8) if out.dtype == torch.float8_e4m3fn else out
    picked = s.index_select(0, src_rows) if src_rows is not None else s[:count]
    if dst_rows is not None:
        o.index_copy_(0, dst_rows, picked)
    else:
        o[:count] = picked
    return out


def move_rows_into(out: torch.Tensor, src: torch.Tensor, dst_rows: torch.Tensor) -> None:
    """out[dst_rows[i]] = src[i] for every row of src, in place (rows of out that are not named keep their contents)."""
    count = int(dst_rows.numel())
    if count == 0:
        return
    rb = _row_bytes(src)
    if src.is_cuda and rb % 16 == 0 and src.is_contiguous() and out.is_contiguous():
        with torch.cuda.device(src.device):
            _lib.check(_lib.load().ag_move_rows(src.data_ptr(), out.data_ptr(), None, dst_rows.data_ptr(), count, rb, _stream(src)))
        return
    out.index_copy_(0, dst_rows, src)


def combine_topk(rows: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor, tokens: int, top_k: int) -> torch.Tensor:
    """y[t] = sum_j weights[t, j] * rows[pos[t*top_k + j]] (fp32 accumulation), as rows.dtype; pos None = t*top_k + j."""
    cols = rows.shape[1]
    if rows.is_cuda and rows.dtype == torch.bfloat16 and cols % 8 == 0 and rows.is_contiguous():
        y = torch.empty((tokens, cols), dtype=torch.bfloat16, device=rows.device)
        w = weights.to(torch.float32).contiguous()
        with torch.cuda.device(rows.device):
            _lib.check(_lib.load().ag_combine_topk(rows.data_ptr(), pos.data_ptr() if pos is not None else None, w.data_ptr(), y.data_ptr(),
                                                   tokens, top_k, cols, _stream(rows)))
        return y
    if rows.is_cuda and rows.dtype == torch.float32 and cols % 4 == 0 and rows.is_contiguous():
        y = torch.empty((tokens, cols), dtype=torch.bfloat16, device=rows.device)
        w = weights.to(torch.float32).contiguous()
        with torch.cuda.device(rows.device):
            _lib.check(_lib.load().ag_combine_topk_f32(rows.data_ptr(), pos.data_ptr(), w.data_ptr(), y.data_ptr(), tokens, top_k, cols,
                                                       _stream(rows)))
        return y
    picked = (rows.index_select(0, pos) if pos is not None else rows[: tokens * top_k]).view(tokens, top_k, cols).float()
    return (picked * weights.unsqueeze(-1).float()).sum(dim=1).to(rows.dtype)
