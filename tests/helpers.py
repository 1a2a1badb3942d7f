"""Shared input builders for the parity tests: seeded tensors in the operators' formats + numpy views for the oracle."""
from __future__ import annotations

import numpy as np
import torch

from asymgemm_b200.utils import (build_contiguous_layout, per_block_cast_to_fp8, per_channel_cast_to_int8,
                                 per_token_cast_to_fp8, per_token_cast_to_int8, per_token_cast_to_nvfp4_e4m3)
from oracle import oracle


def np_bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as numpy (bf16 -> uint16 bit patterns, fp8 -> uint8 bit patterns)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn,):
        return t.view(torch.uint8).numpy()
    return t.numpy()


def pin(t: torch.Tensor) -> torch.Tensor:
    return t.detach().cpu().contiguous().pin_memory()


def rows_zipf(num_experts: int, tokens: int, top_k: int, s: float, gen: torch.Generator) -> list[int]:
    """Per-expert row counts: every token picks top_k distinct experts with popularity ~ 1/rank^s."""
    w = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float64) ** s
    picks = torch.multinomial(w.expand(tokens, -1), top_k, replacement=False, generator=gen)
    return torch.bincount(picks.flatten(), minlength=num_experts).tolist()


def make_contiguous_case(kind: str, rows_per_expert, n: int, k: int, seed: int = 0, device="cuda", b_on_host: bool = True,
                         use_ue8m0: bool = False):
    """Returns dict with operator inputs (torch, on `device`; B pinned on host if asked) and oracle inputs (numpy)."""
    gen = torch.Generator().manual_seed(seed)
    g = len(rows_per_expert)
    offsets, experts, list_size, m_total, segs = build_contiguous_layout(rows_per_expert, device=device)
    a_f = torch.zeros((m_total, k), dtype=torch.float32)
    for e, start, rows in segs:
        a_f[start:start + rows] = torch.randn((rows, k), generator=gen)
    b_f = torch.randn((g, n, k), generator=gen) * 0.02 if kind != "bf16_unit" else torch.randn((g, n, k), generator=gen)
    segments = oracle.contiguous_segments(offsets.cpu().tolist(), experts.cpu().tolist(), None, m_total)
    return _finish_case(kind, a_f, b_f, segments, device, b_on_host, use_ue8m0, gen) | dict(
        offsets=offsets, experts=experts, list_size=list_size, m_total=m_total, segs=segs, n=n, k=k, g=g)


def make_masked_case(kind: str, masked_m, m_max: int, n: int, k: int, seed: int = 0, device="cuda", b_on_host: bool = True,
                     use_ue8m0: bool = False):
    gen = torch.Generator().manual_seed(seed)
    g = len(masked_m)
    a_f = torch.randn((g * m_max, k), generator=gen)
    b_f = torch.randn((g, n, k), generator=gen) * 0.02
    segments = oracle.masked_segments(masked_m, m_max)
    c = _finish_case(kind, a_f, b_f, segments, device, b_on_host, use_ue8m0, gen)
    for key in ("a", "sfa"):
        if c.get(key) is not None:
            c[key] = c[key].view(g, m_max, -1)
    c.update(masked_m=torch.tensor(masked_m, dtype=torch.int32, device=device), m_max=m_max, n=n, k=k, g=g)
    return c


def _finish_case(kind, a_f, b_f, segments, device, b_on_host, use_ue8m0, gen):
    g, n, k = b_f.shape
    place_b = pin if b_on_host else (lambda t: t.to(device))
    c = dict(kind=kind, segments=segments)
    if kind.startswith("bf16"):
        a = a_f.to(torch.bfloat16)
        b = b_f.to(torch.bfloat16)
        c.update(a=a.to(device), sfa=None, b=place_b(b), sfb=None)
        c["ref"] = oracle.gemm_bf16(np_bits(a), np_bits(b), segments)
    elif kind == "fp8":
        a_q, sfa = per_token_cast_to_fp8(a_f, use_ue8m0)
        qs = [per_block_cast_to_fp8(b_f[i], use_ue8m0) for i in range(g)]
        b_q = torch.stack([q for q, _ in qs])
        sfb = torch.stack([s for _, s in qs])
        c.update(a=a_q.to(device), sfa=sfa.to(device), b=place_b(b_q), sfb=place_b(sfb))
        c["ref"] = oracle.gemm_fp8(np_bits(a_q), sfa.numpy(), np_bits(b_q), sfb.numpy(), segments)
    elif kind == "int8":
        a_q, sfa = per_token_cast_to_int8(a_f)
        qs = [per_channel_cast_to_int8(b_f[i]) for i in range(g)]
        b_q = torch.stack([q for q, _ in qs])
        sfb = torch.stack([s for _, s in qs])
        c.update(a=a_q.to(device), sfa=sfa.to(device), b=place_b(b_q), sfb=sfb.to(device))
        c["ref"], c["block_sums"] = oracle.gemm_int8(a_q.numpy(), sfa.numpy(), b_q.numpy(), sfb.numpy(), segments, True)
    elif kind == "fp4":
        a_q, sfa = per_token_cast_to_nvfp4_e4m3(a_f)
        qs = [per_token_cast_to_nvfp4_e4m3(b_f[i]) for i in range(g)]
        b_q = torch.stack([q for q, _ in qs])
        sfb = torch.stack([s for _, s in qs])
        c.update(a=a_q.to(device), sfa=sfa.to(device), b=place_b(b_q), sfb=place_b(sfb))
        c["ref"] = oracle.gemm_nvfp4(a_q.numpy(), np_bits(sfa), b_q.numpy(), np_bits(sfb), segments)
    else:
        raise ValueError(kind)
    return c


def valid_row_mask(segments, rows_total: int) -> np.ndarray:
    mask = np.zeros(rows_total, dtype=bool)
    for _, r0, r1 in segments:
        mask[r0:r1] = True
    return mask
