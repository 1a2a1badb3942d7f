"""HBM cache of hot experts for the asymmetric grouped GEMM.

The reference's unified runtime keeps the most popular experts' weights resident in HBM and streams the rest
(`asym_gemm/unified_moe/runtime.py:1563-1571`, refresh of the cache `:885-893`). Here the same idea sits directly on the
operators: one grouped GEMM call is split into a device-resident part (cached experts) and a host-streamed part (all
others) without touching the host -- both launches see the caller's full segment table, with the segments that belong to
the other part turned into empty row ranges, which the kernel skips before fetching anything. Every weight byte of a
cached expert stays off the host link; the streamed launch moves `(active - cached) / active` of the bytes.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import api


class HotExpertCache:
    """Device copies of up to `capacity` experts of one weight tensor (and of their block scales, when it has any)."""

    def __init__(self, b_host: torch.Tensor, sfb: Optional[torch.Tensor], capacity: int, device="cuda"):
        if b_host.dim() != 3 or not (b_host.is_pinned() or b_host.is_cuda):
            raise RuntimeError("b_host must be a [G, N, K] tensor in pinned host (or device) memory")
        self.b_host = b_host
        self.sfb_full = sfb.to(device) if sfb is not None else None
        self.num_experts = int(b_host.shape[0])
        self.capacity = max(0, min(int(capacity), self.num_experts))
        self.device = torch.device(device)
        self.b_dev = torch.empty((max(self.capacity, 1),) + tuple(b_host.shape[1:]), dtype=b_host.dtype, device=self.device)
        self.sfb_dev = (torch.zeros((max(self.capacity, 1),) + tuple(sfb.shape[1:]), dtype=sfb.dtype, device=self.device)
                        if sfb is not None else None)
        # slot_of[e] = cache slot of expert e, or -1
        self.slot_of = torch.full((self.num_experts,), -1, dtype=torch.int32, device=self.device)
        self.cached: list = []

    def refresh(self, popularity: Sequence[float]) -> int:
        """Make the `capacity` most popular experts resident (copy engine, one cudaMemcpyAsync per newly cached expert, from
        the pinned slab as the reference does). Returns the number of experts copied."""
        if self.capacity == 0:
            return 0
        pop = torch.as_tensor(popularity, dtype=torch.float64)
        want = torch.topk(pop, self.capacity).indices.tolist()
        keep = [e for e in self.cached if e in set(want)]
        new = [e for e in want if e not in set(keep)]
        free = [s for s in range(self.capacity) if s not in {int(self.slot_of[e]) for e in keep}]
        slot_host = self.slot_of.cpu()
        for e in self.cached:
            if e not in keep:
                slot_host[e] = -1
        for e, s in zip(new, free):
            self.b_dev[s].copy_(self.b_host[e], non_blocking=True)
            if self.sfb_dev is not None:
                self.sfb_dev[s].copy_(self.sfb_full[e], non_blocking=True)
            slot_host[e] = s
        self.slot_of.copy_(slot_host)
        self.cached = keep + new
        return len(new)

    def split_tables(self, offsets: torch.Tensor, experts: torch.Tensor) -> Tuple[Tuple[torch.Tensor, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]:
        """(offsets, experts) for the cached launch (expert ids -> cache slots) and for the streamed launch, from the caller's
        contiguous-layout tables. Pure device arithmetic; segments of the other part become empty ranges."""
        n = experts.numel()
        valid = experts >= 0
        slot = self.slot_of[experts.clamp(min=0).long()]
        hit = valid & (slot >= 0)
        pairs = offsets[: 2 * n].view(n, 2) if offsets.numel() >= 2 * n else torch.cat(
            [offsets, offsets.new_zeros(2 * n - offsets.numel())]).view(n, 2)
        empty = torch.zeros_like(pairs)
        off_cached = torch.where(hit.unsqueeze(1), pairs, empty).reshape(-1).contiguous()
        off_stream = torch.where((valid & ~hit).unsqueeze(1), pairs, empty).reshape(-1).contiguous()
        exp_cached = torch.where(hit, slot, torch.where(valid, torch.zeros_like(experts), experts)).to(torch.int32)
        exp_stream = torch.where(valid & ~hit, experts, torch.where(valid, torch.zeros_like(experts), experts)).to(torch.int32)
        return (off_cached, exp_cached), (off_stream, exp_stream)

    def fp8_gemm(self, a, d, offsets, experts, **kw) -> None:
        """`m_grouped_fp8_asym_gemm_nt_contiguous` with cached experts served from HBM and the rest streamed from the host."""
        (oc, ec), (os_, es) = self.split_tables(offsets, experts)
        if self.capacity > 0:
            api.m_grouped_fp8_asym_gemm_nt_contiguous(a, (self.b_dev, self.sfb_dev), d, oc, ec, None, **kw)
        api.m_grouped_fp8_asym_gemm_nt_contiguous(a, (self.b_host, self.sfb_full), d, os_, es, None, **kw)

    def bf16_gemm(self, a, d, offsets, experts) -> None:
        """`m_grouped_bf16_asym_gemm_nt_contiguous` with cached experts served from HBM and the rest streamed from the host."""
        (oc, ec), (os_, es) = self.split_tables(offsets, experts)
        if self.capacity > 0:
            api.m_grouped_bf16_asym_gemm_nt_contiguous(a, self.b_dev, d, oc, ec, None)
        api.m_grouped_bf16_asym_gemm_nt_contiguous(a, self.b_host, d, os_, es, None)

