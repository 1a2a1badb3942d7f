"""Token exchange of the expert-parallel MoE layer over peer memory (NVLink / NVSwitch) instead of NCCL all-to-all.

`PeerExchange` owns, on every rank, four buffers that the other ranks of the node map through CUDA IPC: the quantised
rows and their scales in this rank's padded contiguous layout, a return address per row, and the combine buffer for this
rank's own (token, slot) pairs. One step of the layer is then a handful of kernels of this library (csrc/ep_peer.cu):

    histogram -> [all-gather of the per-expert counts] -> plan -> dispatch (stores into the owners' buffers)
    -> [collective] -> grouped GEMMs on the rows where they landed -> return (stores into the sources' combine buffers)
    -> [collective] -> weighted top-k sum

Rows cross NVLink exactly once each way, written by ordinary stores; nothing is sorted, nothing is gathered into send
buffers, and no split size is read back by the host: the layout only exists on the device (`rows_used`, `offsets`,
`experts`). The bracketed collectives are tiny NCCL calls on the same stream; they order the ranks (a rank's kernel that
reads a buffer runs after the collective that follows every rank's stores into it). With one rank they are skipped.

The reference's callers do the same steps with torch sort / bincount / index kernels on the host's schedule
(asym_gemm/unified_moe/runtime.py:1422-1476) and exchange whole batches with all_gather / reduce_scatter
(asym_gemm/training/ep_vanilla.py:173-282).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib


class _DeviceMemory:
    """A raw device allocation presented to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _align(n: int, a: int = 1024) -> int:
    return (n + a - 1) // a * a


class PeerExchange:
    """Exchange buffers of one layer on one rank, mapped into every rank of `group`."""

    def __init__(self, num_experts: int, row_bytes: int, sf_per_row: int, ret_row_bytes: int, top_k: int, max_tokens: int,
                 expert_ranges: List[Tuple[int, int]], device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 cap_rows: Optional[int] = None):
        """`row_bytes` / `sf_per_row`: bytes of one quantised token row and fp32 scales per row; `ret_row_bytes`: bytes of
        one result row; `max_tokens`: the most tokens one rank brings to a step. `cap_rows`: rows each rank's layout can
        hold; default: every pair of every rank plus padding, which cannot overflow."""
        lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > _lib.EP_MAX_RANKS:
            raise RuntimeError(f"at most {_lib.EP_MAX_RANKS} ranks")
        if row_bytes % 16 or ret_row_bytes % 16:
            raise RuntimeError("rows must be multiples of 16 bytes")
        self.device = device
        self.num_experts, self.top_k, self.max_tokens = num_experts, top_k, max_tokens
        self.row_bytes, self.sf_per_row, self.ret_row_bytes = row_bytes, sf_per_row, ret_row_bytes
        self.expert_ranges = [(int(lo), int(hi)) for lo, hi in expert_ranges]
        self.epr = self.expert_ranges[self.rank][1] - self.expert_ranges[self.rank][0]
        max_epr = max(hi - lo for lo, hi in self.expert_ranges)
        pairs = max_tokens * top_k
        self.cap_rows = int(cap_rows) if cap_rows else _align(self.world * pairs, 128) + 128 * max_epr
        self.pairs_cap = pairs
        sizes = [self.cap_rows * row_bytes, self.cap_rows * sf_per_row * 4, self.cap_rows * 8, max(16, pairs * ret_row_bytes)]
        self._offsets = [0]
        for s in sizes:
            self._offsets.append(self._offsets[-1] + _align(s))
        total = self._offsets[-1]
        with torch.cuda.device(device):
            ptr = ctypes.c_void_p()
            handle = (ctypes.c_ubyte * 64)()
            _lib.check(lib.ag_peer_alloc(total, ctypes.byref(ptr), handle))
            self._own = ptr.value
            self._opened: List[int] = []
            bases = [self._own] * self.world
            if self.world > 1:
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=group)
                failure = ""
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    peer = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
                    if lib.ag_peer_open(buf, ctypes.byref(peer)) != 0:
                        failure = f"rank {self.rank} could not map rank {r}'s buffers: {_lib.last_error()}"
                        break
                    self._opened.append(peer.value)
                    bases[r] = peer.value
                # every rank learns whether every rank could map every buffer, so that all of them fail together
                ok = torch.tensor([0 if failure else 1], dtype=torch.int32, device=device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) == 0:
                    for p in self._opened:
                        lib.ag_peer_close(p)
                    lib.ag_peer_free(self._own)
                    self._own = None
                    raise RuntimeError(failure or "another rank could not map the exchange buffers (CUDA IPC between the GPUs of one node is needed)")
        self.peers = _lib.EpPeers()
        for r in range(self.world):
            self.peers.a[r] = bases[r] + self._offsets[0]
            self.peers.sfa[r] = bases[r] + self._offsets[1]
            self.peers.meta[r] = bases[r] + self._offsets[2]
            self.peers.ret[r] = bases[r] + self._offsets[3]
        # addresses of every rank's combine buffer, on the device: the down GEMM stores its result rows straight into them
        self.ret_bases = torch.tensor([int(self.peers.ret[r]) for r in range(self.world)], dtype=torch.int64, device=device)
        arena = torch.as_tensor(_DeviceMemory(self._own, total), device=device)
        self._arena = arena
        self.a = arena[self._offsets[0]: self._offsets[0] + sizes[0]]          # uint8 [cap_rows * row_bytes]
        self.sfa = arena[self._offsets[1]: self._offsets[1] + sizes[1]].view(torch.float32).view(self.cap_rows, sf_per_row)
        self.meta = arena[self._offsets[2]: self._offsets[2] + sizes[2]].view(torch.int64)
        self.ret = arena[self._offsets[3]: self._offsets[3] + pairs * ret_row_bytes]
        self.meta.fill_(-1)
        # device-side tables of this rank
        lo = [r[0] for r in self.expert_ranges] + [self.expert_ranges[-1][1]]
        self.range_lo = torch.tensor(lo, dtype=torch.int32, device=device)
        self.counts_local = torch.zeros(num_experts, dtype=torch.int32, device=device)
        self.counts_all = torch.zeros((self.world, num_experts), dtype=torch.int32, device=device)
        self.send_base = torch.zeros(num_experts, dtype=torch.int32, device=device)
        self.cursors = torch.zeros(num_experts, dtype=torch.int32, device=device)
        self.offsets = torch.zeros(2 * self.epr, dtype=torch.int32, device=device)
        self.experts = torch.full((self.epr + 1,), -1, dtype=torch.int32, device=device)
        self.rows_used = torch.zeros(2, dtype=torch.int32, device=device)
        self._token = torch.zeros(1, dtype=torch.int32, device=device)
        # one rank: row of every pair in the layout, so that the results are combined where they lie (no return copy)
        self.pair_row = torch.zeros(pairs, dtype=torch.int64, device=device) if self.world == 1 else None
        torch.cuda.synchronize(device)
        if self.world > 1:
            dist.barrier(group=group)      # every rank has mapped every buffer before anyone stores into one

    # ------------------------------------------------------------------ steps (all asynchronous on the current stream)
    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def rendezvous(self) -> None:
        """Stream-ordered meeting point of the ranks: what every rank stored before it is in place after it."""
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    def route(self, topk_ids: torch.Tensor, status: torch.Tensor) -> None:
        """Histogram of this rank's routing, all-gather of every rank's histogram, and the plan: where this rank's rows go
        on every owner, and this rank's own segment table (`offsets`, `experts`, `rows_used`)."""
        lib = _lib.load()
        ids = topk_ids.contiguous()
        if ids.dtype != torch.int64 or not ids.is_cuda:
            raise RuntimeError("topk_ids must be an int64 CUDA tensor")
        if ids.shape[0] > self.max_tokens or ids.shape[1] != self.top_k:
            raise RuntimeError(f"this exchange was built for at most {self.max_tokens} tokens x top-{self.top_k}")
        with torch.cuda.device(self.device):
            _lib.check(lib.ag_ep_histogram(ids.data_ptr(), ids.numel(), self.num_experts, self.counts_local.data_ptr(), status.data_ptr(),
                                           self._stream()))
            if self.world > 1:
                dist.all_gather_into_tensor(self.counts_all.view(-1), self.counts_local, group=self.group)
                counts = self.counts_all
            else:
                counts = self.counts_local
            _lib.check(lib.ag_ep_plan(counts.data_ptr(), self.range_lo.data_ptr(), self.world, self.rank, self.num_experts, self.cap_rows,
                                      self.send_base.data_ptr(), self.cursors.data_ptr(), self.offsets.data_ptr(), self.experts.data_ptr(),
                                      self.epr, self.rows_used.data_ptr(), self.meta.data_ptr(), status.data_ptr(), self._stream()))
        self._ids = ids

    def dispatch(self, x_q: torch.Tensor, sfx: torch.Tensor) -> None:
        """Store every (token, slot) pair's row, scales and return address into its expert's next free row on the owner."""
        lib = _lib.load()
        tokens = self._ids.shape[0]
        if not (x_q.is_contiguous() and sfx.is_contiguous() and x_q.shape[0] == tokens and sfx.dtype == torch.float32):
            raise RuntimeError("x_q / sfx must be contiguous, one row per token, scales in fp32")
        with torch.cuda.device(self.device):
            _lib.check(lib.ag_ep_dispatch(x_q.data_ptr(), sfx.data_ptr(), self._ids.data_ptr(), tokens, self.top_k, self.row_bytes,
                                          self.sf_per_row, self.range_lo.data_ptr(), self.world, self.rank, self.send_base.data_ptr(),
                                          self.cursors.data_ptr(), self.cap_rows,
                                          self.pair_row.data_ptr() if self.pair_row is not None else None,
                                          ctypes.byref(self.peers), self._stream()))
        self.rendezvous()

    def send_back(self, out: torch.Tensor) -> None:
        """Store every valid row of `out` [cap_rows, *] (this rank's layout) into its pair's slot on the source rank."""
        lib = _lib.load()
        if not (out.is_contiguous() and out.shape[0] == self.cap_rows and out[0].numel() * out.element_size() == self.ret_row_bytes):
            raise RuntimeError("out must be contiguous [cap_rows, ret_row_bytes worth of elements]")
        with torch.cuda.device(self.device):
            _lib.check(lib.ag_ep_return(out.data_ptr(), self.meta.data_ptr(), self.rows_used.data_ptr(), self.cap_rows, self.ret_row_bytes,
                                        self.world, ctypes.byref(self.peers), self._stream()))
        self.rendezvous()

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (after every rank has finished using them)."""
        lib = _lib.load()
        if getattr(self, "_own", None) is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._opened:
                lib.ag_peer_close(p)
            self._opened = []
            self._arena = self.a = self.sfa = self.meta = self.ret = None
            lib.ag_peer_free(self._own)
        self._own = None
