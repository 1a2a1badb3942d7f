"""Expert-parallel FP8 MoE layer: experts sharded evenly over the ranks of one node, each rank's expert weights in
pinned host memory on its own host link, tokens exchanged with all-to-all over NCCL.

This is the multi-GPU form of the asymmetric grouped GEMM. The reference's own multi-GPU modes are 2-GPU training
paths (asym_gemm/training/ep_vanilla.py:140-282 gathers every rank's tokens and reduce-scatters partial outputs);
here tokens go only to the rank that owns their expert and weights never leave their rank:

    route -> counts all-to-all -> token all-to-all(v) (fp8 rows + 1x128 scales) -> local contiguous layout
          -> gate+up grouped GEMM -> SiLU(gate)*up -> 1x128 requantisation -> down grouped GEMM
          -> all-to-all(v) back (bf16 rows) -> router-weighted sum over top-k

`EPDispatcher` holds the routing arithmetic and the two exchanges; it is device-agnostic (CPU tensors + gloo in the
tests, CUDA tensors + NCCL in production). `ExpertParallelMoE` adds the weights and the two grouped GEMMs.
The activation between the GEMMs follows the reference's CPU MoE bucket: silu(gate) * up rounded to bf16
(csrc/cpu/module.cpp:337-347), gate = first `inter` output columns, up = the second `inter`.
"""
from __future__ import annotations

import contextlib
import ctypes
import mmap
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import moe_ops

ALIGN = 128


@dataclass
class DispatchState:
    """Everything `combine` needs to send results back and undo the permutations of `dispatch`."""
    order: torch.Tensor          # [T*k] positions of the (token, slot) pairs sorted by expert
    send_splits: List[int]       # rows sent to each rank
    recv_splits: List[int]       # rows received from each rank
    dest_rows: torch.Tensor      # [R] row of every received row in the padded contiguous layout
    rows_per_expert: torch.Tensor  # [experts_per_rank] valid rows of every local expert (device tensor)
    padded_rows: int             # rows allocated for the contiguous layout (upper bound; every expert padded to 128)
    offsets: torch.Tensor        # int32 [2*experts_per_rank] (start, end) pairs; empty experts have start == end
    experts: torch.Tensor        # int32 [experts_per_rank + 1] = 0 .. experts_per_rank-1, -1
    tokens: int
    top_k: int
    src_token: Optional[torch.Tensor] = None   # one rank only: rows were not gathered yet; received row i is token src_token[i]


class EPDispatcher:
    """Token routing for expert parallelism over one process group (expert e lives on rank e // experts_per_rank)."""

    def __init__(self, num_experts: int, group: Optional[dist.ProcessGroup] = None,
                 expert_ranges: Optional[List[Tuple[int, int]]] = None):
        """`expert_ranges[r] = (lo, hi)`: the contiguous experts rank r owns (default: equal shares, expert e on rank
        e // (num_experts / world)); unequal shares let faster host links carry more experts (proportional_expert_ranges)."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if expert_ranges is None:
            if num_experts % self.world != 0:
                raise RuntimeError(f"num_experts ({num_experts}) must be divisible by the number of ranks ({self.world})")
            per = num_experts // self.world
            expert_ranges = [(r * per, (r + 1) * per) for r in range(self.world)]
        if len(expert_ranges) != self.world or expert_ranges[0][0] != 0 or expert_ranges[-1][1] != num_experts or \
                any(expert_ranges[i][1] != expert_ranges[i + 1][0] for i in range(self.world - 1)) or \
                any(hi <= lo for lo, hi in expert_ranges):
            raise RuntimeError(f"expert_ranges must tile [0, {num_experts}) with one non-empty range per rank: {expert_ranges}")
        self.num_experts = num_experts
        self.expert_ranges = [(int(lo), int(hi)) for lo, hi in expert_ranges]
        self.experts_per_rank = self.expert_ranges[self.rank][1] - self.expert_ranges[self.rank][0]   # this rank's experts
        self.max_experts_per_rank = max(hi - lo for lo, hi in self.expert_ranges)
        # slot (r, j) of the [world, max_experts_per_rank] count matrix holds expert lo[r] + j (or nothing when j >= n_r)
        idx = torch.full((self.world, self.max_experts_per_rank), num_experts, dtype=torch.int64)
        for r, (lo, hi) in enumerate(self.expert_ranges):
            idx[r, : hi - lo] = torch.arange(lo, hi)
        self._slot_expert = idx
        self._slot_cache: dict = {}

    # ------------------------------------------------------------------ collectives (identity at world size 1)
    def _all_to_all(self, out: torch.Tensor, inp: torch.Tensor, out_splits=None, in_splits=None) -> None:
        if self.world == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)

    def plan(self, topk_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Sort the (token, slot) pairs by expert and exchange per-expert counts.

        Returns (order [T*k], send_counts int32 [world, max_experts_per_rank], recv_counts int32 [world, experts_per_rank]),
        recv_counts[s, j] = rows rank s sends to this rank's local expert j.
        """
        flat = topk_ids.reshape(-1)
        order = torch.argsort(flat, stable=True)
        per_expert = torch.bincount(flat, minlength=self.num_experts)
        slot = self._slot_cache.get(flat.device)
        if slot is None:
            slot = self._slot_expert.to(flat.device)
            self._slot_cache[flat.device] = slot
        padded = torch.cat([per_expert, per_expert.new_zeros(1)])          # index num_experts = "no expert in this slot"
        send_counts = padded[slot].to(torch.int32).contiguous()
        recv_counts = torch.empty_like(send_counts)
        self._all_to_all(recv_counts, send_counts)
        return order, send_counts, recv_counts[:, : self.experts_per_rank].contiguous()

    def layout(self, recv_counts: torch.Tensor, total_recv: int):
        """Contiguous layout of the received rows: grouped by local expert, each expert padded to 128 rows.

        Pure tensor arithmetic on the device of `recv_counts` [world, experts_per_rank] -- no host synchronisation.
        Received rows arrive ordered by (source rank, expert). Returns (dest_rows [total_recv], rows_per_expert [epr],
        padded_bound, offsets int32 [2*epr], experts int32 [epr+1]): dest_rows[i] = row of received row i in the padded
        layout; every local expert gets a segment (an empty one if it received nothing, which the GEMM skips);
        padded_bound = total_recv rounded up plus 127 rows per expert, an upper bound of the rows the layout can use.
        """
        dev = recv_counts.device
        epr = int(recv_counts.shape[1])       # all local experts, or one group of them (pipelined)
        rc = recv_counts.to(torch.int64)
        per_expert = rc.sum(dim=0)                                   # [epr]
        padded = (per_expert + ALIGN - 1) // ALIGN * ALIGN
        expert_start = torch.cumsum(padded, 0) - padded              # [epr]
        within = torch.cumsum(rc, 0) - rc                            # rows of expert j that come from lower ranks
        block_dest = (expert_start.unsqueeze(0) + within).reshape(-1)    # [world*epr], source-major like the recv order
        block_len = rc.reshape(-1)
        block_recv = torch.cumsum(block_len, 0) - block_len
        shift = torch.repeat_interleave(block_dest - block_recv, block_len, output_size=total_recv)
        dest_rows = shift + torch.arange(total_recv, device=dev)
        offsets = torch.stack([expert_start, expert_start + padded], dim=1).reshape(-1).to(torch.int32)
        experts = torch.cat([torch.arange(epr, device=dev, dtype=torch.int32), torch.full((1,), -1, device=dev, dtype=torch.int32)])
        padded_bound = (total_recv + ALIGN - 1) // ALIGN * ALIGN + epr * ALIGN if total_recv > 0 else 0
        return dest_rows, per_expert, padded_bound, offsets, experts

    def dispatch(self, rows: torch.Tensor, topk_ids: torch.Tensor, extras: Tuple[torch.Tensor, ...] = ()):
        """Send every (token, slot) pair's row to the rank that owns its expert.

        rows [T, H] (any dtype; FP8 rows travel as bytes), extras: more per-token tensors [T, *] sent alongside (scales).
        Returns (state, recv_rows [R, H], recv_extras). With one rank nothing leaves the device and the host never
        waits; with several ranks the split sizes of the exchange are read back once, on a side stream, so the host
        does not wait for GEMMs still running on the compute stream.
        """
        tokens, top_k = topk_ids.shape
        if self.world == 1:
            order, send_counts, recv_counts = self.plan(topk_ids)
            send_splits = recv_splits = [tokens * top_k]
            total_recv = tokens * top_k
        else:
            side = self._side_stream(topk_ids.device)
            if side is not None:
                side.wait_stream(torch.cuda.current_stream(topk_ids.device))
                with torch.cuda.stream(side):
                    order, send_counts, recv_counts = self.plan(topk_ids)
                    counts_host = torch.stack([send_counts.sum(dim=1), recv_counts.sum(dim=1)]).cpu()   # waits for the side stream only
                torch.cuda.current_stream(topk_ids.device).wait_stream(side)
            else:
                order, send_counts, recv_counts = self.plan(topk_ids)
                counts_host = torch.stack([send_counts.sum(dim=1), recv_counts.sum(dim=1)]).cpu()
            send_splits, recv_splits = counts_host[0].tolist(), counts_host[1].tolist()
            total_recv = int(sum(recv_splits))
        src_token = torch.div(order, top_k, rounding_mode="floor")
        outs = []
        for t in (rows,) + tuple(extras):
            if self.world == 1:
                outs.append(t)         # nothing to exchange: the gather is folded into the scatter to the padded layout
                continue
            send = moe_ops.move_rows(t.contiguous(), src_token.numel(), src_rows=src_token)
            as_bytes = send.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else send
            recv = torch.empty((total_recv,) + tuple(as_bytes.shape[1:]), dtype=as_bytes.dtype, device=as_bytes.device)
            self._all_to_all(recv, as_bytes, recv_splits, send_splits)
            outs.append(recv.view(t.dtype) if t.dtype == torch.float8_e4m3fn else recv)
        dest_rows, per_expert, padded_rows, offsets, experts = self.layout(recv_counts, total_recv)
        state = DispatchState(order, send_splits, recv_splits, dest_rows, per_expert, padded_rows, offsets, experts, tokens, top_k,
                              src_token if self.world == 1 else None)
        return state, outs[0], tuple(outs[1:])

    def pipelined(self, rows: torch.Tensor, extras: Tuple[torch.Tensor, ...], topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                  groups: int, expert_fn) -> torch.Tensor:
        """dispatch -> experts -> combine with every rank's experts cut into `groups` groups, so that on a GPU the
        exchanges of one group run while another group is being multiplied.

        Cutting by experts (not by tokens) leaves every weight byte in exactly one round. The exchanges run on a
        communication stream, `expert_fn` on the caller's stream: dispatch of group g+1 and the return of group g-1
        overlap the GEMMs of group g. All ranks issue the collectives in the same order (every dispatch, then the
        returns). `expert_fn(recv_rows, recv_extras, state, first, count)` multiplies the rows received for the local
        experts [first, first + count) -- `state` describes their padded contiguous layout, expert ids relative to
        `first` -- and returns the result in that layout. On CPU tensors the same steps run one after the other.
        Returns y [T, H] like `combine`.
        """
        tokens, top_k = topk_ids.shape
        dev = topk_ids.device
        cuda = dev.type == "cuda"
        main = torch.cuda.current_stream(dev) if cuda else None
        comm = self._side_stream(dev)

        def on_comm():
            return torch.cuda.stream(comm) if cuda else contextlib.nullcontext()

        if cuda:
            comm.wait_stream(main)
        with on_comm():
            order, send_counts, recv_counts = self.plan(topk_ids)
            send_host, recv_host = send_counts.cpu().to(torch.int64), recv_counts.cpu().to(torch.int64)   # waits for this stream only
            src_token = torch.div(order, top_k, rounding_mode="floor")
        groups = max(1, min(int(groups), min(hi - lo for lo, hi in self.expert_ranges)))
        # the (token, slot) pairs sorted by expert are also sorted by (rank, local expert): start of every such block
        flat = send_host.reshape(-1)
        block_start = (torch.cumsum(flat, 0) - flat).reshape(send_host.shape)

        def cut(n, g):
            return g * n // groups

        rounds = []
        for g in range(groups):
            spans, send_splits = [], []
            for r, (lo, hi) in enumerate(self.expert_ranges):
                a, b = cut(hi - lo, g), cut(hi - lo, g + 1)
                cnt = int(send_host[r, a:b].sum())
                send_splits.append(cnt)
                if cnt:
                    spans.append((int(block_start[r, a]), cnt))
            a, b = cut(self.experts_per_rank, g), cut(self.experts_per_rank, g + 1)
            rounds.append((spans, send_splits, [int(v) for v in recv_host[:, a:b].sum(dim=1)], a, b))

        # ---- every dispatch, on the communication stream
        keep, arrived = [], []
        with on_comm():
            for spans, send_splits, recv_splits, a, b in rounds:
                idx = (torch.cat([torch.arange(s0, s0 + cnt, device=dev) for s0, cnt in spans]) if spans
                       else torch.zeros(0, dtype=torch.int64, device=dev))
                rows_src = src_token.index_select(0, idx)
                total = sum(recv_splits)
                recvd = []
                for t in (rows,) + tuple(extras):
                    send = moe_ops.move_rows(t.contiguous(), idx.numel(), src_rows=rows_src)
                    as_bytes = send.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else send
                    recv = torch.empty((total,) + tuple(as_bytes.shape[1:]), dtype=as_bytes.dtype, device=dev)
                    self._all_to_all(recv, as_bytes, recv_splits, send_splits)
                    recvd.append(recv.view(t.dtype) if t.dtype == torch.float8_e4m3fn else recv)
                    keep.append(send)
                ev = None
                if cuda:
                    ev = torch.cuda.Event()
                    ev.record(comm)
                arrived.append((idx, recvd, ev))

        # ---- group by group: multiply on the caller's stream, send the results home on the communication stream
        ret_sorted = None
        for (spans, send_splits, recv_splits, a, b), (idx, recvd, ev) in zip(rounds, arrived):
            if cuda:
                main.wait_event(ev)
            total = sum(recv_splits)
            dest_rows, per_expert, padded, offsets, experts = self.layout(recv_counts[:, a:b], total)
            state = DispatchState(order, send_splits, recv_splits, dest_rows, per_expert, padded, offsets, experts, tokens, top_k)
            out = expert_fn(recvd[0], tuple(recvd[1:]), state, a, b - a)
            back = moe_ops.move_rows(out, total, src_rows=dest_rows)
            done = None
            if cuda:
                done = torch.cuda.Event()
                done.record(main)
            with on_comm():
                if cuda:
                    comm.wait_event(done)
                ret = torch.empty((idx.numel(),) + tuple(back.shape[1:]), dtype=back.dtype, device=dev)
                self._all_to_all(ret, back, send_splits, recv_splits)
                if ret_sorted is None:
                    ret_sorted = torch.empty((tokens * top_k,) + tuple(back.shape[1:]), dtype=back.dtype, device=dev)
                moe_ops.move_rows_into(ret_sorted, ret, idx)
            keep += [out, back, ret, state]          # alive until both streams are done with them
        if cuda:
            main.wait_stream(comm)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=dev)
        y = moe_ops.combine_topk(ret_sorted, inv, topk_weights, tokens, top_k)
        del keep
        return y

    def _side_stream(self, device):
        if device.type != "cuda":
            return None
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=device)
        return self._side

    def combine(self, expert_out: torch.Tensor, state: DispatchState, topk_weights: torch.Tensor, mark=None) -> torch.Tensor:
        """expert_out [padded_rows, H] (contiguous layout) -> y [T, H] = sum_k w[t, k] * out(t, k), in fp32, as expert_out.dtype.
        `mark(name)`, if given, is called between the return exchange and the weighted sum (phase timing)."""
        # inverse of the sort: pair p (token p // k, slot p % k) was sent as sorted row inv[p]
        inv = torch.empty_like(state.order)
        inv[state.order] = torch.arange(state.order.numel(), device=state.order.device)
        if self.world == 1:
            # the sorted rows never left this rank: read them straight out of the padded layout
            pos = state.dest_rows.index_select(0, inv)
            if mark is not None:
                mark("return")
            return moe_ops.combine_topk(expert_out, pos, topk_weights, state.tokens, state.top_k)
        back = moe_ops.move_rows(expert_out, state.dest_rows.numel(), src_rows=state.dest_rows)
        ret = torch.empty((state.tokens * state.top_k, back.shape[1]), dtype=back.dtype, device=back.device)
        self._all_to_all(ret, back, state.send_splits, state.recv_splits)
        if mark is not None:
            mark("return")
        return moe_ops.combine_topk(ret, inv, topk_weights, state.tokens, state.top_k)


def to_contiguous_layout(recv: torch.Tensor, state: DispatchState) -> torch.Tensor:
    """Scatter received rows into the zero-padded contiguous layout the grouped GEMM consumes."""
    return moe_ops.move_rows(recv.contiguous(), state.padded_rows, src_rows=state.src_token, dst_rows=state.dest_rows, zero=True)


# --------------------------------------------------------------------------------------------- pinned weights
_keepalive: list = []


def pinned_empty(shape, dtype: torch.dtype, numa_node: Optional[int] = None, huge_pages: bool = False) -> torch.Tensor:
    """Pinned host tensor for expert weights, optionally bound to one NUMA node and/or backed by transparent huge pages.

    With `numa_node` or `huge_pages`: anonymous mmap -> [madvise(MADV_HUGEPAGE)] -> [mbind(MPOL_BIND)] ->
    cudaHostRegister, the recipe the reference uses for its NUMA-bound slabs
    (asym_gemm/unified_moe/runtime.py:236-279); any failure falls back to torch's pinned allocator.
    Pages are faulted in on first write, so fill the tensor from a thread running on that node.
    """
    numel = 1
    for s in shape:
        numel *= int(s)
    if (numa_node is not None and numa_node >= 0) or huge_pages:
        try:
            nbytes = max(1, numel * torch.empty((), dtype=dtype).element_size())
            two_mb = 2 << 20
            mm = mmap.mmap(-1, (nbytes + two_mb - 1) // two_mb * two_mb + two_mb)
            base = ctypes.addressof(ctypes.c_char.from_buffer(mm))
            addr = (base + two_mb - 1) // two_mb * two_mb          # 2 MB aligned start inside the mapping
            libc = ctypes.CDLL(None, use_errno=True)
            if huge_pages and libc.madvise(ctypes.c_void_p(addr), ctypes.c_size_t((nbytes + two_mb - 1) // two_mb * two_mb), 14) != 0:
                raise OSError("madvise(MADV_HUGEPAGE) failed")
            mask = ctypes.c_ulong(1 << max(numa_node or 0, 0))
            if numa_node is not None and numa_node >= 0 and \
                    libc.syscall(237, ctypes.c_void_p(addr), ctypes.c_size_t(nbytes), 2, ctypes.byref(mask), 65, 0) != 0:
                raise OSError("mbind failed")
            rc = torch.cuda.cudart().cudaHostRegister(addr, nbytes, 0)
            if int(rc) != 0:
                raise OSError(f"cudaHostRegister returned {rc}")
            _keepalive.append(mm)
            return torch.frombuffer(mm, dtype=dtype, count=numel, offset=addr - base).view(*shape)
        except Exception:
            pass
    return torch.empty(*shape, dtype=dtype).pin_memory()


def proportional_expert_ranges(rates: List[float], num_experts: int, tolerance: float = 0.1) -> List[Tuple[int, int]]:
    """Contiguous expert ranges [lo, hi) per rank, sized in proportion to each rank's measured host-link rate.

    Every rank streams its own experts' weights over its own host link and a step ends with the slowest rank, so when the
    links of one machine are not equally fast (on an 8-GPU host four links were measured at 23 GB/s and four at 35 GB/s
    with all eight busy) equal shards leave the fast links idle. Rates within `tolerance` of each other give the even
    split. Every rank keeps at least one expert.
    """
    world = len(rates)
    if world <= 0 or num_experts < world:
        raise RuntimeError("need at least one expert per rank")
    even = [(r * num_experts // world, (r + 1) * num_experts // world) for r in range(world)]
    if min(rates) <= 0 or max(rates) / min(rates) <= 1.0 + tolerance:
        return even
    total = float(sum(rates))
    counts = [max(1, int(num_experts * r / total)) for r in rates]
    # hand out what rounding left over (or take back any excess) where it changes the finishing time least
    while sum(counts) < num_experts:
        i = min(range(world), key=lambda j: (counts[j] + 1) / rates[j])
        counts[i] += 1
    while sum(counts) > num_experts:
        i = max((j for j in range(world) if counts[j] > 1), key=lambda j: counts[j] / rates[j])
        counts[i] -= 1
    out, lo = [], 0
    for c in counts:
        out.append((lo, lo + c))
        lo += c
    return out


def rebalance_expert_ranges(ranges: List[Tuple[int, int]], step_ms: List[float], tolerance: float = 0.06) -> List[Tuple[int, int]]:
    """Expert ranges re-cut from what the ranks just measured: rank r took `step_ms[r]` for a step over its current range, so
    its link moves (hi - lo) / step_ms[r] experts per millisecond under the load the job really produces (every rank
    streaming, the host's memory system shared); the new ranges are proportional to those rates. A short calibration
    before the job cannot see that load -- on one 8-GPU host it read 47 GB/s for links that then ran at 29 GB/s.
    Returns `ranges` itself when the slowest and the fastest rank are within `tolerance` of each other. The caller moves
    the weights of experts that change owner (once, outside any timed region) and may repeat the step."""
    if len(ranges) != len(step_ms) or not ranges:
        raise RuntimeError("one step time per rank is needed")
    if min(step_ms) <= 0:
        return list(ranges)
    if max(step_ms) / min(step_ms) <= 1.0 + tolerance:
        return list(ranges)
    rates = [(hi - lo) / ms for (lo, hi), ms in zip(ranges, step_ms)]
    return proportional_expert_ranges(rates, ranges[-1][1], tolerance=0.0)


def gate_up_interleave_index(inter: int, device=None) -> torch.Tensor:
    """Row permutation for the fused SiLU*mul epilogue: row r of the interleaved weight is row index[r] of the usual
    [gate; up] tensor [2*inter, hidden] -- gate and up rows alternate in groups of 16, so that any 32 consecutive rows hold
    16 gate columns and the same 16 up columns (`epilogue` of the C descriptor)."""
    r = torch.arange(2 * inter, device=device)
    return (r % 32 // 16) * inter + r // 32 * 16 + r % 16


def interleave_gate_up(w13: torch.Tensor) -> torch.Tensor:
    """[..., 2*inter, hidden] weights in the usual [gate; up] order -> the same rows interleaved for the fused SiLU*mul
    epilogue (a new tensor on w13's device; the block scales stay as they are)."""
    inter = w13.shape[-2] // 2
    if inter % 128:
        raise RuntimeError("inter must be a multiple of 128")
    src = w13.view(torch.uint8) if w13.dtype == torch.float8_e4m3fn else w13
    out = src.index_select(-2, gate_up_interleave_index(inter, w13.device))
    return out.view(w13.dtype) if w13.dtype == torch.float8_e4m3fn else out


def gpu_numa_node(device_index: int) -> int:
    """NUMA node of the GPU's PCIe root, or -1 when the platform does not say (single-node VMs)."""
    try:
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        devid = torch.cuda.get_device_properties(device_index).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{devid:02x}.0/numa_node"
        with open(path) as f:
            return int(f.read().strip())
    except Exception:
        return -1


# --------------------------------------------------------------------------------------------- the layer
class ExpertParallelMoE:
    """FP8 MoE layer (gate+up, SiLU*mul, down) with this rank's experts in pinned host memory.

    w13: (fp8 [E_local, 2*inter, hidden] pinned, fp32 block scales [E_local, 2*inter/128, hidden/128])
    w2:  (fp8 [E_local, hidden, inter] pinned,   fp32 block scales [E_local, hidden/128, inter/128])
    """

    def __init__(self, num_experts: int, hidden: int, inter: int, w13, w2, group: Optional[dist.ProcessGroup] = None,
                 expert_ranges: Optional[List[Tuple[int, int]]] = None, ue8m0_scales: bool = False, pipeline_groups: int = 1,
                 comm_sms: int = 24, exchange: str = "nccl", max_tokens: Optional[int] = None, top_k: Optional[int] = None,
                 fused_activation: bool = False, fused_return: bool = True):
        """`ue8m0_scales`: quantise activations with power-of-two scales and let the tensor core apply all block scales
        (the weights must then have been quantised with use_ue8m0=True); default: arbitrary fp32 scales, applied exactly.
        Whether the kernel reads the pinned weights itself or the copy engine stages them is the operators' setting
        (`asymgemm_b200.set_weight_path`). `pipeline_groups` > 1 (several ranks only): the layer runs in that many
        rounds over groups of each rank's experts so that the token exchanges overlap the GEMMs
        (`EPDispatcher.pipelined`); the persistent GEMMs then leave `comm_sms` SMs free for the exchange kernels --
        they are bound by the host link, not by SMs.
        `exchange`: "nccl" (default) sorts the (token, slot) pairs, gathers rows into send buffers and exchanges them with
        all-to-all(v), reading the split sizes back on the host; "peer" routes, lays out and exchanges with this library's
        own kernels, which store rows straight into the owner rank's buffers over NVLink (`ep_peer.PeerExchange`; needs
        `max_tokens`, the most tokens one rank brings to a step, and `top_k`; the ranks must be processes of one node).
        Both give the same output bit for bit.
        `fused_activation`: the gate+up GEMM writes bf16(silu(gate) * up) itself (`epilogue="silu_mul"` of the FP8 operator),
        so the [rows, 2*inter] intermediate is never written; `w13[0]` must then hold the rows of every expert in the
        interleaved order of `interleave_gate_up` (a weight-preparation step; the scales stay as they are). Exact-scale
        mode only; same output bit for bit.
        `fused_return` (peer exchange, more than one rank): the down GEMM's drain stores every result row straight into its
        pair's slot of the source rank's combine buffer (`scatter` of the FP8 operator) instead of writing a local tensor
        that a second kernel then sends home; same output bit for bit."""
        self.fused_activation = bool(fused_activation)
        self.fused_return = bool(fused_return)
        if self.fused_activation and ue8m0_scales:
            raise RuntimeError("fused_activation exists for the exact fp32-scale mode only")
        if exchange not in ("nccl", "peer"):
            raise RuntimeError("exchange must be 'nccl' or 'peer'")
        self.exchange = exchange
        self.peer = None
        self.pipeline_groups = max(1, int(pipeline_groups))
        self.comm_sms = max(0, int(comm_sms))
        self.dispatcher = EPDispatcher(num_experts, group, expert_ranges)
        self.ue8m0_scales = bool(ue8m0_scales)
        self.hidden, self.inter = hidden, inter
        self.w13, self.w2 = w13, w2
        self._weight_views: dict = {}
        # staged weight path only: weights whose first chunks are copied while this layer's results travel home (the next
        # layer's gate+up weights in a model; this layer's own when it is called in a loop). None = no prefetch.
        self.prefetch_next: Optional[torch.Tensor] = None
        # Measurement and test hooks, off by default. `phase_events`: a list that every unpipelined forward() appends
        # (phase name, CUDA event) pairs to, recorded on the caller's stream where one phase ends. `keep_intermediates`:
        # the last experts_forward() leaves its operands and results in `self.intermediates`.
        self.phase_events: Optional[list] = None
        self.keep_intermediates = False
        self.intermediates: Optional[dict] = None
        epr = self.dispatcher.experts_per_rank
        if tuple(w13[0].shape) != (epr, 2 * inter, hidden) or tuple(w2[0].shape) != (epr, hidden, inter):
            raise RuntimeError("weight shapes do not match (experts_per_rank, 2*inter, hidden) / (experts_per_rank, hidden, inter)")
        if exchange == "peer":
            from .ep_peer import PeerExchange
            if not max_tokens or not top_k:
                raise RuntimeError("exchange='peer' needs max_tokens and top_k")
            dev = w13[1].device if w13[1].is_cuda else torch.device("cuda", torch.cuda.current_device())
            self.peer = PeerExchange(num_experts, hidden, (hidden + 127) // 128, hidden * 2, int(top_k), int(max_tokens),
                                     self.dispatcher.expert_ranges, dev, group)

    def _weights_of(self, first: int, count: int):
        """(w13, w2) of the local experts [first, first + count): views made once, because the operators cache prepared
        weight scales by tensor identity."""
        if count >= self.dispatcher.experts_per_rank:
            return self.w13, self.w2
        hit = self._weight_views.get((first, count))
        if hit is None:
            sl = slice(first, first + count)
            hit = self._weight_views[(first, count)] = ((self.w13[0][sl], self.w13[1][sl]), (self.w2[0][sl], self.w2[1][sl]))
        return hit

    def _mark(self, name: str) -> None:
        if self.phase_events is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_events.append((name, ev))

    def experts_forward(self, a_q: torch.Tensor, sfa: torch.Tensor, state: DispatchState, first: int = 0,
                        count: Optional[int] = None, rows_used: Optional[torch.Tensor] = None, scatter=None) -> torch.Tensor:
        """Both grouped GEMMs over the contiguous layout; returns bf16 [padded_rows, hidden]. `first` / `count`: the local
        experts `state` describes (expert id 0 of its segment table = local expert `first`); default: all of them.
        `rows_used`: device int32 holding how many rows of the layout are in use when only the device knows (the
        activation kernel then leaves the rest of the buffer alone). `scatter` = (meta, bases): the down GEMM stores every
        result row into the buffer and row its entry names (the source ranks' combine buffers) instead of the returned tensor."""
        from . import api
        w13, w2 = self._weights_of(first, self.dispatcher.experts_per_rank if count is None else count)
        m = state.padded_rows
        dev = a_q.device
        d2 = torch.empty((m, self.hidden), dtype=torch.bfloat16, device=dev)
        if m == 0:
            return d2
        hw = self.ue8m0_scales
        if self.fused_activation:
            act = torch.empty((m, self.inter), dtype=torch.bfloat16, device=dev)
            api.m_grouped_fp8_asym_gemm_nt_contiguous((a_q, sfa), w13, act, state.offsets, state.experts, None, epilogue="silu_mul")
            self._mark("gemm_gate_up")
            a2, s2 = moe_ops.quant_rows_fp8(act, rows_used=rows_used)
            self._mark("silu_mul_requant")
            api.m_grouped_fp8_asym_gemm_nt_contiguous((a2, s2), w2, d2, state.offsets, state.experts, None, scatter=scatter)
            self._mark("gemm_down")
            if self.keep_intermediates:
                self.intermediates = dict(a_q=a_q, sfa=sfa, act=act, a2=a2, s2=s2, d2=d2, state=state, first=first)
            return d2
        d1 = torch.empty((m, 2 * self.inter), dtype=torch.bfloat16, device=dev)
        api.m_grouped_fp8_asym_gemm_nt_contiguous((a_q, sfa), w13, d1, state.offsets, state.experts, None, ue8m0_scales=hw)
        self._mark("gemm_gate_up")
        a2, s2 = moe_ops.silu_mul_quant_fp8(d1, self.inter, pow2_scales=hw, rows_used=rows_used)
        self._mark("silu_mul_requant")
        api.m_grouped_fp8_asym_gemm_nt_contiguous((a2, s2), w2, d2, state.offsets, state.experts, None, ue8m0_scales=hw, scatter=scatter)
        self._mark("gemm_down")
        if self.keep_intermediates:
            self.intermediates = dict(a_q=a_q, sfa=sfa, d1=d1, a2=a2, s2=s2, d2=d2, state=state, first=first)
        return d2

    def _forward_peer(self, x_q: torch.Tensor, sfx: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """The layer with the peer-memory exchange: rows land in the owner's padded layout directly, the GEMMs run over the
        whole buffer with the device-built segment table, results go home the same way. No host synchronisation."""
        from . import api
        px = self.peer
        tokens, top_k = topk_ids.shape
        px.route(topk_ids, api._status_word(x_q.device))
        px.dispatch(x_q.view(torch.uint8), sfx)
        self._mark("plan_dispatch")
        a_q = px.a.view(torch.float8_e4m3fn).view(px.cap_rows, self.hidden)
        state = DispatchState(None, [], [], None, None, px.cap_rows, px.offsets, px.experts, tokens, top_k)
        self._mark("layout")
        # more than one rank: the down GEMM's drain stores every result row straight into its pair's slot of the source rank's
        # combine buffer (over NVLink, tile by tile while the GEMM runs); there is no separate return pass
        direct = px.pair_row is None and self.fused_return
        out = self.experts_forward(a_q, px.sfa, state, rows_used=px.rows_used[:1], scatter=(px.meta, px.ret_bases) if direct else None)
        if self.prefetch_next is not None and out.is_cuda:      # staged weight path: start the next call's first copies now
            api.prefetch_weights(self.prefetch_next, out.device)
        if px.pair_row is not None:      # one rank: every result already lies in this rank's memory
            self._mark("return")
            y = moe_ops.combine_topk(out, px.pair_row, topk_weights, tokens, top_k)
            self._mark("combine")
            return y
        if direct:
            px.rendezvous()      # every rank's GEMM, and with it every store into this rank's combine buffer, has finished
        else:
            px.send_back(out)
        self._mark("return")
        y = moe_ops.combine_topk(px.ret.view(torch.bfloat16).view(px.pairs_cap, self.hidden), None, topk_weights, tokens, top_k)
        self._mark("combine")
        return y

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """x bf16 [T, hidden] (this rank's tokens), topk_ids int64 [T, k], topk_weights [T, k] -> bf16 [T, hidden]."""
        self._mark("start")
        x_q, sfx = moe_ops.quant_rows_fp8(x.contiguous(), pow2_scales=self.ue8m0_scales)
        self._mark("quantise")
        if self.peer is not None:
            return self._forward_peer(x_q, sfx, topk_ids, topk_weights)
        if self.pipeline_groups > 1 and self.dispatcher.world > 1:
            from . import api

            def group_forward(recv_q, recv_extras, state, first, count):
                a_q = to_contiguous_layout(recv_q, state)
                sfa = to_contiguous_layout(recv_extras[0], state)
                return self.experts_forward(a_q, sfa, state, first, count)

            sms = torch.cuda.get_device_properties(x.device).multi_processor_count
            cap = api.get_num_sms()
            with api.launch_sm_cap(max(8, (cap if 0 < cap < sms else sms) - self.comm_sms)):
                return self.dispatcher.pipelined(x_q, (sfx,), topk_ids, topk_weights, self.pipeline_groups, group_forward)
        state, recv_q, (recv_s,) = self.dispatcher.dispatch(x_q, topk_ids, (sfx,))
        self._mark("plan_dispatch")
        a_q = to_contiguous_layout(recv_q, state)
        sfa = to_contiguous_layout(recv_s, state)
        self._mark("layout")
        out = self.experts_forward(a_q, sfa, state)
        if self.prefetch_next is not None and out.is_cuda:
            from . import api
            api.prefetch_weights(self.prefetch_next, out.device)
        y = self.dispatcher.combine(out, state, topk_weights, self._mark if self.phase_events is not None else None)
        self._mark("combine")
        return y
