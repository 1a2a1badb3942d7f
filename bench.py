#!/usr/bin/env python
"""Benchmark of the m-grouped asymmetric GEMM: grouped-GEMM TFLOP/s and host->GPU weight GB/s against the measured
host-link peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3_fp8|c2_bf16|c1_int8] [--impl ours|reference]

One step = one grouped GEMM over one batch of synthetic, seeded input (the shapes of the benchmark configurations named in WORKLOADS; no
dataset or checkpoint is involved). The default workload is the DeepSeek-V3-shaped FP8 gate+up GEMM: 256 experts,
K=7168, N=4096, 16384 tokens x top-8 with Zipf(0.8) expert popularity, B (7.5 GB) in pinned host memory.
With N > 1 ranks the experts (and the rows routed to them) are split across ranks in contiguous ranges: first in proportion
to each rank's host-link rate measured with all ranks streaming at once for a sustained interval, then re-cut from the
ranks' own step times after the warm-up steps (closed loop; --even-shards forces the even split). Every rank streams its
own shard over its own host link and there is no collective on the data path of the headline number, so total work is
fixed ("strong"). When the job has fewer ranks than the machine has GPUs, the GPUs are chosen by measurement
(asymgemm_b200/linkprobe.py; --device-map identity keeps rank r on GPU r).

Prints ONE JSON line on rank 0. `value` times the kernel with activations already in HBM; `e2e` times the public
operator call with host buffers (pinned A in, D out) inside the timed region. The same line carries `ep_layer` -- the
expert-parallel FP8 MoE layer (two grouped GEMMs, NCCL all-to-all dispatch and combine) timed in the same run at the same
N, with a per-phase breakdown and a parity figure against a dense fp32 restatement -- and, on one GPU, `device_resident`:
the grouped GEMM with the weights in HBM, against the tensor roofline.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: kind, experts, K, N, tokens, top_k, zipf_s
    "c3_fp8": dict(kind="fp8", experts=256, k=7168, n=4096, tokens=16384, top_k=8, zipf=0.8),
    "c2_bf16": dict(kind="bf16", experts=128, k=2048, n=1536, tokens=8192, top_k=8, zipf=1.0),
    "c1_int8": dict(kind="int8", experts=16, k=2048, n=1536, tokens=2048, top_k=4, zipf=0.0),
    "c2b_bf16": dict(kind="bf16", experts=128, k=768, n=2048, tokens=8192, top_k=8, zipf=1.0),
    # NVFP4, masked layout: 1024 rows per expert, valid counts from the routing, capped at the stride
    "c4_fp4": dict(kind="fp4", experts=128, k=4096, n=3072, tokens=16384, top_k=8, zipf=1.0, masked_stride=1024),
    # whole FP8 MoE layer, expert-parallel: gate+up (K=hidden, N=2*inter), SiLU*mul, down (K=inter, N=hidden)
    "c5_moe_fp8": dict(kind="moe", experts=256, hidden=7168, inter=2048, tokens=65536, top_k=8),
}
ELEM_BYTES = {"fp8": 1.0, "bf16": 2.0, "int8": 1.0, "fp4": 0.5}
# DRAM bytes (read + write) per padded row of A/D, from one ncu capture of a cut-down case of each workload with the
# default tile configuration (dram__bytes_read.sum + dram__bytes_write.sum over the padded rows of that launch): HBM
# traffic grows with the rows of the launch, not with the weights, which never touch HBM.
# (bytes, which rows): contiguous workloads scale with the padded rows of A / D, the masked one with its valid rows.
# Captured cuts: c3_fp8 16 experts, c2_bf16 / c2b_bf16 / c4_fp4 32 experts, c1_int8 whole (its 25 MB of D stay in L2).
NCU_DRAM_BYTES_PER_ROW = {"c3_fp8": (18.8e3, "padded"), "c2_bf16": (6.58e3, "padded"), "c2b_bf16": (3.47e3, "padded"),
                          "c1_int8": (2.29e3, "padded"), "c4_fp4": (8.56e3, "valid")}


def rows_per_expert(cfg, seed=0):
    gen = torch.Generator().manual_seed(seed)
    e = cfg["experts"]
    w = 1.0 / torch.arange(1, e + 1, dtype=torch.float64) ** cfg["zipf"]
    picks = torch.multinomial(w.expand(cfg["tokens"], -1), cfg["top_k"], replacement=False, generator=gen)
    return torch.bincount(picks.flatten(), minlength=e).tolist()


def build_workload(cfg, rank, world, device, seed=0, weights_on_device=False, huge_pages=False, expert_range=None, ue8m0=False):
    """Seeded synthetic operands for this rank's expert shard. B is quantised on the GPU and moved to pinned host.
    Every expert's weights and rows come from a generator keyed by the expert's global index, so an expert holds the same
    numbers whichever rank owns it (ranges are re-cut between warm-up and the timed steps)."""
    from asymgemm_b200.testing.moe_reference import expert_generator
    from asymgemm_b200.utils import (build_contiguous_layout, per_block_cast_to_fp8, per_channel_cast_to_int8,
                                     per_token_cast_to_fp8, per_token_cast_to_int8)
    kind, k, n = cfg["kind"], cfg["k"], cfg["n"]
    counts = rows_per_expert(cfg, seed)
    e_total = cfg["experts"]
    per = e_total // world
    lo, hi = expert_range if expert_range is not None else (rank * per, (rank + 1) * per if rank < world - 1 else e_total)
    counts = counts[lo:hi]
    g = len(counts)
    offsets, experts, list_size, m_total, segs = build_contiguous_layout(counts, device=device)
    valid = sum(c for c in counts)

    a_dtype = {"fp8": torch.float8_e4m3fn, "bf16": torch.bfloat16, "int8": torch.int8}[kind]
    a = torch.zeros((m_total, k), dtype=a_dtype, device=device)
    sfa = None if kind == "bf16" else torch.zeros((m_total, (k + 127) // 128), dtype=torch.float32, device=device)
    for e, start, rows in segs:
        x = torch.randn((rows, k), device=device, generator=expert_generator(device, seed, lo + e, 1))
        if kind == "fp8":
            q, s = per_token_cast_to_fp8(x, use_ue8m0=ue8m0)
            a[start:start + rows], sfa[start:start + rows] = q, s
        elif kind == "int8":
            q, s = per_token_cast_to_int8(x)
            a[start:start + rows], sfa[start:start + rows] = q, s
        else:
            a[start:start + rows] = x.to(torch.bfloat16)

    if huge_pages:
        from asymgemm_b200 import ep
        b_host = ep.pinned_empty((g, n, k), a_dtype, None, huge_pages=True)
    else:
        b_host = torch.empty((g, n, k), dtype=a_dtype).pin_memory()
    sfb = None
    if kind == "fp8":
        sfb = torch.empty((g, (n + 127) // 128, (k + 127) // 128), dtype=torch.float32, device=device)
    elif kind == "int8":
        sfb = torch.empty((g, n, k // 128), dtype=torch.float32, device=device)
    for e in range(g):
        w = torch.randn((n, k), device=device, generator=expert_generator(device, seed, lo + e, 0)) * 0.02
        if kind == "fp8":
            q, s = per_block_cast_to_fp8(w, use_ue8m0=ue8m0)
            sfb[e] = s
        elif kind == "int8":
            q, s = per_channel_cast_to_int8(w)
            sfb[e] = s
        else:
            q = w.to(torch.bfloat16)
        b_host[e].copy_(q, non_blocking=True)
    torch.cuda.synchronize(device)
    if weights_on_device:
        b_host = b_host.to(device)
    d = torch.empty((m_total, n), dtype=torch.bfloat16, device=device)
    active = sum(1 for c in counts if c > 0)
    return dict(kind=kind, a=a, sfa=sfa, b=b_host, sfb=sfb, d=d, offsets=offsets, experts=experts, list_size=list_size,
                m_total=m_total, valid_rows=valid, segs=segs, g=g, n=n, k=k, expert_lo=lo,
                flops=2.0 * n * k * valid, host_bytes=active * n * k * ELEM_BYTES[kind])


MOE_SEED = 5


def build_moe(cfg, rank, world, device, group, seed=MOE_SEED, expert_ranges=None, ue8m0=False, pipeline_groups=1, fused=True):
    """This rank's shard of the FP8 MoE layer (weights quantised on the GPU, then moved to pinned host memory, on the
    GPU's NUMA node when the platform exposes one) and this rank's slice of the token batch with its routing. Expert e's
    weights come from a generator keyed by e, so any rank can rebuild any expert for the parity check. `fused`: the gate+up
    weights are stored with gate and up rows interleaved (a weight-preparation step) and the layer fuses SiLU*mul into the
    gate+up GEMM's drain (exact-scale mode only)."""
    from asymgemm_b200 import ep
    from asymgemm_b200.testing.moe_reference import expert_generator, expert_weights
    e_total, h, i = cfg["experts"], cfg["hidden"], cfg["inter"]
    if expert_ranges is None:
        per = e_total // world
        expert_ranges = [(r * per, (r + 1) * per if r < world - 1 else e_total) for r in range(world)]
    lo, hi = expert_ranges[rank]
    epr = hi - lo
    node = ep.gpu_numa_node(device.index)
    w13 = ep.pinned_empty((epr, 2 * i, h), torch.float8_e4m3fn, node)
    w2 = ep.pinned_empty((epr, h, i), torch.float8_e4m3fn, node)
    s13 = torch.empty((epr, 2 * i // 128, h // 128), dtype=torch.float32, device=device)
    s2 = torch.empty((epr, h // 128, i // 128), dtype=torch.float32, device=device)
    fused = fused and not ue8m0
    for e in range(epr):
        q13, sc13, q2, sc2 = expert_weights(seed, lo + e, h, i, device, use_ue8m0=ue8m0)
        if fused:
            q13 = ep.interleave_gate_up(q13)
        w13[e].copy_(q13, non_blocking=True)
        s13[e] = sc13
        w2[e].copy_(q2, non_blocking=True)
        s2[e] = sc2
    torch.cuda.synchronize(device)
    layer = ep.ExpertParallelMoE(e_total, h, i, (w13, s13), (w2, s2), group, expert_ranges, ue8m0_scales=ue8m0,
                                 pipeline_groups=pipeline_groups, fused_activation=fused)
    t_local = cfg["tokens"] // world
    gen = expert_generator(device, seed, 100000 + rank, 3)      # this rank's tokens and router logits
    x = torch.randn((t_local, h), device=device, generator=gen).to(torch.bfloat16)
    logits = torch.randn((t_local, e_total), device=device, generator=gen)
    topk_w, topk_ids = torch.topk(torch.softmax(logits, dim=-1), cfg["top_k"], dim=-1)
    topk_w = topk_w / topk_w.sum(dim=-1, keepdim=True)
    rows = t_local * cfg["top_k"]
    return dict(kind="moe", layer=layer, x=x, ids=topk_ids, w=topk_w, numa_node=node, seed=seed, ue8m0=ue8m0, fused=fused,
                flops=float(rows) * 2.0 * (2 * i * h + h * i), host_bytes=float(epr) * (2 * i * h + h * i),
                nvlink_bytes=float(rows) * (h + h // 128 * 4 + 2 * h) * (world - 1) / world if world > 1 else 0.0)


def build_masked_fp4(cfg, rank, world, device, seed=0):
    """NVFP4 masked-layout operands: A [G, stride, K/2] + e4m3 scales on the device, B and its scales in pinned host memory."""
    from asymgemm_b200.utils import per_token_cast_to_nvfp4_e4m3
    k, n, stride = cfg["k"], cfg["n"], cfg["masked_stride"]
    counts = rows_per_expert(cfg, seed)
    per = cfg["experts"] // world
    counts = [min(c, stride) for c in counts[rank * per:(rank + 1) * per]]
    g = len(counts)
    gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    a = torch.zeros((g, stride, k // 2), dtype=torch.uint8, device=device)
    sfa = torch.zeros((g, stride, k // 16), dtype=torch.float8_e4m3fn, device=device)
    b = torch.empty((g, n, k // 2), dtype=torch.uint8).pin_memory()
    sfb = torch.empty((g, n, k // 16), dtype=torch.float8_e4m3fn).pin_memory()
    for e in range(g):
        if counts[e]:
            q, s = per_token_cast_to_nvfp4_e4m3(torch.randn((counts[e], k), device=device, generator=gen))
            a[e, :counts[e]], sfa[e, :counts[e]] = q, s
        q, s = per_token_cast_to_nvfp4_e4m3(torch.randn((n, k), device=device, generator=gen) * 0.02)
        b[e].copy_(q, non_blocking=True)
        sfb[e].copy_(s, non_blocking=True)
    torch.cuda.synchronize(device)
    valid = sum(counts)
    active = sum(1 for c in counts if c > 0)
    return dict(kind="fp4", a=a, sfa=sfa, b=b, sfb=sfb, d=torch.empty((g, stride, n), dtype=torch.bfloat16, device=device),
                masked_m=torch.tensor(counts, dtype=torch.int32, device=device), counts=counts, g=g, n=n, k=k, m_total=g * stride,
                valid_rows=valid,
                # the weight scales are re-laid out once and then stay on the device, so only the packed values stream per call;
                # host_bytes_with_scales is the figure that counts the (host-resident) scale bytes of the API tensors as well
                flops=2.0 * n * k * valid, host_bytes=active * n * k * 0.5, host_bytes_with_scales=active * n * (k * 0.5 + k / 16.0),
                segs=None)


def run_op(w, a=None, sfa=None, d=None):
    if w.get("cache") is not None:
        a_ = w["a"] if a is None else a
        d_ = w["d"] if d is None else d
        if w["kind"] == "fp8":
            return w["cache"].fp8_gemm((a_, w["sfa"] if sfa is None else sfa), d_, w["offsets"], w["experts"])
        return w["cache"].bf16_gemm(a_, d_, w["offsets"], w["experts"])
    if w["kind"] == "moe":
        return w["layer"].forward(w["x"] if a is None else a, w["ids"], w["w"])
    if w["kind"] == "fp4":
        import asymgemm_b200 as ag
        return ag.m_grouped_fp4_asym_gemm_nt_masked((w["a"] if a is None else a, w["sfa"] if sfa is None else sfa), (w["b"], w["sfb"]),
                                                    w["d"] if d is None else d, w["masked_m"], max(1, sum(w["counts"]) // w["g"]))
    import asymgemm_b200 as ag
    a = w["a"] if a is None else a
    sfa = w["sfa"] if sfa is None else sfa
    d = w["d"] if d is None else d
    if w["kind"] == "fp8":
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((a, sfa), (w["b"], w["sfb"]), d, w["offsets"], w["experts"], None)
    elif w["kind"] == "int8":
        ag.m_grouped_int8_asym_gemm_nt_contiguous((a, sfa), (w["b"], w["sfb"]), d, w["offsets"], w["experts"], None)
    else:
        ag.m_grouped_bf16_asym_gemm_nt_contiguous(a, w["b"], d, w["offsets"], w["experts"], None)


def gemm_launches_per_step(w, args):
    """Grouped-GEMM kernel launches of this library in one step (helper kernels of the MoE layer not counted)."""
    def chunks(g, group_bytes):
        if args.weights != "staged":
            return 1
        per = max(1, min(g, (args.stage_mb << 20) // int(group_bytes)))
        return (g + per - 1) // per
    if w["kind"] == "moe":
        layer = w["layer"]
        g = layer.w13[0].shape[0]
        rounds = layer.pipeline_groups if layer.dispatcher.world > 1 else 1
        if rounds > 1:      # every round launches both GEMMs over its share of the experts
            per = max(1, g // rounds)
            return rounds * (chunks(per, layer.w13[0][0].numel()) + chunks(per, layer.w2[0][0].numel()))
        return chunks(g, layer.w13[0][0].numel()) + chunks(g, layer.w2[0][0].numel())
    if w.get("cache") is not None:
        return 2
    return chunks(w["g"], w["b"][0].numel() * w["b"].element_size())


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for i, nm in enumerate(names):
                if len(r) > 3 + i and r[3 + i].lower().startswith("active"):
                    reasons.add(nm)
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_reference_sample(cfg, w, threads, max_experts):
    """The reference's CPU path on a bounded sample of this workload, all host threads.

    INT8: the reference's own cg_gemm (oracle/_ref) called once per expert, as csrc/cpu/module.cpp:329-373 does.
    Other dtypes: the reference's torch CPU loop `a[s:e] @ w.t()` (asym_gemm/training/frozen_linear.py:986-1008) on
    operands dequantised to bf16 beforehand (dequantisation is not timed).
    Returns (tflops, description, kind, cores).
    """
    from oracle import oracle as O
    kind, n, k = w["kind"], w["n"], w["k"]
    if kind == "fp4":
        return _cpu_reference_fp4(w, threads, max_experts)
    segs = [s for s in w["segs"] if s[2] > 0][:max_experts]
    torch.set_num_threads(threads)
    flops = 0.0
    if kind == "int8":
        from oracle import ref_cpu_gemm as R
        if R.available():
            rt = R.runtime(0)
            ops = []
            for e, start, rows in segs:
                a_f = (w["a"][start:start + rows].float() * w["sfa"][start:start + rows].repeat_interleave(128, 1)).cpu()
                a_bits = O.f32_to_bf16_bits(a_f.numpy())
                b_q = w["b"][e].numpy()
                s = w["sfb"][e].cpu().numpy()[:, 0].copy()   # cg_gemm takes one scale per output channel
                ops.append((a_bits, b_q, s))
                flops += 2.0 * rows * n * k
            t0 = time.perf_counter()
            for a_bits, b_q, s in ops:
                R.gemm_bf16_int8_f32(a_bits, b_q, s, rt)
            dt = time.perf_counter() - t0
            return flops / dt / 1e12, f"{len(segs)} experts of this workload through cg_gemm ({R.backend_name()})", "reference", R.threads(rt)
    ops = []
    for e, start, rows in segs:
        a_t = w["a"][start:start + rows]
        b_t = w["b"][e]
        if kind == "fp8":
            a_f = a_t.float() * w["sfa"][start:start + rows].repeat_interleave(128, 1)[:, :k]
            b_f = b_t.to(a_t.device).float() * w["sfb"][e].repeat_interleave(128, 0).repeat_interleave(128, 1)[:n, :k]
        elif kind == "int8":
            a_f = a_t.float() * w["sfa"][start:start + rows].repeat_interleave(128, 1)
            b_f = b_t.to(a_t.device).float() * w["sfb"][e].repeat_interleave(128, 1)
        else:
            a_f, b_f = a_t.float(), b_t.to(a_t.device).float()
        ops.append((a_f.to(torch.bfloat16).cpu(), b_f.to(torch.bfloat16).cpu()))
        flops += 2.0 * rows * n * k
    ops[0][0] @ ops[0][1].t()  # warm the thread pool
    t0 = time.perf_counter()
    for a_c, b_c in ops:
        a_c @ b_c.t()
    dt = time.perf_counter() - t0
    return flops / dt / 1e12, f"{len(segs)} experts of this workload, torch CPU bf16 `a[s:e] @ w.t()` per expert", "port", threads


def _dequant_fp4(packed, sf):
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32, device=packed.device)
    vals = torch.stack([lut[(packed & 0xF).long()], lut[(packed >> 4).long()]], dim=-1).flatten(-2)
    return vals * sf.float().repeat_interleave(16, dim=-1)


def _cpu_reference_fp4(w, threads, max_experts):
    """torch CPU bf16 loop over the first experts of the masked NVFP4 workload (operands dequantised beforehand)."""
    torch.set_num_threads(threads)
    ops, flops = [], 0.0
    for e in [i for i, c in enumerate(w["counts"]) if c > 0][:max_experts]:
        rows = w["counts"][e]
        a = _dequant_fp4(w["a"][e, :rows], w["sfa"][e, :rows]).to(torch.bfloat16).cpu()
        b = _dequant_fp4(w["b"][e].to(w["a"].device), w["sfb"][e].to(w["a"].device)).to(torch.bfloat16).cpu()
        ops.append((a, b))
        flops += 2.0 * rows * w["n"] * w["k"]
    ops[0][0] @ ops[0][1].t()
    t0 = time.perf_counter()
    for a, b in ops:
        a @ b.t()
    dt = time.perf_counter() - t0
    return flops / dt / 1e12, f"{len(ops)} experts of this workload, torch CPU bf16 `a[:m] @ w.t()` per expert", "port", threads


def pick_device(args, local_rank, world):
    """GPU this rank runs on. With as many ranks as visible GPUs (or one rank) rank r uses GPU r. With fewer ranks than GPUs
    the set of GPUs is chosen by measurement -- GPUs of one machine share host bridges, so which GPUs stream together
    decides the host-link rate more than anything else: local rank 0 runs asymgemm_b200/linkprobe.py in a child process
    (its CUDA contexts on the other GPUs die with it) and hands the map to the other ranks through a file named after
    the launcher's pid. Returns (device index, record for the JSON line or None)."""
    visible = torch.cuda.device_count()
    if world <= 1 or world >= visible or args.device_map == "identity":
        return local_rank, None
    path = Path("/tmp") / f"asymgemm_b200_devmap_{os.getppid()}_{os.environ.get('MASTER_PORT', '0')}.json"
    if local_rank == 0:
        info = None
        try:
            res = subprocess.run([sys.executable, str(ROOT / "asymgemm_b200" / "linkprobe.py"), "--choose", str(world), "--visible", str(visible)],
                                 capture_output=True, text=True, timeout=180)
            if res.returncode == 0:
                info = json.loads(res.stdout.strip().splitlines()[-1])
            else:
                info = {"devices": list(range(world)), "why": "link probe failed: " + res.stderr.strip()[-200:]}
        except Exception as e:  # noqa: BLE001 -- any failure of the probe falls back to the identity map, and says so
            info = {"devices": list(range(world)), "why": f"link probe failed: {type(e).__name__}: {e}"}
        tmp = path.with_suffix(".tmp")
        tmp.write_text(json.dumps(info))
        os.replace(tmp, path)
    else:
        t0 = time.time()
        while not path.exists():
            if time.time() - t0 > 240:
                raise RuntimeError("timed out waiting for local rank 0's device map")
            time.sleep(0.05)
        info = json.loads(path.read_text())
    return int(info["devices"][local_rank]), (info, path)


class RankLinks:
    """This rank's host-link figures, each measured with a barrier between set-up and the streaming interval so that
    "all ranks at once" really overlaps: copy-engine rate alone and together, and the SM-issued TMA read rate together."""

    def __init__(self, lib, _lib, row_bytes, barrier, rank, world):
        self.lib, self._lib = lib, _lib
        ce, tma = _lib.c_void_p(), _lib.c_void_p()
        _lib.check(lib.ag_link_probe_create(-1, 512 << 20, 0, 0, ce))
        _lib.check(lib.ag_link_probe_create(-1, 512 << 20, 1, row_bytes, tma))
        rate = _lib.c_double(0.0)
        self.alone = 0.0
        for r in range(world):          # one rank at a time, the others idle
            barrier()
            if r == rank:
                _lib.check(lib.ag_link_probe_run(ce, 0.25, rate))
                self.alone = rate.value
        barrier()
        _lib.check(lib.ag_link_probe_run(ce, 0.3, rate))
        self.together = rate.value
        barrier()
        _lib.check(lib.ag_link_probe_run(tma, 0.3, rate))
        self.tma_together = rate.value
        barrier()
        lib.ag_link_probe_destroy(ce)
        lib.ag_link_probe_destroy(tma)


def hbm_traffic_model(w, tile_bn=64, chunk_tiles=6, ka=2):
    """HBM bytes of one launch of the host-streamed kernel, from this run's own segment table: A and its scales read once,
    D written once, plus the scratch copy of every (segment, column tile) longer than one accumulator chunk (written once,
    read once per further chunk). A rows are read by every column tile of their segment; tiles that run together share
    them in L2, which is why the measured figure sits between this model and one more pass over A."""
    if w.get("segs") is None:
        return None
    k_bytes = w["a"].shape[1] * w["a"].element_size()
    kpad = (k_bytes + 128 * ka - 1) // (128 * ka) * (128 * ka)
    n_tiles = (w["n"] + tile_bn - 1) // tile_bn
    spill = replay = 0
    for _, _, rows in w["segs"]:
        chunks = ((rows + 127) // 128 + chunk_tiles - 1) // chunk_tiles
        if chunks > 1:
            spill += n_tiles * tile_bn * kpad
            replay += n_tiles * tile_bn * kpad * (chunks - 1)
    a = w["a"].numel() * w["a"].element_size() + (w["sfa"].numel() * 4 if w["sfa"] is not None else 0)
    d = w["valid_rows"] * w["n"] * w["d"].element_size()
    return {"a_and_scales_gb": round(a / 1e9, 3), "d_gb": round(d / 1e9, 3), "scratch_write_gb": round(spill / 1e9, 3),
            "scratch_replay_gb": round(replay / 1e9, 3), "total_gb": round((a + d + spill + replay) / 1e9, 3)}


def timed(fn, steps, barrier):
    """ms per call of fn over `steps` calls, CUDA events on the current stream, barrier + synchronize on both sides."""
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / steps


def measure_device_resident(device, peaks, steps=20):
    """The grouped GEMM with the weights resident in HBM (the tensor-bound regime): the FP8 configuration cut to 32 experts
    (tokens cut in proportion: the routing density of the full config, 0.94 GB of weights) and the BF16 configuration at
    full size (0.8 GB of weights); inputs larger than L2. For every kind the automatic tile and the other device tiles are
    timed and the best is reported with all figures beside it."""
    import asymgemm_b200 as ag
    out = {"note": "weights resident in HBM; peak = bf16_tflops of MEASURED_PEAKS.json (x2 for 8-bit operands), of measured" if peaks else
                   "weights resident in HBM; peak = 1590 TFLOP/s bf16 (x2 for 8-bit), of fallback"}
    bf16_peak = peaks.get("bf16_tflops", 1590.0)
    cases = [("fp8", "c3_fp8", False, (0, 5, 6, 8), 2.0, 32), ("fp8_ue8m0", "c3_fp8", True, (0, 7), 2.0, 32),
             ("bf16", "c2_bf16", False, (0, 1, 6, 7, 8), 1.0, 128), ("int8", "c3_fp8", False, (0, 5), 2.0, 32)]
    for name, wl, ue, tiles, mult, experts in cases:
        cfg = dict(WORKLOADS[wl])
        if name == "int8":
            cfg["kind"] = "int8"      # the FP8 configuration's shapes with INT8 operands and per-channel weight scales
        cfg["tokens"] = max(1, cfg["tokens"] * experts // cfg["experts"])
        cfg["experts"] = experts
        w = build_workload(cfg, 0, 1, device, weights_on_device=True, ue8m0=ue)
        ag.set_fp8_scale_mode("ue8m0" if ue else "fp32")
        best = None
        per_tile = {}
        for t in tiles:
            ag.set_tile_config(t)
            for _ in range(3):
                run_op(w)
            ms = timed(lambda: run_op(w), steps, lambda: torch.cuda.synchronize(device))
            ag.check_status()
            tf = w["flops"] / (ms * 1e-3) / 1e12
            per_tile["auto" if t == 0 else f"tile_config_{t}"] = round(tf, 1)
            if best is None or tf > best[0]:
                best = (tf, t, ms)
        ag.set_tile_config(0)
        ag.set_fp8_scale_mode("fp32")
        peak = mult * bf16_peak
        out[name] = {"tflops": round(best[0], 1), "ms_per_step": round(best[2], 4), "tile_config": best[1], "peak_tflops": round(peak, 1),
                     "frac": round(best[0] / peak, 4), "by_tile_config": per_tile,
                     "workload": f"{wl} with {experts} experts{' and int8 operands' if name == 'int8' else ''}: K={cfg['k']}, N={cfg['n']}, {w['valid_rows']} rows"}
        del w
        torch.cuda.empty_cache()
    # NVFP4 (masked layout, scales applied by the tensor core): the C4 configuration cut to 32 experts, weights moved to HBM
    cfg = dict(WORKLOADS["c4_fp4"])
    cfg["tokens"] = max(1, cfg["tokens"] * 32 // cfg["experts"])
    cfg["experts"] = 32
    w = build_masked_fp4(cfg, 0, 1, device)
    w["b"], w["sfb"] = w["b"].to(device), w["sfb"].to(device)
    per_tile = {}
    best = None
    for t in (0, 1):
        ag.set_tile_config(t)
        for _ in range(3):
            run_op(w)
        ms = timed(lambda: run_op(w), steps, lambda: torch.cuda.synchronize(device))
        ag.check_status()
        tf = w["flops"] / (ms * 1e-3) / 1e12
        per_tile["auto" if t == 0 else f"tile_config_{t}"] = round(tf, 1)
        if best is None or tf > best[0]:
            best = (tf, t, ms)
    ag.set_tile_config(0)
    out["nvfp4"] = {"tflops": round(best[0], 1), "ms_per_step": round(best[2], 4), "tile_config": best[1], "peak_tflops": round(4.0 * bf16_peak, 1),
                    "frac": round(best[0] / (4.0 * bf16_peak), 4), "by_tile_config": per_tile,
                    "workload": f"c4_fp4 with 32 experts (masked layout): K={cfg['k']}, N={cfg['n']}, {w['valid_rows']} rows; peak = 4 x bf16"}
    del w
    torch.cuda.empty_cache()
    return out


def cpu_moe_baseline(cfg, threads):
    """The reference's CPU implementation of the whole MoE layer on a bounded twin of the workload (experts / 8, tokens
    / 16): its INT8 bucket `moe_expert_forward_batch` (csrc/cpu/module.cpp:257-479, compiled from the reference's source into
    oracle/_ref) and, beside it, the torch CPU bf16 per-expert loop (asym_gemm/training/frozen_linear.py:986-1008
    semantics) on the same rows. Returns the record for the JSON line."""
    import numpy as np
    from oracle import oracle as O
    from oracle import ref_cpu_moe as RM
    h, i = cfg["hidden"], cfg["inter"]
    experts = max(1, cfg["experts"] // 8)
    rows_total = max(experts, cfg["tokens"] // 8 * cfg["top_k"])
    rng = np.random.default_rng(0)
    rows = np.full(experts, rows_total // experts, dtype=np.int64)
    off = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    flops = float(off[-1]) * 2.0 * 3 * h * i
    block = rng.standard_normal((min(int(off[-1]), 2048), h), dtype=np.float32)     # N(0,1) rows, repeated: values do not change the timing
    x = np.tile(block, (-(-int(off[-1]) // block.shape[0]), 1))[: int(off[-1])]
    sample = (f"{experts} experts x {int(rows[0])} rows of this layer (hidden {h}, inter {i}): experts / 8 and tokens / 8 of the "
              "workload, balanced routing")
    rec = {"unit": "TFLOP/s", "cores": threads, "sample": sample}
    torch.set_num_threads(threads)
    if RM.available():
        one = rng.integers(-127, 128, size=(i, h), dtype=np.int8)            # one random expert, repeated (1.4 GB of draws otherwise)
        sc = lambda *shape: np.full(shape, 0.02 / 127, dtype=np.float32)
        gate, up = np.ascontiguousarray(np.broadcast_to(one, (experts, i, h))), np.ascontiguousarray(np.broadcast_to(one[::-1], (experts, i, h)))
        down = np.ascontiguousarray(np.broadcast_to(one.reshape(h, i), (experts, h, i)))
        x_bits = O.f32_to_bf16_bits(x)
        out = np.zeros((int(off[-1]), h), dtype=np.float32)
        rt = RM.runtime(0)
        ids = np.arange(experts, dtype=np.int64)
        RM.moe_expert_forward_batch(x_bits[: int(off[1])], off[:2], ids[:1], gate, sc(experts, i), up, sc(experts, i), down, sc(experts, h), rt,
                                    out[: int(off[1])])          # warm the pool
        t0 = time.perf_counter()
        RM.moe_expert_forward_batch(x_bits, off, ids, gate, sc(experts, i), up, sc(experts, i), down, sc(experts, h), rt, out)
        dt = time.perf_counter() - t0
        rec.update({"value": round(flops / dt / 1e12, 4), "kind": "reference", "seconds": round(dt, 2), "cores": int(rt.threads() if callable(rt.threads) else rt.threads),
                    "what": f"reference moe_expert_forward_batch (INT8 weights, bf16 activations, {RM.caps().get('int8_rm_backend')})"})
        del gate, up, down, out, x_bits
    # torch CPU bf16 loop on the same rows
    xt = torch.from_numpy(x).to(torch.bfloat16)
    w13 = (torch.randn((2 * i, h)) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn((h, i)) * 0.02).to(torch.bfloat16)
    (xt[:64] @ w13.t())
    t0 = time.perf_counter()
    for e in range(experts):
        hh = xt[off[e]:off[e + 1]] @ w13.t()
        act = (torch.nn.functional.silu(hh[:, :i].float()) * hh[:, i:].float()).to(torch.bfloat16)
        act @ w2.t()
    dt = time.perf_counter() - t0
    rec["torch_bf16_loop"] = {"value": round(flops / dt / 1e12, 4), "unit": "TFLOP/s", "kind": "port", "cores": threads, "seconds": round(dt, 2)}
    if "value" not in rec:
        rec.update({"value": rec["torch_bf16_loop"]["value"], "kind": "port", "what": "torch CPU bf16 per-expert loop"})
    return rec


def measure_ep_layer(args, cfg, rank, world, device, barrier, ranges, link_alone_sum, steps):
    """The expert-parallel FP8 MoE layer at this N: ms per step (max over ranks), TFLOP/s, weight GB/s (aggregate and per
    rank), per-phase CUDA-event breakdown of an unpipelined step, bytes crossing NVLink, and the parity of a sample of this
    rank's tokens against the dense fp32 restatement (outside the timed region)."""
    import asymgemm_b200 as ag
    import torch.distributed as dist
    from asymgemm_b200 import ep
    from asymgemm_b200.testing import calc_diff, max_rel_err
    from asymgemm_b200.testing.moe_reference import dense_moe_reference, expert_weights
    ue = args.fp8_scales == "ue8m0"
    w = build_moe(cfg, rank, world, device, None, expert_ranges=ranges, ue8m0=ue, pipeline_groups=args.pipeline_groups)
    layer = w["layer"]
    nccl_ms = peer_ms = None
    chosen = "nccl"
    if args.exchange in ("nccl", "both"):
        step = lambda: layer.forward(w["x"], w["ids"], w["w"])
        for _ in range(2):
            y = step()
        ag.check_status()
        nccl_ms = timed(step, steps, barrier)
        ag.check_status()
    peer_layer, peer_error = None, None
    if args.exchange in ("peer", "both") and args.pipeline_groups <= 1:
        try:      # construction fails on every rank together or on none (ep_peer.PeerExchange)
            peer_layer = ep.ExpertParallelMoE(cfg["experts"], cfg["hidden"], cfg["inter"], layer.w13, layer.w2, None, ranges, ue8m0_scales=ue,
                                              exchange="peer", max_tokens=w["x"].shape[0], top_k=cfg["top_k"], fused_activation=w["fused"])
        except RuntimeError as e:
            peer_error = str(e)[:300]
            if args.exchange == "peer":
                raise
    if peer_layer is not None:
        pstep = lambda: peer_layer.forward(w["x"], w["ids"], w["w"])
        for _ in range(2):
            y_peer = pstep()
        ag.check_status()
        peer_ms = timed(pstep, steps, barrier)
        ag.check_status()
        differs = 0.0 if nccl_ms is None or torch.equal(y_peer, y) else 1.0
        # the faster exchange (by the slowest rank's time) is the one the record describes
        both = torch.tensor([nccl_ms if nccl_ms is not None else 1e30, peer_ms, differs], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(both, op=dist.ReduceOp.MAX)
        if both[1].item() <= both[0].item():
            chosen, step, y = "peer", pstep, y_peer
        nccl_all, peer_all = (both[0].item() if nccl_ms is not None else None), both[1].item()
        same = (both[2].item() == 0.0) if nccl_ms is not None else None
    ms = peer_ms if chosen == "peer" else nccl_ms
    if chosen == "peer":
        layer = peer_layer
    # The same layer with the weights moved by the copy engine through an 8-slot ring in HBM that the layer prefetches into
    # while tokens are routed, exchanged and combined (set_weight_path("staged")): the transport the reference's runtime uses.
    staged_ms = staged_same = None
    if args.weights == "host" and not (args.pipeline_groups > 1 and world > 1):
        ag.set_weight_path("staged", chunk_bytes=args.stage_mb << 20, slots=8)
        layer.prefetch_next = layer.w13[0]
        try:
            for _ in range(2):
                y_staged = step()
            ag.check_status()
            staged_ms = timed(step, steps, barrier)
            ag.check_status()
            flags = torch.tensor([staged_ms, 0.0 if torch.equal(y_staged, y) else 1.0], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(flags, op=dist.ReduceOp.MAX)
            staged_ms, staged_same = flags[0].item(), flags[1].item() == 0.0
        finally:
            layer.prefetch_next = None
            ag.set_weight_path("stream", chunk_bytes=args.stage_mb << 20, slots=args.stage_slots)
            torch.cuda.synchronize(device)
    # per-phase breakdown: two more steps with events at the phase boundaries (unpipelined path only)
    phases = None
    if not (args.pipeline_groups > 1 and world > 1):
        acc = {}
        for _ in range(2):
            layer.phase_events = []
            step()
            torch.cuda.synchronize(device)
            ev = layer.phase_events
            for (_, a), (name, b) in zip(ev[:-1], ev[1:]):
                acc[name] = acc.get(name, 0.0) + a.elapsed_time(b) / 2
        layer.phase_events = None
        phases = {k: round(v, 3) for k, v in acc.items()}
    # parity of a sample of this rank's tokens (their experts may live on any rank: weights are rebuilt from the seed)
    sample = min(args.parity_tokens, w["x"].shape[0])
    h, i = cfg["hidden"], cfg["inter"]
    ref = dense_moe_reference(w["x"][:sample], w["ids"][:sample], w["w"][:sample],
                              lambda e: expert_weights(w["seed"], e, h, i, device, use_ue8m0=ue), i, use_ue8m0=ue)
    got = y[:sample].float()
    stats = torch.tensor([ms, w["flops"], w["host_bytes"], w["host_bytes"] / (ms * 1e-3) / 1e9, max_rel_err(got, ref), calc_diff(got, ref),
                          w["nvlink_bytes"]], dtype=torch.float64, device=device)
    if world > 1:
        mx, sm, mn = stats.clone(), stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        if phases is not None:
            keys = sorted(phases)
            pt = torch.tensor([phases[k] for k in keys], dtype=torch.float64, device=device)
            dist.all_reduce(pt, op=dist.ReduceOp.MAX)
            phases = {k: round(v, 3) for k, v in zip(keys, pt.tolist())}
    else:
        mx = sm = mn = stats
    ms_all = mx[0].item()
    rec = {
        "workload": (f"FP8 MoE layer, {cfg['experts']} experts over {world} rank(s), gate+up K={h} N={2 * i}, SiLU*mul, down K={i} N={h}, "
                     f"{cfg['tokens']} tokens x top-{cfg['top_k']} (softmax of N(0,1) logits), weights in pinned host memory per rank"
                     + (", NCCL all-to-all(v) dispatch and combine" if world > 1 else ", one rank: no exchange")),
        "ms_per_step": round(ms_all, 3), "steps": steps,
        "tflops": round(sm[1].item() / (ms_all * 1e-3) / 1e12, 2),
        "weight_gbs": round(sm[2].item() / (ms_all * 1e-3) / 1e9, 2),
        "per_rank_weight_gbs_min_max": [round(mn[3].item(), 2), round(mx[3].item(), 2)],
        "frac_of_link_peak_sum": round(sm[2].item() / (ms_all * 1e-3) / 1e9 / link_alone_sum, 4) if link_alone_sum > 0 else None,
        "phase_ms_max_over_ranks": phases,
        "nvlink_gb_per_step": round(sm[6].item() / 1e9, 3),
        "parity_tokens_per_rank": sample, "parity_max_rel": float(f"{mx[4].item():.3e}"), "parity_calc_diff": float(f"{mx[5].item():.3e}"),
        "parity_against": "dense fp32 restatement of the layer on dequantised operands (asymgemm_b200/testing/moe_reference.py), "
                          "worst rank; tolerance of the FP8 path: max-rel <= 2e-2",
        "experts_per_rank": [hi - lo for lo, hi in ranges] if ranges is not None else [cfg["experts"] // world] * world,
        "gemm_launches_per_step": 2 * (args.pipeline_groups if world > 1 else 1),
        "exchange": {"nccl": "sort + gather + NCCL all-to-all(v), split sizes read back on the host",
                     "peer": "this library's kernels: histogram, plan, rows stored into the owner's layout over NVLink peer memory; the down "
                             "GEMM's drain stores every result row straight into the source rank's combine buffer; no host synchronisation"}[chosen],
    }
    rec["activation"] = ("SiLU*mul fused into the gate+up GEMM's drain (weights stored with gate / up rows interleaved)" if w["fused"]
                         else "separate SiLU*mul + requantisation kernel")
    if staged_ms is not None:
        rec["copy_engine_staged_ring"] = {"ms_per_step": round(staged_ms, 3), "weight_gbs": round(sm[2].item() / (staged_ms * 1e-3) / 1e9, 2),
                                          "outputs_bit_equal": staged_same,
                                          "note": "same layer and exchange with set_weight_path('staged', slots=8) and the layer's prefetch of its "
                                                  "gate+up weights during routing / exchange / combine; the record's own numbers are the in-kernel stream"}
    if peer_error is not None:
        rec["peer_exchange_unavailable"] = peer_error
    if peer_ms is not None:
        rec["exchange_ms_per_step"] = {"nccl": round(nccl_all, 3) if nccl_all is not None else None, "peer": round(peer_all, 3),
                                       "outputs_bit_equal": same}
    if args.pipeline_groups > 1 and world > 1:
        rec["pipeline_groups"] = args.pipeline_groups
    if peer_ms is not None:
        peer_layer.peer.close()
    del w, layer, y
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c3_fp8", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--experts", type=int, default=0, help="shrink the expert count (tokens shrink in proportion); 0 = full size")
    ap.add_argument("--tokens", type=int, default=0,
                    help="override the token count of the workload (decode-sized batches leave experts without rows: the in-kernel "
                         "stream skips those, the staged path copies them all); 0 = the named config")
    ap.add_argument("--pipeline-groups", type=int, default=1,
                    help="MoE layer on several GPUs: run the layer in this many rounds over groups of each rank's experts so that "
                         "the token exchanges overlap the GEMMs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--weights", default="host", choices=["host", "device", "staged"],
                    help="host (default): B in pinned host memory, read by the kernel itself; device: B resident in HBM (tensor-bound "
                         "regime); staged: B in pinned host memory, copied chunk by chunk into an HBM double buffer by the copy engine "
                         "(set_weight_path) -- the alternative the in-kernel stream is compared with")
    ap.add_argument("--stage-mb", type=int, default=128, help="--weights staged: size of one staged chunk of whole experts, MiB")
    ap.add_argument("--stage-slots", type=int, default=2,
                    help="--weights staged: slots of the staging ring (2 = double buffer); more slots let the MoE layer's prefetch bank "
                         "more weight bytes while tokens are exchanged")
    ap.add_argument("--d-host", action="store_true", help="end-to-end leg: let the kernel write D straight into pinned host memory")
    ap.add_argument("--fp8-scales", default="fp32", choices=["fp32", "ue8m0"],
                    help="fp32 (default): arbitrary fp32 block scales applied exactly in the TMEM drain; ue8m0: power-of-two scales "
                         "(use_ue8m0 quantisers) applied by the tensor core, the reference's SM100 numerics")
    ap.add_argument("--cache-experts", type=int, default=0,
                    help="keep this many of the most popular experts resident in HBM (HotExpertCache); the rest stream from the host")
    ap.add_argument("--even-shards", action="store_true",
                    help="N > 1: give every rank the same number of experts (no link calibration, no re-sharding)")
    ap.add_argument("--device-map", default="auto", choices=["auto", "identity"],
                    help="auto (default): with fewer ranks than visible GPUs, choose the GPUs by measuring their host links together; "
                         "identity: rank r on GPU r")
    ap.add_argument("--exchange", default="both", choices=["nccl", "peer", "both"],
                    help="token exchange of the MoE layer: nccl (sort + all-to-all(v)), peer (this library's kernels storing rows into the "
                         "owner's buffers over NVLink), both (default: `ep_layer` times the two and reports the faster as its headline)")
    ap.add_argument("--no-ep-layer", action="store_true", help="skip the `ep_layer` record (the expert-parallel MoE layer at this N)")
    ap.add_argument("--ep-tokens", type=int, default=0, help="token count of the `ep_layer` record (default: the 65536 of the named config)")
    ap.add_argument("--parity-tokens", type=int, default=256, help="tokens per rank checked against the dense restatement in `ep_layer`")
    ap.add_argument("--no-device-resident", action="store_true", help="skip the `device_resident` record (one GPU only)")
    ap.add_argument("--huge-pages", action="store_true", help="back the pinned weights with transparent huge pages (mmap + madvise + cudaHostRegister)")
    ap.add_argument("--tile", type=int, default=0, help="force a tile configuration (0 = automatic)")
    ap.add_argument("--sms", type=int, default=0, help="cap the number of CTAs (0 = all SMs)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cfg = dict(WORKLOADS[args.workload])
    if args.experts and args.experts < cfg["experts"]:
        cfg["tokens"] = max(1, cfg["tokens"] * args.experts // cfg["experts"])
        cfg["experts"] = args.experts
    if args.tokens > 0:
        cfg["tokens"] = args.tokens
    if cfg["kind"] == "moe":
        desc = (f"{args.workload}: FP8 MoE layer (gate+up K={cfg['hidden']} N={2 * cfg['inter']}, SiLU*mul, down K={cfg['inter']} "
                f"N={cfg['hidden']}), {cfg['experts']} experts sharded over the ranks, {cfg['tokens']} tokens x top-{cfg['top_k']} "
                f"(softmax of N(0,1) logits), token all-to-all over NCCL, weights in pinned host DRAM per rank")
    else:
        layout = f"masked (stride {cfg['masked_stride']})" if "masked_stride" in cfg else "contiguous"
        desc = (f"{args.workload}: m-grouped {layout} {cfg['kind']} GEMM, {cfg['experts']} experts, K={cfg['k']}, N={cfg['n']}, "
                f"{cfg['tokens']} tokens x top-{cfg['top_k']}, Zipf({cfg['zipf']}), B in pinned host DRAM")
    config = {"workload": desc, "experts_per_gpu": cfg["experts"] // world,
              "l2": "inputs larger than L2 (weights are re-read from host memory every step)"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        return reference_arm(args, cfg, config)

    dev_index, devmap = pick_device(args, local_rank, world)
    device = torch.device("cuda", dev_index)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    import asymgemm_b200 as ag
    from asymgemm_b200 import _lib
    from asymgemm_b200.ep import proportional_expert_ranges, rebalance_expert_ranges

    if devmap is not None:
        info, path = devmap
        config["device_map"] = {"rank_to_gpu": info["devices"], **{k: v for k, v in info.items() if k != "devices"}}
    moe = cfg["kind"] == "moe"
    on_dev = args.weights == "device"
    lib = _lib.load()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def gather(value):
        t = torch.zeros(world, dtype=torch.float64, device=device)
        t[rank] = value
        if world > 1:
            dist.all_reduce(t)
        return t.tolist()

    # measured host-link figures (sustained, mean): copy engine alone / all ranks at once, TMA reads all ranks at once
    row_bytes = max(128, int(cfg["hidden"] if moe else cfg["k"] * ELEM_BYTES[cfg["kind"]]) // 128 * 128)
    links = RankLinks(lib, _lib, row_bytes, barrier, rank, world)
    link_peak, link_peak_together, stream_ceiling = links.alone, links.together, links.tma_together
    tma_rates = gather(links.tma_together)

    ranges = None
    shard = world > 1 and cfg["kind"] != "fp4" and not on_dev and not args.even_shards
    if shard:
        ranges = proportional_expert_ranges(tma_rates, cfg["experts"])
        config["sharding"] = {"how": "contiguous expert ranges; first cut in proportion to each rank's TMA read rate of pinned memory measured "
                                     "with all ranks streaming at once (mean over 0.3 s; equal when within 10 %), then re-cut from the "
                                     "ranks' own step times after the warm-up steps",
                              "calibration_gbs": [round(x, 1) for x in tma_rates], "first_cut": [hi - lo for lo, hi in ranges]}

    def build(rng):
        if moe:
            return build_moe(cfg, rank, world, device, None, expert_ranges=rng, ue8m0=args.fp8_scales == "ue8m0",
                             pipeline_groups=args.pipeline_groups)
        if cfg["kind"] == "fp4":
            return build_masked_fp4(cfg, rank, world, device)
        return build_workload(cfg, rank, world, device, weights_on_device=on_dev, huge_pages=args.huge_pages,
                              expert_range=rng[rank] if rng is not None else None, ue8m0=args.fp8_scales == "ue8m0")

    w = build(ranges)
    if moe and args.pipeline_groups > 1 and world > 1:
        config["pipeline"] = (f"{args.pipeline_groups} rounds over groups of each rank's experts; exchanges on a second stream "
                              "overlap the GEMMs")
    if args.cache_experts > 0 and cfg["kind"] in ("fp8", "bf16") and not on_dev:
        from asymgemm_b200.expert_cache import HotExpertCache
        cache = HotExpertCache(w["b"], w["sfb"], args.cache_experts, device)
        counts = [0] * w["g"]
        for e, _, r in w["segs"]:
            counts[e] = r
        cache.refresh(counts)
        torch.cuda.synchronize(device)
        w["cache"] = cache
        streamed = sum(1 for e, _, r in w["segs"] if r > 0 and e not in set(cache.cached))
        w["host_bytes"] = streamed * w["n"] * w["k"] * ELEM_BYTES[cfg["kind"]]
        config["hot_expert_cache"] = f"{len(cache.cached)} most popular experts resident in HBM, {streamed} streamed from the host"
    if args.weights == "staged":
        ag.set_weight_path("staged", chunk_bytes=args.stage_mb << 20, slots=args.stage_slots)
        if moe and args.pipeline_groups <= 1:
            # the layer is called in a loop: the first chunks of its gate+up weights are copied while the previous step's
            # results are combined and this step's tokens are routed (a model would prefetch the next layer's weights)
            w["layer"].prefetch_next = w["layer"].w13[0]
        config["staged"] = (f"weights cross the link through the copy engine, about {args.stage_mb} MiB of whole experts per chunk "
                            f"into a ring of {args.stage_slots} slots in HBM; the grouped GEMM of a chunk runs from HBM while the next chunks are copied; every expert "
                            "is copied, the reported GB/s count the active experts' bytes only")
    if args.fp8_scales == "ue8m0":
        ag.set_fp8_scale_mode("ue8m0")
        config["fp8_scales"] = "power-of-two (UE8M0), applied by the tensor core"
    if on_dev:
        config["workload"] = config["workload"].replace("B in pinned host DRAM", "B resident in HBM")
    ag.set_tile_config(args.tile)
    if args.sms:
        ag.set_num_sms(args.sms)

    def warm(wk, n):
        """n untimed steps; returns this rank's mean ms per step over all but the first."""
        ts = []
        for _ in range(n):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            a.record()
            run_op(wk)
            b.record()
            torch.cuda.synchronize(device)
            ts.append(a.elapsed_time(b))
        ag.check_status()
        return sum(ts[1:]) / max(1, len(ts) - 1) if len(ts) > 1 else ts[0]

    my_ms = warm(w, args.warmup)
    # closed loop: re-cut the expert ranges from what the ranks measured on real steps, rebuild, warm up again
    if shard:
        history = []
        for _ in range(2):
            step_ms = gather(my_ms)
            new = rebalance_expert_ranges(ranges, step_ms)
            history.append({"experts_per_rank": [hi - lo for lo, hi in ranges], "ms_per_rank": [round(x, 2) for x in step_ms]})
            if new == ranges:
                break
            ranges = new
            del w
            torch.cuda.empty_cache()
            w = build(ranges)
            my_ms = warm(w, args.warmup)
        config["sharding"]["closed_loop"] = history
        config["experts_per_rank"] = [hi - lo for lo, hi in ranges]

    barrier()
    sampler = ClockSampler(dev_index)
    if rank == 0:
        sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_all0, t_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_all0.record()
    for s in range(args.steps):
        evs[s][0].record()
        run_op(w)
        evs[s][1].record()
    t_all1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ag.check_status()
    total_ms = t_all0.elapsed_time(t_all1)
    kernel_ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps

    # end to end through the operator with host buffers: pinned A (+scales) in, D out, every step
    if moe:
        a_host, sfa_host = w["x"].cpu().pin_memory(), None
        d_host = torch.empty(w["x"].shape, dtype=torch.bfloat16).pin_memory()
        a_dev = torch.empty_like(w["x"])

        def e2e_step():
            a_dev.copy_(a_host, non_blocking=True)
            d_host.copy_(run_op(w, a_dev), non_blocking=True)
    else:
        a_host = w["a"].cpu().pin_memory()
        sfa_host = w["sfa"].cpu().pin_memory() if w["sfa"] is not None else None
        d_host = torch.empty(w["d"].shape, dtype=w["d"].dtype).pin_memory()
        a_dev, d_dev = torch.empty_like(w["a"]), torch.empty_like(w["d"])
        sfa_dev = torch.empty_like(w["sfa"]) if w["sfa"] is not None else None

        # Results leave through a second stream and two device buffers, so the device->host read of step i (the idle
        # direction of the link) overlaps the kernel of step i+1; uploads share the weights' direction and stay in order.
        out_stream = torch.cuda.Stream(device=device)
        d_bufs = [d_dev, torch.empty_like(d_dev)]
        done = [torch.cuda.Event(), torch.cuda.Event()]
        copied = [torch.cuda.Event(), torch.cuda.Event()]
        e2e_count = [0]

        def e2e_step():
            j = e2e_count[0] & 1
            e2e_count[0] += 1
            main = torch.cuda.current_stream(device)
            main.wait_event(copied[j])
            a_dev.copy_(a_host, non_blocking=True)
            if sfa_dev is not None:
                sfa_dev.copy_(sfa_host, non_blocking=True)
            if args.d_host:
                run_op(w, a_dev, sfa_dev, d_host)
                return
            run_op(w, a_dev, sfa_dev, d_bufs[j])
            done[j].record(main)
            with torch.cuda.stream(out_stream):
                out_stream.wait_event(done[j])
                d_host.copy_(d_bufs[j], non_blocking=True)
                copied[j].record(out_stream)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(8, min(args.steps, 16))      # its own loop: the last step's download is not overlapped with anything
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    if not moe:
        torch.cuda.current_stream(device).wait_stream(out_stream)   # the last result has reached the host
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    ag.check_status()

    # the same step and the same end-to-end loop with the weights moved by the copy engine instead of read by the kernel
    alt_ms = alt_e2e_ms = 0.0
    alt = args.weights == "host" and w.get("cache") is None and not args.d_host
    if alt:
        ag.set_weight_path("staged", chunk_bytes=args.stage_mb << 20)
        for _ in range(2):
            run_op(w)
        alt_ms = timed(lambda: run_op(w), args.steps, barrier)
        e2e_step()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(e2e_steps):
            e2e_step()
        if not moe:
            torch.cuda.current_stream(device).wait_stream(out_stream)
        s1.record()
        barrier()
        alt_e2e_ms = s0.elapsed_time(s1) / e2e_steps
        ag.set_weight_path("stream")
        ag.check_status()

    my_gbs = w["host_bytes"] / (total_ms / args.steps * 1e-3) / 1e9
    stats = torch.tensor([total_ms / args.steps, e2e_ms, kernel_ms, w["flops"], w["host_bytes"], link_peak, link_peak_together,
                          stream_ceiling, my_gbs, alt_ms, alt_e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        mn = stats.clone()
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        ms_step, e2e_ms, kernel_ms = mx[0].item(), mx[1].item(), mx[2].item()
        flops, host_bytes = sm[3].item(), sm[4].item()
        link_peak_sum, link_peak_min = sm[5].item(), mn[5].item()
        together_sum, together_min = sm[6].item(), mn[6].item()
        ceil_sum, ceil_min = sm[7].item(), mn[7].item()
        rank_gbs_min, rank_gbs_max = mn[8].item(), mx[8].item()
        alt_ms, alt_e2e_ms = mx[9].item(), mx[10].item()
    else:
        ceil_sum = ceil_min = stream_ceiling
        rank_gbs_min = rank_gbs_max = my_gbs
        ms_step, flops, host_bytes = stats[0].item(), w["flops"], w["host_bytes"]
        link_peak_sum = link_peak_min = link_peak
        together_sum = together_min = link_peak_together

    # what the default line carries beside the headline: the expert-parallel layer at this N, the device-resident regime
    h2d = int(a_host.numel() * a_host.element_size() + (sfa_host.numel() * sfa_host.element_size() if sfa_host is not None else 0))
    d2h = int(d_host.numel() * d_host.element_size())
    rank0_w = {k: w.get(k) for k in ("host_bytes", "flops", "m_total", "valid_rows", "n", "host_bytes_with_scales")}
    traffic_model = hbm_traffic_model(w) if not moe and cfg["kind"] != "fp4" and args.weights == "host" and args.tile == 0 else None
    launches = args.steps * gemm_launches_per_step(w, args)
    extras = {}
    default_line = args.workload == "c3_fp8" and args.weights == "host" and not args.cache_experts
    cpu_sample = None
    if world == 1 and not args.no_cpu_baseline and not moe:
        cpu_sample = cpu_reference_sample(cfg, w, os.cpu_count() or 1, max_experts=8)
    numa = w.get("numa_node")
    del w, a_host, d_host, a_dev
    if not moe:
        del d_bufs, d_dev, sfa_host, sfa_dev
    torch.cuda.empty_cache()
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    if default_line and not args.no_ep_layer:
        ep_cfg = dict(WORKLOADS["c5_moe_fp8"])
        if args.experts and args.experts < ep_cfg["experts"]:
            ep_cfg["tokens"] = max(world, ep_cfg["tokens"] * args.experts // ep_cfg["experts"])
            ep_cfg["experts"] = args.experts
        if args.ep_tokens > 0:
            ep_cfg["tokens"] = args.ep_tokens
        ep_ranges = None
        if ranges is not None and ranges[-1][1] == ep_cfg["experts"]:
            ep_ranges = ranges            # the layer's weights have the same bytes per expert ratio on every rank: same cut
        extras["ep_layer"] = measure_ep_layer(args, ep_cfg, rank, world, device, barrier, ep_ranges, link_peak_sum, steps=max(2, min(args.steps, 5)))
        if world == 1 and not args.no_cpu_baseline and rank == 0:
            extras["ep_layer"]["cpu_baseline"] = cpu_moe_baseline(ep_cfg, os.cpu_count() or 1)
    if default_line and world == 1 and not args.no_device_resident:
        extras["device_resident"] = measure_device_resident(device, peaks)

    if rank == 0:
        tflops = flops / (ms_step * 1e-3) / 1e12
        host_gbs = host_bytes / (ms_step * 1e-3) / 1e9
        # roofline of the one kernel in the step, on this rank's launch (rank 0) -- bound by the host link
        ach = rank0_w["host_bytes"] / (kernel_ms * 1e-3) / 1e9
        tensor_peak = {"fp8": 2.0, "int8": 2.0, "bf16": 1.0, "moe": 2.0, "fp4": 4.0}[cfg["kind"]] * peaks.get("bf16_tflops", 1590.0)
        line = {
            "metric": "grouped-GEMM TFLOPS (with host->GPU weight GB/s vs measured PCIe peak)",
            "value": round(tflops, 3), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"fp8": "fp8_e4m3 (fp32 accumulate)", "bf16": "bf16 (fp32 accumulate)", "int8": "int8 (int32 accumulate)",
                      "moe": "fp8_e4m3 (fp32 accumulate)", "fp4": "nvfp4 e2m1 + ue4m3 block scales (fp32 accumulate)"}[cfg["kind"]],
            "data": "synthetic (seeded; shapes of the named config, random weights)",
            "config": config,
            "host_link": {"weight_gbs": round(host_gbs, 2), "peak_gbs_sum": round(link_peak_sum, 2),
                          "frac_of_measured_peak": round(host_gbs / link_peak_sum, 4), "per_gpu_peak_min_gbs": round(link_peak_min, 2),
                          "peak_all_ranks_at_once_gbs_sum": round(together_sum, 2), "per_gpu_at_once_min_gbs": round(together_min, 2),
                          "frac_of_peak_all_ranks_at_once": round(host_gbs / together_sum, 4),
                          "tma_copy_only_all_ranks_at_once_gbs_sum": round(ceil_sum, 2), "tma_copy_only_per_gpu_min_gbs": round(ceil_min, 2),
                          "per_rank_weight_gbs_min_max": [round(rank_gbs_min, 2), round(rank_gbs_max, 2)],
                          "peak_how": "cudaMemcpyAsync pinned->device, 512 MiB buffer, mean over a sustained 0.25-0.3 s of copies, measured in "
                                      "this run with a barrier between set-up and streaming: peak_gbs_sum adds each rank's rate measured "
                                      "while the others idle, peak_all_ranks_at_once adds the rates measured with every rank copying at "
                                      "the same time; tma_copy_only is a copy-only TMA kernel with the weight producer's access pattern "
                                      "on every SM, all ranks at once (a reference, not a bound). The step ends when the slowest rank "
                                      "ends, so weight_gbs <= sum over ranks of (its experts' bytes / the slowest rank's time)"},
            "roofline": {"bound": "host_link", "achieved": round(ach, 2), "peak": round(link_peak, 2), "unit": "GB/s",
                         "frac": round(ach / link_peak, 4),
                         "frac_of_peak_all_ranks_at_once": round(ach / link_peak_together, 4) if link_peak_together > 0 else None,
                         "traffic": (round(NCU_DRAM_BYTES_PER_ROW[args.workload][0]
                                           * rank0_w["m_total" if NCU_DRAM_BYTES_PER_ROW[args.workload][1] == "padded" else "valid_rows"] / 1e9, 3)
                                     if args.workload in NCU_DRAM_BYTES_PER_ROW and not moe and args.weights == "host" else None),
                         "traffic_unit": "GB of HBM traffic per launch: ncu dram bytes per row (padded rows; valid rows for the masked "
                                         "layout) of a cut-down capture of this workload x the rows of this launch (traffic grows with "
                                         "rows, not with the weights, which never touch HBM)",
                         "traffic_model": traffic_model,
                         "algorithmic_gb": round(rank0_w["host_bytes"] / 1e9, 3),
                         "note": "algorithmic bytes = each active expert's weights once (N*K*bytes); the kernel is bound by the PCIe "
                                 "host link, not HBM or tensor throughput: peak is the copy-engine rate of this rank's link measured "
                                 "alone in this run (frac_of_peak_all_ranks_at_once: against its rate with every rank copying); "
                                 "traffic_model is computed from this run's segment table",
                         "tensor_frac_of_measured": round(rank0_w["flops"] / (kernel_ms * 1e-3) / 1e12 / tensor_peak, 5)},
            "e2e": {"value": round(flops / (e2e_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "weights are read from pinned host memory inside the kernel in both timings"},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if rank0_w.get("host_bytes_with_scales"):
            line["host_link"]["weight_gbs_counting_scale_bytes"] = round(rank0_w["host_bytes_with_scales"] / (ms_step * 1e-3) / 1e9, 2)
            line["host_link"]["scale_bytes_note"] = ("weight_gbs counts the packed values, which cross the link every call; the weight scales "
                                                     "(K/16 bytes per row) are re-laid out once and then stay in HBM, so they are not per-call "
                                                     "traffic; the second figure counts them as the per-call definition of the config does")
        if on_dev and not moe:
            tf = rank0_w["flops"] / (kernel_ms * 1e-3) / 1e12
            line["roofline"] = {"bound": "tensor", "achieved": round(tf, 2), "peak": round(tensor_peak, 1), "unit": "TFLOP/s",
                                "frac": round(tf / tensor_peak, 4), "traffic": None,
                                "note": "weights resident in HBM: bound by the tensor pipe; peak = MEASURED_PEAKS.json bf16_tflops"
                                        " (x2 for 8-bit operands), of measured"}
            line.pop("host_link", None)
        if alt:
            line["copy_engine_staged"] = {
                "ms_per_step": round(alt_ms, 4), "value": round(flops / (alt_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
                "weight_gbs": round(host_bytes / (alt_ms * 1e-3) / 1e9, 2),
                "frac_of_measured_peak": round(host_bytes / (alt_ms * 1e-3) / 1e9 / link_peak_sum, 4),
                "e2e_ms_per_step": round(alt_e2e_ms, 3), "e2e_value": round(flops / (alt_e2e_ms * 1e-3) / 1e12, 3),
                "note": "same workload with set_weight_path('staged'): the copy engine moves the weights through a double buffer "
                        "in HBM and the grouped GEMM runs from there (an option of the operators; `--weights staged` makes it "
                        "the measured path); the headline numbers of this line are the in-kernel stream"}
        if args.weights == "staged":
            line["roofline"]["note"] = ("weights are moved by cudaMemcpyAsync (copy engine), not by the kernel: achieved is the "
                                        "weight bytes over the whole step, against the copy-engine rate measured in this run")
            line["roofline"]["traffic"] = None
            line["e2e"]["note"] = "weights are copied from pinned host memory by the copy engine inside both timings"
        if moe:
            line["metric"] = "MoE-layer TFLOPS (with host->GPU weight GB/s vs measured PCIe peak)"
            line["config"]["numa_node_of_weights"] = numa
            line["roofline"]["note"] += "; the step holds two grouped-GEMM launches plus helper kernels and two NCCL all-to-alls, achieved is over the whole step"
            if world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_moe_baseline(cfg, os.cpu_count() or 1)
        if cpu_sample is not None:
            v, sample, kind, cores = cpu_sample
            line["cpu_baseline"] = {"value": round(v, 4), "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample}
        line.update(extras)
        if "ep_layer" in extras:
            line["gpu_launches"] += extras["ep_layer"]["gemm_launches_per_step"] * (extras["ep_layer"]["steps"] + 4)
        print(json.dumps(line))
        if devmap is not None:
            try:
                devmap[1].unlink()
            except OSError:
                pass
    if world > 1:
        dist.destroy_process_group()
    return 0


def reference_arm(args, cfg, config):
    """--impl reference: the reference's CPU implementation of this path on the host cores (see cpu_reference_sample)."""
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    small = dict(cfg)
    # operands for a bounded sample only: the first experts of the workload, same shapes and routing
    small_experts = min(cfg["experts"], 8)
    w = None
    if device.type == "cuda":
        small["tokens"] = max(1, cfg["tokens"] * small_experts // cfg["experts"])
        small["experts"] = small_experts
        w = build_workload(small, 0, 1, device)
    else:
        print(json.dumps({"impl": "reference", "unavailable": "operands are generated on the GPU; no CUDA device visible"}))
        return 0
    threads = os.cpu_count() or 1
    vals = []
    for i in range(args.warmup + args.steps):
        v, sample, kind, cores = cpu_reference_sample(small, w, threads, max_experts=small_experts)
        if i >= args.warmup:
            vals.append(v)
    v = sum(vals) / len(vals)
    flops_step = sum(2.0 * s[2] * w["n"] * w["k"] for s in w["segs"][:small_experts])
    line = {"impl": "reference", "metric": "grouped-GEMM TFLOPS (with host->GPU weight GB/s vs measured PCIe peak)", "value": round(v, 4),
            "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(flops_step / (v * 1e12) * 1e3, 3), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": cfg["kind"], "data": "synthetic (seeded)", "config": config,
            "cpu_baseline": {"value": round(v, 4), "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": round(v, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
