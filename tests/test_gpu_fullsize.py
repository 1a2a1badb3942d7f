"""Full-size runs (the benchmark configurations of bench.WORKLOADS) checked through size-independent properties: a column checksum of D against
A x (column sum of B), sampled blocks against a torch fp32 product on the device, and run-to-run bit identity."""
import pytest
import torch

import asymgemm_b200 as ag
import bench

pytestmark = pytest.mark.gpu


def _dequant_rows(w, start, rows):
    a = w["a"][start:start + rows].float()
    if w["kind"] in ("fp8", "int8"):
        a = a * w["sfa"][start:start + rows].repeat_interleave(128, 1)[:, : w["k"]]
    return a


def _dequant_b(w, e, n0, n1):
    b = w["b"][e, n0:n1].to(w["a"].device).float()
    if w["kind"] == "fp8":
        s = w["sfb"][e].repeat_interleave(128, 0).repeat_interleave(128, 1)[n0:n1, : w["k"]]
        b = b * s
    elif w["kind"] == "int8":
        b = b * w["sfb"][e, n0:n1].repeat_interleave(128, 1)
    return b


@pytest.mark.parametrize("name,experts", [("c3_fp8", 0), ("c2_bf16", 0), ("c2b_bf16", 0), ("c1_int8", 0)])
def test_full_size_properties(name, experts):
    """Every benchmark configuration of the plain grouped GEMM at its full size: all 256 experts of the FP8 case (7.5 GB of
    weights in pinned memory), both BF16 GEMMs (K = 2048 and the K = 768 one, whose K is not a multiple of the 512-byte
    stage) and the INT8 case."""
    cfg = dict(bench.WORKLOADS[name])
    if experts:
        cfg["tokens"] = cfg["tokens"] * experts // cfg["experts"]
        cfg["experts"] = experts
    w = bench.build_workload(cfg, 0, 1, torch.device("cuda", 0))
    w["d"].fill_(float("nan"))
    bench.run_op(w)
    ag.check_status()
    d1 = w["d"].clone()
    bench.run_op(w)
    ag.check_status()
    assert torch.equal(d1.view(torch.int16), w["d"].view(torch.int16)), "two runs differ"
    gen = torch.Generator().manual_seed(0)
    worst = 0.0
    for e, start, rows in w["segs"]:
        seg = w["d"][start:start + rows].float()
        assert torch.isfinite(seg).all()
        # checksum over all columns of a few experts, in fp64
        if e % 16 == 0:
            a = _dequant_rows(w, start, rows).double()
            colsum = _dequant_b(w, e, 0, w["n"]).double().sum(dim=0)
            want = a @ colsum
            got = seg.double().sum(dim=1)
            scale = (a.abs() @ _dequant_b(w, e, 0, w["n"]).double().abs().sum(dim=0)).clamp_min(1e-9)
            assert ((got - want).abs() / scale).max() < 2e-3
        # one random 128-column block per expert against torch fp32 on the device
        n0 = int(torch.randint(0, w["n"] // 128, (1,), generator=gen)) * 128
        ref = _dequant_rows(w, start, rows) @ _dequant_b(w, e, n0, n0 + 128).t()
        err = (seg[:, n0:n0 + 128] - ref).abs().max() / ref.abs().max().clamp_min(1e-9)
        worst = max(worst, float(err))
    tol = 1e-2 if w["kind"] == "bf16" else 2e-2
    assert worst <= tol, f"max-rel {worst:.3e} > {tol}"


def test_full_size_nvfp4_masked_properties():
    """C4: NVFP4 masked layout, 128 experts x 1024-row stride, K=4096, N=3072, weights and their scales in pinned host
    memory: sampled blocks against a torch fp32 product of the dequantised operands, untouched rows, run-to-run identity."""
    cfg = dict(bench.WORKLOADS["c4_fp4"])
    w = bench.build_masked_fp4(cfg, 0, 1, torch.device("cuda", 0))
    w["d"].fill_(float("nan"))
    bench.run_op(w)
    ag.check_status()
    d1 = w["d"].clone()
    bench.run_op(w)
    ag.check_status()
    assert torch.equal(d1.view(torch.int16), w["d"].view(torch.int16))
    gen = torch.Generator().manual_seed(1)
    worst = 0.0
    assert max(w["counts"]) == 1024 and min(w["counts"]) < 1024   # the routing law caps some experts and not others
    for e, rows in enumerate(w["counts"]):
        assert torch.isnan(w["d"][e, rows:]).all()
        if rows == 0 or e % 8:
            continue
        n0 = int(torch.randint(0, w["n"] // 128, (1,), generator=gen)) * 128
        a = bench._dequant_fp4(w["a"][e, :rows], w["sfa"][e, :rows])
        b = bench._dequant_fp4(w["b"][e, n0:n0 + 128].cuda(), w["sfb"][e, n0:n0 + 128].cuda())
        ref = a @ b.t()
        err = (w["d"][e, :rows, n0:n0 + 128].float() - ref).abs().max() / ref.abs().max().clamp_min(1e-9)
        worst = max(worst, float(err))
    assert worst <= 2e-2, f"max-rel {worst:.3e}"


def test_full_size_moe_down_projection_on_requantised_activations():
    """The down GEMM of the FP8 MoE layer at its full shape (K = 2048, N = 7168) on activations produced the way the layer
    produces them: a bf16 gate|up tensor through the fused SiLU*mul + 1x128 requantisation kernel. 32 experts with the
    layer's 2048 rows per expert on average (Zipf routing makes them ragged); sampled blocks against torch fp32 on the
    dequantised operands, run-to-run bit identity."""
    from asymgemm_b200 import moe_ops
    from asymgemm_b200.utils import build_contiguous_layout, per_block_cast_to_fp8
    dev = torch.device("cuda", 0)
    experts, inter, hidden = 32, 2048, 7168
    counts = bench.rows_per_expert(dict(experts=experts, tokens=8192, top_k=8, zipf=0.8), seed=3)
    offsets, expert_ids, list_size, m_total, segs = build_contiguous_layout(counts, device=dev)
    gen = torch.Generator(device=dev).manual_seed(4)
    gate_up = torch.zeros((m_total, 2 * inter), dtype=torch.bfloat16, device=dev)
    for _, start, rows in segs:
        gate_up[start:start + rows] = (torch.randn((rows, 2 * inter), device=dev, generator=gen) * 1.5).to(torch.bfloat16)
    a2, s2 = moe_ops.silu_mul_quant_fp8(gate_up, inter)
    w2 = torch.empty((experts, hidden, inter), dtype=torch.float8_e4m3fn).pin_memory()
    sf2 = torch.empty((experts, hidden // 128, inter // 128), dtype=torch.float32, device=dev)
    for e in range(experts):
        q, s = per_block_cast_to_fp8(torch.randn((hidden, inter), device=dev, generator=gen) * 0.02, use_ue8m0=False)
        w2[e].copy_(q, non_blocking=True)
        sf2[e] = s
    torch.cuda.synchronize()
    d = torch.full((m_total, hidden), float("nan"), dtype=torch.bfloat16, device=dev)
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((a2, s2), (w2, sf2), d, offsets, expert_ids, None)
    ag.check_status()
    d1 = d.clone()
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((a2, s2), (w2, sf2), d, offsets, expert_ids, None)
    ag.check_status()
    assert torch.equal(d1.view(torch.int16), d.view(torch.int16)), "two runs differ"
    cpu_gen = torch.Generator().manual_seed(0)
    worst = 0.0
    for e, start, rows in segs:
        seg = d[start:start + rows].float()
        assert torch.isfinite(seg).all()
        n0 = int(torch.randint(0, hidden // 128, (1,), generator=cpu_gen)) * 128
        a = a2[start:start + rows].float() * s2[start:start + rows].repeat_interleave(128, 1)
        b = w2[e, n0:n0 + 128].to(dev).float() * sf2[e, n0 // 128].repeat_interleave(128).unsqueeze(0)
        ref = a @ b.t()
        worst = max(worst, float((seg[:, n0:n0 + 128] - ref).abs().max() / ref.abs().max().clamp_min(1e-9)))
    assert worst <= 2e-2, f"max-rel {worst:.3e}"
