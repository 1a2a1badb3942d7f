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


@pytest.mark.parametrize("name,experts", [("c3_fp8", 64), ("c2_bf16", 0), ("c1_int8", 0)])
def test_full_size_properties(name, experts):
    cfg = dict(bench.WORKLOADS[name])
    if experts:  # the 256-expert FP8 case keeps its shapes and routing law but a quarter of the experts (1.9 GB of weights)
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
