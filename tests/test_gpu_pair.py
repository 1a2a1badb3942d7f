"""The CTA-pair kernel (tile configuration 8: two SMs share one 256 x 256 MMA, weights resident in device memory) against
the CPU oracle and against the single-CTA 256-column kernel, through the same operators as every other configuration."""
import random

import numpy as np
import pytest
import torch

import asymgemm_b200 as ag
from tests import helpers as H
from tests.test_gpu_parity import _check, _run_contiguous, _run_masked

pytestmark = pytest.mark.gpu

PAIR, WIDE = 8, 6
KINDS = ["bf16", "fp8", "int8"]


@pytest.fixture
def pair_tile():
    ag.set_tile_config(PAIR)
    yield PAIR
    ag.set_tile_config(0)


@pytest.mark.parametrize("kind", KINDS)
def test_pair_contiguous_ragged(kind, pair_tile):
    """Ragged rows, empty experts, a segment of many 256-row chunks, N and K tails (N = 392 leaves 136 columns in the
    second tile, so the second CTA's half of the weight tile is mostly past the end)."""
    rows = [300, 0, 1, 129, 0, 2300, 64, 513, 256, 257]
    n, k = 392, 640
    c = H.make_contiguous_case(kind, rows, n, k, seed=2, b_on_host=False)
    d = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
    _run_contiguous(c, d)
    ag.check_status()
    d_np = d.float().cpu().numpy()
    _check(kind, d_np, c["ref"], c["segments"])
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], c["m_total"])]).all()
    # the same bits as the single-CTA 256-column kernel: same products, same order of the K blocks
    ag.set_tile_config(WIDE)
    d2 = torch.full_like(d, float("nan"))
    _run_contiguous(c, d2)
    torch.cuda.synchronize()
    mask = torch.from_numpy(H.valid_row_mask(c["segments"], c["m_total"])).cuda()
    assert torch.equal(d[mask].view(torch.int16), d2[mask].view(torch.int16))


@pytest.mark.parametrize("kind", KINDS)
def test_pair_masked(kind, pair_tile):
    masked_m = [64, 0, 96, 384, 1, 200]
    m_max, n, k = 384, 256, 512
    c = H.make_masked_case(kind, masked_m, m_max, n, k, seed=4, b_on_host=False)
    d = torch.full((len(masked_m), m_max, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    _run_masked(c, d)
    ag.check_status()
    d_np = d.float().cpu().numpy().reshape(-1, n)
    _check(kind, d_np, c["ref"], c["segments"])
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], d_np.shape[0])]).all()


def test_pair_fp32_output_and_small_problem(pair_tile):
    """One segment shorter than a tile and fp32 output: the second CTA of the only pair computes rows that do not exist."""
    c = H.make_contiguous_case("bf16", [37], 256, 256, seed=9, b_on_host=False)
    d = torch.full((c["m_total"], 256), float("nan"), dtype=torch.float32, device="cuda")
    _run_contiguous(c, d)
    ag.check_status()
    _check("bf16", d.cpu().numpy(), c["ref"], c["segments"])


def test_pair_fused_silu_mul_equals_gemm_plus_activation(pair_tile):
    from asymgemm_b200 import ep, moe_ops
    rows = [300, 0, 1, 129, 2300, 64]
    inter, k = 384, 640
    c = H.make_contiguous_case("fp8", rows, 2 * inter, k, seed=71, b_on_host=False)
    d1 = torch.zeros((c["m_total"], 2 * inter), dtype=torch.bfloat16, device="cuda")
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (c["b"], c["sfb"]), d1, c["offsets"], c["experts"], c["list_size"])
    q_ref, s_ref = moe_ops.silu_mul_quant_fp8(d1, inter)
    b_il = ep.interleave_gate_up(c["b"].cuda())
    act = torch.full((c["m_total"], inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (b_il, c["sfb"]), act, c["offsets"], c["experts"], c["list_size"],
                                             epilogue="silu_mul")
    ag.check_status()
    mask = torch.from_numpy(H.valid_row_mask(c["segments"], c["m_total"])).cuda()
    assert torch.isnan(act[~mask]).all()
    q, s = moe_ops.quant_rows_fp8(act)
    assert torch.equal(s[mask], s_ref[mask]) and torch.equal(q.view(torch.uint8)[mask], q_ref.view(torch.uint8)[mask])


def test_pair_needs_device_resident_weights(pair_tile):
    c = H.make_contiguous_case("fp8", [130, 64], 256, 512, seed=63, b_on_host=True)
    d = torch.zeros((c["m_total"], 256), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="resident in device memory"):
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["offsets"], c["experts"], c["list_size"])


@pytest.mark.parametrize("seed", range(16))
def test_pair_random_case(seed):
    rng = random.Random(7000 + seed)
    kind = rng.choice(KINDS)
    masked = rng.random() < 0.4
    groups = rng.randint(1, 6)
    n = 8 * rng.randint(1, 90)
    k = {"bf16": 8, "fp8": 16, "int8": 128}[kind] * rng.randint(1, 1024 // {"bf16": 8, "fp8": 16, "int8": 128}[kind])
    counts = [rng.choice([0, rng.randint(1, 700), rng.randint(1, 700), rng.randint(1800, 2600)]) for _ in range(groups)]
    if sum(counts) == 0:
        counts[0] = 5
    ag.set_tile_config(PAIR)
    try:
        if masked:
            m_max = max(counts) + rng.randint(0, 40)
            c = H.make_masked_case(kind, counts, m_max, n, k, seed=seed, b_on_host=False)
            d = torch.full((groups, m_max, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            _run_masked(c, d)
            rows_total = groups * m_max
        else:
            c = H.make_contiguous_case(kind, counts, n, k, seed=seed, b_on_host=False)
            d = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
            _run_contiguous(c, d)
            rows_total = c["m_total"]
        ag.check_status()
    finally:
        ag.set_tile_config(0)
    d_np = d.float().cpu().numpy().reshape(rows_total, n)
    info = f"kind={kind} masked={masked} counts={counts} n={n} k={k}"
    try:
        _check(kind, d_np, c["ref"], c["segments"])
    except AssertionError as e:
        raise AssertionError(f"{e} [{info}]")
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], rows_total)]).all(), info
