"""Seeded random sweep: dtype x layout x weight residency x tile configuration x ragged shapes, each case checked
against the CPU oracle with the tolerances of tests/test_gpu_parity.py."""
import random

import numpy as np
import pytest
import torch

import asymgemm_b200 as ag
from tests import helpers as H
from tests.test_gpu_parity import _check, _run_contiguous, _run_masked

pytestmark = pytest.mark.gpu

K_STEP = {"bf16": 8, "fp8": 16, "int8": 128, "fp4": 32}
TILES = {"bf16": [0, 1, 2, 3, 4, 6, 7], "fp8": [0, 1, 2, 3, 4, 5, 6], "int8": [0, 1, 2, 3, 4, 5, 6], "fp4": [0, 1, 4, 7]}


def _random_case(rng: random.Random):
    kind = rng.choice(["bf16", "fp8", "int8", "fp4"])
    masked = rng.random() < 0.4
    groups = rng.randint(1, 6)
    n = 8 * rng.randint(1, 60)
    k = K_STEP[kind] * rng.randint(1, 1024 // K_STEP[kind])
    if kind == "fp8":
        k = max(k, 16)
    tile = rng.choice(TILES[kind])
    host = rng.random() < 0.6

    def rows():
        r = rng.random()
        if r < 0.15:
            return 0
        if r < 0.25:
            return rng.randint(1800, 2600)      # longer than one accumulator chunk in every configuration
        return rng.randint(1, 400)
    counts = [rows() for _ in range(groups)]
    if sum(counts) == 0:
        counts[0] = 5
    return kind, masked, counts, n, k, tile, host


@pytest.mark.parametrize("seed", range(36))
def test_random_case(seed):
    rng = random.Random(1000 + seed)
    kind, masked, counts, n, k, tile, host = _random_case(rng)
    ag.set_tile_config(tile)
    try:
        if masked:
            m_max = max(counts)
            m_max = -(-m_max // 128) * 128 if kind == "fp4" or rng.random() < 0.5 else m_max + rng.randint(0, 40)
            c = H.make_masked_case(kind, counts, m_max, n, k, seed=seed, b_on_host=host)
            d = torch.full((len(counts), m_max, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            _run_masked(c, d)
            rows_total = len(counts) * m_max
        else:
            c = H.make_contiguous_case(kind, counts, n, k, seed=seed, b_on_host=host)
            d = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
            _run_contiguous(c, d)
            rows_total = c["m_total"]
        ag.check_status()
    finally:
        ag.set_tile_config(0)
    d_np = d.float().cpu().numpy().reshape(rows_total, n)
    info = f"kind={kind} masked={masked} counts={counts} n={n} k={k} tile={tile} host={host}"
    try:
        _check(kind, d_np, c["ref"], c["segments"])
    except AssertionError as e:
        raise AssertionError(f"{e} [{info}]")
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], rows_total)]).all(), info


@pytest.mark.parametrize("seed", range(12))
def test_random_case_fp8_hardware_scaled(seed):
    """The same sweep for FP8 with UE8M0 scales applied by the tensor core (power-of-two scales from the quantisers)."""
    rng = random.Random(5000 + seed)
    masked = rng.random() < 0.4
    groups = rng.randint(1, 5)
    n, k = 8 * rng.randint(1, 60), 16 * rng.randint(1, 64)
    tile = rng.choice([0, 1, 4, 7])
    host = rng.random() < 0.6
    counts = [rng.choice([0, rng.randint(1, 400), rng.randint(1, 400), rng.randint(1800, 2600)]) for _ in range(groups)]
    if sum(counts) == 0:
        counts[0] = 17
    ag.set_tile_config(tile)
    try:
        if masked:
            m_max = -(-max(counts) // 128) * 128
            c = H.make_masked_case("fp8", counts, m_max, n, k, seed=seed, b_on_host=host, use_ue8m0=True)
            d = torch.full((groups, m_max, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            ag.m_grouped_fp8_asym_gemm_nt_masked((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["masked_m"], 64, ue8m0_scales=True)
            rows_total = groups * m_max
        else:
            c = H.make_contiguous_case("fp8", counts, n, k, seed=seed, b_on_host=host, use_ue8m0=True)
            d = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
            ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["offsets"], c["experts"],
                                                     c["list_size"], ue8m0_scales=True)
            rows_total = c["m_total"]
        ag.check_status()
    finally:
        ag.set_tile_config(0)
    d_np = d.float().cpu().numpy().reshape(rows_total, n)
    info = f"masked={masked} counts={counts} n={n} k={k} tile={tile} host={host}"
    try:
        _check("fp8", d_np, c["ref"], c["segments"])
    except AssertionError as e:
        raise AssertionError(f"{e} [{info}]")
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], rows_total)]).all(), info


@pytest.mark.parametrize("seed", range(16))
def test_random_case_staged_weights(seed):
    """The same sweep with host-resident weights moved by the copy engine in chunks of 1..G whole experts."""
    rng = random.Random(9000 + seed)
    kind, masked, counts, n, k, tile, _ = _random_case(rng)
    chunk = rng.randint(1, len(counts))
    ag.set_tile_config(tile)
    try:
        if masked:
            m_max = max(counts)
            m_max = -(-m_max // 128) * 128 if kind == "fp4" or rng.random() < 0.5 else m_max + rng.randint(0, 40)
            c = H.make_masked_case(kind, counts, m_max, n, k, seed=seed, b_on_host=True)
            d = torch.full((len(counts), m_max, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            rows_total = len(counts) * m_max
        else:
            c = H.make_contiguous_case(kind, counts, n, k, seed=seed, b_on_host=True)
            d = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
            rows_total = c["m_total"]
        ag.set_weight_path("staged", chunk_bytes=chunk * (c["b"].numel() * c["b"].element_size() // len(counts)),
                           slots=rng.randint(2, 8))
        (_run_masked if masked else _run_contiguous)(c, d)
        ag.check_status()
    finally:
        ag.set_tile_config(0)
        ag.set_weight_path("stream", chunk_bytes=128 << 20, slots=2)
    d_np = d.float().cpu().numpy().reshape(rows_total, n)
    info = f"kind={kind} masked={masked} counts={counts} n={n} k={k} tile={tile} chunk={chunk}"
    try:
        _check(kind, d_np, c["ref"], c["segments"])
    except AssertionError as e:
        raise AssertionError(f"{e} [{info}]")
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], rows_total)]).all(), info
