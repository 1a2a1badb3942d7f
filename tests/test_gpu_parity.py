"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded inputs.

Tolerances (stated by the task for this path): bf16 outputs within max-rel 1e-2 (BF16) / 2e-2 (FP8, NVFP4) of the
fp32 dequantised reference; INT8 int32 block sums bit-exact; plus the reference's own calc_diff thresholds
(tests/m_grouped/test_sm100_bf16_fp8_fp4_m_grouped.py: 1e-3 BF16, 2e-2 FP8/FP4; tests/test_sm90_int8.py:31: 0.05).
"""
import numpy as np
import pytest
import torch

import asymgemm_b200 as ag
from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu

TOL_MAXREL = {"bf16": 1e-2, "fp8": 2e-2, "int8": 2e-2, "fp4": 2e-2}
TOL_DIFF = {"bf16": 1e-3, "fp8": 2e-2, "int8": 1e-3, "fp4": 2e-2}


def _run_contiguous(c, d):
    kind = c["kind"]
    if kind == "bf16":
        ag.m_grouped_bf16_asym_gemm_nt_contiguous(c["a"], c["b"], d, c["offsets"], c["experts"], c["list_size"])
    elif kind == "fp8":
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["offsets"], c["experts"],
                                                 c["list_size"], recipe=(1, 128, 128))
    elif kind == "int8":
        ag.m_grouped_int8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["offsets"], c["experts"],
                                                  c["list_size"], raw_accumulators=c.get("raw"))
    elif kind == "fp4":
        ag.m_grouped_fp4_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["offsets"], c["experts"],
                                                 c["list_size"], recipe=(1, 1, 16), disable_ue8m0_cast=True)


def _run_masked(c, d):
    kind = c["kind"]
    exp_m = int(max(1, c["masked_m"].float().mean().item()))
    if kind == "bf16":
        ag.m_grouped_bf16_asym_gemm_nt_masked(c["a"], c["b"], d, c["masked_m"], exp_m)
    elif kind == "fp8":
        ag.m_grouped_fp8_asym_gemm_nt_masked((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["masked_m"], exp_m)
    elif kind == "int8":
        ag.m_grouped_int8_asym_gemm_nt_masked((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["masked_m"], exp_m,
                                              raw_accumulators=c.get("raw"))
    elif kind == "fp4":
        ag.m_grouped_fp4_asym_gemm_nt_masked((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["masked_m"], exp_m,
                                             recipe=(1, 1, 16), disable_ue8m0_cast=True)


def _check(kind, d_rows: np.ndarray, ref: np.ndarray, segments, poison_rows_untouched=None):
    mask = H.valid_row_mask(segments, ref.shape[0])
    got = d_rows[mask].astype(np.float32)
    exp = ref[mask]
    assert np.isfinite(got).all()
    mr = oracle.max_rel(got, exp)
    df = oracle.calc_diff(got, exp)
    assert mr <= TOL_MAXREL[kind], f"{kind}: max-rel {mr:.3e} > {TOL_MAXREL[kind]}"
    assert df <= TOL_DIFF[kind], f"{kind}: calc_diff {df:.3e} > {TOL_DIFF[kind]}"


KINDS = ["bf16", "fp8", "int8", "fp4"]


def _skip_unsupported(kind, tile):
    if kind == "fp4" and tile in (2, 3):
        pytest.skip("NVFP4 has 64- and 128-column tile configurations only")
    if tile == 5 and kind not in ("fp8", "int8"):
        pytest.skip("register accumulators exist for the software-scaled kinds only")
    if tile == 6 and kind == "fp4":
        pytest.skip("256-column items exist for bf16, fp8 and int8")
    if tile == 7 and kind in ("fp8", "int8"):
        pytest.skip("the deep activation ring exists for bf16 and the hardware-scaled kinds")


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("b_on_host", [True, False])
def test_contiguous_small(kind, b_on_host):
    """The reference's own smallest case: 2 groups x 128 rows, N=128, K=512 (tests/m_grouped/...:276-291)."""
    c = H.make_contiguous_case(kind, [128, 128], 128, 512, seed=1, b_on_host=b_on_host)
    d = torch.full((c["m_total"], 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    _run_contiguous(c, d)
    torch.cuda.synchronize()
    _check(kind, d.float().cpu().numpy(), c["ref"], c["segments"])


@pytest.fixture
def tile(request):
    """Forces one tile configuration for the test (0 = chosen from where B lives)."""
    ag.set_tile_config(request.param)
    yield request.param
    ag.set_tile_config(0)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("tile", [0, 1, 2, 3, 4, 5, 6, 7], indirect=True)
@pytest.mark.parametrize("b_on_host", [True, False])
def test_contiguous_ragged_multi_tile(kind, tile, b_on_host):
    """Ragged row counts, empty experts, segments longer than one accumulator chunk in every tile configuration
    (scratch replay), N and K tails; every tile configuration with B on the host and on the device."""
    _skip_unsupported(kind, tile)
    rows = [300, 0, 1, 129, 0, 2300, 64, 513]
    n, k = 392, 640
    c = H.make_contiguous_case(kind, rows, n, k, seed=2, b_on_host=b_on_host)
    d = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
    _run_contiguous(c, d)
    torch.cuda.synchronize()
    _check(kind, d.float().cpu().numpy(), c["ref"], c["segments"])


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("tile", [1, 2], indirect=True)
def test_contiguous_no_scratch_matches(kind, tile):
    """Without scratch, long segments re-read B instead; the result must be bit-identical."""
    _skip_unsupported(kind, tile)
    rows = [2500, 260]
    n, k = 256, 512
    c = H.make_contiguous_case(kind, rows, n, k, seed=3)
    d1 = torch.zeros((c["m_total"], n), dtype=torch.bfloat16, device="cuda")
    d2 = torch.zeros_like(d1)
    _run_contiguous(c, d1)
    ag.set_use_scratch(False)
    try:
        _run_contiguous(c, d2)
    finally:
        ag.set_use_scratch(True)
    torch.cuda.synchronize()
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    _check(kind, d1.float().cpu().numpy(), c["ref"], c["segments"])


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("tile", [0, 1, 3, 5, 6, 7], indirect=True)
def test_masked(kind, tile):
    """Masked layout incl. an empty group and a full group (reference case: tests/m_grouped/...:320-342)."""
    _skip_unsupported(kind, tile)
    masked_m = [64, 0, 96, 384, 1]
    m_max, n, k = 384, 256, 512
    c = H.make_masked_case(kind, masked_m, m_max, n, k, seed=4)
    d = torch.full((len(masked_m), m_max, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    _run_masked(c, d)
    torch.cuda.synchronize()
    d_np = d.float().cpu().numpy().reshape(-1, n)
    _check(kind, d_np, c["ref"], c["segments"])
    # rows past masked_m[g] are never written
    mask = H.valid_row_mask(c["segments"], d_np.shape[0])
    assert np.isnan(d_np[~mask]).all()


@pytest.mark.parametrize("b_on_host", [True, False])
def test_int8_block_sums_bit_exact(b_on_host):
    """INT8: the int32 sums per 128-wide K block must equal the oracle's exactly; fp32 output within tolerance.
    Host-resident B runs the TMEM-accumulating drain, device-resident B the register-accumulating one."""
    rows = [200, 128, 3, 640]
    n, k = 256, 1024
    c = H.make_contiguous_case("int8", rows, n, k, seed=5, b_on_host=b_on_host)
    raw = torch.zeros((k // 128, c["m_total"], n), dtype=torch.int32, device="cuda")
    c["raw"] = raw
    d = torch.zeros((c["m_total"], n), dtype=torch.float32, device="cuda")
    _run_contiguous(c, d)
    torch.cuda.synchronize()
    mask = H.valid_row_mask(c["segments"], c["m_total"])
    got = raw.cpu().numpy()[:, mask]
    exp = c["block_sums"][:, mask]
    assert np.array_equal(got, exp)
    # fp32 output: same products, same ascending-K fp32 summation as the oracle -> tight agreement
    got_d = d.cpu().numpy()[mask]
    assert oracle.max_rel(got_d, c["ref"][mask]) < 1e-5


@pytest.mark.parametrize("kind", KINDS)
def test_fp32_output(kind):
    c = H.make_contiguous_case(kind, [130, 257], 136, 384 if kind == "bf16" else 384, seed=6)
    d = torch.full((c["m_total"], 136), float("nan"), dtype=torch.float32, device="cuda")
    _run_contiguous(c, d)
    torch.cuda.synchronize()
    _check(kind, d.cpu().numpy(), c["ref"], c["segments"])


def test_fp8_ue8m0_scales_match_reference_mode():
    """Power-of-two scales (how the reference's SM100 tests quantise, tests/m_grouped/...:114,118)."""
    c = H.make_contiguous_case("fp8", [128, 256], 256, 1024, seed=7, use_ue8m0=True)
    d = torch.zeros((c["m_total"], 256), dtype=torch.bfloat16, device="cuda")
    _run_contiguous(c, d)
    torch.cuda.synchronize()
    _check("fp8", d.float().cpu().numpy(), c["ref"], c["segments"])


def test_empty_problem_and_errors():
    a = torch.zeros((0, 512), dtype=torch.bfloat16, device="cuda")
    b = H.pin(torch.zeros((2, 128, 512), dtype=torch.bfloat16))
    d = torch.zeros((0, 128), dtype=torch.bfloat16, device="cuda")
    off = torch.zeros(4, dtype=torch.int32, device="cuda")
    exp = torch.tensor([-1, -1, -1], dtype=torch.int32, device="cuda")
    ag.m_grouped_bf16_asym_gemm_nt_contiguous(a, b, d, off, exp, 1)  # m == 0: returns
    # unpinned host B must raise, not fault
    a = torch.zeros((128, 512), dtype=torch.bfloat16, device="cuda")
    d = torch.zeros((128, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        ag.m_grouped_bf16_asym_gemm_nt_contiguous(a, torch.zeros((2, 128, 512), dtype=torch.bfloat16), d, off, exp, 1)
    with pytest.raises(RuntimeError):  # shape mismatch
        ag.m_grouped_bf16_asym_gemm_nt_contiguous(a, b, torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda"), off, exp, 1)
    # all-sentinel expert list: nothing written
    d.fill_(7.0)
    ag.m_grouped_bf16_asym_gemm_nt_contiguous(a, b, d, off, exp, 3)
    torch.cuda.synchronize()
    assert (d == 7.0).all()


@pytest.mark.expects_status
def test_wait_limit_expires_with_status_and_context_stays_usable():
    """Failure detection without faulting the GPU: a wait that nothing satisfies gives up after its limit, the kernel
    reports a status word, the host raises, and the next GEMM on the same context is correct."""
    import time
    from asymgemm_b200 import _lib
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _lib.check(lib.ag_selftest_wait_limit(50, status.data_ptr(), torch.cuda.current_stream().cuda_stream))
    out = _lib.c_int32(0)
    rc = lib.ag_read_status(status.data_ptr(), torch.cuda.current_stream().cuda_stream, out)
    dt = time.perf_counter() - t0
    assert rc == _lib.AG_E_DEVICE and (out.value & 0xff) == 9 and "self test" in _lib.last_error()
    assert 0.04 <= dt < 2.0, dt
    c = H.make_contiguous_case("bf16", [128, 128], 128, 512, seed=9)
    d = torch.zeros((c["m_total"], 128), dtype=torch.bfloat16, device="cuda")
    _run_contiguous(c, d)
    ag.check_status()
    _check("bf16", d.float().cpu().numpy(), c["ref"], c["segments"])


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
def test_same_expert_in_two_segments_and_unsorted_experts(kind):
    """Segments need not be sorted by expert and one expert may own two segments (each re-reads its weights)."""
    c = H.make_contiguous_case(kind, [128, 256, 128], 256, 512, seed=31)
    # rewrite the table: expert 2 first, then expert 0 twice (rows of old expert 1 are given to expert 0's weights)
    offsets = torch.tensor([384, 512, 0, 128, 128, 384], dtype=torch.int32, device="cuda")
    experts = torch.tensor([2, 0, 0, -1], dtype=torch.int32, device="cuda")
    segments = [(2, 384, 512), (0, 0, 128), (0, 128, 384)]
    if kind == "bf16":
        ref = oracle.gemm_bf16(H.np_bits(c["a"]), H.np_bits(c["b"]), segments)
        d = torch.zeros((512, 256), dtype=torch.bfloat16, device="cuda")
        ag.m_grouped_bf16_asym_gemm_nt_contiguous(c["a"], c["b"], d, offsets, experts, 4)
    else:
        ref = oracle.gemm_fp8(H.np_bits(c["a"]), c["sfa"].cpu().numpy(), H.np_bits(c["b"]), c["sfb"].cpu().numpy(), segments)
        d = torch.zeros((512, 256), dtype=torch.bfloat16, device="cuda")
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, offsets, experts, 4)
    torch.cuda.synchronize()
    _check(kind, d.float().cpu().numpy(), ref, segments)


@pytest.mark.expects_status
def test_list_size_limits_the_segments_visited_and_bad_expert_is_reported():
    c = H.make_contiguous_case("bf16", [128, 128, 128], 128, 256, seed=32)
    d = torch.zeros((384, 128), dtype=torch.bfloat16, device="cuda")
    ag.m_grouped_bf16_asym_gemm_nt_contiguous(c["a"], c["b"], d, c["offsets"], c["experts"], 2)   # visit 2 entries only
    torch.cuda.synchronize()
    assert (d[256:] == 0).all() and d[:256].abs().sum() > 0
    # an expert id beyond the weight tensor is skipped and reported through the status word, nothing is read out of bounds
    experts = torch.tensor([0, 7, 2, -1], dtype=torch.int32, device="cuda")
    d.zero_()
    ag.m_grouped_bf16_asym_gemm_nt_contiguous(c["a"], c["b"], d, c["offsets"], experts, 4)
    with pytest.raises(RuntimeError, match="expert id"):
        ag.check_status()
    assert (d[128:256] == 0).all() and d[:128].abs().sum() > 0 and d[256:].abs().sum() > 0


@pytest.mark.parametrize("kind", ["bf16", "fp8", "int8"])
def test_masked_stride_not_a_multiple_of_128(kind):
    """M_max = 200: the last tile of a group overlaps the next group's rows in A but only valid rows are written."""
    masked_m = [200, 7, 0, 150]
    c = H.make_masked_case(kind, masked_m, 200, 128, 256, seed=33)
    d = torch.full((4, 200, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    _run_masked(c, d)
    torch.cuda.synchronize()
    d_np = d.float().cpu().numpy().reshape(-1, 128)
    _check(kind, d_np, c["ref"], c["segments"])
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], 800)]).all()


def test_masked_call_is_capturable_in_a_cuda_graph():
    """The masked layout has a grid that does not depend on routing: capture once, replay with new row counts
    (the property the reference calls CUDA-graph safe, csrc/jit_kernels/impls/sm100_fp8_asym_gemm_1d1d.hpp:284-292)."""
    c = H.make_masked_case("bf16", [128, 128, 128], 128, 128, 256, seed=34)
    d = torch.zeros((3, 128, 128), dtype=torch.bfloat16, device="cuda")
    ag.m_grouped_bf16_asym_gemm_nt_masked(c["a"], c["b"], d, c["masked_m"], 128)   # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ag.m_grouped_bf16_asym_gemm_nt_masked(c["a"], c["b"], d, c["masked_m"], 128)
    full = c["ref"].reshape(3, 128, 128)
    for counts in ([128, 0, 5], [1, 128, 64]):
        c["masked_m"].copy_(torch.tensor(counts, dtype=torch.int32))
        d.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        got = d.float().cpu().numpy()
        for g, r in enumerate(counts):
            if r:
                assert oracle.max_rel(got[g, :r], full[g, :r]) <= 1e-2
            assert np.isnan(got[g, r:]).all()
    ag.check_status()


@pytest.mark.parametrize("kind", KINDS)
def test_device_resident_split_matches_whole_segments(kind):
    """With B in device memory long segments are split into row chunks across CTAs; the result must not change."""
    rows = [1500, 0, 700, 40, 2600]
    c = H.make_contiguous_case(kind, rows, 384, 512, seed=41, b_on_host=False)
    d1 = torch.zeros((c["m_total"], 384), dtype=torch.bfloat16, device="cuda")
    d2 = torch.zeros_like(d1)
    _run_contiguous(c, d1)
    ag.set_split_segments(False)
    try:
        _run_contiguous(c, d2)
    finally:
        ag.set_split_segments(True)
    torch.cuda.synchronize()
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    _check(kind, d1.float().cpu().numpy(), c["ref"], c["segments"])


def test_two_streams_do_not_share_replay_scratch():
    """Two long-segment GEMMs issued back to back on different streams may overlap; each must get its own scratch."""
    cases = [H.make_contiguous_case("fp8", [2600, 1900], 256, 1024, seed=51 + i) for i in range(2)]
    outs = [torch.zeros((c["m_total"], 256), dtype=torch.bfloat16, device="cuda") for c in cases]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for _ in range(3):
        for c, d, st in zip(cases, outs, streams):
            with torch.cuda.stream(st):
                _run_contiguous(c, d)
    torch.cuda.synchronize()
    for c, d in zip(cases, outs):
        _check("fp8", d.float().cpu().numpy(), c["ref"], c["segments"])


@pytest.mark.parametrize("tile", [0, 1, 4, 7], indirect=True)
@pytest.mark.parametrize("b_on_host", [True, False])
def test_fp8_hardware_ue8m0_scaling_contiguous(tile, b_on_host):
    """FP8 with the block scales applied by the tensor core (UE8M0): exact for power-of-two scales, so it must agree with
    the oracle and, up to fp32 summation order, with the exact-fp32-scale path. Ragged rows, long segments, N and K tails."""
    rows = [300, 0, 1, 129, 2300, 64]
    n, k = 392, 640
    c = H.make_contiguous_case("fp8", rows, n, k, seed=61, b_on_host=b_on_host, use_ue8m0=True)
    d_hw = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
    d_sw = torch.full_like(d_hw, float("nan"))
    args = ((c["a"], c["sfa"]), (c["b"], c["sfb"]))
    ag.m_grouped_fp8_asym_gemm_nt_contiguous(*args, d_hw, c["offsets"], c["experts"], c["list_size"], ue8m0_scales=True)
    if tile == 7:   # the deep-ring configuration exists for the hardware-scaled kinds only: the exact path runs its default
        ag.set_tile_config(0)
    ag.m_grouped_fp8_asym_gemm_nt_contiguous(*args, d_sw, c["offsets"], c["experts"], c["list_size"], ue8m0_scales=False)
    torch.cuda.synchronize()
    _check("fp8", d_hw.float().cpu().numpy(), c["ref"], c["segments"])
    mask = H.valid_row_mask(c["segments"], c["m_total"])
    a, b = d_hw.float().cpu().numpy()[mask], d_sw.float().cpu().numpy()[mask]
    assert oracle.max_rel(a, b) <= 2 ** -7          # at most one bf16 ulp apart anywhere
    assert (a != b).mean() < 0.05


@pytest.mark.parametrize("tile", [0, 1, 2, 3, 4, 5, 6], indirect=True)
@pytest.mark.parametrize("b_on_host", [True, False])
def test_fp8_fused_silu_mul_epilogue_equals_gemm_plus_activation_kernel(tile, b_on_host):
    """The gate+up GEMM with the activation fused into its drain (weights interleaved gate / up in groups of 16) against the
    plain GEMM followed by the activation kernel: bf16(silu(gate) * up) must be the same bits, in every tile configuration,
    with ragged rows, a long segment and an empty expert; valid rows only are written."""
    from asymgemm_b200 import ep, moe_ops
    rows = [300, 0, 1, 129, 2300, 64]
    inter, k = 384, 640
    c = H.make_contiguous_case("fp8", rows, 2 * inter, k, seed=71, b_on_host=b_on_host)
    d1 = torch.zeros((c["m_total"], 2 * inter), dtype=torch.bfloat16, device="cuda")
    args = ((c["a"], c["sfa"]), (c["b"], c["sfb"]))
    ag.m_grouped_fp8_asym_gemm_nt_contiguous(*args, d1, c["offsets"], c["experts"], c["list_size"])
    q_ref, s_ref = moe_ops.silu_mul_quant_fp8(d1, inter)
    b_il = ep.interleave_gate_up(c["b"].cuda())
    b_il = b_il if not b_on_host else H.pin(b_il)
    act = torch.full((c["m_total"], inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (b_il, c["sfb"]), act, c["offsets"], c["experts"], c["list_size"],
                                             epilogue="silu_mul")
    torch.cuda.synchronize()
    mask = torch.from_numpy(H.valid_row_mask(c["segments"], c["m_total"])).cuda()
    assert torch.isnan(act[~mask]).all()
    q, s = moe_ops.quant_rows_fp8(act)
    assert torch.equal(s[mask], s_ref[mask]) and torch.equal(q.view(torch.uint8)[mask], q_ref.view(torch.uint8)[mask])
    # and against torch's formulation of the activation on the unfused output (exp implementations may differ in the last bit)
    g, u = d1[:, :inter].float(), d1[:, inter:].float()
    want = ((g / (1.0 + torch.exp(-g))) * u).to(torch.bfloat16)
    assert (act[mask].float() - want[mask].float()).abs().max() <= 2 ** -7 * want[mask].float().abs().max()
    assert (act[mask] != want[mask]).float().mean() < 1e-2
    with pytest.raises(RuntimeError, match="n % 256"):
        c2 = H.make_contiguous_case("fp8", [64], 128, 128, seed=72)
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((c2["a"], c2["sfa"]), (c2["b"], c2["sfb"]),
                                                 torch.zeros((c2["m_total"], 64), dtype=torch.bfloat16, device="cuda"),
                                                 c2["offsets"], c2["experts"], c2["list_size"], epilogue="silu_mul")


def test_nvfp4_coarser_scale_recipe_is_replicated():
    """Recipe (1, 1, 32): one E4M3 scale per 32 elements. The operator replicates every scale over its two 16-element
    groups (the reference does the same before its kernel, csrc/apis/gemm.hpp:271-275), so the result equals the
    (1, 1, 16) call on the replicated scale tensors bit for bit."""
    c = H.make_contiguous_case("fp4", [200, 0, 130], 256, 512, seed=81)
    sfa32 = c["sfa"].view(torch.uint8)[:, 0::2].contiguous().view(torch.float8_e4m3fn)            # keep every other scale
    sfb32 = H.pin(c["sfb"].view(torch.uint8)[:, :, 0::2].contiguous()).view(torch.float8_e4m3fn)
    sfa16 = sfa32.view(torch.uint8).repeat_interleave(2, dim=-1).contiguous().view(torch.float8_e4m3fn)
    sfb16 = H.pin(sfb32.view(torch.uint8).repeat_interleave(2, dim=-1).contiguous()).view(torch.float8_e4m3fn)
    d32 = torch.zeros((c["m_total"], 256), dtype=torch.bfloat16, device="cuda")
    d16 = torch.zeros_like(d32)
    ag.m_grouped_fp4_asym_gemm_nt_contiguous((c["a"], sfa32), (c["b"], sfb32), d32, c["offsets"], c["experts"], c["list_size"],
                                             recipe=(1, 1, 32), disable_ue8m0_cast=True)
    ag.m_grouped_fp4_asym_gemm_nt_contiguous((c["a"], sfa16), (c["b"], sfb16), d16, c["offsets"], c["experts"], c["list_size"],
                                             recipe=(1, 1, 16), disable_ue8m0_cast=True)
    torch.cuda.synchronize()
    assert torch.equal(d32.view(torch.int16), d16.view(torch.int16)) and d16.abs().sum() > 0
    ref = oracle.gemm_nvfp4(c["a"].cpu().numpy(), H.np_bits(sfa16), c["b"].numpy(), H.np_bits(sfb16), c["segments"])
    _check("fp4", d32.float().cpu().numpy(), ref, c["segments"])
    with pytest.raises(RuntimeError, match="Unknown SF transformation"):
        ag.m_grouped_fp4_asym_gemm_nt_contiguous((c["a"], sfa32), (c["b"], sfb32), d32, c["offsets"], c["experts"], c["list_size"],
                                                 recipe=(1, 1, 24))


def test_c_abi_error_surfaces_as_runtime_error_through_the_operator():
    """A descriptor the library refuses (a tile configuration that does not exist for the operand kind) comes back as the
    RuntimeError the reference API raises, with the library's message, and leaves the context usable."""
    c = H.make_contiguous_case("fp8", [130, 64], 128, 512, seed=63)
    d = torch.zeros((c["m_total"], 128), dtype=torch.bfloat16, device="cuda")
    args = ((c["a"], c["sfa"]), (c["b"], c["sfb"]))
    ag.set_tile_config(7)
    try:
        with pytest.raises(RuntimeError, match="tile_config 7 does not exist"):
            ag.m_grouped_fp8_asym_gemm_nt_contiguous(*args, d, c["offsets"], c["experts"], c["list_size"])
        ag.set_tile_config(5)
        with pytest.raises(RuntimeError, match="tile_config 5 does not exist"):
            ag.m_grouped_bf16_asym_gemm_nt_contiguous(c["a"].view(torch.uint8)[:, :256].contiguous().view(torch.bfloat16),
                                                      c["b"].view(torch.uint8)[:, :, :256].contiguous().pin_memory().view(torch.bfloat16),
                                                      d, c["offsets"], c["experts"], c["list_size"])
    finally:
        ag.set_tile_config(0)
    ag.m_grouped_fp8_asym_gemm_nt_contiguous(*args, d, c["offsets"], c["experts"], c["list_size"])
    torch.cuda.synchronize()
    _check("fp8", d.float().cpu().numpy(), c["ref"], c["segments"])


def test_fp8_hardware_ue8m0_scaling_masked_and_mode_switch():
    masked_m = [64, 0, 128, 384, 1]
    c = H.make_masked_case("fp8", masked_m, 384, 256, 512, seed=62, use_ue8m0=True)
    d = torch.full((5, 384, 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    ag.set_fp8_scale_mode("ue8m0")
    try:
        ag.m_grouped_fp8_asym_gemm_nt_masked((c["a"], c["sfa"]), (c["b"], c["sfb"]), d, c["masked_m"], 100)
    finally:
        ag.set_fp8_scale_mode("fp32")
    torch.cuda.synchronize()
    d_np = d.float().cpu().numpy().reshape(-1, 256)
    _check("fp8", d_np, c["ref"], c["segments"])
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], d_np.shape[0])]).all()
    # scales that are not powers of two lose their mantissa on this path, exactly as in the reference's SM100 kernel:
    # the result equals the oracle evaluated with floored scales
    c2 = H.make_contiguous_case("fp8", [128, 200], 128, 256, seed=63, use_ue8m0=False)
    d2 = torch.zeros((c2["m_total"], 128), dtype=torch.bfloat16, device="cuda")
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((c2["a"], c2["sfa"]), (c2["b"], c2["sfb"]), d2, c2["offsets"], c2["experts"],
                                             c2["list_size"], ue8m0_scales=True)
    torch.cuda.synchronize()
    floor2 = lambda t: np.exp2(np.floor(np.log2(t)))
    ref = oracle.gemm_fp8(H.np_bits(c2["a"]), floor2(c2["sfa"].cpu().numpy()), H.np_bits(c2["b"]), floor2(c2["sfb"].cpu().numpy()),
                          c2["segments"])
    _check("fp8", d2.float().cpu().numpy(), ref, c2["segments"])


@pytest.mark.parametrize("capacity", [0, 2, 5])
def test_hot_expert_cache_matches_plain_call(capacity):
    """Cached experts are served from HBM, the rest streamed; together they must give the plain call's result."""
    from asymgemm_b200.expert_cache import HotExpertCache
    rows = [300, 40, 0, 900, 129]
    c = H.make_contiguous_case("fp8", rows, 256, 512, seed=71)
    cache = HotExpertCache(c["b"], c["sfb"], capacity)
    assert cache.refresh(rows) == capacity
    if capacity == 2:
        assert sorted(cache.cached) == [0, 3]
        assert cache.refresh([0, 0, 5, 9, 0]) == 1 and sorted(cache.cached) == [2, 3]      # one expert replaced, one kept
        assert cache.refresh(rows) == 1
    d = torch.full((c["m_total"], 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    cache.fp8_gemm((c["a"], c["sfa"]), d, c["offsets"], c["experts"])
    torch.cuda.synchronize()
    _check("fp8", d.float().cpu().numpy(), c["ref"], c["segments"])
    cb = H.make_contiguous_case("bf16", rows, 256, 512, seed=72)
    cache_b = HotExpertCache(cb["b"], None, capacity)
    cache_b.refresh(rows)
    db = torch.full((cb["m_total"], 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    cache_b.bf16_gemm(cb["a"], db, cb["offsets"], cb["experts"])
    torch.cuda.synchronize()
    _check("bf16", db.float().cpu().numpy(), cb["ref"], cb["segments"])


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("layout", ["contiguous", "masked256", "masked192"])
def test_staged_weight_path_matches_in_kernel_stream(kind, layout):
    """`set_weight_path("staged")` makes the operators move host-resident weights with the copy engine, chunks of whole
    experts through a double buffer in HBM; results must equal the in-kernel stream's bit for bit, also on a second call,
    which reuses the buffers."""
    from asymgemm_b200 import api
    if kind == "fp4" and layout == "masked192":
        pytest.skip("the masked NVFP4 operator wants a stride that is a multiple of 128")
    if layout == "contiguous":
        c = H.make_contiguous_case(kind, [300, 40, 0, 900, 129], 256, 512, seed=81)
        shape, run = (c["m_total"], 256), _run_contiguous
    else:
        m_max = int(layout[6:])
        c = H.make_masked_case(kind, [min(200, m_max), 0, m_max, 17, 129], m_max, 256, 512, seed=82)
        shape, run = (5, m_max, 256), _run_masked
    plain = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    run(c, plain)
    group_bytes = c["b"].numel() * c["b"].element_size() // 5
    api._stager_cache.clear()
    ag.set_weight_path("staged", chunk_bytes=2 * group_bytes + 1, slots=2 if layout == "contiguous" else 3)   # chunks of 2, 2, 1 experts
    try:
        assert ag.get_weight_path() == "staged"
        for _ in range(2):
            d = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
            run(c, d)
            torch.cuda.synchronize()
            assert torch.equal(d.view(torch.int16), plain.view(torch.int16))
        assert len(api._stager_cache) == 1          # the staged path ran (and did not fall back to the in-kernel stream)
        if kind == "fp8" and layout != "masked192":
            hw_plain, hw = torch.zeros_like(plain), torch.zeros_like(plain)
            args = ((c["a"], c["sfa"]), (c["b"], c["sfb"]))
            ag.set_weight_path("stream")
            if layout == "contiguous":
                ag.m_grouped_fp8_asym_gemm_nt_contiguous(*args, hw_plain, c["offsets"], c["experts"], None, ue8m0_scales=True)
                ag.set_weight_path("staged")
                ag.m_grouped_fp8_asym_gemm_nt_contiguous(*args, hw, c["offsets"], c["experts"], None, ue8m0_scales=True)
            else:
                ag.m_grouped_fp8_asym_gemm_nt_masked(*args, hw_plain, c["masked_m"], 100, ue8m0_scales=True)
                ag.set_weight_path("staged")
                ag.m_grouped_fp8_asym_gemm_nt_masked(*args, hw, c["masked_m"], 100, ue8m0_scales=True)
            torch.cuda.synchronize()
            assert torch.equal(hw.view(torch.int16), hw_plain.view(torch.int16))
    finally:
        ag.set_weight_path("stream", chunk_bytes=128 << 20, slots=2)
    _check(kind, plain.float().cpu().numpy().reshape(-1, 256), c["ref"], c["segments"])


def test_prepare_weights_registers_pageable_memory_in_place():
    """Weights in an ordinary CPU tensor are refused; after `prepare_weights` the same memory serves as B and gives the
    result of a pinned copy; `release_weights` undoes it and refuses memory it did not register."""
    c = H.make_contiguous_case("fp8", [200, 0, 129], 256, 512, seed=91)
    plain = torch.zeros((c["m_total"], 256), dtype=torch.bfloat16, device="cuda")
    _run_contiguous(c, plain)
    pageable = torch.empty(c["b"].shape, dtype=torch.uint8).copy_(c["b"].view(torch.uint8)).view(torch.float8_e4m3fn)
    assert not pageable.is_pinned()
    d = torch.zeros_like(plain)
    with pytest.raises(RuntimeError, match="pinned"):
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (pageable, c["sfb"]), d, c["offsets"], c["experts"], None)
    assert ag.prepare_weights(pageable) is pageable and pageable.is_pinned()
    try:
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (pageable, c["sfb"]), d, c["offsets"], c["experts"], None)
        torch.cuda.synchronize()
        assert torch.equal(d.view(torch.int16), plain.view(torch.int16))
    finally:
        ag.release_weights(pageable)
    assert not pageable.is_pinned()
    with pytest.raises(RuntimeError, match="not registered"):
        ag.release_weights(pageable)
    assert ag.prepare_weights(c["b"]) is c["b"]          # already pinned: nothing to do, nothing to release


def test_prefetch_of_staged_weights_is_used_or_discarded_correctly():
    """`prefetch_weights` copies the first chunks early; the next staged call on the same weights must give the plain
    result, and so must a call on other weights that finds a prefetch it cannot use -- for a double buffer and for rings."""
    c1 = H.make_contiguous_case("fp8", [300, 40, 0, 900, 129], 256, 512, seed=95)
    c2 = H.make_contiguous_case("fp8", [10, 700, 64, 0, 200], 256, 512, seed=96)
    want = []
    for c in (c1, c2):
        d = torch.zeros((c["m_total"], 256), dtype=torch.bfloat16, device="cuda")
        _run_contiguous(c, d)
        want.append(d)
    group_bytes = c1["b"].numel() // 5

    def check_all():
        for first, second in ((c1, c1), (c1, c2), (c2, c1)):
            ag.prefetch_weights(first["b"])
            ag.prefetch_weights(first["b"])           # twice in a row: the second simply copies again
            for c in (second, first):
                d = torch.zeros((c["m_total"], 256), dtype=torch.bfloat16, device="cuda")
                _run_contiguous(c, d)
                torch.cuda.synchronize()
                assert torch.equal(d.view(torch.int16), want[0 if c is c1 else 1].view(torch.int16))

    try:
        for slots, per_chunk in ((2, 2), (4, 1), (8, 1)):       # 3, 5 and 5 chunks; the ring holds 2, 4 and all of them
            ag.set_weight_path("staged", chunk_bytes=per_chunk * group_bytes, slots=slots)
            check_all()
            ag.set_weight_path("stream", chunk_bytes=per_chunk * group_bytes, slots=slots)
            check_all()                 # prefetching is a no-op on the in-kernel path
    finally:
        ag.set_weight_path("stream", chunk_bytes=128 << 20, slots=2)
    ag.check_status()


@pytest.mark.parametrize("kind", ["fp8", "bf16", "fp4"])
@pytest.mark.parametrize("b_on_host", [True, False])
def test_segment_list_longer_than_the_shared_memory_table(kind, b_on_host):
    """1100 segments (more than the 1024 whose entries a CTA keeps in shared memory; NVFP4 keeps 256): every role then walks
    the segment list in device memory instead of reading the per-CTA item table, and must enumerate the same items."""
    rng = np.random.default_rng(5)
    rows = [int(r) for r in rng.choice([0, 1, 3, 17, 128, 130], size=1100)]
    n, k = 64, 128
    c = H.make_contiguous_case(kind, rows, n, k, seed=91, b_on_host=b_on_host)
    d = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
    _run_contiguous(c, d)
    ag.check_status()
    d_np = d.float().cpu().numpy()
    _check(kind, d_np, c["ref"], c["segments"])
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], c["m_total"])]).all()


@pytest.mark.parametrize("kind", ["fp8", "bf16", "fp4"])
@pytest.mark.parametrize("b_on_host", [True, False])
def test_more_items_per_cta_than_the_shared_memory_table(kind, b_on_host):
    """One CTA for 600 to 2000 items, depending on the tile (the table holds 512 per CTA; NVFP4 128): the first items come from the table, the rest from
    the walk, and the two must join without a gap or a repeat."""
    rows = [200, 0, 1, 129, 300, 64, 513, 130] * 8
    n, k = 2048, 128
    c = H.make_contiguous_case(kind, rows, n, k, seed=92, b_on_host=b_on_host)
    d = torch.full((c["m_total"], n), float("nan"), dtype=torch.bfloat16, device="cuda")
    with ag.launch_sm_cap(1):
        _run_contiguous(c, d)
    ag.check_status()
    d_np = d.float().cpu().numpy()
    _check(kind, d_np, c["ref"], c["segments"])
    assert np.isnan(d_np[~H.valid_row_mask(c["segments"], c["m_total"])]).all()


def test_two_issuers_keep_the_tensor_core_busy_where_one_does_not():
    """The issue-rate probe behind the kernels' two MMA-issuing threads: with the issuer's own instruction sequence and no
    loads, two threads reach the tensor core's rate for 256-column MMAs (512 cycles per step of four); one thread needs
    more cycles per step than two."""
    from asymgemm_b200.testing import probes
    one, two = probes.mma_issue_cycles(1, 256), probes.mma_issue_cycles(2, 256)
    assert 500.0 <= two <= 540.0, (one, two)
    assert one >= two - 1.0, (one, two)
    with pytest.raises(RuntimeError, match="issuers must be 1 or 2"):
        probes.mma_issue_cycles(3)


@pytest.mark.parametrize("b_on_host", [True, False])
@pytest.mark.parametrize("fused", [False, True])
def test_fp8_result_scatter_equals_plain_gemm_plus_row_move(b_on_host, fused):
    """`scatter=(meta, bases)`: every result row goes to the buffer and row its entry names instead of d[r] (what the
    expert-parallel layer's down GEMM uses to send results home). Two destination buffers, a random permutation of the
    valid rows over them, negative entries dropped: the bits of the plain GEMM, moved; nothing else is written."""
    from asymgemm_b200 import ep
    rows = [300, 0, 1, 129, 2300, 64]
    n, k = (768, 640) if fused else (392, 640)
    c = H.make_contiguous_case("fp8", rows, n, k, seed=95, b_on_host=b_on_host)
    b = c["b"]
    if fused:
        b = ep.interleave_gate_up(b.cuda())
        b = H.pin(b) if b_on_host else b
    cols = n // 2 if fused else n
    kw = dict(epilogue="silu_mul") if fused else {}
    d = torch.zeros((c["m_total"], cols), dtype=torch.bfloat16, device="cuda")
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (b, c["sfb"]), d, c["offsets"], c["experts"], c["list_size"], **kw)
    mask = torch.from_numpy(H.valid_row_mask(c["segments"], c["m_total"])).cuda()
    valid = torch.nonzero(mask).flatten()
    gen = torch.Generator().manual_seed(7)
    perm = torch.randperm(valid.numel(), generator=gen).cuda()
    dropped = perm[:37]                                     # these rows get a negative entry: not stored anywhere
    bufs = [torch.full((valid.numel(), cols), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    meta = torch.full((c["m_total"],), -1, dtype=torch.int64, device="cuda")
    which = (torch.arange(valid.numel(), device="cuda") % 2).to(torch.int64)
    meta[valid[perm]] = (which << 32) | torch.arange(valid.numel(), device="cuda", dtype=torch.int64)
    meta[valid[dropped]] = -1
    bases = torch.tensor([t.data_ptr() for t in bufs], dtype=torch.int64, device="cuda")
    untouched = torch.full_like(d, float("nan"))
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (b, c["sfb"]), untouched, c["offsets"], c["experts"], c["list_size"],
                                             scatter=(meta, bases), **kw)
    ag.check_status()
    assert torch.isnan(untouched).all()                      # d itself is not written
    src = valid[perm]
    for i, buf in enumerate(bufs):
        sel = (which == i)
        sel[:37] = False
        slots = torch.nonzero(sel).flatten()
        assert torch.equal(buf[slots].view(torch.int16), d[src[slots]].view(torch.int16))
        rest = torch.ones(valid.numel(), dtype=torch.bool, device="cuda")
        rest[slots] = False
        assert torch.isnan(buf[rest]).all()
    with pytest.raises(RuntimeError, match="scatter"):
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (b, c["sfb"]), untouched, c["offsets"], c["experts"], c["list_size"],
                                                 scatter=(meta.int(), bases), **kw)


def test_operand_feed_probe_runs_and_loads_cost_cycles():
    """The operand-feed probe (the kernels' rings with real TMA loads and nothing else): without loads it runs close to
    the tensor core's 1024 cycles per K atom; with both operands loaded it cannot be faster than without."""
    from asymgemm_b200.testing import probes
    none, both = probes.operand_feed_cycles(False, False), probes.operand_feed_cycles(True, True)
    assert 1000.0 <= none <= 1250.0, (none, both)
    assert both >= none - 5.0 and both < 4000.0, (none, both)
