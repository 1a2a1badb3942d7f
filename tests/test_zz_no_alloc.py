"""The static-scratch FP8 entry point (for callers that cannot allocate device memory), called through the C ABI and
compared with the ordinary entry point on the same inputs, twice in a row: the second call finds the first call's
leftovers in the shared scratch array and must not be affected by them.

Collected last on purpose (file name), so a run that stops at the first failure has already run every other test.
The test itself allocates its tensors with torch before the calls; the entry point under test allocates nothing.
"""

import pytest
import torch

import asymgemm_b200 as ag
from asymgemm_b200 import _lib
from oracle import oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _desc(c, d, status, tile=0, num_sms=0):
    g = _lib.GemmDesc()
    g.layout = _lib.LAYOUT_CONTIGUOUS
    g.d_dtype = _lib.D_BF16
    g.a, g.sfa = c["a"].data_ptr(), c["sfa"].data_ptr()
    g.b, g.sfb = c["b"].data_ptr(), c["sfb_dev"].data_ptr()
    g.d = d.data_ptr()
    g.offsets, g.experts = c["offsets"].data_ptr(), c["experts"].data_ptr()
    g.max_segments = c["list_size"]
    g.m, g.n, g.k, g.num_groups = c["m_total"], c["n"], c["k"], c["g"]
    g.status = status.data_ptr()
    g.stream = torch.cuda.current_stream().cuda_stream
    g.tile_config = tile
    g.num_sms = num_sms
    return g


@pytest.mark.parametrize("tile", [0, 2])
def test_static_scratch_matches_regular_entry_point_twice(tile):
    lib = _lib.load()
    # segments longer than one accumulator chunk, so that the scratch replay path runs
    c = H.make_contiguous_case("fp8", [2100, 0, 130, 3000, 64], 384, 1024, seed=21)
    c["sfb_dev"] = c["sfb"].cuda()
    d_ref = torch.zeros((c["m_total"], c["n"]), dtype=torch.bfloat16, device="cuda")
    ag.m_grouped_fp8_asym_gemm_nt_contiguous((c["a"], c["sfa"]), (c["b"], c["sfb"]), d_ref, c["offsets"], c["experts"], c["list_size"])
    ag.check_status()
    mask = H.valid_row_mask(c["segments"], c["m_total"])
    assert oracle.max_rel(d_ref.float().cpu().numpy()[mask], c["ref"][mask]) <= 2e-2

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call in range(2):
        d = torch.full_like(d_ref, float("nan"))
        rc = lib.ag_m_grouped_fp8_gemm_nt_static_scratch(_desc(c, d, status, tile=tile))
        assert rc == _lib.AG_OK, _lib.last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        got = d.float().cpu().numpy()[mask]
        # tolerance of the FP8 parity tests; in practice the two entry points agree bit for bit
        assert oracle.max_rel(got, d_ref.float().cpu().numpy()[mask]) <= 2e-2, f"call {call}"
        assert oracle.max_rel(got, c["ref"][mask]) <= 2e-2, f"call {call}"


def _need(lib, desc):
    out = _lib.c_uint64(0)
    assert lib.ag_scratch_bytes_for(_lib.KIND_FP8, desc, out) == _lib.AG_OK, _lib.last_error()
    return int(out.value)


def test_static_scratch_with_device_resident_weights():
    """Weights already in HBM. By default long segments are cut into one-chunk items that never replay, so the call needs
    no scratch at all and K is not limited by the array (K = 7168 here, beyond what 148 CTAs x 128 rows would fit). With
    no_split = 1 the replay runs from the built-in array: a first call with other weights leaves its columns there, and the
    second call's result must not depend on them."""
    lib = _lib.load()
    c = H.make_contiguous_case("fp8", [700, 130, 0, 64], 256, 7168, seed=23, b_on_host=False)
    c["sfb_dev"] = c["sfb"]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mask = H.valid_row_mask(c["segments"], c["m_total"])
    d = torch.full((c["m_total"], c["n"]), float("nan"), dtype=torch.bfloat16, device="cuda")
    g = _desc(c, d, status)
    assert _need(lib, g) == 0
    assert lib.ag_m_grouped_fp8_gemm_nt_static_scratch(g) == _lib.AG_OK, _lib.last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert oracle.max_rel(d.float().cpu().numpy()[mask], c["ref"][mask]) <= 2e-2

    # replay from the array: whole segments per item, segments longer than one accumulator chunk
    small = H.make_contiguous_case("fp8", [2100, 0, 130, 3000, 64], 384, 1024, seed=24, b_on_host=False)
    small["sfb_dev"] = small["sfb"]
    other = H.make_contiguous_case("fp8", [2100, 0, 130, 3000, 64], 384, 1024, seed=25, b_on_host=False)   # same shapes, other numbers
    other["sfb_dev"] = other["sfb"]
    smask = H.valid_row_mask(small["segments"], small["m_total"])
    outs = []
    for case in (other, small):
        d = torch.full((case["m_total"], case["n"]), float("nan"), dtype=torch.bfloat16, device="cuda")
        g = _desc(case, d, status)
        g.no_split = 1
        need = _need(lib, g)
        assert 0 < need <= lib.ag_static_scratch_bytes()
        assert lib.ag_m_grouped_fp8_gemm_nt_static_scratch(g) == _lib.AG_OK, _lib.last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        outs.append(d)
    assert oracle.max_rel(outs[1].float().cpu().numpy()[smask], small["ref"][smask]) <= 2e-2
    # the same call through the ordinary entry point with a scratch buffer of the caller's: same bits
    d_ref = torch.full_like(outs[1], float("nan"))
    g = _desc(small, d_ref, status)
    g.no_split = 1
    need = _need(lib, g)
    buf = torch.empty(need + 1024, dtype=torch.uint8, device="cuda")
    off = (-buf.data_ptr()) % 1024
    g.scratch, g.scratch_bytes = buf.data_ptr() + off, need
    assert lib.ag_m_grouped_fp8_gemm_nt(g) == _lib.AG_OK, _lib.last_error()
    torch.cuda.synchronize()
    m = torch.from_numpy(smask).cuda()
    assert torch.equal(outs[1][m].view(torch.int16), d_ref[m].view(torch.int16))


def test_static_scratch_limit_is_the_launch_plans_own_figure():
    """Accept / reject right at the limit: the scratch a launch would use comes from ag_scratch_bytes_for (the arithmetic
    of the launch itself), and the entry point refuses exactly the descriptors whose figure exceeds the array."""
    lib = _lib.load()
    c = H.make_contiguous_case("fp8", [128, 128], 128, 512, seed=26)
    c["sfb_dev"] = c["sfb"].cuda()
    d = torch.zeros((c["m_total"], c["n"]), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    limit = int(lib.ag_static_scratch_bytes())
    # host-resident weights, default tile (64 rows per CTA, K padded to 256 bytes), N and segments large enough for a full grid.
    # Only the sizes are claimed; the oversized descriptor is refused before anything is launched, the one that fits is
    # only asked for its figure.
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    k_fit = limit // (sms * 64) // 256 * 256
    for k, fits in ((k_fit, True), (k_fit + 256, False)):
        g = _desc(c, d, status)
        g.k, g.n, g.max_segments = k, 1 << 14, 64
        need = _need(lib, g)
        assert need == sms * 64 * k
        assert (need <= limit - 1024) == fits or (need <= limit) == fits
        if not fits:
            assert lib.ag_m_grouped_fp8_gemm_nt_static_scratch(g) == _lib.AG_E_INVALID
            assert "built-in scratch" in _lib.last_error()
    # a lower CTA cap brings the same K back under the limit
    g = _desc(c, d, status, num_sms=sms // 2)
    g.k, g.n, g.max_segments = k_fit + 256, 1 << 14, 64
    assert _need(lib, g) == (sms // 2) * 64 * (k_fit + 256) <= limit
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def test_static_scratch_rejects_oversized_problems_and_missing_status():
    lib = _lib.load()
    c = H.make_contiguous_case("fp8", [128], 128, 512, seed=22)
    c["sfb_dev"] = c["sfb"].cuda()
    d = torch.zeros((c["m_total"], c["n"]), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = _desc(c, d, status)
    g.status = None
    assert lib.ag_m_grouped_fp8_gemm_nt_static_scratch(g) == _lib.AG_E_INVALID
    assert "status" in _lib.last_error()
    # claim a problem whose scratch need (CTAs x 64 rows x K bytes) exceeds the built-in array: rejected before any launch
    g = _desc(c, d, status)
    g.k, g.n, g.max_segments = 1 << 16, 1 << 14, 64
    assert lib.ag_m_grouped_fp8_gemm_nt_static_scratch(g) == _lib.AG_E_INVALID
    assert "built-in scratch" in _lib.last_error()
    assert lib.ag_static_scratch_bytes() == 80 << 20
    torch.cuda.synchronize()
    assert int(status.item()) == 0
