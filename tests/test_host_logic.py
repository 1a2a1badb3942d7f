"""Host-side logic without a GPU: quantisers against the reference's (golden fixtures), layout builder, argument checks,
and the C ABI's exported symbols."""
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import asymgemm_b200 as ag
from asymgemm_b200 import _lib
from asymgemm_b200.utils import (build_contiguous_layout, get_tma_aligned_size, per_block_cast_to_fp8, per_channel_cast_to_int8,
                                 per_token_cast_to_fp8, per_token_cast_to_int8, per_token_cast_to_nvfp4_e4m3)
from oracle import oracle

ROOT = Path(__file__).resolve().parents[1]
GOLD = ROOT / "tests" / "golden"


def _inputs():
    g = np.load(GOLD / "inputs.npz")
    return torch.from_numpy(g["x"].astype(np.float32)), torch.from_numpy(g["w"].astype(np.float32))


@pytest.mark.parametrize("ue", [False, True])
def test_fp8_quantisers_match_reference(ue):
    x, w = _inputs()
    g = np.load(GOLD / ("fp8_ue8m0_contiguous.npz" if ue else "fp8_fp32scale_contiguous.npz"))
    q, s = per_token_cast_to_fp8(x, ue)
    assert np.array_equal(q.view(torch.uint8).numpy(), g["a"]) and np.array_equal(s.numpy(), g["sfa"])
    for i in range(w.shape[0]):
        q, s = per_block_cast_to_fp8(w[i], ue)
        assert np.array_equal(q.view(torch.uint8).numpy(), g["b"][i]) and np.array_equal(s.numpy(), g["sfb"][i])


def test_int8_quantisers_match_reference():
    x, w = _inputs()
    g = np.load(GOLD / "int8_contiguous.npz")
    q, s = per_token_cast_to_int8(x)
    assert np.array_equal(q.numpy(), g["a"]) and np.array_equal(s.numpy(), g["sfa"])
    q, s = per_channel_cast_to_int8(w[3])
    assert np.array_equal(q.numpy(), g["b"][3]) and np.array_equal(s.numpy(), g["sfb"][3])


def test_nvfp4_quantiser_matches_reference():
    x, _ = _inputs()
    g = np.load(GOLD / "fp4_contiguous.npz")
    q, s = per_token_cast_to_nvfp4_e4m3(x)
    assert np.array_equal(q.numpy(), g["a_math"]) and np.array_equal(s.view(torch.uint8).numpy(), g["sfa_math"])
    # dequantising it reproduces x to within half an E2M1 step of the block scale
    deq = oracle.dequant_nvfp4(q.numpy(), s.view(torch.uint8).numpy())
    scale = np.repeat(oracle.decode_e4m3(s.view(torch.uint8).numpy()), 16, axis=1)
    assert (np.abs(deq - x.numpy()) <= scale * 1.0 + 1e-6).all()


def test_remaining_quantisers_match_reference():
    """per_channel_cast_to_fp8, per_custom_dims_cast_to_fp8, per_token_cast_to_fp4 and transpose_packed_fp4 against the
    reference's outputs on the shared inputs (fixture written by tests/golden/make_golden.py from the reference's functions)."""
    from asymgemm_b200.utils import per_channel_cast_to_fp8, per_custom_dims_cast_to_fp8, per_token_cast_to_fp4, transpose_packed_fp4
    x, w = _inputs()
    xs = x[:256]
    g = np.load(GOLD / "quantisers_extra.npz")
    for tag, ue in (("f32", False), ("ue8m0", True)):
        q, s = per_channel_cast_to_fp8(xs, ue)
        assert np.array_equal(q.view(torch.uint8).numpy(), g[f"chan_q_{tag}"]) and np.array_equal(s.numpy(), g[f"chan_s_{tag}"])
        q, s = per_custom_dims_cast_to_fp8(w, (0, 2), ue)
        assert np.array_equal(q.view(torch.uint8).numpy(), g[f"dims_q_{tag}"]) and np.array_equal(s.numpy(), g[f"dims_s_{tag}"])
        q, s = per_token_cast_to_fp4(xs, ue, 128)
        assert np.array_equal(q.numpy(), g[f"fp4_q_{tag}"]) and np.array_equal(s.numpy(), g[f"fp4_s_{tag}"])
    packed, _ = per_token_cast_to_fp4(xs, False, 128)
    t = transpose_packed_fp4(packed)
    assert np.array_equal(t.numpy(), g["fp4_transposed"])
    assert torch.equal(transpose_packed_fp4(t), packed)          # an involution on even-sized matrices


def test_contiguous_layout_builder():
    off, exp, list_size, total, segs = build_contiguous_layout([130, 0, 1, 256], device="cpu")
    assert off.tolist() == [0, 256, 256, 384, 384, 640]
    assert exp.tolist() == [0, 2, 3, -1] and list_size == 4 and total == 640
    assert segs == [(0, 0, 130), (2, 256, 1), (3, 384, 256)]
    assert oracle.contiguous_segments(off.tolist(), exp.tolist()) == [(0, 0, 256), (2, 256, 384), (3, 384, 640)]
    assert oracle.contiguous_segments(off.tolist(), exp.tolist(), max_segments=1) == [(0, 0, 256)]
    assert ag.get_mk_alignment_for_contiguous_layout() == 128
    assert get_tma_aligned_size(5, 4) == 8 and get_tma_aligned_size(16, 1) == 16


def test_argument_checks_raise_runtime_error_on_cpu_tensors():
    a = torch.zeros((128, 512), dtype=torch.bfloat16)
    b = torch.zeros((2, 128, 512), dtype=torch.bfloat16)
    d = torch.zeros((128, 128), dtype=torch.bfloat16)
    off = torch.zeros(4, dtype=torch.int32)
    exp = torch.zeros(3, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        ag.m_grouped_bf16_asym_gemm_nt_contiguous(a, b, d, off, exp, 1)  # nothing is on the GPU
    with pytest.raises(RuntimeError):
        ag.m_grouped_bf16_asym_gemm_nt_contiguous(a, b, d, off, exp, 1, transpose_b=True)
    with pytest.raises(RuntimeError):
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((a, a), (b, b), d, off, exp, 1, recipe=(1, 1, 128))


def test_shared_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "asymgemm_b200.h").read_text()
    declared = set(re.findall(r"\b(ag_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = _lib.load()
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, f"declared but not exported: {missing}"
    assert declared == set(_lib.EXPORTS)
    assert lib.ag_get_mk_alignment_for_contiguous_layout() == 128
    assert b"sm_100a" in lib.ag_version()


def test_c_abi_rejects_bad_descriptors_without_a_gpu():
    lib = _lib.load()
    desc = _lib.GemmDesc()
    desc.layout = 7
    assert lib.ag_m_grouped_bf16_gemm_nt(desc) == _lib.AG_E_INVALID
    assert "layout" in _lib.last_error()
    desc.layout = 0
    desc.n, desc.k, desc.num_groups, desc.m = 128, 512, 2, 0
    assert lib.ag_m_grouped_bf16_gemm_nt(desc) == _lib.AG_OK  # m == 0: nothing to do
    assert lib.ag_fp4_sf_blocked_bytes(2, 130, 16) == 2 * 2 * 32 * 512  # 2 groups x 2 row tiles x K runs padded to 32


def test_helper_kernels_reject_misaligned_pointers_without_launching():
    """The row quantisers and the top-k combine use vector loads and stores; a pointer that is not aligned for them is
    refused on the host (a launch would fault the context). No GPU is needed: the checks run before any CUDA call."""
    lib = _lib.load()
    base = 0x7F0000000000   # never dereferenced
    ok = base
    assert lib.ag_quant_rows_fp8(ok + 2, ok, ok, 4, 256, 0, None) == _lib.AG_E_INVALID      # x only 2-byte aligned
    assert "aligned" in _lib.last_error()
    assert lib.ag_quant_rows_fp8(ok, ok + 2, ok, 4, 256, 0, None) == _lib.AG_E_INVALID      # q only 2-byte aligned
    assert lib.ag_silu_mul_quant_fp8(ok + 4, ok, ok, 4, 256, 0, None) == _lib.AG_E_INVALID  # gate_up only 4-byte aligned
    assert lib.ag_silu_mul_quant_fp8(ok, ok + 1, ok, 4, 256, 0, None) == _lib.AG_E_INVALID
    assert lib.ag_combine_topk(ok + 8, ok, ok, ok, 4, 2, 256, None) == _lib.AG_E_INVALID    # rows only 8-byte aligned
    assert lib.ag_combine_topk(ok, ok, ok, ok + 8, 4, 2, 256, None) == _lib.AG_E_INVALID    # y only 8-byte aligned
    assert lib.ag_combine_topk_f32(ok + 4, ok, ok, ok, 4, 2, 256, None) == _lib.AG_E_INVALID
    assert lib.ag_combine_topk_f32(ok, ok, ok, ok + 4, 4, 2, 256, None) == _lib.AG_E_INVALID
    assert lib.ag_move_rows(ok + 8, ok, None, None, 4, 256, None) == _lib.AG_E_INVALID
    assert lib.ag_quant_rows_int8(ok + 1, ok, ok, 4, 256, None) == _lib.AG_E_INVALID
    assert lib.ag_silu_mul_quant_int8(ok + 2, ok, ok, 4, 256, None) == _lib.AG_E_INVALID
    # zero rows with aligned pointers: accepted, nothing launched
    assert lib.ag_quant_rows_fp8(ok, ok, ok, 0, 256, 0, None) == _lib.AG_OK


def test_weight_scale_cache_is_tied_to_the_tensor_object():
    """A new tensor that reuses a freed tensor's address must not be served the old tensor's cached copy."""
    from asymgemm_b200 import api

    cache: dict = {}
    dev = torch.device("cpu")
    dev = type("D", (), {"index": 0})()
    t1 = torch.zeros(8)
    api._cache_put(cache, t1, dev, "copy-of-t1")
    assert api._cache_get(cache, t1, dev) == "copy-of-t1"
    t1.add_(1)                                   # in-place change bumps the version counter
    assert api._cache_get(cache, t1, dev) is None
    api._cache_put(cache, t1, dev, "copy-of-t1-v2")
    t2 = torch.zeros(8)
    assert api._cache_get(cache, t2, dev) is None
    key = (id(t1), 0)
    del t1                                       # entry stays but can never match another object
    fake = torch.ones(8)
    cache[(id(fake), 0)] = cache.pop(key)
    assert api._cache_get(cache, fake, dev) is None


def test_scale_layout_helpers_keep_the_reference_shapes_and_strides():
    sf = torch.rand(2, 70, 6) + 0.5
    out = ag.get_mn_major_tma_aligned_tensor(sf)
    assert out.shape == sf.shape and out.stride() == (6 * 72, 1, 72) and torch.equal(out, sf)
    pw = torch.exp2(torch.randint(-8, 8, (70, 6)).float())
    packed = ag.get_mn_major_tma_aligned_packed_ue8m0_tensor(pw)
    assert packed.shape == (70, 2) and packed.dtype == torch.int32 and packed.stride() == (1, 72)
    # byte j of word w is the biased exponent of column 4*w + j; columns past k are zero
    exp = (torch.log2(pw) + 127).to(torch.int32)
    assert torch.equal(packed[:, 0] & 0xFF, exp[:, 0]) and torch.equal((packed[:, 1] >> 8) & 0xFF, exp[:, 5])
    assert ((packed[:, 1] >> 16) == 0).all()
    # weight scales: 128-row blocks are broadcast to rows first
    sfb = torch.exp2(torch.randint(-4, 4, (3, 2, 4)).float())
    t = ag.transform_sf_into_required_layout(sfb, 200, 512, (1, 128, 128), num_groups=3, is_sfa=False)
    assert t.shape == (3, 200, 1)
    assert torch.equal(t[1, 130, 0] & 0xFF, (torch.log2(sfb[1, 1, 0]) + 127).to(torch.int32))
    with pytest.raises(RuntimeError):
        ag.transform_sf_into_required_layout(sfb, 200, 512, (1, 64, 64))
    ag.set_tc_util(80); ag.set_compile_mode(1)
    assert ag.get_tc_util() == 80 and ag.get_compile_mode() == 1


def test_proportional_expert_ranges():
    from asymgemm_b200.ep import proportional_expert_ranges as pr
    assert pr([50.0, 51.0, 49.5, 50.2], 256) == [(0, 64), (64, 128), (128, 192), (192, 256)]      # within tolerance: even
    r = pr([23.0] * 4 + [35.0] * 4, 256)
    sizes = [hi - lo for lo, hi in r]
    assert sum(sizes) == 256 and r[0][0] == 0 and r[-1][1] == 256 and all(r[i][1] == r[i + 1][0] for i in range(7))
    assert all(25 <= n <= 26 for n in sizes[:4]) and all(38 <= n <= 39 for n in sizes[4:])
    # finishing time (experts / rate) is balanced to within one expert
    t = [n / rate for n, rate in zip(sizes, [23.0] * 4 + [35.0] * 4)]
    assert max(t) - min(t) <= 1 / 23.0 + 1e-9
    assert [hi - lo for lo, hi in pr([1.0, 100.0], 4)] == [1, 3]
    with pytest.raises(RuntimeError):
        pr([1.0, 1.0, 1.0], 2)


def test_rebalance_expert_ranges_from_step_times():
    """Closed loop of the sharding: ranks that took longer per step hand experts to ranks that took less."""
    from asymgemm_b200.ep import rebalance_expert_ranges as rb
    even = [(0, 64), (64, 128), (128, 192), (192, 256)]
    assert rb(even, [38.0, 38.5, 37.9, 38.2]) == even                    # within tolerance: untouched
    new = rb(even, [64.0, 64.0, 38.0, 38.0])                              # two ranks on a shared, slower host bridge
    sizes = [hi - lo for lo, hi in new]
    assert sum(sizes) == 256 and new[0][0] == 0 and new[-1][1] == 256 and all(new[i][1] == new[i + 1][0] for i in range(3))
    assert sizes[0] < 64 < sizes[2] and abs(sizes[0] - sizes[1]) <= 1 and abs(sizes[2] - sizes[3]) <= 1
    # predicted step times with the measured rates (experts per ms) are balanced to within one expert
    rates = [64 / 64.0, 64 / 64.0, 64 / 38.0, 64 / 38.0]
    t = [n / r for n, r in zip(sizes, rates)]
    assert max(t) - min(t) <= 1.0 / min(rates) + 1e-9
    # a second round on the new cut with times that now agree changes nothing
    assert rb(new, t) == new
    with pytest.raises(RuntimeError):
        rb(even, [1.0, 2.0])


def test_link_probe_candidate_sets():
    """Choice of GPUs from concurrent link rates: groups by rate, and candidate sets that spread over the groups."""
    from asymgemm_b200 import linkprobe as lp
    rates = [23.1, 22.8, 23.4, 23.0, 35.2, 34.8, 35.0, 34.5]             # two host bridges, one more loaded
    assert lp.rate_groups(rates) == [[4, 5, 6, 7], [0, 1, 2, 3]]
    assert lp.rate_groups([50.0, 50.5, 49.8]) == [[0, 1, 2]]
    sets = lp.candidate_sets(rates, 4)
    assert [0, 1, 2, 3] == sets[0] and [4, 5, 6, 7] in sets and [0, 1, 4, 5] in sets and [0, 2, 4, 6] in sets
    assert all(len(s) == 4 and len(set(s)) == 4 for s in sets)
    assert lp.candidate_sets(rates, 8) == [list(range(8))]
    assert lp.candidate_sets([50.0] * 8, 2)[0] == [0, 1]
    assert lp.choose_devices(8, 8)["devices"] == list(range(8))         # nothing to choose: no probe, no GPU needed


def test_gate_up_interleave_index():
    """Row order of the fused-activation weights: every 32 consecutive rows are 16 gate rows and the matching 16 up rows."""
    from asymgemm_b200 import ep
    inter = 256
    idx = ep.gate_up_interleave_index(inter)
    assert sorted(idx.tolist()) == list(range(2 * inter))
    assert idx[:16].tolist() == list(range(16)) and idx[16:32].tolist() == list(range(inter, inter + 16))
    assert idx[32:48].tolist() == list(range(16, 32)) and idx[48:64].tolist() == list(range(inter + 16, inter + 32))
    w = torch.arange(2 * inter * 4, dtype=torch.float32).view(2 * inter, 4)
    wi = ep.interleave_gate_up(w)
    for r in (0, 15, 16, 31, 32, 100, 2 * inter - 1):
        assert torch.equal(wi[r], w[(r % 32 // 16) * inter + r // 32 * 16 + r % 16])
    with pytest.raises(RuntimeError):
        ep.interleave_gate_up(torch.zeros(2 * 100, 8))


def test_hot_expert_cache_table_split():
    from asymgemm_b200.expert_cache import HotExpertCache
    c = HotExpertCache.__new__(HotExpertCache)
    c.slot_of = torch.tensor([-1, 0, -1, 1], dtype=torch.int32)      # experts 1 and 3 are cached in slots 0 and 1
    offsets = torch.tensor([0, 128, 128, 384, 384, 512, 0, 0], dtype=torch.int32)
    experts = torch.tensor([3, 0, 1, -1], dtype=torch.int32)
    (oc, ec), (os_, es) = c.split_tables(offsets, experts)
    assert oc.tolist() == [0, 128, 0, 0, 384, 512, 0, 0] and ec.tolist() == [1, 0, 0, -1]
    assert os_.tolist() == [0, 0, 128, 384, 0, 0, 0, 0] and es.tolist() == [0, 0, 0, -1]
    # every row range lands in exactly one of the two launches
    assert (oc.view(-1, 2) + os_.view(-1, 2)).reshape(-1).tolist() == offsets.tolist()


def test_torch_extension_loads_and_registers_the_launch_op():
    """The operators launch through `torch.ops.asymgemm_b200.m_grouped_gemm_nt`; it has a CUDA kernel only, so a call
    with CPU tensors is refused by the dispatcher instead of computing anything on the host."""
    from asymgemm_b200 import _lib
    ops = _lib.torch_ops()
    schema = str(ops.m_grouped_gemm_nt.default._schema)
    assert "Tensor(a!) d" in schema and "Tensor? stage" in schema and "int stage_chunk_bytes" in schema and "int num_sms" in schema and "int epilogue" in schema and "Tensor? scatter_meta" in schema and "Tensor? scatter_bases" in schema
    z = torch.zeros(4, 4)
    with pytest.raises(NotImplementedError):
        ops.m_grouped_gemm_nt(0, 0, z, None, z, None, z, None, None, 0, None, 4, 4, 4, 1, None,
                              torch.zeros(1, dtype=torch.int32), 0, None, 1.0, 0, 0, None, 0, 0, 0, None, None)


def test_auto_weight_path_rule():
    """"auto" stages only host-resident weights of at least 256 MiB in calls that can have rows for every expert."""
    from asymgemm_b200 import _lib, api
    big = torch.empty((64, 2048, 2048), dtype=torch.uint8)           # 256 MiB, 64 experts
    small = torch.empty((64, 256, 256), dtype=torch.uint8)
    C, M = _lib.LAYOUT_CONTIGUOUS, _lib.LAYOUT_MASKED
    try:
        api.set_weight_path("auto")
        assert api._use_staging(big, 64, 64 * 128, C, None)
        assert not api._use_staging(big, 64, 64 * 128 - 1, C, None)      # some expert is certainly idle
        assert api._use_staging(big, 64, 64 * 8, M, None) and not api._use_staging(big, 64, 64 * 7, M, None)
        assert not api._use_staging(small, 64, 1 << 20, C, None)
        assert not api._use_staging(big, 64, 1 << 20, C, object())        # the INT8 debug dump keeps the plain path
        api.set_weight_path("staged")
        assert api._use_staging(small, 64, 1, C, None)
        api.set_weight_path("stream")
        assert not api._use_staging(big, 64, 1 << 20, C, None)
        with pytest.raises(RuntimeError):
            api.set_weight_path("pipelined")
    finally:
        api.set_weight_path("stream")


def test_plain_c_program_compiles_against_the_header_and_links():
    """include/asymgemm_b200.h is a C header: a C99 program built with gcc and nothing else must compile with all
    warnings on, link against the library and get error codes (not crashes) for malformed requests, without a GPU."""
    import shutil
    import subprocess
    import tempfile
    from pathlib import Path
    from asymgemm_b200 import _lib
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    root = Path(__file__).resolve().parent.parent
    lib_dir = _lib.LIB_PATH.parent
    assert _lib.LIB_PATH.exists()
    with tempfile.TemporaryDirectory() as tmp:
        exe = Path(tmp) / "consumer"
        subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", str(root / "include"),
                        str(root / "tests" / "c_abi" / "consumer.c"), "-o", str(exe), "-L", str(lib_dir), "-lasymgemm_b200",
                        f"-Wl,-rpath,{lib_dir}"], check=True, capture_output=True, text=True)
        res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "c_abi consumer: ok" in res.stdout


def test_expert_range_and_layout_invariants_random():
    """Random link rates and routing counts: the ranges always tile the experts with one non-empty range per rank and
    never make the slowest finisher worse than the even split; the device-built layout puts every received row in its
    expert's 128-aligned segment exactly once."""
    import random
    from asymgemm_b200.ep import EPDispatcher, proportional_expert_ranges
    rng = random.Random(11)
    for _ in range(200):
        world = rng.randint(1, 8)
        experts = rng.randint(world, 64)
        rates = [rng.uniform(5.0, 60.0) for _ in range(world)]
        ranges = proportional_expert_ranges(rates, experts)
        assert ranges[0][0] == 0 and ranges[-1][1] == experts
        assert all(hi > lo for lo, hi in ranges) and all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
        even = [(r * experts // world, (r + 1) * experts // world) for r in range(world)]
        finish = lambda rr: max((hi - lo) / rate for (lo, hi), rate in zip(rr, rates))
        assert finish(ranges) <= finish(even) * (1 + 1e-9) + 1.0 / min(rates)       # at most one expert's time worse
    disp = EPDispatcher(6)                    # one rank owning six experts
    for _ in range(50):
        world_src = rng.randint(1, 4)
        counts = torch.tensor([[rng.choice([0, 0, 1, 5, 130, 257]) for _ in range(6)] for _ in range(world_src)], dtype=torch.int32)
        total = int(counts.sum())
        dest, per_expert, bound, offsets, experts_t = disp.layout(counts, total)
        assert per_expert.tolist() == counts.sum(dim=0).tolist() and experts_t.tolist() == [0, 1, 2, 3, 4, 5, -1]
        off = offsets.view(-1, 2).tolist()
        assert all(s % 128 == 0 and e % 128 == 0 and e - s >= n for (s, e), n in zip(off, per_expert.tolist()))
        assert all(off[i][1] == off[i + 1][0] for i in range(5)) and (total == 0 or off[-1][1] <= bound)
        # rows arrive ordered by (source rank, expert): row i of expert j from source s lands inside expert j's segment
        assert len(set(dest.tolist())) == total
        pos = 0
        seen = [0] * 6
        for s in range(world_src):
            for j in range(6):
                for _ in range(int(counts[s, j])):
                    d = int(dest[pos])
                    assert off[j][0] <= d < off[j][0] + int(per_expert[j])
                    seen[j] += 1
                    pos += 1
        assert seen == per_expert.tolist()


def test_documented_ctypes_mirror_matches_the_library():
    """The ctypes stub printed in INTEGRATION.md (for hosts without this package) is executed as written: its structure must
    have the size the library reports for ag_gemm_desc_t, and the documented op call must name as many arguments as the
    registered schema has."""
    import ctypes
    import re
    from pathlib import Path
    from asymgemm_b200 import _lib
    text = (Path(__file__).resolve().parents[1] / "INTEGRATION.md").read_text()
    m = re.search(r"class Desc\(ctypes\.Structure\):.*?\n(    _fields_ = \[.*?\]\n)", text, re.S)
    assert m, "the ctypes stub is missing from INTEGRATION.md"
    ns = {}
    exec("import ctypes\nclass Desc(ctypes.Structure):\n" + m.group(1), ns)
    lib = _lib.load()
    lib.ag_gemm_desc_size.restype = ctypes.c_uint64
    assert lib.ag_gemm_desc_size() == ctypes.sizeof(ns["Desc"]) == ctypes.sizeof(_lib.GemmDesc)
    call = re.search(r"m_grouped_gemm_nt\((kind, layout.*?)\)\n", text, re.S)
    assert call, "the op call is missing from INTEGRATION.md"
    documented = [a.strip() for a in call.group(1).replace("\n", " ").split(",") if a.strip()]
    schema = str(_lib.torch_ops().m_grouped_gemm_nt.default._schema)
    registered = schema[schema.index("(") + 1: schema.rindex(") ->")].split(",")
    assert len(documented) == len(registered) == 28, (len(documented), len(registered))
