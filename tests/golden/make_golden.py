#!/usr/bin/env python
"""Generates the golden fixtures in this directory by IMPORTING the reference's own Python code.

Run once in a container that has the reference checkout (pass its path with --reference); the fixtures are committed, the
checkout is not needed to run the tests. What is imported from bytedance-iaas/AsymGEMM:
  * asym_gemm/utils/math.py          -- the quantisers that define the FP8 / INT8 / NVFP4 formats
  * tests/test_fp4_asym_gemm.py      -- _quantize_nvfp4_e4m3, _manual_dequant_reference (NVFP4 dequantised reference)
  * tests/test_sm90_int8.py          -- ref_2d / dequant (INT8 float reference)
  * tests/m_grouped/test_sm100_bf16_fp8_fp4_m_grouped.py -- _fp4_masked_reference (masked NVFP4 reference)
  * oracle/_ref (csrc/cpu/cpu_gemm)  -- exact int32 block sums through the reference's cg_gemm
The compiled extension `asym_gemm._C` cannot be built here; a stub package stands in for it so that the pure-Python
helpers import. The reference's GPU kernels themselves are never run.

    python tests/golden/make_golden.py [--reference <checkout of the reference>]
"""
from __future__ import annotations

import argparse
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _install_reference(ref: Path):
    math_mod = _load(ref / "asym_gemm" / "utils" / "math.py", "asym_gemm.utils.math")
    numeric = _load(ref / "asym_gemm" / "testing" / "numeric.py", "asym_gemm.testing.numeric")
    pkg = types.ModuleType("asym_gemm")
    pkg.__path__ = []
    pkg.get_mk_alignment_for_contiguous_layout = lambda: 128
    utils = types.ModuleType("asym_gemm.utils")
    utils.__path__ = []
    for k in dir(math_mod):
        if not k.startswith("__"):
            setattr(utils, k, getattr(math_mod, k))
    utils.math = math_mod
    utils.get_mk_alignment_for_contiguous_layout = lambda: 128
    testing = types.ModuleType("asym_gemm.testing")
    testing.calc_diff = numeric.calc_diff
    testing.count_bytes = numeric.count_bytes
    testing.get_arch_major = lambda: 10
    testing.ignore_env = lambda *a, **k: (lambda f: f)
    testing.bench_kineto = testing.bench = None
    pkg.utils, pkg.testing = utils, testing
    sys.modules.update({"asym_gemm": pkg, "asym_gemm.utils": utils, "asym_gemm.testing": testing})
    fp4 = _load(ref / "tests" / "test_fp4_asym_gemm.py", "ref_test_fp4")
    int8 = _load(ref / "tests" / "test_sm90_int8.py", "ref_test_int8")
    # tests/m_grouped/... imports its NVFP4 helpers from a module name that does not exist in the repository
    # (`test_nvfp4`); they live in tests/test_fp4_asym_gemm.py, so that module stands in under the missing name.
    sys.modules["test_nvfp4"] = fp4
    global MG
    MG = _load(ref / "tests" / "m_grouped" / "test_sm100_bf16_fp8_fp4_m_grouped.py", "ref_test_m_grouped")
    return math_mod, numeric, fp4, int8


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def segments_table(rows):
    """(offsets, experts) the way the reference's tests build them: 128-aligned segments, -1 terminator."""
    offsets, experts, start = [], [], 0
    segs = []
    for e, r in enumerate(rows):
        if r == 0:
            continue
        padded = -(-r // 128) * 128
        offsets += [start, start + padded]
        experts.append(e)
        segs.append((e, start, r))
        start += padded
    experts.append(-1)
    return np.array(offsets, np.int32), np.array(experts, np.int32), start, segs


def extra_quantisers(M, x, w):
    """The reference's remaining quantisers (asym_gemm/utils/math.py:37-45,82-88,103-119,142-155) on the shared inputs."""
    xs = x[:256]                                    # per_channel_cast_to_fp8 wants rows % 128 == 0
    out = {}
    for tag, ue in (("f32", False), ("ue8m0", True)):
        q, s = M.per_channel_cast_to_fp8(xs, use_ue8m0=ue)
        out[f"chan_q_{tag}"], out[f"chan_s_{tag}"] = bits(q), s.numpy()
        q, s = M.per_custom_dims_cast_to_fp8(w, (0, 2), use_ue8m0=ue)
        out[f"dims_q_{tag}"], out[f"dims_s_{tag}"] = bits(q), s.numpy()
        q, s = M.per_token_cast_to_fp4(xs, use_ue8m0=ue, gran_k=128)
        out[f"fp4_q_{tag}"], out[f"fp4_s_{tag}"] = q.numpy(), s.numpy()
    packed, _ = M.per_token_cast_to_fp4(xs, use_ue8m0=False, gran_k=128)
    out["fp4_transposed"] = M.transpose_packed_fp4(packed).numpy()
    np.savez_compressed(HERE / "quantisers_extra.npz", **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of bytedance-iaas/AsymGEMM (its quantisers and test-side "
                                                       "references are imported from there)")
    ap.add_argument("--only-extra", action="store_true", help="write quantisers_extra.npz only (from the committed inputs.npz)")
    args = ap.parse_args()
    ref = Path(args.reference)
    M, numeric, fp4, int8 = _install_reference(ref)
    if args.only_extra:
        g0 = np.load(HERE / "inputs.npz")
        extra_quantisers(M, torch.from_numpy(g0["x"].astype(np.float32)), torch.from_numpy(g0["w"].astype(np.float32)))
        return

    torch.manual_seed(0)
    np.random.seed(0)
    rows = [70, 0, 33, 130]
    g, n, k = len(rows), 72, 256
    offsets, experts, m_total, segs = segments_table(rows)
    x = torch.zeros((m_total, k))
    for e, s, r in segs:
        x[s:s + r] = torch.randn((r, k)).half().float()   # fp16-representable so the inputs store compactly
    w = (torch.randn((g, n, k)) * 0.02).half().float()
    common = dict(offsets=offsets, experts=experts, rows=np.array(rows, np.int32))
    np.savez_compressed(HERE / "inputs.npz", x=x.numpy().astype(np.float16), w=w.numpy().astype(np.float16), **common)
    extra_quantisers(M, x, w)

    def per_seg(fn):
        out = torch.zeros((m_total, n), dtype=torch.float32)
        for e, s, r in segs:
            out[s:s + r] = fn(e, s, r)
        return out

    # ---- BF16: a.float() @ b[g].float().t() -> bf16 (tests/m_grouped/...:99-109)
    a16, b16 = x.to(torch.bfloat16), w.to(torch.bfloat16)
    ref16 = per_seg(lambda e, s, r: a16[s:s + r].float() @ b16[e].float().t())
    np.savez_compressed(HERE / "bf16_contiguous.npz", a=bits(a16), b=bits(b16), ref_f32=ref16.numpy(),
                        ref_bf16=bits(ref16.to(torch.bfloat16)), **common)

    # ---- FP8: reference quantisers (both scale modes) + dequantised fp32 product + the tests' unquantised ground truth
    for tag, ue in (("fp32scale", False), ("ue8m0", True)):
        aq, sfa = M.per_token_cast_to_fp8(x, use_ue8m0=ue)
        bq, sfb = zip(*[M.per_block_cast_to_fp8(w[i], use_ue8m0=ue) for i in range(g)])
        bq, sfb = torch.stack(bq), torch.stack(sfb)
        a_deq = aq.float() * sfa.repeat_interleave(128, 1)[:, :k]
        b_deq = bq.float() * sfb.repeat_interleave(128, 1).repeat_interleave(128, 2)[:, :n, :k]
        ref8 = per_seg(lambda e, s, r: a_deq[s:s + r] @ b_deq[e].t())
        gt = per_seg(lambda e, s, r: a16[s:s + r].float() @ b16[e].float().t())
        np.savez_compressed(HERE / f"fp8_{tag}_contiguous.npz", a=bits(aq), sfa=sfa.numpy(), b=bits(bq), sfb=sfb.numpy(),
                            ref_f32=ref8.numpy(), ref_unquantised=gt.numpy(), **common)

    # ---- INT8: reference quantisers, ref_2d float reference (tests/test_sm90_int8.py:39-54), exact sums via cg_gemm
    k8 = k
    aq, sfa = M.per_token_cast_to_int8(x)
    bq, sfb = zip(*[M.per_channel_cast_to_int8(w[i]) for i in range(g)])
    bq, sfb = torch.stack(bq), torch.stack(sfb)
    ref_i8 = per_seg(lambda e, s, r: int8.ref_2d(aq[s:s + r], sfa[s:s + r], bq[e], sfb[e], k8))
    from oracle import ref_cpu_gemm as R
    sums = np.zeros((k8 // 128, m_total, n), np.int32)
    a_np = aq.numpy()
    for e, s, r in segs:
        # cg_gemm quantises each row of A by amax/127: rows are exact only when every K block holds a +-127, which
        # per_token_cast_to_int8 guarantees (the block's amax maps to +-127) unless the block is all zero.
        blk_ok = np.abs(a_np[s:s + r].reshape(r, -1, 128).astype(np.int32)).max(axis=2) == 127
        assert blk_ok.all()
        sums[:, s:s + r] = R.exact_int32_block_sums(a_np[s:s + r], bq[e].numpy())
    np.savez_compressed(HERE / "int8_contiguous.npz", a=a_np, sfa=sfa.numpy(), b=bq.numpy(), sfb=sfb.numpy(),
                        ref_f32=ref_i8.numpy(), block_sums=sums, cg_backend=np.array(R.backend_name()), **common)

    # ---- NVFP4: both reference quantisers (numpy test helper and utils/math.py) + _manual_dequant_reference
    a_p, a_s = fp4._quantize_a_nvfp4_e4m3(x.numpy(), 16)
    b_ps = [fp4._quantize_b_nvfp4_e4m3(w[i].numpy(), 16) for i in range(g)]
    b_p = np.stack([p for p, _ in b_ps])
    b_s = np.stack([s for _, s in b_ps])
    m_indices = torch.full((m_total,), -1, dtype=torch.int32)
    for e, s, r in segs:
        m_indices[s:s + r] = e
    ref4 = fp4._manual_dequant_reference(a_p, a_s, b_p, b_s, m_indices, 16)
    a_p2, a_s2 = M.per_token_cast_to_nvfp4_e4m3(x, 16)
    np.savez_compressed(HERE / "fp4_contiguous.npz", a=a_p, sfa=a_s, b=b_p, sfb=b_s, ref_f32=ref4.numpy(),
                        a_math=a_p2.numpy(), sfa_math=bits(a_s2), m_indices=m_indices.numpy(), **common)

    # ---- masked layout (FP8): [G, M_max, K], masked_m (tests/m_grouped/...:320-342 semantics)
    m_max = 128
    masked_m = np.array([64, 0, 96, 128], np.int32)
    xm = torch.randn((g, m_max, k)).half().float()
    aq, sfa = zip(*[M.per_token_cast_to_fp8(xm[i], use_ue8m0=True) for i in range(g)])
    aq, sfa = torch.stack(aq), torch.stack(sfa)
    bq, sfb = zip(*[M.per_block_cast_to_fp8(w[i], use_ue8m0=True) for i in range(g)])
    bq, sfb = torch.stack(bq), torch.stack(sfb)
    a_deq = aq.float() * sfa.repeat_interleave(128, 2)[..., :k]
    b_deq = bq.float() * sfb.repeat_interleave(128, 1).repeat_interleave(128, 2)[:, :n, :k]
    refm = torch.einsum("gmk,gnk->gmn", a_deq, b_deq)
    np.savez_compressed(HERE / "fp8_masked.npz", a=bits(aq), sfa=sfa.numpy(), b=bits(bq), sfb=sfb.numpy(), masked_m=masked_m,
                        ref_f32=refm.numpy(), xm=xm.numpy().astype(np.float16))
    # ---- masked layout, the other dtypes, on the same activations xm and weights w
    a16m, b16m = xm.to(torch.bfloat16), w.to(torch.bfloat16)
    ref16m = torch.einsum("gmk,gnk->gmn", a16m.float(), b16m.float())          # tests/m_grouped/...: _bf16_masked_case
    np.savez_compressed(HERE / "bf16_masked.npz", a=bits(a16m), b=bits(b16m), masked_m=masked_m, ref_f32=ref16m.numpy(),
                        ref_bf16=bits(ref16m.to(torch.bfloat16)))
    aq, sfa = zip(*[M.per_token_cast_to_int8(xm[i]) for i in range(g)])
    aq, sfa = torch.stack(aq), torch.stack(sfa)
    bq, sfb = zip(*[M.per_channel_cast_to_int8(w[i]) for i in range(g)])
    bq, sfb = torch.stack(bq), torch.stack(sfb)
    ref8m = torch.stack([int8.ref_2d(aq[i], sfa[i], bq[i], sfb[i], k) for i in range(g)])   # tests/test_sm90_int8.py:51-54
    np.savez_compressed(HERE / "int8_masked.npz", a=aq.numpy(), sfa=sfa.numpy(), b=bq.numpy(), sfb=sfb.numpy(), masked_m=masked_m,
                        ref_f32=ref8m.numpy())
    a_ps = [fp4._quantize_a_nvfp4_e4m3(xm[i].numpy(), 16) for i in range(g)]
    a_p4, a_s4 = np.stack([p for p, _ in a_ps]), np.stack([s_ for _, s_ in a_ps])
    ref4m = MG._fp4_masked_reference(a_p4, a_s4, b_p, b_s, torch.from_numpy(masked_m), 16)
    np.savez_compressed(HERE / "fp4_masked.npz", a=a_p4, sfa=a_s4, b=b_p, sfb=b_s, masked_m=masked_m, ref_f32=ref4m.numpy())
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
