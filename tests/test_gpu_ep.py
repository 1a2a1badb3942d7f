"""Expert-parallel FP8 MoE layer on the GPU: one rank against a dense fp32 reference, and 2 ranks over NCCL (when two
GPUs are visible) where every rank checks its own tokens against the same dense reference."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _make_weights(num_experts, hidden, inter, device):
    """All experts' FP8 weights from a fixed seed (every rank can rebuild them for the dense reference)."""
    from asymgemm_b200.utils import per_block_cast_to_fp8
    gen = torch.Generator(device="cpu").manual_seed(7)
    w13, s13, w2, s2 = [], [], [], []
    for _ in range(num_experts):
        q, s = per_block_cast_to_fp8(torch.randn((2 * inter, hidden), generator=gen) * 0.05, use_ue8m0=False)
        w13.append(q); s13.append(s)
        q, s = per_block_cast_to_fp8(torch.randn((hidden, inter), generator=gen) * 0.05, use_ue8m0=False)
        w2.append(q); s2.append(s)
    return torch.stack(w13), torch.stack(s13), torch.stack(w2), torch.stack(s2)


def _deq_block(q, s):
    n, k = q.shape
    return q.float() * s.repeat_interleave(128, 0).repeat_interleave(128, 1)[:n, :k]


def _dense_reference(x, ids, wts, w13, s13, w2, s2, inter):
    """Same arithmetic as the layer with fp32 matmuls on dequantised operands, token by expert."""
    from asymgemm_b200.utils import per_token_cast_to_fp8
    xq, sx = per_token_cast_to_fp8(x.float(), use_ue8m0=False)
    xd = xq.float() * sx.repeat_interleave(128, 1)[:, : x.shape[1]]
    y = torch.zeros_like(xd)
    for e in ids.unique().tolist():
        tok, slot = (ids == e).nonzero(as_tuple=True)
        h = (xd[tok] @ _deq_block(w13[e], s13[e]).t()).to(torch.bfloat16).float()
        act = (h[:, :inter] * torch.sigmoid(h[:, :inter]) * h[:, inter:]).to(torch.bfloat16).float()
        aq, sa = per_token_cast_to_fp8(act, use_ue8m0=False)
        ad = aq.float() * sa.repeat_interleave(128, 1)[:, :inter]
        out = (ad @ _deq_block(w2[e], s2[e]).t()).to(torch.bfloat16).float()
        y.index_add_(0, tok, out * wts[tok, slot].unsqueeze(1).float())
    return y


def _case(rank, world, device, weight_path="stream"):
    from asymgemm_b200 import ep
    num_experts, hidden, inter, tokens, top_k = 8, 512, 256, 300 + 17 * rank, 2
    w13, s13, w2, s2 = _make_weights(num_experts, hidden, inter, device)
    epr = num_experts // world
    lo = rank * epr
    layer = ep.ExpertParallelMoE(num_experts, hidden, inter,
                                 (w13[lo:lo + epr].contiguous().pin_memory(), s13[lo:lo + epr].contiguous().to(device)),
                                 (w2[lo:lo + epr].contiguous().pin_memory(), s2[lo:lo + epr].contiguous().to(device)))
    gen = torch.Generator().manual_seed(50 + rank)
    x = torch.randn((tokens, hidden), generator=gen).to(torch.bfloat16).to(device)
    logits = torch.randn((tokens, num_experts), generator=gen)
    logits[:, 6] += 2.0    # a hot expert
    logits[:, 1] -= 50.0   # an expert nobody picks
    wts, ids = torch.topk(torch.softmax(logits, -1), top_k, dim=-1)
    wts = (wts / wts.sum(-1, keepdim=True)).to(device)
    ids = ids.to(device)
    y = layer.forward(x, ids, wts)
    if world > 1:
        # rounds over groups of each rank's experts, exchanges on a second stream: every row's result is unchanged
        for groups in (2, 4):
            piped = ep.ExpertParallelMoE(num_experts, hidden, inter, layer.w13, layer.w2, pipeline_groups=groups)
            assert torch.equal(piped.forward(x, ids, wts), y), f"pipeline_groups={groups}"
            assert torch.equal(piped.forward(x, ids, wts), y), f"pipeline_groups={groups}, second call"
    # routing, layout and both exchanges by this library's own kernels over peer memory: the same output bit for bit, also
    # on a second call, which finds the previous call's rows, return addresses and results in the buffers
    peer = ep.ExpertParallelMoE(num_experts, hidden, inter, layer.w13, layer.w2, exchange="peer",
                                max_tokens=300 + 17 * (world - 1), top_k=top_k)
    try:
        assert torch.equal(peer.forward(x, ids, wts), y), "peer exchange"
        assert torch.equal(peer.forward(x[:250].contiguous(), ids[:250].contiguous(), wts[:250].contiguous()), layer.forward(
            x[:250].contiguous(), ids[:250].contiguous(), wts[:250].contiguous())), "peer exchange, fewer tokens"
        assert torch.equal(peer.forward(x, ids, wts), y), "peer exchange, third call"
    finally:
        peer.peer.close()
    # the activation fused into the gate+up GEMM's drain (weights interleaved gate / up): same output bit for bit
    w13_il = ep.interleave_gate_up(layer.w13[0].to(device)).cpu().pin_memory()
    fused = ep.ExpertParallelMoE(num_experts, hidden, inter, (w13_il, layer.w13[1]), layer.w2, fused_activation=True)
    assert torch.equal(fused.forward(x, ids, wts), y), "fused activation"
    if weight_path == "staged":
        # the copy engine moves the same bytes the kernel would read: same result, also when the staging buffers are reused
        import asymgemm_b200 as ag
        ag.set_weight_path("staged", chunk_bytes=3 * 2 * inter * hidden, slots=3)      # three gate+up experts per chunk
        layer.prefetch_next = layer.w13[0]     # the next call finds its first chunks already in the ring
        peer2 = ep.ExpertParallelMoE(num_experts, hidden, inter, layer.w13, layer.w2, exchange="peer",
                                     max_tokens=300 + 17 * (world - 1), top_k=top_k)
        peer2.prefetch_next = layer.w13[0]     # and the same through the peer-memory exchange
        try:
            assert torch.equal(layer.forward(x, ids, wts), y) and torch.equal(layer.forward(x, ids, wts), y)
            assert torch.equal(peer2.forward(x, ids, wts), y) and torch.equal(peer2.forward(x, ids, wts), y), "peer exchange, staged weights"
        finally:
            layer.prefetch_next = None
            peer2.peer.close()
            ag.set_weight_path("stream", chunk_bytes=128 << 20, slots=2)
    ref = _dense_reference(x, ids, wts, w13.to(device), s13.to(device), w2.to(device), s2.to(device), inter)
    err = float((y.float() - ref).abs().max() / ref.abs().max())
    yd, rd = y.double(), ref.double()
    diff = float(1 - 2 * (yd * rd).sum() / ((yd * yd).sum() + (rd * rd).sum()))
    assert diff < 1e-3, f"calc_diff {diff:.3e}"
    return err


def test_moe_layer_single_rank():
    import asymgemm_b200 as ag
    err = _case(0, 1, torch.device("cuda", 0))
    ag.check_status()
    # two chained FP8 GEMMs with a requantisation in between: a one-ulp difference in the activation (expf vs torch's
    # sigmoid) can move single FP8 codes, so the layer is held to 3e-2 max-rel and 1e-3 calc_diff
    assert err <= 3e-2, f"max-rel {err:.3e}"


def test_moe_layer_stages_meet_the_gemm_tolerance_on_their_own_inputs():
    """The FP8 tolerance of this path (max-rel <= 2e-2 against the fp32 dequantised reference) is stated per GEMM. The layer
    chains two of them with a requantisation in between, where a one-ulp difference in a bf16 intermediate can move an FP8
    code of the next stage's input; so the end-to-end figure of the tests above is held to 3e-2, and this test holds every
    stage to the stated tolerance on the operands the layer itself produced: gate+up GEMM and down GEMM against the CPU
    oracle, the activation + requantisation against the quantiser applied to the layer's own gate+up output."""
    import numpy as np
    from asymgemm_b200 import ep
    from asymgemm_b200.utils import per_token_cast_to_fp8
    from oracle import oracle
    from tests import helpers as H
    device = torch.device("cuda", 0)
    num_experts, hidden, inter, tokens, top_k = 8, 512, 256, 300, 2
    w13, s13, w2, s2 = _make_weights(num_experts, hidden, inter, device)
    layer = ep.ExpertParallelMoE(num_experts, hidden, inter, (w13.contiguous().pin_memory(), s13.contiguous().to(device)),
                                 (w2.contiguous().pin_memory(), s2.contiguous().to(device)))
    layer.keep_intermediates = True
    gen = torch.Generator().manual_seed(77)
    x = torch.randn((tokens, hidden), generator=gen).to(torch.bfloat16).to(device)
    wts, ids = torch.topk(torch.softmax(torch.randn((tokens, num_experts), generator=gen), -1), top_k, dim=-1)
    layer.forward(x, ids.to(device), (wts / wts.sum(-1, keepdim=True)).to(device))
    torch.cuda.synchronize()
    it = layer.intermediates
    state = it["state"]
    segments = oracle.contiguous_segments(state.offsets.cpu().tolist(), state.experts.cpu().tolist(), None, state.padded_rows)
    valid = np.zeros(state.padded_rows, dtype=bool)
    rows_per_expert = state.rows_per_expert.cpu().tolist()
    for e, r0, _ in segments:
        valid[r0:r0 + rows_per_expert[e]] = True
    # stage 1: gate+up GEMM on the layer's quantised tokens
    ref1 = oracle.gemm_fp8(H.np_bits(it["a_q"]), it["sfa"].cpu().numpy(), H.np_bits(w13), s13.numpy(), segments)
    got1 = it["d1"].float().cpu().numpy()
    assert oracle.max_rel(got1[valid], ref1[valid]) <= 2e-2
    # stage 2: bf16(silu(gate) * up) of the layer's own d1, quantised 1x128: scales agree to fp32 rounding, codes differ only
    # where the device's expf and torch's exp round a bf16 activation differently
    d1 = it["d1"].float()
    g, u = d1[:, :inter], d1[:, inter:]
    act = ((g / (1.0 + torch.exp(-g))) * u).to(torch.bfloat16).float()
    q_ref, sf_ref = per_token_cast_to_fp8(act, use_ue8m0=False)
    vmask = torch.from_numpy(valid).to(device)
    assert ((it["s2"] - sf_ref).abs()[vmask] <= 1e-2 * sf_ref[vmask]).all()
    assert (it["a2"].view(torch.uint8)[vmask] != q_ref.view(torch.uint8)[vmask]).float().mean() < 1e-2
    deq = it["a2"].float() * it["s2"].repeat_interleave(128, 1)[:, :inter]
    amax = act.view(act.shape[0], -1, 128).abs().amax(dim=2).repeat_interleave(128, 1)
    assert ((deq - act).abs()[vmask] <= (amax * 0.0625 + 1e-6)[vmask]).all()      # within half an e4m3 step of the block maximum
    # stage 3: down GEMM on the layer's own requantised activations
    ref2 = oracle.gemm_fp8(H.np_bits(it["a2"]), it["s2"].cpu().numpy(), H.np_bits(w2), s2.numpy(), segments)
    got2 = it["d2"].float().cpu().numpy()
    assert oracle.max_rel(got2[valid], ref2[valid]) <= 2e-2
    assert oracle.calc_diff(got2[valid], ref2[valid]) <= 1e-3


def test_moe_layer_single_rank_staged_weights():
    import asymgemm_b200 as ag
    err = _case(0, 1, torch.device("cuda", 0), weight_path="staged")
    ag.check_status()
    assert err <= 3e-2, f"max-rel {err:.3e}"


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        device = torch.device("cuda", rank)
        torch.cuda.set_device(device)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        import asymgemm_b200 as ag
        err = _case(rank, world, device)
        ag.check_status()
        dist.barrier()
        q.put((rank, err))
    except Exception as e:  # pragma: no cover
        q.put((rank, f"error: {type(e).__name__}: {e}"))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_moe_layer_two_ranks_nccl():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    for r in range(2):
        assert isinstance(res[r], float), res
        assert res[r] <= 3e-2, res


def test_helper_kernels_match_torch():
    """The fused helper kernels against the torch formulation of the same steps."""
    from asymgemm_b200 import moe_ops
    from asymgemm_b200.utils import per_token_cast_to_fp8
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn((333, 640), device="cuda", generator=gen) * 3).to(torch.bfloat16)
    x[5] = 0                                            # an all-zero row hits the 1e-4 clamp
    q, sf = moe_ops.quant_rows_fp8(x)
    q_ref, sf_ref = per_token_cast_to_fp8(x.float(), use_ue8m0=False)
    assert torch.equal(sf, sf_ref) and torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))

    inter = 384
    gu = (torch.randn((257, 2 * inter), device="cuda", generator=gen) * 2).to(torch.bfloat16)
    q, sf = moe_ops.silu_mul_quant_fp8(gu, inter)
    g, u = gu[:, :inter].float(), gu[:, inter:].float()
    act = (g * torch.sigmoid(g) * u).to(torch.bfloat16).float()
    got = q.float() * sf.repeat_interleave(128, 1)[:, :inter]
    # 1x128 FP8 of the same activation: within half an e4m3 step (2^-4 relative) of the block maximum
    amax = act.view(257, -1, 128).abs().amax(dim=2).repeat_interleave(128, 1)
    assert ((got - act).abs() <= amax * 0.0625 + 1e-6).all()
    q_ref, sf_ref = per_token_cast_to_fp8(act, use_ue8m0=False)
    assert (sf - sf_ref).abs().max() <= 1e-2 * sf_ref.abs().max()
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-2   # expf vs torch.sigmoid: rare 1-ulp flips

    rows = torch.randn((100, 256), device="cuda", generator=gen).to(torch.bfloat16)
    idx = torch.randperm(100, device="cuda", generator=gen)[:60]
    out = moe_ops.move_rows(rows, 300, src_rows=idx, dst_rows=idx * 3, zero=True)
    ref = torch.zeros((300, 256), dtype=torch.bfloat16, device="cuda")
    ref[idx * 3] = rows[idx]
    assert torch.equal(out, ref)

    tokens, k = 50, 3
    pos = torch.randint(0, 100, (tokens * k,), device="cuda", generator=gen)
    w = torch.rand((tokens, k), device="cuda", generator=gen)
    y = moe_ops.combine_topk(rows, pos, w, tokens, k)
    ref = (rows[pos].view(tokens, k, -1).float() * w.unsqueeze(-1)).sum(1)
    assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max()


def test_wide_quantiser_kernels_equal_the_narrow_ones():
    """Rows that are 16-byte aligned take the wide kernels (16-byte loads, two 128-column blocks per warp); the same data at
    an address that is only 8-byte aligned takes the narrow ones. Values and scales must agree bit for bit."""
    from asymgemm_b200 import moe_ops
    gen = torch.Generator(device="cuda").manual_seed(7)

    def misaligned(t):
        flat = torch.empty(t.numel() + 4, dtype=t.dtype, device=t.device)
        view = flat[4:].view(t.shape)
        view.copy_(t)
        assert view.data_ptr() % 16 == 8 and t.data_ptr() % 16 == 0 and view.is_contiguous()
        return view

    for rows, cols in ((333, 640), (64, 128), (17, 1000), (5, 7168)):          # odd block counts, a ragged last block
        x = (torch.randn((rows, cols), device="cuda", generator=gen) * 3).to(torch.bfloat16)
        x[rows // 2] = 0
        for pow2 in (False, True):
            q1, s1 = moe_ops.quant_rows_fp8(x, pow2_scales=pow2)
            q2, s2 = moe_ops.quant_rows_fp8(misaligned(x), pow2_scales=pow2)
            assert torch.equal(s1, s2) and torch.equal(q1.view(torch.uint8), q2.view(torch.uint8)), (rows, cols, pow2)
    for rows, inter in ((257, 384), (33, 128), (9, 2048), (21, 200)):
        gu = (torch.randn((rows, 2 * inter), device="cuda", generator=gen) * 2).to(torch.bfloat16)
        for pow2 in (False, True):
            q1, s1 = moe_ops.silu_mul_quant_fp8(gu, inter, pow2_scales=pow2)
            q2, s2 = moe_ops.silu_mul_quant_fp8(misaligned(gu), inter, pow2_scales=pow2)
            assert torch.equal(s1, s2) and torch.equal(q1.view(torch.uint8), q2.view(torch.uint8)), (rows, inter, pow2)


def test_pow2_quantiser_and_hardware_scaled_layer():
    """Row quantiser with power-of-two scales against the torch quantiser with use_ue8m0=True, and the MoE layer on the
    hardware-scaled FP8 path against the same layer on the exact path (same inputs, weights quantised with UE8M0 scales)."""
    import asymgemm_b200 as ag
    from asymgemm_b200 import ep, moe_ops
    from asymgemm_b200.utils import per_block_cast_to_fp8, per_token_cast_to_fp8
    gen = torch.Generator(device="cuda").manual_seed(9)
    x = (torch.randn((300, 512), device="cuda", generator=gen) * 2).to(torch.bfloat16)
    q, sf = moe_ops.quant_rows_fp8(x, pow2_scales=True)
    q_ref, sf_ref = per_token_cast_to_fp8(x.float(), use_ue8m0=True)
    assert torch.equal(torch.log2(sf), torch.log2(sf).round())                 # powers of two
    assert (sf != sf_ref).float().mean() < 1e-3                                # log2f-based torch version: rare edge cases only
    same = sf == sf_ref
    assert torch.equal(q.view(torch.uint8)[same.repeat_interleave(128, 1)], q_ref.view(torch.uint8)[same.repeat_interleave(128, 1)])

    num_experts, hidden, inter, tokens, top_k = 4, 512, 256, 260, 2
    cpu_gen = torch.Generator().manual_seed(10)
    def qw(n, k):
        return per_block_cast_to_fp8(torch.randn((n, k), generator=cpu_gen) * 0.05, use_ue8m0=True)
    w13 = [qw(2 * inter, hidden) for _ in range(num_experts)]
    w2 = [qw(hidden, inter) for _ in range(num_experts)]
    pack = lambda ws: (torch.stack([q for q, _ in ws]).pin_memory(), torch.stack([s for _, s in ws]).cuda())
    ids = torch.stack([torch.randperm(num_experts, generator=cpu_gen)[:top_k] for _ in range(tokens)]).cuda()
    wts = torch.rand((tokens, top_k), generator=cpu_gen).cuda()
    xin = torch.randn((tokens, hidden), generator=cpu_gen).to(torch.bfloat16).cuda()
    outs = []
    for hw in (True, False):
        layer = ep.ExpertParallelMoE(num_experts, hidden, inter, pack(w13), pack(w2), ue8m0_scales=hw)
        # both layers quantise activations with power-of-two scales so that they see identical operands
        layer_out = None
        x_q, sfx = moe_ops.quant_rows_fp8(xin, pow2_scales=True)
        state, recv_q, (recv_s,) = layer.dispatcher.dispatch(x_q, ids, (sfx,))
        a_q, sfa = ep.to_contiguous_layout(recv_q, state), ep.to_contiguous_layout(recv_s, state)
        d1 = torch.empty((state.padded_rows, 2 * inter), dtype=torch.bfloat16, device="cuda")
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((a_q, sfa), layer.w13, d1, state.offsets, state.experts, None, ue8m0_scales=hw)
        a2, s2 = moe_ops.silu_mul_quant_fp8(d1, inter, pow2_scales=True)
        d2 = torch.zeros((state.padded_rows, hidden), dtype=torch.bfloat16, device="cuda")
        ag.m_grouped_fp8_asym_gemm_nt_contiguous((a2, s2), layer.w2, d2, state.offsets, state.experts, None, ue8m0_scales=hw)
        outs.append(layer.dispatcher.combine(d2, state, wts))
    ag.check_status()
    err = float((outs[0].float() - outs[1].float()).abs().max() / outs[1].float().abs().max())
    assert err <= 2e-2, f"hardware-scaled vs exact layer: max-rel {err:.3e}"
    y = ep.ExpertParallelMoE(num_experts, hidden, inter, pack(w13), pack(w2), ue8m0_scales=True).forward(xin, ids, wts)
    assert float((y.float() - outs[0].float()).abs().max()) == 0.0
