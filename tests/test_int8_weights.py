"""The INT8 expert-weight format on disk (the reference's offline converter layout) and the INT8 MoE layer."""
import json
import os

import pytest
import torch

from asymgemm_b200 import int8_moe as W


def _masters(g=3, inter=128, hidden=256, seed=0):
    gen = torch.Generator().manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, generator=gen) * 0.05).to(torch.bfloat16)
    return mk(g, inter, hidden), mk(g, inter, hidden), mk(g, hidden, inter)


def test_per_channel_quantiser_contract():
    w = (torch.randn(64, 256) * 0.1).to(torch.bfloat16)
    w[3] = 0
    q, s = W.quantize_per_channel_int8(w)
    assert q.dtype == torch.int8 and s.dtype == torch.float32 and s.shape == (64,)
    assert s[3] == pytest.approx(1e-12) and (q[3] == 0).all()
    amax = w.float().abs().amax(dim=1)
    assert torch.allclose(s[amax > 0], (amax / 127.0)[amax > 0])
    assert (q.abs().amax(dim=1)[amax > 0] == 127).all()
    assert ((q.float() * s[:, None] - w.float()).abs() <= s[:, None] * 0.501 + 1e-7).all()


def test_layer_file_roundtrip_and_manifest(tmp_path):
    gate, up, down = _masters()
    path = str(tmp_path)
    W.save_int8_layer(path, 7, gate, up, down)
    W.write_manifest(path, [7], {"hidden_size": 256})
    m = W.read_manifest(path)
    assert m["converted_layers"] == [7] and m["layer_file_pattern"] == "layer_{layer_id}.safetensors"
    assert m["quant"]["gran_k"] == 128 and m["quant"]["scale"] == "amax/127"
    from safetensors import safe_open
    with safe_open(os.path.join(path, "layer_7.safetensors"), framework="pt") as f:
        assert sorted(f.keys()) == ["down_int8", "down_scales", "gate_int8", "gate_scales", "up_int8", "up_scales"]
        assert f.get_tensor("gate_int8").shape == (3, 128, 256) and f.get_tensor("down_scales").shape == (3, 256)
    ew = W.load_int8_layer(path, 7, device="cpu")
    assert ew.w13.shape == (3, 256, 256) and ew.w2.shape == (3, 256, 128)
    assert ew.sf13.shape == (3, 256, 2) and ew.sf2.shape == (3, 256, 1)
    q, s = W.quantize_per_channel_int8(up[1])
    assert torch.equal(ew.w13[1, 128:], q) and torch.equal(ew.sf13[1, 128:, 0], s) and torch.equal(ew.sf13[1, :, 0], ew.sf13[1, :, 1])
    with pytest.raises(RuntimeError):
        W.load_int8_layer(path, 8, device="cpu")          # not in the manifest
    bad = json.load(open(os.path.join(path, W.MANIFEST_NAME)))
    bad["quant"]["gran_k"] = 64
    json.dump(bad, open(os.path.join(path, W.MANIFEST_NAME), "w"))
    with pytest.raises(RuntimeError):
        W.read_manifest(path)


@pytest.mark.gpu
def test_int8_moe_layer_against_dense_reference(tmp_path):
    """Weights written in the offline format, loaded into pinned memory, layer output against the same arithmetic done
    densely with fp32 matmuls (per-token INT8 activations, fp32 GEMM outputs, bf16-rounded SwiGLU, per-token requant)."""
    import asymgemm_b200 as ag
    g, inter, hidden, tokens, top_k = 6, 256, 512, 333, 2
    gate, up, down = _masters(g, inter, hidden, seed=2)
    W.save_int8_layer(str(tmp_path), 0, gate, up, down)
    W.write_manifest(str(tmp_path), [0])
    ew = W.load_int8_layer(str(tmp_path), 0, device="cuda")
    assert ew.w13.is_pinned() and ew.sf13.is_cuda
    layer = W.Int8MoELayer(ew)
    gen = torch.Generator().manual_seed(5)
    x = torch.randn((tokens, hidden), generator=gen).to(torch.bfloat16).cuda()
    logits = torch.randn((tokens, g), generator=gen)
    logits[:, 4] -= 40.0
    wts, ids = torch.topk(torch.softmax(logits, -1), top_k, dim=-1)
    wts, ids = wts.cuda(), ids.cuda()
    y = layer.forward(x, ids, wts)
    ag.check_status()

    def q_rows(t):   # quantize_per_token_int8_gpu of the reference (runtime.py:573-583)
        s = (t.float().abs().amax(dim=1) / 127.0).clamp(min=1e-12)
        return (t.float() * (1.0 / s)[:, None]).round().clamp(-127, 127), s
    w13 = ew.w13.cuda().float() * ew.sf13[:, :, 0].unsqueeze(-1)
    w2 = ew.w2.cuda().float() * ew.sf2[:, :, 0].unsqueeze(-1)
    ref = torch.zeros((tokens, hidden), device="cuda")
    for e in ids.unique().tolist():
        tok, slot = (ids == e).nonzero(as_tuple=True)
        q, s = q_rows(x[tok])
        gu = (q * s[:, None]) @ w13[e].t()
        act = (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]).to(torch.bfloat16)
        q2, s2 = q_rows(act)
        out = (q2 * s2[:, None]) @ w2[e].t()
        ref.index_add_(0, tok, out * wts[tok, slot].unsqueeze(1))
    err = float((y.float() - ref).abs().max() / ref.abs().max())
    assert err <= 2e-2, f"max-rel {err:.3e}"
