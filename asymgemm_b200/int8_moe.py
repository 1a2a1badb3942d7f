"""INT8 expert weights: the reference's offline format on disk, pinned host residency, and the INT8 MoE layer on top of
the grouped INT8 GEMM.

On-disk format (scripts/convert_int8_weights.py:17-25,392-416 of the reference): one ``layer_{L}.safetensors`` per MoE
layer with six tensors -- ``gate_int8 [G, inter, hidden]``, ``up_int8 [G, inter, hidden]``, ``down_int8 [G, hidden,
inter]`` (int8) and ``gate_scales [G, inter]``, ``up_scales [G, inter]``, ``down_scales [G, hidden]`` (fp32, one scale per
output channel, amax/127) -- plus ``asym_int8_manifest.json``. Files written by the reference's converter load here and
files written here load there.

Layer arithmetic follows the reference's GPU bucket (asym_gemm/unified_moe/runtime.py:1521-1645): per-token INT8
activations (one scale per row, broadcast over the K blocks), fused gate+up grouped GEMM with fp32 output,
``silu(gate) * up`` rounded to bf16, per-token requantisation, down GEMM with fp32 output, router-weighted sum.
Weights stay in pinned host memory and are streamed by the GEMM kernel; only the small scale tensors live on the GPU.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from . import moe_ops
from .ep import EPDispatcher, pinned_empty, to_contiguous_layout

GRAN_K = 128
MANIFEST_NAME = "asym_int8_manifest.json"
FORMAT_VERSION = 1
LAYER_FILE_PATTERN = "layer_{layer_id}.safetensors"


def quantize_per_channel_int8(w_bf16: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[N, K] bf16 -> (int8 [N, K], fp32 [N]): scale = max(amax/127, 1e-12) per output channel, round to nearest even,
    clamp to +-127 (the contract of quantize_per_channel_int8, asym_gemm/unified_moe/runtime.py:559-570)."""
    assert w_bf16.dtype == torch.bfloat16 and w_bf16.dim() == 2
    w = w_bf16.to(torch.float32)
    scales = (w.abs().amax(dim=1) / 127.0).clamp(min=1e-12)
    q = (w * (1.0 / scales)[:, None]).round().clamp(-127, 127).to(torch.int8)
    return q, scales.to(torch.float32)


def save_int8_layer(path: str, layer_id: int, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> str:
    """Quantise one layer's bf16 expert weights (gate/up [G, inter, hidden], down [G, hidden, inter]) and write its file."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    out = {}
    for name, w in (("gate", gate), ("up", up), ("down", down)):
        qs = [quantize_per_channel_int8(w[g].to(torch.bfloat16).cpu()) for g in range(w.shape[0])]
        out[f"{name}_int8"] = torch.stack([q for q, _ in qs]).contiguous()
        out[f"{name}_scales"] = torch.stack([s for _, s in qs]).contiguous()
    file = os.path.join(path, LAYER_FILE_PATTERN.format(layer_id=layer_id))
    save_file(out, file)
    return file


def write_manifest(path: str, converted_layers: List[int], model_config: Optional[dict] = None, source_model: str = "") -> str:
    manifest = {
        "format_version": FORMAT_VERSION,
        "producer": "asymgemm_b200.int8_moe",
        "source_model": source_model,
        "layer_file_pattern": LAYER_FILE_PATTERN,
        "converted_layers": sorted(int(x) for x in converted_layers),
        "quant": {"scheme": "per_channel_symmetric_int8", "scale": "amax/127", "gran_k": GRAN_K, "weight_dtype": "int8",
                  "scale_dtype": "float32", "gate_up_split": "sglang silu_and_mul (w13[:inter]=gate, w13[inter:]=up)"},
        "model": model_config or {},
    }
    file = os.path.join(path, MANIFEST_NAME)
    with open(file, "w") as f:
        json.dump(manifest, f, indent=2)
    return file


def read_manifest(path: str) -> dict:
    with open(os.path.join(path, MANIFEST_NAME)) as f:
        m = json.load(f)
    if int(m.get("format_version", -1)) != FORMAT_VERSION:
        raise RuntimeError(f"unsupported INT8 weight format version {m.get('format_version')}")
    q = m.get("quant", {})
    if q.get("scheme") != "per_channel_symmetric_int8" or int(q.get("gran_k", 0)) != GRAN_K:
        raise RuntimeError(f"unsupported quantisation in manifest: {q}")
    return m


@dataclass
class Int8ExpertWeights:
    """One layer's experts: int8 values in pinned host memory, scales expanded to the GEMM's per-K-block form on the GPU."""
    w13: torch.Tensor       # int8 [G, 2*inter, hidden] pinned host (gate rows first, then up)
    w2: torch.Tensor        # int8 [G, hidden, inter] pinned host
    sf13: torch.Tensor      # fp32 [G, 2*inter, hidden/128] device
    sf2: torch.Tensor       # fp32 [G, hidden, inter/128] device
    hidden: int
    inter: int

    @property
    def num_experts(self) -> int:
        return int(self.w13.shape[0])


def _expand_scales(per_channel: torch.Tensor, kb: int, device) -> torch.Tensor:
    """fp32 [G, N] -> [G, N, kb]: the same channel scale in every K block (what the grouped INT8 GEMM takes as sfb)."""
    return per_channel.to(device, torch.float32).unsqueeze(-1).expand(-1, -1, kb).contiguous()


def pack_int8_layer(tensors: dict, device, numa_node: Optional[int] = None) -> Int8ExpertWeights:
    """Six tensors of one layer file -> pinned fused gate+up / down weights and device scale tensors."""
    gate, up, down = tensors["gate_int8"], tensors["up_int8"], tensors["down_int8"]
    g, inter, hidden = gate.shape
    if tuple(up.shape) != (g, inter, hidden) or tuple(down.shape) != (g, hidden, inter):
        raise RuntimeError("inconsistent expert weight shapes in layer file")
    if hidden % GRAN_K or inter % GRAN_K:
        raise RuntimeError("hidden and inter must be multiples of 128")
    pinned = torch.cuda.is_available()
    make = (lambda shape: pinned_empty(shape, torch.int8, numa_node)) if pinned else (lambda shape: torch.empty(shape, dtype=torch.int8))
    w13 = make((g, 2 * inter, hidden))
    w13[:, :inter].copy_(gate)
    w13[:, inter:].copy_(up)
    w2 = make((g, hidden, inter))
    w2.copy_(down)
    sf13 = _expand_scales(torch.cat([tensors["gate_scales"], tensors["up_scales"]], dim=1), hidden // GRAN_K, device)
    sf2 = _expand_scales(tensors["down_scales"], inter // GRAN_K, device)
    return Int8ExpertWeights(w13, w2, sf13, sf2, hidden, inter)


def load_int8_layer(path: str, layer_id: int, device="cuda", numa_node: Optional[int] = None) -> Int8ExpertWeights:
    """Read ``layer_{layer_id}.safetensors`` under `path` (checked against the manifest) into pinned host memory."""
    from safetensors import safe_open
    manifest = read_manifest(path)
    if layer_id not in manifest.get("converted_layers", []):
        raise RuntimeError(f"layer {layer_id} is not listed in {MANIFEST_NAME}")
    file = os.path.join(path, manifest.get("layer_file_pattern", LAYER_FILE_PATTERN).format(layer_id=layer_id))
    with safe_open(file, framework="pt", device="cpu") as f:
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    missing = {"gate_int8", "up_int8", "down_int8", "gate_scales", "up_scales", "down_scales"} - set(tensors)
    if missing:
        raise RuntimeError(f"{file} lacks tensors {sorted(missing)}")
    return pack_int8_layer(tensors, device, numa_node)


class Int8MoELayer:
    """INT8 MoE layer on one GPU with host-resident expert weights (the reference's GPU bucket, runtime.py:1521-1645)."""

    def __init__(self, weights: Int8ExpertWeights):
        self.w = weights
        self.dispatcher = EPDispatcher(weights.num_experts)

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """x bf16 [T, hidden], topk_ids int64 [T, k], topk_weights fp32 [T, k] -> bf16 [T, hidden]."""
        from . import api
        w = self.w
        # route rows into the padded contiguous layout first (bf16), then quantise per row there: padding rows are zero,
        # their scale clamps to 1e-12 and their outputs are never read
        state, rows, _ = self.dispatcher.dispatch(x.contiguous(), topk_ids)
        a_bf16 = to_contiguous_layout(rows, state)
        m = state.padded_rows
        if m == 0:
            return torch.zeros_like(x)
        a_q, sfa = moe_ops.quant_rows_int8(a_bf16)
        d_gu = torch.empty((m, 2 * w.inter), dtype=torch.float32, device=x.device)
        api.m_grouped_int8_asym_gemm_nt_contiguous((a_q, sfa), (w.w13, w.sf13), d_gu, state.offsets, state.experts, None)
        a2, s2 = moe_ops.silu_mul_quant_int8(d_gu, w.inter)
        d_down = torch.empty((m, w.hidden), dtype=torch.float32, device=x.device)
        api.m_grouped_int8_asym_gemm_nt_contiguous((a2, s2), (w.w2, w.sf2), d_down, state.offsets, state.experts, None)
        return self.dispatcher.combine(d_down, state, topk_weights)
