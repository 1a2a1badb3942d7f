"""Binding of the reference's own CPU MoE bucket (`_cpu_C.moe_expert_forward_batch`, csrc/cpu/module.cpp:418-479 of
bytedance-iaas/AsymGEMM), compiled from its source in place into ``oracle/_ref`` by ``oracle/Makefile`` -- TEST
INFRASTRUCTURE ONLY (oracle pin and the timed CPU baseline of the MoE-layer workload). Nothing of the product loads it.

The module is the reference's pybind11 extension as it is; it is imported from its file, not installed.
"""
from __future__ import annotations

import importlib.util
import sysconfig
from pathlib import Path

import numpy as np

MODULE_PATH = Path(__file__).resolve().parent / "_ref" / ("_cpu_C" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

_mod = None
_rt = {}


def available() -> bool:
    return MODULE_PATH.exists()


def load():
    global _mod
    if _mod is None:
        spec = importlib.util.spec_from_file_location("_cpu_C", str(MODULE_PATH))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    return _mod


def runtime(threads: int = 0):
    """The reference's worker pool (`Runtime(threads)`, 0 = all hardware threads), one per size for the process."""
    if threads not in _rt:
        _rt[threads] = load().Runtime(threads)
    return _rt[threads]


def caps() -> dict:
    return dict(load().caps())


def moe_expert_forward_batch(x_bits: np.ndarray, m_offsets, expert_ids, gate_q, gate_s, up_q, up_s, down_q, down_s,
                             rt=None, out: np.ndarray = None) -> np.ndarray:
    """out fp32 [sum_m, hidden] = the layer's CPU bucket over work items (m_offsets, expert_ids); x_bits = bf16 bit
    patterns [sum_m, hidden]; weights int8 [G, inter, hidden] x2 and [G, hidden, inter] with fp32 per-channel scales."""
    mod = load()
    rt = rt if rt is not None else runtime(0)
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    g, inter, hidden = gate_q.shape
    if out is None:
        out = np.zeros((x.shape[0], hidden), dtype=np.float32)
    e8, ef = np.zeros((0,), np.int8), np.zeros((0,), np.float32)
    mod.moe_expert_forward_batch(rt, x, np.ascontiguousarray(m_offsets, dtype=np.int64), np.ascontiguousarray(expert_ids, dtype=np.int64),
                                 gate_q, gate_s, up_q, up_s, down_q, down_s, e8, ef, e8, ef, e8, ef, out, int(inter), int(hidden))
    return out
