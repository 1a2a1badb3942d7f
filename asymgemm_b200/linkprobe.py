"""Host-link probes across the GPUs of one machine, and the choice of which GPUs a job of N ranks should use.

Every rank of the asymmetric GEMM streams its experts' weights over its own GPU's host link, so a job is as fast as the
links it runs on -- and on multi-GPU hosts the links are not independent: GPUs behind the same host bridge share a
ceiling (on one 8-GPU machine four GPUs shared ~116 GB/s while each reached 55 GB/s alone). When a job uses fewer ranks
than the machine has GPUs, the set of GPUs matters more than anything the kernel does.

`LinkProbes(devices).run(...)` measures the given GPUs streaming at the same time (one host thread per GPU, all behind one
barrier, copy engine, mean over the run). `choose_devices(n, ...)` first checks whether the default GPUs 0..n-1 slow each
other down; only if they do, it measures all visible GPUs together, builds a few candidate sets of n GPUs (the first n,
the n fastest, one spread over the groups that the rates fall into, one strided over the device order) and keeps the
candidate whose own concurrent measurement has the highest sum.

The module only needs ctypes and the C library (ag_link_probe_* in include/asymgemm_b200.h); run as a script
(`python asymgemm_b200/linkprobe.py --choose N`) it prints one JSON object and does not import torch, which is how a
launcher can call it before any rank has picked its device.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import sys
import threading
from pathlib import Path
from typing import Dict, List, Optional, Sequence

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libasymgemm_b200.so"
_lib = None


def _load():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m asymgemm_b200.build`")
        lib = ctypes.CDLL(str(LIB_PATH))
        lib.ag_link_probe_create.argtypes = [ctypes.c_int32, ctypes.c_uint64, ctypes.c_int32, ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p)]
        lib.ag_link_probe_create.restype = ctypes.c_int32
        lib.ag_link_probe_run.argtypes = [ctypes.c_void_p, ctypes.c_double, ctypes.POINTER(ctypes.c_double)]
        lib.ag_link_probe_run.restype = ctypes.c_int32
        lib.ag_link_probe_destroy.argtypes = [ctypes.c_void_p]
        lib.ag_link_probe_destroy.restype = ctypes.c_int32
        lib.ag_last_error.restype = ctypes.c_char_p
        _lib = lib
    return _lib


class LinkProbes:
    """Probes on several GPUs of this process, created once and run together as often as wanted."""

    def __init__(self, devices: Sequence[int], nbytes: int = 256 << 20, mode: int = 0, row_bytes: int = 0):
        lib = _load()
        self.devices = list(devices)
        self.handles: Dict[int, ctypes.c_void_p] = {}
        errors: List[str] = []

        def create(dev):
            h = ctypes.c_void_p()
            if lib.ag_link_probe_create(dev, nbytes, mode, row_bytes, ctypes.byref(h)) != 0:
                errors.append(f"GPU {dev}: {lib.ag_last_error().decode('utf-8', 'replace')}")   # message of the failing thread
            else:
                self.handles[dev] = h

        threads = [threading.Thread(target=create, args=(d,)) for d in self.devices]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            self.close()
            raise RuntimeError("link probe: " + "; ".join(errors))

    def run(self, devices: Optional[Sequence[int]] = None, seconds: float = 0.3) -> List[float]:
        """Mean GB/s of each of `devices` (default: all) while all of them stream at once."""
        lib = _load()
        devs = list(self.devices if devices is None else devices)
        gate = threading.Barrier(len(devs))
        out: Dict[int, float] = {}

        def go(dev):
            rate = ctypes.c_double(0.0)
            gate.wait()
            rc = lib.ag_link_probe_run(self.handles[dev], seconds, ctypes.byref(rate))
            out[dev] = rate.value if rc == 0 else 0.0

        threads = [threading.Thread(target=go, args=(d,)) for d in devs]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        return [out[d] for d in devs]

    def close(self) -> None:
        lib = _load()
        for h in self.handles.values():
            lib.ag_link_probe_destroy(h)
        self.handles = {}


def rate_groups(rates: Sequence[float], gap: float = 0.12) -> List[List[int]]:
    """Indices grouped by rate: sorted from fast to slow, a new group starts wherever the rate drops by more than `gap`
    relative to the previous one. GPUs that share a bottleneck measure alike when all stream at once."""
    order = sorted(range(len(rates)), key=lambda i: -rates[i])
    groups: List[List[int]] = []
    for i in order:
        if groups and rates[i] >= (1.0 - gap) * rates[groups[-1][-1]]:
            groups[-1].append(i)
        else:
            groups.append([i])
    return [sorted(g) for g in groups]


def candidate_sets(rates: Sequence[float], n: int) -> List[List[int]]:
    """A few sets of n of the len(rates) GPUs worth measuring: the first n, the n fastest, and one that takes GPUs in
    turn from every rate group (GPUs of one group may share a ceiling that fewer of them would not hit)."""
    v = len(rates)
    if n >= v:
        return [list(range(v))]
    sets = [list(range(n)), sorted(sorted(range(v), key=lambda i: -rates[i])[:n])]
    groups = [list(g) for g in rate_groups(rates)]
    spread: List[int] = []
    while len(spread) < n:
        for g in groups:
            if g and len(spread) < n:
                spread.append(g.pop(0))
    sets.append(sorted(spread))
    # evenly strided over the device order as well: neighbours in the enumeration often sit behind one bridge
    sets.append(sorted({(i * v) // n for i in range(n)}))
    uniq = []
    for s in sets:
        if len(s) == n and s not in uniq:
            uniq.append(s)
    return uniq


def choose_devices(n: int, visible: int, seconds: float = 0.2, nbytes: int = 128 << 20, margin: float = 0.05,
                   contention: float = 0.9) -> dict:
    """Which `n` of the `visible` GPUs to run on. Returns {"devices": [...], "why": ..., and what was measured}.

    Two stages, so that GPUs the job will not use are touched only when it pays. First the default set (GPUs 0..n-1)
    alone: each link by itself, then all n at once. If together they keep at least `contention` of the sum of their
    stand-alone rates, they do not get in each other's way and stay the choice; no other GPU is touched. Otherwise all
    visible GPUs are measured at once, candidate sets are built from the groups their rates fall into, each candidate
    is measured streaming at once, and the best one wins if it beats the default set by more than `margin`."""
    if n >= visible:
        return {"devices": list(range(visible))[:n], "why": "every visible GPU is used"}
    first = list(range(n))
    probes = LinkProbes(first, nbytes)
    try:
        alone = [probes.run([d], seconds / 2)[0] for d in first]
        together = probes.run(first, seconds)
    finally:
        probes.close()
    rec = {"first_gpus_alone_gbs": [round(x, 2) for x in alone], "first_gpus_at_once_gbs": [round(x, 2) for x in together]}
    if sum(together) >= contention * sum(alone):
        rec.update({"devices": first, "why": f"the first {n} GPUs keep {sum(together) / sum(alone):.2f} of their stand-alone host-link rates "
                                            "when they stream at once: no other GPU was measured"})
        return rec
    probes = LinkProbes(range(visible), nbytes)
    try:
        all_rates = probes.run(None, seconds)
        cands = []
        for s in candidate_sets(all_rates, n):
            r = probes.run(s, seconds)
            cands.append({"devices": s, "gbs": [round(x, 2) for x in r], "sum_gbs": round(sum(r), 2)})
    finally:
        probes.close()
    best = max(cands, key=lambda c: c["sum_gbs"])
    pick = best if best["sum_gbs"] > (1.0 + margin) * cands[0]["sum_gbs"] else cands[0]
    rec.update({"devices": pick["devices"], "all_gpus_at_once_gbs": [round(x, 2) for x in all_rates], "candidates": cands,
                "why": f"the first {n} GPUs keep only {sum(together) / sum(alone):.2f} of their stand-alone host-link rates when they stream "
                       "at once (a shared host bridge), so candidate sets of GPUs were measured streaming at once (copy engine, mean "
                       f"over {seconds} s each) before any rank started; the chosen set is the fastest one. The measurement used the copy "
                       "engines of all visible GPUs for about a second; everything after it runs on the chosen GPUs only"})
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--choose", type=int, default=0, help="print the choice of this many GPUs")
    ap.add_argument("--visible", type=int, default=0, help="GPUs visible to the process (default: ask the driver via nvidia-smi -L)")
    ap.add_argument("--seconds", type=float, default=0.2)
    args = ap.parse_args(argv)
    visible = args.visible
    if visible <= 0:
        import os
        import subprocess
        cvd = os.environ.get("CUDA_VISIBLE_DEVICES")
        if cvd is not None and cvd.strip() != "":
            visible = len([x for x in cvd.split(",") if x.strip() != ""])
        else:
            visible = len([ln for ln in subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True).stdout.splitlines()
                           if ln.startswith("GPU ")])
    if args.choose > 0:
        print(json.dumps(choose_devices(args.choose, visible, args.seconds)))
    else:
        probes = LinkProbes(range(visible))
        try:
            print(json.dumps({"all_at_once_gbs": [round(x, 2) for x in probes.run(None, args.seconds)]}))
        finally:
            probes.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
