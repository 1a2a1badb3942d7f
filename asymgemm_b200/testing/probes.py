"""Hardware probes of the library, for tuning and for the record (not used by any operator)."""
from __future__ import annotations

import ctypes

from .. import _lib


def mma_issue_cycles(issuers: int, n_cols: int = 256, steps: int = 4096) -> float:
    """SM cycles per step of four bf16 `tcgen05.mma` (M128 x N`n_cols` x K16) when `issuers` threads per CTA issue them
    against producers that only arrive on the barriers, worst CTA of the current device (`ag_probe_mma_issue`). The
    tensor core's own time for a step is 2 * n_cols cycles."""
    lib = _lib.load()
    out = ctypes.c_double(0.0)
    _lib.check(lib.ag_probe_mma_issue(int(issuers), int(n_cols), int(steps), ctypes.byref(out)))
    return out.value


def operand_feed_cycles(load_a: bool, load_b: bool) -> float:
    """SM cycles per 128-byte K atom (two steps of four 256-column bf16 MMAs; tensor time 1024) of the kernels' producer /
    issuer rings with real TMA loads of the activations and / or the weights from device memory and nothing else
    (`ag_probe_operand_feed`; allocates 1 GB while it runs)."""
    lib = _lib.load()
    out = ctypes.c_double(0.0)
    _lib.check(lib.ag_probe_operand_feed(int(bool(load_a)), int(bool(load_b)), ctypes.byref(out)))
    return out.value


if __name__ == "__main__":
    import json

    print(json.dumps({f"issuers={i} n_cols={n}": round(mma_issue_cycles(i, n), 1) for n in (256, 128) for i in (1, 2)}))
    print(json.dumps({f"loads a={int(a)} b={int(b)}": round(operand_feed_cycles(a, b), 1) for a, b in ((False, False), (True, False), (False, True), (True, True))}))
