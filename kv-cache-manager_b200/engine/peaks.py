"""The roofline denominators: measured copy bandwidth and bf16 GEMM throughput of this machine's
GPU, from ``MEASURED_PEAKS.json`` beside the package when the file is there, else an earlier
measurement of the same kind of GPU (and ``source`` says which)."""
from __future__ import annotations

import json
import os

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks() -> dict:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    out = dict(FALLBACK, source="fallback")
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        for k in FALLBACK:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out
