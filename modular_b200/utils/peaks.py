"""Roofline denominators.

``measured_peaks()`` returns the copy bandwidth and cuBLAS bf16 throughput measured on
this pool's B200s when the driver-written ``MEASURED_PEAKS.json`` sits at the repository
root, and otherwise the fallback figures of an earlier measurement on the same pool
(6.65 TB/s, 1.59 PFLOP/s burst, 1.4 PFLOP/s sustained).
"""

from __future__ import annotations

import json
from pathlib import Path

_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
             "source": "fallback"}


def measured_peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    except Exception:  # noqa: BLE001
        return dict(_FALLBACK)


NVLINK_PEER_GBS = 770.0      # measured peer copy, per direction per GPU
NVLINK_ALLREDUCE_BUSBW_GBS = 725.0  # measured 8-rank all-reduce bus bandwidth at 1 GiB
