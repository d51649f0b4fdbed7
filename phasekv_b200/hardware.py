"""Roofline figures of the GPU this package is written for, in the shape the reference's planner reads them.

``planner.HardwareSpec`` of the reference (``src/phasekv/planner.py:43-59``) carries a name, an effective half-precision
matrix throughput and a memory bandwidth, defaulting to an RTX 4080 SUPER (50 TFLOP/s, 736 GB/s); its roofline helpers
and ``PlanInput.hardware`` only read ``peak_flops``, ``hbm_bandwidth`` and ``ridge_intensity``.  ``HardwareSpec`` here has
the same fields, and ``b200()`` fills them for a B200: with the copy bandwidth and the cuBLAS bf16 throughput measured
on the machine when a ``MEASURED_PEAKS.json`` is at hand (keys ``hbm_gbs``, ``bf16_tflops``), otherwise with an earlier
measurement of the same GPU model.  Pass the object where the reference's planner takes a ``HardwareSpec``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional

B200_HBM_BYTES_PER_S = 6.65e12      # STREAM-style copy, measured on B200s (nominal 7.7e12)
B200_BF16_FLOPS = 1.59e15           # cuBLAS bf16 GEMM burst, measured (nominal dense 2.25e15)


@dataclass
class HardwareSpec:
    name: str = "B200"
    peak_flops: float = B200_BF16_FLOPS
    hbm_bandwidth: float = B200_HBM_BYTES_PER_S

    @property
    def ridge_intensity(self) -> float:
        """FLOP per byte above which a kernel is compute-bound, below which bandwidth-bound."""
        return self.peak_flops / self.hbm_bandwidth


def b200(measured_peaks: Optional[str] = None) -> HardwareSpec:
    """``HardwareSpec`` of a B200; ``measured_peaks`` names a JSON file with ``hbm_gbs`` and ``bf16_tflops``."""
    spec = HardwareSpec()
    if measured_peaks and os.path.exists(measured_peaks):
        with open(measured_peaks) as f:
            data = json.load(f)
        if "hbm_gbs" in data:
            spec.hbm_bandwidth = float(data["hbm_gbs"]) * 1e9
        if "bf16_tflops" in data:
            spec.peak_flops = float(data["bf16_tflops"]) * 1e12
        spec.name = "B200 (measured)"
    return spec
