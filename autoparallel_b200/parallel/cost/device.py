"""Device limits used by the compute cost model.

The B200 entry carries *measured* figures for this class of machine (a STREAM-style copy and a
cuBLAS bf16 GEMM sustained under the power cap) next to the nominal ones; the planner prices
compute with the measured numbers, so no blanket "70 % of peak" factor is applied for B200.
Other entries are nominal with a 0.7 efficiency factor, like the reference's table
(autoparallel/cost_models/compute_estimation.py:67-275).  A ``cpu`` entry exists so planning
runs on machines without a GPU (the reference requires a CUDA device name).
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Optional

import torch


@dataclasses.dataclass(frozen=True)
class DeviceLimit:
    name: str
    hbm_gbs: float  # achievable memory bandwidth, GB/s
    tflops: dict  # dtype -> achievable dense TFLOP/s
    efficiency: float = 1.0  # multiplier on both (1.0 when the figures are measured)
    launch_us: float = 3.0
    sm_count: int = 0
    hbm_gb: float = 0.0

    def flops_per_us(self, dtype: torch.dtype) -> float:
        t = self.tflops.get(dtype) or self.tflops.get(torch.float32)
        return t * 1e6 * self.efficiency  # TFLOP/s -> FLOP/us

    def bytes_per_us(self) -> float:
        return self.hbm_gbs * 1e3 * self.efficiency  # GB/s -> B/us


_f32, _bf16, _f16, _f64 = torch.float32, torch.bfloat16, torch.float16, torch.float64

DEVICE_LIMITS = {
    # measured: 6.54 TB/s copy, 1352 TFLOP/s sustained bf16 (nominal 7.7 TB/s, 2250 TFLOP/s)
    "B200": DeviceLimit("B200", 6538.6, {_bf16: 1351.9, _f16: 1351.9, _f32: 75.0, _f64: 37.0}, 1.0, 3.0, 148, 180.0),
    "GB200": DeviceLimit("GB200", 6538.6, {_bf16: 1351.9, _f16: 1351.9, _f32: 75.0, _f64: 37.0}, 1.0, 3.0, 148, 186.0),
    "H200": DeviceLimit("H200", 4800.0, {_bf16: 989.0, _f16: 989.0, _f32: 67.0, _f64: 34.0}, 0.7, 5.0, 132, 141.0),
    "H100": DeviceLimit("H100", 3350.0, {_bf16: 989.0, _f16: 989.0, _f32: 67.0, _f64: 34.0}, 0.7, 5.0, 132, 80.0),
    "A100": DeviceLimit("A100", 1555.0, {_bf16: 312.0, _f16: 312.0, _f32: 19.5, _f64: 9.7}, 0.7, 7.0, 108, 80.0),
    "A10G": DeviceLimit("A10G", 600.0, {_bf16: 70.0, _f16: 70.0, _f32: 31.2, _f64: 0.5}, 0.7, 7.0, 80, 24.0),
    "V100": DeviceLimit("V100", 900.0, {_f16: 125.0, _bf16: 125.0, _f32: 15.7, _f64: 7.8}, 0.7, 7.0, 80, 32.0),
    "T4": DeviceLimit("T4", 300.0, {_f16: 65.0, _bf16: 65.0, _f32: 8.1, _f64: 0.25}, 0.7, 7.0, 40, 16.0),
    "A30": DeviceLimit("A30", 933.0, {_bf16: 165.0, _f16: 165.0, _f32: 10.3, _f64: 5.2}, 0.7, 7.0, 56, 24.0),
    "P100": DeviceLimit("P100", 732.0, {_f16: 21.2, _bf16: 21.2, _f32: 10.6, _f64: 5.3}, 0.7, 7.0, 56, 16.0),
    # planning only (the kernels of this package are sm_100a): nominal figures of other vendors' parts, so that a plan
    # can be made for them and compared
    "MI200X": DeviceLimit("MI200X", 3276.8, {_bf16: 383.0, _f16: 383.0, _f32: 47.9, _f64: 47.9}, 0.7, 7.0, 220, 128.0),
    "MI300X": DeviceLimit("MI300X", 5300.0, {_bf16: 1307.4, _f16: 1307.4, _f32: 163.4, _f64: 81.7}, 0.7, 7.0, 304, 192.0),
    "MI325X": DeviceLimit("MI325X", 6000.0, {_bf16: 1307.4, _f16: 1307.4, _f32: 163.4, _f64: 81.7}, 0.7, 7.0, 304, 256.0),
    "MI350X": DeviceLimit("MI350X", 8000.0, {_bf16: 2300.0, _f16: 2300.0, _f32: 144.2, _f64: 72.1}, 0.7, 7.0, 256, 288.0),
    "MI355X": DeviceLimit("MI355X", 8000.0, {_bf16: 2500.0, _f16: 2500.0, _f32: 157.3, _f64: 78.6}, 0.7, 7.0, 256, 288.0),
    "Max1550": DeviceLimit("Max1550", 3276.8, {_bf16: 832.0, _f16: 832.0, _f32: 52.0, _f64: 52.0}, 0.7, 7.0, 128, 128.0),
    "cpu": DeviceLimit("cpu", 100.0, {_f32: 2.0, _bf16: 2.0, _f16: 2.0, _f64: 1.0}, 0.7, 1.0, 0, 64.0),
}

_override: Optional[DeviceLimit] = None


def set_device_limit(limit: Optional[DeviceLimit]) -> None:
    """Force the device the planner prices for (e.g. plan for B200 on a CPU-only host)."""
    global _override
    _override = limit


def load_measured_peaks(path: str, base: str = "B200") -> DeviceLimit:
    """Build a limit from a measured-peaks JSON (keys ``hbm_gbs``, ``bf16_tflops_sustained``)."""
    with open(path) as f:
        m = json.load(f)
    b = DEVICE_LIMITS[base]
    tf = dict(b.tflops)
    tf[_bf16] = tf[_f16] = float(m.get("bf16_tflops_sustained", m.get("bf16_tflops", tf[_bf16])))
    return dataclasses.replace(b, hbm_gbs=float(m.get("hbm_gbs", b.hbm_gbs)), tflops=tf)


def get_device_limit(device_type: str = "cuda") -> DeviceLimit:
    if _override is not None:
        return _override
    env = os.environ.get("APB200_PLAN_DEVICE")
    if env:
        return DEVICE_LIMITS[env]
    if device_type == "cuda" and torch.cuda.is_available():
        name = torch.cuda.get_device_name(0)
        for key in ("GB200", "B200", "H200", "H100", "A100", "A10G", "A30", "V100", "P100", "T4",
                    "MI355X", "MI350X", "MI325X", "MI300X", "MI200X", "Max1550"):
            if key in name:
                return DEVICE_LIMITS[key]
        return DEVICE_LIMITS["A100"]
    if device_type == "cuda":
        return DEVICE_LIMITS["B200"]  # planning for the target machine from a GPU-less host
    return DEVICE_LIMITS["cpu"]
