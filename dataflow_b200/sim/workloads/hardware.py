"""Hardware rows for the analytic workload compiler.

A row prices a hardware-free cost term: peak tensor throughput per dtype times an efficiency, memory bandwidth for
elementwise work, per-direction scale-up (NVLink) bandwidth for collectives, and the two host-link lanes that the
simulator's ``from_slow`` / ``to_slow`` tracks model.  Same role as the reference's
``src/dataflow_sim/workloads/common/hardware.py:6-97`` (H100, GB300, RTX 5090, SRAM accelerator); the B200 row carries
bandwidth and GEMM throughput measured on this hardware instead of data-sheet peaks.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field


@dataclass(frozen=True)
class HardwareSpec:
    name: str
    peak_tflops: dict = field(default_factory=dict)          # dtype -> dense TFLOP/s
    matmul_efficiency: float = 0.75
    attention_efficiency: float = 0.45
    hbm_gbs: float = 3000.0
    memory_efficiency: float = 0.85
    from_slow_gbs: float = 50.0
    to_slow_gbs: float = 50.0
    scale_up_bw_gbs: float = 0.0
    fast_memory_gib: float = 80.0
    launch_us: float = 4.0                                    # fixed cost added per sub-op

    def tflops(self, dtype: str) -> float:
        if dtype in self.peak_tflops:
            return float(self.peak_tflops[dtype])
        if dtype.startswith("fp8") and "fp8" in self.peak_tflops:
            return float(self.peak_tflops["fp8"])
        return float(self.peak_tflops.get("bf16", 1.0))

    def to_dict(self) -> dict:
        return asdict(self)


HARDWARE_PRESETS: dict[str, HardwareSpec] = {
    "B200": HardwareSpec("B200", {"bf16": 1669.0, "fp16": 1669.0, "fp8": 3300.0, "fp4": 6600.0, "tf32": 830.0, "fp32": 75.0},
                         0.84, 0.45, 6524.0, 0.90, 52.0, 52.0, 770.0, 180.0, 3.0),
    "H100": HardwareSpec("H100", {"bf16": 989.0, "fp16": 989.0, "fp8": 1979.0, "tf32": 494.0, "fp32": 67.0},
                         0.72, 0.55, 3350.0, 0.85, 52.0, 50.0, 450.0, 80.0, 4.0),
    "GB300": HardwareSpec("GB300", {"bf16": 2500.0, "fp16": 2500.0, "fp8": 5000.0, "fp4": 15000.0, "tf32": 1250.0, "fp32": 80.0},
                          0.78, 0.45, 8000.0, 0.88, 200.0, 200.0, 900.0, 288.0, 3.0),
    "RTX_5090": HardwareSpec("RTX_5090", {"bf16": 210.0, "fp16": 210.0, "fp8": 420.0, "fp4": 840.0, "tf32": 105.0, "fp32": 105.0},
                             0.70, 0.45, 1792.0, 0.85, 52.0, 52.0, 0.0, 32.0, 4.0),
    "SRAM_ACCELERATOR": HardwareSpec("SRAM_ACCELERATOR", {"bf16": 750.0, "fp16": 750.0, "fp8": 1500.0},
                                     0.80, 0.60, 80000.0, 0.90, 300.0, 300.0, 100.0, 0.22, 1.0),
}


def get_hardware(name: str) -> HardwareSpec:
    key = name.upper().replace("-", "_").replace(" ", "_")
    for k, v in HARDWARE_PRESETS.items():
        if k.upper() == key:
            return v
    raise KeyError(f"unknown hardware preset {name!r}; known: {sorted(HARDWARE_PRESETS)}")
