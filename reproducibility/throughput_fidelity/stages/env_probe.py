"""What the study ran on: software versions, the device, its clocks and limits as found (read only), and the rates that
bound a step: device copy bandwidth, bf16 GEMM throughput (burst), host-to-device and device-to-host bandwidth from
pinned memory.  Without a device the probe records the host only."""
from __future__ import annotations

import json
import os
import platform
import subprocess

SMI_FIELDS = "name,driver_version,clocks.sm,clocks.max.sm,clocks.mem,power.draw,power.limit,temperature.gpu,clocks_event_reasons.active"


def smi_query(device: int) -> dict:
    """One read-only ``nvidia-smi --query-gpu`` sample; {} when the tool is missing."""
    try:
        out = subprocess.run(["nvidia-smi", f"--query-gpu={SMI_FIELDS}", "--format=csv,noheader,nounits", "-i", str(device)],
                             capture_output=True, text=True, timeout=20)
    except (OSError, subprocess.TimeoutExpired):
        return {}
    if out.returncode != 0 or not out.stdout.strip():
        return {}
    vals = [v.strip() for v in out.stdout.strip().splitlines()[0].split(",")]
    return dict(zip(SMI_FIELDS.split(","), vals))


def _timed(fn, reps: int) -> float:
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / reps


def env_probe(device: int | None, root: str) -> dict:
    import torch
    info = {"python": platform.python_version(), "torch": torch.__version__, "host": platform.node(), "cpus": os.cpu_count(),
            "device": "cpu"}
    try:
        import psutil
        info["host_memory_gib"] = psutil.virtual_memory().total / 2 ** 30
    except ImportError:
        pass
    if device is None or not torch.cuda.is_available():
        return info
    torch.cuda.set_device(device)
    p = torch.cuda.get_device_properties(device)
    info.update(device=p.name, sms=p.multi_processor_count, memory_gib=p.total_memory / 2 ** 30, cuda=torch.version.cuda,
                capability=f"{p.major}.{p.minor}", smi=smi_query(device))
    n = 1 << 28                                                   # 256 MiB: larger than the L2
    a = torch.empty(n, dtype=torch.uint8, device=device)
    b = torch.empty(n, dtype=torch.uint8, device=device)
    info["copy_gbs"] = 2 * n / _timed(lambda: b.copy_(a), 10) / 1e9
    m = 8192
    x = torch.randn(m, m, dtype=torch.bfloat16, device=device)
    y = torch.randn(m, m, dtype=torch.bfloat16, device=device)
    info["bf16_tflops_burst"] = 2 * m ** 3 / _timed(lambda: torch.mm(x, y), 10) / 1e12
    h = torch.empty(n, dtype=torch.uint8).pin_memory()
    info["h2d_gbs"] = n / _timed(lambda: a.copy_(h, non_blocking=True), 5) / 1e9
    info["d2h_gbs"] = n / _timed(lambda: h.copy_(a, non_blocking=True), 5) / 1e9
    peaks = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(peaks):
        with open(peaks) as f:
            info["measured_peaks"] = json.load(f)
    return info
