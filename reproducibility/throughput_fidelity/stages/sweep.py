"""Measure the selected cells, one at a time, each result appended to ``measure.jsonl`` as soon as it exists: a study that
is killed keeps what it measured, and ``--resume`` measures only the cells that are missing.  A cell that fails is a
row with its error, not the end of the sweep.  While a cell runs on a device the clocks are sampled (read only) and the
row carries the median SM clock and every throttle reason seen, so that a cell measured on a throttled device can be
recognised and measured again."""
from __future__ import annotations

import os
import subprocess
import threading
import time

from .common import append_jsonl, read_jsonl


class ClockSampler:
    """Samples ``nvidia-smi`` every ``period`` seconds on a thread; silent when the tool is missing."""
    FIELDS = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, device: int | None, period: float = 0.5):
        self.device, self.period = device, period
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._t: threading.Thread | None = None

    def __enter__(self):
        if self.device is not None:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()
        return self

    def _loop(self):
        while not self._stop.wait(self.period):
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.device)],
                                     capture_output=True, text=True, timeout=10)
            except (OSError, subprocess.TimeoutExpired):
                return
            if out.returncode == 0 and out.stdout.strip():
                self.samples.append([v.strip() for v in out.stdout.strip().splitlines()[0].split(",")])

    def __exit__(self, *exc):
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=15)
        return False

    def summary(self) -> dict:
        if not self.samples:
            return {}
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": int(self.samples[0][1]) if self.samples[0][1].isdigit() else None,
                "samples": len(self.samples), "reasons": reasons}


def sweep(out: str, cells: list[tuple], chosen: list[int], measure_cell, resume: bool) -> list[dict]:
    """``cells[i] = (opt, (family, cfg, budget))``; ``measure_cell(family, cfg, budget) -> row``."""
    path = os.path.join(out, "measure.jsonl")
    if not resume and os.path.exists(path):
        os.remove(path)
    done = {r["cell"]: r for r in read_jsonl(path) if "cell" in r and "error" not in r}
    rows = []
    for i in chosen:
        if i in done:
            print(f"[measure] cell {i} kept")
            rows.append(done[i])
            continue
        opt, (fam, cfg, budget) = cells[i]
        t0 = time.time()
        device = getattr(measure_cell, "device", None)
        try:
            with ClockSampler(device) as clocks:
                row = measure_cell(fam, cfg, budget)
            row.update(opt=opt, cell=i, wall_s=time.time() - t0)
            c = clocks.summary()
            if c:
                row["clocks"] = c
        except Exception as e:   # noqa: BLE001  (a cell that cannot run is a result of the study)
            row = {"cell": i, "opt": opt, "budget": budget, "seq": cfg.seq_len, "error": f"{type(e).__name__}: {str(e)[:300]}"}
        append_jsonl(path, row)
        rows.append(row)
        print(f"[measure] cell {i}: " + (f"ratio {row['ratio']:.3f}" if "ratio" in row else row.get("error", "")))
    return rows
