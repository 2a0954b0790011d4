#!/usr/bin/env python
"""Was the device throttled while something ran?  Samples clocks, power and throttle reasons (read only) while ``--``
``command`` runs, or summarises a ``clocks.csv`` recorded earlier (the format of ``nvidia-smi --query-gpu=... --format=csv
-lms``), and says whether a measurement taken in that window can be trusted: hardware or thermal slowdown rejects it, a
power cap is noted, an SM clock stuck far below its maximum with no reason given points at a clock lock left by someone else.

    python reproducibility/throughput_fidelity/diagnostics/throttle_probe.py --device 0 -- python bench.py --steps 3
    python reproducibility/throughput_fidelity/diagnostics/throttle_probe.py --csv clocks.csv
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import subprocess
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

BAD = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")


def verdict(sm_mhz: list[int], sm_max: int | None, reasons: set[str]) -> dict:
    sm_mhz = sorted(sm_mhz)
    med = sm_mhz[len(sm_mhz) // 2] if sm_mhz else None
    out = {"samples": len(sm_mhz), "sm_mhz_median": med, "sm_mhz_min": sm_mhz[0] if sm_mhz else None, "sm_max_mhz": sm_max,
           "reasons": sorted(reasons)}
    if any(r in reasons for r in BAD):
        out.update(ok=False, why="slowdown active: " + ", ".join(r for r in BAD if r in reasons))
    elif med is not None and sm_max and med < 0.6 * sm_max and not reasons:
        out.update(ok=False, why=f"SM clock {med} MHz of {sm_max} with no reason given: a clock lock left on the device?")
    else:
        out.update(ok=True, why="power cap active (normal under dense load)" if "sw_power_cap" in reasons else "no throttling seen")
    return out


def from_csv(path: str) -> dict:
    mhz, reasons, sm_max = [], set(), None
    with open(path, newline="") as f:
        rows = list(csv.reader(f))
    if not rows:
        return verdict([], None, set())
    head = [h.strip().split(" ")[0] for h in rows[0]]
    col = {h: i for i, h in enumerate(head)}
    for r in rows[1:]:
        r = [c.strip() for c in r]
        try:
            mhz.append(int(r[col["clocks.sm"]].split()[0]))
            sm_max = int(r[col["clocks.max.sm"]].split()[0])
        except (KeyError, ValueError, IndexError):
            continue
        for name in BAD + ("sw_power_cap",):
            i = col.get("clocks_event_reasons." + name)
            if i is not None and i < len(r) and r[i].lower().startswith("active"):
                reasons.add(name)
    return verdict(mhz, sm_max, reasons)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="0")
    ap.add_argument("--csv", default=None)
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    if a.csv:
        res = from_csv(a.csv)
    else:
        from stages.sweep import ClockSampler
        cmd = [c for c in a.command if c != "--"]
        if not cmd:
            ap.error("give --csv FILE or a command after --")
        with ClockSampler(None if a.device == "cpu" else int(a.device), period=0.2) as clocks:
            rc = subprocess.call(cmd)
        s = clocks.summary()
        res = verdict([int(x[0]) for x in clocks.samples if x[0].isdigit()], s.get("sm_max_mhz"), set(s.get("reasons", [])))
        res["command_exit"] = rc
    print(json.dumps(res))
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
