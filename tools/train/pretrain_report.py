"""Report on one or more training runs from their result files (``train.py ... --out run.json``).

Text (always): per run the first / final / best loss, the loss at fixed shares of the run, tokens/s (median of the steady
steps), step-time percentiles, the slowest steps, and a coarse plot of the curve.
HTML (``--html report.html``): the same table plus figures as inline SVG: loss against tokens for every run on one plot (raw
and exponentially smoothed), tokens/s against step, step-time histogram; and, when two runs are given with ``--band``, where
the second leaves a relative band around the first (the way two precisions or two budgets of one recipe are compared).
Checkpoint evaluations written by ``eval_checkpoint.py --json`` can be added with ``--evals`` and appear as points.

    python tools/train/pretrain_report.py run_a.json run_b.json --html report.html --band 0.02

Reference role: ``tools/train/pretrain_report.py`` (HTML study reports with inline SVG).
"""
from __future__ import annotations

import argparse
import html
import json
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402

COLORS = ["#4c8bf5", "#e5534b", "#57ab5a", "#d4a72c", "#986ee2", "#3fb6b2", "#e0823d", "#8b949e"]


def spark(values, width=48):
    values = [v for v in values if math.isfinite(v)]
    if not values:
        return ""
    bars = " .:-=+*#%@"
    step = max(len(values) // width, 1)
    pts = [sum(values[i:i + step]) / len(values[i:i + step]) for i in range(0, len(values), step)]
    lo, hi = min(pts), max(pts)
    return "".join(bars[int((v - lo) / (hi - lo + 1e-12) * (len(bars) - 1))] for v in pts)


def ema(values, alpha: float = 0.1):
    out, m = [], None
    for v in values:
        m = v if m is None else (1 - alpha) * m + alpha * v
        out.append(m)
    return out


def load_run(path: str, warmup: int) -> dict:
    with open(path) as f:
        d = json.load(f)
    losses = list(d.get("losses") or d.get("curve") or [])
    times = list(d.get("step_wall_s") or d.get("step_s") or [])
    tok = d.get("tokens_per_step") or 0
    steady = sorted(times[warmup:]) or sorted(times)
    q = lambda p: steady[min(int(len(steady) * p), len(steady) - 1)] if steady else None   # noqa: E731
    slow = sorted(((t, i + 1) for i, t in enumerate(times)), reverse=True)[:3]
    meta = d.get("meta") or {}
    return {"run": os.path.basename(path), "steps": len(losses), "losses": losses, "times": times, "tokens_per_step": tok,
            "first": losses[0] if losses else None, "final": losses[-1] if losses else None, "best": min((v for v in losses if math.isfinite(v)), default=None),
            "at_25": losses[len(losses) // 4] if losses else None, "at_50": losses[len(losses) // 2] if losses else None,
            "s_step_p50": q(0.5), "s_step_p90": q(0.9), "s_step_max": steady[-1] if steady else None,
            "tok_s": tok / q(0.5) if steady and tok else None, "slowest": [f"step {i}: {t:.3f} s" for t, i in slow],
            "tokens_total": tok * len(losses), "curve": spark(losses), "preset": meta.get("preset", ""), "world": meta.get("world", 1),
            "policy": meta.get("policy", ""), "non_finite": sum(1 for v in losses if not math.isfinite(v))}


def band_report(a: dict, b: dict, band: float) -> dict:
    """Where run ``b`` leaves the relative band around run ``a`` (smoothed curves, common steps)."""
    n = min(len(a["losses"]), len(b["losses"]))
    if n == 0:
        return {"steps": 0}
    sa, sb = ema(a["losses"][:n]), ema(b["losses"][:n])
    rel = [abs(y - x) / max(abs(x), 1e-12) for x, y in zip(sa, sb)]
    out = [i + 1 for i, r in enumerate(rel) if r > band]
    return {"steps": n, "band": band, "max_rel": max(rel), "at_step": rel.index(max(rel)) + 1, "final_rel": rel[-1], "steps_outside": len(out),
            "first_outside": out[0] if out else None, "within": not out}


# ------------------------------------------------------------------------------------------------------------------- figures
def _frame(w, h, pad, title, xlab, ylab, x0, x1, y0, y1):
    sx = lambda v: pad + (v - x0) / ((x1 - x0) or 1.0) * (w - pad - 16)      # noqa: E731
    sy = lambda v: h - pad - (v - y0) / ((y1 - y0) or 1.0) * (h - pad - 28)  # noqa: E731
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" viewBox="0 0 {w} {h}" width="{w}" height="{h}" font-family="sans-serif" font-size="11">',
           f'<rect width="{w}" height="{h}" fill="#fff"/><text x="{w / 2}" y="16" text-anchor="middle" font-size="13">{html.escape(title)}</text>',
           f'<line x1="{pad}" y1="{h - pad}" x2="{w - 16}" y2="{h - pad}" stroke="#333"/><line x1="{pad}" y1="{h - pad}" x2="{pad}" y2="28" stroke="#333"/>',
           f'<text x="{w / 2}" y="{h - 10}" text-anchor="middle">{html.escape(xlab)}</text>',
           f'<text x="12" y="{h / 2}" text-anchor="middle" transform="rotate(-90 12 {h / 2})">{html.escape(ylab)}</text>']
    for k in range(5):
        xv, yv = x0 + (x1 - x0) * k / 4, y0 + (y1 - y0) * k / 4
        out.append(f'<text x="{sx(xv):.1f}" y="{h - pad + 14}" text-anchor="middle">{xv:.4g}</text>'
                   f'<text x="{pad - 5}" y="{sy(yv) + 4:.1f}" text-anchor="end">{yv:.4g}</text>'
                   f'<line x1="{pad}" y1="{sy(yv):.1f}" x2="{w - 16}" y2="{sy(yv):.1f}" stroke="#eee"/>')
    return out, sx, sy


def loss_figure(runs: list[dict], evals: list[dict]) -> str:
    pts = [(r["tokens_per_step"] * (i + 1) or (i + 1), v) for r in runs for i, v in enumerate(r["losses"]) if math.isfinite(v)]
    if not pts:
        return ""
    xs, ys = [p[0] for p in pts], [p[1] for p in pts]
    unit = "tokens" if all(r["tokens_per_step"] for r in runs) else "step"
    out, sx, sy = _frame(720, 420, 56, "Training loss", unit, "loss", 0, max(xs), min(ys) - 0.02 * (max(ys) - min(ys) or 1), max(ys))
    for k, r in enumerate(runs):
        col = COLORS[k % len(COLORS)]
        step = r["tokens_per_step"] or 1
        raw = [(step * (i + 1), v) for i, v in enumerate(r["losses"]) if math.isfinite(v)]
        sm = list(zip([p[0] for p in raw], ema([p[1] for p in raw])))
        out.append(f'<polyline fill="none" stroke="{col}" stroke-opacity="0.3" stroke-width="1" points="' + " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in raw) + '"/>')
        out.append(f'<polyline fill="none" stroke="{col}" stroke-width="1.6" points="' + " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in sm) + '"/>')
        out.append(f'<text x="700" y="{40 + 14 * k}" text-anchor="end" fill="{col}">{html.escape(r["run"])}</text>')
    for e in evals:
        x = e.get("tokens_seen") or e.get("checkpoint", 0) * (runs[0]["tokens_per_step"] or 1)
        if e.get("loss") is not None and math.isfinite(e["loss"]):
            out.append(f'<circle cx="{sx(x):.1f}" cy="{sy(e["loss"]):.1f}" r="4" fill="none" stroke="#1b1f24"><title>held-out loss {e["loss"]:.4f} at checkpoint {e.get("checkpoint")}</title></circle>')
    return "\n".join(out) + "\n</svg>"


def throughput_figure(runs: list[dict], warmup: int) -> str:
    series = [(r, [r["tokens_per_step"] / t if r["tokens_per_step"] else 1.0 / t for t in r["times"] if t > 0]) for r in runs if r["times"]]
    if not series:
        return ""
    top = max(max(s[warmup:] or s) for _, s in series)
    n = max(len(s) for _, s in series)
    out, sx, sy = _frame(720, 300, 56, "Throughput per step", "step", "tokens / s" if runs[0]["tokens_per_step"] else "steps / s", 1, max(n, 2), 0, top * 1.05)
    for k, (r, s) in enumerate(series):
        out.append(f'<polyline fill="none" stroke="{COLORS[k % len(COLORS)]}" stroke-width="1.2" points="' +
                   " ".join(f"{sx(i + 1):.1f},{sy(min(v, top * 1.05)):.1f}" for i, v in enumerate(s)) + '"/>')
    return "\n".join(out) + "\n</svg>"


def step_time_histogram(runs: list[dict], warmup: int, bins: int = 24) -> str:
    ts = [t for r in runs for t in r["times"][warmup:]]
    if len(ts) < 2:
        return ""
    lo, hi = min(ts), max(ts)
    hi = hi if hi > lo else lo + 1e-9
    out, sx, sy = _frame(720, 260, 56, "Step time after warm-up", "seconds", "steps", lo, hi, 0, 1)
    width = (720 - 56 - 16) / bins / max(len(runs), 1)
    tallest = 1
    counts = []
    for r in runs:
        c = [0] * bins
        for t in r["times"][warmup:]:
            c[min(int((t - lo) / (hi - lo) * bins), bins - 1)] += 1
        counts.append(c)
        tallest = max(tallest, max(c))
    for k, c in enumerate(counts):
        for b, v in enumerate(c):
            if v:
                x = sx(lo + (hi - lo) * b / bins) + k * width
                out.append(f'<rect x="{x:.1f}" y="{sy(v / tallest):.1f}" width="{max(width - 1, 1):.1f}" height="{sy(0) - sy(v / tallest):.1f}" fill="{COLORS[k % len(COLORS)]}"><title>{v} steps</title></rect>')
    return "\n".join(out) + "\n</svg>"


def render_html(runs: list[dict], band: dict | None, evals: list[dict], warmup: int) -> str:
    head = ["run", "preset", "ranks", "steps", "tokens", "first", "25 %", "50 %", "final", "best", "s/step p50", "p90", "max", "tokens/s", "planner"]
    fmt = lambda v, f="{:.4f}": "-" if v is None else f.format(v)      # noqa: E731
    body = ["<tr>" + "".join(f"<th>{h}</th>" for h in head) + "</tr>"]
    for r in runs:
        cells = [r["run"], r["preset"], r["world"], r["steps"], f"{r['tokens_total']:,}", fmt(r["first"]), fmt(r["at_25"]), fmt(r["at_50"]), fmt(r["final"]),
                 fmt(r["best"]), fmt(r["s_step_p50"]), fmt(r["s_step_p90"]), fmt(r["s_step_max"]), fmt(r["tok_s"], "{:,.0f}"), r["policy"]]
        body.append("<tr>" + "".join(f"<td>{html.escape(str(c))}</td>" for c in cells) + "</tr>")
    notes = []
    for r in runs:
        if r["non_finite"]:
            notes.append(f"<p><b>{html.escape(r['run'])}: {r['non_finite']} steps with a non-finite loss.</b></p>")
        if r["slowest"]:
            notes.append(f"<p>{html.escape(r['run'])}, slowest steps: {html.escape(', '.join(r['slowest']))}</p>")
    if band and band.get("steps"):
        verdict = "stays inside" if band["within"] else f"leaves it at step {band['first_outside']} ({band['steps_outside']} steps outside)"
        notes.append(f"<p>Band of {100 * band['band']:.1f} % around <i>{html.escape(runs[0]['run'])}</i>: <i>{html.escape(runs[1]['run'])}</i> {verdict}; "
                     f"largest relative distance {band['max_rel']:.2e} at step {band['at_step']}, final {band['final_rel']:.2e} (smoothed curves, {band['steps']} common steps).</p>")
    figs = [f for f in (loss_figure(runs, evals), throughput_figure(runs, warmup), step_time_histogram(runs, warmup)) if f]
    style = "body{font:14px/1.45 sans-serif;max-width:1200px;margin:24px auto}table{border-collapse:collapse}td,th{border:1px solid #ccc;padding:3px 8px;text-align:right}td:first-child{text-align:left}"
    return (f"<!doctype html><html><head><meta charset='utf-8'><title>Training report</title><style>{style}</style></head><body><h1>Training report</h1>"
            f"<table>{''.join(body)}</table>{''.join(notes)}{''.join(f'<figure>{f}</figure>' for f in figs)}</body></html>\n")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("runs", nargs="+")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--html", default=None, help="write an HTML report with inline figures here")
    ap.add_argument("--band", type=float, default=None, help="relative band around the first run that the second must stay in")
    ap.add_argument("--evals", nargs="*", default=[], help="JSON lines of eval_checkpoint.py (held-out loss per checkpoint)")
    a = ap.parse_args(argv)
    runs = [load_run(p, a.warmup) for p in a.runs]
    print(table(runs, [("run", "{}"), ("steps", "{}"), ("first", "{:.4f}"), ("at_50", "{:.4f}"), ("final", "{:.4f}"), ("best", "{:.4f}"), ("s_step_p50", "{:.4f}"),
                       ("s_step_p90", "{:.4f}"), ("tok_s", "{:.0f}"), ("curve", "{}")]))
    band = None
    if a.band is not None and len(runs) >= 2:
        band = band_report(runs[0], runs[1], a.band)
        if band.get("steps"):
            print(f"band {100 * a.band:.1f} %: max relative distance {band['max_rel']:.2e} at step {band['at_step']}; "
                  + ("inside" if band["within"] else f"outside from step {band['first_outside']}"))
    evals = []
    for p in a.evals:
        with open(p) as f:
            for line in f:
                line = line.strip()
                if line.startswith("{"):
                    evals.append(json.loads(line))
    if a.html:
        with open(a.html, "w") as f:
            f.write(render_html(runs, band, evals, a.warmup))
        print(f"wrote {a.html}")
    return 0 if band is None or not band.get("steps") or band["within"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
