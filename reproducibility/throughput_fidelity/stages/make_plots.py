"""The study's figures as stand-alone SVG text (no plotting library): predicted against measured step time with the
diagonal and the +-10 % band; measured / predicted against the device budget, one series per geometry; tokens per second
against the budget, predicted and measured."""
from __future__ import annotations

import math

W, H, PAD = 640, 420, 56
COLORS = ["#4c8bf5", "#e5534b", "#57ab5a", "#d4a72c", "#986ee2", "#3fb6b2", "#e0823d", "#8b949e"]


def _axes(xlab: str, ylab: str, xt, yt, sx, sy, title: str) -> list[str]:
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" viewBox="0 0 {W} {H}" width="{W}" height="{H}" font-family="sans-serif" font-size="11">',
           f'<rect width="{W}" height="{H}" fill="#fff"/>', f'<text x="{W / 2}" y="18" text-anchor="middle" font-size="13">{title}</text>',
           f'<line x1="{PAD}" y1="{H - PAD}" x2="{W - 16}" y2="{H - PAD}" stroke="#333"/>', f'<line x1="{PAD}" y1="{H - PAD}" x2="{PAD}" y2="28" stroke="#333"/>',
           f'<text x="{W / 2}" y="{H - 12}" text-anchor="middle">{xlab}</text>',
           f'<text x="14" y="{H / 2}" text-anchor="middle" transform="rotate(-90 14 {H / 2})">{ylab}</text>']
    for v in xt:
        out.append(f'<line x1="{sx(v):.1f}" y1="{H - PAD}" x2="{sx(v):.1f}" y2="{H - PAD + 4}" stroke="#333"/><text x="{sx(v):.1f}" y="{H - PAD + 16}" text-anchor="middle">{v:g}</text>')
    for v in yt:
        out.append(f'<line x1="{PAD - 4}" y1="{sy(v):.1f}" x2="{PAD}" y2="{sy(v):.1f}" stroke="#333"/><text x="{PAD - 7}" y="{sy(v) + 4:.1f}" text-anchor="end">{v:g}</text>'
                   f'<line x1="{PAD}" y1="{sy(v):.1f}" x2="{W - 16}" y2="{sy(v):.1f}" stroke="#eee"/>')
    return out


def _ticks(lo: float, hi: float, n: int = 5) -> list[float]:
    if hi <= lo:
        hi = lo + 1.0
    step = 10 ** math.floor(math.log10((hi - lo) / n))
    for m in (1, 2, 5, 10):
        if (hi - lo) / (step * m) <= n:
            step *= m
            break
    first = math.ceil(lo / step) * step
    return [round(first + i * step, 10) for i in range(int((hi - first) / step) + 1)]


def _scales(xs, ys, pad_frac: float = 0.06):
    x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
    dx, dy = (x1 - x0) or 1.0, (y1 - y0) or 1.0
    x0, x1, y0, y1 = x0 - dx * pad_frac, x1 + dx * pad_frac, y0 - dy * pad_frac, y1 + dy * pad_frac
    sx = lambda v: PAD + (v - x0) / (x1 - x0) * (W - 16 - PAD)       # noqa: E731
    sy = lambda v: H - PAD - (v - y0) / (y1 - y0) * (H - PAD - 28)   # noqa: E731
    return sx, sy, (x0, x1), (y0, y1)


def scatter_pred_vs_meas(meas: list[dict]) -> str:
    pts = [(m["pred_s"], m["meas_s"], m.get("cell")) for m in meas if "ratio" in m]
    if not pts:
        return ""
    lo, hi = min(min(p[0], p[1]) for p in pts), max(max(p[0], p[1]) for p in pts)
    sx, sy, (x0, x1), _ = _scales([lo, hi], [lo, hi])
    sy2 = lambda v: H - PAD - (v - x0) / (x1 - x0) * (H - PAD - 28)     # the same scale on both axes  # noqa: E731
    out = _axes("predicted step time, s", "measured step time, s", _ticks(x0, x1), _ticks(x0, x1), sx, sy2, "Predicted against measured")
    band = " ".join(f"{sx(v):.1f},{sy2(v * 1.1):.1f}" for v in (x0, x1)) + " " + " ".join(f"{sx(v):.1f},{sy2(v * 0.9):.1f}" for v in (x1, x0))
    out.append(f'<polygon points="{band}" fill="#4c8bf5" fill-opacity="0.12"/>')
    out.append(f'<line x1="{sx(x0):.1f}" y1="{sy2(x0):.1f}" x2="{sx(x1):.1f}" y2="{sy2(x1):.1f}" stroke="#333" stroke-dasharray="5 4"/>')
    for p, m, c in pts:
        out.append(f'<circle cx="{sx(p):.1f}" cy="{sy2(m):.1f}" r="4" fill="#e5534b"><title>cell {c}: predicted {p:.4f} s, measured {m:.4f} s</title></circle>')
    return "\n".join(out) + "\n</svg>\n"


def _series(meas: list[dict], ykey, ylab: str, title: str, extra=None) -> str:
    good = [m for m in meas if "ratio" in m and m.get("budget") is not None]
    if not good:
        return ""
    groups: dict = {}
    for m in good:
        groups.setdefault((m.get("opt"), m["seq"], m["t_round"], m["rounds"]), []).append(m)
    xs = [m["budget"] for m in good]
    ys = [ykey(m) for m in good] + ([extra(m) for m in good] if extra else [])
    sx, sy, xr, yr = _scales(xs, ys)
    out = _axes("device budget, GiB", ylab, _ticks(*xr), _ticks(*yr), sx, sy, title)
    for gi, (key, rows) in enumerate(sorted(groups.items(), key=str)):
        rows.sort(key=lambda m: m["budget"])
        col = COLORS[gi % len(COLORS)]
        out.append(f'<polyline fill="none" stroke="{col}" stroke-width="1.5" points="' + " ".join(f"{sx(m['budget']):.1f},{sy(ykey(m)):.1f}" for m in rows) + '"/>')
        if extra:
            out.append(f'<polyline fill="none" stroke="{col}" stroke-width="1" stroke-dasharray="4 3" points="' + " ".join(f"{sx(m['budget']):.1f},{sy(extra(m)):.1f}" for m in rows) + '"/>')
        for m in rows:
            out.append(f'<circle cx="{sx(m["budget"]):.1f}" cy="{sy(ykey(m)):.1f}" r="3" fill="{col}"><title>{key}: {ykey(m):.4g} at {m["budget"]} GiB</title></circle>')
        out.append(f'<text x="{W - 20}" y="{40 + 14 * gi}" text-anchor="end" fill="{col}">{key[0]} seq {key[1]} x {key[2]} x {key[3]}</text>')
    return "\n".join(out) + "\n</svg>\n"


def ratio_by_budget(meas: list[dict]) -> str:
    return _series(meas, lambda m: m["ratio"], "measured / predicted", "Fidelity against the device budget")


def throughput_by_budget(meas: list[dict]) -> str:
    return _series(meas, lambda m: m["tok_s"], "tokens / s (solid: measured, dashed: predicted)", "Throughput against the device budget",
                   extra=lambda m: m["tok_s"] * m["ratio"])


def make_plots(meas: list[dict]) -> dict[str, str]:
    plots = {"pred_vs_meas.svg": scatter_pred_vs_meas(meas), "ratio_by_budget.svg": ratio_by_budget(meas),
             "throughput_by_budget.svg": throughput_by_budget(meas)}
    return {k: v for k, v in plots.items() if v}
