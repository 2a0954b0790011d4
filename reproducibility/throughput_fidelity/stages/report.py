"""``report.md`` (tables) and ``report.html`` (the same with the figures inline) from the stages' results."""
from __future__ import annotations

import html


def _env_lines(env: dict) -> list[str]:
    if not env:
        return []
    bits = [f"device `{env.get('device')}`", f"torch {env.get('torch')}", f"python {env.get('python')}"]
    for k, unit in (("copy_gbs", "GB/s device copy"), ("bf16_tflops_burst", "TFLOP/s bf16 GEMM (burst)"), ("h2d_gbs", "GB/s host to device"),
                    ("d2h_gbs", "GB/s device to host")):
        if env.get(k):
            bits.append(f"{env[k]:.1f} {unit}")
    smi = env.get("smi") or {}
    if smi:
        bits.append(f"SM clock {smi.get('clocks.sm')} of {smi.get('clocks.max.sm')} MHz, power {smi.get('power.draw')} of {smi.get('power.limit')} W, "
                    f"reasons {smi.get('clocks_event_reasons.active')}")
    return ["Environment: " + "; ".join(bits) + ".", ""]


def report_md(preset: str, env: dict, pred: list[dict], meas: list[dict], ana: dict) -> str:
    lines = ["# Throughput fidelity", ""]
    lines += _env_lines(env)
    if ana.get("cells"):
        w = ana["worst"]
        lines += [f"preset `{preset}`, {ana['cells']} measured cells of {len(pred)} predicted ({ana['failed']} failed); "
                  f"geometric mean measured / predicted = {ana['geomean_ratio']:.3f}; median {ana['median_ratio']:.3f}, "
                  f"10th-90th percentile {ana['p10_ratio']:.3f}-{ana['p90_ratio']:.3f}; {100 * ana['within_5pct']:.0f} % of cells within 5 %, "
                  f"{100 * ana['within_10pct']:.0f} % within 10 %; worst cell {w['ratio']:.3f} (budget {w['budget']}).", ""]
    else:
        lines += [f"preset `{preset}`: no cell was measured ({ana.get('failed', 0)} failed).", ""]
    lines += ["| opt | seq | t_round | rounds | budget GiB | predicted s | measured s | ratio | tok/s | recompute % | replay gap % | SM MHz | throttle |",
              "|---|---|---|---|---|---|---|---|---|---|---|---|---|"]
    for r in meas:
        if "error" in r:
            lines.append(f"| {r.get('opt')} | {r.get('seq')} | | | {r.get('budget')} | | | failed: {r['error'][:80]} | | | | | |")
            continue
        c = r.get("clocks") or {}
        lines.append(f"| {r['opt']} | {r['seq']} | {r['t_round']} | {r['rounds']} | {r['budget']} | {r['pred_s']:.4f} | {r['meas_s']:.4f} | "
                     f"{r['ratio']:.3f} | {r['tok_s']:.0f} | {r['recomp_pct']:.1f} | {r.get('replay_gap_pct', 0.0):.1f} | {c.get('sm_mhz', '')} | "
                     f"{', '.join(c.get('reasons', []))} |")
    for axis, groups in (ana.get("by_axis") or {}).items():
        if len(groups) < 2:
            continue
        lines += ["", f"By {axis.replace('_', ' ')}:", "", "| value | cells | geometric mean ratio | worst |", "|---|---|---|---|"]
        lines += [f"| {k} | {g['cells']} | {g['geomean_ratio']:.3f} | {g['worst']:.3f} |" for k, g in groups.items()]
    if ana.get("off_by_more_than_10pct"):
        lines += ["", "Cells off by more than 10 %:", "", "| cell | budget GiB | ratio | what the measurement says |", "|---|---|---|---|"]
        lines += [f"| {o['cell']} | {o['budget']} | {o['ratio']:.3f} | {o['why']} |" for o in ana["off_by_more_than_10pct"]]
    infeasible = [r for r in pred if not r.get("s_step")]
    if infeasible:
        lines += ["", f"{len(infeasible)} predicted cells had no plan (budget too small for the geometry)."]
    return "\n".join(lines) + "\n"


def report_html(md: str, plots: dict[str, str]) -> str:
    body = []
    in_table = False
    for line in md.splitlines():
        if line.startswith("|"):
            cells = [c.strip() for c in line.strip("|").split("|")]
            if set(line) <= set("|-: "):
                continue
            if not in_table:
                body.append("<table>")
                in_table = True
                body.append("<tr>" + "".join(f"<th>{html.escape(c)}</th>" for c in cells) + "</tr>")
            else:
                body.append("<tr>" + "".join(f"<td>{html.escape(c)}</td>" for c in cells) + "</tr>")
            continue
        if in_table:
            body.append("</table>")
            in_table = False
        if line.startswith("# "):
            body.append(f"<h1>{html.escape(line[2:])}</h1>")
        elif line.strip():
            body.append(f"<p>{html.escape(line)}</p>")
    if in_table:
        body.append("</table>")
    figs = "".join(f"<figure>{svg}<figcaption>{html.escape(name)}</figcaption></figure>" for name, svg in plots.items())
    style = "body{font:14px/1.45 sans-serif;max-width:1100px;margin:24px auto}table{border-collapse:collapse}td,th{border:1px solid #ccc;padding:3px 8px;text-align:right}"
    return f"<!doctype html><html><head><meta charset='utf-8'><title>Throughput fidelity</title><style>{style}</style></head><body>" + \
        "\n".join(body) + figs + "</body></html>\n"
