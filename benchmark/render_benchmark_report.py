#!/usr/bin/env python3
"""Render ``results.json`` of the experiment suite as one self-contained HTML page.

One chart per experiment group; one line per ``method | A=.. B=.. C=.. | rep=..`` series with
x = the varied dimension and y = median TFLOP/s; an optional dashed "theoretical max" line;
check boxes to show / hide methods and experiment groups; a table of all rows.  Input schema
and grouping are those of the reference's renderer (benchmark/render_benchmark_report.py:21-117);
the charts are drawn as inline SVG by a few lines of script, so the page also works without
network access (the reference loads Plotly from a CDN).
"""
from __future__ import annotations

import argparse
import html
import json
import pathlib
from typing import Any

PALETTE = ["#2563eb", "#dc2626", "#059669", "#d97706", "#7c3aed", "#0891b2", "#be185d", "#4d7c0f", "#475569",
           "#ea580c", "#0d9488", "#9333ea"]


def load_results(path: pathlib.Path) -> dict[str, Any]:
    payload = json.loads(path.read_text(encoding="utf-8"))
    if "results" not in payload:
        raise ValueError(f"Expected 'results' in {path}")
    return payload


def series_name(row: dict[str, Any]) -> str:
    return (f"{row['method']} | A={row['a_partition']} B={row['b_partition']} C={row['c_partition']} | "
            f"rep={row['replication_factor']}")


def group_rows(rows: list[dict[str, Any]]) -> dict[str, dict[str, Any]]:
    groups: dict[str, dict[str, Any]] = {}
    for row in rows:
        g = groups.setdefault(row["experiment_group"], {
            "experiment_group": row["experiment_group"], "experiment_label": row["experiment_label"],
            "varied_dim": row["varied_dim"], "series": {}, "theoretical_tflops": row.get("theoretical_tflops")})
        g["series"].setdefault(series_name(row), []).append(row)
        if g["theoretical_tflops"] is None and row.get("theoretical_tflops") is not None:
            g["theoretical_tflops"] = row["theoretical_tflops"]
    for g in groups.values():
        for name in g["series"]:
            g["series"][name].sort(key=lambda r: r["varied_value"])
    return groups


def build_plots(groups: dict[str, dict[str, Any]], methods: set[str] | None, only_groups: set[str] | None) -> list[dict]:
    plots = []
    for key in sorted(groups):
        if only_groups and key not in only_groups:
            continue
        g = groups[key]
        traces, xs_all = [], set()
        for name, rows in g["series"].items():
            method = name.split("|", 1)[0].strip()
            if methods and method not in methods:
                continue
            xs = [int(r["varied_value"]) for r in rows]
            xs_all.update(xs)
            traces.append({"name": name, "x": xs, "y": [float(r["median_tflops"]) for r in rows],
                           "meta": {"method": method, "kind": "series"}})
        if not traces:
            continue
        theo = g.get("theoretical_tflops")
        if theo is not None and xs_all:
            xs = sorted(xs_all)
            traces.append({"name": f"Theoretical max ({float(theo):.2f} TFLOPs)", "x": xs, "y": [float(theo)] * len(xs),
                           "meta": {"method": "theoretical", "kind": "theoretical"}})
        plots.append({"id": key, "title": g["experiment_label"], "x_title": f"Varied {g['varied_dim']}",
                      "y_title": "Achieved TFLOPs (median)", "traces": traces})
    return plots


_SCRIPT = r"""
const PAL = __PALETTE__;
const plots = __PLOTS__;
const root = document.getElementById('plots-root');
const expBox = document.getElementById('experiment-toggles');
function enabledMethods() {
  return new Set(Array.from(document.querySelectorAll('.method-toggle')).filter(x => x.checked).map(x => x.value));
}
function draw(p, host) {
  const W = 900, H = 420, L = 70, R = 20, T = 16, B = 56;
  const on = enabledMethods();
  const tr = p.traces.filter(t => t.meta.kind === 'theoretical' || on.has(t.meta.method));
  const xs = [...new Set(tr.flatMap(t => t.x))].sort((a, b) => a - b);
  const ymax = Math.max(1e-9, ...tr.flatMap(t => t.y)) * 1.08;
  const xpos = v => L + (xs.length < 2 ? 0.5 : xs.indexOf(v) / (xs.length - 1)) * (W - L - R);
  const ypos = v => H - B - (v / ymax) * (H - T - B);
  let s = `<svg viewBox="0 0 ${W} ${H}" class="plot">`;
  for (let i = 0; i <= 5; i++) {
    const v = ymax * i / 5, y = ypos(v);
    s += `<line x1="${L}" x2="${W - R}" y1="${y}" y2="${y}" stroke="#e2e8f0"/>`;
    s += `<text x="${L - 8}" y="${y + 4}" text-anchor="end" font-size="11">${v.toFixed(v < 10 ? 2 : 0)}</text>`;
  }
  for (const v of xs) s += `<text x="${xpos(v)}" y="${H - B + 18}" text-anchor="middle" font-size="11">${v.toLocaleString()}</text>`;
  s += `<text x="${(L + W - R) / 2}" y="${H - 14}" text-anchor="middle" font-size="12">${p.x_title}</text>`;
  s += `<text transform="translate(16 ${(T + H - B) / 2}) rotate(-90)" text-anchor="middle" font-size="12">${p.y_title}</text>`;
  let legend = '';
  tr.forEach((t, i) => {
    const c = t.meta.kind === 'theoretical' ? '#0f172a' : PAL[p.traces.indexOf(t) % PAL.length];
    const dash = t.meta.kind === 'theoretical' ? ' stroke-dasharray="6 4"' : '';
    const pts = t.x.map((x, j) => `${xpos(x)},${ypos(t.y[j])}`).join(' ');
    s += `<polyline fill="none" stroke="${c}" stroke-width="2"${dash} points="${pts}"/>`;
    if (t.meta.kind !== 'theoretical') t.x.forEach((x, j) => {
      s += `<circle cx="${xpos(x)}" cy="${ypos(t.y[j])}" r="3.5" fill="${c}"><title>${t.name}: ${t.y[j].toFixed(2)} TFLOPs at ${x}</title></circle>`;
    });
    legend += `<span class="key"><i style="background:${c}"></i>${t.name}</span>`;
  });
  s += '</svg>';
  host.innerHTML = s + `<div class="legend">${legend}</div>`;
}
const handles = [];
for (const p of plots) {
  const card = document.createElement('div'); card.className = 'plot-card'; card.dataset.expId = p.id;
  const h = document.createElement('h3'); h.textContent = p.title; card.appendChild(h);
  const host = document.createElement('div'); card.appendChild(host); root.appendChild(card);
  const lab = document.createElement('label');
  lab.innerHTML = `<input type="checkbox" class="exp-toggle" value="${p.id}" checked> ${p.title}`;
  expBox.appendChild(lab);
  handles.push({p, card, host}); draw(p, host);
}
document.addEventListener('change', ev => {
  if (ev.target.classList.contains('method-toggle')) handles.forEach(h => draw(h.p, h.host));
  if (ev.target.classList.contains('exp-toggle')) {
    const on = new Set(Array.from(document.querySelectorAll('.exp-toggle')).filter(x => x.checked).map(x => x.value));
    handles.forEach(h => { h.card.style.display = on.has(h.p.id) ? 'block' : 'none'; });
  }
});
"""

_STYLE = """
body { font-family: "Segoe UI", system-ui, sans-serif; margin: 0; padding: 24px; background: #f1f5f9; color: #0f172a; }
.controls { position: sticky; top: 0; background: #ffffffee; border: 1px solid #cbd5e1; border-radius: 10px; padding: 12px; margin-bottom: 18px; }
.controls-row { display: flex; gap: 16px; flex-wrap: wrap; margin-bottom: 6px; }
.plot-card { background: #fff; border: 1px solid #cbd5e1; border-radius: 10px; padding: 10px 14px 16px; margin-bottom: 18px; }
.plot { width: 100%; max-width: 1100px; }
.legend { display: flex; flex-wrap: wrap; gap: 6px 18px; font-size: 12px; }
.key i { display: inline-block; width: 12px; height: 12px; margin-right: 6px; border-radius: 2px; }
table { border-collapse: collapse; font-size: 12px; background: #fff; }
td, th { border: 1px solid #cbd5e1; padding: 3px 8px; text-align: right; }
th { background: #e2e8f0; }
"""


def render_html(plots: list[dict], rows: list[dict], output_path: pathlib.Path, methods: list[str], meta: dict) -> None:
    controls = "\n".join(f'<label><input type="checkbox" class="method-toggle" value="{html.escape(m)}" checked> '
                         f'{html.escape(m)}</label>' for m in methods)
    cols = ["experiment_group", "m", "n", "k", "method", "a_partition", "b_partition", "c_partition",
            "replication_factor", "world_size", "median_seconds", "median_tflops", "max_tflops"]
    head = "".join(f"<th>{c}</th>" for c in cols)
    body = ""
    for r in rows:
        cells = []
        for c in cols:
            v = r.get(c, "")
            cells.append(f"<td>{v:.4g}</td>" if isinstance(v, float) else f"<td>{html.escape(str(v))}</td>")
        body += "<tr>" + "".join(cells) + "</tr>\n"
    info = html.escape(", ".join(f"{k}={meta[k]}" for k in ("created_at", "host", "nproc_per_node", "warmup_iters",
                                                             "measure_iters") if k in meta))
    script = _SCRIPT.replace("__PALETTE__", json.dumps(PALETTE)).replace("__PLOTS__", json.dumps(plots))
    page = f"""<!doctype html>
<html lang="en"><head><meta charset="utf-8"><meta name="viewport" content="width=device-width, initial-scale=1">
<title>Universal GEMM Benchmark Report</title><style>{_STYLE}</style></head>
<body><h1>Universal GEMM Benchmark Report</h1><p>{info}</p>
<div class="controls"><div class="controls-row"><strong>Methods:</strong> {controls}</div>
<div class="controls-row" id="experiment-toggles"></div></div>
<div id="plots-root"></div>
<h2>All rows</h2><table><thead><tr>{head}</tr></thead><tbody>
{body}</tbody></table>
<script>{script}</script></body></html>
"""
    output_path.write_text(page, encoding="utf-8")


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Render the interactive HTML benchmark report")
    p.add_argument("--results-json", type=str, required=True)
    p.add_argument("--output-html", type=str, default=None)
    p.add_argument("--methods", type=str, default="dtensor,stationary_c,stationary_b,auto",
                   help="Comma-separated method filter for the rendered report")
    p.add_argument("--groups", type=str, default="", help="Optional comma-separated experiment group filter")
    return p.parse_args(argv)


def main(argv=None) -> None:
    args = parse_args(argv)
    results_path = pathlib.Path(args.results_json)
    out = pathlib.Path(args.output_html) if args.output_html else results_path.with_name("report.html")
    payload = load_results(results_path)
    methods = {x.strip() for x in args.methods.split(",") if x.strip()}
    groups = {x.strip() for x in args.groups.split(",") if x.strip()} or None
    plots = build_plots(group_rows(payload["results"]), methods or None, groups)
    present = sorted({t["meta"]["method"] for p in plots for t in p["traces"] if t["meta"]["kind"] == "series"})
    render_html(plots, payload["results"], out, present, payload)
    print(f"Wrote report: {out}")


if __name__ == "__main__":
    main()
