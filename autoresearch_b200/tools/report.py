"""Static benchmark page from result lines (role of docs/index.html + docs/charts/*.svg, a page of bar charts of
the reference's early results; no JavaScript or plotting library is needed here: the charts are inline SVG).

    python bench.py --steps 3 --warmup 3 >> results.jsonl          # one JSON line per run, any number of runs
    python -m autoresearch_b200.tools.report results.jsonl --out report.html

Every input line that parses as a JSON object with "value" and "config" becomes a bar; runs are grouped by
metric, labelled by implementation, model, parallelism and GPU count.  Lines of the form
{"impl": "reference", "unavailable": "..."} are listed under the charts with their reason.
"""
from __future__ import annotations

import argparse
import html
import json


def load(paths):
    runs, notes = [], []
    for path in paths:
        with open(path, errors="replace") as f:
            for line in f:
                line = line.strip()
                if not line.startswith("{"):
                    continue
                try:
                    d = json.loads(line)
                except ValueError:
                    continue
                if not isinstance(d, dict):
                    continue
                if "unavailable" in d:
                    notes.append(f'{d.get("impl", "?")}: {d["unavailable"]}')
                elif "value" in d and isinstance(d.get("config"), dict):
                    runs.append(d)
    return runs, notes


def label(d) -> str:
    c = d["config"]
    parts = [str(d.get("impl", "own")), str(c.get("model", "?")), str(c.get("parallelism", "")), f'{d.get("n_gpus", 1)} GPU']
    return " | ".join(p for p in parts if p)


def bar_chart(title, rows, unit) -> str:
    """rows: (label, value, note).  Horizontal bars scaled to the largest value."""
    top = max((v for _, v, _ in rows), default=1.0) or 1.0
    h = 28 * len(rows) + 50
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="960" height="{h}" viewBox="0 0 960 {h}">',
           f'<text x="8" y="20" font-size="15" font-family="sans-serif" font-weight="bold">{html.escape(title)}</text>']
    for i, (lab, v, note) in enumerate(rows):
        y = 36 + 28 * i
        w = 420.0 * v / top
        out.append(f'<text x="8" y="{y + 15}" font-size="12" font-family="sans-serif">{html.escape(lab[:60])}</text>')
        out.append(f'<rect x="390" y="{y}" width="{w:.1f}" height="20" fill="#1f77b4"/>')
        out.append(f'<text x="{396 + w:.1f}" y="{y + 15}" font-size="12" font-family="sans-serif">'
                   f'{v:,.0f} {html.escape(unit)}{html.escape(note)}</text>')
    out.append("</svg>")
    return "\n".join(out)


def render(runs, notes) -> str:
    by_metric = {}
    for d in runs:
        by_metric.setdefault((d.get("metric", "value"), d.get("unit", "")), []).append(d)
    body = ["<!doctype html><html><head><meta charset='utf-8'><title>autoresearch_b200 benchmarks</title></head>",
            "<body style='font-family:sans-serif;max-width:980px;margin:2em auto'>", "<h1>Benchmarks</h1>"]
    for (metric, unit), ds in by_metric.items():
        rows = []
        for d in ds:
            note = ""
            if d.get("vs_baseline") is not None:
                note += f'  ({d["vs_baseline"]:.2f}x published reference)'
            if isinstance(d.get("e2e"), dict) and "value" in d["e2e"]:
                note += f'  e2e {d["e2e"]["value"]:,.0f}'
            rows.append((label(d), float(d["value"]), note))
        body.append(bar_chart(metric, rows, unit))
        body.append("<table border='1' cellspacing='0' cellpadding='4' style='font-size:12px;border-collapse:collapse'>"
                    "<tr><th>run</th><th>ms / step</th><th>steps</th><th>dtype</th><th>SM MHz (median)</th><th>clock reasons</th><th>data</th></tr>")
        for d in ds:
            ck = d.get("clocks") or {}
            body.append("<tr>" + "".join(f"<td>{html.escape(str(x))}</td>" for x in (
                label(d), d.get("ms_per_step", ""), d.get("steps", ""), d.get("dtype", ""), ck.get("sm_mhz", ""),
                ", ".join(ck.get("reasons", []) or []), d.get("data", ""))) + "</tr>")
        body.append("</table>")
    if notes:
        body.append("<h2>Not measured</h2><ul>" + "".join(f"<li>{html.escape(n)}</li>" for n in notes) + "</ul>")
    body.append("</body></html>\n")
    return "\n".join(body)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("results", nargs="+", help="files of JSON result lines (the one-line output of bench.py)")
    ap.add_argument("--out", default="report.html")
    a = ap.parse_args(argv)
    runs, notes = load(a.results)
    with open(a.out, "w") as f:
        f.write(render(runs, notes))
    print(f"{len(runs)} runs, {len(notes)} notes -> {a.out}")


if __name__ == "__main__":
    main()
