"""Loss and validation curves of a run as an SVG file, from its log (role of plot_live.sh, which scrapes the
``[eval] step N ... val_bpb X`` lines over ssh and draws a matplotlib PNG; no plotting library is needed here).

    python -m autoresearch_b200.tools.plot_live train.log --out curves.svg [--follow]
"""
from __future__ import annotations

import argparse
import time

from . import monitor


def _polyline(xs, ys, x0, x1, y0, y1, box, color):
    bx, by, bw, bh = box
    pts = []
    for x, y in zip(xs, ys):
        px = bx + (x - x0) / max(x1 - x0, 1e-12) * bw
        py = by + bh - (y - y0) / max(y1 - y0, 1e-12) * bh
        pts.append(f"{px:.1f},{py:.1f}")
    return f'<polyline fill="none" stroke="{color}" stroke-width="1.5" points="{" ".join(pts)}"/>'


def _panel(title, xs, ys, box, color):
    bx, by, bw, bh = box
    out = [f'<rect x="{bx}" y="{by}" width="{bw}" height="{bh}" fill="none" stroke="#888"/>',
           f'<text x="{bx}" y="{by - 6}" font-size="13" font-family="sans-serif">{title}</text>']
    if len(xs) >= 1:
        x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
        if y1 - y0 < 1e-9:
            y0, y1 = y0 - 0.5, y1 + 0.5
        out.append(_polyline(xs, ys, x0, x1, y0, y1, box, color))
        for frac in (0.0, 0.5, 1.0):
            v = y0 + frac * (y1 - y0)
            py = by + bh - frac * bh
            out.append(f'<text x="{bx + bw + 4}" y="{py + 4:.1f}" font-size="11" font-family="sans-serif">{v:.4g}</text>')
        out.append(f'<text x="{bx}" y="{by + bh + 14}" font-size="11" font-family="sans-serif">step {x0:g}</text>')
        out.append(f'<text x="{bx + bw - 60}" y="{by + bh + 14}" font-size="11" font-family="sans-serif">step {x1:g}</text>')
    return "\n".join(out)


def render(parsed) -> str:
    steps = parsed["steps"]
    evals = [e for e in parsed["evals"] if e["step"] is not None]
    body = [_panel("training loss (EMA)", [s["step"] for s in steps], [s["loss"] for s in steps], (40, 30, 520, 180), "#1f77b4"),
            _panel("val_bpb", [e["step"] for e in evals], [e["val_bpb"] for e in evals], (40, 260, 520, 180), "#d62728")]
    return ('<svg xmlns="http://www.w3.org/2000/svg" width="640" height="470" viewBox="0 0 640 470">\n'
            '<rect width="640" height="470" fill="white"/>\n' + "\n".join(body) + "\n</svg>\n")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("log")
    ap.add_argument("--out", default="curves.svg")
    ap.add_argument("--follow", action="store_true")
    ap.add_argument("--interval", type=float, default=60.0)
    a = ap.parse_args(argv)
    while True:
        with open(a.log, errors="replace") as f:
            parsed = monitor.parse(f)
        with open(a.out, "w") as f:
            f.write(render(parsed))
        print(f"{a.out}: {len(parsed['steps'])} step lines, {len(parsed['evals'])} eval lines", flush=True)
        if not a.follow:
            return 0
        time.sleep(a.interval)


if __name__ == "__main__":
    main()
