"""Bandwidth-vs-size plot from the JSON lines of bench/sweep.py, the counterpart of the
reference's notebook (plot.ipynb:167-175: log-log "NCCL" vs "Ours").  Pure Python: writes an
SVG (no matplotlib needed) with one line per implementation / algorithm.

    python bench/plot.py results/sweep8.jsonl --collective allreduce --out results/allreduce8.svg
"""
import argparse
import json
import math


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("jsonl")
    ap.add_argument("--collective", default="allreduce")
    ap.add_argument("--metric", default="busbw_gbs", choices=["busbw_gbs", "algbw_gbs", "p50_us"])
    ap.add_argument("--graph", type=int, default=0)
    ap.add_argument("--out", default="plot.svg")
    a = ap.parse_args()
    series = {}
    for line in open(a.jsonl):
        r = json.loads(line)
        if r.get("collective") != a.collective or r.get("graph", 0) != a.graph or r.get("ctas"):
            continue
        v = r.get(a.metric)
        if v and v > 0:
            series.setdefault(f"{r['impl']}:{r['algo']}" if r["impl"] != r["algo"] else r["algo"], []).append((r["bytes"], v))
    if not series:
        raise SystemExit("nothing to plot")
    W, H, L, B = 900, 560, 70, 50
    xs = [x for s in series.values() for x, _ in s]
    ys = [y for s in series.values() for _, y in s]
    lx0, lx1 = math.log10(min(xs)), math.log10(max(xs))
    ly0, ly1 = math.floor(math.log10(min(ys))), math.ceil(math.log10(max(ys)))
    px = lambda x: L + (math.log10(x) - lx0) / max(lx1 - lx0, 1e-9) * (W - L - 180)
    py = lambda y: H - B - (math.log10(y) - ly0) / max(ly1 - ly0, 1e-9) * (H - B - 30)
    colors = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#17becf", "#7f7f7f", "#bcbd22"]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="12">',
           f'<rect width="{W}" height="{H}" fill="white"/>',
           f'<text x="{W / 2 - 100}" y="18" font-size="14">{a.collective}: {a.metric} vs message bytes</text>']
    for e in range(int(ly0), int(ly1) + 1):
        y = py(10 ** e)
        out.append(f'<line x1="{L}" y1="{y:.1f}" x2="{W - 180}" y2="{y:.1f}" stroke="#ddd"/>'
                   f'<text x="{L - 8}" y="{y + 4:.1f}" text-anchor="end">1e{e}</text>')
    e = math.ceil(lx0)
    while e <= lx1:
        x = px(10 ** e)
        out.append(f'<line x1="{x:.1f}" y1="30" x2="{x:.1f}" y2="{H - B}" stroke="#eee"/>'
                   f'<text x="{x:.1f}" y="{H - B + 16}" text-anchor="middle">1e{int(e)}</text>')
        e += 1
    for i, (name, pts) in enumerate(sorted(series.items())):
        pts.sort()
        c = colors[i % len(colors)]
        d = " ".join(f"{px(x):.1f},{py(y):.1f}" for x, y in pts)
        out.append(f'<polyline points="{d}" fill="none" stroke="{c}" stroke-width="2"/>')
        out.append(f'<text x="{W - 170}" y="{40 + 16 * i}" fill="{c}">{name}</text>')
    out.append("</svg>")
    with open(a.out, "w") as f:
        f.write("\n".join(out))
    print(f"wrote {a.out} ({len(series)} series)")


if __name__ == "__main__":
    main()
