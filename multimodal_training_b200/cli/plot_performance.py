"""Throughput table (and bar chart when matplotlib is present) from sweep results.

    python -m multimodal_training_b200.cli.plot_performance --results experiments/generated/results.txt

``tokens/s = vision patches before the 2x2 merge x batch size / average iteration seconds`` and, per
sequence length, the largest batch size that ran is reported: the reference's definitions
(scripts/plot_performance.py:37-44,146-147 there).  Several result files can be compared
(``--results a.txt b.txt --labels ours baseline``).
"""
from __future__ import annotations

import argparse
import re

TOKEN_COUNT_MAPPING = {"1k_tokens": 1024, "4k_tokens": 4096, "9k_tokens": 9216, "16k_tokens": 16384,
                       "25k_tokens": 25600, "64k_tokens": 65536}


def parse_results(path: str) -> dict:
    """{(model, size, vision_parallelism): {batch_size: seconds or 'OOM'}}"""
    out: dict = {}
    for line in open(path):
        m = re.match(r"(\w+?)_(\d+k_tokens)_(\w+)_bs(\d+)\s+(OK|OOM|FAILED)(?:.*?([0-9.]+)s)?", line.strip())
        if not m:
            continue
        model, size, vp, bs, status, secs = m.groups()
        out.setdefault((model, size, vp), {})[int(bs)] = float(secs) if status == "OK" and secs else status
    return out


def best_throughput(runs: dict) -> tuple[int, float] | None:
    ok = {bs: s for bs, s in runs.items() if isinstance(s, float) and s > 0}
    if not ok:
        return None
    bs = max(ok)
    return bs, 0.0 + bs / ok[bs]


def table(results: dict) -> list[tuple]:
    rows = []
    for (model, size, vp), runs in sorted(results.items()):
        b = best_throughput(runs)
        tok = TOKEN_COUNT_MAPPING[size]
        rows.append((model, size, vp, b[0] if b else None, tok * b[1] if b else None))
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--results", nargs="+", required=True)
    ap.add_argument("--labels", nargs="*")
    ap.add_argument("--output", default="performance.png")
    a = ap.parse_args(argv)
    labels = a.labels or a.results
    tables = [table(parse_results(p)) for p in a.results]
    for lab, rows in zip(labels, tables):
        print(f"== {lab}")
        for model, size, vp, bs, tps in rows:
            print(f"{model:>4} {size:>11} {vp:>9} bs={bs} " + (f"{tps:,.0f} tok/s" if tps else "no successful run"))
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        print("matplotlib is not installed: table only")
        return 0
    fig, ax = plt.subplots(figsize=(10, 4))
    width = 0.8 / max(len(tables), 1)
    for i, (lab, rows) in enumerate(zip(labels, tables)):
        xs = [j + i * width for j in range(len(rows))]
        ax.bar(xs, [r[4] or 0 for r in rows], width=width, label=lab)
    ax.set_xticks(range(len(tables[0])))
    ax.set_xticklabels([f"{r[0]} {r[1]} {r[2]}" for r in tables[0]], rotation=60, ha="right", fontsize=7)
    ax.set_ylabel("vision tokens / s")
    ax.legend()
    fig.tight_layout()
    fig.savefig(a.output, dpi=150)
    print("wrote", a.output)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
