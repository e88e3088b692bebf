"""Offline tools for ``training_metrics.jsonl``: ``info`` lists the recorded series, ``plot`` draws selected
series as stacked panels with a centred moving average and writes an image file (SVG / PNG by extension).

    python -m async_grpo_nccl_b200.utils.plot info  runs/exp1/training_metrics.jsonl
    python -m async_grpo_nccl_b200.utils.plot plot  runs/exp1/training_metrics.jsonl -v training/avg_loss -v training/batch_avg_reward -o curves.svg

Same job as the reference's parse_logs.py / plot.py (parse_logs.py:7-131, plot.py:11-153); files only, no interactive
window (the GPU machines are headless). matplotlib is imported lazily; without it ``plot`` writes the smoothed series as
CSV next to the requested path instead.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
from typing import Dict, List, Optional, Sequence, Tuple


def parse_experiment_logs(path: str) -> Dict[str, List[Tuple[float, float]]]:
    """{series: [(x, value), ...]} with x = total samples seen when logged, else the record's step / index."""
    series: Dict[str, List[Tuple[float, float]]] = {}
    with open(path, "r", encoding="utf-8") as f:
        for i, line in enumerate(f):
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            x = rec.get("total_samples_seen", rec.get("trainer_step", rec.get("_step", i)))
            for k, v in rec.items():
                if k.startswith("_") or isinstance(v, bool) or not isinstance(v, (int, float)):
                    continue
                series.setdefault(k, []).append((float(x), float(v)))
    return series


def moving_average(values: Sequence[float], window: int) -> List[float]:
    """Centred moving average; the window shrinks at the edges."""
    n = len(values)
    if window <= 1 or n == 0:
        return list(values)
    half = window // 2
    out = []
    for i in range(n):
        lo, hi = max(0, i - half), min(n, i + half + 1)
        out.append(sum(values[lo:hi]) / (hi - lo))
    return out


def plot_experiments_variables(paths: Sequence[str], variables: Sequence[str], output: str, smooth: int = 10,
                               labels: Optional[Sequence[str]] = None) -> str:
    runs = [(labels[i] if labels else os.path.basename(os.path.dirname(p)) or p, parse_experiment_logs(p)) for i, p in enumerate(paths)]
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        out_csv = os.path.splitext(output)[0] + ".csv"
        with open(out_csv, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["run", "series", "x", "value", "smoothed"])
            for name, ser in runs:
                for var in variables:
                    pts = ser.get(var, [])
                    sm = moving_average([v for _, v in pts], smooth)
                    for (x, v), s in zip(pts, sm):
                        w.writerow([name, var, x, v, s])
        return out_csv
    fig, axes = plt.subplots(len(variables), 1, figsize=(9, 2.8 * len(variables)), sharex=True, squeeze=False)
    for ax, var in zip(axes[:, 0], variables):
        for name, ser in runs:
            pts = ser.get(var, [])
            if not pts:
                continue
            xs = [x for x, _ in pts]
            ax.plot(xs, [v for _, v in pts], alpha=0.25)
            ax.plot(xs, moving_average([v for _, v in pts], smooth), label=name)
        ax.set_ylabel(var)
        ax.grid(True, alpha=0.3)
        ax.legend(fontsize=7)
    axes[-1, 0].set_xlabel("samples seen / step")
    fig.tight_layout()
    fig.savefig(output)
    plt.close(fig)
    return output


def fetch_if_remote(path: str) -> str:
    """``host:/path/metrics.jsonl`` is copied with scp into a temporary file first (parse_logs.py:7-41 offers the same);
    local paths are returned unchanged."""
    import os
    import subprocess
    import tempfile

    if ":" not in path or os.path.exists(path) or path[1:3] == ":\\":
        return path
    fd, local = tempfile.mkstemp(suffix=".jsonl", prefix="metrics_")
    os.close(fd)
    subprocess.run(["scp", "-q", path, local], check=True)
    return local


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="plot")
    sub = ap.add_subparsers(dest="cmd", required=True)
    pi = sub.add_parser("info")
    pi.add_argument("path")
    pp = sub.add_parser("plot")
    pp.add_argument("paths", nargs="+")
    pp.add_argument("-v", "--var", action="append", required=True)
    pp.add_argument("-o", "--output", default="metrics.svg")
    pp.add_argument("-s", "--smooth", type=int, default=10)
    args = ap.parse_args(argv)
    if args.cmd == "info":
        ser = parse_experiment_logs(fetch_if_remote(args.path))
        for k in sorted(ser):
            vals = [v for _, v in ser[k]]
            print(f"{k:50s} n={len(vals):6d} last={vals[-1]:.6g} min={min(vals):.6g} max={max(vals):.6g}")
        return 0
    print(plot_experiments_variables([fetch_if_remote(p) for p in args.paths], args.var, args.output, args.smooth))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
