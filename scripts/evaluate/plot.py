#!/usr/bin/env python3
"""Plots for ``evaluate.py sweep`` results (needs matplotlib).

    python plot.py compare --source "No Spec=nospec/perf_results.csv" --source "Eagle3=eagle3/perf_results.csv" --metric latency
    python plot.py speedup --baseline "No Spec=nospec/perf_results.csv" --target "Eagle3=eagle3/perf_results.csv" --metric itl

``compare`` overlays smoothed metric-vs-request-rate curves of several versions (all
subsets pooled); ``speedup`` draws baseline and target curves per subset with the gap
shaded by the speed-up ratio (blue = faster, red = regression) and prints the ratio's
summary.  CLI parity: scripts/evaluate/plot.py:375 of the reference.
"""

from __future__ import annotations

import argparse
import sys
from collections import defaultdict
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
import perf_utils as pu  # noqa: E402

COLORS = ("#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f")


def _pyplot():
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt

        return plt
    except ImportError:
        print("[ERROR] matplotlib is required for plotting (pip install -r scripts/evaluate/requirements.txt)", file=sys.stderr)
        raise SystemExit(1) from None


def collect(sources: dict[str, list[Path]], metric: str) -> dict[str, dict[str, list[tuple[float, float]]]]:
    """``{label: {subset: points}}`` pooled over the label's files."""
    out: dict[str, dict[str, list]] = defaultdict(lambda: defaultdict(list))
    for label, paths in sources.items():
        for path in paths:
            try:
                for subset, pts in pu.load_data(path, metric).items():
                    out[label][subset].extend(pts)
            except (ValueError, FileNotFoundError) as err:
                print(f"[WARN] {err}", file=sys.stderr)
    return out


def speedup_curves(base_pts, target_pts, *, increasing: bool):
    """Dense x over the common rate range, both smoothed curves on it, and their ratio
    (> 1 = target better).  ``None`` when the ranges do not overlap."""
    import numpy as np

    bx, by = pu.smooth_curve(*zip(*base_pts))
    tx, ty = pu.smooth_curve(*zip(*target_pts))
    lo, hi = max(bx.min(), tx.min()), min(bx.max(), tx.max())
    if lo >= hi:
        return None
    x = np.linspace(lo, hi, 200)
    yb, yt = np.interp(x, bx, by), np.interp(x, tx, ty)
    ratio = yb / np.maximum(yt, 1e-12) if increasing else yt / np.maximum(yb, 1e-12)
    return x, yb, yt, ratio


def run_compare(args: argparse.Namespace) -> int:
    plt = _pyplot()
    sources = pu.parse_source_args(args.source)
    keep = set(args.subsets.split(",")) if args.subsets else None
    args.output_dir.mkdir(parents=True, exist_ok=True)
    for metric in args.metric or ["latency"]:
        data = collect(sources, metric)
        fig, ax = plt.subplots(figsize=(8, 5))
        drawn = False
        for i, label in enumerate(sources):
            pts = sorted(p for subset, ps in data[label].items() if keep is None or subset in keep for p in ps)
            if not pts:
                continue
            xs, ys = zip(*pts)
            ax.scatter(xs, ys, color=COLORS[i % len(COLORS)], alpha=0.35, s=25, zorder=3)
            ax.plot(*pu.smooth_curve(xs, ys), color=COLORS[i % len(COLORS)], linewidth=2.5, label=label, zorder=4)
            drawn = True
        if not drawn:
            print(f"[WARN] No data found for metric '{metric}'", file=sys.stderr)
            plt.close(fig)
            continue
        ax.set_title(pu.METRICS[metric]["label"], fontsize=14, fontweight="bold")
        ax.set_xlabel("Requests per Second", fontsize=12)
        ax.set_ylabel(pu.METRICS[metric]["label"], fontsize=12)
        ax.legend(framealpha=0.9)
        ax.grid(True, alpha=0.3)
        fig.tight_layout()
        fig.savefig(args.output_dir / f"compare_{metric}.png", dpi=150)
        plt.close(fig)
        print(f"[INFO] Saved {args.output_dir / f'compare_{metric}.png'}")
    return 0


def run_speedup(args: argparse.Namespace) -> int:
    plt = _pyplot()
    import numpy as np
    from matplotlib.colors import TwoSlopeNorm

    base, target = pu.parse_source_args(args.baseline), pu.parse_source_args(args.target)
    (b_label,), (t_label,) = list(base)[:1], list(target)[:1]
    keep = set(args.subsets.split(",")) if args.subsets else None
    args.output_dir.mkdir(parents=True, exist_ok=True)
    for metric in args.metric or ["latency"]:
        cfg = pu.METRICS[metric]
        b_data, t_data = collect(base, metric)[b_label], collect(target, metric)[t_label]
        subsets = sorted(set(b_data) & set(t_data) & (keep or set(b_data)))
        if not subsets:
            print(f"[WARN] No common subsets for metric '{metric}'", file=sys.stderr)
            continue
        cols = min(3, len(subsets))
        rows = -(-len(subsets) // cols)
        fig, axes = plt.subplots(rows, cols, figsize=(6 * cols, 4.2 * rows), squeeze=False)
        for ax, subset in zip(axes.flat, subsets):
            curves = speedup_curves(b_data[subset], t_data[subset], increasing=cfg["increasing"])
            if curves is None:
                ax.set_visible(False)
                continue
            x, yb, yt, ratio = curves
            norm = TwoSlopeNorm(vmin=min(0.5, ratio.min()), vcenter=1.0, vmax=max(2.0, ratio.max()))
            cmap = plt.get_cmap("RdBu")
            for j in range(len(x) - 1):  # shade the gap strip by strip with the local ratio
                ax.fill_between(x[j:j + 2], yb[j:j + 2], yt[j:j + 2], color=cmap(norm(ratio[j])), alpha=0.6, linewidth=0)
            ax.plot(x, yb, color="#444444", linewidth=2, label=b_label)
            ax.plot(x, yt, color="#1f77b4", linewidth=2, label=t_label)
            ax.set_title(f"{pu.pretty_subset(subset)}  (mean x{np.mean(ratio):.2f})", fontsize=11)
            ax.set_xlabel("Requests per Second")
            ax.set_ylabel(cfg["label"])
            ax.grid(True, alpha=0.3)
            ax.legend(fontsize=8)
            print(f"[INFO] {metric} {subset}: speedup mean {np.mean(ratio):.3f} min {ratio.min():.3f} max {ratio.max():.3f}")
        for ax in list(axes.flat)[len(subsets):]:
            ax.set_visible(False)
        fig.suptitle(" ".join(filter(None, [args.title, f"{cfg['label']}: {t_label} vs {b_label}"])), fontweight="bold")
        fig.tight_layout()
        fig.savefig(args.output_dir / f"speedup_{metric}.png", dpi=150)
        plt.close(fig)
        print(f"[INFO] Saved {args.output_dir / f'speedup_{metric}.png'}")
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="plot", description="Performance visualization for speculative decoding benchmarks.")
    sub = ap.add_subparsers(dest="command", required=True)
    metric_help = f"metric(s) to plot (default latency); choices: {', '.join(pu.METRICS)}"
    cmp_ = sub.add_parser("compare", help="overlay several versions")
    cmp_.add_argument("--source", action="append", required=True, metavar="LABEL=PATH", help="repeatable; equal labels pool repetitions")
    spd = sub.add_parser("speedup", help="baseline vs target with ratio shading")
    spd.add_argument("--baseline", action="append", required=True, metavar="LABEL=PATH")
    spd.add_argument("--target", action="append", required=True, metavar="LABEL=PATH")
    spd.add_argument("--title", default=None)
    for p, fn in ((cmp_, run_compare), (spd, run_speedup)):
        p.add_argument("--metric", action="append", choices=list(pu.METRICS), metavar="METRIC", help=metric_help)
        p.add_argument("--output-dir", type=Path, default=Path())
        p.add_argument("--subsets", default=None, help="comma-separated subset filter")
        p.set_defaults(func=fn)
    return ap


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        return args.func(args)
    except (ValueError, FileNotFoundError) as err:
        print(f"[ERROR] {err}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
