#!/usr/bin/env python
"""Compare two ``--save-stats`` files (e.g. a single-GPU baseline and a DDP run).

    python examples/benchmark_throughput.py baseline.json ddp.json --out bench

Prints throughput / mean step time / speed-up, writes ``<out>.npz`` with the step-time and
loss series and, when matplotlib is available, ``<out>.png`` (step time and loss curves)
and ``<out>_bars.png`` (throughput bars) like the reference's
examples/benchmark_throughput.py:103-243.
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def load(path):
    with open(path, encoding="utf-8") as f:
        return json.load(f)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("baseline")
    ap.add_argument("ddp")
    ap.add_argument("--out", default="bench")
    args = ap.parse_args()
    a, b = load(args.baseline), load(args.ddp)
    rows = []
    for s in (a, b):
        rows.append((s["mode"], s["world_size"], s["throughput_samples_per_sec"], s["avg_step_time_s"] * 1e3,
                     s["losses"][-1] if s["losses"] else float("nan")))
    print(f"{'mode':<14}{'world':>6}{'samples/s':>14}{'ms/step':>12}{'final loss':>12}")
    for r in rows:
        print(f"{r[0]:<14}{r[1]:>6}{r[2]:>14.1f}{r[3]:>12.2f}{r[4]:>12.4f}")
    ratio = a["throughput_samples_per_sec"] / max(b["throughput_samples_per_sec"], 1e-12)
    print(f"baseline/ddp throughput ratio: {ratio:.2f}x  (ddp speed-up {1 / max(ratio, 1e-12):.2f}x on {b['world_size']} ranks)")
    np.savez(args.out + ".npz", baseline_step_times=np.array(a["step_times"]), ddp_step_times=np.array(b["step_times"]),
             baseline_losses=np.array(a["losses"]), ddp_losses=np.array(b["losses"]))
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        print("matplotlib not available: skipped the plots")
        return
    fig, (top, bot) = plt.subplots(2, 1, figsize=(9, 7))
    for s, c in ((a, "tab:gray"), (b, "tab:green")):
        t = np.array(s["step_times"]) * 1e3
        top.plot(t, color=c, label=f"{s['mode']} (mean {t.mean():.1f} ms/step)")
        bot.plot(np.cumsum(s["step_times"]), s["losses"], color=c, label=s["mode"])
    top.set_ylabel("ms / step"); top.legend(); bot.set_xlabel("wall seconds"); bot.set_ylabel("loss"); bot.legend()
    fig.savefig(args.out + ".png", dpi=120)
    fig2, ax = plt.subplots(figsize=(5, 4))
    ax.bar([a["mode"], b["mode"]], [a["throughput_samples_per_sec"], b["throughput_samples_per_sec"]],
           color=["tab:gray", "tab:green"])
    ax.set_ylabel("samples / s"); ax.set_title(f"baseline/ddp = {ratio:.2f}x")
    fig2.savefig(args.out + "_bars.png", dpi=120)


if __name__ == "__main__":
    main()
