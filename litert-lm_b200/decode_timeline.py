"""Per-phase device timeline of one decode step (persistent decode modes).

    python litert-lm_b200/decode_timeline.py [--model gemma3-1b] [--mode 2] [--prompt 1024]

Prints, for every phase class (qkv, attention, o-proj, gate/up, down, head, arg-max), the
time the slowest CTA worked, the barrier latency seen by the last CTA to arrive, and their
sum over the step.  Built on B200Lm_TraceDecodeStep.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402


def summarise(stamps: np.ndarray, khz: int, n_layers: int):
    """stamps [n_barriers, n_cta, 2] -> rows (phase, work_max_us, work_mean_us, barrier_us)."""
    nb = stamps.shape[0]
    arrive, release = stamps[:, :, 0].astype(np.float64), stamps[:, :, 1].astype(np.float64)
    us = 1e3 / khz
    work = np.zeros_like(arrive)
    work[1:] = arrive[1:] - release[:-1]
    work[0] = np.nan                      # phase 0 includes kernel start-up
    wait = release - arrive
    names = []
    for _ in range(n_layers):
        names += ["qkv", "attention", "o-proj", "gate/up", "down"]
    names += ["head", "arg-max"]
    rows = {}
    for b in range(nb):
        r = rows.setdefault(names[b], [0.0, 0.0, 0.0, 0])
        if b > 0:
            r[0] += np.nanmax(work[b]) * us
            r[1] += np.nanmean(work[b]) * us
        r[2] += wait[b].min() * us
        r[3] += 1
    return rows


def summarise_chained(pts: np.ndarray, khz: int, n_layers: int) -> None:
    """Chained kernel: pts [n_phases, n_cta, 8] SM-clock stamps taken by thread 0 of every CTA:
    0 phase begin, 1 input seen (poll done), 2 prologue done, 3 / 4 points inside, 7 phase end.
    SM clocks are not synchronised with each other, so only differences inside one CTA are used."""
    us = 1e3 / khz
    names = []
    for _ in range(n_layers):
        names += ["qkv", "attention", "o-proj", "ffn", "reduce"]
    names += ["head", "arg-max"]
    p = pts.astype(np.float64)
    beg, end = p[:, :, 0], p[:, :, 7]
    dur = np.where((beg > 0) & (end > 0), (end - beg) * us, np.nan)
    worked = p[:, :, 1] > 0                      # CTAs that polled an input in the phase
    print(f"{'phase':10s} {'count':>5s} {'us/phase (CTA 0)':>17s} {'mean working CTA':>17s} {'max CTA':>9s} {'working CTAs':>13s}")
    total0 = 0.0
    for cls in ["qkv", "attention", "o-proj", "ffn", "reduce", "head", "arg-max"]:
        idx = [b for b, n in enumerate(names) if n == cls]
        d0 = np.nanmean(dur[idx, 0])
        w = np.where(worked[idx], dur[idx], np.nan)
        total0 += np.nansum(dur[idx, 0])
        print(f"{cls:10s} {len(idx):5d} {d0:17.2f} {np.nanmean(w):17.2f} {np.nanmax(dur[idx]):9.2f} {worked[idx].sum() / len(idx):13.1f}")
    hb = len(names) - 1
    if p[hb, :, 4:7].any():
        print("head phase, warp 0 of every CTA, mean us: wait for slot %.2f, tiles x int8 MMA %.2f, finalise + store + release %.2f" %
              tuple(np.mean(p[hb, :, k]) * us for k in (4, 5, 6)))
    gaps = np.where((p[1:, 0, 0] > 0) & (p[:-1, 0, 7] > 0), (p[1:, 0, 0] - p[:-1, 0, 7]) * us, np.nan)
    print(f"CTA 0: sum of phases {total0:.1f} us, gaps between phases {np.nansum(gaps):.1f} us")
    segs = [(0, 1, "begin->input seen"), (1, 2, "->prologue done"), (2, 3, "->3"), (3, 4, "->4"), (4, 7, "->end"), (2, 7, "prologue->end"),
            (1, 7, "seen->end"), (3, 7, "3->end"), (2, 5, "prologue->weights there"), (5, 7, "weights there->end"),
            (5, 3, "gate/up math"), (4, 6, "wait down weights"), (6, 7, "down math")]
    print("segments, mean over working CTAs and layers / CTA 0 (us):")
    for cls in ["qkv", "attention", "o-proj", "ffn", "reduce", "head", "arg-max"]:
        idx = [b for b, n in enumerate(names) if n == cls]
        out = []
        for lo, hi, nm in segs:
            ok = (p[idx][:, :, lo] > 0) & (p[idx][:, :, hi] > 0)
            if not ok.any():
                continue
            dd = np.where(ok, (p[idx][:, :, hi] - p[idx][:, :, lo]) * us, np.nan)
            out.append(f"{nm}={np.nanmean(dd):.2f}/{np.nanmean(dd[:, 0]):.2f}")
        print(f"  {cls:10s} " + "  ".join(out))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gemma3-1b")
    ap.add_argument("--mode", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=1024)
    args = ap.parse_args()
    sys.path.insert(0, ROOT)
    import bench
    graft.build()
    pkg = graft.load_package()
    cfg, rec, img = bench.load_model(args.model)
    ex = pkg.B200LlmExecutor(img, decode_mode=args.mode)
    ids = np.random.Generator(np.random.PCG64(cfg.seed)).integers(0, cfg.vocab, args.prompt).astype(np.int32)
    ex.Prefill(ids)
    for _ in range(3):
        ex.Decode()
    tok, stamps, khz = ex.TraceDecodeStep()
    if ex.GetDecodeMode() == pkg.DECODE_CHAINED:
        print(f"model={cfg.name} mode=chained n_cta={stamps.shape[1]} phases={stamps.shape[0]} sm_clock_khz={khz}")
        summarise_chained(ex.last_trace_points, khz, cfg.n_layers)
        log = stamps.reshape(-1)[:12000].reshape(-1, 3).astype(np.float64)
        ok = (log[:, 0] > 0) & (log[:, 1] > 0) & (log[:, 2] > 0)
        n = int(ok.sum())
        if n:
            us = 1e3 / khz
            t0 = log[ok][:, 1].min()
            print("CTA 0 fills: index, issue (us since first wait), lead of the copy over the wait start, time waited")
            for i in np.nonzero(ok)[0][200:260]:
                print(f"  {i:5d} issue {((log[i,0]-t0)*us):9.2f}  lead {((log[i,1]-log[i,0])*us):8.2f}  waited {((log[i,2]-log[i,1])*us):7.2f}")
            print("  total waited over the step: %.1f us in %d fills; fills with lead < 2 us: %d" %
                  ((log[ok][:, 2] - log[ok][:, 1]).sum() * us, n, int(((log[ok][:, 1] - log[ok][:, 0]) * us < 2.0).sum())))
        return
    rows = summarise(stamps, khz, cfg.n_layers)
    total = 0.0
    print(f"model={cfg.name} mode={args.mode} n_cta={stamps.shape[1]} barriers={stamps.shape[0]} sm_clock_khz={khz}")
    print(f"{'phase':10s} {'count':>5s} {'slowest-CTA work us':>20s} {'mean-CTA work us':>17s} {'barrier us':>11s} {'per-phase us':>13s}")
    for name, (wmax, wmean, bar, n) in rows.items():
        total += wmax + bar
        print(f"{name:10s} {n:5d} {wmax:20.1f} {wmean:17.1f} {bar:11.1f} {(wmax + bar) / n:13.2f}")
    print(f"step total (work of slowest CTA + barrier latency): {total:.1f} us")
    pts = getattr(ex, "last_trace_points", None)
    if pts is not None and pts.any():
        names = []
        for _ in range(cfg.n_layers):
            names += ["qkv", "attention", "o-proj", "gate/up", "down"]
        names += ["head", "arg-max"]
        us = 1e3 / khz
        points = [0, 1, 3, 4, 5, 6]           # stamps taken by the streaming kernel (2 is unused)
        labels = ["wait staged", "prologue", "mma", "epilogue", "tail rounds"]
        print("segments inside a phase, mean over CTAs that reached both points (us):")
        for cls in ["qkv", "attention", "o-proj", "gate/up", "down", "head"]:
            idx = [b for b in range(1, len(names)) if names[b] == cls]
            seg = []
            rel = stamps[[b - 1 for b in idx], :, 1].astype(np.float64)
            p = pts[idx].astype(np.float64)
            first = np.where(p[:, :, 0] > 0, (p[:, :, 0] - rel) * us, np.nan)
            seg.append(("release->start", np.nanmean(first)))
            for k in range(len(points) - 1):
                lo, hi = points[k], points[k + 1]
                ok = (p[:, :, lo] > 0) & (p[:, :, hi] > 0)
                d = np.where(ok, (p[:, :, hi] - p[:, :, lo]) * us, np.nan)
                seg.append((labels[k], float(np.nanmean(d)) if ok.any() else float("nan")))
            inner = (((1, 2, "stage q/k/v"), (2, 7, "append + ranges"), (7, 3, "scores"), (3, 5, "P.V"), (5, 6, "reduce + write partials"))
                     if cls == "attention" else ((1, 2, "loads+sums"), (2, 7, "block reduce"), (7, 3, "quantize")))
            for lo, hi, nm in inner:
                ok = (p[:, :, lo] > 0) & (p[:, :, hi] > 0)
                if ok.any():
                    seg.append((nm, float(np.nanmean(np.where(ok, (p[:, :, hi] - p[:, :, lo]) * us, np.nan)))))
            arr = stamps[idx, :, 0].astype(np.float64)
            lastp = np.where(p[:, :, 6] > 0, (arr - p[:, :, 6]) * us, np.nan)
            seg.append(("end->arrive", float(np.nanmean(lastp)) if np.isfinite(lastp).any() else float("nan")))
            print(f"  {cls:10s} " + "  ".join(f"{n}={v:.2f}" for n, v in seg))


if __name__ == "__main__":
    main()
