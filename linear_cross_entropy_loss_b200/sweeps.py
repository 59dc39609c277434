"""Speed, peak-memory and accuracy sweeps of the fused loss over N, H and V.

    python -m linear_cross_entropy_loss_b200.sweeps --mode speed|memory|accuracy [--over N H V]
           [--acc bf16 fp16 fp16-mixed] [--out DIR] [--quick] [--forward-only]

Re-creates the three sweep families of the reference's benchmark script (bench_fusions.py:210-226 speed,
:318-334 memory, :448-467 accuracy of the reference project) around its default point N=16384, H=2048,
V=131072, and writes one CSV per (precision, swept variable) with the reference's file names and column
layout -- first column the swept variable, then one column per provider (here ``lce-b200``) -- so that the
files can be plotted next to the published ones.

* speed: fwd+bwd TFLOP/s with the reference's flop count 3 * (2 N H V + 3 N V) (bench_fusions.py:287-293),
  median of CUDA-event timings, inputs ``x~randn``, ``y~randint``, ``A~randn`` as there (:241-245).
* memory: ``max_memory_allocated - memory_allocated`` around one fwd+bwd, in GiB (:304-315).
* accuracy: ``torch.dist`` of the loss (``fwd``) and the mean of ``torch.dist`` of both gradients (``bwd``) against
  a float64 chunked torch computation on the GPU, inputs ``x = 0.1 A[y] + randn`` (:400-445, :480-512).
"""
from __future__ import annotations

import argparse
import csv
import os
import statistics
from pathlib import Path

import torch

from . import linear_cross_entropy

DEFAULTS = {"N": 16384, "H": 2048, "V": 131072}
RANGES = {  # powers of two, as in the reference (range_dict, bench_fusions.py:113 and :448)
    "speed": {"H": range(8, 14), "V": range(8, 18), "N": range(8, 17)},
    "memory": {"H": range(8, 14), "V": range(8, 18), "N": range(8, 17)},
    "accuracy": {"H": range(8, 14), "V": range(8, 18), "N": range(8, 16)},
}
# provider column; a fixed slab mode (LCE_SLAB_MODE=row|tile, see ops.SlabModePolicy) is named in it
PROVIDER = "lce-b200" + {"row": "-slab-per-row", "tile": "-slab-per-tile"}.get(os.environ.get("LCE_SLAB_MODE", ""), "")


def _dtype(acc: str) -> torch.dtype:
    return {"fp16": torch.float16, "bf16": torch.bfloat16, "fp16-mixed": torch.float32}[acc]


def _call(x, y, At, acc):
    if acc == "fp16-mixed":  # fp32 tensors under fp16 autocast, like the reference's "fp16-mixed" (:261-266)
        with torch.autocast(device_type="cuda", dtype=torch.float16):
            return linear_cross_entropy(x, y, At)[0]
    return linear_cross_entropy(x, y, At)[0]


def _inputs(N, H, V, acc, low_loss: bool, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dtype = _dtype(acc)
    A = torch.randn(V, H, device="cuda", generator=g)
    y = torch.randint(0, V, (N,), device="cuda", generator=g)
    x = torch.randn(N, H, device="cuda", generator=g)
    if low_loss:
        x = 0.1 * A[y] + x
    At = A.t().contiguous().to(dtype).requires_grad_(True)
    return x.to(dtype).requires_grad_(True), y, At


def speed_point(N, H, V, acc, reps, forward_only=False):
    x, y, At = _inputs(N, H, V, acc, low_loss=False)

    def step():
        if forward_only:  # evaluation: nothing requires grad, so no slab is written and no gradient kernel runs
            with torch.no_grad():
                _call(x, y, At, acc)
        else:
            _call(x, y, At, acc).backward()
            x.grad = At.grad = None

    for _ in range(3):
        step()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    flop = (1 if forward_only else 3) * (2 * N * H * V + 3 * N * V)
    return flop * 1e-12 / (ms * 1e-3)


def memory_point(N, H, V, acc):
    x, y, At = _inputs(N, H, V, acc, low_loss=False)
    _call(x, y, At, acc).backward()
    x.grad = At.grad = None
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    _call(x, y, At, acc).backward()
    torch.cuda.synchronize()
    return (torch.cuda.max_memory_allocated() - before) / 1024 ** 3


def _reference_fp64(x, y, At, chunk=512):
    """float64 loss and gradients, rows in chunks so that only chunk x V logits are alive."""
    xd = x.detach().double()
    Ad = At.detach().double()
    N = xd.shape[0]
    dx = torch.empty_like(xd)
    dA = torch.zeros_like(Ad)
    total = torch.zeros((), dtype=torch.float64, device=x.device)
    for r0 in range(0, N, chunk):
        z = xd[r0:r0 + chunk] @ Ad
        lse = torch.logsumexp(z, dim=-1)
        yy = y[r0:r0 + chunk]
        total += (lse - z.gather(1, yy[:, None])[:, 0]).sum()
        dz = torch.exp(z - lse[:, None])
        dz.scatter_add_(1, yy[:, None], -torch.ones_like(yy[:, None], dtype=torch.float64))
        dx[r0:r0 + chunk] = dz @ Ad.t() / N
        dA += xd[r0:r0 + chunk].t() @ dz / N
    return total / N, dx, dA


def accuracy_point(N, H, V, acc):
    x, y, At = _inputs(N, H, V, acc, low_loss=True)
    ref_loss, ref_dx, ref_dA = _reference_fp64(x, y, At)
    loss = _call(x, y, At, acc)
    loss.backward()
    torch.cuda.synchronize()
    loss_err = torch.dist(loss.double(), ref_loss).item()
    x_err = torch.dist(x.grad.double(), ref_dx).item()
    a_err = torch.dist(At.grad.double(), ref_dA).item()
    return loss_err, 0.5 * (x_err + a_err)


def file_name(mode, acc, var, sub=None):
    tail = "Defaults: N=B*S=16384, H=2048, V=131072.csv"
    if mode == "speed":
        return f"{acc} fwd-bwd-Linear+Loss Performance over {var}. {tail}"
    if mode == "memory":
        return f"{acc} fwd-bwd-Linear+Loss Memory Peak over {var}. {tail}"
    return f" {sub} {acc} Linear+Loss Accuracy over {var}. {tail}"


def write_csv(path: Path, var, rows):
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow([var, PROVIDER])
        for xval, val in rows:
            w.writerow([f"{float(xval):f}", "" if val is None else f"{val:f}"])


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mode", choices=["speed", "memory", "accuracy"], required=True)
    ap.add_argument("--over", nargs="+", default=["H", "N", "V"], choices=["H", "N", "V"])
    ap.add_argument("--acc", nargs="+", default=["fp16", "bf16"], choices=["fp16", "bf16", "fp16-mixed"])
    ap.add_argument("--out", default="sweeps_out")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--quick", action="store_true", help="every other point of each range")
    ap.add_argument("--forward-only", action="store_true",
                    help="speed mode: time the loss under torch.no_grad() (one third of the flop count); CSVs go to "
                         "bench-fwd/ (the reference has no such sweep)")
    args = ap.parse_args()
    out = Path(args.out) / {"speed": "bench", "memory": "bench-mem", "accuracy": "bench-acc"}[args.mode]
    if args.forward_only:
        assert args.mode == "speed", "--forward-only goes with --mode speed"
        out = Path(args.out) / "bench-fwd"

    for acc in args.acc:
        for var in args.over:
            exps = list(RANGES[args.mode][var])
            if args.quick:
                exps = exps[::2]
            rows, rows_bwd = [], []
            for e in exps:
                shape = dict(DEFAULTS)
                shape[var] = 2 ** e
                try:
                    if args.mode == "speed":
                        rows.append((shape[var], speed_point(shape["N"], shape["H"], shape["V"], acc, args.reps,
                                                             args.forward_only)))
                    elif args.mode == "memory":
                        rows.append((shape[var], memory_point(shape["N"], shape["H"], shape["V"], acc)))
                    else:
                        fwd, bwd = accuracy_point(shape["N"], shape["H"], shape["V"], acc)
                        rows.append((shape[var], fwd))
                        rows_bwd.append((shape[var], bwd))
                except (RuntimeError, AssertionError) as err:  # e.g. out of memory: leave the cell empty
                    print(f"{args.mode} {acc} {var}={shape[var]}: {type(err).__name__}: {err}")
                    rows.append((shape[var], None))
                    if args.mode == "accuracy":
                        rows_bwd.append((shape[var], None))
                torch.cuda.empty_cache()
                print(f"{args.mode} {acc} {var}={shape[var]}: {rows[-1][1]}"
                      + (f" / {rows_bwd[-1][1]}" if rows_bwd else ""), flush=True)
            if args.mode == "accuracy":
                write_csv(out / file_name("accuracy", acc, var, "fwd"), var, rows)
                write_csv(out / file_name("accuracy", acc, var, "bwd"), var, rows_bwd)
            else:
                write_csv(out / file_name(args.mode, acc, var), var, rows)


if __name__ == "__main__":
    main()
