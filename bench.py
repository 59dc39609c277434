#!/usr/bin/env python
"""Benchmark of the fused linear + cross-entropy path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME] [--scaling weak|strong]

A step is one forward+backward of ``linear_cross_entropy`` over one batch of synthetic inputs (loss, dx and dW),
the quantity the reference's own benchmark times (bench_fusions.py:261-266 of the reference). The metric is the
reference's: fwd+bwd TFLOP/s = 6*N*H*V / t. One JSON line is printed by rank 0.

N = 1: the default point of the reference's sweeps in bf16 (N=16384, H=2048, V=131072, N_chunk_size=4096).
N > 1 (launched by torch.distributed.run, one rank per GPU): the weight is sharded by vocabulary columns over the
ranks (linear_cross_entropy_loss_b200/sharded.py). ``--scaling weak`` (default) keeps one 131072-column slab per
rank, so the global vocabulary is N_gpus * 131072; ``--scaling strong`` shards the named configuration itself.

``--impl reference`` times the reference's torch statement of the path (float32, CPU, all host threads) through
the oracle's port of it on a bounded sample of the same workload; rank 0 only.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "fwd+bwd TFLOP/s (6NHV/t)"
# published number for this metric at the default point in bf16 (fused Triton kernel, unknown 48 GB GPU):
# reference file "bench/bf16 fwd-bwd-Linear+Loss Performance over N. ...csv", line 8
PUBLISHED_BF16_DEFAULT_TFLOPS = 86.75
# fallback roofline denominators when the measured-peaks file is absent (earlier measurement on this pool)
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of each contraction kernel, from ncu
# captures of the quarter-size case (N=4096, H=2048, V=32768, bf16; summary kept under profiles/). All three grow in
# proportion to V; the figures are scaled by V_local / 32768 at run time (only for N_chunk_size=4096, H=2048, which
# the captures used). dW: average over the four launches of a four-chunk pass (the first writes the sum and residual
# arrays, the middle ones read and write both, the last reads both and writes the sum), from the two-chunk capture.
NCU_DRAM_BYTES_V32768 = {"fwd": 388.3e6, "dx": 735.7e6, "dw": 728.6e6}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", default="headline_bf16")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--n-chunk-size", type=int, default=0,
                    help="override the configuration's N_chunk_size (0 = keep it; the metric's point uses 4096)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (N=1, rank 0)")
    ap.add_argument("--no-parity", action="store_true",
                    help="skip the float64 check of the last timed step's loss and gradients (after the timed region)")
    ap.add_argument("--no-strong", action="store_true",
                    help="skip the short strong-scaling sub-record on the 65536 x 4096 x 131072 LM-head configuration")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU work of the baseline leg")
    ap.add_argument("--triton-ref", choices=["full", "trimmed", "off"], default="full",
                    help="N=1: also time the reference's own Triton op on this GPU (outside the timed region of the "
                         "CUDA path) with its full autotune lists, with lists trimmed to three entries each, or not")
    ap.add_argument("--ref-budget", type=float, default=100.0,
                    help="--impl reference: seconds of CPU work over all warm-up and timed steps together")
    return ap.parse_args()


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi polling in the background; only the samples taken inside [mark_start, mark_end] count."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    @staticmethod
    def _parse_time(text):
        import datetime
        try:
            return datetime.datetime.strptime(text.strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 10:
                continue
            ts = self._parse_time(parts[0])
            if ts is not None and self.t0 is not None and self.t1 is not None and not (self.t0 <= ts <= self.t1 + 0.05):
                continue
            try:
                sm.append(float(parts[2]))
                smax.append(float(parts[3]))
                power.append(float(parts[4]))
            except ValueError:
                continue
            for name, val in zip(names, parts[6:10]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v.strip() for v in vis.split(",") if v.strip()]
        if local_rank < len(ids) and ids[local_rank].isdigit():
            return int(ids[local_rank])
    return local_rank


# ---------------------------------------------------------------------------------------------------
# CPU legs (the reference's torch path, ported in oracle/oracle.py)
# ---------------------------------------------------------------------------------------------------
def cpu_reference_rate(cfg, seconds, steps=1, warmup=0):
    """Times oracle.cpu_baseline_step on a bounded row/column sample of cfg. Returns (tflops, ms_per_step, info)."""
    import torch

    from oracle import oracle

    torch.manual_seed(0)
    # all host cores this process may use (torchrun exports OMP_NUM_THREADS=1 for multi-rank launches)
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    if torch.get_num_threads() < avail:
        torch.set_num_threads(avail)
    cores = torch.get_num_threads()
    V = min(cfg.V, 131072)
    H = cfg.H
    g = torch.Generator().manual_seed(cfg.seed)
    W = torch.randn(H, V, generator=g).clamp_(-2, 2).mul_(H ** -0.5)

    def run(rows):
        x = torch.randn(rows, H, generator=g)
        y = torch.randint(0, V, (rows,), generator=g)
        y[torch.rand(rows, generator=g) < cfg.frac_ignored] = cfg.ignore_index
        t0 = time.perf_counter()
        oracle.cpu_baseline_step(x, y, W, cfg.ignore_index, cfg.z_regularization, cfg.logit_scale,
                                 chunk_rows=min(rows, 1024))
        return time.perf_counter() - t0

    run(128)                                   # touches the pages, spins up the thread pool
    t = run(128)
    rate = 6.0 * 128 * H * V / t               # flop/s estimate
    rows = int(seconds * rate / (6.0 * H * V)) // 128 * 128
    rows = max(128, min(rows, cfg.N))
    for _ in range(warmup):
        run(rows)
    times = [run(rows) for _ in range(max(1, steps))]
    t = sum(times) / len(times)
    tflops = 6.0 * rows * H * V / t / 1e12
    info = {"kind": "port", "cores": cores, "value": tflops, "unit": "TFLOP/s",
            "sample": f"{rows} of {cfg.N} rows x H={H} x {V} of {cfg.V} vocabulary columns per step, float32, "
                      f"torch CPU F.linear + F.cross_entropy + autograd (the reference's reference_torch), "
                      f"{len(times)} timed step(s)"}
    return tflops, t * 1e3, info


def triton_reference_leg(cfg, x, y, W, mode):
    """Times the reference's own Triton implementation (unmodified, from oracle/_ref) on the same inputs, on this GPU.
    A baseline leg like cpu_baseline: it runs after the CUDA path's timed regions and never touches them."""
    try:
        import triton

        from oracle import ref_triton

        ref_triton.load()
        if mode == "trimmed":
            ref_triton.trim_configs()
        ms, loss, chosen = ref_triton.time_fwd_bwd(
            x.detach(), y, W.detach(), cfg.ignore_index, cfg.z_regularization, cfg.logit_scale, cfg.N_chunk_size,
            cfg.monitoring, steps=10, warmup=3)
        return {"tflops": cfg.flops / (ms * 1e-3) / 1e12, "ms_per_step": ms, "loss": loss,
                "triton_version": triton.__version__, "autotune_lists": mode, "chosen_configs": chosen,
                "note": "reference linear_cross_entropy (Triton kernels JIT-compiled for this GPU), forward+backward, "
                        "10 steps after the autotune call and 3 warm-up calls, CUDA events"}
    except Exception as err:  # noqa: BLE001 -- not installed, Triton cannot compile for this GPU, out of resources ...
        return {"unavailable": f"reference Triton unavailable on this box: {type(err).__name__}: {err}"[:600]}


def parity_record(cfg, x, y, W, dx, dW, loss_value, rank, world, v_local):
    """Correctness of the very tensors the timed steps produced, checked here in float64 (rows / columns subsets) and
    float32-product / float64-reduction (the loss over all rows), with plain torch on the GPU. At world > 1 every
    rank handles its own vocabulary slab and the pieces are combined with NCCL collectives, so this also covers the
    sharded data path (row partials exchange, dx reduction) in the run that is being timed.
    Returns {"loss_rel_err", "dx_cos", "dw_cos", "ok"}; tolerances: loss 1e-3 relative, cosines 0.9999."""
    import torch
    import torch.distributed as dist

    dev = x.device
    N, H = x.shape
    scale, zreg, ign = cfg.logit_scale, cfg.z_regularization, cfg.ignore_index
    off = rank * v_local
    valid = y != ign
    n_valid = int(valid.sum())
    y_loc = y - off
    owned = valid & (y_loc >= 0) & (y_loc < v_local)

    def all_sum(t):
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t

    def all_max(t):
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t

    # log-sum-exp and target logit of every row: float32 products (no TF32), float64 reductions
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    Wf = W.detach().float()
    m_loc = torch.empty(N, dtype=torch.float64, device=dev)
    s_loc = torch.empty(N, dtype=torch.float64, device=dev)
    t_loc = torch.zeros(N, dtype=torch.float64, device=dev)
    for r0 in range(0, N, 1024):
        z = (x[r0:r0 + 1024].detach().float() @ Wf).double() * scale
        m = z.max(dim=1).values
        m_loc[r0:r0 + 1024] = m
        s_loc[r0:r0 + 1024] = torch.exp(z - m[:, None]).sum(dim=1)
        o = owned[r0:r0 + 1024]
        t_loc[r0:r0 + 1024][o] = z[o, y_loc[r0:r0 + 1024][o]]
        del z
    del Wf
    torch.backends.cuda.matmul.allow_tf32 = prev
    m_all = all_max(m_loc.clone())
    lse = m_all + torch.log(all_sum(s_loc * torch.exp(m_loc - m_all)))
    t_all = all_sum(t_loc)
    want_loss = (((lse - t_all) * valid).sum() + zreg * ((lse * lse) * valid).sum()).item() / n_valid
    loss_rel = abs(loss_value - want_loss) / abs(want_loss)

    # dx of 32 rows (same rows on every rank) in float64
    g = torch.Generator().manual_seed(1234)
    rows = torch.randperm(N, generator=g)[:32].to(dev)
    xs = x[rows].detach().double()
    dx_rows = torch.zeros((32, H), dtype=torch.float64, device=dev)
    for v0 in range(0, v_local, 16384):
        Wb = W[:, v0:v0 + 16384].detach().double()
        z = (xs @ Wb) * scale
        dz = torch.exp(z - lse[rows][:, None]) * (1 + 2 * zreg * lse[rows])[:, None]
        yl = y_loc[rows] - v0
        hit = owned[rows] & (yl >= 0) & (yl < Wb.shape[1])
        dz[hit.nonzero()[:, 0], yl[hit]] -= 1
        dz *= valid[rows].double()[:, None]
        dx_rows += dz @ Wb.T
    dx_rows = all_sum(dx_rows) * (scale / n_valid)
    got = dx[rows].double()
    dx_cos = float((got * dx_rows).sum() / (got.norm() * dx_rows.norm() + 1e-300))

    # 64 columns of this rank's dW in float64 (its four most frequent label columns among them, when it owns some)
    cols = torch.cat([torch.arange(4), torch.randperm(v_local - 4, generator=g)[:60] + 4]).to(dev)
    Wc = W[:, cols].detach().double()
    want_dw = torch.zeros((H, 64), dtype=torch.float64, device=dev)
    for r0 in range(0, N, 8192):
        xb = x[r0:r0 + 8192].detach().double()
        l = lse[r0:r0 + 8192]
        dz = torch.exp((xb @ Wc) * scale - l[:, None]) * (1 + 2 * zreg * l)[:, None]
        dz -= (y_loc[r0:r0 + 8192][:, None] == cols[None, :]).double()
        dz *= valid[r0:r0 + 8192].double()[:, None]
        want_dw += xb.T @ dz
    want_dw *= scale / n_valid
    got = dW[:, cols].double()
    cos_t = torch.stack([(got * want_dw).sum(), (got * got).sum(), (want_dw * want_dw).sum()])
    cos_t = all_sum(cos_t)  # one cosine over the columns of all ranks
    dw_cos = float(cos_t[0] / (cos_t[1].sqrt() * cos_t[2].sqrt() + 1e-300))
    ok = loss_rel <= 1e-3 and dx_cos >= 0.9999 and dw_cos >= 0.9999
    return {"loss_rel_err": loss_rel, "dx_cos": dx_cos, "dw_cos": dw_cos, "ok": bool(ok),
            "checked": "loss over all rows (fp32 products, fp64 reductions); dx of 32 rows and 64 dW columns per rank "
                       "in float64; tolerances 1e-3 / 0.9999 / 0.9999"}


def run_reference_arm(args, cfg, n_gpus):
    per_step = max(0.25, args.ref_budget / max(1, args.steps + args.warmup))
    tflops, ms, info = cpu_reference_rate(cfg, per_step, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling if n_gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(cfg, n_gpus, args),
        "cpu_baseline": info,
        "ms_per_step_note": "a step of this arm is one bounded row sample (cpu_baseline.sample), not the whole "
                            "workload: only the rate compares with the GPU arm, and it scales with cpu_baseline.cores",
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def config_dict(cfg, n_gpus, args):
    return {
        "workload": f"{cfg.name}: N={cfg.N} H={cfg.H} V={cfg.V} {str(cfg.dtype).split('.')[-1]} "
                    f"N_chunk_size={cfg.N_chunk_size} logit_scale={cfg.logit_scale} "
                    f"z_regularization={cfg.z_regularization} monitoring={cfg.monitoring}",
        "N": cfg.N, "H": cfg.H, "V": cfg.V, "N_chunk_size": cfg.N_chunk_size,
        "vocab_sharding": f"{n_gpus} x {cfg.V // n_gpus} columns" if n_gpus > 1 else "none",
        "dx_exchange": ("none" if n_gpus == 1 else
                        "peer stores fused into the dx contraction" if os.environ.get("LCE_PEER_DX") == "1"
                        else "NCCL all-reduce per chunk, in stream order" if os.environ.get("LCE_DX_REDUCE") == "chunk"
                        else "one NCCL all-reduce of dx per pass"
                        + (" (fp32 partial sums for fp16 inputs)" if str(cfg.dtype) == "torch.float16" else "")),
        "row_partials_exchange": ("none" if n_gpus == 1 else
                                  "NCCL all-gather per chunk" if (os.environ.get("LCE_PEER_PARTS", "0") != "1"
                                                                  or os.environ.get("LCE_PEER_DX") == "1")
                                  else "stores into peer memory + flags, chunks software-pipelined on two slabs"),
        "l2": "inputs larger than L2 (the weight alone is >= 512 MiB per GPU); no explicit flush",
        "gemm_variant": "CTA-pair 256x256 tiles",
    }


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.gpus > 1 and world == 1 and args.impl == "ours":
        # convenience: relaunch under torch.distributed.run, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 400), str(Path(__file__))]
        sys.exit(subprocess.call(cmd + sys.argv[1:]))

    from linear_cross_entropy_loss_b200 import synthetic

    n_gpus = max(args.gpus, world)
    base = synthetic.CONFIGS[args.config]
    if args.n_chunk_size > 0:
        base = synthetic.scaled(base, N_chunk_size=args.n_chunk_size, name=f"{base.name}_chunk{args.n_chunk_size}")
    cfg = base
    if n_gpus > 1 and args.scaling == "weak":
        cfg = synthetic.scaled(base, V=base.V * n_gpus, name=f"{base.name}_x{n_gpus}vocab")

    if args.impl == "reference":
        if rank == 0:
            run_reference_arm(args, cfg, n_gpus)
        return

    import torch
    import torch.distributed as dist

    from linear_cross_entropy_loss_b200 import _native, linear_cross_entropy
    from linear_cross_entropy_loss_b200.sharded import linear_cross_entropy_sharded

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sharded = world > 1
    if sharded:
        dist.init_process_group("nccl", device_id=dev)
    v_local = cfg.V // world
    x, y, W = synthetic.make_inputs(cfg, device=dev,
                                    vocab_slice=(rank * v_local, (rank + 1) * v_local) if sharded else None)
    x.requires_grad_(True)
    W.requires_grad_(True)

    def fwd_bwd(xx, yy, keep_grads=False):
        if sharded:
            loss = linear_cross_entropy_sharded(xx, yy, W, None, cfg.ignore_index, cfg.z_regularization,
                                                cfg.logit_scale, cfg.N_chunk_size, cfg.monitoring)[0]
        else:
            loss = linear_cross_entropy(xx, yy, W, cfg.ignore_index, cfg.z_regularization, cfg.logit_scale,
                                        cfg.N_chunk_size, cfg.monitoring)[0]
        loss.backward()
        if not keep_grads:
            xx.grad = None
            W.grad = None
        return loss

    def barrier():
        if sharded:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if not sharded:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # ---- device-resident throughput -----------------------------------------------------------------
    sampler = ClockSampler(physical_gpu_index(local_rank))
    if rank == 0:
        sampler.start()   # started before the warm-up so that it is polling by the time the timed region begins
    for _ in range(max(3, args.warmup)):
        warm_loss = fwd_bwd(x, y)
    barrier()
    # a pass that is not finite after the warm-up (for instance an exchange between ranks that timed out: the library
    # then returns NaN) is not worth timing: every rank learns of it and the run ends with an error instead
    bad = torch.tensor([0.0 if math.isfinite(warm_loss.item()) else 1.0], device=dev)
    if sharded:
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    if bad.item() != 0:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "error": "the loss of a warm-up step is not finite", "n_gpus": world}),
                  flush=True)
        if sharded:
            dist.destroy_process_group()
        sys.exit(4)
    torch.cuda.reset_peak_memory_stats()
    mem_before = torch.cuda.memory_allocated()
    _native.profile_read()
    _native.profile_enable(True)
    launches_before = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark_start()
    e0.record()
    marks = []
    for i in range(args.steps):
        loss = fwd_bwd(x, y, keep_grads=(i == args.steps - 1))  # the last timed step's gradients are checked below
        marks.append(torch.cuda.Event(enable_timing=True))
        marks[-1].record()                                       # per-step durations for the quantiles (no sync)
    e1.record()
    barrier()
    sampler.mark_end()
    launches = _native.launch_count() - launches_before
    _native.profile_enable(False)
    kernel_ms, kernel_launches = _native.profile_read()
    # every rank's own time inside the three contractions per step: with a sharded run the step is set by the slowest
    # rank (each GPU settles at its own clock under its power cap), and this shows how far apart the ranks are
    mine = torch.tensor([sum(kernel_ms.values()) / args.steps], dtype=torch.float64, device=dev)
    if sharded:
        all_ranks = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(all_ranks, mine)
        rank_contraction_ms = [round(t.item(), 3) for t in all_ranks]
    else:
        rank_contraction_ms = [round(mine.item(), 3)]
    clocks = sampler.stop() if rank == 0 else None
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = ms_total / args.steps
    per_step = sorted(a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks))  # this rank's steps
    quantiles = [per_step[min(len(per_step) - 1, int(q * len(per_step)))] for q in (0.2, 0.5, 0.8)]
    peak_extra = torch.cuda.max_memory_allocated() - mem_before
    value = cfg.flops / (ms_per_step * 1e-3) / 1e12
    loss_value = loss.item()
    parity = None
    if not args.no_parity:
        parity = parity_record(cfg, x, y, W, x.grad, W.grad, loss_value, rank, world, v_local)
    x.grad = None
    W.grad = None

    # ---- end to end through the public call, inputs in pinned host memory ------------------------------
    # Input pipeline as a training loop would have it: two device buffers; the copy of step i+1's inputs is issued
    # on a copy stream while step i computes. Every step's x and y still cross PCIe inside the timed region, and
    # every step ends with the device -> host read of its loss.
    x_host = x.detach().to("cpu").pin_memory()
    y_host = y.to("cpu").pin_memory()
    bufs = [(torch.empty_like(x_host, device=dev).requires_grad_(True), torch.empty_like(y_host, device=dev))
            for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    compute_stream = torch.cuda.current_stream(dev)
    copied = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]

    def upload(i):
        xb, yb = bufs[i % 2]
        with torch.cuda.stream(copy_stream), torch.no_grad():
            copy_stream.wait_event(consumed[i % 2])      # the step that last used this buffer pair is done with it
            xb.copy_(x_host, non_blocking=True)
            yb.copy_(y_host, non_blocking=True)
            copied[i % 2].record(copy_stream)

    def e2e_run(n):
        for ev in consumed:
            ev.record(compute_stream)
        upload(0)
        for i in range(n):
            if i + 1 < n:
                upload(i + 1)
            compute_stream.wait_event(copied[i % 2])
            xb, yb = bufs[i % 2]
            loss_i = fwd_bwd(xb, yb)
            consumed[i % 2].record(compute_stream)
            loss_i.item()                                 # device -> host read of the loss

    e2e_run(3)
    barrier()
    e0.record()
    e2e_run(args.steps)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    e2e_value = cfg.flops / (e2e_ms * 1e-3) / 1e12

    # ---- roofline of the dominant kernel --------------------------------------------------------------
    peaks, peak_source = load_peaks()
    peak_tflops = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    # each of the three contractions does 2*N*H*V_local flop per step, spread over its launches of that step
    per_step_flops = 2.0 * cfg.N * cfg.H * v_local
    kernels = {}
    for k in ("fwd", "dx", "dw"):
        if kernel_launches[k] > 0:
            per_step = kernel_launches[k] / args.steps
            avg_ms = kernel_ms[k] / kernel_launches[k]
            kernels[k] = {"launches_per_step": per_step, "avg_ms": avg_ms,
                          "flops_per_launch": per_step_flops / per_step,
                          "tflops": per_step_flops / per_step / (avg_ms * 1e-3) / 1e12,
                          "share_of_step": kernel_ms[k] / (ms_per_step * args.steps)}
    dominant = max(kernels, key=lambda k: kernels[k]["avg_ms"] * kernels[k]["launches_per_step"]) if kernels else None
    roofline = None
    if dominant is not None:
        achieved = kernels[dominant]["tflops"]
        base = NCU_DRAM_BYTES_V32768.get(dominant)
        traffic = (base * v_local / 32768.0) if (base and cfg.H == 2048 and min(cfg.N, cfg.N_chunk_size) == 4096) \
            else None
        roofline = {"bound": "tensor", "kernel": f"lce_gemm_pair_kernel[{dominant}]", "achieved": achieved,
                    "peak": peak_tflops, "unit": "TFLOP/s", "frac": achieved / peak_tflops,
                    "peak_source": f"{peak_source} cuBLAS bf16 GEMM, sustained",
                    "traffic": traffic,
                    "flops_per_launch": kernels[dominant]["flops_per_launch"], "kernels": kernels,
                    "whole_step_frac": (value / world) / peak_tflops}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
        "ms_per_step_quantiles": {"p20": quantiles[0], "p50": quantiles[1], "p80": quantiles[2],
                                  "note": "rank 0's individual steps (the reference's benchmark reports median and "
                                          "20 / 80 % quantiles, bench_fusions.py:271,280)"},
        "higher_is_better": True,
        "scaling": args.scaling if world > 1 else "weak",
        "vs_baseline": value / PUBLISHED_BF16_DEFAULT_TFLOPS if (world == 1 and cfg.name == "headline_bf16") else None,
        "dtype": str(cfg.dtype).split(".")[-1].replace("bfloat16", "bf16").replace("float16", "f16").replace("float32", "tf32"),
        "data": "synthetic", "config": config_dict(cfg, world, args), "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": x_host.numel() * x_host.element_size() + y_host.numel() * 8,
                "d2h_bytes_per_step": 4},
        "gpu_launches": launches, "roofline": roofline, "loss": loss_value, "parity": parity,
        "contraction_ms_per_step_by_rank": rank_contraction_ms,
        "peak_extra_bytes": peak_extra, "peak_budget_bytes": min(cfg.N, cfg.N_chunk_size) * v_local * 4,
        # the same without the gradients the caller receives and the residual array of dW (together what the
        # reference's fp32 gradient buffers hold)
        "peak_extra_bytes_excl_grads": peak_extra - cfg.N * cfg.H * x.element_size()
        - cfg.H * v_local * (4 if cfg.N > cfg.N_chunk_size else W.element_size()),
    }

    if rank == 0 and world == 1 and args.triton_ref != "off":
        line["triton_reference"] = triton_reference_leg(cfg, x, y, W, args.triton_ref)
    if not args.no_strong and args.config == "headline_bf16":
        # The configuration the 8-GPU scaling target is quoted on (65536 x 4096 x 131072, bf16, Zipf labels), with
        # its vocabulary split over the ranks: total work fixed, so value(N) / (N * value(1)) is the strong-scaling
        # efficiency. A short run (2 warm-up + 3 timed steps) beside the main measurement.
        del x, y, W, bufs, x_host, y_host
        torch.cuda.empty_cache()
        c4 = synthetic.CONFIGS["c4_llama8b_bf16"]
        vl4 = c4.V // world
        x4, y4, W4 = synthetic.make_inputs(c4, device=dev, vocab_slice=(rank * vl4, (rank + 1) * vl4) if sharded else None)
        x4.requires_grad_(True)
        W4.requires_grad_(True)

        def step4():
            if sharded:
                l4 = linear_cross_entropy_sharded(x4, y4, W4, None, c4.ignore_index, c4.z_regularization,
                                                  c4.logit_scale, c4.N_chunk_size, c4.monitoring)[0]
            else:
                l4 = linear_cross_entropy(x4, y4, W4, c4.ignore_index, c4.z_regularization, c4.logit_scale,
                                          c4.N_chunk_size, c4.monitoring)[0]
            l4.backward()
            x4.grad = None
            W4.grad = None
            return l4

        for _ in range(2):
            step4()
        barrier()
        e0.record()
        for _ in range(3):
            l4 = step4()
        e1.record()
        barrier()
        ms4 = max_over_ranks(e0.elapsed_time(e1)) / 3
        line["strong_scaling_c4"] = {"config": "c4_llama8b_bf16: N=65536 H=4096 V=131072 bf16 N_chunk_size=8192, "
                                               f"vocabulary split over {world} rank(s)",
                                     "value": c4.flops / (ms4 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms4,
                                     "steps": 3, "warmup": 2, "scaling": "strong", "loss": l4.item()}
        del x4, y4, W4
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        _, _, info = cpu_reference_rate(cfg, args.cpu_seconds)
        line["cpu_baseline"] = info
    if rank == 0:
        print(json.dumps(line), flush=True)
    if sharded:
        dist.barrier()
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        sys.exit(3)  # the timed steps produced results outside the stated tolerance


if __name__ == "__main__":
    main()
