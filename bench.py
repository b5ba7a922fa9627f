#!/usr/bin/env python
"""Headline benchmark of the sampling hot path: sampled rows/s at 1024 x 262144 f32 logits with penalties + top-k + top-p
(+ min-p), per GPU, rows sharded across N GPUs with no data-path collective (weak scaling: 1024 rows per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W]                    # this library on the GPU(s)
    python bench.py --impl reference [--gpus N] [--steps K] [--warmup W]   # the reference's CPU sampler on the host cores
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...       # N > 1: one rank per GPU

Prints ONE JSON line (rank 0).  `value` is rows/s with the logits already in HBM; `e2e` is rows/s through
whirl_sample_rows_host with pinned HOST logits, every copy inside the timed region; `roofline` compares the algorithmic
bytes of one step with the measured HBM copy bandwidth; `cpu_baseline` is the CPU oracle timed on a bounded sample.
Synthetic inputs stand in for real logits: N(0, 2.5^2) rows and Zipf(1.1) token histories, seeded.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIST = 4096
SETTINGS = dict(rep=1.1, pres=0.5, freq=0.3, temp=0.8, top_k=50, top_p=0.9, min_p=0.05)


def algorithmic_bytes_per_row(vocab: int, esize: int, hist: int) -> int:
    # the logits once + the history ids + the uniform; the 4-byte token is ignored
    return vocab * esize + 4 * hist + 8


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def splitmix_u01(seed: int, idx: np.ndarray) -> np.ndarray:
    """The reference's counter-hash uniform (Sampler::uniform) for output indices idx, vectorised."""
    m = np.uint64(0xFFFFFFFFFFFFFFFF)
    with np.errstate(over="ignore"):
        z = (np.uint64(seed) + (idx.astype(np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)) & m
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return (z >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                       "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except Exception:
            self.p.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [t.strip() for t in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for nme, v in zip(names, f[2:6]):
                if v == "Active":
                    reasons.add(nme)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": float(np.max(mx)) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs(torch, device, rows, vocab, dtype, nbuf, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    xs = []
    for _ in range(nbuf):
        x = torch.empty((rows, vocab), dtype=torch.float32, device=device)
        x.normal_(0.0, 2.5, generator=g)
        xs.append(x if dtype == "f32" else x.to(torch.bfloat16))
    # Zipf(1.1) ranks by the inverse CDF of the continuous power law, scattered over the id space
    u = torch.rand((rows, HIST), generator=g, device=device, dtype=torch.float64)
    a = 1.0 - 1.1
    hi = float(vocab + 1) ** a
    rank = torch.floor((1.0 + u * (hi - 1.0)) ** (1.0 / a)).to(torch.int64) - 1
    rank.clamp_(0, vocab - 1)
    hist = ((rank * 2654435761 + seed) % vocab).to(torch.int32).contiguous()
    return xs, hist


def run_ours(args):
    import torch
    from whirl_llm_b200 import api

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    rows, vocab, esize = args.rows, args.vocab, (4 if args.dtype == "f32" else 2)
    nbuf = 3
    xs, hist = make_inputs(torch, dev, rows, vocab, args.dtype, nbuf, 1234 + rank)
    f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device=dev)
    us = [torch.from_numpy(splitmix_u01(1234 + rank, np.arange(rows) + b * rows)).to(dev) for b in range(nbuf)]
    base = dict(inv_t=f32(1.0 / SETTINGS["temp"]), top_k=torch.full((rows,), SETTINGS["top_k"], dtype=torch.int32, device=dev),
                top_p=torch.full((rows,), SETTINGS["top_p"], dtype=torch.float64, device=dev),
                min_p=torch.full((rows,), SETTINGS["min_p"], dtype=torch.float64, device=dev),
                hist=hist, hist_len=torch.full((rows,), HIST, dtype=torch.int32, device=dev),
                rep=f32(SETTINGS["rep"]), pres=f32(SETTINGS["pres"]), freq=f32(SETTINGS["freq"]))
    base["top_k"].fill_(args.top_k)
    if args.no_penalties:
        for k in ("hist", "hist_len", "rep", "pres", "freq"):
            base[k] = None
    if args.greedy:
        base["greedy"] = torch.ones(rows, dtype=torch.uint8, device=dev)
    params = [api.RowParams(u=us[b], **base) for b in range(nbuf)]
    ws = torch.zeros(api.workspace_bytes(rows, vocab), dtype=torch.uint8, device=dev)
    # tokens only, as a serving engine asks: no row statistics, so rows closed by their top_k skip the normaliser
    res = api.sample_rows(xs[0], params[0], ws=ws, want_stats=False)
    torch.cuda.synchronize()
    assert int((res.status != 0).sum().item()) == 0, "unresolved rows in the benchmark workload"

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def step(i):
        api.sample_rows(xs[i % nbuf], params[i % nbuf], ws=ws, result=res)

    for i in range(args.warmup):
        step(i)
    sync_all()
    clocks = ClockSampler(local)
    lc0 = api.launch_counts()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    sync_all()
    lc1 = api.launch_counts()
    ms = e0.elapsed_time(e1)
    clk = clocks.stop()
    if dist is not None:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = world * rows / (ms_per_step * 1e-3)
    launches = sum(lc1.values()) - sum(lc0.values())

    # ---- end to end: pinned host logits through whirl_sample_rows_host, copies inside the timed region
    if args.no_e2e:
        print(json.dumps({"variant": vars(args), "ms_per_step": ms_per_step, "rows_per_s": value,
                          "frac": rows * algorithmic_bytes_per_row(vocab, esize, 0 if args.no_penalties else HIST) / (ms_per_step * 1e-3) / 1e9 / measured_peak_gbs()[0]}))
        return
    x_host = torch.empty((rows, vocab), dtype=xs[0].dtype).pin_memory()
    x_host.copy_(xs[0])
    hp = {k: (v.cpu().pin_memory() if v is not None else None) for k, v in dict(u=us[0], **base).items()}
    ho = dict(token=torch.empty(rows, dtype=torch.int32).pin_memory())
    e2e_steps = max(1, min(args.steps, 5))
    api.sample_rows_host(x_host, hp, rows, vocab, api.F32 if args.dtype == "f32" else api.BF16, ho, device=local)
    same = bool((ho["token"].to(dev) == api.sample_rows(xs[0], params[0], ws=ws).token).all().item())
    sync_all()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        api.sample_rows_host(x_host, hp, rows, vocab, api.F32 if args.dtype == "f32" else api.BF16, ho, device=local)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([dt], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    e2e_value = world * rows * e2e_steps / dt
    h2d = rows * vocab * esize + sum(v.numel() * v.element_size() for v in hp.values() if v is not None)
    d2h = rows * 4

    # ---- roofline of the dominant kernel (the single-pass sampler; the step's helper launches are inside the time)
    peak, peak_kind = measured_peak_gbs()
    per_row = algorithmic_bytes_per_row(vocab, esize, HIST)
    achieved = rows * per_row / (ms_per_step * 1e-3) / 1e9
    traffic = None
    tp = os.path.join(ROOT, "profiles", "single_pass_kernel_traffic.txt")
    if os.path.exists(tp):
        try:
            tj = json.load(open(tp))
            traffic = float(tj["dram_bytes_per_row"]) * rows
        except Exception:
            traffic = None

    line = {
        "metric": "sampled rows/s at 1024x262144 fp32 logits (penalties + top-k + top-p), % of HBM roofline",
        "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": f"penalised sampling {rows}x{vocab} {args.dtype} per GPU, history {HIST} Zipf(1.1), " +
                               ", ".join(f"{k} {v}" for k, v in SETTINGS.items()),
                   "rows_per_gpu": rows, "vocab": vocab, "parallelism": f"rows sharded x{world}, no collective",
                   "l2": f"{nbuf} rotating logits buffers of {rows * vocab * esize / 2**30:.2f} GiB each (each larger than L2)",
                   "e2e_matches_device_path": same},
        "clocks": clk,
        "e2e": {"value": e2e_value, "unit": "rows/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "steps": e2e_steps},
        "gpu_launches": int(launches),
        "launches_by_kernel": {k: int(lc1[k] - lc0[k]) for k in lc1},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_kind": peak_kind, "algorithmic_bytes_per_row": per_row,
                     "kernel": "single_pass_kernel<float>" if args.dtype == "f32" else "single_pass_kernel<uint16_t>"},
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(xs[0], hist, us[0], rows, vocab, args.dtype)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def cpu_params(n, u):
    f = lambda v, dt=np.float32: np.full(n, v, dtype=dt)
    return dict(inv_t=f(1.0 / SETTINGS["temp"]), top_k=f(SETTINGS["top_k"], np.uint32), top_p=f(SETTINGS["top_p"], np.float64),
                min_p=f(SETTINGS["min_p"], np.float64), u=u, hist_len=f(HIST, np.uint32), rep=f(SETTINGS["rep"]),
                pres=f(SETTINGS["pres"]), freq=f(SETTINGS["freq"]))


def cpu_baseline(x_dev, hist_dev, u_dev, rows, vocab, dtype):
    """The CPU oracle (a port of the reference's host path plus this build's penalties) on a bounded sample of the same
    rows, all host cores."""
    from oracle import oracle as orc
    o = orc.Oracle()
    cores = os.cpu_count() or 1
    n = int(min(rows, max(8, cores * 2)))
    x = x_dev[:n].float().cpu().numpy()
    hist = hist_dev[:n].cpu().numpy()
    u = u_dev[:n].cpu().numpy()
    t0 = time.perf_counter()
    o.sample_rows(x, threads=cores, hist=hist, **cpu_params(n, u))
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": "rows/s", "cores": cores, "kind": "port",
            "sample": f"{n} rows of the same workload, one pass, {cores} threads"}


def run_reference(args):
    """The reference's own CPU sampler (oracle/_ref: SampleBuffers -> filterCands -> sampleRow over its host top-k) on the
    host cores.  The reference has no penalties: the oracle's penalty rule is applied to the rows first (a cheap O(H)
    step), then the reference code samples.  Falls back to the oracle port where oracle/_ref was not built."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from oracle import oracle as orc
    cores = os.cpu_count() or 1
    o = orc.Oracle()
    ref = orc.Reference() if orc.have_reference() else None
    rows, vocab = args.rows, args.vocab
    n = int(min(rows, max(8, cores)))
    rng = np.random.default_rng(1234)
    x = (rng.standard_normal((n, vocab), dtype=np.float32) * np.float32(2.5))
    a = 1.0 - 1.1
    rank_ = np.floor((1.0 + rng.random((n, HIST)) * (float(vocab + 1) ** a - 1.0)) ** (1.0 / a)).astype(np.int64) - 1
    hist = ((np.clip(rank_, 0, vocab - 1) * 2654435761 + 1234) % vocab).astype(np.int32)

    def step(i):
        u = splitmix_u01(1234, np.arange(n) + i * n)
        if ref is not None:
            xp = x.copy()
            for r in range(n):
                xp[r], _ = o.apply_penalties(xp[r], hist[r], SETTINGS["rep"], SETTINGS["pres"], SETTINGS["freq"])
            p = cpu_params(n, None)
            ref.sample_rows(xp, threads=cores, inv_t=p["inv_t"], top_k=p["top_k"], top_p=p["top_p"], min_p=p["min_p"],
                            seed=np.full(n, 1234, np.uint64), pos_idx=(np.arange(n) + i * n).astype(np.uint64))
        else:
            o.sample_rows(x, threads=cores, hist=hist, **cpu_params(n, u))

    for i in range(min(args.warmup, 1)):
        step(i)
    steps = min(args.steps, 5)
    t0 = time.perf_counter()
    for i in range(steps):
        step(i)
    dt = time.perf_counter() - t0
    value = n * steps / dt
    kind = "reference" if ref is not None else "port"
    sample = f"{n} rows per step of the same workload ({steps} steps), {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": "sampled rows/s at 1024x262144 fp32 logits (penalties + top-k + top-p), % of HBM roofline",
        "value": value, "unit": "rows/s", "n_gpus": world, "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"penalised sampling, {n}-row sample of {rows}x{vocab} f32, history {HIST} Zipf(1.1), " +
                               ", ".join(f"{k} {v}" for k, v in SETTINGS.items())},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=1024)
    ap.add_argument("--vocab", type=int, default=262144)
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-penalties", action="store_true", help="variant: no token history (not the headline workload)")
    ap.add_argument("--greedy", action="store_true", help="variant: greedy rows (not the headline workload)")
    ap.add_argument("--top-k", type=int, default=SETTINGS["top_k"], help="variant: another top-k (not the headline workload)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (variants only)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
