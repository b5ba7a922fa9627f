#!/usr/bin/env python
"""Benchmark of the sampling hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W]                    # this library on the GPU(s): the headline
    python bench.py --config 4 ...                                         # the continuous-batching mix (bf16, per-row settings)
    python bench.py --impl reference [--gpus N] [--steps K] [--warmup W]   # the reference's CPU sampler on the host cores
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...       # N > 1: one rank per GPU

Headline workload: penalised sampling of 1024 x 262144 f32 logits per GPU (history 4096 Zipf(1.1), repetition 1.1,
presence 0.5, frequency 0.3, temperature 0.8, top-k 50, top-p 0.9, min-p 0.05); rows are independent, so N GPUs take N
batches with no data-path collective (weak scaling).

Prints ONE JSON line (rank 0).  `value` is rows/s with the logits already in HBM: the median over `regions.n` timed
regions of exactly K steps each, every region bracketed by a barrier and a device synchronisation, timed with CUDA events
on the launching stream, maximum over ranks.  `e2e` is rows/s through whirl_sample_rows_host with pinned HOST logits,
every copy inside the timed region.  `roofline` compares the algorithmic bytes of one step with the measured HBM copy
bandwidth.  `cpu_baseline` is the reference's CPU sampler (or the oracle port where the reference was not built) on
the host cores, and `parity` compares the GPU's tokens with the oracle's on the same rows.  With two or more ranks a
`vocab_sharded` block times the tensor-parallel form (256 x 262144 split over the ranks, 1024 candidates per slice, one
all-gather, global top-p 0.9).  Synthetic inputs stand in for real logits, seeded.
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
METRIC = "sampled rows/s at 1024x262144 fp32 logits (penalties + top-k + top-p), % of HBM roofline"


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
    """nvidia-smi clocks and throttle reasons sampled every 50 ms while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                       "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
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


def zipf_history(torch, g, device, rows, vocab, seed):
    # Zipf(1.1) ranks by the inverse CDF of the continuous power law, scattered over the id space
    u = torch.rand((rows, HIST), generator=g, device=device, dtype=torch.float64)
    a = 1.0 - 1.1
    hi = float(vocab + 1) ** a
    rank = torch.floor((1.0 + u * (hi - 1.0)) ** (1.0 / a)).to(torch.int64) - 1
    rank.clamp_(0, vocab - 1)
    return ((rank * 2654435761 + seed) % vocab).to(torch.int32).contiguous()


def make_workload(torch, api, args, dev, rank):
    """Logits buffers (each larger than L2, rotated between steps) and the per-row settings of the chosen workload.
    Returns (xs, [RowParams per buffer], host dict of the settings as CPU tensors, description)."""
    rows, vocab = args.rows, args.vocab
    seed = 1234 + rank
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    nbuf = 3
    xs = []
    for _ in range(nbuf):
        x = torch.empty((rows, vocab), dtype=torch.float32, device=dev)
        if args.config == 4:
            x.normal_(0.0, 3.0, generator=g)
            x += 10.0 * (torch.rand((rows, vocab), generator=g, device=dev) < 0.01)  # 1 % of the entries + 10
        else:
            x.normal_(0.0, 2.5, generator=g)
        xs.append(x if args.dtype == "f32" else x.to(torch.bfloat16))
        del x
    us = [torch.from_numpy(splitmix_u01(seed, np.arange(rows) + b * rows)).to(dev) for b in range(nbuf)]
    f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device=dev)
    if args.config == 4:
        # 25 % greedy rows; the others temperature U[0.5, 1.2], top-k U{1..1024}, top-p U[0.8, 1.0]
        r = torch.rand((4, rows), generator=g, device=dev, dtype=torch.float64)
        base = dict(inv_t=(1.0 / (0.5 + 0.7 * r[0])).to(torch.float32), top_k=(1 + torch.floor(r[1] * 1024)).clamp_(1, 1024).to(torch.int32),
                    top_p=(0.8 + 0.2 * r[2]).contiguous(), greedy=(r[3] < 0.25).to(torch.uint8))
        what = f"continuous-batching mix {rows}x{vocab} {args.dtype} per GPU: 25% greedy, temperature U[0.5,1.2], top-k U{{1..1024}}, top-p U[0.8,1.0]"
    else:
        base = dict(inv_t=f32(1.0 / SETTINGS["temp"]), top_k=torch.full((rows,), args.top_k, dtype=torch.int32, device=dev),
                    top_p=torch.full((rows,), SETTINGS["top_p"], dtype=torch.float64, device=dev),
                    min_p=torch.full((rows,), SETTINGS["min_p"], dtype=torch.float64, device=dev))
        if not args.no_penalties:
            base.update(hist=zipf_history(torch, g, dev, rows, vocab, seed), hist_len=torch.full((rows,), HIST, dtype=torch.int32, device=dev),
                        rep=f32(SETTINGS["rep"]), pres=f32(SETTINGS["pres"]), freq=f32(SETTINGS["freq"]))
        if args.greedy:
            base["greedy"] = torch.ones(rows, dtype=torch.uint8, device=dev)
        what = (f"penalised sampling {rows}x{vocab} {args.dtype} per GPU, history {HIST} Zipf(1.1), " +
                ", ".join(f"{k} {v}" for k, v in SETTINGS.items()))
    params = [api.RowParams(u=us[b], **base) for b in range(nbuf)]
    return xs, params, us, base, what


def host_settings(base, u):
    """The per-row settings as numpy arrays in the oracle's argument names and dtypes."""
    conv = dict(inv_t=np.float32, top_k=np.uint32, top_p=np.float64, min_p=np.float64, greedy=np.uint8, hist=np.int32,
                hist_len=np.uint32, rep=np.float32, pres=np.float32, freq=np.float32)
    out = {k: base[k].cpu().numpy().astype(conv[k]) for k in base if base.get(k) is not None}
    out["u"] = u.cpu().numpy()
    return out


def parity_block(torch, api, x, params, host, ws, n):
    """GPU tokens against the oracle's on the first n rows of one batch.  A row whose draw lies within 1e-6 of a
    cumulative-probability boundary of its kept set may differ by design: such rows are counted apart."""
    from oracle import oracle as orc
    o = orc.Oracle()
    cap = 64
    res = api.sample_rows(x, params, ws=ws, kept_cap=cap, want_stats=False)
    torch.cuda.synchronize()
    got = res.token[:n].cpu().numpy().astype(np.int64)
    xn = x[:n].float().cpu().numpy() if x.dtype == torch.float32 else x[:n].view(torch.int16).cpu().numpy().view(np.uint16)
    want = o.sample_rows(xn, kept_cap=cap, threads=os.cpu_count() or 1, **{k: v[:n] for k, v in host.items()})
    diff = np.nonzero(got != want["token"].astype(np.int64))[0]
    boundary = 0
    for r in diff:
        k = min(int(want["n"][r]), cap)
        cum = np.cumsum(want["kept_p"][r, :k])
        boundary += bool((np.abs(cum - host["u"][r]) < 1e-6).any())
    unresolved = int((res.status[:n] != 0).sum().item())
    return {"rows": int(n), "mismatch": int(len(diff) - boundary), "boundary": int(boundary), "unresolved": unresolved,
            "against": "oracle port, same rows and uniforms"}


def cpu_baseline(x_dev, host, rows, vocab, seed, budget_s=8.0):
    """The reference's own CPU sampler (oracle/_ref, persistent threads over SampleBuffers -> filterCands -> sampleRow, this
    build's penalty rule applied to each row first) on the rows of one GPU batch, all host cores; the oracle port where
    the reference was not built.  Repeats the pass until about budget_s seconds of work."""
    from oracle import oracle as orc
    cores = os.cpu_count() or 1
    x = x_dev.float().cpu().numpy()
    n = x.shape[0]
    p = {k: v for k, v in host.items() if k != "u"}
    if orc.have_reference():
        ref = orc.Reference()
        p.update(seed=np.full(n, seed, np.uint64), pos_idx=np.arange(n, dtype=np.uint64))
        sec, _ = ref.bench_rows(x, threads=cores, reps=1, **p)
        reps = int(max(1, min(50, budget_s / max(sec, 1e-3))))
        sec, _ = ref.bench_rows(x, threads=cores, reps=reps, **p)
        kind = "reference"
    else:
        o = orc.Oracle()
        t0 = time.perf_counter()
        o.sample_rows(x, threads=cores, **host)
        one = time.perf_counter() - t0
        reps = int(max(1, min(50, budget_s / max(one, 1e-3))))
        t0 = time.perf_counter()
        for _ in range(reps):
            o.sample_rows(x, threads=cores, **host)
        sec = time.perf_counter() - t0
        kind = "port"
    return {"value": n * reps / sec, "unit": "rows/s", "cores": cores, "kind": kind,
            "sample": f"{n} rows of the same workload x {reps} passes ({sec:.1f} s), {cores} persistent threads, {n // cores} rows per thread and pass"}


def vocab_sharded_block(torch, dist, api, dev, world, rank, steps, warmup):
    """The tensor-parallel form at its stated size: 256 rows x 262144 tokens split over the ranks, 1024 candidates per
    slice, ONE all-gather of the packed blocks, merge and global top-p 0.9 on every rank.  Device-timed, max over ranks."""
    from whirl_llm_b200 import sharded
    rows, n_total, ks = 256, 262144, 1024
    vs = sharded.VocabShardedSampler(rows, n_total, ks, dev)
    g = torch.Generator(device=dev)
    g.manual_seed(77 + rank)
    nbuf = 4  # 4 x 32 MiB slices at 8 ranks: rotate so that the slices do not sit in L2
    xs = [torch.empty((rows, n_total // world), dtype=torch.float32, device=dev).normal_(0.0, 3.0, generator=g) for _ in range(nbuf)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    prm = api.RowParams(inv_t=torch.ones(rows, dtype=torch.float32, device=dev), top_k=torch.full((rows,), ks, dtype=torch.int32, device=dev),
                        top_p=torch.full((rows,), 0.9, dtype=torch.float64, device=dev),
                        u=torch.from_numpy(splitmix_u01(99, np.arange(rows))).to(dev))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    parts = np.zeros(3)
    res = None
    for i in range(warmup + steps):
        flush.zero_()  # the slices of one step are smaller than L2: flush it between steps
        ev[0].record()
        vs.select(xs[i % nbuf])
        ev[1].record()
        vs.exchange()
        ev[2].record()
        res = vs.merge(prm)
        ev[3].record()
        torch.cuda.synchronize()
        if i >= warmup:
            parts += [ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2]), ev[2].elapsed_time(ev[3])]
    t = torch.tensor(parts / steps, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sel, exc, mer = (float(v) for v in t.tolist())
    tok = res.token.clone()
    dist.broadcast(tok, 0)
    same = torch.tensor([int(torch.equal(tok, res.token))], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    unresolved = int((res.status != 0).sum().item())
    peak, _ = measured_peak_gbs()
    slice_bytes = rows * (n_total // world) * 4
    return {"rows": rows, "vocab": n_total, "shards": world, "k_s": ks, "top_p": 0.9, "ms_select": sel, "ms_exchange": exc, "ms_merge": mer,
            "ms_per_step": sel + exc + mer, "rows_per_s": rows / ((sel + exc + mer) * 1e-3), "block_bytes_per_rank": int(vs.block.numel() * 4),
            "select_frac_of_hbm_peak": slice_bytes / (sel * 1e-3) / 1e9 / peak, "tokens_equal_on_all_ranks": bool(same.item()),
            "unresolved_rows": unresolved, "l2": "256 MiB flush between steps, 4 rotating slices",
            "layout": "packed [ids|vals|stats] block per rank, one all_gather_into_tensor, merged in place"}


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
        import datetime
        # stdout carries the one JSON line only: what NCCL prints when its communicator comes up (its version line) goes to
        # stderr, by pointing file descriptor 1 there until the first collective has run
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    rows, vocab, esize = args.rows, args.vocab, (4 if args.dtype == "f32" else 2)
    xs, params, us, base, what = make_workload(torch, api, args, dev, rank)
    nbuf = len(xs)
    ws = torch.zeros(api.workspace_bytes(rows, vocab), dtype=torch.uint8, device=dev)
    # tokens only, as a serving engine asks: no row statistics, so rows closed by their top_k skip the normaliser
    res = api.sample_rows(xs[0], params[0], ws=ws, want_stats=False)
    torch.cuda.synchronize()
    assert int((res.status != 0).sum().item()) == 0, "unresolved rows in the benchmark workload"
    assert api.check(ws, rows) == 0, "a device-side wait ran out"

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
    # ---- timed regions of exactly K steps each; enough of them for about a second of device time (at least 10)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    sync_all()
    est = max(e0.elapsed_time(e1), 1e-3)
    if dist is not None:  # every rank must run the same number of regions: take the slowest rank's estimate
        te = torch.tensor([est], dtype=torch.float64, device=dev)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        est = float(te.item())
    n_regions = args.regions if args.regions > 0 else int(min(400, max(10, 1000.0 / est)))
    clocks = ClockSampler(local)
    lc0 = api.launch_counts()
    region_ms = []
    for _ in range(n_regions):
        sync_all()
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        sync_all()
        region_ms.append(e0.elapsed_time(e1))
    lc1 = api.launch_counts()
    clk = clocks.stop()
    t = torch.tensor(region_ms, dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # per region: the slowest rank
    per_step = np.sort(t.cpu().numpy()) / args.steps
    ms_per_step = float(np.median(per_step))
    value = world * rows / (ms_per_step * 1e-3)
    launches = (sum(lc1.values()) - sum(lc0.values())) // n_regions
    assert api.check(ws, rows) == 0, "a device-side wait ran out during the timed regions"
    hist_ids = 0 if base.get("hist") is None else HIST
    peak, peak_kind = measured_peak_gbs()
    per_row = algorithmic_bytes_per_row(vocab, esize, hist_ids)
    achieved = rows * per_row / (ms_per_step * 1e-3) / 1e9

    if args.no_e2e:
        if rank == 0:
            print(json.dumps({"variant": {k: v for k, v in vars(args).items() if k not in ("impl", "gpus")}, "ms_per_step": ms_per_step,
                              "ms_min": float(per_step[0]), "ms_max": float(per_step[-1]), "regions": n_regions, "rows_per_s": value,
                              "frac": achieved / peak}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end to end: pinned host logits through whirl_sample_rows_host, copies inside the timed region
    dt_code = api.F32 if args.dtype == "f32" else api.BF16
    x_host = torch.empty((rows, vocab), dtype=xs[0].dtype).pin_memory()
    x_host.copy_(xs[0])
    hp = {k: (v.cpu().pin_memory() if v is not None else None) for k, v in dict(u=us[0], **base).items()}
    ho = dict(token=torch.empty(rows, dtype=torch.int32).pin_memory())
    e2e_steps = max(1, min(args.steps, 10))
    api.sample_rows_host(x_host, hp, rows, vocab, dt_code, ho, device=local)
    same = bool((ho["token"].to(dev) == api.sample_rows(xs[0], params[0], ws=ws).token).all().item())
    sync_all()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        api.sample_rows_host(x_host, hp, rows, vocab, dt_code, ho, device=local)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if dist is not None:
        tt = torch.tensor([dt], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
    e2e_value = world * rows * e2e_steps / dt
    h2d = rows * vocab * esize + sum(v.numel() * v.element_size() for v in hp.values() if v is not None)
    d2h = rows * 4 + 32

    traffic = None
    tp = None
    if args.config != 4 and args.dtype == "f32":
        tp = os.path.join(ROOT, "profiles", "single_pass_kernel_traffic.txt")
    elif args.config == 4:
        tp = os.path.join(ROOT, "profiles", "single_pass_kernel_bf16_mix_traffic.txt")
    if tp and os.path.exists(tp):
        try:
            traffic = float(json.load(open(tp))["dram_bytes_per_row"]) * rows
        except Exception:
            traffic = None

    line = {
        "metric": METRIC if args.config != 4 else "sampled rows/s at 1024x262144 bf16 logits (continuous-batching mix), % of HBM roofline",
        "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": what, "rows_per_gpu": rows, "vocab": vocab, "parallelism": f"rows sharded x{world}, no collective",
                   "l2": f"{nbuf} rotating logits buffers of {rows * vocab * esize / 2**30:.2f} GiB each (each larger than L2)",
                   "e2e_matches_device_path": same},
        "regions": {"n": n_regions, "steps_each": args.steps, "ms_per_step_median": ms_per_step, "ms_per_step_min": float(per_step[0]),
                    "ms_per_step_max": float(per_step[-1]), "ms_per_step_p10": float(per_step[len(per_step) // 10]),
                    "ms_per_step_p90": float(per_step[(len(per_step) * 9) // 10])},
        "clocks": clk,
        "e2e": {"value": e2e_value, "unit": "rows/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "steps": e2e_steps},
        "gpu_launches": int(launches),
        "launches_by_kernel": {k: int((lc1[k] - lc0[k]) // n_regions) for k in lc1},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_kind": peak_kind, "algorithmic_bytes_per_row": per_row,
                     "kernel": "single_pass_kernel<float>" if args.dtype == "f32" else "single_pass_kernel<uint16_t>",
                     "timed": "whole step (error-word memset + single-pass kernel + multi-pass kernel over the leftover list)"},
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        host = host_settings(base, us[0])
        line["parity"] = parity_block(torch, api, xs[0], params[0], host, ws, rows)
        line["cpu_baseline"] = cpu_baseline(xs[0], host, rows, vocab, 1234 + rank)
    if world > 1 and not args.no_sharded:
        del xs, params
        torch.cuda.empty_cache()
        line["vocab_sharded"] = vocab_sharded_block(torch, dist, api, dev, world, rank, max(args.steps, 10), args.warmup)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_reference(args):
    """The reference's own CPU sampler (oracle/_ref: SampleBuffers -> filterCands -> sampleRow over its host top-k, behind
    persistent worker threads) on the host cores.  The reference has no penalties: this build's penalty rule is applied
    to each row first (a cheap O(H) step), then the reference code samples.  Falls back to the oracle port where
    oracle/_ref was not built.  One step = one pass over a bounded sample of the workload: at least 16 rows per thread."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from oracle import oracle as orc
    cores = os.cpu_count() or 1
    rows, vocab = args.rows, args.vocab
    n = int(min(rows, max(256, 64 * cores)))
    rng = np.random.default_rng(1234)
    x = (rng.standard_normal((n, vocab), dtype=np.float32) * np.float32(2.5))
    a = 1.0 - 1.1
    rank_ = np.floor((1.0 + rng.random((n, HIST)) * (float(vocab + 1) ** a - 1.0)) ** (1.0 / a)).astype(np.int64) - 1
    hist = ((np.clip(rank_, 0, vocab - 1) * 2654435761 + 1234) % vocab).astype(np.int32)
    f = lambda v, dt=np.float32: np.full(n, v, dtype=dt)
    p = dict(inv_t=f(1.0 / SETTINGS["temp"]), top_k=f(SETTINGS["top_k"], np.uint32), top_p=f(SETTINGS["top_p"], np.float64),
             min_p=f(SETTINGS["min_p"], np.float64), hist=hist, hist_len=f(HIST, np.uint32), rep=f(SETTINGS["rep"]),
             pres=f(SETTINGS["pres"]), freq=f(SETTINGS["freq"]))
    warm, steps = min(args.warmup, 2), max(1, min(args.steps, 40))
    if orc.have_reference():
        ref = orc.Reference()
        p.update(seed=f(1234, np.uint64), pos_idx=np.arange(n, dtype=np.uint64))
        if warm:
            ref.bench_rows(x, threads=cores, reps=warm, **p)
        dt, _ = ref.bench_rows(x, threads=cores, reps=steps, **p)
        kind = "reference"
    else:
        o = orc.Oracle()
        p["u"] = splitmix_u01(1234, np.arange(n))
        for _ in range(warm):
            o.sample_rows(x, threads=cores, **p)
        t0 = time.perf_counter()
        for _ in range(steps):
            o.sample_rows(x, threads=cores, **p)
        dt = time.perf_counter() - t0
        kind = "port"
    value = n * steps / dt
    sample = f"{n} rows per step of the same workload ({steps} steps, {dt:.1f} s), {cores} persistent threads, {n // cores} rows per thread and step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": steps, "warmup": warm,
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
    ap.add_argument("--config", type=int, default=2, choices=[2, 4],
                    help="2: the headline (penalised sampling, scaled to 1024 x 262144); 4: the continuous-batching mix (bf16)")
    ap.add_argument("--rows", type=int, default=1024)
    ap.add_argument("--vocab", type=int, default=262144)
    ap.add_argument("--dtype", default=None, choices=["f32", "bf16"])
    ap.add_argument("--regions", type=int, default=0, help="timed regions of K steps (0: about a second's worth, at least 10)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline and parity legs")
    ap.add_argument("--no-sharded", action="store_true", help="skip the vocab_sharded block at N > 1")
    ap.add_argument("--no-penalties", action="store_true", help="variant: no token history (not the headline workload)")
    ap.add_argument("--greedy", action="store_true", help="variant: greedy rows (not the headline workload)")
    ap.add_argument("--top-k", type=int, default=SETTINGS["top_k"], help="variant: another top-k (not the headline workload)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (variants only)")
    args = ap.parse_args()
    if args.dtype is None:
        args.dtype = "bf16" if args.config == 4 else "f32"
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
