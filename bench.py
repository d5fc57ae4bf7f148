#!/usr/bin/env python
"""Benchmark of the sampling hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2|c1|c3|c5] [--impl reference]

A step is one sampling pass over one batch of synthetic logits (default: the batched server-decode
configuration, 256 rows x 151,936 fp32 logits, 512-token Zipf histories, mixed per-row
parameters).  Prints ONE JSON line:

  value      rows/s over all ranks with every input already resident in HBM (CUDA events, max over
             ranks); the inputs rotate through 3 copies (467 MB) so no step finds its rows in L2
  e2e        the same metric through the public host API with HOST arrays: pinned logits, histories
             and uniforms are copied host->device and the tokens device->host inside the timed
             region, every step
  roofline   achieved HBM GB/s of the one kernel a step launches (algorithmic bytes / mean launch
             duration measured with per-launch CUDA events) against the measured copy bandwidth
  cpu_baseline  the CPU oracle (the reference's algorithm restated in C) timed on this host's cores
                on the same rows, single thread, as the reference's serial per-row loop runs it

With --impl reference the reference's CPU algorithm (the oracle; its C# cannot be built without a
.NET toolchain) is timed on all host threads instead and printed in the same format.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sampled rows/s (B=256 x V=151,936 fp32 server-decode batch per GPU)"


def metric_name(w) -> str:
    """The headline metric is quoted on the C2 batch; other configurations say their own shape."""
    if w.name.startswith("c2"):
        return METRIC
    dt = "fp32" if w.logits.dtype == np.float32 else "bf16"
    return f"sampled rows/s (B={w.rows} x V={w.vocab:,} {dt} {w.name} batch per GPU)"
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic(name: str):
    """dram bytes per launch from the committed ncu summary, if one exists for this workload."""
    path = os.path.join(ROOT, "profiles", f"{name}.traffic.json")
    try:
        with open(path) as f:
            return int(json.load(f)["bytes_per_step"])
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows = []
        self.proc = None
        self.index = device_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for t, line in self.rows:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clock = float(parts[1])
                mx = float(parts[2])
            except ValueError:
                continue
            if t0 - 0.05 <= t <= t1 + 0.05:
                sm.append(clock)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        if not sm:  # region shorter than the sampling period: use the closest samples
            for t, line in self.rows[-3:]:
                parts = [x.strip() for x in line.split(",")]
                try:
                    sm.append(float(parts[1]))
                    mx = float(parts[2])
                except (ValueError, IndexError):
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def to_device(w):
    """Device copies of a workload's arrays (the timed region starts with inputs resident in HBM)."""
    import torch

    dev = {}
    lg = torch.from_numpy(w.logits.view(np.int16) if w.logits.dtype == np.uint16 else w.logits).cuda()
    dev["logits"] = lg.view(torch.bfloat16) if w.logits.dtype == np.uint16 else lg
    dev["uniforms"] = torch.from_numpy(w.uniforms).cuda()
    if w.history_ids is not None:
        dev["history_ids"] = torch.from_numpy(w.history_ids).cuda()
    if w.mask is not None:
        dev["mask"] = torch.from_numpy(w.mask.view(np.int32)).cuda()
    return dev


def make_workload(name: str, rank: int):
    from opentail.stingray_b200 import workloads as W

    if name == "c1":
        return W.config1(seed=0 + 100 * rank)
    if name == "c2":
        return W.config2(seed=1 + 100 * rank)
    if name == "c3":
        return W.config3(seed=2 + 100 * rank)
    if name == "c5":
        return W.config5(rows=512, seed=4 + 100 * rank)
    raise SystemExit(f"unknown config {name}")


def cpu_rows_per_s(w, threads: int, max_rows: int, repeats: int = 1):
    """Times the oracle's serial per-row loop over the first max_rows rows on `threads` threads."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as orc

    rows = min(w.rows, max_rows)
    u = w.uniforms.astype(np.float64)

    def run_slice(lo, hi):
        ho = hi_ids = None
        if w.history_ids is not None:
            ho = (w.history_offsets[lo:hi + 1] - w.history_offsets[lo]).astype(np.int32)
            hi_ids = w.history_ids[w.history_offsets[lo]:w.history_offsets[hi]]
        orc.sample_rows(w.logits[lo:hi], w.params[lo:hi], u[lo:hi], hi_ids, ho,
                        None if w.mask is None else w.mask[lo:hi])

    orc.lib()
    bounds = np.linspace(0, rows, threads + 1).astype(int)
    # interleave rows so every thread gets a similar mix of paths: here slices are contiguous but
    # the per-row parameters are i.i.d., so contiguous slices are already balanced
    t0 = time.perf_counter()
    for _ in range(repeats):
        if threads == 1:
            run_slice(0, rows)
        else:
            with ThreadPoolExecutor(threads) as ex:
                list(ex.map(lambda i: run_slice(bounds[i], bounds[i + 1]), range(threads)))
    dt = time.perf_counter() - t0
    return rows * repeats / dt, rows, dt


def run_reference(args, rank, world):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    w = make_workload(args.config, 0)
    sample_rows = w.rows if cores >= 8 else min(w.rows, 64)
    for _ in range(min(args.warmup, 1)):
        cpu_rows_per_s(w, cores, sample_rows)
    times = []
    for _ in range(max(1, min(args.steps, 5))):
        rps, rows, dt = cpu_rows_per_s(w, cores, sample_rows)
        times.append(dt)
    ms = 1000.0 * sum(times) / len(times)
    value = sample_rows / (ms / 1000.0)
    line = {
        "impl": "reference", "metric": metric_name(w), "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "rows": w.rows, "vocab": w.vocab,
                   "note": "reference C# cannot be built here (no .NET toolchain); this is its algorithm restated "
                           "in C (oracle/sampler_oracle.c), rows spread over all host threads"},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port",
                         "sample": f"{sample_rows} of {w.rows} rows per step"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_spec(args, rank, local, world):
    """Config 4: one speculative verification step (32 sequences x (9 target + 8 draft) rows of
    151,936 fp32 logits).  The unit is a verified sequence; same timing rules as the sampling step."""
    import torch
    import torch.distributed as dist

    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import workloads as W

    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    w = W.config4(seed=3 + 100 * rank)
    n_seq, lp1, vocab = w.target.shape
    L = lp1 - 1
    bs = BatchSampler(max_rows=n_seq * lp1, max_vocab=vocab, max_history=1, max_top_k=8, max_spec_draft=L, device=local)
    n_copies = 2  # 2 x 331 MB > 126 MB L2
    devs = [(torch.from_numpy(w.target).cuda(), torch.from_numpy(w.draft).cuda(),
             torch.from_numpy(w.draft_tokens).cuda(), torch.from_numpy(w.uniforms).cuda()) for _ in range(n_copies)]

    def step(i):
        t, d, tok, u = devs[i % n_copies]
        return bs.spec_verify(t, d, tok, w.params, u)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    launches0 = bs.stats()["kernel_launches"]
    clocks = ClockSampler(local)
    clocks.start()
    time.sleep(0.25)
    barrier()
    t_wall0 = time.time()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    torch.cuda.synchronize()
    clock_info = clocks.stop(t_wall0, time.time())
    ms_step = ev0.elapsed_time(ev1) / args.steps
    launches = bs.stats()["kernel_launches"] - launches0
    # end to end: pinned host logits in, accepted lengths and correction tokens out
    pt, pd = torch.from_numpy(w.target).pin_memory(), torch.from_numpy(w.draft).pin_memory()
    dt, dd = torch.empty_like(devs[0][0]), torch.empty_like(devs[0][1])
    e2e_steps = max(3, min(args.steps, 5))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        dt.copy_(pt, non_blocking=True)
        dd.copy_(pd, non_blocking=True)
        out = bs.spec_verify(dt, dd, w.draft_tokens, w.params, w.uniforms)
        acc = out["accepted"].cpu()
        corr = out["correction"].cpu()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    t = torch.tensor([ms_step, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms = [float(x) for x in t.cpu()]
    peak, peak_kind = measured_peak()
    alg = w.algorithmic_bytes()
    if rank == 0:
        line = {
            "metric": "verified sequences/s (32 seq x (9 target + 8 draft) x V=151,936 fp32 per GPU)",
            "value": n_seq * world / (ms_step / 1000.0), "unit": "sequences/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w.name, "sequences_per_gpu": n_seq, "draft_len": L, "vocab": vocab,
                       "sharding": f"sequences x{world}", "l2": f"{n_copies} rotating input copies, "
                       f"{n_copies * (w.target.nbytes + w.draft.nbytes) / 1e6:.0f} MB > 126 MB L2"},
            "roofline": {"bound": "hbm", "achieved": alg / (ms_step / 1000.0) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (ms_step / 1000.0) / 1e9 / peak, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": alg, "traffic": None},
            "e2e": {"value": n_seq * world / (e2e_ms / 1000.0), "unit": "sequences/s",
                    "h2d_bytes_per_step": w.target.nbytes + w.draft.nbytes + w.draft_tokens.nbytes + w.uniforms.nbytes,
                    "d2h_bytes_per_step": 8 * n_seq, "ms_per_step": e2e_ms},
            "gpu_launches": launches, "clocks": clock_info,
            "accepted_mean": float(acc.float().mean()),
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--config", default="c2")
    ap.add_argument("--impl", default="native")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampling path has no CPU fallback")
    if args.config == "c4":
        run_spec(args, rank, local, world)
        return
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))

    from opentail.stingray_b200 import BatchSampler

    w = make_workload(args.config, rank)
    hist_max = int(np.diff(w.history_offsets).max()) if w.history_offsets is not None else 0
    bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=max(hist_max, 1),
                      max_top_k=max(int(w.params["top_k"].max()), 1), device=local)
    n_copies = 3
    devs = [to_device(w) for _ in range(n_copies)]

    def step(i):
        d = devs[i % n_copies]
        kw = dict(uniforms=d["uniforms"])
        if w.history_ids is not None:
            kw.update(history_ids=d["history_ids"], history_offsets=w.history_offsets)
        if w.mask is not None:
            kw.update(mask=d["mask"])
        return bs.sample_rows(d["logits"], w.params, **kw)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    launches0 = bs.stats()["kernel_launches"]
    clocks = ClockSampler(local)
    clocks.start()
    time.sleep(0.25)
    barrier()
    t_wall0 = time.time()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    ms_total = ev0.elapsed_time(ev1)
    launches = bs.stats()["kernel_launches"] - launches0

    # per-launch durations of the step's kernel (roofline numerator), same stream, same inputs
    pairs = []
    for i in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step(i)
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    clock_info = clocks.stop(t_wall0, time.time())
    launch_ms = [a.elapsed_time(b) for a, b in pairs]
    launch_ms_mean = sum(launch_ms) / len(launch_ms)

    # end to end through the host API: pinned host arrays in, tokens out, every step
    pin = {"logits": torch.from_numpy(w.logits.view(np.int16) if w.logits.dtype == np.uint16 else w.logits).pin_memory()}
    host_logits = pin["logits"].numpy().view(w.logits.dtype)
    kw_host = dict(uniforms=w.uniforms)
    h2d = w.logits.nbytes + w.uniforms.nbytes
    if w.history_ids is not None:
        pin["hist"] = torch.from_numpy(w.history_ids).pin_memory()
        kw_host.update(history_ids=pin["hist"].numpy(), history_offsets=w.history_offsets)
        h2d += w.history_ids.nbytes
    if w.mask is not None:
        pin["mask"] = torch.from_numpy(w.mask.view(np.int32)).pin_memory()
        kw_host.update(mask=pin["mask"].numpy().view(np.uint32))
        h2d += w.mask.nbytes
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        bs.sample_rows(host_logits, w.params, **kw_host)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        out = bs.sample_rows(host_logits, w.params, **kw_host)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    t = torch.tensor([ms_total, e2e_ms, launch_ms_mean], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, launch_ms_mean = [float(x) for x in t.cpu()]
    ms_step = ms_total / args.steps
    total_rows = w.rows * world
    value = total_rows / (ms_step / 1000.0)
    peak, peak_kind = measured_peak()
    alg_bytes = w.algorithmic_bytes()
    achieved = alg_bytes / (launch_ms_mean / 1000.0) / 1e9

    if rank == 0:
        line = {
            "metric": metric_name(w), "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32" if w.logits.dtype == np.float32 else "bf16", "data": "synthetic",
            "config": {"workload": w.name, "rows_per_gpu": w.rows, "vocab": w.vocab, "history": hist_max,
                       "sharding": f"rows x{world}", "l2": f"{n_copies} rotating input copies, "
                       f"{n_copies * w.logits.nbytes / 1e6:.0f} MB > 126 MB L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_8TBs": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": alg_bytes, "launch_ms": launch_ms_mean,
                         "traffic": ncu_traffic(f"k_sample_{args.config}")},
            "e2e": {"value": total_rows / (e2e_ms / 1000.0), "unit": "rows/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4 * w.rows, "ms_per_step": e2e_ms},
            "gpu_launches": launches,
            "clocks": clock_info,
        }
        if not args.no_cpu and world >= 1:
            rps, rows, dt = cpu_rows_per_s(w, 1, 256)
            reps = int(min(20, max(1, round(12.0 / max(dt, 0.05)) - 1)))  # about 12 s of CPU work in all
            if reps > 0:
                rps2, _, dt2 = cpu_rows_per_s(w, 1, 256, repeats=reps)
                rps, dt = (rows * (1 + reps)) / (dt + dt2), dt + dt2
            line["cpu_baseline"] = {"value": rps, "unit": "rows/s", "cores": 1, "kind": "port",
                                    "sample": f"{rows} rows of the same batch, {1 + reps} passes ({dt:.1f} s), single "
                                              f"thread as the reference's serial loop"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
