#!/usr/bin/env python
"""Benchmark of the sampling hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2|c1|c3|c4|c5] [--impl reference]
                    [--no-cpu] [--no-legs]

A step is one sampling pass over one batch of synthetic logits (default: the batched server-decode
configuration, 256 rows x 151,936 fp32 logits, 512-token Zipf histories, mixed per-row
parameters).  Prints ONE JSON line:

  value      rows/s over all ranks with every input already resident in HBM (CUDA events, max over
             ranks); the inputs rotate through 3 copies (467 MB) so no step finds its rows in L2
  e2e        the same metric through the public host API with HOST arrays: pinned logits, histories
             and uniforms are copied host->device and the tokens device->host inside the timed
             region, every step
  roofline   achieved HBM GB/s of a step's kernels (algorithmic bytes / mean duration of one step's
             launches measured with per-step CUDA events) against the measured copy bandwidth
  cpu_baseline  the CPU oracle (the reference's algorithm restated in C) timed on this host's cores
                on the same rows, single thread, as the reference's serial per-row loop runs it
  parity     the tokens of the last timed step compared with the tokens that CPU pass computed: a
             mismatch is tolerated only where the oracle reports the draw within 1e-6 of a CDF
             boundary, anything else makes the run exit non-zero
  configs    short legs (a few steps each) over the other configurations: c1, c3, c4, a 512-row
             shard of c5, three homogeneous batches of the c2 shape, a leg whose per-row history
             grows every step (plan and history upload inside the timed region), the reference's
             own CUDA arg-max kernel beside stg_argmax_rows, and - with more than one rank - both
             shardings of ONE 4096-row c5 batch (rows; vocabulary columns + NCCL all-gather)

With --impl reference the reference's CPU algorithm (the oracle; its C# cannot be built without a
.NET toolchain) is timed on all host threads instead and printed in the same format.
"""
from __future__ import annotations

import argparse
import ctypes
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
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126e6
BOUNDARY = 1e-6


def metric_name(w) -> str:
    """The headline metric is quoted on the C2 batch; other configurations say their own shape."""
    if w.name.startswith("c2"):
        return METRIC
    dt = "fp32" if w.logits.dtype == np.float32 else "bf16"
    return f"sampled rows/s (B={w.rows} x V={w.vocab:,} {dt} {w.name} batch per GPU)"


def config_block(w, world: int, n_copies: int) -> dict:
    """The `config` object, identical in the native and the reference arm."""
    hist_max = int(np.diff(w.history_offsets).max()) if w.history_offsets is not None else 0
    return {"workload": w.name, "rows_per_gpu": w.rows, "vocab": w.vocab, "history": hist_max,
            "sharding": f"rows x{world}",
            "l2": f"{n_copies} rotating input copies, {n_copies * w.logits.nbytes / 1e6:.0f} MB vs 126 MB L2"}


def copies_for(nbytes: int) -> int:
    """Rotating input copies needed for the working set to exceed L2 (at least 3)."""
    return max(3, int(np.ceil(1.25 * L2_BYTES / max(nbytes, 1))))


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

    def _nvml_loop(self):
        # the same counters nvidia-smi prints, read through NVML every few milliseconds: the timed region
        # of the headline run is a few tens of milliseconds, shorter than nvidia-smi's own sampling period
        import pynvml as nv

        R = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
             "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        while not self.stop_flag:
            try:
                clock = nv.nvmlDeviceGetClockInfo(self.nvml_dev, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.nvml_dev)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.nvml_dev)
                self.nvml_rows.append((time.time(), float(clock), [n for n, bit in R.items() if mask & bit]))
            except Exception:
                break
            time.sleep(0.004)

    def start(self):
        self.nvml_rows, self.stop_flag, self.nvml_dev = [], False, None
        try:
            import pynvml as nv

            nv.nvmlInit()
            # NVML numbers devices like nvidia-smi; CUDA_VISIBLE_DEVICES may renumber CUDA's
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if self.index < len(ids) and ids[self.index].isdigit():
                    phys = int(ids[self.index])
            self.nvml_dev = nv.nvmlDeviceGetHandleByIndex(phys)
            self.nvml_max = float(nv.nvmlDeviceGetMaxClockInfo(self.nvml_dev, nv.NVML_CLOCK_SM))
            self.nvml_thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.nvml_thread.start()
        except Exception:
            self.nvml_dev = None
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
        self.stop_flag = True
        if self.nvml_dev is not None:
            inside = [r for r in self.nvml_rows if t0 <= r[0] <= t1]
            if len(inside) >= 3:
                if self.proc is not None:
                    self.proc.terminate()
                reasons = sorted({n for r in inside for n in r[2]})
                return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": self.nvml_max,
                        "reasons": reasons, "samples": len(inside), "source": "NVML, every 4 ms during the timed region"}
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
    if name == "c2_all_greedy":
        # the C2 logits with every row a plain arg-max row: the step that is one HBM pass and nothing else
        w = W.config2(seed=1 + 100 * rank)
        return W.SampleWorkload("c2_all_greedy", w.logits, W._params(w.rows, temperature=0.0), w.uniforms, None, None, None)
    raise SystemExit(f"unknown config {name}")


def oracle_pass(w, threads: int, max_rows: int):
    """One pass of the oracle's serial per-row loop over the first max_rows rows on `threads`
    threads; returns (seconds, tokens, traces)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as orc

    rows = min(w.rows, max_rows)
    u = w.uniforms.astype(np.float64)

    def run_slice(lo, hi):
        ho = hi_ids = None
        if w.history_ids is not None:
            ho = (w.history_offsets[lo:hi + 1] - w.history_offsets[lo]).astype(np.int32)
            hi_ids = w.history_ids[w.history_offsets[lo]:w.history_offsets[hi]]
        return orc.sample_rows(w.logits[lo:hi], w.params[lo:hi], u[lo:hi], hi_ids, ho,
                               None if w.mask is None else w.mask[lo:hi])

    orc.lib()
    bounds = np.linspace(0, rows, threads + 1).astype(int)
    t0 = time.perf_counter()
    if threads == 1:
        parts = [run_slice(0, rows)]
    else:
        with ThreadPoolExecutor(threads) as ex:
            parts = list(ex.map(lambda i: run_slice(bounds[i], bounds[i + 1]), range(threads)))
    dt = time.perf_counter() - t0
    tokens = np.concatenate([p[0] for p in parts])
    traces = np.concatenate([p[1] for p in parts])
    return dt, tokens, traces


def run_reference(args, rank, world):
    """The reference arm: the reference's CPU algorithm for the path (the oracle port; the C# itself
    needs a .NET toolchain that is absent) on all host threads, same workload and config keys."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    if args.config == "c4":
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm covers the sampling configurations "
                          "(c1, c2, c3, c5); the speculative step is timed by the native arm's c4 leg only"}))
        return
    w = make_workload(args.config, 0)
    sample_rows = w.rows if cores >= 8 else min(w.rows, 64)
    for _ in range(args.warmup):
        oracle_pass(w, cores, sample_rows)
    times = [oracle_pass(w, cores, sample_rows)[0] for _ in range(max(1, args.steps))]
    ms = 1000.0 * sum(times) / len(times)
    value = sample_rows / (ms / 1000.0)
    line = {
        "impl": "reference", "metric": metric_name(w), "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32" if w.logits.dtype == np.float32 else "bf16",
        "data": "synthetic",
        "config": config_block(w, world, copies_for(w.logits.nbytes)),
        "note": "the reference's C# cannot be built here (no .NET toolchain); this is its algorithm restated in C "
                "(oracle/sampler_oracle.c), rows spread over all host threads; one rank runs it",
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port",
                         "sample": f"{sample_rows} of {w.rows} rows per step"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- timing helpers ----------------------------------------------------------------------------------

class L2Flush:
    """Writes a buffer larger than L2 between timed iterations (for inputs smaller than L2)."""

    def __init__(self):
        import torch

        self.buf = torch.empty(int(2 * L2_BYTES), dtype=torch.uint8, device="cuda")

    def __call__(self):
        self.buf.fill_(1)


def timed_each(step, steps: int, warmup: int, flush=None) -> float:
    """Mean device time (ms) of step(i), each call bracketed by its own pair of CUDA events on the
    launching stream; `flush` runs between calls, outside the brackets."""
    import torch

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    pairs = []
    for i in range(steps):
        if flush is not None:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step(i)
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)


def timed_loop(step, steps: int, warmup: int) -> float:
    """Mean device time (ms) per step of `steps` calls issued back to back between one pair of CUDA
    events on the launching stream - the way the headline number is taken."""
    import torch

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        step(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def sampling_leg(w, steps=12, warmup=3, device=0, bs=None, params=None, use_history=True, flush=None):
    """ms per step of one sampling configuration with device-resident inputs."""
    import torch
    from opentail.stingray_b200 import BatchSampler

    params = w.params if params is None else params
    own = bs is None
    if own:
        hist_max = int(np.diff(w.history_offsets).max()) if w.history_offsets is not None else 0
        bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=max(hist_max, 1),
                          max_top_k=max(int(params["top_k"].max()), 1), device=device)
    n_copies = copies_for(w.logits.nbytes) if flush is None else 1
    devs = [to_device(w) for _ in range(n_copies)]

    outs = [None] * n_copies

    def step(i):
        d = devs[i % n_copies]
        kw = dict(uniforms=d["uniforms"])
        if use_history and w.history_ids is not None:
            kw.update(history_ids=d["history_ids"], history_offsets=w.history_offsets)
        if w.mask is not None:
            kw.update(mask=d["mask"])
        outs[i % n_copies] = bs.sample_rows(d["logits"], params, out=outs[i % n_copies], **kw)
        return outs[i % n_copies]

    # every input copy is seen twice before the timed steps (the second sighting captures the step's graph)
    # rotating copies: the steps back to back, as in the headline run; one copy: each step on its own,
    # the L2 flushed before it
    warm = max(warmup, 2 * n_copies + 1)
    ms = timed_loop(step, steps, warm) if flush is None else timed_each(step, steps, warm, flush)
    if own:
        bs.close()
    del devs
    torch.cuda.empty_cache()
    alg = w.algorithmic_bytes() - (0 if use_history or w.history_ids is None else w.history_ids.nbytes)
    peak, _ = measured_peak()
    gbs = alg / (ms / 1000.0) / 1e9
    return {"ms_per_step": ms, "rows_per_s": w.rows / (ms / 1000.0), "achieved_gbs": gbs, "frac": gbs / peak,
            "l2": (f"{n_copies} rotating copies, {n_copies * w.logits.nbytes / 1e6:.0f} MB, steps back to back" if flush is None
                   else "L2 flushed between steps")}


def kernel_times_leg(w, steps=8, warmup=4, device=0):
    """Device time of every kernel of a sampling step, measured live: a handle created with the
    library's event timer on (STG_KERNEL_TIMES=1 at stg_create) records a CUDA event on the launching
    stream after each kernel of a step, and stg_debug_kernel_times returns the intervals.  The steps
    run back to back on rotating input copies exactly as in the timed region, so the numbers are
    warm-pipeline times (unlike a profiler's serialised, cache-flushed launches); the extra event
    records cost a few microseconds per step, which is why this leg is not the headline."""
    import torch
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import _native as N

    hist_max = int(np.diff(w.history_offsets).max()) if w.history_offsets is not None else 0
    os.environ["STG_KERNEL_TIMES"] = "1"
    try:
        bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=max(hist_max, 1),
                          max_top_k=max(int(w.params["top_k"].max()), 1), device=device)
    finally:
        del os.environ["STG_KERNEL_TIMES"]
    lib = N.load()
    n_copies = copies_for(w.logits.nbytes)
    devs = [to_device(w) for _ in range(n_copies)]
    acc, names = None, None
    for i in range(warmup + steps):
        d = devs[i % n_copies]
        kw = dict(uniforms=d["uniforms"])
        if w.history_ids is not None:
            kw.update(history_ids=d["history_ids"], history_offsets=w.history_offsets)
        if w.mask is not None:
            kw.update(mask=d["mask"])
        bs.sample_rows(d["logits"], w.params, **kw)
        us = np.zeros(32, np.float32)
        nm = ctypes.create_string_buffer(32 * 24)
        k = ctypes.c_int32(0)
        if lib.stg_debug_kernel_times(bs._h, us.ctypes.data, nm, 24, 32, ctypes.byref(k)) != 0:
            break
        if i >= warmup:
            acc = us[:k.value].copy() if acc is None else acc + us[:k.value]
            names = [nm.raw[j * 24:(j + 1) * 24].split(b"\0")[0].decode() for j in range(k.value)]
    bs.close()
    del devs
    torch.cuda.empty_cache()
    if acc is None:
        return {"unavailable": "the event timer returned nothing"}
    acc = acc / steps
    peak, _ = measured_peak()
    out = {"us": {n: round(float(t), 2) for n, t in zip(names, acc)}, "sum_us": round(float(acc.sum()), 1)}
    if "flat_stream" in out["us"]:
        # the one kernel that reads the logits from HBM: algorithmic bytes of the step over its own time
        gbs = w.algorithmic_bytes() / (out["us"]["flat_stream"] * 1e-6) / 1e9
        out["flat_stream_gbs"] = round(gbs, 1)
        out["flat_stream_frac"] = round(gbs / peak, 4)
    return out


def spec_leg(steps=4, warmup=3, device=0):
    """Config 4: one speculative verification step, 32 sequences x (9 target + 8 draft) rows."""
    import torch
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import workloads as W

    w = W.config4(seed=3)
    n_seq, lp1, vocab = w.target.shape
    L = lp1 - 1
    bs = BatchSampler(max_rows=n_seq * lp1, max_vocab=vocab, max_history=1, max_top_k=8, max_spec_draft=L, device=device)
    n_copies = 2  # 2 x 331 MB > 126 MB L2
    devs = [(torch.from_numpy(w.target).cuda(), torch.from_numpy(w.draft).cuda(),
             torch.from_numpy(w.draft_tokens).cuda(), torch.from_numpy(w.uniforms).cuda()) for _ in range(n_copies)]

    def step(i):
        t, d, tok, u = devs[i % n_copies]
        return bs.spec_verify(t, d, tok, w.params, u)

    ms = timed_each(step, steps, warmup)
    acc = step(0)["accepted"].float().mean().item()
    bs.close()
    del devs
    torch.cuda.empty_cache()
    alg = w.algorithmic_bytes()
    peak, _ = measured_peak()
    gbs = alg / (ms / 1000.0) / 1e9
    return {"ms_per_step": ms, "sequences_per_s": n_seq / (ms / 1000.0), "achieved_gbs": gbs, "frac": gbs / peak,
            "accepted_mean": acc, "l2": f"{n_copies} rotating copies, {n_copies * (w.target.nbytes + w.draft.nbytes) / 1e6:.0f} MB"}


def vary_plan_leg(w, steps=6, warmup=3, device=0):
    """The c2 batch as a decode loop sees it: every step each row's history is one token longer, so
    the per-step plan and the host-resident CSR history are uploaded inside the timed region."""
    import torch
    from opentail.stingray_b200 import BatchSampler

    hist_len = int(np.diff(w.history_offsets).max())
    bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=hist_len, max_top_k=int(w.params["top_k"].max()),
                      device=device)
    n_copies = copies_for(w.logits.nbytes)
    devs = [to_device(w) for _ in range(n_copies)]
    hist = w.history_ids.reshape(w.rows, hist_len)
    total = steps + warmup
    variants = []
    for i in range(total):
        n = hist_len - total + 1 + i  # grows by one token per step, ends at the full history
        ids = torch.from_numpy(np.ascontiguousarray(hist[:, :n]).reshape(-1)).pin_memory()
        variants.append((ids, (np.arange(w.rows + 1) * n).astype(np.int32)))
    uploads0 = bs.stats()["plan_uploads"]

    def run(i):
        d = devs[i % n_copies]
        ids, off = variants[i]
        return bs.sample_rows(d["logits"], w.params, uniforms=d["uniforms"], history_ids=ids.numpy(), history_offsets=off,
                              host_outputs=False)

    for i in range(warmup):
        run(i)
    torch.cuda.synchronize()
    pairs = []
    for i in range(warmup, total):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run(i)
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in pairs) / len(pairs)
    uploads = bs.stats()["plan_uploads"] - uploads0
    bs.close()
    del devs
    torch.cuda.empty_cache()
    return {"ms_per_step": ms, "rows_per_s": w.rows / (ms / 1000.0), "plan_uploads": uploads, "steps": total,
            "history_h2d_bytes_per_step": int(variants[-1][0].numel() * 4)}


def reference_gpu_argmax_leg(w, steps=6, warmup=3, device=0):
    """The reference's own device arg-max kernel (llm_argmax_rows, compiled from the reference's source
    text into oracle/_ref/ by oracle/build_ref_argmax.py and launched as the reference launches it:
    one 256-thread block per row) beside stg_argmax_rows on the same all-greedy batch."""
    import torch
    from opentail.stingray_b200 import BatchSampler

    so = os.path.join(ROOT, "oracle", "_ref", "libref_argmax.so")
    n_copies = copies_for(w.logits.nbytes)
    xs = [torch.from_numpy(w.logits).cuda() for _ in range(n_copies)]
    bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=1, max_top_k=1, device=device)
    # argmax_rows hands out new output arrays every call (torch's allocator alternates between two blocks):
    # enough warm-up for every (input copy, output block) pair to have been seen twice, after which the
    # library replays the step
    ours_ms = timed_each(lambda i: bs.argmax_rows(xs[i % n_copies]), steps, max(warmup, 4 * n_copies + 1))
    idx, val = bs.argmax_rows(xs[0])
    out = {"stg_argmax_rows_ms": ours_ms, "stg_argmax_rows_gbs": w.logits.nbytes / (ours_ms / 1000.0) / 1e9}
    bs.close()
    if not os.path.exists(so):
        out["reference_kernel"] = "unavailable: oracle/_ref/libref_argmax.so was not built (no reference tree at build time)"
        return out
    lib = ctypes.CDLL(so)
    lib.ref_argmax_rows.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    pairs = torch.empty((w.rows, 2), dtype=torch.int32, device="cuda")

    def ref(i):
        rc = lib.ref_argmax_rows(xs[i % n_copies].data_ptr(), w.rows, w.vocab, w.vocab, pairs.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
        assert rc == 0, f"ref_argmax_rows: CUDA error {rc}"

    ref_ms = timed_each(ref, steps, warmup)
    ref(0)
    torch.cuda.synchronize()
    same = bool(torch.equal(pairs[:, 0], idx) and torch.equal(pairs[:, 1], val.view(torch.int32)))
    out.update({"llm_argmax_rows_ms": ref_ms, "llm_argmax_rows_gbs": w.logits.nbytes / (ref_ms / 1000.0) / 1e9,
                "speedup": ref_ms / ours_ms, "identical_pairs": same})
    del xs
    torch.cuda.empty_cache()
    return out


# ---- one 4096-row c5 batch over the ranks (multi-GPU legs) --------------------------------------------

C5_ROWS, C5_VOCAB, C5_HIST, C5_BLOCK = 4096, 256_000, 256, 64


def c5_block(block: int, device):
    """Rows [block * 64, block * 64 + 64) of the 4096-row c5 batch, generated on the device from a
    seed that depends only on the block: every rank sees the same global batch."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(40_000 + block)
    logits = torch.randn((C5_BLOCK, C5_VOCAB), generator=g, device=device, dtype=torch.float32) * 3.0
    hist = torch.randint(0, C5_VOCAB, (C5_BLOCK, C5_HIST), generator=g, device=device, dtype=torch.int32)
    u = (torch.randint(0, 1 << 24, (C5_BLOCK,), generator=g, device=device).double() + 0.5) / float(1 << 24)
    return logits, hist, u.float()


def c5_sharded_legs(rank, world, local, steps=4, warmup=3):
    """Both shardings of ONE 4096-row c5 batch: (i) rank r samples rows [r*4096/N, (r+1)*4096/N) over the
    full vocabulary, no collective; (ii) rank r holds columns [r*V/N, (r+1)*V/N) of every row: local
    candidates (stg_shard_select), one NCCL all-gather (stg_shard_allgather), merge and finish
    (stg_shard_finish).  The tokens of (ii) are compared with those of (i) on this rank's rows."""
    import torch
    import torch.distributed as dist
    from opentail.stingray_b200 import BatchSampler
    from opentail.stingray_b200 import workloads as W

    dev = torch.device(f"cuda:{local}")
    rows_per = C5_ROWS // world
    cols_per = C5_VOCAB // world
    assert cols_per % 8 == 0
    r_lo = rank * rows_per
    c_lo = rank * cols_per
    my_rows = torch.empty((rows_per, C5_VOCAB), dtype=torch.float32, device=dev)
    my_cols = torch.empty((C5_ROWS, cols_per), dtype=torch.float32, device=dev)
    hist_all = torch.empty((C5_ROWS, C5_HIST), dtype=torch.int32, device=dev)
    u_all = torch.empty((C5_ROWS,), dtype=torch.float32, device=dev)
    for b in range(C5_ROWS // C5_BLOCK):
        lg, hs, u = c5_block(b, dev)
        lo = b * C5_BLOCK
        my_cols[lo:lo + C5_BLOCK] = lg[:, c_lo:c_lo + cols_per]
        hist_all[lo:lo + C5_BLOCK] = hs
        u_all[lo:lo + C5_BLOCK] = u
        if r_lo <= lo < r_lo + rows_per:
            my_rows[lo - r_lo:lo - r_lo + C5_BLOCK] = lg
        del lg
    params_all = W._params(C5_ROWS, top_k=50, top_p=0.9, repetition_penalty=1.05, repeat_last_n=0)
    off_all = (np.arange(C5_ROWS + 1) * C5_HIST).astype(np.int32)
    hist_rows = hist_all[r_lo:r_lo + rows_per].contiguous().view(-1)
    off_rows = (np.arange(rows_per + 1) * C5_HIST).astype(np.int32)
    hist_flat = hist_all.view(-1)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        for _ in range(warmup):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {}
    peak, _ = measured_peak()
    # (i) rows sharded: rows_per x 1 GB-per-1000-rows exceeds L2 at every N up to 8 (512 rows = 524 MB)
    bs = BatchSampler(max_rows=rows_per, max_vocab=C5_VOCAB, max_history=C5_HIST, max_top_k=50, device=local)
    res = {}

    def row_step():
        res["out"] = bs.sample_rows(my_rows, params_all[:rows_per], uniforms=u_all[r_lo:r_lo + rows_per],
                                    history_ids=hist_rows, history_offsets=off_rows, out=res.get("out"))
        res["tok"] = res["out"]["tokens"]

    ms = timed(row_step)
    row_tokens = res["tok"].clone()
    bs.close()
    alg = C5_ROWS * (C5_VOCAB * 4 + C5_HIST * 4 + 48)
    out["c5_row_sharded"] = {"ms_per_step": ms, "rows_per_s": C5_ROWS / (ms / 1000.0), "rows_per_rank": rows_per,
                             "scaling": "strong", "achieved_gbs_all_ranks": alg / (ms / 1000.0) / 1e9,
                             "frac_per_gpu": alg / world / (ms / 1000.0) / 1e9 / peak, "collective": "none"}
    del my_rows
    torch.cuda.empty_cache()
    # (ii) vocabulary sharded
    vs = BatchSampler(max_rows=C5_ROWS, max_vocab=cols_per, max_history=C5_HIST, max_top_k=50, device=local)
    if rank == 0:
        uid = torch.frombuffer(bytearray(BatchSampler.comm_unique_id()), dtype=torch.uint8).to(dev)
    else:
        uid = torch.empty(128, dtype=torch.uint8, device=dev)
    dist.broadcast(uid, 0)
    vs.comm_init(bytes(uid.cpu().numpy().tobytes()), rank, world)

    def vocab_step():
        vs.shard_select(my_cols, params_all, c_lo, C5_VOCAB, history_ids=hist_flat, history_offsets=off_all)
        vs.shard_allgather()
        res["vtok"] = vs.shard_finish(C5_ROWS, cols_per, params_all, C5_VOCAB, history_ids=hist_flat,
                                      history_offsets=off_all, uniforms=u_all)["tokens"]

    ms_v = timed(vocab_step)
    # the exchange alone
    ms_x = timed(lambda: vs.shard_allgather())
    vtok = res["vtok"]
    same = int((vtok[r_lo:r_lo + rows_per] == row_tokens).sum().item())
    agree = torch.tensor([same, rows_per], dtype=torch.int64, device=dev)
    dist.all_reduce(agree)
    xbytes = vs.exchange_bytes()
    vs.close()
    out["c5_vocab_sharded"] = {"ms_per_step": ms_v, "rows_per_s": C5_ROWS / (ms_v / 1000.0), "columns_per_rank": cols_per,
                               "scaling": "strong", "allgather_ms": ms_x, "allgather_bytes_sent_per_rank": xbytes,
                               "allgather_bytes_received_per_rank": xbytes * world, "collective": "1 ncclAllGather per step",
                               "achieved_gbs_all_ranks": alg / (ms_v / 1000.0) / 1e9,
                               "frac_per_gpu": alg / world / (ms_v / 1000.0) / 1e9 / peak,
                               "tokens_equal_to_row_sharded": int(agree[0].item()), "tokens_compared": int(agree[1].item())}
    return out


# ---- the headline run ------------------------------------------------------------------------------------

def run_spec(args, rank, local, world):
    """--config c4 as the headline: the speculative verification step."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    clocks = ClockSampler(local)
    clocks.start()
    t0 = time.time()
    leg = spec_leg(steps=args.steps, warmup=max(args.warmup, 3), device=local)
    clock_info = clocks.stop(t0, time.time())
    t = torch.tensor([leg["ms_per_step"]], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    peak, peak_kind = measured_peak()
    if rank == 0:
        print(json.dumps({
            "metric": "verified sequences/s (32 seq x (9 target + 8 draft) x V=151,936 fp32 per GPU)",
            "value": 32 * world / (ms / 1000.0), "unit": "sequences/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "c4_spec_verify", "sequences_per_gpu": 32, "draft_len": 8, "vocab": 151936,
                       "sharding": f"sequences x{world}", "l2": leg["l2"]},
            "roofline": {"bound": "hbm", "achieved": leg["achieved_gbs"], "peak": peak, "unit": "GB/s",
                         "frac": leg["achieved_gbs"] / peak, "peak_kind": peak_kind, "traffic": None},
            "clocks": clock_info, "accepted_mean": leg["accepted_mean"]}))
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
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline and parity leg")
    ap.add_argument("--no-legs", action="store_true", help="skip the short legs over the other configurations")
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
    # the engine's stream: every call, copy and timing event of the run goes on it.  The legacy default
    # stream cannot be captured, and the library replays a repeated step as a CUDA graph where it can.
    torch.cuda.set_stream(torch.cuda.Stream(device=local))

    from opentail.stingray_b200 import BatchSampler

    w = make_workload(args.config, rank)
    hist_max = int(np.diff(w.history_offsets).max()) if w.history_offsets is not None else 0
    bs = BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=max(hist_max, 1),
                      max_top_k=max(int(w.params["top_k"].max()), 1), device=local, host_logits=True)
    n_copies = copies_for(w.logits.nbytes)
    devs = [to_device(w) for _ in range(n_copies)]

    outs = [None] * n_copies  # fixed output buffers, one set per input copy, as an engine keeps them

    def step(i):
        d = devs[i % n_copies]
        kw = dict(uniforms=d["uniforms"])
        if w.history_ids is not None:
            kw.update(history_ids=d["history_ids"], history_offsets=w.history_offsets)
        if w.mask is not None:
            kw.update(mask=d["mask"])
        outs[i % n_copies] = bs.sample_rows(d["logits"], w.params, want_flags=True, out=outs[i % n_copies], **kw)
        return outs[i % n_copies]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 2 * n_copies + 1)  # each input copy twice: the second sighting captures the step's graph
    for i in range(warmup):
        step(i)
    barrier()
    launches0 = bs.stats()["kernel_launches"]
    replays0 = bs.stats()["graph_replays"]
    clocks = ClockSampler(local)
    clocks.start()
    time.sleep(0.25)
    barrier()
    t_wall0 = time.time()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        last = step(i)
    ev1.record()
    torch.cuda.synchronize()
    ms_total = ev0.elapsed_time(ev1)
    launches = bs.stats()["kernel_launches"] - launches0
    replays = bs.stats()["graph_replays"] - replays0
    gpu_tokens = last["tokens"].cpu().numpy()
    gpu_flags = last["flags"].cpu().numpy().view(np.uint32)

    # per-step durations of the step's kernels (roofline numerator), same stream, same inputs
    launch_ms_mean = timed_each(step, args.steps, 0)
    clock_info = clocks.stop(t_wall0, time.time())

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
    e2e_tokens = np.asarray(out["tokens"])
    # the bound of the end-to-end step: the same bytes as one plain pinned host-to-device copy, no compute
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    devs[0]["logits"].view(torch.int16 if w.logits.dtype == np.uint16 else torch.float32).copy_(pin["logits"], non_blocking=True)
    torch.cuda.synchronize()
    c0.record()
    for _ in range(3):
        devs[0]["logits"].view(torch.int16 if w.logits.dtype == np.uint16 else torch.float32).copy_(pin["logits"], non_blocking=True)
    c1.record()
    torch.cuda.synchronize()
    copy_ms = c0.elapsed_time(c1) / 3

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
    bs.close()
    del devs, pin
    torch.cuda.empty_cache()

    legs = {}
    if not args.no_legs and args.config == "c2":
        if world > 1:
            legs.update(c5_sharded_legs(rank, world, local))
        if rank == 0:
            from opentail.stingray_b200 import workloads as W

            flush = L2Flush()
            legs["c1_single_row"] = sampling_leg(W.config1(), device=local, flush=flush)
            legs["c3_grammar_masked"] = sampling_leg(W.config3(), device=local)
            legs["c4_spec_verify"] = spec_leg(device=local)
            legs["c5_shard_512_rows"] = sampling_leg(W.config5(rows=512), steps=8, device=local)
            greedy = W._params(w.rows, temperature=0.0)
            topk = W._params(w.rows, top_k=50, top_p=0.95)
            topk_pen = W._params(w.rows, top_k=50, top_p=0.95, frequency_penalty=0.5, presence_penalty=0.3)
            legs["c2_all_greedy"] = sampling_leg(w, device=local, params=greedy, use_history=False)
            legs["c2_all_top_k_50"] = sampling_leg(w, device=local, params=topk, use_history=False)
            legs["c2_all_top_k_50_history_512"] = sampling_leg(w, device=local, params=topk_pen)
            legs["c2_vary_plan"] = vary_plan_leg(w, device=local)
            legs["c2_kernel_times"] = kernel_times_leg(w, device=local)
            legs["reference_gpu_argmax"] = reference_gpu_argmax_leg(w, device=local)
            del flush
            torch.cuda.empty_cache()

    rc = 0
    if rank == 0:
        line = {
            "metric": metric_name(w), "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32" if w.logits.dtype == np.float32 else "bf16", "data": "synthetic",
            "config": config_block(w, world, n_copies),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_8TBs": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": alg_bytes, "launch_ms": launch_ms_mean,
                         "traffic": ncu_traffic(f"sample_step_{args.config}")},
            "e2e": {"value": total_rows / (e2e_ms / 1000.0), "unit": "rows/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4 * w.rows, "ms_per_step": e2e_ms,
                    "h2d_gbs_per_rank": h2d / (e2e_ms / 1000.0) / 1e9,
                    "pinned_copy_of_the_logits_alone_ms": copy_ms, "copy_share_of_step": copy_ms / e2e_ms},
            "gpu_launches": launches,
            "graph_replays": replays,
            "clocks": clock_info,
        }
        if not args.no_cpu:
            dt, tokens, traces = oracle_pass(w, 1, 256)
            rows = tokens.size
            total_dt, passes = dt, 1
            reps = int(min(20, max(0, round(12.0 / max(dt, 0.05)) - 1)))  # about 12 s of CPU work in all
            for _ in range(reps):
                total_dt += oracle_pass(w, 1, 256)[0]
                passes += 1
            line["cpu_baseline"] = {"value": rows * passes / total_dt, "unit": "rows/s", "cores": 1, "kind": "port",
                                    "sample": f"{rows} rows of the same batch, {passes} passes ({total_dt:.1f} s), "
                                              f"single thread as the reference's serial loop"}
            # parity of the timed step (device inputs) and of the end-to-end step (host inputs)
            diff = np.nonzero(gpu_tokens[:rows] != tokens)[0]
            boundary = int(sum(1 for r in diff if float(traces["margin"][r]) <= BOUNDARY))
            ties = int(((gpu_flags[:rows] >> 4) & 1).sum())
            line["parity"] = {"rows": int(rows), "mismatch": int(diff.size), "boundary": boundary, "tie_rows": ties,
                              "near_cut_rows": int(((traces["cut_margin"] > 0) & (traces["cut_margin"] <= BOUNDARY)).sum()),
                              "e2e_tokens_equal_device_tokens": bool(np.array_equal(e2e_tokens, gpu_tokens)),
                              "checker": "oracle/sampler_oracle.c, same rows, same uniforms"}
            if diff.size != boundary or not line["parity"]["e2e_tokens_equal_device_tokens"]:
                rc = 3
        if legs:
            line["configs"] = legs
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rc:
        sys.stderr.write("bench.py: sampled tokens differ from the oracle's outside the boundary rule\n")
        sys.exit(rc)


if __name__ == "__main__":
    main()
