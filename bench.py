#!/usr/bin/env python3
"""Benchmark of the hot path: Q4_K decode mat-mul (MUL_MAT with one activation row) over
the four weight shapes of the quantized sweep, reported as HBM GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass over the four shapes (4096x4096, 14336x4096, 4096x14336,
128256x4096; 371 MB of Q4_K weights, more than L2, so no flush is needed between
steps).  `value` has the activations resident in HBM; `e2e` goes through the
host-buffer entry point (pinned host activations in, results out, every step).
`--impl reference` times the CPU restatement of the reference's route on the host
cores.  One JSON line is printed by rank 0.
"""
import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "tests"))

Q4_K = 12
SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]  # (n rows, k)
DISTINCT_ROWS = 4096  # rows quantized for real; larger matrices repeat them (timing does not depend on values)
METRIC = "q4_K_decode_mat_mul_hbm_gbs"


def algorithmic_bytes(n, k, m=1):
    """quantized weight bytes + f32 activations in + f32 results out"""
    return n * k * 144 // 256 + 4 * m * k + 4 * m * n


def load_pkg():
    spec = importlib.util.spec_from_file_location("llama_rust_b200", os.path.join(ROOT, "llama.rust_b200", "__init__.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["llama_rust_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def synth_weights(n, k, seed):
    import orc  # the oracle's restatement of quantize_row_q4_K_ref makes the synthetic weights
    rng = np.random.default_rng(seed)
    rows = min(n, DISTINCT_ROWS)
    w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    q = orc.quantize_rows(Q4_K, w)
    if rows < n:
        q = np.tile(q, ((n + rows - 1) // rows, 1))[:n]
    return np.ascontiguousarray(q)


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        self.idx = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(n_gpus):
    """(rank, world, barrier, reduce_max).  torch.distributed only carries the barrier and the max."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return 0, 1, (lambda: None), (lambda v: v)
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    dist.init_process_group(backend=backend)
    dev = torch.device("cuda", local) if backend == "nccl" else torch.device("cpu")

    def barrier():
        dist.barrier()

    def reduce_max(v):
        t = torch.tensor([float(v)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    return rank, world, barrier, reduce_max


def cpu_step(orc, reps_w, x_list, outs, threads):
    for (ty, n, k, wrep), x, out in zip(reps_w, x_list, outs):
        r = orc.lib().orc_mul_mat_repacked(ty, n, k, 1, wrep.ctypes.data, x.ctypes.data, out.ctypes.data, threads)
        assert r > 0


def cpu_prepare(orc):
    """weights in the CPU path's 8x8 interleaved layout, built before timing as the
    reference's warm_repack does"""
    reps, xs, outs = [], [], []
    for i, (n, k) in enumerate(SHAPES):
        W = synth_weights(n, k, seed=100 + i)
        reps.append((Q4_K, n, k, orc.repack_8x8(Q4_K, W, n, k)))
        xs.append(np.random.default_rng(200 + i).standard_normal((1, k)).astype(np.float32))
        outs.append(np.zeros((1, n), dtype=np.float32))
    return reps, xs, outs


def run_reference(args, rank, world):
    """The CPU route the reference takes for this workload (8x8 interleaved Q4_K gemv on Q8_K
    activations), restated in C++ because the Rust reference cannot be built here."""
    if rank != 0:
        return
    import orc
    threads = orc.lib().orc_num_threads()
    reps, xs, outs = cpu_prepare(orc)
    total = sum(algorithmic_bytes(n, k) for n, k in SHAPES)
    for _ in range(args.warmup):
        cpu_step(orc, reps, xs, outs, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(orc, reps, xs, outs, threads)
    dt = time.perf_counter() - t0
    gbs = total * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8xint4 dot, f32 accumulate", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"the full step (4 shapes, {total} algorithmic bytes) x {args.steps}"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config():
    return {"workload": "MUL_MAT Q4_K x f32, 1 activation row, shapes (n x k) " +
                        ", ".join(f"{n}x{k}" for n, k in SHAPES),
            "weights": "N(0,0.02) through quantize_row_q4_K_ref, seeded", "activations": "N(0,1), seeded",
            "l2": "371 MB of weights per step exceed the 126 MB L2; no flush between steps",
            "parallelism": "replicas"}


def run_b200(args, rank, world, barrier, reduce_max):
    b = load_pkg()
    if b.device_count() == 0:
        raise SystemExit("bench.py: no CUDA device; the CUDA library is the only compute path")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    b.set_device(local)
    weights, dxs, douts, acts, hxs, houts = [], [], [], [], [], []
    for i, (n, k) in enumerate(SHAPES):
        weights.append(b.Weight(Q4_K, synth_weights(n, k, seed=100 + i), k))
        x = np.random.default_rng(200 + i).standard_normal((1, k)).astype(np.float32)
        hxs.append(x)
        dxs.append(b.device_array(x))
        douts.append(b.DeviceBuffer(4 * n))
        acts.append(b.DeviceBuffer(b.lib.b200_act_scratch_nbytes(1, k)))
        houts.append(np.zeros((1, n), dtype=np.float32))
    total = sum(algorithmic_bytes(n, k) for n, k in SHAPES)

    def step_device():
        for w, dx, do in zip(weights, dxs, douts):
            b.mul_mat_device(w, dx, 1, do)

    def step_host():
        for w, hx, ho in zip(weights, hxs, houts):
            b.check(b.lib.b200_mul_mat_host(w.ty, w.n_rows, w.k, 1, w.ptr, hx.ctypes.data, ho.ctypes.data, 0, None),
                    "mul_mat_host")

    # ---- device-resident throughput -------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step_device()
    b.synchronize()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = b.Event(), b.Event()
    e0.record()
    for _ in range(args.steps):
        step_device()
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_ms(e1)
    barrier()
    ms = reduce_max(ms)

    # ---- the mat-mul kernel alone (activations already quantized): roofline ---------
    # Per shape: back-to-back launches rotating over enough weight copies to exceed twice the L2, one
    # pair of CUDA events around the batch (the stream is what a decode step looks like: launches queue
    # behind each other and each kernel's weight prefetch overlaps the tail of the one before).
    kern_ms, per_shape = [], {}
    launches = max(4 * args.steps, 100)
    for (n, k), w0, dx, do, act in zip(SHAPES, weights, dxs, douts, acts):
        b.check(b.lib.b200_quantize_activations_device(b.ACT_Q8_K, 1, k, dx.ptr, k, act.ptr, None), "quantize")
        wbytes = n * k * 144 // 256
        copies = max(2, min(32, (300 << 20) // wbytes + 1))
        ws = [w0] + [b.Weight(Q4_K, w0.download(), k) for _ in range(copies - 1)]

        def launch(i):
            w = ws[i % copies]
            b.check(b.lib.b200_mul_mat_q8(Q4_K, n, k, 1, w.ptr, act.ptr, b.ACT_Q8_K, do.ptr, n, 0, None), "mul_mat_q8")

        for i in range(copies):
            launch(i)
        b.synchronize()
        a, z = b.Event(), b.Event()
        a.record()
        for i in range(launches):
            launch(i)
        z.record()
        z.synchronize()
        t = a.elapsed_ms(z) / launches
        per_shape[f"{n}x{k}"] = {"us": t * 1e3, "gbs": algorithmic_bytes(n, k) / (t * 1e-3) / 1e9, "copies": copies}
        kern_ms.append(t)
        del ws
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the host-buffer entry point -------------------------------
    for _ in range(3):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    b.synchronize()
    e2e_s = reduce_max(time.perf_counter() - t0)

    if rank != 0:
        return
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    kern_gbs = total / (sum(kern_ms) * 1e-3) / 1e9
    value = world * total * args.steps / (ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8xint4 dot, f32 accumulate", "data": "synthetic", "config": workload_config(),
        "clocks": clocks,
        "e2e": {"value": world * total * args.steps / e2e_s / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": sum(4 * k for _, k in SHAPES), "d2h_bytes_per_step": sum(4 * n for n, _ in SHAPES)},
        "gpu_launches": args.steps * 2 * len(SHAPES),
        "roofline": {"bound": "hbm", "kernel": "gemv_q4_K_kernel<1,0> / gemv_q4_K_stream_kernel (Q4_K decode mat-mul)",
                     "achieved": kern_gbs, "peak": peak,
                     "peak_source": peak_src, "unit": "GB/s", "frac": kern_gbs / peak, "traffic": None,
                     "per_shape": per_shape},
    }
    # CPU baseline on the host cores: the same workload through the CPU route, a few repetitions
    try:
        import orc
        threads = orc.lib().orc_num_threads()
        reps_w, xs, outs = cpu_prepare(orc)
        cpu_step(orc, reps_w, xs, outs, threads)
        n_rep, t0 = 0, time.perf_counter()
        while n_rep < 3 or (time.perf_counter() - t0 < 10.0 and n_rep < 50):
            cpu_step(orc, reps_w, xs, outs, threads)
            n_rep += 1
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": total * n_rep / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"the full step x {n_rep} repetitions ({dt:.1f} s)"}
    except Exception as exc:  # the baseline is a reported extra, never the measured path
        line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {exc}"}
    print(json.dumps(line), flush=True)


def run_profile_case(args):
    """A small case for ncu: `--only NxK --launches R` runs R decode mat-muls of one shape,
    rotating over enough weight copies to stay out of L2, and prints the event-timed mean."""
    b = load_pkg()
    b.set_device(0)
    n, k = (int(v) for v in args.only.lower().split("x"))
    wbytes = n * k * 144 // 256
    copies = max(2, min(32, (300 << 20) // wbytes + 1))
    W = synth_weights(n, k, seed=7)
    weights = [b.Weight(Q4_K, W, k) for _ in range(copies)]
    x = np.random.default_rng(8).standard_normal((1, k)).astype(np.float32)
    dx, do = b.device_array(x), b.DeviceBuffer(4 * n)
    act = b.DeviceBuffer(b.lib.b200_act_scratch_nbytes(1, k))
    b.check(b.lib.b200_quantize_activations_device(b.ACT_Q8_K, 1, k, dx.ptr, k, act.ptr, None), "quantize")

    def launch(i):
        w = weights[i % copies]
        b.check(b.lib.b200_mul_mat_q8(Q4_K, n, k, 1, w.ptr, act.ptr, b.ACT_Q8_K, do.ptr, n, 0, None), "mul_mat_q8")

    for i in range(copies):
        launch(i)
    b.synchronize()
    e0, e1 = b.Event(), b.Event()
    e0.record()
    for i in range(args.launches):
        launch(i)
    e1.record()
    e1.synchronize()
    us = e0.elapsed_ms(e1) * 1e3 / args.launches
    print(json.dumps({"case": args.only, "copies": copies, "launches": args.launches, "us_per_launch": us,
                      "gbs": algorithmic_bytes(n, k) / us / 1e3}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, help="profile case: one shape NxK, see --launches")
    ap.add_argument("--launches", type=int, default=64)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    if args.only:
        run_profile_case(args)
        return
    rank, world, barrier, reduce_max = dist_setup(args.gpus)
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_b200(args, rank, world, barrier, reduce_max)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
