#!/usr/bin/env python3
"""Benchmark of the hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-llama]

The JSON line's headline (`metric`, `value`, `roofline`, `e2e`) is the Q4_K decode mat-mul (MUL_MAT with
one activation row) over the four weight shapes of the quantized sweep, in HBM GB/s: one step = one pass
over 4096x4096, 14336x4096, 4096x14336 and 128256x4096 (371 MB of Q4_K weights, more than L2, so no
flush is needed between steps).  `value` has the activations resident in HBM; `e2e` goes through the
host-buffer entry point (host activations in, results out, every step).

The second half of the metric rides in the same line under `llama_8b`: a Llama-3-8B-shaped decoder with
synthetic Q4_K_M weights run by the decode driver (include/llama_b200.h) — a 512-token prompt (pp512)
and 128 greedy steps after it (tg128), in tokens/s, end to end through the driver's host-buffer call
(token ids in, argmax out, every step) and device-only (the step's graph replayed on the stream).

`--impl reference` times the CPU restatement of the reference's routes on the host cores for the same
workloads.  One JSON line is printed by rank 0.  `--case` runs one small case for a profiler.
"""
import argparse
import importlib
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))

Q4_K = 12
SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]  # (n rows, k)
METRIC = "q4_K_decode_mat_mul_hbm_gbs"
# the CPU arm is the oracle's C++ restatement of the reference's routes (no Rust toolchain here) with AVX2 / AVX-512 VNNI
# bodies for the Q4_K 8x8 core and the Q6_K row dot, as the reference's CPU path has (bit-identical to the scalar loops)
CPU_KIND = "port-simd"
SIMD_NAMES = {0: "scalar", 1: "AVX2", 2: "AVX-512 VNNI"}
# measured DRAM bytes / algorithmic bytes of one launch of the decode kernel in use (gemv_q4_K_row_kernel on
# 14336 x 4096: dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture whose summary is kept with the other
# profile summaries); weights are read once whatever the shape
NCU_TRAFFIC_RATIO = 33.052416 / 33.103872
PROMPT, GEN = 512, 128


def algorithmic_bytes(n, k, m=1):
    """quantized weight bytes + f32 activations in + f32 results out"""
    return n * k * 144 // 256 + 4 * m * k + 4 * m * n


def load_pkg():
    if "llama_rust_b200" not in sys.modules:
        spec = importlib.util.spec_from_file_location("llama_rust_b200", os.path.join(ROOT, "llama.rust_b200", "__init__.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules["llama_rust_b200"] = mod
        spec.loader.exec_module(mod)
    return sys.modules["llama_rust_b200"]


def load_standalone(name):
    """llama.rust_b200/<name>.py loaded by path, WITHOUT the package (and so without libggml-b200.so): the CPU arms
    build the same synthetic inputs as the GPU arm and map nothing but the oracle"""
    key = f"_b200_standalone_{name}"
    if key not in sys.modules:
        spec = importlib.util.spec_from_file_location(key, os.path.join(ROOT, "llama.rust_b200", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[key] = mod
        spec.loader.exec_module(mod)
    return sys.modules[key]


def synth_weights(n, k, seed, ty=Q4_K):
    """random well-formed blocks (llama.rust_b200/synth.py); timing does not depend on the values"""
    return load_standalone("synth").blocks(ty, n, k, seed=seed)


def load_oracle():
    """the CPU restatement under oracle/, for the reference arm and the cpu_baseline legs only"""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import orc
    import orc_glue
    return orc, orc_glue


def host_threads(orc):
    """all host cores: torch.distributed.run exports OMP_NUM_THREADS=1 to its workers, which is not what the
    CPU arm should run with (the oracle's entry points take the thread count and set it themselves)"""
    return max(orc.lib().orc_num_threads(), len(os.sched_getaffinity(0)))


def note(msg):
    """progress on stderr, so that a run that stops short shows where"""
    print(f"[bench {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)


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
        # name the device: the CUDA library switches the process's current device as it works, and a barrier that
        # guessed another device would try to build a second communicator there and wait for peers that never come
        if backend == "nccl":
            dist.barrier(device_ids=[local])
        else:
            dist.barrier()

    def reduce_max(v):
        t = torch.tensor([float(v)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    return rank, world, barrier, reduce_max


def peak_hbm():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- the decode mat-mul ---------------------------------------------------------------------------------
def gemv_config():
    return {"workload": "MUL_MAT Q4_K x f32, 1 activation row, shapes (n x k) " + ", ".join(f"{n}x{k}" for n, k in SHAPES),
            "weights": "seeded random well-formed Q4_K blocks (decoded spread ~0.05)", "activations": "N(0,1), seeded",
            "l2": "371 MB of weights per step exceed the 126 MB L2; no flush between steps",
            "parallelism": "replicas"}


def cpu_gemv_prepare(orc):
    """weights in the CPU path's 8x8 interleaved layout, built before timing as the reference's warm_repack does"""
    reps, xs, outs = [], [], []
    for i, (n, k) in enumerate(SHAPES):
        W = synth_weights(n, k, seed=100 + i)
        reps.append((Q4_K, n, k, orc.repack_8x8(Q4_K, W, n, k)))
        xs.append(np.random.default_rng(200 + i).standard_normal((1, k)).astype(np.float32))
        outs.append(np.zeros((1, n), dtype=np.float32))
    return reps, xs, outs


def cpu_gemv_step(orc, reps_w, x_list, outs, threads):
    for (ty, n, k, wrep), x, out in zip(reps_w, x_list, outs):
        r = orc.lib().orc_mul_mat_repacked(ty, n, k, 1, wrep.ctypes.data, x.ctypes.data, out.ctypes.data, threads)
        assert r > 0


def cpu_gemv_baseline(orc, seconds=10.0):
    threads = host_threads(orc)
    total = sum(algorithmic_bytes(n, k) for n, k in SHAPES)
    reps_w, xs, outs = cpu_gemv_prepare(orc)
    cpu_gemv_step(orc, reps_w, xs, outs, threads)
    n_rep, t0 = 0, time.perf_counter()
    while n_rep < 3 or (time.perf_counter() - t0 < seconds and n_rep < 5000):
        cpu_gemv_step(orc, reps_w, xs, outs, threads)
        n_rep += 1
    dt = time.perf_counter() - t0
    level = orc.simd_level()
    return {"value": total * n_rep / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": CPU_KIND if level else "port",
            "simd": SIMD_NAMES[level], "sample": f"the full step x {n_rep} repetitions ({dt:.1f} s)"}


def run_gemv(b, args, rank, world, barrier, reduce_max, local):
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
            b.check(b.lib.b200_mul_mat_host(w.ty, w.n_rows, w.k, 1, w.ptr, hx.ctypes.data, ho.ctypes.data, 0, None), "mul_mat_host")

    warm = max(args.warmup, 3)
    for _ in range(warm):
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

    # the mat-mul kernel alone (activations already quantized), per shape: launches rotating over enough weight copies
    # to exceed twice the L2, captured into ONE CUDA graph and replayed, CUDA events around the replay on the launching
    # stream (b200_bench_mul_mat_q8): what the kernel costs inside a decode step, where a replayed graph issues the
    # launches; a host loop over the entry point measures the host's launch rate for the small shapes
    kern_ms, per_shape = [], {}
    launches = max(4 * args.steps, 100)
    for (n, k), w0, dx, do, act in zip(SHAPES, weights, dxs, douts, acts):
        b.check(b.lib.b200_quantize_activations_device(b.ACT_Q8_K, 1, k, dx.ptr, k, act.ptr, None), "quantize")
        wbytes = n * k * 144 // 256
        copies = max(2, min(32, (300 << 20) // wbytes + 1))
        ws = [w0] + [b.Weight(Q4_K, w0.download(), k) for _ in range(copies - 1)]
        t = b.bench_mul_mat_q8(ws, act, b.ACT_Q8_K, do, 1, launches) * 1e-3
        per_shape[f"{n}x{k}"] = {"us": t * 1e3, "gbs": algorithmic_bytes(n, k) / (t * 1e-3) / 1e9, "frac": algorithmic_bytes(n, k) / (t * 1e-3) / 1e9 / peak_hbm()[0],
                                 "copies": copies}
        kern_ms.append(t)
        del ws
    clocks = sampler.stop() if rank == 0 else None

    for _ in range(3):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    b.synchronize()
    e2e_s = reduce_max(time.perf_counter() - t0)
    peak, peak_src = peak_hbm()
    kern_gbs = total / (sum(kern_ms) * 1e-3) / 1e9
    return {
        "value": world * total * args.steps / (ms * 1e-3) / 1e9, "ms_per_step": ms / args.steps, "clocks": clocks, "warmup": warm,
        "e2e": {"value": world * total * args.steps / e2e_s / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": sum(4 * k for _, k in SHAPES), "d2h_bytes_per_step": sum(4 * n for n, _ in SHAPES)},
        "gpu_launches": args.steps * 2 * len(SHAPES),
        "roofline": {"bound": "hbm", "kernel": "gemv_q4_K_row_kernel (Q4_K decode mat-mul, one activation row)",
                     "achieved": kern_gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": kern_gbs / peak,
                     "timing": "per shape: launches over rotating weight copies (> 2 x L2) replayed as one CUDA graph, CUDA events on the launching stream",
                     # bytes per step (the four launches)
                     "traffic": total * NCU_TRAFFIC_RATIO, "traffic_source": "ncu capture of this kernel on 14336x4096 (profiles/), scaled by algorithmic bytes",
                     "per_shape": per_shape},
    }


# ---- the Llama-3-8B-shaped decoder ------------------------------------------------------------------------
def llama_hparams(n_layer, shape="8b"):
    """(shapes module, hyper-parameters); pure Python, no library"""
    sh = load_standalone("shapes")
    hp = dict(sh.LLAMA3_70B if shape == "70b" else sh.LLAMA3_8B)
    hp["n_layer"] = n_layer
    return sh, hp


def llama_weight_bytes(ll, hp):
    """bytes of quantized weights one decode step streams: every matrix once, one row of token_embd"""
    syn = load_standalone("synth")
    total = 0
    for name, (ne0, ne1) in ll.tensor_shapes(hp).items():
        ty = ll.q4_k_m_type(name, hp["n_layer"])
        if ty == 0:
            total += 4 * ne0
        else:
            per, size = syn.BLOCK[ty]
            total += (1 if name == "token_embd.weight" else ne1) * (ne0 // per) * size
    return total


def build_llama(n_layer, n_ctx=1024, n_batch=PROMPT, keep_host=False, device=0, shape="8b"):
    load_pkg()
    sh, hp = llama_hparams(n_layer, shape)
    ll = importlib.import_module("llama_rust_b200.llama")
    syn = load_standalone("synth")
    gpu = ll.Llama(hp, n_ctx, n_batch, device=device, cpu_threads=8)
    host = {}
    for name, ty, arr, ne0, ne1 in syn.llama_tensors(hp, lambda n: sh.q4_k_m_type(n, n_layer), tensor_shapes=sh.tensor_shapes):
        gpu.set_tensor(name, ty, arr, ne0, ne1)
        if keep_host:
            host[name] = (ty, arr, ne0, ne1)
    return ll, hp, gpu, host


N_SEQ = 16


def run_llama_batch16(gpu, hp, world, barrier, reduce_max):
    """16 parallel sequences in the unified cache: 16 prompts of 512 tokens (one sequence per call), then 128
    steps of one token per sequence; tokens/s over all sequences, end to end through the driver call"""
    rng = np.random.default_rng(1)
    prompts = rng.integers(0, hp["n_vocab"], (N_SEQ, PROMPT)).astype(np.int32)
    pos = np.arange(PROMPT, dtype=np.int32)
    seqs = np.arange(N_SEQ, dtype=np.int32)

    def one_pass():
        gpu.kv_clear()
        nxt = np.zeros(N_SEQ, dtype=np.int32)
        t0 = time.perf_counter()
        for s in range(N_SEQ):
            _, am = gpu.decode_seqs(prompts[s], pos, np.full(PROMPT, s, dtype=np.int32), [PROMPT - 1], logits=False, argmax=True)
            nxt[s] = am[0]
        t1 = time.perf_counter()
        for i in range(GEN):
            _, am = gpu.decode_seqs(nxt, np.full(N_SEQ, PROMPT + i, dtype=np.int32), seqs, seqs, logits=False, argmax=True)
            nxt = am.astype(np.int32)
        t2 = time.perf_counter()
        return t1 - t0, (t2 - t1) / GEN, gpu.replay(8) / 8 * 1e-3

    one_pass()
    barrier()
    res = [one_pass() for _ in range(2)]
    barrier()
    pp, tg, tg_dev = (reduce_max(min(r[k] for r in res)) for k in range(3))
    return {"sequences": N_SEQ, "pp512_e2e_tok_s": world * N_SEQ * PROMPT / pp, "tg128_e2e_tok_s": world * N_SEQ / tg,
            "tg128_tok_s": world * N_SEQ / tg_dev, "tg128_ms_per_step": tg_dev * 1e3,
            "cache": f"unified, {N_SEQ * (PROMPT + GEN)} cells in use at the end; a row's mask hides the other sequences' cells"}


def time_llama_passes(gpu, hp, world, barrier, reduce_max, warm=2, reps=3):
    """pp512 + tg128 of one driver in the library's current numerics mode -> (pp_e2e, pp_dev, tg_e2e, tg_dev, tokens)"""
    prompt = np.random.default_rng(0).integers(0, hp["n_vocab"], PROMPT).astype(np.int32)
    pos = np.arange(PROMPT, dtype=np.int32)

    def one_pass():
        gpu.kv_clear()
        t0 = time.perf_counter()
        tok = gpu.decode(prompt, pos, logits=False, argmax=True)
        t1 = time.perf_counter()
        pp_dev = gpu.replay(1)
        toks = []
        t2 = time.perf_counter()
        for i in range(GEN):
            tok = gpu.decode([tok], [PROMPT + i], logits=False, argmax=True)
            toks.append(tok)
        t3 = time.perf_counter()
        tg_dev = gpu.replay(GEN) / GEN
        return t1 - t0, pp_dev * 1e-3, (t3 - t2) / GEN, tg_dev * 1e-3, toks

    for _ in range(warm):   # warm-up passes: allocations, graph capture
        one_pass()
    barrier()
    res = [one_pass() for _ in range(reps)]
    barrier()
    return tuple(reduce_max(statistics.median(r[k] for r in res)) for k in range(4)) + (res[-1][4],)


PARITY_PROMPT, PARITY_STEPS = 16, 4
CPU_TG_STEPS = 64   # single-token steps the CPU leg times (the first PARITY_STEPS of them are the parity comparison)


def gpu_greedy_trace(gpu, hp):
    """the logits of a 16-token prompt's last token and of 4 greedy steps after it, with the tokens fed (the same
    prompt the CPU leg of the benchmark runs)"""
    prompt = np.random.default_rng(0).integers(0, hp["n_vocab"], PARITY_PROMPT).astype(np.int32)
    gpu.kv_clear()
    logits, tok = gpu.decode(prompt, np.arange(PARITY_PROMPT), logits=True, argmax=True)
    trace, toks = [logits], [int(tok)]
    for i in range(PARITY_STEPS):
        logits, tok = gpu.decode([toks[-1]], [PARITY_PROMPT + i], logits=True, argmax=True)
        trace.append(logits)
        toks.append(int(tok))
    return trace, toks


def compare_greedy(gpu_trace, gpu_toks, cpu_trace, cpu_toks):
    """greedy-stream parity of a GPU run against the CPU port: are the token streams identical, where do they first
    differ, and how far apart are the logits while the streams still agree"""
    first, worst, bits = None, 0.0, True
    for i, (g, c) in enumerate(zip(gpu_trace, cpu_trace)):
        worst = max(worst, float(np.abs(g - c).max() / max(float(np.abs(c).max()), 1e-30)))
        bits = bits and bool(np.array_equal(g.view(np.uint32), c.view(np.uint32)))
        if gpu_toks[i] != cpu_toks[i]:
            first = i
            break
    return {"identical": first is None, "first_divergence": first, "steps_compared": len(gpu_trace) if first is None else first + 1,
            "max_rel_logit_err": worst, "logits_bit_identical": bits if first is None else False,
            "tokens": gpu_toks, "cpu_tokens": cpu_toks}


def run_llama(b, args, rank, world, barrier, reduce_max):
    """pp512 + tg128, batch 1, one replica per rank; the fast numerics mode (the library's default) and the exact one"""
    ll, hp, gpu, _ = build_llama(args.layers, n_ctx=N_SEQ * (PROMPT + GEN), device=int(os.environ.get("LOCAL_RANK", "0")))
    peak, peak_src = peak_hbm()
    wbytes = llama_weight_bytes(ll, hp)
    out = {"config": {"workload": f"Llama-3-8B shape ({hp['n_layer']} layers, d_model 4096, 32/8 heads, FFN 14336, vocab 128256), "
                                  "Q4_K_M tensor types, F16 KV cache, batch 1: 512-token prompt then 128 greedy steps",
                      "weights": "seeded random well-formed blocks", "tokens": "uniform random prompt ids, seeded",
                      "device_time": "tg128_tok_s / pp512_tok_s: the step's captured CUDA graph replayed on the stream with the last "
                                     "step's inputs (kernel time of a step); *_e2e_*: the driver call per step, host ids in, argmax out"}}
    traces = {}
    for mode, name in ((b.FAST, "fast"), (b.EXACT, "exact")):
        b.set_numerics(mode)
        pp_e2e, pp_dev, tg_e2e, tg_dev, toks = time_llama_passes(gpu, hp, world, barrier, reduce_max, warm=2 if name == "fast" else 1,
                                                                 reps=3 if name == "fast" else 2)
        res = {"pp512_tok_s": world * PROMPT / pp_dev, "pp512_e2e_tok_s": world * PROMPT / pp_e2e,
               "tg128_tok_s": world / tg_dev, "tg128_e2e_tok_s": world / tg_e2e,
               "pp512_ms": pp_dev * 1e3, "tg128_ms_per_token": tg_dev * 1e3,
               "roofline": {"bound": "hbm", "what": "tg128: quantized weight bytes one step streams / device time of the step",
                            "bytes_per_token": wbytes, "achieved": wbytes / tg_dev / 1e9, "peak": peak, "peak_source": peak_src,
                            "unit": "GB/s", "frac": wbytes / tg_dev / 1e9 / peak},
               "greedy_tokens_head": [int(t) for t in toks[:8]]}
        if name == "fast":
            out.update(res)
            out["numerics"] = "fast (the library's default: attention accumulates in f32, 1e-6 from float64; every mat-mul bit-exact)"
            out["e2e_bytes_per_step"] = {"h2d": "token ids, positions, F16 mask, cache row indices", "d2h": "4 (argmax)"}
            out["batch16"] = run_llama_batch16(gpu, hp, world, barrier, reduce_max)
        else:
            out["exact_numerics"] = res
        if world == 1:
            traces[name] = gpu_greedy_trace(gpu, hp)
    b.set_numerics(b.FAST)
    gpu.close()
    if world == 1 and not args.no_persistent:
        try:
            out["persistent_step_kernel"] = run_llama_persistent(b, args, out.get("greedy_tokens_head"))
        except Exception as exc:   # an optional leg: say why it is missing
            out["persistent_step_kernel"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    return out, traces


def run_llama_persistent(b, args, node_path_tokens):
    """The same single-token steps with the whole step as ONE persistent kernel (opt-in: B200_DECODE_PERSISTENT=1): tokens/s,
    the greedy tokens against the node-by-node run, and the mean time CTA 0 spends in each phase of a layer"""
    import ctypes
    old = os.environ.get("B200_DECODE_PERSISTENT")
    os.environ["B200_DECODE_PERSISTENT"] = "1"   # read when the backend is created
    try:
        ll, hp, gpu, _ = build_llama(args.layers, n_ctx=2 * (PROMPT + GEN), device=int(os.environ.get("LOCAL_RANK", "0")))
    finally:
        if old is None:
            del os.environ["B200_DECODE_PERSISTENT"]
        else:
            os.environ["B200_DECODE_PERSISTENT"] = old
    b.set_numerics(b.FAST)
    before = b.lib.b200_debug_decode_step_launches()
    ident = lambda x: x
    pp_e2e, pp_dev, tg_e2e, tg_dev, toks = time_llama_passes(gpu, hp, 1, lambda: None, ident, warm=1, reps=2)
    steps = b.lib.b200_debug_decode_step_launches() - before
    n = hp["n_layer"] * 5 + 1
    buf = (ctypes.c_ulonglong * n)()
    b.lib.b200_debug_decode_step_times.argtypes = [ctypes.c_void_p, ctypes.c_int]
    got = b.lib.b200_debug_decode_step_times(buf, n)
    phases = {}
    if got == n:
        d = np.diff(np.array(buf[:got], dtype=np.float64)) / 1e3
        for i, nm in enumerate(("qkv", "attention", "attn_output", "gate_up", "ffn_down")):
            phases[nm] = float(np.mean(d[i::5][:hp["n_layer"]]))
        phases["output"] = None   # the last phase ends with the kernel, not at a barrier
    gpu.close()
    return {"tg128_tok_s": 1.0 / tg_dev, "tg128_e2e_tok_s": 1.0 / tg_e2e, "tg128_ms_per_token": tg_dev * 1e3, "steps_run_as_one_kernel": int(steps),
            "greedy_tokens_head": [int(t) for t in toks[:8]], "same_tokens_as_node_path": node_path_tokens == [int(t) for t in toks[:8]] if node_path_tokens else None,
            "us_per_layer_phase_cta0": phases,
            "note": "opt-in: slower than the node-by-node step of the same run; the phase times (grid barrier to grid barrier) show where"}


def run_llama_70b_one_gpu(b, args):
    """the 70B shape on ONE GPU (40 GB of Q4_K_M weights fit): the base of the tensor-parallel strong-scaling curve"""
    ll, hp, gpu, _ = build_llama(80 if args.layers == 32 else args.layers, n_ctx=1024, shape="70b")
    ident = lambda v: v
    pp_e2e, pp_dev, tg_e2e, tg_dev, _ = time_llama_passes(gpu, hp, 1, (lambda: None), ident, warm=1, reps=2)
    wbytes = llama_weight_bytes(ll, hp)
    peak, peak_src = peak_hbm()
    gpu.close()
    return {"tp": 1, "shape": "70b", "pp512_tok_s": PROMPT / pp_dev, "pp512_e2e_tok_s": PROMPT / pp_e2e, "tg128_tok_s": 1.0 / tg_dev,
            "tg128_e2e_tok_s": 1.0 / tg_e2e, "pp512_ms": pp_dev * 1e3, "tg128_ms_per_token": tg_dev * 1e3,
            "roofline": {"bound": "hbm", "bytes_per_token": wbytes, "achieved": wbytes / tg_dev / 1e9, "peak": peak, "peak_source": peak_src,
                         "unit": "GB/s", "frac": wbytes / tg_dev / 1e9 / peak}}


def run_llama_tp(b, args, rank, world, local, barrier, reduce_max, shape):
    """The same pp512 + tg128, one model split row-wise over all ranks (NCCL all-reduce after attn_output and
    ffn_down, all-gather of the logits): tokens/s of the group, strong scaling.  Each rank makes its own
    random shard, already cut."""
    import torch
    import torch.distributed as dist
    ll = importlib.import_module("llama_rust_b200.llama")
    syn = load_standalone("synth")
    hp = dict(ll.LLAMA3_70B if shape == "70b" else ll.LLAMA3_8B)
    if args.layers != 32:   # a shortened model for a quick check of the multi-rank path
        hp["n_layer"] = args.layers
    ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        ident = torch.tensor(list(ll.tp_unique_id()), dtype=torch.uint8, device="cuda")
    dist.broadcast(ident, 0)
    gpu = ll.Llama(hp, 1024, PROMPT, device=local, cpu_threads=8, tp_rank=rank, tp_size=world, tp_id=bytes(ident.cpu().tolist()))
    rng = np.random.default_rng(1000 + rank)
    for i, (name, (ne0, ne1)) in enumerate(ll.tensor_shapes(hp).items()):
        ty = ll.q4_k_m_type(name, hp["n_layer"])
        _, l0, l1 = ll.tp_shard_shape(name, ty, ne0, ne1, world)
        if ty == 0:
            gpu.set_tensor_shard(name, ty, (1.0 + 0.1 * rng.standard_normal(l0)).astype(np.float32), l0, l1)
        else:
            gpu.set_tensor_shard(name, ty, syn.blocks(ty, l1, l0, seed=7919 * rank + i), l0, l1)
    prompt = np.random.default_rng(0).integers(0, hp["n_vocab"], PROMPT).astype(np.int32)
    pos = np.arange(PROMPT, dtype=np.int32)

    def one_pass():
        gpu.kv_clear()
        barrier()
        t0 = time.perf_counter()
        tok = gpu.decode(prompt, pos, logits=False, argmax=True)
        t1 = time.perf_counter()
        pp_dev = gpu.replay(1)
        barrier()
        t2 = time.perf_counter()
        for i in range(GEN):
            tok = gpu.decode([tok], [PROMPT + i], logits=False, argmax=True)
        t3 = time.perf_counter()
        tg_dev = gpu.replay(GEN) / GEN
        return t1 - t0, pp_dev * 1e-3, (t3 - t2) / GEN, tg_dev * 1e-3

    kind = gpu.tp_exchange_kind()
    for _ in range(2):
        one_pass()
    res = [one_pass() for _ in range(3)]
    barrier()
    pp_e2e, pp_dev, tg_e2e, tg_dev = (reduce_max(statistics.median(r[k] for r in res)) for k in range(4))
    gpu.close()
    return {"tp": world, "scaling": "strong", "shape": shape,
            "collectives": ("decode steps: one kernel of the library per all-reduce / all-gather over peer-mapped memory (NVLink), partial sums "
                            "added in rank order, inside the step's CUDA graph; prompt batches (> 131072 floats per rank): NCCL")
                           if kind == 1 else "NCCL (the peer-memory exchange was not available or was switched off)",
            "config": {"workload": f"Llama-3-{shape.upper()} shape, Q4_K_M tensor types, row-split over {world} GPUs, batch 1: "
                                   "512-token prompt then 128 greedy steps", "weights": "seeded random well-formed blocks, one shard per rank"},
            "pp512_tok_s": PROMPT / pp_dev, "pp512_e2e_tok_s": PROMPT / pp_e2e, "tg128_tok_s": 1.0 / tg_dev, "tg128_e2e_tok_s": 1.0 / tg_e2e,
            "pp512_ms": pp_dev * 1e3, "tg128_ms_per_token": tg_dev * 1e3}


def cpu_llama_baseline(orc, orc_glue, n_layer, prompt_tokens=PARITY_PROMPT, gen_tokens=CPU_TG_STEPS):
    """The CPU restatement's Llama forward on the same shape: a prompt batch and a few greedy single-token steps.
    Weights are interleaved once, outside the timed region, as the reference does at load.  Also returns the logits
    and tokens of the run (the greedy-stream parity check of the GPU arm compares with them)."""
    sh, hp = llama_hparams(n_layer)
    syn = load_standalone("synth")
    tensors = {name: (ty, arr) for name, ty, arr, _, _ in syn.llama_tensors(hp, lambda n: sh.q4_k_m_type(n, n_layer), tensor_shapes=sh.tensor_shapes)}
    ohp = dict(n_vocab=hp["n_vocab"], n_embd=hp["n_embd"], n_head=hp["n_head"], n_head_kv=hp["n_head_kv"],
               head_dim=hp["n_embd_head"], n_ff=hp["n_ff"], n_layer=n_layer, rope_mode=0, n_ctx_orig=hp["n_ctx_train"],
               norm_eps=hp["norm_rms_eps"], freq_base=hp["rope_freq_base"], freq_scale=1.0)
    threads = host_threads(orc)
    cpu = orc_glue.Llama(ohp, tensors, 256)
    wide = bool(__builtin_cpu_wide_silu())

    def fwd(toks, p0):
        n = len(toks)
        mask = np.full((n, 256), 0xFC00, dtype=np.uint16)
        for i in range(n):
            mask[i, :p0 + i + 1] = 0
        return cpu.forward(toks, np.arange(p0, p0 + n), 256, mask, np.arange(p0, p0 + n), [n - 1], n_threads=threads,
                           wide_silu=wide, keep_repacked=True)[0]

    prompt = np.random.default_rng(0).integers(0, hp["n_vocab"], prompt_tokens).astype(np.int32)
    fwd(prompt[:4], 0)            # interleaves every weight (untimed), like the reference's load
    fwd(prompt[:1], 4)
    t0 = time.perf_counter()
    trace = [fwd(prompt, 0)]
    t1 = time.perf_counter()
    toks = [int(orc_glue.argmax(trace[-1]))]
    for i in range(gen_tokens):
        trace.append(fwd(np.array([toks[-1]], dtype=np.int32), prompt_tokens + i))
        toks.append(int(orc_glue.argmax(trace[-1])))
    t2 = time.perf_counter()
    orc_glue.L().orc_llama_drop_repacked()
    res = {"pp_tok_s": prompt_tokens / (t1 - t0), "tg_tok_s": gen_tokens / (t2 - t1), "unit": "tok/s", "cores": threads, "kind": CPU_KIND,
           "sample": f"{n_layer}-layer model of the same shape, one {prompt_tokens}-token prompt batch ({t1 - t0:.1f} s) and "
                     f"{gen_tokens} greedy single-token steps ({t2 - t1:.1f} s) at positions {prompt_tokens}.."}
    return res, trace, toks


def __builtin_cpu_wide_silu():
    """does this host take the 16-lane SILU (AVX512F + DQ)?  Read from /proc/cpuinfo: the CPU arm loads no GPU library"""
    try:
        flags = open("/proc/cpuinfo").read()
        return "avx512f" in flags and "avx512dq" in flags
    except OSError:
        return False


# ---- the quantized mat-mul sweep, MUL_MAT_ID and FLASH_ATTN_EXT configurations ---------------------------------
SWEEP_TYPES = {"Q8_0": (8, 34, 32), "Q4_K": (12, 144, 256), "Q6_K": (14, 210, 256), "MXFP4": (39, 17, 32)}   # id, block bytes, block elements


def peak_tensor():
    """dense int8 peak taken as twice the measured sustained bf16 GEMM rate (the int8 MMA rate is twice the bf16 one)"""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["bf16_tflops_sustained"]), "measured"
    return 1400.0, "fallback"


def event_time(b, fn, reps, warm=2):
    for _ in range(warm):
        fn()
    b.synchronize()
    e0, e1 = b.Event(), b.Event()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_ms(e1) / reps


def run_sweep(b):
    """BASELINE's mat-mul sweep (one weight shape per regime), the MUL_MAT_ID configuration and the FLASH_ATTN_EXT
    configurations, each with its roofline: HBM for the decode-shaped cases, the tensor pipe for the prompt-shaped ones"""
    hbm, hbm_src = peak_hbm()
    tc, tc_src = peak_tensor()
    out = {"peaks": {"hbm_gbs": hbm, "hbm_source": hbm_src, "bf16_tflops_sustained": tc, "tensor_source": tc_src,
                     "int8_dense_tops": 2 * tc, "note": "int8 dense peak taken as 2 x the measured sustained bf16 GEMM rate"}}
    mm = {}
    for name, (ty, bb, be) in SWEEP_TYPES.items():
        entry = {}
        # decode-shaped and small batches: the 128256 x 4096 weights (279 to 558 MB: more than L2, nothing to flush)
        n, k = 128256, 4096
        w = b.Weight(ty, synth_weights(n, k, seed=50 + ty, ty=ty), k)
        for m in (1, 8, 32):
            x = np.random.default_rng(60 + m).standard_normal((m, k)).astype(np.float32)
            dx, do = b.device_array(x), b.DeviceBuffer(4 * n * m)
            ms = event_time(b, lambda: b.mul_mat_device(w, dx, m, do), 20)
            byts = n * k * bb // be + 4 * m * k + 4 * m * n
            entry[f"m{m}"] = {"shape": f"{n}x{k}", "us": ms * 1e3, "gbs": byts / ms / 1e6, "frac_hbm": byts / ms / 1e6 / hbm,
                              "includes": "activation quantization + mat-mul, device-resident f32 in and out"}
        del w
        # prompt-shaped: 14336 x 4096 (the FFN up shape)
        n, k = 14336, 4096
        w = b.Weight(ty, synth_weights(n, k, seed=51 + ty, ty=ty), k)
        for m in (512, 2048):
            x = np.random.default_rng(61 + m).standard_normal((m, k)).astype(np.float32)
            dx, do = b.device_array(x), b.DeviceBuffer(4 * n * m)
            ms = event_time(b, lambda: b.mul_mat_device(w, dx, m, do), 5 if name in ("Q8_0", "MXFP4") and m == 2048 else 10)
            tops = 2.0 * n * k * m / ms / 1e9
            entry[f"m{m}"] = {"shape": f"{n}x{k}", "us": ms * 1e3, "tops": tops, "frac_int8_peak": tops / (2 * tc), "frac_bf16_peak": tops / tc,
                              "includes": "activation quantization + mat-mul, device-resident f32 in and out",
                              "note": "Q4_K / Q6_K under the fast numerics policy run f16 MMAs (compare with the bf16 peak), the others int8 MMAs"}
            if m == 512 and name in ("Q4_K", "Q6_K", "Q8_0"):
                # the fast numerics mode's distance from the exact mode (= the CPU route's bits), as the reference defines
                # the mat-mul tolerance: |fast - exact| / sum_k |w_k x_k| per output, over the first 256 weight rows
                before = b.get_numerics()
                fast = do.download(np.float32, n * m).reshape(m, n)[:, :256].astype(np.float64)
                b.set_numerics(b.EXACT)
                t0 = event_time(b, lambda: b.mul_mat_device(w, dx, m, do), 3)
                exact = do.download(np.float32, n * m).reshape(m, n)[:, :256].astype(np.float64)
                b.set_numerics(before)
                wd = b.Weight(ty, w.download()[:256], k).dequantize().astype(np.float64)
                denom = np.abs(x).astype(np.float64) @ np.abs(wd).T
                entry[f"m{m}"].update({"exact_numerics_us": t0 * 1e3,
                                       "max_fast_minus_exact_over_sum_abs_wx": float((np.abs(fast - exact) / np.maximum(denom, 1e-30)).max()),
                                       "tolerance": 1e-5})
        del w
        mm[name] = entry
    out["mul_mat"] = mm
    out["kernel_error_after_mul_mat"] = b.kernel_error()

    # MUL_MAT_ID: 128 experts of 768 x 2048 MXFP4, 512 tokens, top-8 ids drawn without replacement per token
    ne, n, k, n_tok, top = 128, 768, 2048, 512, 8
    w = b.ExpertWeights(39, synth_weights(ne * n, k, seed=70, ty=39), n, k)
    rng = np.random.default_rng(71)
    ids = np.stack([rng.permutation(ne)[:top] for _ in range(n_tok)]).astype(np.int32)
    for ne11, label in ((1, "gate_up_form_b_2048x1x512"), (top, "down_form_b_2048x8x512")):
        xb = rng.standard_normal((n_tok, ne11, k)).astype(np.float32)
        db, dids, dst = b.device_array(xb), b.device_array(ids), b.DeviceBuffer(4 * n_tok * top * n)
        ms = event_time(b, lambda: b.check(b.lib.b200_mul_mat_id(39, n, k, ne, ne11, n_tok, top, w.ptr, db.ptr, dids.ptr, dst.ptr, 0, None),
                                           "mul_mat_id"), 10)
        byts = ne * n * k * 17 // 32 + 4 * n_tok * ne11 * k + 4 * n_tok * top * n
        out.setdefault("mul_mat_id", {})[label] = {"us": ms * 1e3, "algorithmic_bytes": byts, "gbs": byts / ms / 1e6, "frac_hbm": byts / ms / 1e6 / hbm,
                                                   "gflop": 2.0 * n_tok * top * n * k / 1e9, "tops": 2.0 * n_tok * top * n * k / ms / 1e9}
    del w

    # FLASH_ATTN_EXT: D 128, 32 query heads on 8 KV heads, causal mask, F16 cache laid out like the KV cache
    H, HK, D = 32, 8, 128
    fa = {}
    for n_kv in (512, 4096, 32768):
        rng = np.random.default_rng(80 + n_kv)
        kk = rng.standard_normal((HK, n_kv, D)).astype(np.float16).view(np.uint16)
        vv = rng.standard_normal((HK, n_kv, D)).astype(np.float16).view(np.uint16)
        kv = b.KvCacheView(kk, vv)
        for T in (1, 512):
            q = rng.standard_normal((H, T, D)).astype(np.float32)
            mask = np.where(np.arange(n_kv)[None, :] <= np.arange(T)[:, None] + (n_kv - T), 0.0, -np.inf).astype(np.float16).view(np.uint16)
            dq, dm, dst = b.device_array(q), b.device_array(mask), b.DeviceBuffer(4 * T * H * D)
            a = b.FlashAttnArgs()
            a.dk, a.dv, a.n_tok, a.n_head, a.n_head_kv, a.n_kv = D, D, T, H, HK, n_kv
            a.q, a.q_nb1, a.q_nb2 = dq.ptr, D * 4, T * D * 4
            a.k, a.k_nb1, a.k_nb2 = kv.k.ptr, kv.k_nb1, kv.k_nb2
            a.v, a.v_nb1, a.v_nb2 = kv.v.ptr, kv.v_nb1, kv.v_nb2
            a.mask, a.mask_nb1, a.sinks = dm.ptr, n_kv * 2, None
            a.scale, a.max_bias, a.logit_softcap, a.dst, a.n_chunks = 1.0 / np.sqrt(D), 0.0, 0.0, dst.ptr, 8
            # T = 1: the flash-decoding kernel against the bit-exact one; T = 512: the tensor-core prompt kernel against the bit-exact tiled one
            modes = ((1, "fast"), (2, "exact"))
            for mode, label in modes:
                a.mode = mode
                import ctypes
                ms = event_time(b, lambda: b.check(b.lib.b200_flash_attn_ext(ctypes.byref(a), None), "flash_attn_ext"), 20 if T == 1 else 3)
                visible = sum(min(n_kv, t + n_kv - T + 1) for t in range(T))
                byts = 2 * n_kv * HK * D * 2 + 2 * n_kv * T + 2 * 4 * T * H * D
                flops = 4.0 * D * H * visible
                e = {"us": ms * 1e3}
                if T == 1:
                    e.update({"algorithmic_bytes": byts, "gbs": byts / ms / 1e6, "frac_hbm": byts / ms / 1e6 / hbm,
                              "note": "16.8 MB (n_kv 4096) and smaller caches sit in the 126 MB L2 across repetitions" if n_kv < 32768 else "134 MB of K/V per call: more than L2"})
                else:
                    e.update({"gflop": flops / 1e9, "tflops": flops / ms / 1e9, "frac_bf16_peak": flops / ms / 1e9 / tc})
                fa[f"n_kv{n_kv}_T{T}_{label}"] = e
    out["flash_attn"] = fa
    out["kernel_error"] = b.kernel_error()
    return out


# ---- arms -------------------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """The CPU routes the reference takes for these workloads, restated in C++ because the Rust reference
    cannot be built here; all host threads.  This arm maps the oracle only: the synthetic inputs are made by
    modules loaded without the CUDA library."""
    if rank != 0:
        return
    orc, orc_glue = load_oracle()
    threads = host_threads(orc)
    reps, xs, outs = cpu_gemv_prepare(orc)
    total = sum(algorithmic_bytes(n, k) for n, k in SHAPES)
    for _ in range(args.warmup):
        cpu_gemv_step(orc, reps, xs, outs, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_gemv_step(orc, reps, xs, outs, threads)
    dt = time.perf_counter() - t0
    gbs = total * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8xint4 dot, f32 accumulate", "data": "synthetic", "config": gemv_config(),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": CPU_KIND,
                         "sample": f"the full step (4 shapes, {total} algorithmic bytes) x {args.steps}"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if not args.no_llama:
        del reps, xs, outs
        try:
            line["llama_8b"] = cpu_llama_baseline(orc, orc_glue, args.cpu_layers)[0]
        except Exception as exc:
            line["llama_8b"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    print(json.dumps(line), flush=True)


def run_b200(args, rank, world, barrier, reduce_max):
    b = load_pkg()
    if b.device_count() == 0:
        raise SystemExit("bench.py: no CUDA device; the CUDA library is the only compute path")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    b.set_device(local)
    note(f"rank {rank}: decode mat-mul")
    g = run_gemv(b, args, rank, world, barrier, reduce_max, local)
    llama, traces = None, {}
    if not args.no_llama:
        note(f"rank {rank}: llama 8b replica")
        llama, traces = run_llama(b, args, rank, world, barrier, reduce_max)
    tp_runs = {}
    if world > 1 and not args.no_llama:
        for shape in ("8b", "70b"):
            note(f"rank {rank}: llama {shape} tensor parallel x{world}")
            try:
                tp_runs[f"llama_{shape}_tp"] = run_llama_tp(b, args, rank, world, local, barrier, reduce_max, shape)
            except Exception as exc:   # a shape that does not split this many ways, or no room: reported, not fatal
                tp_runs[f"llama_{shape}_tp"] = {"tp": world, "unavailable": f"{type(exc).__name__}: {exc}"}
    if world == 1 and not args.no_llama and not args.no_70b:
        note("llama 70b on one GPU")
        try:
            tp_runs["llama_70b_tp"] = run_llama_70b_one_gpu(b, args)
        except Exception as exc:
            tp_runs["llama_70b_tp"] = {"tp": 1, "unavailable": f"{type(exc).__name__}: {exc}"}
    sweep = None
    if world == 1 and not args.no_sweep:
        note("mat-mul sweep, mul_mat_id, flash_attn")
        try:
            sweep = run_sweep(b)
        except Exception as exc:
            sweep = {"unavailable": f"{type(exc).__name__}: {exc}"}
    if rank != 0:
        return
    config = gemv_config()
    # the other halves of the metric, where the driver's record keeps them: tokens/s of the Llama shapes
    measured = {}
    if llama is not None:
        measured["llama_8b_one_gpu_replicas"] = {k: llama[k] for k in ("tg128_tok_s", "pp512_tok_s", "tg128_e2e_tok_s", "pp512_e2e_tok_s")}
        measured["llama_8b_one_gpu_replicas"]["tg128_frac_hbm"] = llama["roofline"]["frac"] if world == 1 else None
    for key, r in tp_runs.items():
        if "unavailable" not in r:
            measured[f"{key}{r['tp']}"] = {k: r[k] for k in ("tg128_tok_s", "pp512_tok_s", "tg128_e2e_tok_s", "tg128_ms_per_token")}
    config["measured"] = measured
    line = {
        "metric": METRIC, "value": g["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": g["warmup"],
        "ms_per_step": g["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8xint4 dot, f32 accumulate", "data": "synthetic", "config": config, "clocks": g["clocks"],
        "e2e": g["e2e"], "gpu_launches": g["gpu_launches"], "roofline": g["roofline"],
    }
    if world > 1:   # the CPU baseline is a single-GPU extra
        if llama is not None:
            line["llama_8b"] = llama
        line.update(tp_runs)
        print(json.dumps(line), flush=True)
        return
    # CPU baselines on the host cores: the same workloads through the CPU routes, bounded samples
    note("cpu baselines")
    try:
        orc, orc_glue = load_oracle()
        line["cpu_baseline"] = cpu_gemv_baseline(orc)
        if llama is not None:
            try:
                llama["cpu_baseline"], cpu_trace, cpu_toks = cpu_llama_baseline(orc, orc_glue, args.cpu_layers)
                # greedy-stream parity: the same 16-token prompt and 4 greedy steps on the GPU (both numerics modes) and on the CPU port
                if args.cpu_layers == args.layers:
                    llama["greedy_parity"] = {name: compare_greedy(tr, tk, cpu_trace, cpu_toks) for name, (tr, tk) in traces.items()}
                    llama["greedy_parity"]["what"] = (f"{PARITY_PROMPT}-token prompt + {PARITY_STEPS} greedy steps of the full model, GPU against the CPU port "
                                                      "on the same synthetic weights: token streams, first divergence, logits while the streams agree")
                    config["measured"]["greedy_parity_exact_identical"] = llama["greedy_parity"].get("exact", {}).get("identical")
                    config["measured"]["greedy_parity_fast_first_divergence"] = llama["greedy_parity"].get("fast", {}).get("first_divergence")
            except Exception as exc:
                llama["cpu_baseline"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    except Exception as exc:  # the baseline is a reported extra, never the measured path
        line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": CPU_KIND, "sample": f"failed: {exc}"}
    # extras last (the tail of the line is what a truncated log keeps): sweep first, the Llama numbers at the very end
    if sweep is not None:
        line["sweep"] = sweep
    line.update(tp_runs)
    if llama is not None:
        line["llama_8b"] = llama
    print(json.dumps(line), flush=True)


# ---- small cases for a profiler --------------------------------------------------------------------------
def case_gemv(args):
    """`--case gemv --only NxK --launches R`: R decode mat-muls of one shape, rotating over enough weight
    copies to stay out of L2; prints the event-timed mean."""
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
    us_graph = b.bench_mul_mat_q8(weights, act, b.ACT_Q8_K, do, 1, args.launches)
    print(json.dumps({"case": f"gemv {args.only}", "copies": copies, "launches": args.launches, "us_per_launch_host_loop": us,
                      "us_per_launch": us_graph, "gbs": algorithmic_bytes(n, k) / us_graph / 1e3}), flush=True)


def case_gemm(args):
    """`--case gemm --only NxK --cols M --launches R`: R prompt-shaped Q4_K mat-muls (M activation rows,
    quantization included, device-resident f32 in and out); prints the event-timed mean and the integer
    multiply-add rate."""
    b = load_pkg()
    b.set_device(0)
    n, k = (int(v) for v in args.only.lower().split("x"))
    m = args.cols
    ty = SWEEP_TYPES[args.wtype][0]
    w = b.Weight(ty, synth_weights(n, k, seed=7, ty=ty), k)
    x = np.random.default_rng(8).standard_normal((m, k)).astype(np.float32)
    dx, do = b.device_array(x), b.DeviceBuffer(4 * n * m)
    for _ in range(3):
        b.mul_mat_device(w, dx, m, do)
    b.synchronize()
    e0, e1 = b.Event(), b.Event()
    e0.record()
    for _ in range(args.launches):
        b.mul_mat_device(w, dx, m, do)
    e1.record()
    e1.synchronize()
    us = e0.elapsed_ms(e1) * 1e3 / args.launches
    out = {"case": f"gemm {args.wtype} {args.only} x {m}", "launches": args.launches, "us_per_call": us, "tops": 2.0 * n * k * m / us / 1e6, "kernel_error": b.kernel_error()}
    if m < 32:
        # a batched decode step's mat-mul: activations quantized beforehand, weight copies rotated to stay out of L2, launches replayed as one graph
        wbytes = n * k * SWEEP_TYPES[args.wtype][1] // SWEEP_TYPES[args.wtype][2]
        copies = max(2, min(32, (300 << 20) // max(wbytes, 1) + 1))
        weights = [w] + [b.Weight(ty, synth_weights(n, k, seed=7, ty=ty), k) for _ in range(copies - 1)]
        act = b.DeviceBuffer(b.lib.b200_act_scratch_nbytes(m, k))
        kind = b.act_kind_for(ty, n, m)
        b.check(b.lib.b200_quantize_activations_device(kind, m, k, dx.ptr, k, act.ptr, None), "quantize")
        out["us_per_launch_graph"] = b.bench_mul_mat_q8(weights, act, kind, do, m, args.launches)
        out["copies"] = copies
    if os.environ.get("B200_GEMM_FAST_PROFILE") in ("1", "2", "3", "4"):
        # SM clocks per launch of one thread per role of the fast kernel's first CTA (csrc/gemm_tcgen05_fast.cu)
        import ctypes
        buf = (ctypes.c_ulonglong * 16)()
        b.check(b.lib.b200_debug_gemm_fast_profile(buf, 16), "gemm_fast_profile")
        names = ["epi_wait_acc", "epi_drain", "mma_wait_stage", "mma_wait_tmem", "mma_issue", "load_wait_free", "load_issue", "prod_wait_free", "prod_fetch_ahead",
                 "prod_convert_store", "prod_fence_arrive", "-", "cta_total"]
        out["clocks_per_launch"] = {nm: int(buf[i]) // (args.launches + 3) for i, nm in enumerate(names)}
    print(json.dumps(out), flush=True)


def case_fa(args):
    """`--case fa --tokens T --n-kv N --fa-mode M --launches R`: R FLASH_ATTN_EXT calls of the benchmark's head geometry (32 query
    heads on 8 KV heads of 128, causal mask, F16 cache) with T query rows over N cached positions; mode 1 = the fast kernels,
    2 = the bit-exact ones; prints the event-timed mean."""
    import ctypes
    b = load_pkg()
    b.set_device(0)
    H, HK, D, T, n_kv = 32, 8, 128, args.tokens, args.n_kv
    rng = np.random.default_rng(80 + n_kv)
    kv = b.KvCacheView(rng.standard_normal((HK, n_kv, D)).astype(np.float16).view(np.uint16), rng.standard_normal((HK, n_kv, D)).astype(np.float16).view(np.uint16))
    q = rng.standard_normal((H, T, D)).astype(np.float32)
    mask = np.where(np.arange(n_kv)[None, :] <= np.arange(T)[:, None] + (n_kv - T), 0.0, -np.inf).astype(np.float16).view(np.uint16)
    dq, dm, dst = b.device_array(q), b.device_array(mask), b.DeviceBuffer(4 * T * H * D)
    a = b.FlashAttnArgs()
    a.dk, a.dv, a.n_tok, a.n_head, a.n_head_kv, a.n_kv = D, D, T, H, HK, n_kv
    a.q, a.q_nb1, a.q_nb2 = dq.ptr, D * 4, T * D * 4
    a.k, a.k_nb1, a.k_nb2 = kv.k.ptr, kv.k_nb1, kv.k_nb2
    a.v, a.v_nb1, a.v_nb2 = kv.v.ptr, kv.v_nb1, kv.v_nb2
    a.mask, a.mask_nb1, a.sinks = dm.ptr, n_kv * 2, None
    a.scale, a.max_bias, a.logit_softcap, a.dst, a.n_chunks, a.mode = 1.0 / np.sqrt(D), 0.0, 0.0, dst.ptr, 8, args.fa_mode
    ms = event_time(b, lambda: b.check(b.lib.b200_flash_attn_ext(ctypes.byref(a), None), "flash_attn_ext"), args.launches)
    visible = sum(min(n_kv, t + n_kv - T + 1) for t in range(T))
    print(json.dumps({"case": f"fa T {T} n_kv {n_kv} mode {args.fa_mode}", "launches": args.launches, "us_per_call": ms * 1e3,
                      "tflops": 4.0 * D * H * visible / ms / 1e9, "cache_gbs": 2 * n_kv * HK * D * 2 / ms / 1e6, "kernel_error": b.kernel_error()}), flush=True)


def case_llama(args):
    """`--case llama_tg|llama_pp|llama_b16 --layers L [--launches R]`: an L-layer model of the 8B shape; one prompt
    batch (llama_pp), R single-token steps after a 16-token prompt (llama_tg) or R steps of 16 sequences after
    512-token prompts (llama_b16), eager launches (no CUDA graph) so that a profiler sees every kernel."""
    os.environ["B200_CUDA_GRAPHS"] = "0"
    b = load_pkg()
    b.set_device(0)
    ll, hp, gpu, _ = build_llama(args.layers, n_ctx=N_SEQ * (PROMPT + GEN) if args.case == "llama_b16" else 1024)
    rng = np.random.default_rng(0)
    if args.case == "llama_b16":
        # 16 sequences with 512-token prompts in the unified cache, then R steps of one token per sequence
        seqs = np.arange(N_SEQ, dtype=np.int32)
        nxt = np.zeros(N_SEQ, dtype=np.int32)
        for s in range(N_SEQ):
            _, am = gpu.decode_seqs(rng.integers(0, hp["n_vocab"], PROMPT).astype(np.int32), np.arange(PROMPT, dtype=np.int32),
                                    np.full(PROMPT, s, dtype=np.int32), [PROMPT - 1], logits=False, argmax=True)
            nxt[s] = am[0]
        t0 = time.perf_counter()
        for i in range(args.launches):
            _, am = gpu.decode_seqs(nxt, np.full(N_SEQ, PROMPT + i, dtype=np.int32), seqs, seqs, logits=False, argmax=True)
            nxt = am.astype(np.int32)
        print(json.dumps({"case": "llama_b16", "layers": args.layers, "steps": args.launches,
                          "ms_per_step": (time.perf_counter() - t0) * 1e3 / args.launches}), flush=True)
        gpu.close()
        return
    if args.case == "llama_pp":
        prompt = rng.integers(0, hp["n_vocab"], PROMPT).astype(np.int32)
        t0 = time.perf_counter()
        gpu.decode(prompt, np.arange(PROMPT), logits=False, argmax=True)
        print(json.dumps({"case": "llama_pp", "layers": args.layers, "ms": (time.perf_counter() - t0) * 1e3,
                          "replay_ms": gpu.replay(1)}), flush=True)
    else:
        np_ = max(1, min(args.prompt, PROMPT))   # --prompt 512: the split-KV attention of the bench's tg128 steps
        tok = gpu.decode(rng.integers(0, hp["n_vocab"], np_).astype(np.int32), np.arange(np_), logits=False, argmax=True)
        t0 = time.perf_counter()
        for i in range(args.launches):
            tok = gpu.decode([tok], [np_ + i], logits=False, argmax=True)
        print(json.dumps({"case": "llama_tg", "layers": args.layers, "steps": args.launches,
                          "ms_per_token": (time.perf_counter() - t0) * 1e3 / args.launches}), flush=True)
    gpu.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, choices=["gemv", "gemm", "fa", "llama_tg", "llama_pp", "llama_b16"], help="one small case for a profiler")
    ap.add_argument("--only", default="4096x4096", help="--case gemv / gemm: the shape NxK")
    ap.add_argument("--cols", type=int, default=512, help="--case gemm: activation rows")
    ap.add_argument("--wtype", default="Q4_K", choices=["Q4_K", "Q6_K"], help="--case gemm: weight type")
    ap.add_argument("--tokens", type=int, default=512, help="--case fa: query rows")
    ap.add_argument("--n-kv", type=int, default=4096, help="--case fa: cached positions")
    ap.add_argument("--fa-mode", type=int, default=1, help="--case fa: 1 fast kernels, 2 bit-exact kernels")
    ap.add_argument("--prompt", type=int, default=16, help="--case llama_tg: prompt tokens before the timed steps")
    ap.add_argument("--launches", type=int, default=64)
    ap.add_argument("--layers", type=int, default=32, help="layers of the 8B-shaped model (32 = the full model)")
    ap.add_argument("--cpu-layers", type=int, default=32, help="layers of the model the CPU baseline times")
    ap.add_argument("--no-llama", action="store_true", help="skip the Llama half of the metric")
    ap.add_argument("--no-70b", action="store_true", help="skip the 70B shape on one GPU (N = 1)")
    ap.add_argument("--no-persistent", action="store_true", help="skip the persistent step-kernel leg of the Llama entry")
    ap.add_argument("--no-sweep", action="store_true", help="skip the mat-mul sweep / MUL_MAT_ID / FLASH_ATTN_EXT entries (N = 1)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    if args.case == "gemv":
        return case_gemv(args)
    if args.case == "fa":
        return case_fa(args)
    if args.case == "gemm":
        return case_gemm(args)
    if args.case:
        return case_llama(args)
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
