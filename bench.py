#!/usr/bin/env python
"""Benchmark of the hot path: the data-parallel PPO actor-critic update of benchmark configuration 5.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl ours|reference] [--mode tf32x3|tf32|fp32]
                    [--sections ppo,gemm,hbm,cpu,host]

A step is one optimizer step: forward, per-sample PPO loss, backward, gradient all-reduce (N > 1)
and Adam on one minibatch of 65 536 transitions PER GPU (obs 64 -> 256 -> 256 tanh trunk, 16-way
policy head + value head, clip 0.2, Adam 3e-4).  Rank r owns a contiguous shard of the 1 048 576
synthetic transitions, resident in HBM; minibatches are consecutive unshuffled chunks.  One JSON line
is printed by rank 0.  `--impl reference` times the CPU restatement of the reference's algorithm
(the oracle) on the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_TOTAL, OBS, HID, ACT, MB, EPOCHS = 1048576, 64, 256, 16, 65536, 4
FLOP_PER_SAMPLE = 484864            # algorithmic: forward 172 544 + backward without dX0 312 320
WORKLOAD = "ppo_update_c5: 1048576 transitions, obs64->256->256 tanh, 16 actions + value, minibatch 65536/GPU, 4 epochs, Adam 3e-4"


def peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """SM clock and throttle-reason samples taken during the timed region: an NVML polling thread (a sample every
    2 ms, read-only queries), or nvidia-smi as a child process when the NVML binding is not importable."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index):
        self.sm, self.mx, self.reasons = [], [], set()
        self.p = None; self.f = None; self.thread = None; self.stop_flag = False
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[gpu_index]) if visible and all(t.strip().isdigit() for t in visible.split(",")) else gpu_index
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.mx.append(float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)))
            bits = {"hw_slowdown": pynvml.nvmlClocksThrottleReasonHwSlowdown, "hw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonSwThermalSlowdown, "sw_power_cap": pynvml.nvmlClocksThrottleReasonSwPowerCap}

            def poll():
                while not self.stop_flag:
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        r = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                        for name, bit in bits.items():
                            if r & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    time.sleep(0.002)
            self.thread = threading.Thread(target=poll, daemon=True); self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "20"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag = True; self.thread.join(timeout=1.0)
        elif self.p is not None:
            time.sleep(0.03)
            self.p.terminate()
            try:
                self.p.wait(timeout=5)
            except Exception:
                self.p.kill()
            self.f.flush(); self.f.seek(0)
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for line in self.f.read().splitlines():
                c = [x.strip() for x in line.split(",")]
                if len(c) < 9:
                    continue
                try:
                    self.sm.append(float(c[1])); self.mx.append(float(c[2]))
                except ValueError:
                    continue
                for name, v in zip(names, c[5:9]):
                    if v.lower().startswith("active"):
                        self.reasons.add(name)
            os.unlink(self.f.name)
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(self.mx) if self.mx else None, "reasons": sorted(self.reasons), "samples": len(sm)}


def synth_shard(talos, rank, world):
    """Seeded synthetic transitions of this rank's shard (host, fp32), generated block by block so that
    every rank can build its own part: block b of 65 536 transitions uses seeds 30..33 + 16*b."""
    import numpy as np
    n_local = N_TOTAL // world
    blocks = range(rank * n_local // MB, (rank + 1) * n_local // MB) if n_local >= MB else [rank]
    rows = MB if n_local >= MB else n_local
    obs = np.empty((len(blocks) * rows, OBS), dtype=np.float32); act = np.empty(len(blocks) * rows, dtype=np.int32)
    adv = np.empty(len(blocks) * rows, dtype=np.float32); ret = np.empty_like(adv)
    for i, b in enumerate(blocks):
        s = slice(i * rows, (i + 1) * rows)
        talos.lib.talos_rng_normal_host(30 + 16 * b, 0.0, 1.0, talos.ptr(obs[s]), rows * OBS)
        talos.lib.talos_rng_bounded_host(31 + 16 * b, ACT, talos.ptr(act[s]), rows)
        talos.lib.talos_rng_normal_host(32 + 16 * b, 0.0, 1.0, talos.ptr(adv[s]), rows)
        talos.lib.talos_rng_normal_host(33 + 16 * b, 0.0, 1.0, talos.ptr(ret[s]), rows)
    return obs, act, adv, ret


def init_params(talos):
    """Xavier-uniform weights (limit sqrt(6/(in+out)), src/nn.rs:22) from seeds 34..37, zero biases."""
    import numpy as np
    p = {}
    for name, seed, fi, fo in (("w1", 34, OBS, HID), ("w2", 35, HID, HID), ("wp", 36, HID, ACT), ("wv", 37, HID, 1)):
        lim = float(np.sqrt(6.0 / (fi + fo))); a = np.empty((fi, fo), dtype=np.float32)
        talos.lib.talos_rng_uniform_host(seed, -lim, lim, talos.ptr(a), a.size); p[name] = a
    p["b1"] = np.zeros(HID, np.float32); p["b2"] = np.zeros(HID, np.float32); p["bp"] = np.zeros(ACT, np.float32); p["bv"] = np.zeros(1, np.float32)
    return p


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


def bench_config(world):
    """The `config` object both arms print (same keys, same workload string)."""
    return {"workload": WORKLOAD, "global_batch": MB * world, "parallelism": "dp%d" % world,
            "l2": "per-step working set ~330 MB > 126 MB L2: no flush needed between steps"}


def cpu_baseline(sample=MB, steps=12, budget_s=25.0, threads=None):
    """The oracle (CPU restatement of the reference's algorithm, f64, row-parallel like Rayon) on a bounded sample of
    the same workload: up to `steps` optimizer steps of `sample` transitions each (one minibatch per step), stopping
    early once `budget_s` seconds of CPU time are spent.  Returns (samples/s, threads, seconds, steps done)."""
    import numpy as np
    import oracle as orc
    from oracle import model as om
    threads = threads or os.cpu_count() or 1
    obs = orc.f32r(orc.rng_normal(30, (sample, OBS))); act = orc.rng_bounded(31, sample, ACT)
    adv = orc.f32r(orc.rng_normal(32, (sample,))); ret = orc.f32r(orc.rng_normal(33, (sample,)))
    params = {}
    for name, seed, fi, fo in (("w1", 34, OBS, HID), ("w2", 35, HID, HID), ("wp", 36, HID, ACT), ("wv", 37, HID, 1)):
        lim = float(np.sqrt(6.0 / (fi + fo))); params[name] = orc.f32r(orc.rng_uniform(seed, (fi, fo), -lim, lim))
    params.update(b1=np.zeros(HID), b2=np.zeros(HID), bp=np.zeros(ACT), bv=np.zeros(1))
    model = om.MlpActorCritic(params)
    old = model.log_prob(obs, act, threads)
    om.ppo_update(model, obs[:1024], act[:1024], old[:1024], adv[:1024], ret[:1024], 1, 1024, threads=threads)   # warm-up
    done = 0; t0 = time.perf_counter()
    while done < steps:
        om.ppo_update(model, obs, act, old, adv, ret, 1, sample, threads=threads)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return sample * done / dt, threads, dt, done


def cpu_baseline_entry(v, threads, dt, done):
    return {"value": v, "unit": "samples/s", "cores": threads, "kind": "port", "cpu": cpu_model(), "host_threads_available": os.cpu_count(),
            "sample": "%d optimizer steps x %d transitions through the oracle (C f64 restatement of the reference, %d threads, %.1f s)" % (done, MB, threads, dt)}


def run_reference(args):
    """The reference's own CPU implementation of the path, timed on the host cores.  The Rust crate cannot be built in
    this image (no cargo / rustc), so this is the oracle port with all host threads; a step is one optimizer step on
    one 65 536-transition minibatch, the same unit as the GPU arm's step.  --warmup W runs W untimed steps first
    (each ~1 s of CPU work), --steps K is bounded to 64 steps / 150 s."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.warmup:
        cpu_baseline(MB, args.warmup, budget_s=30.0)
    value, threads, dt, done = cpu_baseline(MB, max(1, min(args.steps, 64)), budget_s=150.0)
    cpu = cpu_baseline_entry(value, threads, dt, done)
    out = {"impl": "reference", "metric": "ppo_update_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": args.gpus, "steps": done,
           "warmup": args.warmup, "ms_per_step": 1e3 * dt / done, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f64", "data": "synthetic", "config": bench_config(args.gpus), "cpu_baseline": cpu,
           "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(out), flush=True)


class Timer:
    """CUDA-event timing of single launches on torch's current stream (the stream the library context was created
    on), with the L2 flushed by a 256 MB write between launches when the operands would otherwise stay resident."""

    def __init__(self):
        import torch
        self.torch = torch
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def time(self, fn, reps=20, flush=True, warm=3):
        torch = self.torch
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(reps):
            if flush:
                self.flush.zero_()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); torch.cuda.synchronize(); ts.append(e0.elapsed_time(e1))
        ts.sort()
        return {"ms": sum(ts) / len(ts), "ms_median": ts[len(ts) // 2], "ms_min": ts[0], "ms_max": ts[-1], "launches": reps}


def dominant_kernel(talos, ctx, mode, mb, timer, reps=20, profile=False):
    """CUDA-event durations of the layer-2 forward GEMM [mb,256]x[256,256] with the bias+tanh epilogue, launched alone
    on the ctx stream with the L2 flushed between launches."""
    import ctypes
    import torch
    M, N, K = mb, HID, HID
    A = torch.randn(M, K, device="cuda"); B = torch.randn(K, N, device="cuda") * 0.05; C = torch.empty(M, N, device="cuda"); bias = torch.zeros(N, device="cuda")
    epi = talos.Epilogue(bias=talos.ptr(bias), act=talos.ACT_TANH)
    call = lambda: talos.lib.talos_gemm(ctx.handle, 0, 0, M, N, K, talos.ptr(A), K, talos.ptr(B), N, talos.ptr(C), N, mode, ctypes.byref(epi))
    for _ in range(3): call()
    if profile:                                           # `ncu --profile-from-start off` captures from here
        torch.cuda.synchronize(); torch.cuda.profiler.start()
    r = timer.time(call, reps=reps, warm=0)
    if profile:
        torch.cuda.profiler.stop()
    return r


def kernel_only(talos, ctx, mode, timer, which):
    """Small cases for ncu captures (a few hundred MB on the device, inputs larger than L2, three profiled launches):
    gemm      the dominant kernel of the PPO step, 65 536 x 256 x 256 with bias + tanh, in --mode
    gemm4096  the north-star 4096^3 product A.B in --mode (the CTA-pair kernel)
    attention the fused attention forward at benchmark configuration 4's head shape, a quarter of its batch (TF32)"""
    import torch
    L, P = talos.lib, talos.ptr
    if which == "gemm":
        return dominant_kernel(talos, ctx, mode, MB, timer, reps=3, profile=True)["ms"]
    if which == "gemm4096":
        n = 4096
        A = torch.rand(n, n, device="cuda") * 2 - 1; B = torch.rand(n, n, device="cuda") * 2 - 1; C = torch.empty(n, n, device="cuda")
        call = lambda: L.talos_gemm(ctx.handle, 0, 0, n, n, n, P(A), n, P(B), n, P(C), n, mode, None)
    else:
        BH, S, dqk, dv = 1024, 128, 96, 64
        q = torch.randn(BH, S, dqk, device="cuda"); k = torch.randn_like(q); v = torch.randn(BH, S, dv, device="cuda"); o = torch.empty_like(v)
        call = lambda: L.talos_attention_fwd(ctx.handle, P(q), P(k), P(v), P(o), None, BH, S, dqk, dv, 0.1, 0, talos.MODE_TF32)
    for _ in range(3): call()
    torch.cuda.synchronize(); torch.cuda.profiler.start()
    r = timer.time(call, reps=3, warm=0)
    torch.cuda.profiler.stop()
    return r["ms"]


def gemm_section(talos, ctx, timer, pk, pk_kind, local, reps=20):
    """The GEMM half of the metric: 4096^3 in both tensor-core modes and the three forms (A.B, A.B^T, A^T.B), cuBLAS
    TF32 on the same box as a yard-stick, and benchmark configuration 1 (512^3) with the oracle's CPU time beside it.
    Each figure: >= 20 single launches, L2 flushed between them, clocks sampled while they run."""
    import torch
    L, P = talos.lib, talos.ptr
    tf32_peak = pk["bf16_tflops"] / 2.0
    out = {"peak_tf32_tflops": tf32_peak, "peak_tf32x3_tflops": tf32_peak / 3.0,
           "peak_source": pk_kind + " bf16 burst / 2 (TF32 rate); / 3 for the three-product fp32-faithful mode", "cases": []}
    for size in (4096, 512):
        A = torch.rand(size, size, device="cuda") * 2 - 1; B = torch.rand(size, size, device="cuda") * 2 - 1; C = torch.empty(size, size, device="cuda")
        flop = 2.0 * size ** 3
        sampler = ClockSampler(local)
        for mode_name, mode in (("tf32", 2), ("tf32x3", 1)):
            for form, (oa, ob) in (("A.B", (0, 0)), ("A.B^T", (0, 1)), ("A^T.B", (1, 0))):
                r = timer.time(lambda: L.talos_gemm(ctx.handle, oa, ob, size, size, size, P(A), size, P(B), size, P(C), size, mode, None), reps=reps)
                peak = tf32_peak if mode == 2 else tf32_peak / 3.0
                tf = flop / (r["ms"] * 1e-3) / 1e12
                out["cases"].append(dict(shape=[size] * 3, form=form, mode=mode_name, tflops=tf, frac=tf / peak, **r))
        torch.backends.cuda.matmul.allow_tf32 = True
        r = timer.time(lambda: torch.matmul(A, B, out=C), reps=reps)
        out["cases"].append(dict(shape=[size] * 3, form="A.B", mode="cublas_tf32_yardstick", tflops=flop / (r["ms"] * 1e-3) / 1e12,
                                 frac=flop / (r["ms"] * 1e-3) / 1e12 / tf32_peak, **r))
        out["clocks_%d" % size] = sampler.stop()
    # benchmark configuration 1 on the host: the oracle's restatement of Tensor::matmul and its two backward products
    import numpy as np
    import oracle as orc
    a = orc.rng_uniform(42, (512, 512), -1.0, 1.0); b = orc.rng_uniform(123, (512, 512), -1.0, 1.0)
    threads_all = os.cpu_count() or 1
    cpu = {}
    for label, th in (("all", threads_all), ("minus_one", max(1, threads_all - 1))):
        orc.matmul(a, b, threads=th)
        t0 = time.perf_counter(); n = 0
        while n < 5 or time.perf_counter() - t0 < 0.5:
            orc.matmul(a, b, threads=th); n += 1
        fwd = (time.perf_counter() - t0) / n
        t0 = time.perf_counter(); n = 0
        while n < 3 or time.perf_counter() - t0 < 0.5:
            orc.matmul_bwd(a, b, a, threads=th); n += 1
        bwd = (time.perf_counter() - t0) / n
        cpu[label] = {"threads": th, "A.B_ms": fwd * 1e3, "A.B_gflops": 2.0 * 512 ** 3 / fwd / 1e9, "both_backward_products_ms": bwd * 1e3,
                      "backward_gflops": 4.0 * 512 ** 3 / bwd / 1e9}
    out["config1_cpu_oracle"] = dict(cpu=cpu_model(), kind="port", **cpu)
    return out


def hbm_section(talos, ctx, timer, pk, pk_kind, local, reps=20):
    """RMSNorm / softmax / RoPE at the transformer-block shapes of the benchmark configurations (inputs larger than
    L2, so no flush): achieved HBM GB/s = algorithmic bytes / CUDA-event time, as a fraction of the measured copy rate."""
    import torch
    L, P = talos.lib, talos.ptr
    hbm = pk["hbm_gbs"]
    out = {"peak_gbs": hbm, "peak_source": pk_kind + " copy bandwidth", "nominal_gbs": 8000.0, "cases": []}
    sampler = ClockSampler(local)

    def add(name, shape, gbytes, fn):
        r = timer.time(fn, reps=reps, flush=False)
        gbs = gbytes / (r["ms"] * 1e-3)
        out["cases"].append(dict(kernel=name, shape=shape, gbs=gbs, frac=gbs / hbm, frac_of_nominal=gbs / 8000.0, **r))

    rows, dim = 65536 * 4, 256            # config 3: 65 536 token rows of 256 (x4 so the input exceeds L2)
    x = torch.randn(rows, dim, device="cuda"); g = torch.ones(dim, device="cuda"); y = torch.empty_like(x); inv = torch.empty(rows, device="cuda")
    add("rmsnorm_fwd", [rows, dim], (2.0 * rows * dim + rows + dim) * 4 / 1e9, lambda: L.talos_rmsnorm_fwd(ctx.handle, P(x), P(g), 1e-6, rows, dim, P(y), P(inv)))
    dy = torch.randn_like(x); dx = torch.empty_like(x); dg = torch.empty(dim, device="cuda")
    add("rmsnorm_bwd", [rows, dim], (3.0 * rows * dim + rows) * 4 / 1e9, lambda: L.talos_rmsnorm_bwd(ctx.handle, P(dy), P(x), P(g), P(inv), rows, dim, P(dx), P(dg), 0))
    del x, y, dy, dx
    for srows, slen in ((524288 * 2, 64), (524288, 128)):   # config 3: 8192 x 64 rows of 64 (x2); config 4: 4096 x 128 rows of 128
        s = torch.randn(srows, slen, device="cuda"); o = torch.empty_like(s)
        add("softmax_fwd", [srows, slen], 2.0 * srows * slen * 4 / 1e9, lambda: L.talos_softmax_fwd(ctx.handle, P(s), P(o), srows, slen, 0.125, 0))
        gs = torch.randn_like(s); ds = torch.empty_like(s)
        add("softmax_bwd", [srows, slen], 3.0 * srows * slen * 4 / 1e9, lambda: L.talos_softmax_bwd(ctx.handle, P(o), P(gs), P(ds), srows, slen, 0.125, 0))
    Bq, S, H, dr = 2048, 128, 8, 32       # config 4 rotary part (batch x4)
    c = torch.empty(S * dr // 2, device="cuda"); sn = torch.empty_like(c); L.talos_rope_table(ctx.handle, dr, S, 10000.0, P(c), P(sn))
    xr = torch.randn(Bq, S, H, dr, device="cuda"); yr = torch.empty_like(xr)
    add("rope", [Bq, S, H, dr], 2.0 * xr.numel() * 4 / 1e9, lambda: L.talos_rope(ctx.handle, P(xr), P(yr), P(c), P(sn), c.numel(), Bq, S, H, dr, 0, 0, 0))
    del xr, yr
    n = 1 << 25                           # rollout buffer: GAE scan + advantage normalisation (src/ppo.rs:650-675)
    rw = torch.randn(n, device="cuda"); vl = torch.randn(n, device="cuda"); tm = (torch.rand(n, device="cuda") < 0.02).to(torch.int32)
    adv = torch.empty(n, device="cuda"); ret = torch.empty(n, device="cuda")
    add("gae", [n], (2 * 12.0 + 8.0) * n / 1e9, lambda: L.talos_gae(ctx.handle, P(rw), P(vl), P(tm), n, 0.99, 0.95, 0.0, 1.0, P(adv), P(ret)))   # two passes read r, V, terminal; the second writes A and R
    add("normalize_slice", [n], 16.0 * n / 1e9, lambda: L.talos_normalize_slice(ctx.handle, P(adv), n, P(ret), None))                          # three reads, one write
    del rw, vl, tm, adv, ret
    BH, S, dqk, dv = 4096, 128, 96, 64    # config 4 attention core
    q = torch.randn(BH, S, dqk, device="cuda"); k = torch.randn_like(q); v = torch.randn(BH, S, dv, device="cuda"); o = torch.empty_like(v)
    att = []
    for mname in ("tf32", "tf32x3"):
        r = timer.time(lambda: L.talos_attention_fwd(ctx.handle, P(q), P(k), P(v), P(o), None, BH, S, dqk, dv, 0.1, 0, talos.MODES[mname]), reps=reps, flush=False)
        att.append(dict(kernel="attention_fwd", mode=mname, shape=[BH, S, dqk, dv], tflops=2.0 * BH * S * S * (dqk + dv) / (r["ms"] * 1e-3) / 1e12, **r))
    out["attention_core_config4"] = att
    out["clocks"] = sampler.stop()
    return out


def host_route_section(mode):
    """The two training routes that go through the Tensor / autograd mirror of the crate's API rather than the fused PPO
    trainer -- a dueling double-DQN train step at batch 64 (src/dqn.rs:482-584) and a LuckTransformer(8, 64) forward +
    backward on [64, 16, 8] -- timed by the C++ host program (host clock between two stream synchronisations), with the
    oracle's time for the same arithmetic on the host cores beside it.  Every tensor of those routes comes from the
    context's caching allocator; the counters show whether the timed loop reached the CUDA driver."""
    exe = os.path.join(ROOT, "tests", "cpp", "bin", "host_driver")
    if not os.path.exists(exe):
        return {"unavailable": "tests/cpp/bin/host_driver is not built"}
    r = subprocess.run([exe, "time", str(mode), os.devnull, "7", "200", "64"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    if r.returncode != 0:
        return {"unavailable": "host_driver failed: " + r.stdout[-300:]}
    out = json.loads(r.stdout.strip().splitlines()[-1])
    import numpy as np
    import oracle as orc
    from oracle import model as om
    th = os.cpu_count() or 1
    lt = om.LuckTransformer(8, 64, 7); x = orc.f32r(orc.lcg_rand((64, 16, 8), -0.5, 0.5, 10)); g = np.full((64, 16, 64), 1.0 / (64 * 16 * 64))
    lt.forward_backward(x, g)
    t0 = time.perf_counter(); n = 0
    while n < 3 or time.perf_counter() - t0 < 1.0:
        lt.forward_backward(x, g); n += 1
    out["cpu_oracle_luck_fwd_bwd_ms"] = (time.perf_counter() - t0) / n * 1e3
    # the DQN step's arithmetic with the oracle's pieces: three forwards, targets, loss, backward, clipped Adam, soft update
    W = [om.linear_init_lcg(8, 64, True, 7), om.linear_init_lcg(64, 64, True, 8), om.linear_init_lcg(64, 1, True, 9), om.linear_init_lcg(64, 5, True, 10)]
    P = [np.array(t) for w in W for t in w]; T = [p.copy() for p in P]; m = [np.zeros_like(p) for p in P]; v = [np.zeros_like(p) for p in P]
    s0 = orc.lcg_rand((64, 8), -1.0, 1.0, 8); s1 = orc.lcg_rand((64, 8), -1.0, 1.0, 9)
    act = np.arange(64) % 5; rew = 0.1 * (np.arange(64) % 7) - 0.3; done = (np.arange(64) % 9 == 0).astype(np.float64)

    def fwd(Q, s):
        z1 = om.linear_fwd(s, Q[0], Q[1]); h1 = np.maximum(z1, 0); z2 = om.linear_fwd(h1, Q[2], Q[3]); h2 = np.maximum(z2, 0)
        return (z1, h1, z2, h2), om.dueling_combine(om.linear_fwd(h2, Q[4], Q[5]), om.linear_fwd(h2, Q[6], Q[7]))

    def dqn_step(t):
        (z1, h1, z2, h2), q = fwd(P, s0); _, qe = fwd(P, s1); _, qt = fwd(T, s1)
        _, dq = om.dqn_loss_fwd_bwd(q, act, om.dqn_target(qe, qt, rew, done))
        dv, da = om.dueling_combine_bwd(dq)
        dh_v, gWv, gbv = om.linear_bwd(h2, P[4], dv, True); dh_a, gWa, gba = om.linear_bwd(h2, P[6], da, True)
        d2 = (dh_v + dh_a) * (z2 > 0); dh1, gW2, gb2 = om.linear_bwd(h1, P[2], d2, True)
        d1 = dh1 * (z1 > 0); _, gW1, gb1 = om.linear_bwd(s0, P[0], d1, True, need_dx=False)
        om.adam_step(P, [gW1, gb1, gW2, gb2, gWv, gbv, gWa, gba], m, v, t, 1e-3, clip_norm=1.0)
        for i in range(len(T)):
            T[i] = om.soft_update(T[i], P[i], 0.005)
    dqn_step(1)
    t0 = time.perf_counter(); n = 0
    while n < 5 or time.perf_counter() - t0 < 1.0:
        n += 1; dqn_step(n + 1)
    out["cpu_oracle_dqn_train_step_ms"] = (time.perf_counter() - t0) / n * 1e3
    out["cpu_threads"] = th; out["cpu"] = cpu_model(); out["mode"] = mode
    return out


def params_digest(tr):
    import hashlib
    import numpy as np
    p = tr.get_params()
    h = hashlib.sha256()
    for k in tr.NAMES:
        h.update(np.ascontiguousarray(p[k]).tobytes())
    return h.hexdigest()


def data_parallel_checks(talos, ctx, comm, dist, rank, world, mode, params, steps=2):
    """Correctness evidence for N > 1, outside the timed region: (1) after `steps` optimizer steps from the same
    initial weights every rank must hold bit-identical parameters; (2) rank 0 repeats the same steps as ONE rank on
    the concatenated global minibatches (world x 65 536 transitions per step) -- gradients are sums divided by the
    global count, so the two runs must agree to fp32 reduction-order noise."""
    import numpy as np
    import torch
    n_local = N_TOTAL // world
    first = rank * n_local // MB

    def block(b):
        obs = np.empty((MB, OBS), np.float32); act = np.empty(MB, np.int32); adv = np.empty(MB, np.float32); ret = np.empty(MB, np.float32)
        talos.lib.talos_rng_normal_host(30 + 16 * b, 0.0, 1.0, talos.ptr(obs), MB * OBS)
        talos.lib.talos_rng_bounded_host(31 + 16 * b, ACT, talos.ptr(act), MB)
        talos.lib.talos_rng_normal_host(32 + 16 * b, 0.0, 1.0, talos.ptr(adv), MB)
        talos.lib.talos_rng_normal_host(33 + 16 * b, 0.0, 1.0, talos.ptr(ret), MB)
        return [torch.from_numpy(a).cuda() for a in (obs, act, adv, ret)]

    def run(trainer, batches, n):
        for obs, act, adv, ret in batches:
            old = torch.empty(n, device="cuda"); trainer.log_prob(obs, act, n, old)
            trainer.step(obs, act, old, adv, ret, n)
        return trainer.get_params()

    tr = talos.PPOTrainer(ctx, talos.PpoConfig(OBS, HID, ACT, MB, mode), comm); tr.set_params(params)
    got = run(tr, [block(first + s) for s in range(steps)], MB)
    digest = params_digest(tr); tr.close()
    digests = [None] * world
    dist.all_gather_object(digests, digest)
    out = {"ranks_bit_identical": len(set(digests)) == 1, "checked_steps": steps}
    if rank == 0:
        n_local_blocks = n_local // MB
        one = talos.PPOTrainer(ctx, talos.PpoConfig(OBS, HID, ACT, MB * world, mode), None); one.set_params(params)
        batches = []
        for s in range(steps):
            parts = [block(r * n_local_blocks + s) for r in range(world)]
            batches.append([torch.cat([p[i] for p in parts]) for i in range(4)])
        ref = run(one, batches, MB * world); one.close()
        num = den = unum = uden = 0.0
        for k in tr.NAMES:
            a = got[k].astype(np.float64); b = ref[k].astype(np.float64); p0 = np.asarray(params[k], np.float64).reshape(a.shape)
            num += float(((a - b) ** 2).sum()); den += float((b ** 2).sum())
            unum += float((((a - p0) - (b - p0)) ** 2).sum()); uden += float(((b - p0) ** 2).sum())
        out["dp_equiv_rel_err"] = (num / den) ** 0.5
        out["dp_equiv_update_rel_err"] = (unum / uden) ** 0.5 if uden > 0 else 0.0
    dist.barrier()
    return out


def traffic_from_profiles(mode_name):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, as written by the profiling step
    (one ncu capture of `bench.py --kernel-only`) into profiles/dominant_kernel_traffic.json; null when absent."""
    try:
        t = json.load(open(os.path.join(ROOT, "profiles", "dominant_kernel_traffic.json")))
        return float(t[mode_name]["dram_bytes_per_launch"])
    except Exception:
        return None


def run_ours(args):
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    talos = load_package()
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device: the library has no CPU path"
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = talos.torch_context(local)
    comm = None
    if world > 1:
        uid = [talos.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        comm = talos.Comm(ctx, uid[0], world, rank)

    mode = talos.MODES[args.mode]
    timer = Timer()
    if args.kernel_only:                 # profiling aid: one kernel, three launches between cudaProfilerStart/Stop (`ncu --profile-from-start off`)
        print(json.dumps({"kernel": args.kernel_only, "kernel_only_ms": kernel_only(talos, ctx, mode, timer, args.kernel_only)}))
        return
    sections = set(args.sections.split(",")) if args.sections else {"ppo", "gemm", "hbm", "cpu", "host"}
    pk, pk_kind = peaks()
    if "ppo" not in sections:            # kernel figures only (what the committed profiles' commands run)
        out = {}
        if "gemm" in sections: out["gemm"] = gemm_section(talos, ctx, timer, pk, pk_kind, local)
        if "hbm" in sections: out["hbm_kernels"] = hbm_section(talos, ctx, timer, pk, pk_kind, local)
        if "host" in sections: out["host_autograd_routes"] = host_route_section(mode)
        print(json.dumps(out), flush=True)
        return
    obs_h, act_h, adv_h, ret_h = synth_shard(talos, rank, world)
    n_local = obs_h.shape[0]; mb = min(MB, n_local)
    params = init_params(talos)

    def make_trainer(m):
        tr = talos.PPOTrainer(ctx, talos.PpoConfig(OBS, HID, ACT, mb, m), comm); tr.set_params(params); return tr
    tr = make_trainer(mode)
    dev = lambda a: torch.from_numpy(a).cuda(local)
    obs, act, adv, ret = dev(obs_h), dev(act_h), dev(adv_h), dev(ret_h)
    old = torch.empty(n_local, device="cuda")
    tr.log_prob(obs, act, n_local, old)            # the stored rollout log-probabilities under the initial weights
    ctx.synchronize()
    n_mb = n_local // mb

    def one_step(trainer, i):
        s = (i % n_mb) * mb
        trainer.step(obs[s:], act[s:], old[s:], adv[s:], ret[s:], mb)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(trainer, steps, warmup):
        for i in range(warmup):
            one_step(trainer, i)
        barrier()
        l0 = ctx.launches
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            one_step(trainer, warmup + i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = t.item()
        return ms, ctx.launches - l0

    # The timed region (exactly --steps steps between two barriers) is repeated; `value` is the MEDIAN region.
    sampler = ClockSampler(local) if rank == 0 else None
    regions = []
    launches = 0
    for r in range(max(1, args.repeats)):
        ms_r, launches = timed(tr, args.steps, args.warmup if r == 0 else 1)
        regions.append(ms_r)
    clocks = sampler.stop() if sampler else None
    srt = sorted(regions); ms = srt[len(srt) // 2]
    value = args.steps * mb * world / (ms * 1e-3)
    repeats = {"timed_regions": len(regions), "steps_per_region": args.steps, "ms_per_step_median": ms / args.steps,
               "ms_per_step_min": srt[0] / args.steps, "ms_per_step_max": srt[-1] / args.steps, "value_is": "median region"}
    # Per-launch device times of the step, warm (the way the step runs them, not the cold serialised times a profiler
    # shows): five more steps with an event behind every launch; median per position.  Outside the timed regions.
    step_launches = None
    if rank == 0 and world == 1:
        per_step = launches // max(1, args.steps)
        ctx.timeline_begin()
        for i in range(5):
            one_step(tr, i)
        marks = ctx.timeline_end()
        if per_step > 0 and len(marks) == 5 * per_step:
            step_launches = []
            for j in range(per_step):
                us = sorted(marks[k * per_step + j][1] for k in range(1, 5))      # (the first step's first mark includes the begin call)
                step_launches.append([marks[per_step + j][0], round((us[1] + us[2]) / 2, 2)])
    if args.mode != "fp32" and not ctx.tensor_cores_active:
        raise SystemExit("bench.py: the tensor-core path is disabled on this context (its start-up self-check failed; run with "
                         "TALOS_DEBUG=1 to see which case): refusing to report the fp32 fallback as a %s figure" % args.mode)

    # ---- end to end: ONE talos_ppo_update_host call over this rank's whole shard, 4 epochs, from pinned host buffers
    # (the H2D copy of every transition and the per-epoch KL read-back are inside the timed call)
    pin = lambda a: torch.from_numpy(a).pin_memory()
    p_obs, p_act, p_adv, p_ret = pin(obs_h), pin(act_h), pin(adv_h), pin(ret_h)
    p_old = old.cpu().pin_memory()
    e2e_steps = EPOCHS * n_mb
    tr.update(p_obs, p_act, p_old, p_adv, p_ret, n_local, 1, host=True)    # warm-up at full size: the device staging buffer is allocated here, not in the timed call
    e2e_runs = []
    for _ in range(3):
        barrier()
        t0 = time.perf_counter()
        tr.update(p_obs, p_act, p_old, p_adv, p_ret, n_local, EPOCHS, host=True)             # returns after the last epoch's KL read-back
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if dist is not None:
            t = torch.tensor([dt], device="cuda", dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); dt = t.item()
        e2e_runs.append(dt)
    dt = sorted(e2e_runs)[1]
    # What the call cannot hide: the first minibatch has to arrive before the first step can start.  Its copy is timed
    # alone (pinned host -> device, all ranks at once, as in the call) so that the line carries the call's floor.
    d_first = torch.empty((mb, OBS), device="cuda")
    h2d_ms = []
    for _ in range(5):
        barrier()
        c0 = torch.cuda.Event(enable_timing=True); c1 = torch.cuda.Event(enable_timing=True)
        c0.record(); d_first.copy_(p_obs[:mb], non_blocking=True); c1.record(); torch.cuda.synchronize()
        h2d_ms.append(c0.elapsed_time(c1))
    first_copy_s = sorted(h2d_ms)[2] * 1e-3 * (OBS + 4) / OBS          # + the four per-transition scalars
    if dist is not None:
        t = torch.tensor([first_copy_s], device="cuda", dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); first_copy_s = t.item()
    del d_first
    e2e = {"value": e2e_steps * mb * world / dt, "unit": "samples/s", "h2d_bytes_per_step": n_local * (OBS + 4) * 4 // e2e_steps, "d2h_bytes_per_step": 16,
           "steps": e2e_steps, "epochs": EPOCHS, "shard_transitions": n_local, "api": "talos_ppo_update_host (one call: whole shard, 4 epochs)",
           "seconds_median_of_3": dt, "seconds_all": e2e_runs,
           "first_minibatch_copy_seconds": first_copy_s, "first_minibatch_copy_gbs": mb * (OBS + 4) * 4 / first_copy_s / 1e9,
           "floor_seconds": first_copy_s + e2e_steps * (ms / args.steps) * 1e-3,
           "floor_is": "copy of the first minibatch (nothing to overlap it with) + steps x the resident ms_per_step"}

    dp = None
    if world > 1:
        dp = data_parallel_checks(talos, ctx, comm, dist, rank, world, mode, params)

    # ---- the dominant kernel alone: the 65536 x 256 x 256 tensor-core GEMM (three of them per step: layer-2 forward, dH1, dW2)
    roof = None; other_modes = {}; gemm = None; hbm = None; host_route = None
    if rank == 0:
        M, N, K = mb, HID, HID
        ksamp = ClockSampler(local)
        kr = dominant_kernel(talos, ctx, mode, mb, timer)
        kclk = ksamp.stop()
        k_ms = kr["ms"]
        alg_bytes = 4.0 * (M * K + K * N + M * N + N); alg_flop = 2.0 * M * N * K
        traffic = traffic_from_profiles(args.mode) if mb == MB else None
        if args.mode == "tf32":      # 64 flop/byte is under the TF32 ridge: HBM-bound
            ach = alg_bytes / (k_ms * 1e-3) / 1e9
            roof = {"kernel": "gemm_tc_kernel (65536x256x256, bias+tanh epilogue)", "bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": ach / pk["hbm_gbs"], "traffic": traffic, "peak_source": pk_kind + " copy bandwidth", "ms_per_launch": k_ms}
        else:
            div = 3.0 if args.mode == "tf32x3" else None
            peak = pk["bf16_tflops"] / 2.0 / 3.0 if div else 75.0
            ach = alg_flop / (k_ms * 1e-3) / 1e12
            roof = {"kernel": "gemm_tc_kernel 3xTF32 (65536x256x256, bias+tanh epilogue)" if div else "gemm_fp32_kernel", "bound": "tensor", "achieved": ach,
                    "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": traffic, "ms_per_launch": k_ms,
                    "peak_source": (pk_kind + " bf16 burst / 2 (TF32 rate) / 3 (three TF32 products per term)") if div else "nominal fp32 FFMA"}
        roof.update(launches_timed=kr["launches"], ms_min=kr["ms_min"], ms_max=kr["ms_max"], clocks=kclk,
                    step_frac_of_roof=(value / world) * FLOP_PER_SAMPLE / 1e12 / (pk["bf16_tflops"] / 2.0 / (3.0 if args.mode == "tf32x3" else 1.0)) if args.mode != "fp32" else None)
        # the same step in the other arithmetic modes, for context
        for name in ("tf32", "tf32x3"):
            if name == args.mode or world > 1:
                continue
            t2 = make_trainer(talos.MODES[name]); ms2, _ = timed(t2, min(args.steps, 16), 3); t2.close()
            other_modes[name] = {"value": min(args.steps, 16) * mb / (ms2 * 1e-3), "unit": "samples/s"}
        if world == 1 and "gemm" in sections:
            gemm = gemm_section(talos, ctx, timer, pk, pk_kind, local)
        if world == 1 and "hbm" in sections:
            hbm = hbm_section(talos, ctx, timer, pk, pk_kind, local)
        if world == 1 and "host" in sections:
            host_route = host_route_section(mode)

    cpu = None
    if rank == 0 and world == 1 and "cpu" in sections and not args.no_cpu:
        threads_all = os.cpu_count() or 1
        cpu = cpu_baseline_entry(*cpu_baseline(MB, 16, budget_s=12.0, threads=threads_all))
        if threads_all > 1:      # the reference reserves one core for the main thread by default (src/worker.rs:60-67)
            cpu["minus_one_core"] = cpu_baseline_entry(*cpu_baseline(MB, 16, budget_s=10.0, threads=threads_all - 1))

    if rank == 0:
        out = {"metric": "ppo_update_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
               "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
               "config": bench_config(world), "tensor_cores_active": ctx.tensor_cores_active,
               "tflops": value * FLOP_PER_SAMPLE / 1e12, "repeats": repeats, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
               "cpu_baseline": cpu, "other_modes": other_modes}
        if step_launches is not None:
            out["step_launches_warm_us"] = step_launches
        if dp is not None:
            out.update(dp)
        if gemm is not None:
            out["gemm"] = gemm
        if hbm is not None:
            out["hbm_kernels"] = hbm
        if host_route is not None:
            out["host_autograd_routes"] = host_route
        print(json.dumps(out), flush=True)
    tr.close()
    if comm is not None:
        comm.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10, help="how many times the timed region of --steps steps is run (value = the median region)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="tf32x3", choices=["tf32x3", "tf32", "fp32"])
    ap.add_argument("--sections", default="", help="comma list of ppo,gemm,hbm,cpu,host (default: all; without ppo only the kernel figures are printed)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--kernel-only", nargs="?", const="gemm", default=None, choices=["gemm", "gemm4096", "attention"],
                    help="profiling aid: run only this kernel, three launches inside cudaProfilerStart/Stop")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
