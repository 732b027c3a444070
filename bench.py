#!/usr/bin/env python
"""Benchmark of the hot path: the data-parallel PPO actor-critic update of benchmark configuration 5.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--mode tf32x3|tf32|fp32]

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


def run_reference(args):
    """The reference's own CPU implementation of the path, timed on the host cores.  The Rust crate cannot be built in
    this image (no cargo / rustc), so this is the oracle port with all host threads; a step is one optimizer step on
    one 65 536-transition minibatch, the same unit as the GPU arm's step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    warm = min(args.warmup, 1)
    if warm:
        cpu_baseline(8192, 1)
    value, threads, dt, done = cpu_baseline(MB, max(1, min(args.steps, 64)), budget_s=150.0)
    out = {"impl": "reference", "metric": "ppo_update_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": args.gpus, "steps": done,
           "warmup": warm, "ms_per_step": 1e3 * dt / done, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f64", "data": "synthetic", "config": {"workload": WORKLOAD, "sample": "%d transitions per step (one minibatch), %d steps" % (MB, done)},
           "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port",
                            "sample": "%d steps x %d transitions through the oracle (C f64 restatement of the reference, %d threads, %.1f s)" % (done, MB, threads, dt)},
           "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(out), flush=True)


def dominant_kernel(talos, ctx, mode, mode_name, mb, reps=10, profile=False):
    """Average CUDA-event duration (ms) of the layer-2 forward GEMM [mb,256]x[256,256] with the bias+tanh
    epilogue, launched alone on the ctx stream with the L2 flushed between launches."""
    import ctypes
    import torch
    M, N, K = mb, HID, HID
    A = torch.randn(M, K, device="cuda"); B = torch.randn(K, N, device="cuda") * 0.05; C = torch.empty(M, N, device="cuda"); bias = torch.zeros(N, device="cuda")
    epi = talos.Epilogue(bias=talos.ptr(bias), act=talos.ACT_TANH)
    call = lambda: talos.lib.talos_gemm(ctx.handle, 0, 0, M, N, K, talos.ptr(A), K, talos.ptr(B), N, talos.ptr(C), N, mode, ctypes.byref(epi))
    for _ in range(3): call()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    tot = 0.0
    if profile:                                           # `ncu --profile-from-start off` captures from here
        torch.cuda.synchronize(); torch.cuda.profiler.start()
    for _ in range(reps):
        flush.zero_()                                     # evict the operands from L2 between timed launches
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(); call(); e1.record(); torch.cuda.synchronize(); tot += e0.elapsed_time(e1)
    if profile:
        torch.cuda.profiler.stop()
    return tot / reps


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
    if args.kernel_only:                 # profiling aid: only the dominant kernel runs (`ncu --profile-from-start off -k regex:gemm_tc`)
        print(json.dumps({"kernel_only_ms": dominant_kernel(talos, ctx, mode, args.mode, MB, reps=3, profile=True)}))
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

    sampler = ClockSampler(local) if rank == 0 else None
    ms, launches = timed(tr, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    value = args.steps * mb * world / (ms * 1e-3)
    if args.mode != "fp32" and not ctx.tensor_cores_active:
        raise SystemExit("bench.py: the tensor-core path is disabled on this context (its start-up self-check failed; run with "
                         "TALOS_DEBUG=1 to see which case): refusing to report the fp32 fallback as a %s figure" % args.mode)

    # ---- end to end through the host-buffer entry point: H2D of every step's transitions inside the timed region
    e2e_steps = min(args.steps, n_mb)
    pin = lambda a: torch.from_numpy(a[:e2e_steps * mb]).pin_memory()
    p_obs, p_act, p_adv, p_ret = pin(obs_h), pin(act_h), pin(adv_h), pin(ret_h)
    p_old = old[:e2e_steps * mb].cpu().pin_memory()
    tr.update(p_obs, p_act, p_old, p_adv, p_ret, e2e_steps * mb, 1, host=True)               # warm-up at full size: the device staging buffer is allocated here, not in the timed call
    barrier()
    t0 = time.perf_counter()
    tr.update(p_obs, p_act, p_old, p_adv, p_ret, e2e_steps * mb, 1, host=True)             # ends with the epoch's KL read-back
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([dt], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); dt = t.item()
    e2e = {"value": e2e_steps * mb * world / dt, "unit": "samples/s", "h2d_bytes_per_step": mb * (OBS + 4) * 4, "d2h_bytes_per_step": 16,
           "steps": e2e_steps, "api": "talos_ppo_update_host"}

    # ---- the dominant kernel alone: the 65536 x 256 x 256 tensor-core GEMM (three of them per step: layer-2 forward, dH1, dW2)
    pk, pk_kind = peaks()
    roof = None; other_modes = {}
    if rank == 0:
        M, N, K = mb, HID, HID
        k_ms = dominant_kernel(talos, ctx, mode, args.mode, mb)
        alg_bytes = 4.0 * (M * K + K * N + M * N + N); alg_flop = 2.0 * M * N * K
        # dram__bytes_read.sum + dram__bytes_write.sum per launch of this very kernel and shape, from the ncu capture
        # summarised in profiles/gemm_tc_65536x256x256_bias_tanh.md (cold caches; the write count is below the 64 MB of C
        # because the tail of C is still dirty in L2 when the kernel ends).  Not captured for the fp32 CUDA-core kernel.
        traffic = {"tf32": 79.9e6, "tf32x3": 84.4e6}.get(args.mode) if mb == MB else None
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
        # the same step in the other arithmetic modes, for context
        for name in ("tf32", "tf32x3"):
            if name == args.mode or world > 1:
                continue
            t2 = make_trainer(talos.MODES[name]); ms2, _ = timed(t2, min(args.steps, 16), 3); t2.close()
            other_modes[name] = {"value": min(args.steps, 16) * mb / (ms2 * 1e-3), "unit": "samples/s"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, threads, dt, done = cpu_baseline(MB, 16, budget_s=12.0)
        cpu = {"value": v, "unit": "samples/s", "cores": threads, "kind": "port",
               "sample": "%d optimizer steps x %d transitions through the oracle (C f64 restatement of the reference, %d threads, %.1f s)" % (done, MB, threads, dt)}

    if rank == 0:
        out = {"metric": "ppo_update_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
               "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
               "config": {"workload": WORKLOAD, "global_batch": mb * world, "parallelism": "dp%d" % world, "l2": "per-step working set ~330 MB > 126 MB L2",
                          "tensor_cores_active": ctx.tensor_cores_active},
               "tflops": value * FLOP_PER_SAMPLE / 1e12, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
               "other_modes": other_modes}
        print(json.dumps(out), flush=True)
    tr.close()
    if comm is not None:
        comm.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="tf32x3", choices=["tf32x3", "tf32", "fp32"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--kernel-only", action="store_true", help="run only the dominant kernel (profiling aid)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
