#!/usr/bin/env python
"""Per-kernel throughput of the dense path against the B200 roofline (one JSON line per kernel).

    python talos-xii_b200/kernel_bench.py [--quick]

GEMM 512^3 and 4096^3 in the three forms (A.B, A.B^T, A^T.B) and three arithmetic modes -> TFLOP/s;
RMSNorm, softmax, RoPE at the transformer-block shapes of the benchmark configs -> achieved HBM GB/s
(algorithmic bytes / CUDA-event time) as a fraction of the measured copy bandwidth.  Inputs of the
memory-bound kernels are larger than L2 (126 MB); GEMM operands are flushed from L2 between launches."""
import argparse
import ctypes
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser(); ap.add_argument("--quick", action="store_true"); args = ap.parse_args()
    import torch
    from __graft_entry__ import load_package
    talos = load_package()
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))); src = "measured"
    except Exception:
        pk = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}; src = "fallback"
    ctx = talos.torch_context(0)
    L, P = talos.lib, talos.ptr
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn, reps=10, do_flush=True):
        for _ in range(3): fn()
        tot = 0.0
        for _ in range(reps):
            if do_flush: flush.zero_()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); torch.cuda.synchronize(); tot += e0.elapsed_time(e1)
        return tot / reps

    def emit(**kw):
        print(json.dumps(kw), flush=True)

    tf32_peak = pk["bf16_tflops"] / 2.0
    for size in ((512,) if args.quick else (512, 4096)):
        A = torch.rand(size, size, device="cuda") * 2 - 1; B = torch.rand(size, size, device="cuda") * 2 - 1; C = torch.empty(size, size, device="cuda")
        for mode_name, mode in (("tf32", 2), ("tf32x3", 1), ("fp32", 0)):
            for form, (oa, ob) in (("A.B", (0, 0)), ("A.B^T", (0, 1)), ("A^T.B", (1, 0))):
                ms = timeit(lambda: L.talos_gemm(ctx.handle, oa, ob, size, size, size, P(A), size, P(B), size, P(C), size, mode, None), reps=5 if mode == 0 else 10)
                tf = 2.0 * size ** 3 / (ms * 1e-3) / 1e12
                peak = tf32_peak if mode == 2 else tf32_peak / 3 if mode == 1 else 75.0
                emit(kernel="gemm", shape=[size] * 3, form=form, mode=mode_name, ms=ms, tflops=tf, frac_of_peak=tf / peak,
                     peak_tflops=peak, peak_source=(src + " bf16 burst / 2" + (" / 3" if mode == 1 else "")) if mode else "nominal fp32 FFMA")
        torch.backends.cuda.matmul.allow_tf32 = True
        ms = timeit(lambda: torch.matmul(A, B, out=C))
        emit(kernel="cublas_tf32_yardstick", shape=[size] * 3, ms=ms, tflops=2.0 * size ** 3 / (ms * 1e-3) / 1e12)

    hbm = pk["hbm_gbs"]
    rows, dim = 65536 * (1 if args.quick else 4), 256            # config 3: 65 536 token rows of 256 (x4 so the input exceeds L2)
    x = torch.randn(rows, dim, device="cuda"); g = torch.ones(dim, device="cuda"); y = torch.empty_like(x); inv = torch.empty(rows, device="cuda")
    ms = timeit(lambda: L.talos_rmsnorm_fwd(ctx.handle, P(x), P(g), 1e-6, rows, dim, P(y), P(inv)), do_flush=False)
    gb = (2.0 * rows * dim + rows + dim) * 4 / 1e9
    emit(kernel="rmsnorm_fwd", shape=[rows, dim], ms=ms, gbps=gb / (ms * 1e-3), frac_of_hbm=gb / (ms * 1e-3) / hbm, hbm_peak_gbps=hbm, peak_source=src)
    dy = torch.randn_like(x); dx = torch.empty_like(x); dg = torch.empty(dim, device="cuda")
    ms = timeit(lambda: L.talos_rmsnorm_bwd(ctx.handle, P(dy), P(x), P(g), P(inv), rows, dim, P(dx), P(dg), 0), do_flush=False)
    gb = (3.0 * rows * dim + rows) * 4 / 1e9
    emit(kernel="rmsnorm_bwd", shape=[rows, dim], ms=ms, gbps=gb / (ms * 1e-3), frac_of_hbm=gb / (ms * 1e-3) / hbm, hbm_peak_gbps=hbm, peak_source=src)
    for srows, slen in ((524288 * (1 if args.quick else 2), 64), (524288, 128)):   # config 3: 8192 x 64 rows of 64; config 4: 4096 x 128 rows of 128
        s = torch.randn(srows, slen, device="cuda"); o = torch.empty_like(s)
        ms = timeit(lambda: L.talos_softmax_fwd(ctx.handle, P(s), P(o), srows, slen, 0.125, 0), do_flush=False)
        gb = 2.0 * srows * slen * 4 / 1e9
        emit(kernel="softmax_fwd", shape=[srows, slen], ms=ms, gbps=gb / (ms * 1e-3), frac_of_hbm=gb / (ms * 1e-3) / hbm, hbm_peak_gbps=hbm, peak_source=src)
        gs = torch.randn_like(s); ds = torch.empty_like(s)
        ms = timeit(lambda: L.talos_softmax_bwd(ctx.handle, P(o), P(gs), P(ds), srows, slen, 0.125, 0), do_flush=False)
        gb = 3.0 * srows * slen * 4 / 1e9
        emit(kernel="softmax_bwd", shape=[srows, slen], ms=ms, gbps=gb / (ms * 1e-3), frac_of_hbm=gb / (ms * 1e-3) / hbm, hbm_peak_gbps=hbm, peak_source=src)
    Bq, S, H, dr = 512 * (1 if args.quick else 4), 128, 8, 32    # config 4 rotary part
    c = torch.empty(S * dr // 2, device="cuda"); sn = torch.empty_like(c); L.talos_rope_table(ctx.handle, dr, S, 10000.0, P(c), P(sn))
    xr = torch.randn(Bq, S, H, dr, device="cuda"); yr = torch.empty_like(xr)
    ms = timeit(lambda: L.talos_rope(ctx.handle, P(xr), P(yr), P(c), P(sn), c.numel(), Bq, S, H, dr, 0, 0, 0), do_flush=False)
    gb = 2.0 * xr.numel() * 4 / 1e9
    emit(kernel="rope", shape=[Bq, S, H, dr], ms=ms, gbps=gb / (ms * 1e-3), frac_of_hbm=gb / (ms * 1e-3) / hbm, hbm_peak_gbps=hbm, peak_source=src)
    n = 1 << (22 if args.quick else 25)                          # rollout buffer: GAE scan + advantage normalisation
    rw = torch.randn(n, device="cuda"); vl = torch.randn(n, device="cuda"); tm = (torch.rand(n, device="cuda") < 0.02).to(torch.int32)
    adv = torch.empty(n, device="cuda"); ret = torch.empty(n, device="cuda")
    ms = timeit(lambda: L.talos_gae(ctx.handle, P(rw), P(vl), P(tm), n, 0.99, 0.95, 0.0, 1.0, P(adv), P(ret)), do_flush=False)
    gb = (2 * 12.0 + 8.0) * n / 1e9                               # two passes read r, V, terminal; the second writes A and R
    emit(kernel="gae", shape=[n], ms=ms, gbps=gb / (ms * 1e-3), frac_of_hbm=gb / (ms * 1e-3) / hbm, hbm_peak_gbps=hbm, peak_source=src)
    ms = timeit(lambda: L.talos_normalize_slice(ctx.handle, P(adv), n, P(ret), None), do_flush=False)
    gb = 16.0 * n / 1e9                                           # three reads, one write
    emit(kernel="normalize_slice", shape=[n], ms=ms, gbps=gb / (ms * 1e-3), frac_of_hbm=gb / (ms * 1e-3) / hbm, hbm_peak_gbps=hbm, peak_source=src)
    BH, S, dqk, dv = 4096, 128, 96, 64                           # config 4 attention core
    q = torch.randn(BH, S, dqk, device="cuda"); k = torch.randn_like(q); v = torch.randn(BH, S, dv, device="cuda"); o = torch.empty_like(v)
    for mname in ("tf32", "tf32x3", "fp32"):
        md = talos.MODES[mname]
        ms = timeit(lambda: L.talos_attention_fwd(ctx.handle, P(q), P(k), P(v), P(o), None, BH, S, dqk, dv, 0.1, 0, md), do_flush=False, reps=5)
        emit(kernel="attention_fwd", mode=mname, shape=[BH, S, dqk, dv], ms=ms, tflops=2.0 * BH * S * S * (dqk + dv) / (ms * 1e-3) / 1e12)


if __name__ == "__main__":
    main()
