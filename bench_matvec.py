"""Decode matvec sweep: the counterpart of the reference's `llamd-bench`
(crates/llamd-bench/src/main.rs:25-32, 79-128, 163-198).

For each of the model's matvec shapes and each batch size it reports
  - the CPU oracle's time (one thread, and row-parallel over the host cores),
  - the host-facing API call (host activations in, host result out),
  - kernel-only time, cold: the launches rotate over enough copies of the
    weights (>= 1 GiB) that no launch finds its matrix in L2, timed with CUDA
    events around a captured graph of `iters` launches,
and the algorithmic GB/s = (weights + activations in + results out) / time,
against the measured HBM copy bandwidth and the nominal 8 TB/s.

    python bench_matvec.py                 # every shape, Q6_K and Q8_0, batch 1 2 4 8
    python bench_matvec.py --shapes lm_head --types q6k --batch 1 --iters 3 --no-cpu
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from llamd_rs_b200 import backend, synth  # noqa: E402
from llamd_rs_b200._lib import lib  # noqa: E402

# (name, rows, k): crates/llamd-bench/src/main.rs:25-32
SHAPES = [("attn_q", 4096, 2048), ("attn_k", 512, 2048), ("attn_out", 2048, 4096), ("expert_gate", 768, 2048),
          ("expert_down", 2048, 768), ("lm_head", 151936, 2048)]


def weight_bytes(ty, rows, k):
    return rows * (k // 256) * 210 if ty == "q6k" else rows * (k // 32) * 34


def algorithmic_bytes(ty, rows, k, batch):
    act = batch * (k + (k // 256) * 4) if ty == "q6k" else batch * k * 4
    return weight_bytes(ty, rows, k) + act + batch * rows * 4


def kernel_only_cold(ty, w_host, rows, k, batch, iters, min_total=1 << 30):
    """ms per launch with the weights HBM-cold."""
    L = lib()
    wb = weight_bytes(ty, rows, k)
    copies = max(2, min(64, -(-min_total // wb)))
    if ty == "q6k":
        bufs = [backend.DeviceWeights.upload(w_host, rows, k // 256) for _ in range(copies)]
    else:
        bufs = [backend.Q80Weights.upload(w_host, rows, k // 32) for _ in range(copies)]
    x = synth.normal_f32(batch * k, 1, "bench.x")
    dx = backend.DevBuf.from_array(x)
    dout = backend.DevBuf(batch * rows * 4)
    if ty == "q6k":
        dq, dd = backend.DevBuf(batch * k), backend.DevBuf(batch * (k // 256) * 4)
        L.llamd_fwd_quantize(dx.ptr, dq.ptr, dd.ptr, batch * (k // 256))

        def launch(i):
            L.llamd_fwd_matvec_batch(bufs[i % copies].ptr, dq.ptr, dd.ptr, dout.ptr, k // 256, rows, batch)
    else:
        def launch(i):
            L.llamd_fwd_matvec_q8_0(bufs[i % copies].ptr, dx.ptr, dout.ptr, k // 32, rows, batch)
    for i in range(copies):  # warm (code, not data: the rotation keeps data cold)
        launch(i)
    backend.sync()
    L.llamd_fwd_graph_destroy()
    L.llamd_fwd_begin_capture()
    for i in range(iters):
        launch(i)
    if L.llamd_fwd_end_capture() != 0:
        raise backend.Other("capture failed: " + backend._last_error())
    L.llamd_fwd_graph_launch()  # one untimed replay
    backend.sync()
    ms = C.c_float(0)
    L.llamd_fwd_timer_start()
    L.llamd_fwd_graph_launch()
    L.llamd_fwd_timer_stop(C.byref(ms))
    L.llamd_fwd_graph_destroy()
    backend.check()
    for b in bufs:
        b.free()
    return ms.value / iters, copies


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="all")
    ap.add_argument("--types", default="q6k,q8_0")
    ap.add_argument("--batch", default="1,2,4,8")
    ap.add_argument("--iters", type=int, default=64)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--json", default="", help="also append one JSON line per row to this file")
    args = ap.parse_args(argv)
    if not backend.available():
        raise SystemExit("bench_matvec needs a CUDA device (there is no CPU fallback)")
    backend.stream_init()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    import oracle  # the CPU column is the oracle port; the GPU columns never touch it

    names = [s[0] for s in SHAPES] if args.shapes == "all" else args.shapes.split(",")
    cores = os.cpu_count() or 1
    print(f"# peak HBM {peak:.0f} GB/s ({'measured' if 'hbm_gbs' in peaks else 'fallback'}); host cores {cores}")
    print(f"{'shape':12} {'type':5} {'B':>2} {'MiB':>7} {'cpu1 ms':>9} {'cpuN ms':>9} {'api ms':>8} {'kernel us':>10} {'GB/s':>8} {'%meas':>6} {'%8TB/s':>7}")
    for name, rows, k in SHAPES:
        if name not in names:
            continue
        for ty in args.types.split(","):
            w = synth.q6k_blocks(rows * k // 256, 0, "bench", name) if ty == "q6k" else synth.q8_0_blocks(rows * k // 32, 0, "bench", name)
            for batch in [int(b) for b in args.batch.split(",")]:
                x = synth.normal_f32(batch * k, 1, "bench.x")
                cpu1 = cpun = float("nan")
                if not args.no_cpu and batch == 1:
                    f = (lambda th: oracle.matvec_q6k(w, x[:k], k, rows, threads=th)) if ty == "q6k" else \
                        (lambda th: oracle.matvec_dequant(oracle.Q8_0, w, x[:k], k, rows, threads=th))
                    f(cores)
                    t = time.perf_counter(); f(1); cpu1 = (time.perf_counter() - t) * 1e3
                    t = time.perf_counter(); f(cores); cpun = (time.perf_counter() - t) * 1e3
                dw = backend.DeviceWeights.upload(w, rows, k // 256) if ty == "q6k" else backend.Q80Weights.upload(w, rows, k // 32)
                dw.matvec_f32(x, batch)
                t = time.perf_counter()
                for _ in range(5):
                    dw.matvec_f32(x, batch)
                api = (time.perf_counter() - t) / 5 * 1e3
                dw.free()
                ms, copies = kernel_only_cold(ty, w, rows, k, batch, args.iters)
                gbs = algorithmic_bytes(ty, rows, k, batch) / (ms * 1e-3) / 1e9
                print(f"{name:12} {ty:5} {batch:2d} {weight_bytes(ty, rows, k) / 2**20:7.1f} {cpu1:9.3f} {cpun:9.3f} {api:8.3f} {ms * 1e3:10.2f} "
                      f"{gbs:8.1f} {100 * gbs / peak:6.1f} {100 * gbs / 8000:7.1f}", flush=True)
                if args.json:
                    with open(args.json, "a") as fjs:
                        fjs.write(json.dumps(dict(shape=name, rows=rows, k=k, type=ty, batch=batch, cpu1_ms=cpu1, cpuN_ms=cpun, cores=cores,
                                                  api_ms=api, kernel_us=ms * 1e3, gbs=gbs, frac_measured=gbs / peak, frac_8tbs=gbs / 8000,
                                                  copies=copies, iters=args.iters)) + "\n")


if __name__ == "__main__":
    main()
