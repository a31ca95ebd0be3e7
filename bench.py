#!/usr/bin/env python
"""Headline benchmark: Q6_K MoE decode tokens/s (batch 1) on B200.

Workload ("decode_qwen3moe_q6k_b1"): the Qwen3MoE-architecture model of the
decode configuration -- 48 layers, hidden 2048, 32/4 heads of 128, 128 experts
(8 active, FFN 768), vocab 151936, every linear weight Q6_K, f32 router,
random-init from seed 0 -- after a prompt of `--prompt` uniform token ids. A
step is one greedy decode pass (one token). Synthetic weights and ids stand in
for the real checkpoint, which is not available.

  value     tokens/s with everything resident: K passes queued back to back,
            each token fed to the next on the device, timed with CUDA events on
            the library stream.
  e2e       tokens/s through the public call `CudaModel.forward(token, pos)`:
            per step 8 bytes host->device, the pass, 4 bytes device->host and
            one synchronise, timed on the host between synchronises.
  roofline  the Q6_K matvec kernel: algorithmic bytes of one token's matvec
            launches / their device time (events), against the measured HBM
            copy bandwidth. Each token streams ~2.5 GB of weights out of a
            24 GB model, so every launch reads HBM-cold data (inputs larger than L2).
  cpu_baseline  the CPU oracle (a port of the reference's scalar CPU path) on
            the host cores, on a bounded sample (see `sample`).

`--impl reference` times that CPU port as the main line: the reference is Rust
and cannot be built here, so the oracle port stands in for llamd-cpu.

Multi-GPU (torchrun): one process per GPU, each decoding its own sequence on
its own replica of the model (scaling "weak"); value is the sum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def matvec_bytes_per_token(hp):
    """Algorithmic bytes of one token's Q6_K matvec launches: weights read once
    plus the Q8_K activations in and the f32 rows out of every launch."""
    E, qd, kvd = hp["n_embd"], hp["n_head"] * hp["head_dim"], hp["n_head_kv"] * hp["head_dim"]
    ffe, nu, V, L = hp["n_ff_expert"], hp["n_expert_used"], hp["n_vocab"], hp["n_layer"]
    q6 = lambda rows, k: rows * (k // 256) * 210
    act = lambda k: k + (k // 256) * 4
    w_layer = q6(qd, E) + 2 * q6(kvd, E) + q6(E, qd) + nu * (2 * q6(ffe, E) + q6(E, ffe))
    io_layer = act(E) + (qd + 2 * kvd) * 4 + act(qd) + E * 4 + act(E) + 2 * nu * ffe * 4 + nu * act(ffe) + nu * E * 4
    weights = L * w_layer + q6(V, E)
    io = L * io_layer + act(E) + V * 4
    return weights, io


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm)}


def decode_config(args, hp, world, ep, data_plane):
    """What names the workload: the same object in the repo arm's line and in the reference arm's."""
    return {"workload": "decode_qwen3moe_q6k_b1", "layers": hp["n_layer"], "experts": "128x8", "hidden": 2048, "vocab": 151936,
            "batch": 1, "prompt": args.prompt, "weights": "Q6_K random-init seed 0", "kv": args.kv,
            "l2": "each token reads ~2.5 GB of a 24 GB model: inputs larger than L2",
            "parallelism": (f"ep{world}: experts sharded {128 // world} per GPU; {data_plane}" if ep else f"replicas x{world}"),
            "arith": args.arith}


class CpuPort:
    """The oracle's decode pass, a whole token at a time, on the host cores.

    All 48 layers run. Only `n_sample` distinct layers of weights are generated (a layer with its 128 experts is
    0.5 GB; 48 of them would not fit every host): layer il computes with the weights of layer il % n_sample, which
    changes no operation count and no byte read. The KV cache is filled to `start_pos` positions with N(0,1) rows,
    so attention does the work of a token that follows a `start_pos`-token prompt.
    """

    def __init__(self, hp, seed, n_sample, threads, start_pos, room, kv_f16=False):
        import oracle
        from llamd_rs_b200 import synth

        self.oracle, self.hp, self.n_sample = oracle, hp, n_sample
        t0 = time.time()
        sample = [synth.layer_weights(hp, seed, il, with_experts=True) for il in range(n_sample)]
        self.w = dict(tok_embd=synth.q6k_blocks(hp["n_vocab"] * hp["n_embd"] // 256, seed, "tok_embd"),
                      output_norm=np.ones(hp["n_embd"], np.float32),
                      output=synth.q6k_blocks(hp["n_vocab"] * hp["n_embd"] // 256, seed, "output"),
                      layers=[sample[il % n_sample] for il in range(hp["n_layer"])])
        self.om = oracle.Model(hp, self.w, threads=threads)
        self.om.kv_new(start_pos + room, f16=kv_f16)
        kvd = hp["n_head_kv"] * hp["head_dim"]
        if start_pos:
            for il in range(hp["n_layer"]):
                kv = synth.normal_f32(2 * start_pos * kvd, seed, "cpu.kv", il)
                if kv_f16:
                    kv = kv.astype(np.float16).astype(np.float32)
                self.om.kv_fill(il, 0, kv[:start_pos * kvd], kv[start_pos * kvd:])
        self.pos = self.start = start_pos
        self.tok = int(synth.token_ids(1, hp["n_vocab"], seed, "cpu.first")[0])
        log(f"[cpu] {n_sample} sampled layers + embeddings + a {start_pos}-position KV cache ready in {time.time() - t0:.1f}s")

    def step(self, threads=None):
        """One greedy token; returns its wall time in seconds."""
        if threads is not None:
            self.om.m.threads = threads
        t = time.perf_counter()
        logits = self.om.forward(self.tok, self.pos)
        self.tok = self.oracle.argmax(logits)
        dt = time.perf_counter() - t
        self.pos += 1
        return dt

    def sample_text(self, what, threads):
        return (f"{what}; every step runs all {self.hp['n_layer']} layers (weights of {self.n_sample} generated layers cycled: same work), "
                f"output norm, lm_head and argmax on {threads} threads, at positions from {self.start} on (KV cache pre-filled with N(0,1) rows)")


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path: the oracle port, all host threads. Every step is a whole token."""
    if rank != 0:
        return
    from llamd_rs_b200 import synth

    hp = dict(synth.QWEN3MOE_30B)
    hp["n_layer"] = args.layers
    threads = os.cpu_count() or 1
    total = args.warmup + args.steps
    port = CpuPort(hp, 0, 2, threads, args.prompt, total + 2, kv_f16=args.kv == "f16")
    for _ in range(args.warmup):
        port.step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        port.step()
    sec_per_tok = (time.perf_counter() - t0) / args.steps
    single = port.step(threads=1)  # the reference's own configuration: one thread
    v = 1.0 / sec_per_tok
    ep = world > 1 and args.parallelism == "ep"
    line = {"impl": "reference", "metric": "q6k_moe_decode_tok_s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * sec_per_tok, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "i8xi8->i32, f32 tail", "data": "synthetic",
            "config": decode_config(args, hp, world, ep, data_plane_text(args)),
            "cpu_baseline": {"value": v, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": port.sample_text(f"{args.steps} decode steps after {args.warmup} warm-up steps", threads),
                             "single_thread": {"value": 1.0 / single, "unit": "tok/s", "cores": 1, "sample": "1 step"}},
            "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def data_plane_text(args):
    return ("NCCL all-gather dispatch + all-to-all combine per layer" if args.ep_nccl else
            "peer stores + system-scope arrival counters over NVLink per layer, NCCL for set-up only")


def measured_peaks():
    """(HBM GB/s, where it came from, the file's content): the pool's measured copy bandwidth when the file is there, else the
    stated fallback."""
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        peaks = {}
    if "hbm_gbs" in peaks:
        return float(peaks["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)", peaks
    return 6650.0, "fallback 6650", peaks


def run_prefill(args, m, hp, prompt, rank, world, backend, dist):
    """Prompt throughput: K passes of the tiled prefill over the same prompt from position 0 (pp<prompt>)."""
    import ctypes as C

    from llamd_rs_b200._lib import lib as _lib

    L = _lib()
    K, W = args.steps, args.warmup
    # the library default (512) is the reference's; larger tiles fold each expert's weights for more tokens at once
    m.prefill_tile = args.tile if args.tile > 0 else min(len(prompt), 2048)
    m.set_prefill_gemm({"exact": 1, "dp4a": 0, "tc": 2}[args.gemm])
    if args.prefold:
        m.set_option("prefill_prefold", 1)
    for _ in range(W):
        m.prefill(prompt, 0)
    backend.sync()
    if dist:
        dist.barrier()
    launches0 = L.llamd_fwd_launch_count()
    ms = C.c_float(0)
    t1 = time.perf_counter()
    L.llamd_fwd_timer_start()
    for _ in range(K):
        tok = m.prefill(prompt, 0)
    L.llamd_fwd_timer_stop(C.byref(ms))
    backend.sync()
    wall = time.perf_counter() - t1
    if dist:
        import torch

        t = torch.tensor([ms.value, wall], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms.value, wall = float(t[0]), float(t[1])
    n = len(prompt)
    wbytes = hp["n_layer"] * (15482880 + 128 * 3 * 1290240)  # a 512-token tile touches every expert of every layer
    peak, peak_src, peaks = measured_peaks()
    # the matmuls of one pass as multiply-adds: per token and layer QKV + attn_out + 8 experts x (gate, up, down)
    macs = n * hp["n_layer"] * (2048 * 5120 + 4096 * 2048 + 8 * 3 * 768 * 2048)
    tops = 2.0 * macs / (ms.value / K * 1e-3) / 1e12
    line = {"metric": "q6k_moe_prefill_tok_s", "value": world * n * K / (ms.value * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms.value / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 pairs -> f32 (tcgen05, tolerance level)" if args.gemm == "tc" else "i8xi8->i32, f32 tail", "data": "synthetic",
            "config": {"workload": f"prefill_qwen3moe_q6k_pp{n}", "layers": hp["n_layer"], "tile": m.prefill_tile, "gemm": args.gemm, "prefold": bool(args.prefold),
                       "l2": "a tile streams every expert of every layer (23.8 GB): inputs larger than L2"},
            "e2e": {"value": world * n * K / wall, "unit": "tok/s", "h2d_bytes_per_step": 8 * n, "d2h_bytes_per_step": 4},
            "gpu_launches": int(L.llamd_fwd_launch_count() - launches0), "last_token": int(tok),
            "roofline": {"bound": "hbm", "achieved": wbytes / (ms.value / K * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": wbytes / (ms.value / K * 1e-3) / 1e9 / peak,
                         # one ncu capture of the grouped GEMM read 1.006x its algorithmic bytes (pre-folded: 816.7 MB for the 811 MB of
                         # gate+up images); the matmuls' weights are the pass's traffic to within that
                         "traffic": 1.006 * hp["n_layer"] * (15482880 + 128 * 3 * 1290240 * (2.016 / 0.8203 if args.prefold else 1.0))
                         if world == 1 else None,
                         "peak_source": peak_src,
                         "matmul_tops": tops, "matmul_frac_of_bf16_peak": tops / float(peaks.get("bf16_tflops_sustained", 1400.0)),
                         "note": "weight bytes of one pass / pass time against the copy peak; matmul_tops = 2 x multiply-adds of the "
                                 "pass's matmuls / pass time, against the measured sustained bf16 GEMM rate for scale (the exact path "
                                 "runs integer MMAs and is bound by folding Q6_K blocks into operands on the CUDA cores)"}}
    if rank == 0:
        print(json.dumps(line), flush=True)
    m.free()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prompt", type=int, default=512, help="prompt length consumed before the timed decode")
    ap.add_argument("--layers", type=int, default=48, help="(debug) fewer layers; the JSON line says so")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill"],
                    help="decode: the headline (one token per step). prefill: one pass over a --prompt token prompt per step")
    ap.add_argument("--parallelism", default="", choices=["", "replicas", "ep"],
                    help="N > 1: ep (default) = experts sharded 128/N per GPU, dispatch/combine per MoE layer, each rank decodes "
                         "its own sequence; replicas = one full model per GPU, no exchange")
    ap.add_argument("--arith", default="exact", choices=["exact", "fast"],
                    help="exact: every f32 reduction in the reference's order (token ids bit-exact against the CPU path; what `value` "
                         "is unless asked otherwise). fast: the long sums of a decode token as reduction trees, same launches "
                         "(tolerance-level floats; with --resident 1 through the resident kernel). An exact run on one GPU also times the fast mode and reports it in detail.fast_arith")
    ap.add_argument("--kv", default="f32", choices=["f32", "f16"],
                    help="K/V cache element type. f32: the reference's (every backend of it), and what the committed CPU run of the "
                         "benchmark used. f16: binary16, rounded once at the store (model option kv_f16; the oracle has the same mode)")
    ap.add_argument("--gemm", default="exact", choices=["exact", "dp4a", "tc"],
                    help="prefill workload: exact = integer tensor path (mma.sync), bit-identical to decode (default); dp4a = the same "
                         "bits, 8 tokens per weight pass; tc = tcgen05 on f16 pairs, tolerance level")
    ap.add_argument("--prefold", action="store_true", help="prefill workload: keep the expert matrices a second time, folded for the integer "
                    "GEMM (model option prefill_prefold; +58 GB on the 48-layer model; same bits)")
    ap.add_argument("--tile", type=int, default=0, help="prefill workload: tokens per prefill tile (0: min(prompt, 2048))")
    ap.add_argument("--ep-nccl", action="store_true", help="with --parallelism ep: the two exchanges per layer as NCCL collectives "
                    "(all-gather + grouped send/recv) instead of peer stores with arrival counters")
    ap.add_argument("--gguf", default="", help="load the model through the GGUF reader instead of tensor by tensor: a path to an "
                    "existing file, or a path that does not exist yet, where the same random-init model is written first")
    ap.add_argument("--resident", type=int, default=-1, help="1: decode through the resident kernel (one cooperative launch per token); "
                    "0: the per-op pass; default: the library's own default")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--set", default="", help="(A/B) comma list of model options name=value set before the run, e.g. early_loads=0; "
                                              "the JSON line's detail.options repeats it")
    ap.add_argument("--ep-rank-arrive", action="store_true", help="(A/B) expert parallelism: one arrival per rank and launch on the return "
                    "path instead of one per CTA of the down projection (measured 0.8 %% slower at 4 GPUs)")
    ap.add_argument("--no-pdl", action="store_true", help="serialise kernels instead of programmatic dependent launch (A/B)")
    ap.add_argument("--prefetch", action="store_true", help="(experiment) matvec launches ask L2 for the next matvec's weights; measured slightly slower")
    ap.add_argument("--batch-sweep", default="", help="(secondary) comma list of batch sizes: time forward_batch over that many "
                    "independent sequences (crates/llamd-runtime/src/device.rs:741-962) and print tok/s per batch size to stderr")
    ap.add_argument("--resident-phases", action="store_true", help="(diagnostic) per-phase time inside the resident decode kernel, then exit")
    ap.add_argument("--phases", action="store_true", help="(diagnostic) print the per-phase time of an un-graphed pass and exit")
    ap.add_argument("--pdl-sweep", default="", help="(experiment) comma list of PDL class masks to time, e.g. 0,1,5,15")
    ap.add_argument("--no-graph", action="store_true", help="queue every launch instead of replaying the captured graph "
                    "(for a profiler's launch list; the timed numbers are then not the headline)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if not args.parallelism:
        args.parallelism = "ep" if env_int("WORLD_SIZE", 1) > 1 else "replicas"

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group(backend="gloo")  # host-side barrier / max only: the data path has no collective
        dist = dist_mod

    from llamd_rs_b200 import backend, synth
    from llamd_rs_b200.model import CudaModel

    if not backend.available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    backend.set_device(local)
    backend.stream_init()
    info = backend.device_info(local)
    ep = world > 1 and args.parallelism == "ep"
    if ep:
        # NCCL's version banner goes to stdout, where the one JSON line lives
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        from llamd_rs_b200 import model as _M

        def _share(b):
            obj = [b]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]

        _M.ep_init(rank, world, _share)

    hp = dict(synth.QWEN3MOE_30B)
    hp["n_layer"] = args.layers
    K, W = args.steps, args.warmup
    max_kv = args.prompt + 2 * (K + W) + 8 + (8 * (K + W) if args.batch_sweep else 0)
    t0 = time.time()
    max_seq = max([int(b) for b in args.batch_sweep.split(",")]) if args.batch_sweep else 1
    if args.gguf:
        from llamd_rs_b200 import gguf as _gguf

        if not os.path.exists(args.gguf):
            if rank == 0:
                n = _gguf.write_synthetic(args.gguf + ".part", hp, 0)
                os.replace(args.gguf + ".part", args.gguf)
                log(f"[rank 0] wrote {args.gguf}: {n / 2**30:.2f} GiB in {time.time() - t0:.1f}s")
            if world > 1:
                dist.barrier()
        t0 = time.time()
        m = CudaModel.open_gguf(args.gguf, max_kv=max_kv, max_seq=max_seq)
    else:
        m = CudaModel.load_synthetic(hp, 0, max_kv=max_kv, max_seq=max_seq)
    log(f"[rank {rank}] model resident: {m.weight_bytes() / 2**30:.2f} GiB in {time.time() - t0:.1f}s on {info.name}")
    if args.ep_rank_arrive:
        m.set_option("ep_rank_arrive", 1)
    if args.kv == "f16":
        m.set_option("kv_f16", 1)  # (before the attach: the caches are re-allocated)
    if ep and not args.ep_nccl:
        if args.batch_sweep:
            m.prefill_tile = max(max_seq, 8)  # the tile exchange's capacity is fixed at the attach: size it for the batches

        def _gather(b):
            out = [None] * world
            dist.all_gather_object(out, b)
            return out

        m.ep_p2p_attach(_gather)
        dist.barrier()
    if args.no_graph:
        m.use_graph = False
    if args.no_pdl:
        from llamd_rs_b200._lib import lib as _l

        _l().llamd_fwd_set_pdl(0)
    if args.prefetch:
        m.set_option("prefetch", 1)
    for kv in [t for t in args.set.split(",") if t]:
        name, _, val = kv.partition("=")
        m.set_option(name.strip(), int(val))
    if args.resident >= 0 and not ep:
        m.set_option("resident", args.resident)
    if args.arith == "fast":
        if ep:
            raise SystemExit("--arith fast is a single-GPU decode mode (replicas); not available with expert parallelism")
        m.set_option("arith", 1)

    prompt = synth.token_ids(args.prompt, hp["n_vocab"], 0, "prompt", rank)
    if args.workload == "prefill":
        run_prefill(args, m, hp, prompt, rank, world, backend, dist)
        return
    # each rank decodes its own sequence
    t0 = time.time()
    tok = m.prefill(prompt, 0)
    log(f"[rank {rank}] prompt of {args.prompt} consumed in {time.time() - t0:.2f}s")
    pos = args.prompt

    def barrier():
        backend.sync()
        if dist:
            dist.barrier()

    def max_over_ranks(v):
        if not dist:
            return v
        import torch

        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.batch_sweep:
        import numpy as _np

        for B in [int(b) for b in args.batch_sweep.split(",")]:
            toks = _np.array([int(t) for t in synth.token_ids(B, hp["n_vocab"], 3, "batch")], dtype=_np.int32)
            p0 = 0
            for _ in range(args.prompt if B > 1 else 0):  # fill each sequence's cache to the same depth as the headline
                toks = m.forward_batch(toks, [p0] * B)
                p0 += 1
            p0 = max(p0, pos if B == 1 else p0)
            for _ in range(W):
                toks = m.forward_batch(toks, [p0] * B)
                p0 += 1
            backend.sync()
            barrier()
            t1 = time.perf_counter()
            for _ in range(K):
                toks = m.forward_batch(toks, [p0] * B)
                p0 += 1
            backend.sync()
            barrier()
            dt = max_over_ranks(time.perf_counter() - t1)
            if rank == 0:
                log(f"[batch-sweep] batch {B} per GPU x {world} GPU(s){' expert-parallel' if ep else ''}: {world * B * K / dt:.1f} tok/s aggregate, "
                    f"{dt / K * 1e3:.3f} ms/pass, position ~{p0}")
        return
    if args.resident_phases:
        m.set_option("resident", 1)
        for _ in range(4):
            tok = m.forward(tok, pos)
            pos += 1
        m.set_option("resident_profile", 1)
        n = 16
        for _ in range(n):
            tok = m.forward(tok, pos)
            pos += 1
        backend.sync()
        prof = m.resident_profile()
        raw = m.resident_profile_raw()
        if raw[31]:
            log(f"[resident] SM clock inside the kernel: {raw[30]} cycles / {raw[31]} ns = {raw[30] / raw[31] * 1e3:.0f} MHz")
        tot = sum(prof.values())
        for k, v in prof.items():
            log(f"[resident] {k:28s} {v / n / 1e3:9.1f} us/token {v / n / hp['n_layer'] / 1e3:7.2f} us/layer {100 * v / max(tot, 1):5.1f} %")
        log(f"[resident] total {tot / n / 1e6:.3f} ms/token inside the kernel (CTA 0's clock)")
        return
    if args.phases:
        m.forward(tok, pos)
        acc = {}
        for i in range(8):
            for k, v in m.profile_pass(tok, pos).items():
                acc[k] = acc.get(k, 0.0) + v / 8
        tot = sum(acc.values())
        for k, v in acc.items():
            log(f"[phase] {k:10s} {v * 1e3:9.1f} us/token {v / hp['n_layer'] * 1e3:7.2f} us/layer {100 * v / tot:5.1f} %")
        log(f"[phase] total {tot:.3f} ms (events between launches serialise the pass)")
        return
    if args.pdl_sweep:
        from llamd_rs_b200._lib import lib as _l

        for mask in [int(v) for v in args.pdl_sweep.split(",")]:
            _l().llamd_fwd_set_pdl(mask if mask != 1 else 1 | 0x100)
            m._L.llamd_model_set_option(m._h, b"pdl", mask if mask != 1 else 0x101)
            for _ in range(3):
                m.decode(tok, pos, 8)
            _, ms = m.decode(tok, pos, K)
            mv, _n = m.bench_matvecs(8)
            log(f"[pdl-sweep] mask {mask}: {ms / K:.3f} ms/token, matvec-only {mv / 8:.3f} ms")
        return

    # ---- warm-up (both paths) ----
    first_tok, warm_tokens = tok, []
    for _ in range(W):
        tok = m.forward(tok, pos)
        warm_tokens.append(tok)
        pos += 1

    from llamd_rs_b200._lib import lib as _lib

    log(f"[launch-index] timed region starts after {_lib().llamd_fwd_launch_count()} launches; "
        f"{m.launches_per_pass()} launches per pass")
    sampler = ClockSampler(local)
    sampler.start()
    # ---- e2e: the public per-token call, host token in / host token out ----
    barrier()
    t1 = time.perf_counter()
    e2e_tokens = []
    for _ in range(K):
        tok = m.forward(tok, pos)
        e2e_tokens.append(tok)
        pos += 1
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t1)

    # ---- value: resident loop, device-timed ----
    barrier()
    tok0, pos0 = tok, pos
    toks, ms = m.decode(tok, pos, K)
    barrier()
    dev_ms = max_over_ranks(ms)
    pos += K
    clocks = sampler.stop()

    # ---- the other arithmetic mode over the same K positions (one GPU, exact runs only): how fast, and whether it chose the same tokens
    fast_arith = None
    if args.arith == "exact" and not ep and world == 1 and args.workload == "decode":
        try:
            m.set_option("arith", 1)
            m.decode(tok0, pos0, min(K, 8))
            ftoks, fms = m.decode(tok0, pos0, K)
            same = [int(a) == int(b) for a, b in zip(ftoks, toks)]
            fast_arith = {"value": K / (fms * 1e-3), "unit": "tok/s", "ms_per_step": fms / K, "tokens_equal_exact": all(same),
                          "first_difference_at_step": None if all(same) else same.index(False), "steps": K,
                          "note": "the same K positions decoded again, same launches, with reduction trees for the two norms' "
                                  "sums, the router's dots and attention's sums (model option arith = 1); everything else as in "
                                  "the exact mode"}
            m.set_option("arith", 0)
            m.decode(tok0, pos0, K)  # leave the cache as the exact run left it
        except Exception as e:
            fast_arith = {"unavailable": str(e)}

    # ---- roofline of the dominant kernel ----
    iters = max(4, min(K, 16))
    wbytes, iobytes = matvec_bytes_per_token(hp)
    if ep:
        # sharded experts: the matvec-only replay is not available; report this rank's share of a token's
        # bytes over the whole pass time instead (a lower bound on the kernel's rate)
        mv_ms, mv_launches = dev_ms / K * iters, 193
    else:
        mv_ms, mv_launches = m.bench_matvecs(iters)
    achieved = (wbytes + iobytes) / (mv_ms / iters * 1e-3) / 1e9
    peak, peak_src, _ = measured_peaks()

    # what was decoded, so that a run can be checked against the CPU path's tokens for the same inputs
    decoded = [int(first_tok)] + [int(t) for t in warm_tokens] + [int(t) for t in e2e_tokens] + [int(t) for t in toks]
    tokens_hash = synth.checksum(np.asarray(decoded, np.int32))
    inputs_hash = synth.checksum(np.asarray(prompt, np.int32), synth.layer_weights(hp, 0, 0, with_experts=False)["attn_q"])
    golden_check = None
    golden_path = os.path.join(ROOT, "tests", "golden", "decode_seed0.npz")
    if rank == 0 and args.prompt == 512 and hp["n_layer"] == 48 and args.kv == "f32" and args.arith == "exact" and os.path.exists(golden_path):
        # the CPU oracle's greedy run of this very workload (rank 0's prompt): token ids must be the same
        g = np.load(golden_path)
        want = [int(t) for t in g["chosen"][args.prompt - 1:args.prompt - 1 + len(decoded)]]
        n_cmp = min(len(want), len(decoded))
        golden_check = {"tokens_compared": n_cmp, "equal": decoded[:n_cmp] == want[:n_cmp]}
    hashes = [tokens_hash]
    if dist:
        hashes = [None] * world
        dist.all_gather_object(hashes, tokens_hash)
    detail = {"token_gbs": (wbytes + iobytes) / (dev_ms / K * 1e-3) / 1e9, "ms_per_token_per_rank": dev_ms / K,
              "graph": not args.no_graph, "pdl": not args.no_pdl, "l2_prefetch": args.prefetch, "options": args.set,
              "inputs_hash": inputs_hash, "tokens_hash": hashes[0], "tokens_hash_per_rank": hashes,
              "tokens_head": decoded[:8], "n_tokens_hashed": len(decoded), "tokens_vs_cpu_golden": golden_check, "fast_arith": fast_arith,
              "hash_note": "crc32 of (prompt ids, layer-0 attn_q bytes) and of the int32 token ids chosen after the prompt: "
                           "the prefill's token, the warm-up tokens, the e2e tokens, the device-loop tokens"}
    line = {
        "metric": "q6k_moe_decode_tok_s", "value": world * K / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "i8xi8->i32, f32 tail", "data": "synthetic",
        "config": decode_config(args, hp, world, ep, data_plane_text(args)),
        "detail": detail,
        "e2e": {"value": world * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4},
        "gpu_launches": int(m.launches_per_pass()) * K,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # DRAM bytes per token's matvec launches: an ncu capture of the lm_head launch read+wrote 1.016x its
                     # algorithmic bytes; every weight byte is streamed once from cold HBM in every launch, so the ratio
                     # carries over to the token's launches.
                     "traffic": 1.016 * (wbytes + iobytes),
                     "kernel": "matvec_q6k_kernel<1>", "launches_per_token": mv_launches, "avg_launch_us": mv_ms / iters / mv_launches * 1e3,
                     "algorithmic_bytes_per_token": wbytes + iobytes, "peak_source": peak_src,
                     "frac_of_nominal_8tbs": achieved / 8000.0},
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:  # (the CPU port is timed beside the single-GPU run only)
        threads = os.cpu_count() or 1
        port = CpuPort(dict(synth.QWEN3MOE_30B), 0, 2, threads, args.prompt, 8, kv_f16=args.kv == "f16")
        port.step()
        secs = [port.step() for _ in range(3)]
        single = port.step(threads=1)
        line["cpu_baseline"] = {"value": 1.0 / float(np.mean(secs)), "unit": "tok/s", "cores": threads, "kind": "port",
                                "sample": port.sample_text("3 decode steps after 1 warm step", threads),
                                "single_thread": {"value": 1.0 / single, "unit": "tok/s", "cores": 1, "sample": "1 step"}}
    if rank == 0:
        print(json.dumps(line), flush=True)
    m.free()
    if dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
