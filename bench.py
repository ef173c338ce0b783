#!/usr/bin/env python
"""Benchmark of the hot path: RNN-T greedy decode of synthetic 10 s utterances (1000 frames x 240
features, batch 1 per stream, random-init weights of the benchmark architecture).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--streams-total S] [--impl reference]

One "step" = the benchmark configuration's 1024 utterance streams, sharded over the N ranks (1024 / N per rank,
decoded in one call per rank: encoder groups of 128 utterances, one greedy launch).  Utterances are independent, so ranks share nothing on the data path
("strong" scaling: the total is fixed; no collective); torch.distributed is used only for the barrier and the
max-over-ranks of the device time.  The same line carries the stand-alone LSTM (C1) and GEMV (C2) figures of the
baseline metric under the keys `lstm_c1` and `gemv`.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

T_FRAMES = 1000
# dram__bytes_read.sum + dram__bytes_write.sum of one lstm_persistent_pipe_kernel<16,2,4> launch of 500 timesteps x 128
# sequences (1.059 GB + 0.127 GB, the capture summarised under profiles/), per timestep: the fp32 gate pre-activations
# read once and the fp16 outputs written once; traffic grows in proportion to the timesteps of a launch
TRAFFIC_PER_TIMESTEP_128 = (1.058840e9 + 0.126854e9) / 500.0
WORKLOAD = "C3: RNN-T greedy decode, 1000x240 frames per utterance, batch 1 per stream, 1024 streams"
STREAMS_TOTAL = 1024
TENSOR_PIPE_ACTIVE_PCT_NCU = 46.4   # sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active, same capture


def base_config(streams_total: int) -> dict:
    """The workload description both arms print (identical keys and values)."""
    return {"workload": WORKLOAD, "frames": T_FRAMES, "streams_total": streams_total,
            "parallelism": "independent utterance streams sharded over the ranks, no collective",
            "l2": "GPU arm: 256 MB flush write between timed steps; the per-step working set (90.6 MB weights + "
                  "features + activations) also exceeds the 126 MB L2"}


RECURRENCE_KERNEL = "lstm_persistent_pipe_kernel<16,2,4> (W_hh recurrence, all T steps of 128 sequences per launch)"


def load_tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), "measured burst (MEASURED_PEAKS.json)"
    return 1590.0, "fallback"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples during the timed region (reads settings only)."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 9:
                        continue
                    try:
                        sm.append(float(parts[1]))
                        smax.append(float(parts[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                          "sw_power_cap"), parts[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(smax)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


from pimaicompiler_b200.replica import barrier, env_rank, init_process_group, max_over_ranks  # noqa: E402


def dist_setup(n_gpus: int):
    rank, world, local = env_rank()
    init_process_group(world, local, torch.cuda.is_available())
    return rank, world, local


# ------------------------------------------------------------------------------------------------
# CPU arm: the libtorch CPU implementation of the same ops (what the reference's default executors call)
# ------------------------------------------------------------------------------------------------
CPU_SAMPLE_SECONDS = 20.0   # the CPU arm stops taking new streams after this many seconds of work


def host_threads() -> int:
    """Threads the CPU arm uses: the cores this process may run on (affinity mask, cgroup CPU quota), at most 32.  More
    threads than cores make the libtorch calls of a batch-1 decode crawl (spinning barriers on tiny products), and under
    torchrun the other ranks' processes are busy waiting at the same time."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()
        if quota != "max":
            n = min(n, max(1, int(int(quota) / int(period))))
    except (OSError, ValueError):
        pass
    return max(1, min(n, 32))


def cpu_rnnt_throughput(n_utts: int, seed0: int):
    """Decodes n_utts synthetic utterances on the host cores; returns (utt/s, seconds, cores)."""
    from oracle import torch_oracle as to
    cfg = to.RnntConfig()
    w = to.make_rnnt_weights(cfg, seed=0)
    cores = host_threads()
    torch.set_num_threads(cores)
    feats = [to.make_features(T_FRAMES, cfg, seed0 + i) for i in range(n_utts)]
    to.rnnt_greedy(w, feats[0][:100], cfg)  # warm the thread pool
    t0 = time.perf_counter()
    done = 0
    for f in feats:
        to.rnnt_greedy(w, f, cfg)
        done += 1
        if time.perf_counter() - t0 > CPU_SAMPLE_SECONDS:
            break
    dt = time.perf_counter() - t0
    return done / dt, dt, cores


def run_reference(args, rank, world):
    if rank != 0:
        return
    n = min(args.cpu_sample, 32)
    for _ in range(args.warmup):
        cpu_rnnt_throughput(1, 999)
    vals, secs, cores = [], 0.0, 1
    for k in range(args.steps):
        v, dt, cores = cpu_rnnt_throughput(n, 5000 + k * n)
        vals.append(v)
        secs += dt
    value = statistics.median(vals)
    sample = (f"up to {n} utterances per step (no new one after {CPU_SAMPLE_SECONDS:.0f} s), libtorch {torch.__version__} CPU fp32 "
              f"(at::lstm/at::linear), {cores} threads")
    line = {
        "impl": "reference", "metric": "rnnt_greedy_utterances_per_s", "value": value, "unit": "utt/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs / max(args.steps, 1) * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": base_config(args.streams_total),
        "sample_streams_per_step": n,
        "cpu_baseline": {"value": value, "unit": "utt/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "utt/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_gpu(args, rank, world, local):
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the hot path has no CPU fall-back")
    from pimaicompiler_b200 import synthetic as to
    from pimaicompiler_b200 import build
    from pimaicompiler_b200.rnnt import RnntDecoder
    build.build()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = to.RnntConfig()
    w = to.make_rnnt_weights(cfg, seed=0)
    d = lambda t: t.to(torch.float16).to(dev).contiguous()
    dec = RnntDecoder(cfg, [d(p) for p in w.pre], [d(p) for p in w.post], d(w.embedding), [d(p) for p in w.pred],
                      d(w.w1), d(w.b1), d(w.w2), d(w.b2))
    if args.encoder_batch:
        dec.set_encoder_batch(args.encoder_batch)
    # this rank's shard of the configuration's streams, decoded in calls of `chunk` utterances
    streams_total = args.streams_per_gpu * world if args.streams_per_gpu else args.streams_total
    S = (streams_total + world - 1) // world
    chunk = min(args.streams_per_call, S) if args.streams_per_call > 0 else S
    Tp = T_FRAMES // cfg.stack_factor
    g = torch.Generator().manual_seed(1000 + rank)
    feats_host = torch.randn(S, T_FRAMES, cfg.feat_dim, generator=g).to(torch.float16).pin_memory()
    feats = feats_host.to(dev)
    feats_stage = torch.empty(chunk, T_FRAMES, cfg.feat_dim, dtype=torch.float16, device=dev)
    tokens = torch.zeros(S, Tp, dtype=torch.int32, device=dev)
    n_tokens = torch.zeros(S, dtype=torch.int32, device=dev)
    tokens_host = torch.zeros(S, Tp, dtype=torch.int32).pin_memory()
    n_tokens_host = torch.zeros(S, dtype=torch.int32).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2

    def step_device():
        for c in range(0, S, chunk):
            e = min(c + chunk, S)
            dec.decode_into(feats[c:e], tokens[c:e], n_tokens[c:e], None)

    def step_e2e():
        # host features in, token ids out, per call of `chunk` utterances
        for c in range(0, S, chunk):
            e = min(c + chunk, S)
            f = feats_stage[: e - c]
            f.copy_(feats_host[c:e], non_blocking=True)
            dec.decode_into(f, tokens[c:e], n_tokens[c:e], None)
            tokens_host[c:e].copy_(tokens[c:e], non_blocking=True)
            n_tokens_host[c:e].copy_(n_tokens[c:e], non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step_device()
    torch.cuda.synchronize()
    dec.check_status("warm-up decode")

    # ---- device-resident throughput: K steps, each bracketed by CUDA events, L2 flushed between steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dec.profile(True)
    barrier(world)
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for k in range(args.steps):
        flush.fill_(k & 0xff)
        ev[k][0].record()
        step_device()
        ev[k][1].record()
    torch.cuda.synchronize()
    barrier(world)
    step_ms = [a.elapsed_time(b) for a, b in ev]
    prof = dec.profile_read()
    dec.profile(False)
    dec.check_status("timed decode")
    total_ms = max_over_ranks(sum(step_ms), world)
    clocks = sampler.stop() if rank == 0 else {}

    # per-utterance latency (batch 1, one utterance per call), p50 over a few utterances
    lat = []
    for i in range(min(S, 9)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush.fill_(i)
        a.record()
        dec.decode_into(feats[i:i + 1], tokens[i:i + 1], n_tokens[i:i + 1], None)
        b.record()
        torch.cuda.synchronize()
        lat.append(a.elapsed_time(b))
    p50_ms = statistics.median(lat)

    # ---- end to end through the public call with host buffers
    for _ in range(2):
        step_e2e()
    barrier(world)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_e2e()
    e2e_s = max_over_ranks(time.perf_counter() - t0, world)
    barrier(world)
    dec.check_status("end-to-end decode")

    utts_total = S * world * args.steps
    value = utts_total / (total_ms * 1e-3)
    e2e_value = utts_total / e2e_s

    # ---- roofline of the dominant kernel (the LSTM recurrence), timed live with CUDA events
    peak, peak_src = load_peaks()
    tpeak, tpeak_src = load_tensor_peak()
    rec_s = prof["ms"] * 1e-3
    achieved = prof["bytes"] / rec_s / 1e9 if rec_s > 0 else 0.0
    share = prof["ms"] / sum(step_ms) if sum(step_ms) > 0 else 0.0
    eb = min(args.encoder_batch or 128, chunk)
    # the same launches as a contraction: 2 flop per weight element and sequence and timestep
    flops = prof["bytes"] / 2.0 * 2.0 * eb
    tflops = flops / rec_s / 1e12 if rec_s > 0 else 0.0
    # per call of `chunk` utterances: per group of encoder-batch utterances (projection GEMM + recurrence) per LSTM
    # layer; then the joint's encoder-half GEMM and one greedy kernel for the whole call
    calls = (S + chunk - 1) // chunk
    launches_per_step = calls * (((chunk + eb - 1) // eb) * 2 * (cfg.pre_layers + cfg.post_layers) + 2)

    extras = {}
    if rank == 0 and world == 1 and not args.no_extras:        # the op sweeps ride on the one-GPU line only
        del feats, flush
        torch.cuda.empty_cache()
        extras["lstm_c1"] = measure_c1(max(args.steps, 3))["persistent"]
        extras["gemv"] = measure_c2(max(args.steps, 3), batches=(32,), shapes_batched=((4096, 1024),), rowops=False)["results"]
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:   # timed on rank 0 at N = 1 only: the other ranks would wait
        v, dt, cores = cpu_rnnt_throughput(args.cpu_sample, 7000)
        cpu = {"value": v, "unit": "utt/s", "cores": cores, "kind": "port",
               "sample": f"up to {args.cpu_sample} of the same synthetic utterances (no new one after {CPU_SAMPLE_SECONDS:.0f} s), libtorch {torch.__version__} CPU fp32 "
                         f"(the at::lstm/at::linear calls of the reference's default executors), {dt:.1f} s"}
    barrier(world)
    if rank != 0:
        return
    line = {
        "metric": "rnnt_greedy_utterances_per_s", "value": value, "unit": "utt/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage / f32 accumulate",
        "data": "synthetic",
        "config": base_config(S * world),
        "streams_per_gpu": S, "streams_per_call": chunk, "greedy_kernel": dec.info(),
        "p50_ms_per_utt": p50_ms,
        "e2e": {"value": e2e_value, "unit": "utt/s",
                "h2d_bytes_per_step": int(feats_host.numel() * 2),
                "d2h_bytes_per_step": int(tokens_host.numel() * 4 + n_tokens_host.numel() * 4)},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "kernel": RECURRENCE_KERNEL,
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_src,
                     # DRAM bytes of an average launch, scaled from the committed ncu capture by its timesteps (a launch of
                     # fewer than 128 sequences moves proportionally less; the capture is the 128-sequence case)
                     "traffic": TRAFFIC_PER_TIMESTEP_128 * (eb / 128.0) * prof["bytes"] / max(prof["recurrences"], 1) /
                                (4.0 * cfg.enc_hidden * cfg.enc_hidden * 2.0 * (2 if eb > 64 else 1)),
                     "launches": prof["recurrences"], "avg_launch_ms": prof["ms"] / max(prof["recurrences"], 1),
                     "us_per_timestep": prof["ms"] * 1e3 / max(prof["bytes"] / (4.0 * cfg.enc_hidden * cfg.enc_hidden * 2.0), 1.0),
                     "sequences_per_launch": eb,
                     # what batch-1-per-stream execution would have to stream: every sequence its own W_hh per step
                     "per_stream_equivalent_gbs": achieved * eb,
                     "share_of_step_time": share,
                     # the weight-stationary kernel's own bound is the tensor pipe (and the L2 exchange), not HBM:
                     # the same launches as flops against the measured dense bf16 peak, and the pipe's active share
                     # from the committed ncu capture
                     "tensor": {"achieved_tflops": tflops, "peak_tflops": tpeak, "frac": tflops / tpeak,
                                "peak_source": tpeak_src, "pipe_active_pct_ncu": TENSOR_PIPE_ACTIVE_PCT_NCU},
                     "note": "algorithmic bytes = T * 4H*H * 2 per launch (W_hh once per timestep, the streamed "
                             "formulation); the kernel keeps them in registers as mma fragments"},
        "clocks": clocks,
    }
    line.update(extras)
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# secondary workloads: the stand-alone op sweeps of the baseline (C2 GEMV/GEMM, C1 single aten::lstm)
# ------------------------------------------------------------------------------------------------
def _graph_time_us(calls, reps):
    """Average device time of one call: all calls are captured into one CUDA graph (no host launch cost between
    kernels), replayed `reps` times between two CUDA events on the launching stream."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for f in calls[:2]:
            f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in calls:
            f()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(calls))


def measure_c2(reps_base, batches=(8, 32, 128), shapes_batched=None, rowops=True, shapes=None):
    """C2: y = Wx + b at batch 1 for the five (N,K) shapes (weights rotated over > 126 MB so every call streams from
    HBM), and the same layers at batch 8/32/128 through the batched-stream GEMM."""
    from pimaicompiler_b200 import ops
    ops.init()
    peak, peak_src = load_peaks()
    dev = torch.device("cuda", torch.cuda.current_device())
    shapes = shapes or [(4096, 1024), (4096, 2048), (1024, 1024), (32320, 1024), (29, 512)]
    g = torch.Generator().manual_seed(1)
    results = []
    for (N, K) in shapes:
        nb = max(2, min(96, int(400e6 // (N * K * 2)) + 1))       # > 126 MB of distinct weights where it matters
        k = 1.0 / K ** 0.5
        Ws = [((torch.rand(N, K, generator=g) * 2 - 1) * k).half().to(dev) for _ in range(nb)]
        b = ((torch.rand(N, generator=g) * 2 - 1) * k).half().to(dev)
        x = torch.randn(K, generator=g).half().to(dev)
        y = torch.empty(N, dtype=torch.float16, device=dev)
        us = _graph_time_us([(lambda W=W: ops.gemv_mv(W, x, b, out=y)) for W in Ws], reps_base * 10)
        us_l2 = _graph_time_us([(lambda: ops.gemv_mv(Ws[0], x, b, out=y)) for _ in range(nb)], reps_base * 10)
        As = [W.t().contiguous() for W in Ws[: min(nb, 24)]]
        us_vm = _graph_time_us([(lambda A=A: ops.gemv_vm(x, A, b, out=y)) for A in As], reps_base * 10)
        nbytes = 2 * (N * K + K + 2 * N)
        row = {"N": N, "K": K, "B": 1, "bytes": nbytes, "mv_us": us, "mv_gbs": nbytes / us / 1e3,
               "mv_frac_of_measured_hbm": nbytes / us / 1e3 / peak, "mv_l2_resident_us": us_l2,
               "vm_us": us_vm, "vm_gbs": nbytes / us_vm / 1e3, "weights_rotated_mb": nb * N * K * 2 / 1e6}
        results.append(row)
        for B in batches:
            if shapes_batched is not None and (N, K) not in shapes_batched:
                continue
            X = torch.randn(B, K, generator=g).half().to(dev)
            Y = torch.empty(B, N, dtype=torch.float16, device=dev)
            usb = _graph_time_us([(lambda W=W: ops.gemm_wx(W, X, b, out=Y)) for W in Ws], reps_base * 10)
            bb = 2 * (N * K + B * K + N + B * N)
            results.append({"N": N, "K": K, "B": B, "bytes": bb, "gemm_us": usb, "gemm_gbs": bb / usb / 1e3,
                            "gemm_frac_of_measured_hbm": bb / usb / 1e3 / peak,
                            "gemm_tflops": 2.0 * B * N * K / usb / 1e6})
        del Ws, As
    # row-wise glue of a decode step at its benchmark sizes: the 32320-wide GNMT / 29-wide RNN-T logit rows, a 512-wide
    # model vector, 8 heads x 40 attention scores (one launch each, 16 calls per graph)
    rows_out = []
    if rowops:
        for name, rows, cols in (("logits_gnmt", 1, 32320), ("logits_rnnt", 1, 29), ("model_vec", 1, 512), ("attn", 8, 40)):
            xr = (torch.randn(rows, cols, generator=g) * 3).half().to(dev)
            yr = torch.empty_like(xr)
            t_sm = _graph_time_us([(lambda: ops.softmax(xr, out=yr)) for _ in range(16)], reps_base * 10)
            t_am = _graph_time_us([(lambda: ops.argmax(xr)) for _ in range(16)], reps_base * 10)
            t_ln = _graph_time_us([(lambda: ops.layer_norm(xr)) for _ in range(16)], reps_base * 10)
            rows_out.append({"case": name, "rows": rows, "cols": cols, "softmax_us": t_sm, "argmax_us": t_am,
                             "layer_norm_us": t_ln})
    return {"results": results, "rowops": rows_out, "peak": peak, "peak_src": peak_src}


def run_c2(args):
    from pimaicompiler_b200 import build
    build.build()
    sampler = ClockSampler(0)
    sampler.start()
    if args.c2_shape:   # a restricted sweep (one shape, chosen batches, no row ops): the small case a profiler capture uses
        n, k = (int(v) for v in args.c2_shape.lower().split("x"))
        batches = tuple(int(v) for v in args.c2_batches.split(",")) if args.c2_batches else ()
        m = measure_c2(args.steps, batches=batches, rowops=False, shapes=[(32320, 1024), (n, k)] if (n, k) != (32320, 1024) else [(n, k)],
                       shapes_batched=[(n, k)])
    else:
        m = measure_c2(args.steps)
    results, rowops, peak, peak_src = m["results"], m["rowops"], m["peak"], m["peak_src"]
    clocks = sampler.stop()
    big = next(r for r in results if r["N"] == 32320 and r["B"] == 1)
    line = {"metric": "gemv_mv_hbm_gbs", "value": big["mv_gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": 3, "ms_per_step": big["mv_us"] / 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 storage / f32 accumulate", "data": "synthetic",
            "config": {"workload": "C2: aten::linear batch-1 GEMV sweep + batch 8/32/128 GEMM", "headline_shape": [32320, 1024],
                       "l2": "weights rotated over more distinct buffers than fit the 126 MB L2",
                       "timing": "CUDA graph of the rotated calls, CUDA events around the replays"},
            "roofline": {"bound": "hbm", "kernel": "gemv_mv_vec_kernel<4> (32320x1024)", "achieved": big["mv_gbs"],
                         "peak": peak, "unit": "GB/s", "frac": big["mv_gbs"] / peak, "peak_source": peak_src,
                         "traffic": None},
            "results": results, "rowops": rowops, "clocks": clocks, "gpu_launches": None}
    print(json.dumps(line), flush=True)


def measure_c1(reps_base):
    """C1: one aten::lstm, 2 layers, input 240, hidden 1024, T=200, batch 1 (seed 0), streamed and persistent."""
    from pimaicompiler_b200 import ops
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(0)
    T, I, H, L = 200, 240, 1024, 2
    x = torch.randn(T, 1, I, generator=gen).half().to(dev)
    ps = []
    for l in range(L):
        Il = I if l == 0 else H
        ps += [((torch.rand(4 * H, Il, generator=gen) * 2 - 1) / 32).half().to(dev),
               ((torch.rand(4 * H, H, generator=gen) * 2 - 1) / 32).half().to(dev),
               ((torch.rand(4 * H, generator=gen) * 2 - 1) / 32).half().to(dev),
               ((torch.rand(4 * H, generator=gen) * 2 - 1) / 32).half().to(dev)]
    m = ops.Lstm(ps, L, False, I, H, True)
    peak, _ = load_peaks()
    res = {}
    for name, v in (("streamed", ops.LSTM_STREAMED), ("persistent", ops.LSTM_AUTO)):
        m.set_variant(v)
        out = m.forward(x)
        for _ in range(3):
            m.forward(x, out=out)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps_base * 5):
            m.forward(x, out=out)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps_base * 5)
        gbs = T * L * 4 * H * H * 2 / us / 1e3
        res[name] = {"us_per_call": us, "us_per_layer_step": us / (T * L), "w_hh_stream_gbs": gbs,
                     "frac_of_measured_hbm": gbs / peak,
                     "config": "aten::lstm L=2 I=240 H=1024 T=200 B=1, whole call (projection GEMMs included)"}
    assert m.last_status() == 0
    return res


def run_c1(args):
    from pimaicompiler_b200 import build
    build.build()
    res = measure_c1(args.steps)
    peak, peak_src = load_peaks()
    best = res["persistent"]
    line = {"metric": "lstm_c1_us_per_call", "value": best["us_per_call"], "unit": "us", "n_gpus": 1,
            "steps": args.steps, "warmup": 3, "ms_per_step": best["us_per_call"] / 1e3, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage / f32 accumulate", "data": "synthetic",
            "config": {"workload": "C1: aten::lstm L=2 I=240 H=1024 T=200 B=1"},
            "roofline": {"bound": "hbm", "kernel": "persistent recurrence", "achieved": best["w_hh_stream_gbs"],
                         "peak": peak, "unit": "GB/s", "frac": best["w_hh_stream_gbs"] / peak, "peak_source": peak_src,
                         "traffic": None, "note": "whole call (projection GEMMs included); bytes = T*L*4H*H*2"},
            "results": res, "gpu_launches": None}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# C4 / C5: translation workloads, stream-sharded like C3 (sentences round-robin over the ranks, no collective)
# ------------------------------------------------------------------------------------------------
class _Translate:
    """What differs between the GNMT (C4) and the Transformer (C5) workload."""

    def __init__(self, kind: str):
        from pimaicompiler_b200 import synthetic as syn
        self.kind = kind
        if kind == "c4":
            self.total, self.metric, self.unit, self.group = 512, "gnmt_greedy_sentences_per_s", "sentences/s", 512
            self.cfg = syn.GnmtConfig()
            self.make_weights = syn.make_gnmt_weights
            self.desc = ("C4: GNMT greedy translation (4+4 LSTM layers, hidden 1024, vocabulary 32320, normalised Bahdanau "
                         "attention), sentences of 20..50 tokens, 80 decode steps")
            self.l2 = "one step touches 160 MB of weights, more than the 126 MB L2"
        else:
            self.total, self.metric, self.unit, self.group = 2048, "transformer_greedy_sequences_per_s", "sequences/s", 2048
            self.cfg = syn.TransformerConfig()
            self.make_weights = syn.make_transformer_weights
            self.desc = ("C5: Transformer-base greedy translation (6+6 layers, width 512, 8 heads, feed-forward 2048, "
                         "vocabulary 32000, key / value cache), sources of 16..64 tokens, 64 decode steps")
            self.l2 = "a 256 MB buffer is rewritten between timed steps (one step's weights, 84 MB, would fit the L2)"

    def config(self, total: int, group: int) -> dict:
        return {"workload": self.desc, "streams_total": total, "lockstep_group": group, "max_steps": self.cfg.max_steps,
                "sharding": "streams round-robin over the ranks, no collective on the data path", "l2": self.l2}

    def translator(self, w, group, dev):
        if self.kind == "c4":
            from pimaicompiler_b200.gnmt import GnmtTranslator
            return GnmtTranslator(self.cfg, w, group=group, device=dev)
        from pimaicompiler_b200.transformer import TransformerTranslator
        return TransformerTranslator(self.cfg, w, group=group, device=dev)

    def step_bytes(self, group: int, mean_len: float) -> float:
        """Bytes one decode step of one group has to stream: every decoder matrix once (whatever the group size) plus each
        stream's attention keys and values."""
        c = self.cfg
        if self.kind == "c4":
            H, V = c.hidden, c.vocab
            return 2.0 * (2 * 4 * H * H + 3 * (4 * H * 2 * H + 4 * H * H) + H * H + V * H) + group * 2 * mean_len * H * 2
        d, f, V, nl = c.d_model, c.ffn, c.vocab, c.layers
        weights = 2.0 * (nl * (3 * d * d + d * d + d * d + d * d + 2 * d * f) + V * d)
        kv = group * nl * 2.0 * (mean_len + c.max_steps / 2.0) * d * 2      # cross keys/values + half-full self cache
        return weights + kv

    def cpu_throughput(self, n: int, seed: int):
        """Translates n synthetic streams on the host cores with the libtorch oracle; (streams/s, seconds, cores)."""
        from oracle import torch_oracle as to
        w = self.make_weights(self.cfg, seed=0)
        cores = host_threads()
        torch.set_num_threads(cores)
        seqs = to.make_sentences(n, self.cfg, seed)
        fn = to.gnmt_translate if self.kind == "c4" else to.transformer_translate
        fn(w, seqs[0], self.cfg, 4)
        t0 = time.perf_counter()
        done = 0
        for s_ in seqs:
            fn(w, s_, self.cfg)
            done += 1
            if time.perf_counter() - t0 > CPU_SAMPLE_SECONDS:
                break
        dt = time.perf_counter() - t0
        return done / dt, dt, cores


def run_reference_translate(args, rank, world):
    if rank != 0:
        return
    wl = _Translate(args.workload)
    n = max(1, min(args.cpu_sample, 8 if wl.kind == "c4" else 128))
    vals, secs, cores = [], 0.0, 1
    for k in range(args.steps):
        v, dt, cores = wl.cpu_throughput(n, 9000 + k)
        vals.append(v)
        secs += dt
    value = statistics.median(vals)
    total = args.streams_total or wl.total
    line = {"impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs / max(args.steps, 1) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": wl.config(total, min(args.group or wl.group, (total + args.gpus - 1) // args.gpus)), "sample_streams_per_step": n,
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": cores, "kind": "port",
                             "sample": f"{n} streams per step, libtorch {torch.__version__} CPU fp32, {cores} threads"},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_translate(args, rank, world, local):
    """C4 / C5: the configuration's streams sharded over the ranks; each rank translates its shard in lock-step groups
    (encoder over the padded group, then every greedy step from a CUDA graph).  `value` has the staged token ids resident
    in HBM; `e2e` goes through the translator's translate() with host token lists in and out."""
    from pimaicompiler_b200 import build
    from pimaicompiler_b200 import synthetic as syn
    build.build()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    wl = _Translate(args.workload)
    cfg = wl.cfg
    w = wl.make_weights(cfg, seed=0)
    total = args.streams_total or wl.total
    mine = syn.make_sentences(total, cfg, seed=11)[rank::world]
    S = len(mine)
    group = min(args.group or wl.group, S)
    tr = wl.translator(w, group, dev)
    staged = tr.stage(mine)
    dev_groups = [tr.to_device(g_) for g_ in staged]
    out_tokens = torch.zeros(len(staged), cfg.max_steps, group, dtype=torch.int64, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2

    def step_device(events=None):
        for gi, grp in enumerate(dev_groups):
            tr.encode(grp)
            if events is not None:
                events[gi][0].record()
            toks, _ = tr.decode(cfg.max_steps)
            if events is not None:
                events[gi][1].record()
            out_tokens[gi].copy_(toks)

    for _ in range(max(args.warmup, 3)):
        step_device()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier(world)
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    dec_ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in dev_groups]
              for _ in range(args.steps)]
    for k in range(args.steps):
        flush.fill_(k & 0xff)
        ev[k][0].record()
        step_device(dec_ev[k])
        ev[k][1].record()
    torch.cuda.synchronize()
    barrier(world)
    step_ms = [a.elapsed_time(b) for a, b in ev]
    decode_ms = sum(a.elapsed_time(b) for row in dec_ev for a, b in row)
    total_ms = max_over_ranks(sum(step_ms), world)
    clocks = sampler.stop() if rank == 0 else {}

    for _ in range(2):
        tr.translate(mine)
    barrier(world)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        res = tr.translate(mine)
    e2e_s = max_over_ranks(time.perf_counter() - t0, world)
    barrier(world)

    n_streams = S * world * args.steps
    value = n_streams / (total_ms * 1e-3)
    e2e_value = n_streams / e2e_s
    peak, peak_src = load_peaks()
    mean_len = sum(int(x.shape[0]) for x in mine) / max(S, 1)
    step_bytes = wl.step_bytes(group, mean_len)
    n_steps = len(dev_groups) * cfg.max_steps * args.steps
    achieved = step_bytes * n_steps / (decode_ms * 1e-3) / 1e9 if decode_ms > 0 else 0.0
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:   # timed on rank 0 at N = 1 only: the other ranks would wait
        n_cpu = max(1, min(args.cpu_sample, 8 if wl.kind == "c4" else 128))
        v, dt, cores = wl.cpu_throughput(n_cpu, 9100)
        cpu = {"value": v, "unit": wl.unit, "cores": cores, "kind": "port",
               "sample": f"{n_cpu} synthetic streams of the same distribution, libtorch {torch.__version__} CPU fp32 "
                         f"(the at:: calls of the reference's default executors, one stream at a time), {dt:.1f} s"}
    barrier(world)
    if rank != 0:
        return
    h2d = sum(tr.h2d_bytes(g_) for g_ in staged)
    line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage / f32 accumulate",
            "data": "synthetic", "config": wl.config(S * world, group), "streams_per_gpu": S,
            "us_per_decode_step": decode_ms * 1e3 / max(n_steps, 1), "decode_share_of_step_time": decode_ms / max(sum(step_ms), 1e-9),
            "tokens_checksum": int(sum(sum(t) for t in res) % 1000003),
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": len(staged) * cfg.max_steps * group * 8},
            "gpu_launches": (len(dev_groups) * (cfg.max_steps * tr.launches_per_step + 24)) * args.steps,
            "roofline": {"bound": "hbm", "kernel": f"one decode step of {group} streams ({tr.launches_per_step} launches inside a "
                                                    "CUDA graph: projection GEMMs, attention, vocabulary GEMM, arg max)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                         "traffic": None, "bytes_per_step": step_bytes,
                         "per_stream_equivalent_gbs": achieved * group,
                         "note": "algorithmic bytes = every decoder matrix once per step plus each stream's keys and "
                                 "values; one stream at a time would read the same matrices once per stream"},
            "clocks": clocks}
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c3", choices=["c3", "c2", "c1", "c4", "c5"],
                    help="c3 = RNN-T greedy decode (the headline); c2 = GEMV/GEMM sweep; c1 = single aten::lstm; "
                         "c4 / c5 = GNMT / Transformer greedy translation of 512 / 2048 streams in lock-step groups")
    ap.add_argument("--streams-total", type=int, default=0,
                    help="streams of one step, sharded over the ranks (0 = the configuration's own: 1024 utterances for "
                         "c3, 512 sentences for c4, 2048 sequences for c5)")
    ap.add_argument("--group", type=int, default=0,
                    help="c4 / c5: streams decoded in lock step per group (0 = the rank's whole shard, at most 512 / 2048)")
    ap.add_argument("--streams-per-gpu", type=int, default=0,
                    help="overrides --streams-total with a per-rank count (profiling runs on small cases)")
    ap.add_argument("--streams-per-call", type=int, default=0,
                    help="utterances per decode call (0 = the rank's whole shard in one call: the encoder still advances "
                         "groups of up to 128 utterances, the greedy kernel takes all of them at once)")
    ap.add_argument("--no-extras", action="store_true", help="skip the C1 / C2 figures of the default line")
    ap.add_argument("--c2-shape", default="", help="with --workload c2: only this NxK shape (plus the headline shape), e.g. 4096x1024")
    ap.add_argument("--c2-batches", default="", help="with --c2-shape: the batched-stream sizes to time, e.g. 8,32")
    ap.add_argument("--cpu-sample", type=int, default=64, help="utterances decoded on the CPU per baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--encoder-batch", type=int, default=0, help="utterances per lock-step encoder group (0 = default)")
    args = ap.parse_args()
    if args.workload == "c3" and not args.streams_total:
        args.streams_total = STREAMS_TOTAL
    if args.impl == "reference":
        # CPU arm: rank 0 alone works, the others leave at once; no process group is needed
        ref = {"c4": run_reference_translate, "c5": run_reference_translate}.get(args.workload, run_reference)
        ref(args, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")))
        return
    if args.workload in ("c1", "c2"):
        if int(os.environ.get("RANK", "0")) == 0:
            {"c1": run_c1, "c2": run_c2}[args.workload](args)
        return
    rank, world, local = dist_setup(args.gpus)
    try:
        {"c3": run_gpu, "c4": run_translate, "c5": run_translate}[args.workload](args, rank, world, local)
    finally:
        if world > 1:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
