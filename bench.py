"""Benchmark of the quantized decode hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): configuration 1 of the baseline -- the Q4_K matvec, W 4096x4096 in raw
GGUF Q4_K blocks, x fp32[4096], batch 1 -- repeated over a stack of LAYERS distinct weight
tensors (default 128, 1.2 GB, far larger than the 126 MB L2, so every launch streams its
weights from HBM).  One step = one pass over the stack: LAYERS matvec launches back to back.

  value     GB/s of algorithmic bytes (blocks + x + y per matvec), inputs resident in HBM,
            timed with CUDA events on the launching stream;
  e2e       the same metric through the host-pointer C ABI: a step is one skn_matmul_async per layer (x copied
            from pinned host memory, y copied back to pinned host memory, every layer) and one skn_sync; the
            figure of the blocking call (skn_matmul per layer, a synchronisation per layer) is reported beside
            it as e2e.blocking_call;
  roofline  the streaming matvec kernel against the measured HBM copy bandwidth;
  cpu_baseline  the CPU oracle (a C restatement; the reference's Kotlin cannot run here)
            timed on this host's cores on a bounded sample of the same workload.

With --gpus N > 1 (launched by torchrun, one rank per GPU) every rank streams its own row
shard of an N-times taller stack (column-parallel: rank r owns rows [r*4096, (r+1)*4096) of
each [N*4096, 4096] layer) and the y slices of the whole stack are all-gathered over NCCL once
per step (the layers of this stack are independent of one another);
per-GPU work is fixed, so scaling is weak.

--impl reference times the CPU oracle alone (all host threads) and prints the same line.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_ROWS, N_COLS = 4096, 4096
Q4_K = 12
W_BYTES = N_ROWS * (N_COLS // 256) * 144
ALG_BYTES = W_BYTES + 4 * N_COLS + 4 * N_ROWS      # 9 469 952 per matvec
# dram__bytes_read.sum + dram__bytes_write.sum of one skn_matvec_mma<0, 2, 1, true, 0> launch on this
# workload, from the ncu capture summarised in profiles/q4k_matvec_cfg1.md
DRAM_TRAFFIC_PER_LAUNCH = 9489408
METRIC = "q4k_matvec_gbs"
UNIT = "GB/s"


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [c.strip() for c in r.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(seconds: float = 10.0, threads: int = 0):
    """The CPU restatement on a bounded sample: repeated cfg1 matvecs (fused dequant-dot,
    fp64 accumulate, rows over OpenMP threads) for about `seconds`."""
    from oracle import oracle
    from skainet_b200 import synth
    w, x = synth.cfg1(0)
    cores = threads or (os.cpu_count() or 1)
    oracle.matmul(Q4_K, w, N_ROWS, N_COLS, x, threads=cores)   # warm-up
    reps, t0 = 0, time.perf_counter()
    while True:
        oracle.matmul(Q4_K, w, N_ROWS, N_COLS, x, threads=cores)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or reps >= 2000:
            break
    gbs = reps * ALG_BYTES / dt / 1e9
    return {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{reps} cfg1 matvecs (Q4_K 4096x4096, M=1) in {dt:.1f} s, fused dequant-dot in fp64, "
                      f"OpenMP over rows; the reference's Kotlin has no JVM to run on"}, dt / reps


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    per_step_s = min(3.0, 60.0 / (steps + args.warmup))
    from oracle import oracle
    from skainet_b200 import synth
    w, x = synth.cfg1(0)
    cores = os.cpu_count() or 1
    times = []
    reps_per_step = None
    for it in range(args.warmup + steps):
        reps, t0 = 0, time.perf_counter()
        while True:
            oracle.matmul(Q4_K, w, N_ROWS, N_COLS, x, threads=cores)
            reps += 1
            if (reps_per_step is not None and reps >= reps_per_step) or \
               (reps_per_step is None and time.perf_counter() - t0 >= per_step_s):
                break
        dt = time.perf_counter() - t0
        if reps_per_step is None:
            reps_per_step = reps
        if it >= args.warmup:
            times.append(dt)
    tot = sum(times)
    gbs = steps * reps_per_step * ALG_BYTES / tot / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * tot / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "cfg1: Q4_K matvec 4096x4096, M=1", "sample_matvecs_per_step": reps_per_step},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{reps_per_step} cfg1 matvecs per step on the CPU oracle (C restatement; the "
                                   "reference is Kotlin and has no quantized kernels or JVM here)"},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    import skainet_b200 as skn
    from skainet_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    layers = args.layers
    ctx = skn.Context(local)
    # a stream of our own: handle 0 (the legacy default stream) would mean "the context's own
    # stream" to skn_ctx_set_stream, and the timing events must sit on the launching stream
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    ctx.set_relaxed_order(args.order == "relaxed")

    # Synthetic stack: one seeded cfg1-distribution weight, then `layers` variants of it
    # (bytes rotated per layer) so that each layer is a distinct buffer with the same value
    # distributions, without spending minutes in the host generator.
    g = synth.rng(1000 + rank)
    base = synth.make_weight(g, Q4_K, N_ROWS, N_COLS)
    x_host = torch.from_numpy(synth.make_activations(g, 1, N_COLS)[0].copy()).pin_memory()
    tensors = []
    for i in range(layers):
        wi = np.roll(base, i, axis=0) if i else base
        tensors.append(skn.QuantTensor(ctx, (N_ROWS, N_COLS), Q4_K, wi))
    x_dev = x_host.to(dev)
    y_dev = torch.empty((layers, N_ROWS), dtype=torch.float32, device=dev)
    y_all = torch.empty((world, layers, N_ROWS), dtype=torch.float32, device=dev) if world > 1 else None
    y_host = torch.empty(N_ROWS, dtype=torch.float32).pin_memory()

    def step_device():
        for i, t in enumerate(tensors):
            t.matmul_t_dev(x_dev, 1, y_dev[i])
        if world > 1:
            # the layers of the stack are independent: their y slices are exchanged once per step
            dist.all_gather_into_tensor(y_all, y_dev)

    from skainet_b200 import _ffi
    L = _ffi.lib()
    xh_ptr, yh_ptr = x_host.data_ptr(), y_host.data_ptr()

    def step_e2e_blocking():
        for t in tensors:
            rc = L.skn_matmul(ctx.handle, t.handle, xh_ptr, 1, N_COLS, None, yh_ptr)
            if rc != 0:
                raise RuntimeError(L.skn_last_error(ctx.handle).decode())

    # every layer's result in its own pinned row: nothing is overwritten before the step's synchronisation
    y_host_all = torch.empty((layers, N_ROWS), dtype=torch.float32).pin_memory()
    yh_all_ptr = y_host_all.data_ptr()

    def step_e2e():
        for i, t in enumerate(tensors):
            rc = L.skn_matmul_async(ctx.handle, t.handle, xh_ptr, 1, N_COLS, None, yh_all_ptr + i * 4 * N_ROWS)
            if rc != 0:
                raise RuntimeError(L.skn_last_error(ctx.handle).decode())
        rc = L.skn_sync(ctx.handle)
        if rc != 0:
            raise RuntimeError(L.skn_last_error(ctx.handle).decode())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing --------------------------------------------------------
    # The launch loop of one step is captured once into a CUDA graph (a matvec lasts a few
    # microseconds, less than a host-side launch); the timed region replays the graph.
    step_device()          # first call plans each tensor's launch geometry (not capturable)
    barrier()

    def time_device(order):
        ctx.set_relaxed_order(order == "relaxed")
        graph, run = None, step_device
        if not args.no_graph:
            cap_stream = torch.cuda.Stream()
            cap_stream.wait_stream(stream)
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(cap_stream):
                    ctx.set_stream(cap_stream.cuda_stream)
                    with torch.cuda.graph(graph, stream=cap_stream):
                        step_device()
                run = graph.replay
            except Exception as exc:   # capture unsupported for this configuration: launch eagerly
                sys.stderr.write(f"[bench] CUDA graph capture failed ({exc}); launching eagerly\n")
                graph, run = None, step_device
            finally:
                ctx.set_stream(stream.cuda_stream)
            torch.cuda.synchronize()
        for _ in range(max(3, args.warmup)):
            run()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        barrier()
        ctx.sync()
        t = e0.elapsed_time(e1)
        if world > 1:
            tt = torch.tensor([t], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        return t, graph is not None

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    other = "stream" if args.order == "relaxed" else "relaxed"
    ms_other, _ = time_device(other) if world == 1 else (None, False)
    ms, graphed = time_device(args.order)
    graph = graphed or None

    # ---- end to end through the host-pointer ABI ----------------------------------------
    for _ in range(2):
        step_e2e()
    barrier()
    e2e_steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    step_e2e_blocking()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e_blocking()
    torch.cuda.synchronize()
    e2e_blocking_s = time.perf_counter() - t0
    if world > 1:
        te = torch.tensor([e2e_s, e2e_blocking_s], device=dev)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s, e2e_blocking_s = float(te[0].item()), float(te[1].item())
    clocks = sampler.stop() if rank == 0 else None

    # sanity: results are finite and the same from both paths
    y_chk = y_dev[-1].cpu()
    assert torch.isfinite(y_chk).all()
    assert torch.equal(y_chk, y_host), "device-pointer and host-pointer paths disagree"
    assert torch.equal(y_chk, y_host_all[-1]), "device-pointer and asynchronous host-pointer paths disagree"

    if rank == 0:
        launches_per_step = layers
        total_bytes = world * layers * ALG_BYTES
        value = total_bytes * args.steps / (ms * 1e-3) / 1e9
        e2e_value = total_bytes * e2e_steps / e2e_s / 1e9
        peak, peak_kind = measured_peak()
        per_launch_us = ms * 1e3 / (args.steps * layers)
        achieved = ALG_BYTES / (per_launch_us * 1e-6) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "cfg1: Q4_K matvec 4096x4096, M=1, fp32 x", "layers_per_step": layers,
                       "launch_order": ("relaxed: the layers of a step are independent and declared so "
                                        "(SKN_OPT_RELAXED_ORDER)") if args.order == "relaxed" else
                       "stream order: every launch waits for the previous one",
                       "parallelism": (f"tp{world}" + (", exchange fused into the matvecs" if (args.fused_exchange == "on" or (args.fused_exchange == "auto" and world >= 4)) and B <= 2 else "")) if world > 1 else "none",
                   "launch": "CUDA graph replay of one step" if graph is not None else "eager launches",
                       "l2_policy": f"inputs larger than L2: {layers} distinct weights = "
                                    f"{layers * W_BYTES / 1e6:.0f} MB streamed per step",
                       "sharding": "none" if world == 1 else
                       f"column-parallel rows over {world} ranks, one NCCL all-gather of the y slices per step",
                       "pct_of_8TBs": 100.0 * value / world / 8000.0,
                       "other_order": None if ms_other is None else
                       {"order": other, "value": total_bytes * args.steps / (ms_other * 1e-3) / 1e9, "unit": UNIT}},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": layers * 4 * N_COLS,
                    "d2h_bytes_per_step": layers * 4 * N_ROWS, "steps": e2e_steps,
                    "api": "per step: skn_matmul_async for every layer (pinned host x in, pinned host y out), then skn_sync",
                    "blocking_call": {"value": total_bytes * e2e_steps / e2e_blocking_s / 1e9, "unit": UNIT,
                                      "api": "skn_matmul per layer (returns with y in host memory)"}},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "kernel": "skn_matvec_mma<0, 2, 1, true, 0>", "achieved": achieved,
                         "peak": peak, "peak_kind": peak_kind, "unit": UNIT, "frac": achieved / peak,
                         "us_per_launch": per_launch_us, "traffic": DRAM_TRAFFIC_PER_LAUNCH},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            cb, _ = cpu_baseline(args.cpu_seconds)
            line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)

    for t in tensors:
        t.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# Secondary workloads (not the headline line): --workload ffn | attn | sweep.  Single GPU.
# --------------------------------------------------------------------------------------------
def _events_ms(torch, stream, fn, steps, warmup):
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_ffn(args):
    """Config 3: SwiGLU FFN prefill, X fp32 [512,4096], W_gate/W_up 14336x4096 Q4_K, W_down
    4096x14336 Q6_K, on the tensor cores.  Inputs (229 MB of weights + activations) exceed L2."""
    import torch
    import skainet_b200 as skn
    from skainet_b200 import _ffi, synth
    M, K, F = 512, 4096, 14336
    dev = torch.device("cuda", 0)
    ctx = skn.Context(0)
    # a stream of our own: handle 0 (the legacy default stream) would mean "the context's own
    # stream" to skn_ctx_set_stream, and the timing events must sit on the launching stream
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    g = synth.rng(2)
    x = torch.from_numpy(synth.make_activations(g, M, K)).to(dev)
    base = synth.make_weight(g, 12, F, K)
    wg = skn.QuantTensor(ctx, (F, K), 12, base)
    wu = skn.QuantTensor(ctx, (F, K), 12, np.roll(base, 1, axis=0))
    wd = skn.QuantTensor(ctx, (K, F), 14, synth.make_weight(g, 14, K, F))
    y = torch.empty((M, K), dtype=torch.float32, device=dev)
    L = _ffi.lib()

    def step():
        rc = L.skn_ffn_swiglu_dev(ctx.handle, wg.handle, wu.handle, wd.handle, x.data_ptr(), M, y.data_ptr())
        assert rc == 0, L.skn_last_error(ctx.handle)

    sampler = ClockSampler(0)
    sampler.start()
    ms = _events_ms(torch, stream, step, args.steps, args.warmup)
    clocks = sampler.stop()
    ctx.sync()
    flops = 3 * 2 * M * K * F
    tfl = flops / (ms * 1e-3) / 1e12
    peak = 1672.7
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    print(json.dumps({
        "metric": "ffn_prefill_tflops", "value": tfl, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg3: SwiGLU FFN prefill M=512, 4096 -> 14336 (Q4_K gate/up) -> 4096 (Q6_K down)",
                   "tokens_per_s": M / (ms * 1e-3)},
        "gpu_launches": 3 * args.steps,
        "roofline": {"bound": "tensor", "kernel": "skn_matmul_tc_kernel", "achieved": tfl, "peak": peak,
                     "peak_kind": "measured burst", "unit": "TFLOP/s", "frac": tfl / peak, "traffic": None},
        "clocks": clocks}), flush=True)


def run_attn(args):
    """Config 4: decode attention, 32 query / 8 kv heads, head_dim 128, batch 8, fp32 cache
    pre-filled (lengths uniform 1024..4096); a step appends one token and attends.  The
    cache (1.1 GB) exceeds L2."""
    import torch
    import skainet_b200 as skn
    from skainet_b200 import _ffi, synth
    B, Hq, Hkv, D, T = 8, 32, 8, 128, 4096
    steps = min(args.steps, 128)
    cap = T + 128 + 8
    dev = torch.device("cuda", 0)
    ctx = skn.Context(0)
    # a stream of our own: handle 0 (the legacy default stream) would mean "the context's own
    # stream" to skn_ctx_set_stream, and the timing events must sit on the launching stream
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    g = synth.rng(3)
    kv = skn.KVCache(ctx, B, Hkv, D, cap, dtype=args.kv_dtype)
    eb = 2 if args.kv_dtype == "f16" else 4             # bytes per cached element
    lens = g.integers(1024, 4097, size=B).astype(np.int32)
    kc = g.standard_normal((B, Hkv, T, D), dtype=np.float32)
    kv.load(kc, kc[:, ::-1].copy(), lens)
    q = torch.randn((B, Hq, D), device=dev)
    kn = torch.randn((B, Hkv, D), device=dev)
    out = torch.empty_like(q)
    L = _ffi.lib()
    scale = 1.0 / float(np.sqrt(D))

    def step():
        assert L.skn_kv_append_dev(kv.handle, kn.data_ptr(), kn.data_ptr()) == 0
        assert L.skn_attn_decode_dev(kv.handle, q.data_ptr(), Hq, scale, out.data_ptr(), None) == 0

    warm = 3
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # bytes: K and V of every cached token of every kv head, mean length over the timed steps
    mean_len = float(lens.mean()) + warm + (steps + 1) / 2.0
    alg = B * mean_len * Hkv * D * eb * 2 + B * Hkv * D * 4 * 2 + 2 * B * Hq * D * 4
    gbs = alg / (ms * 1e-3) / 1e9
    peak, kind = measured_peak()
    print(json.dumps({
        "metric": "attn_decode_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg4: GQA decode attention B=8, 32q/8kv heads, D=128, ctx 1024..4096 (+1 per step)",
                   "kv_cache": args.kv_dtype + (" (the configuration's cache)" if args.kv_dtype == "f32" else
                                                " (beyond the configuration: K and V rounded to fp16 once, arithmetic fp32)"),
                   "mean_len": mean_len, "steps_per_s": 1e3 / ms},
        "gpu_launches": 3 * steps,
        "roofline": {"bound": "hbm", "kernel": "skn_attn_stream_kernel + merge + append", "achieved": gbs, "peak": peak, "peak_kind": kind,
                     "unit": "GB/s", "frac": gbs / peak, "traffic": None}}), flush=True)


def run_sweep(args):
    """Config 2 (and the Q4_K / Q6_K analogues): matvec / small-batch matmul GB/s per type,
    shape and M.  Each case cycles over enough distinct weights to exceed L2."""
    import torch
    import skainet_b200 as skn
    from skainet_b200 import synth
    dev = torch.device("cuda", 0)
    ctx = skn.Context(0)
    # a stream of our own: handle 0 (the legacy default stream) would mean "the context's own
    # stream" to skn_ctx_set_stream, and the timing events must sit on the launching stream
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    ctx.set_relaxed_order(args.order == "relaxed")
    g = synth.rng(1)
    rows = []
    for qt in (2, 8, 12, 14):
        e, bb = synth.GEOMETRY[qt]
        for (N, K) in ((4096, 4096), (14336, 4096), (4096, 14336)):
            wbytes = N * K // e * bb
            nl = max(2, int(400e6 // wbytes) + 1)
            base = synth.make_weight(g, qt, N, K)
            ts = [skn.QuantTensor(ctx, (N, K), qt, np.roll(base, i, axis=0)) for i in range(nl)]
            for M in (1, 4, 16, 64):
                x = torch.randn((M, K), device=dev)
                y = torch.empty((nl, M, N), device=dev)

                def step():
                    for i, t in enumerate(ts):
                        t.matmul_t_dev(x, M, y[i])
                reps = 3 if M >= 16 else 5
                ms = _events_ms(torch, stream, step, reps, 3) / nl
                alg = wbytes + 4 * M * (K + N)
                rows.append({"type": synth.TYPE_NAMES[qt], "N": N, "K": K, "M": M, "us": ms * 1e3,
                             "gbs": alg / (ms * 1e-3) / 1e9, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12})
            for t in ts:
                t.close()
    peak, kind = measured_peak()
    print(json.dumps({"metric": "matvec_sweep_gbs", "unit": "GB/s", "n_gpus": 1, "data": "synthetic",
                      "config": {"workload": "cfg2 sweep over types, shapes, M", "order": args.order},
                      "peak": peak, "peak_kind": kind, "cases": rows}), flush=True)


def run_decode(args):
    """Configuration 5: Llama-style decoder, 32 layers, d_model 4096, FFN 14336, 32q/8kv heads,
    head_dim 128, vocab 32000, Q4_K projections, Q6_K embedding / LM head.  512-token prefill of
    uniform-random ids, then 128 greedy decode steps (ids fed back on the device, one CUDA graph
    replay per step).  One layer's random blocks are uploaded 32 times (distinct device buffers).
    4 GB of weights per step far exceed L2.

    Under torchrun (WORLD_SIZE > 1) the decoder is tensor-parallel: every rank keeps its share of
    the heads, FFN columns and vocabulary and the partial products meet in the library's own
    exchange (two per layer); the step time is the maximum over the ranks ("strong" scaling:
    the model and batch are fixed)."""
    import torch
    import torch.distributed as dist
    import skainet_b200 as skn
    from skainet_b200 import synth
    from skainet_b200.llama import LlamaConfig, LlamaDecoder
    from skainet_b200.parallel import Exchange
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    B, T, steps = args.batch, 512, min(args.steps, 128)
    cfg = LlamaConfig(n_layers=args.layers if args.layers != 128 else 32)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = skn.Context(local)
    exchange = Exchange.connect_processes(ctx, B * T * cfg.d_model) if world > 1 else None
    ctx.set_fused_exchange({"auto": None, "on": True, "off": False}[args.fused_exchange])
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    g = synth.rng(4)
    qd, kd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    shapes = {"wq": (qd, cfg.d_model), "wk": (kd, cfg.d_model), "wv": (kd, cfg.d_model), "wo": (cfg.d_model, qd),
              "w_gate": (cfg.ffn_dim, cfg.d_model), "w_up": (cfg.ffn_dim, cfg.d_model), "w_down": (cfg.d_model, cfg.ffn_dim)}
    layer = {k: synth.make_weight(g, cfg.proj_type, *shp) for k, shp in shapes.items()}
    emb = synth.make_weight(g, cfg.head_type, cfg.vocab, cfg.d_model)
    dec = LlamaDecoder(ctx, cfg, batch=B, max_tokens=T, max_ctx=T + 136, exchange=exchange, kv_dtype=args.kv_dtype)
    ones = np.ones(cfg.d_model, dtype=np.float32)
    for i in range(cfg.n_layers):
        dec.set_layer(i, layer, ones, ones)
    dec.set_head(emb, ones, np.roll(emb, 1, axis=0))
    prompt = torch.from_numpy(g.integers(0, cfg.vocab, size=(B, T)).astype(np.int32)).to(dev)

    def prefill():
        dec.reset()
        dec.forward_dev(prompt, T)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    prefill()
    dec.forward_dev(None, 1)          # sizes every scratch buffer of the decode path
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    prefill()
    e1.record(stream)
    barrier()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1))
    graph = None
    if not args.no_graph:
        try:
            cap = torch.cuda.Stream()
            cap.wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(cap):
                ctx.set_stream(cap.cuda_stream)
                with torch.cuda.graph(graph, stream=cap):
                    dec.forward_dev(None, 1)
        except Exception as exc:
            sys.stderr.write(f"[bench] CUDA graph capture failed ({exc}); launching eagerly\n")
            graph = None
        finally:
            ctx.set_stream(stream.cuda_stream)
        torch.cuda.synchronize()
    # the capture itself advanced the host-side position by one: start over
    prefill()
    step = graph.replay if graph is not None else (lambda: dec.forward_dev(None, 1))
    for _ in range(3):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1) / steps)
    ctx.sync()
    if rank != 0:
        dec.close()
        if world > 1:
            dist.destroy_process_group()
        return
    wbytes = cfg.n_layers * sum(n * (k // 256) * 144 for n, k in shapes.values()) + cfg.vocab * (cfg.d_model // 256) * 210
    peak, kind = measured_peak()
    gbs = wbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "decode_tok_s", "value": B * 1e3 / ms, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": 3,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"cfg5: Llama-style decoder, {cfg.n_layers} layers, Q4_K / Q6_K, batch {B}, "
                               f"{T}-token prefill then greedy decode",
                   "parallelism": (f"tp{world}" + (", exchange fused into the matvecs" if (args.fused_exchange == "on" or (args.fused_exchange == "auto" and world >= 4)) and B <= 2 else "")) if world > 1 else "none",
                   "launch": "CUDA graph replay of one step" if graph is not None else "eager launches",
                   "prefill_ms": prefill_ms, "prefill_tok_s": B * T * 1e3 / prefill_ms,
                   "kv_cache": args.kv_dtype, "weight_bytes_per_step": wbytes},
        "roofline": {"bound": "hbm", "kernel": "decode step (weight stream, all GPUs)", "achieved": gbs, "peak": peak * world,
                     "peak_kind": kind, "unit": "GB/s", "frac": gbs / (peak * world), "traffic": None},
        "clocks": clocks}), flush=True)
    dec.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=128)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--order", default="relaxed", choices=["relaxed", "stream"],
                    help="relaxed: the layers of a step are declared independent (SKN_OPT_RELAXED_ORDER) and "
                         "may overlap; stream: each launch waits for the one before it")
    ap.add_argument("--batch", type=int, default=1, help="decode workload: sequences per step")
    ap.add_argument("--kv-dtype", default="f32", choices=["f32", "f16"],
                    help="attn / decode workloads: element type of the KV cache (f32 is what the configurations specify)")
    ap.add_argument("--fused-exchange", default="auto", choices=["auto", "on", "off"],
                    help="tensor-parallel decode: push partial sums from the matvec epilogue (SKN_OPT_FUSED_EXCHANGE); "
                         "auto = on from four ranks")
    ap.add_argument("--workload", default="matvec", choices=["matvec", "ffn", "attn", "sweep", "decode"],
                    help="matvec is the headline line; the others print one secondary JSON line (1 GPU)")
    args = ap.parse_args()
    if args.impl == "ours" and args.workload != "matvec":
        return {"ffn": run_ffn, "attn": run_attn, "sweep": run_sweep, "decode": run_decode}[args.workload](args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
