"""Benchmark of the quantized decode hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): configuration 1 of the baseline -- the Q4_K matvec, W 4096x4096 in raw
GGUF Q4_K blocks, x fp32[4096], batch 1 -- repeated over a stack of LAYERS distinct weight
tensors (default 128, 1.2 GB, far larger than the 126 MB L2, so every launch streams its
weights from HBM), every layer with an x of its own.  One pass = LAYERS matvec launches back to
back; one step = PASSES passes (default 80, so that the K timed steps last about half a second
and the sampled clocks describe a sustained run).

  value     GB/s of algorithmic bytes (blocks + x + y per matvec), inputs resident in HBM,
            timed with CUDA events on the launching stream;
  e2e       the same metric through the host-pointer C ABI: a pass is one skn_matmul_async per layer (x copied
            from pinned host memory, y copied back to pinned host memory, every layer) and one skn_sync; the
            figure of the blocking call (skn_matmul per layer, a synchronisation per layer) is reported beside
            it as e2e.blocking_call;
  roofline  the matvec kernel against the measured HBM copy bandwidth;
  decode    configuration 5 (Llama-style decoder, tok/s at batch 1 and 16) on the same ranks,
            tensor-parallel through the library's own exchange when N > 1 (strong scaling); the legs
            run under a deadline (--decode-deadline): a leg that fails or does not finish is reported
            in its place and never costs the line;
  cpu_baseline  the CPU oracle (a C restatement; the reference's Kotlin cannot run here)
            timed on this host's cores on a bounded sample of the same workload.

With --gpus N > 1 (launched by torchrun, one rank per GPU) every rank streams its own row
shard of an N-times taller stack (column-parallel: rank r owns rows [r*4096, (r+1)*4096) of
each [N*4096, 4096] layer) and the y slices of every pass are all-gathered over NCCL beside the
matvecs of the next pass (the layers of this stack are independent of one another);
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the matvec kernel on this workload (one ncu
# capture of a 16-layer stack, 151 MB of weights)
DRAM_TRAFFIC_PER_LAUNCH = 9495040
KERNEL_NAME = "skn_matvec_mma<0, 2, 1, true, 0>"
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


def workload_config(world: int, layers: int) -> dict:
    """The `config` object both arms print: what is computed, never how."""
    return {
        "workload": "cfg1: Q4_K matvec 4096x4096, M=1, fp32 x",
        "layers_per_pass": layers,
        "l2_policy": f"inputs larger than the last-level cache: {layers} distinct weights = "
                     f"{layers * W_BYTES / 1e6:.0f} MB streamed per pass over the stack",
        "sharding": "none" if world == 1 else
        f"column-parallel rows over {world} ranks, the y slices of a pass all-gathered over NCCL",
    }


def _stack_host(layers: int, seed: int):
    """One seeded cfg1-distribution weight and `layers` variants of it (rows rotated per layer): distinct
    buffers with the same value distributions without minutes in the host generator; one x per layer."""
    from skainet_b200 import synth
    g = synth.rng(seed)
    base = synth.make_weight(g, Q4_K, N_ROWS, N_COLS)
    xs = synth.make_activations(g, layers, N_COLS)
    return base, xs


def cpu_baseline(seconds: float = 10.0, threads: int = 0, layers: int = 128):
    """The CPU restatement on a bounded sample of the bench workload: passes over the stack of distinct
    weights (fused dequant-dot, fp64 accumulate, rows over OpenMP threads) for about `seconds`, and beside
    it the reference-faithful single-thread form (fp64 weights, a transposed copy per call, k-outer loops:
    DoublesTensor.kt:362-387 + :255-264) on a few matvecs."""
    from oracle import oracle
    base, xs = _stack_host(min(layers, 16), 1000)
    ws = [np.roll(base, i, axis=0) if i else base for i in range(min(layers, 16))]
    cores = threads or (os.cpu_count() or 1)
    oracle.matmul(Q4_K, ws[0], N_ROWS, N_COLS, xs[0], threads=cores)   # warm-up
    reps, t0 = 0, time.perf_counter()
    while True:
        i = reps % len(ws)
        oracle.matmul(Q4_K, ws[i], N_ROWS, N_COLS, xs[i], threads=cores)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or reps >= 4000:
            break
    gbs = reps * ALG_BYTES / dt / 1e9
    # B1: what the reference's own Linear.forward would cost on these weights held as fp64
    w64 = oracle.dequant_f64(Q4_K, ws[0], N_ROWS, N_COLS)
    b1_reps, t1 = 0, time.perf_counter()
    while b1_reps < 3 and (b1_reps == 0 or time.perf_counter() - t1 < 6.0):
        oracle.linear_ref(Q4_K, ws[0], N_ROWS, N_COLS, xs[0], W64=w64)
        b1_reps += 1
    b1_dt = (time.perf_counter() - t1) / b1_reps
    return {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{reps} cfg1 matvecs over {len(ws)} distinct weights in {dt:.1f} s, fused dequant-dot in fp64, "
                      f"OpenMP over rows; the reference's Kotlin has no JVM to run on",
            "reference_faithful_single_thread": {
                "value": ALG_BYTES / b1_dt / 1e9, "unit": UNIT, "cores": 1, "ms_per_matvec": 1e3 * b1_dt,
                "sample": f"{b1_reps} matvecs: fp64 weights, per-call transposed copy and k-outer loops "
                          "(DoublesTensor.kt:362-387, :255-264); GB/s counts the same Q4_K algorithmic bytes"}}, dt / reps


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    per_step_s = min(3.0, 60.0 / (steps + args.warmup))
    from oracle import oracle
    nw = min(args.layers, 16)
    base, xs = _stack_host(nw, 1000)
    ws = [np.roll(base, i, axis=0) if i else base for i in range(nw)]
    cores = os.cpu_count() or 1
    times = []
    reps_per_step = None
    k = 0
    for it in range(args.warmup + steps):
        reps, t0 = 0, time.perf_counter()
        while True:
            oracle.matmul(Q4_K, ws[k % nw], N_ROWS, N_COLS, xs[k % nw], threads=cores)
            reps += 1
            k += 1
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
        "config": workload_config(world, args.layers),
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{reps_per_step} cfg1 matvecs per step over {nw} distinct weights on the CPU oracle "
                                   "(C restatement, OpenMP over rows; the reference is Kotlin and has no quantized "
                                   "kernels or JVM here)"},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


DECODE_WORKLOAD = ("cfg5: Llama-style decoder, 32 layers, Q4_K projections, Q6_K embedding / LM head, "
                   "512-token prefill then greedy decode, batch 1 and batch 16")


def _decode_object(legs: dict) -> dict:
    out = dict(legs)
    out["tok_s"] = out.get("batch1", {}).get("tok_s")
    out["unit"] = "tok/s"
    out["scaling"] = "strong"
    out["workload"] = DECODE_WORKLOAD
    return out


def guarded_decode_legs(run_leg, batches, deadline_s: float, on_give_up, on_leg_failed=None) -> dict:
    """The `decode` object of the line: run_leg(B) for every batch size, a failed leg replaced by its error.
    Ranks that fall out of step inside a leg (one raises, the others sit in a collective) would wait for one
    another for ever, so every rank carries the same deadline: when it passes, on_give_up(decode object with
    the legs finished so far, the others marked unfinished) is called from a timer thread; the bench prints
    the headline line from there and leaves the process."""
    legs: dict = {}
    lock = threading.Lock()
    state = {"done": False}

    def expire():
        with lock:
            if state["done"]:
                return
            state["done"] = True
            partial = dict(legs)
        for B in batches:
            partial.setdefault(f"batch{B}", {"error": f"not finished within {deadline_s:.0f} s"})
        on_give_up(_decode_object(partial))

    timer = threading.Timer(deadline_s, expire)
    timer.daemon = True
    timer.start()
    try:
        for B in batches:
            try:
                r = run_leg(B)
            except Exception as exc:      # the headline line must survive a failure of the secondary leg
                r = {"error": f"{type(exc).__name__}: {exc}"[:300]}
                if on_leg_failed is not None:
                    on_leg_failed()
            with lock:
                if state["done"]:
                    break
                legs[f"batch{B}"] = r
    finally:
        timer.cancel()
        with lock:
            state["done"] = True
    return _decode_object(legs)


def decode_parallelism(world: int, fused_exchange: str, batch: int) -> str:
    """How the decoder is spread over the ranks, as the bench line words it."""
    if world <= 1:
        return "none"
    fused = fused_exchange == "on" and batch <= 2          # (automatic = off in the library)
    return f"tp{world}" + (", exchange fused into the matvecs" if fused else "")


def make_line(*, world, steps, warmup, layers, passes, order, ms, ms_other, graphed, e2e_s, e2e_blocking_s,
              e2e_steps, e2e_passes, clocks, peak, peak_kind, decode=None, cpu=None) -> dict:
    """The headline JSON line from the measured times (pure: no device, no clock).  ms / ms_other: the
    timed region of `steps` steps in the chosen / the other launch order, each step = `passes` passes over
    the stack of `layers` weights; e2e_s / e2e_blocking_s: wall time of e2e_steps steps of e2e_passes passes
    through the host-pointer calls."""
    launches_per_step = layers * passes
    total_bytes = world * layers * passes * ALG_BYTES            # per step, all ranks
    value = total_bytes * steps / (ms * 1e-3) / 1e9
    per_launch_us = ms * 1e3 / (steps * launches_per_step)
    achieved = ALG_BYTES / (per_launch_us * 1e-6) / 1e9
    e2e_bytes = world * layers * e2e_passes * ALG_BYTES * e2e_steps
    other = "stream" if order == "relaxed" else "relaxed"
    sm_mhz = (clocks or {}).get("sm_mhz")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(world, layers),
        "detail": {
            "passes_per_step": passes, "launches_per_step": launches_per_step, "timed_region_s": ms * 1e-3,
            "launch_order": ("relaxed: the layers of a pass are independent and declared so "
                             "(SKN_OPT_RELAXED_ORDER)") if order == "relaxed" else
            "stream order: every launch waits for the previous one",
            "launch": "CUDA graph replay of one pass" if graphed else "eager launches",
            "exchange": "none" if world == 1 else "the all-gather of pass p runs beside the matvecs of pass p + 1",
            "pct_of_8TBs": 100.0 * value / world / 8000.0,
            "us_per_launch_x_sm_mhz": None if not sm_mhz else per_launch_us * sm_mhz,
            "other_order": None if ms_other is None else
            {"order": other, "value": total_bytes * steps / (ms_other * 1e-3) / 1e9, "unit": UNIT},
        },
        "e2e": {"value": e2e_bytes / e2e_s / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": layers * e2e_passes * 4 * N_COLS,
                "d2h_bytes_per_step": layers * e2e_passes * 4 * N_ROWS, "steps": e2e_steps, "passes_per_step": e2e_passes,
                "api": "per pass: skn_matmul_async for every layer (its own pinned host x in, pinned host y out), "
                       "then skn_sync",
                "blocking_call": {"value": e2e_bytes / e2e_blocking_s / 1e9, "unit": UNIT,
                                  "api": "skn_matmul per layer (returns with y in host memory)"}},
        "gpu_launches": launches_per_step * steps,
        "roofline": {"bound": "hbm", "kernel": KERNEL_NAME, "achieved": achieved,
                     "peak": peak, "peak_kind": peak_kind, "unit": UNIT, "frac": achieved / peak,
                     "us_per_launch": per_launch_us, "traffic": DRAM_TRAFFIC_PER_LAUNCH},
        "clocks": clocks,
    }
    if decode is not None:
        line["decode"] = decode
    if cpu is not None:
        line["cpu_baseline"] = cpu
    return line


def run_ours(args):
    import torch
    import torch.distributed as dist

    import skainet_b200 as skn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    layers, passes = args.layers, max(1, args.passes)
    ctx = skn.Context(local)
    # a stream of our own: handle 0 (the legacy default stream) would mean "the context's own
    # stream" to skn_ctx_set_stream, and the timing events must sit on the launching stream
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    ctx.set_relaxed_order(args.order == "relaxed")

    base, xs = _stack_host(layers, 1000 + rank)
    x_host = torch.from_numpy(xs.copy()).pin_memory()               # [layers][K]: every layer has its own x
    tensors = []
    for i in range(layers):
        wi = np.roll(base, i, axis=0) if i else base
        tensors.append(skn.QuantTensor(ctx, (N_ROWS, N_COLS), Q4_K, wi))
    x_dev = x_host.to(dev)
    # two result buffers: while pass p writes one, the other (pass p - 1) is all-gathered
    y_dev = [torch.empty((layers, N_ROWS), dtype=torch.float32, device=dev) for _ in range(2 if world > 1 else 1)]
    y_all = torch.empty((world, layers, N_ROWS), dtype=torch.float32, device=dev) if world > 1 else None
    y_host = torch.empty((layers, N_ROWS), dtype=torch.float32).pin_memory()

    def pass_device(which=0):
        for i, t in enumerate(tensors):
            t.matmul_t_dev(x_dev[i], 1, y_dev[which][i])

    from skainet_b200 import _ffi
    L = _ffi.lib()
    xh_ptr, yh_ptr = x_host.data_ptr(), y_host.data_ptr()

    def check(rc):
        if rc != 0:
            raise RuntimeError(L.skn_last_error(ctx.handle).decode())

    def pass_e2e_blocking():
        for i, t in enumerate(tensors):
            check(L.skn_matmul(ctx.handle, t.handle, xh_ptr + i * 4 * N_COLS, 1, N_COLS, None, yh_ptr + i * 4 * N_ROWS))

    def pass_e2e():
        for i, t in enumerate(tensors):
            check(L.skn_matmul_async(ctx.handle, t.handle, xh_ptr + i * 4 * N_COLS, 1, N_COLS, None, yh_ptr + i * 4 * N_ROWS))
        check(L.skn_sync(ctx.handle))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing --------------------------------------------------------
    # The launch loop of one pass is captured once into a CUDA graph (a matvec lasts a few
    # microseconds, less than a host-side launch); a step replays it `passes` times.  With several ranks
    # there are two graphs: each forks a side stream that all-gathers the buffer the previous pass wrote.
    pass_device(0)          # first call plans each tensor's launch geometry (not capturable)
    barrier()
    side = torch.cuda.Stream() if world > 1 else None

    def pass_with_exchange(which):
        if world > 1:
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                dist.all_gather_into_tensor(y_all, y_dev[1 - which])
        pass_device(which)
        if world > 1:
            torch.cuda.current_stream().wait_stream(side)

    def time_device(order):
        ctx.set_relaxed_order(order == "relaxed")
        graphs, runs = [], [lambda: pass_with_exchange(0), lambda: pass_with_exchange(1)]
        if not args.no_graph:
            cap_stream = torch.cuda.Stream()
            cap_stream.wait_stream(stream)
            try:
                with torch.cuda.stream(cap_stream):
                    ctx.set_stream(cap_stream.cuda_stream)
                    for which in range(len(y_dev)):
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g, stream=cap_stream):
                            pass_with_exchange(which)
                        graphs.append(g)
                runs = [g.replay for g in graphs]
            except Exception as exc:   # capture unsupported for this configuration: launch eagerly
                sys.stderr.write(f"[bench] CUDA graph capture failed ({exc}); launching eagerly\n")
                graphs = []
            finally:
                ctx.set_stream(stream.cuda_stream)
            torch.cuda.synchronize()
        nrun = len(runs) if world > 1 else 1

        def step():
            for p in range(passes):
                runs[p % nrun]()
        for _ in range(max(3, args.warmup)):
            step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        ctx.sync()
        t = e0.elapsed_time(e1)
        if world > 1:
            tt = torch.tensor([t], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        return t, bool(graphs)

    sampler = ClockSampler(local)
    other = "stream" if args.order == "relaxed" else "relaxed"
    ms_other, _ = time_device(other) if world == 1 else (None, False)
    if rank == 0:
        sampler.start()
    ms, graphed = time_device(args.order)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the host-pointer ABI ----------------------------------------
    # relaxed order stays on, as in the device-timed region: the library keeps each call's own
    # fetch -> product chain in order, only the calls are independent of one another
    e2e_passes = max(1, min(passes, args.e2e_passes))
    e2e_steps = max(1, min(args.steps, 5))
    for _ in range(2):
        pass_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps * e2e_passes):
        pass_e2e()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    y_async = y_host.clone()
    y_host.zero_()
    pass_e2e_blocking()
    t0 = time.perf_counter()
    for _ in range(e2e_steps * e2e_passes):
        pass_e2e_blocking()
    torch.cuda.synchronize()
    e2e_blocking_s = time.perf_counter() - t0
    if world > 1:
        te = torch.tensor([e2e_s, e2e_blocking_s], device=dev)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s, e2e_blocking_s = float(te[0].item()), float(te[1].item())

    # sanity: every layer's result is finite and the same from all three paths
    ctx.set_relaxed_order(False)
    pass_device(0)
    ctx.sync()
    y_chk = y_dev[0].cpu()
    assert torch.isfinite(y_chk).all()
    assert torch.equal(y_chk, y_host), "device-pointer and host-pointer paths disagree"
    assert torch.equal(y_chk, y_async), "device-pointer and asynchronous host-pointer paths disagree"
    assert not torch.equal(y_chk[0], y_chk[1])

    for t in tensors:
        t.close()
    tensors = []
    del x_dev, y_dev, y_all
    torch.cuda.empty_cache()

    # ---- the line without its decode object: what a stuck decode leg must not cost -----------------
    def build_line(decode):
        peak, peak_kind = measured_peak()
        cpu = None
        if world == 1 and not args.no_cpu:
            cpu, _ = cpu_baseline(args.cpu_seconds, layers=layers)
        return make_line(world=world, steps=args.steps, warmup=max(3, args.warmup), layers=layers, passes=passes,
                         order=args.order, ms=ms, ms_other=ms_other, graphed=graphed, e2e_s=e2e_s,
                         e2e_blocking_s=e2e_blocking_s, e2e_steps=e2e_steps, e2e_passes=e2e_passes, clocks=clocks,
                         peak=peak, peak_kind=peak_kind, decode=decode, cpu=cpu)

    # ---- the decoder of configuration 5 on the same ranks (tok/s, strong scaling) ------------
    decode = None
    if not args.no_decode:
        def leg(B):
            return decode_measure(args, ctx, stream, world, rank, local, B, min(args.decode_steps, 128))

        def leg_failed():
            torch.cuda.synchronize()

        def give_up(partial):
            # (timer thread: the main thread may sit in a collective for good)
            if rank == 0:
                saved = args.no_cpu
                args.no_cpu = True               # no CPU leg from here
                print(json.dumps(build_line(partial)), flush=True)
                args.no_cpu = saved
            os._exit(0)

        decode = guarded_decode_legs(leg, (1, 16), args.decode_deadline, give_up, leg_failed)

    if rank == 0:
        print(json.dumps(build_line(decode)), flush=True)

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
    eb = {"f32": 4, "f16": 2, "q8_0": 1.0625}[args.kv_dtype]             # bytes per cached element
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
                   "kv_cache": args.kv_dtype + {"f32": " (the configuration's cache)",
                                                "f16": " (beyond the configuration: K and V rounded to fp16 once, arithmetic fp32)",
                                                "q8_0": " (beyond the configuration: K and V in Q8_0-style blocks, arithmetic fp32)"}[args.kv_dtype],
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


def decode_measure(args, ctx, stream, world, rank, local, B, steps, n_layers=None):
    """Configuration 5 on the ranks of this job: 512-token prefill of uniform-random ids, then `steps`
    greedy decode steps (ids fed back on the device, one CUDA graph replay per step).  One layer's random
    blocks are uploaded n_layers times (distinct device buffers; 4 GB of weights per step far exceed L2).
    With several ranks the decoder is tensor-parallel through the library's own exchange (skn_comm_*);
    times are the maximum over the ranks.  Returns a dict (the same on every rank)."""
    import torch
    import torch.distributed as dist
    from skainet_b200 import synth
    from skainet_b200.llama import LlamaConfig, LlamaDecoder
    from skainet_b200.parallel import Exchange
    T = 512
    cfg = LlamaConfig(n_layers=n_layers or args.decode_layers)
    dev = torch.device("cuda", local)
    exchange = Exchange.connect_processes(ctx, B * T * cfg.d_model) if world > 1 else None
    ctx.set_fused_exchange({"auto": None, "on": True, "off": False}[args.fused_exchange])
    ctx.set_relaxed_order(False)
    g = synth.rng(4)
    qd, kd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    shapes = {"wq": (qd, cfg.d_model), "wk": (kd, cfg.d_model), "wv": (kd, cfg.d_model), "wo": (cfg.d_model, qd),
              "w_gate": (cfg.ffn_dim, cfg.d_model), "w_up": (cfg.ffn_dim, cfg.d_model), "w_down": (cfg.d_model, cfg.ffn_dim)}
    layer = {k: synth.make_weight(g, cfg.proj_type, *shp) for k, shp in shapes.items()}
    emb = synth.make_weight(g, cfg.head_type, cfg.vocab, cfg.d_model)
    dec = LlamaDecoder(ctx, cfg, batch=B, max_tokens=T, max_ctx=T + 136, exchange=exchange, kv_dtype=args.kv_dtype)
    try:
        ones = np.ones(cfg.d_model, dtype=np.float32)
        for i in range(cfg.n_layers):
            dec.set_layer(i, layer, ones, ones)
        dec.set_head(emb, ones, np.roll(emb, 1, axis=0))
        prompt = torch.from_numpy(g.integers(0, cfg.vocab, size=(B, T)).astype(np.int32)).to(dev)
        if world > 1:
            # the ranks finish their uploads seconds apart: they enter the first exchange together, and the bound of
            # the exchange waits is far above any skew that remains (a wait that runs out on one rank only would
            # put the ranks out of step)
            ctx.set_wait_limit_ms(30000)
            torch.cuda.synchronize()
            dist.barrier()

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
    finally:
        dec.close()
        if exchange is not None:
            exchange.close()
        if world > 1:
            ctx.set_wait_limit_ms(0)
    wbytes = cfg.n_layers * sum(n * (k // 256) * 144 for n, k in shapes.values()) + cfg.vocab * (cfg.d_model // 256) * 210
    peak, kind = measured_peak()
    gbs = wbytes / (ms * 1e-3) / 1e9
    return {"tok_s": B * 1e3 / ms, "ms_per_step": ms, "batch": B, "steps": steps, "n_gpus": world, "layers": cfg.n_layers,
            "parallelism": decode_parallelism(world, args.fused_exchange, B),
            "launch": "CUDA graph replay of one step" if graph is not None else "eager launches",
            "prefill_ms": prefill_ms, "prefill_tok_s": B * T * 1e3 / prefill_ms, "kv_cache": args.kv_dtype,
            "weight_bytes_per_step": wbytes,
            "roofline": {"bound": "hbm", "kernel": "decode step (weight stream, all GPUs)", "achieved": gbs,
                         "peak": peak * world, "peak_kind": kind, "unit": "GB/s", "frac": gbs / (peak * world)},
            "clocks": clocks}


def run_decode(args):
    """--workload decode: configuration 5 alone (see decode_measure), one JSON line."""
    import torch
    import torch.distributed as dist
    import skainet_b200 as skn
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = skn.Context(local)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    B = args.batch
    r = decode_measure(args, ctx, stream, world, rank, local, B, min(args.steps, 128),
                       n_layers=args.layers if args.layers != 128 else args.decode_layers)
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tok_s", "value": r["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": r["steps"], "warmup": 3,
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"cfg5: Llama-style decoder, {r['layers']} layers, Q4_K / Q6_K, batch {B}, "
                                   f"512-token prefill then greedy decode",
                       "parallelism": r["parallelism"], "launch": r["launch"], "prefill_ms": r["prefill_ms"],
                       "prefill_tok_s": r["prefill_tok_s"], "kv_cache": r["kv_cache"],
                       "weight_bytes_per_step": r["weight_bytes_per_step"]},
            "roofline": dict(r["roofline"], traffic=None), "clocks": r["clocks"]}), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=128)
    ap.add_argument("--passes", type=int, default=80, help="passes over the stack per timed step")
    ap.add_argument("--e2e-passes", type=int, default=20, help="passes per step of the host-pointer (e2e) leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the configuration-5 decoder leg of the headline line")
    ap.add_argument("--decode-steps", type=int, default=128)
    ap.add_argument("--decode-deadline", type=float, default=300.0,
                    help="seconds after which unfinished decode legs are given up and the line is printed without them")
    ap.add_argument("--decode-layers", type=int, default=32)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--order", default="relaxed", choices=["relaxed", "stream"],
                    help="relaxed: the layers of a step are declared independent (SKN_OPT_RELAXED_ORDER) and "
                         "may overlap; stream: each launch waits for the one before it")
    ap.add_argument("--batch", type=int, default=1, help="decode workload: sequences per step")
    ap.add_argument("--kv-dtype", default="f32", choices=["f32", "f16", "q8_0"],
                    help="attn / decode workloads: element type of the KV cache (f32 is what the configurations specify)")
    ap.add_argument("--fused-exchange", default="auto", choices=["auto", "on", "off"],
                    help="tensor-parallel decode: push partial sums from the matvec epilogue (SKN_OPT_FUSED_EXCHANGE); "
                         "auto = the library's choice (off)")
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
